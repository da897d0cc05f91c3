"""Whole-decoder parity through the session ABI: logits, greedy tokens, prefill vs decode."""
import numpy as np
import pytest

import fixtures_ref as fx
import helpers
from dyninfer_b200 import DynInferError, checkpoint as ck, synth
from dyninfer_b200.runtime import GenerateConfig, ModelLoader, PerfConfig, SessionConfig, generate_greedy, run_perf

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def greedy_match(got, want_tokens, margins, tie=1e-3):
    """Identical greedy tokens except where the oracle's top-2 margin is a near-tie (< 1e-3)."""
    for i, (g, w) in enumerate(zip(got, want_tokens)):
        if g != w:
            assert margins[i] < tie, f"step {i}: token {g} != {w} with margin {margins[i]}"
            return i
    return len(want_tokens)


def oracle_run(oracle, cat, prompt, steps, kv_round=0, kv_cap=512, cfg_over=None):
    cfg = dict(cat.config, **(cfg_over or {}))
    m = oracle.Model(cfg, helpers.catalog_weights(oracle, cat), kv_cap=kv_cap, kv_round=kv_round, fast=True)
    logits, tok = m.forward(prompt)
    all_logits, toks, margins = [logits], [tok], []
    for _ in range(steps):
        top2 = np.partition(all_logits[-1], -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        logits, tok = m.forward([toks[-1]])
        all_logits.append(logits)
        toks.append(tok)
    top2 = np.partition(all_logits[-1], -2)[-2:]
    margins.append(float(top2[1] - top2[0]))
    return all_logits, toks, margins


@pytest.mark.parametrize("kind", ["f32", "gguf_mixed", "mlx_u4"])
def test_reference_tiny_fixtures(native_lib, oracle, tmp_path, kind):
    """The reference's differential e2e: logits within 1e-3 of reference.rs, tokens [1,2,3,0]
    (crates/dyninfer-runtime/src/e2e.rs:43-140,245-306,364-409)."""
    tens = fx.encoded_tensors(fx.TINY, kind)
    if kind == "mlx_u4":
        path = helpers.write_fixture_mlx(str(tmp_path / "m"), fx.TINY, tens)
    else:
        path = helpers.write_fixture_gguf(str(tmp_path / "t.gguf"), fx.TINY, tens, arch="llama")
    model = ModelLoader().load(path, max_kv=128, chunk_size=4)
    model.catalog.config.update(qk_norm=False, rope=False)     # the M1 fixture has neither
    want = fx.reference_rs_forward(fx.roundtrip_weights(fx.TINY, kind), [1, 2, 3, 0])
    with model.create_session(SessionConfig(max_sequence_length=128)) as s:
        got = s.prefill([1, 2, 3, 0]).values
        assert np.abs(got - want).max() < 1e-3
        assert s.position() == 4
        s.reset()
        s.prefill([1, 2, 3])
        step = s.decode(0).values                               # prefill(3) + decode(1) == prefill(4)
        assert np.abs(step - got).max() < 1e-3
        assert s.prefill_argmax([1, 2, 3, 0]) == int(np.argmax(want))


def test_gqa_rope_qknorm_prefill_vs_decode(native_lib, oracle, tmp_path):
    """e2e.rs:412-464,509-552: GQA + RoPE + QK-norm, prefill vs step decode < 1e-2 (here 1e-4)."""
    tens = fx.encoded_tensors(fx.GQA, "f32")
    path = helpers.write_fixture_gguf(str(tmp_path / "g.gguf"), fx.GQA, tens)
    model = ModelLoader().load(path, max_kv=8, chunk_size=4)
    cat = ck.open_catalog(path)
    want, _, _ = oracle_run(oracle, cat, [5, 17, 3, 41], 0, kv_cap=8)
    with model.create_session(SessionConfig(max_sequence_length=8)) as s:
        full = s.prefill([5, 17, 3, 41]).values
        assert np.abs(full - want[0]).max() < 1e-4
        s.reset()
        lg = s.prefill([5]).values
        for t in [17, 3, 41]:
            lg = s.decode(t).values
        assert np.abs(lg - full).max() < 1e-4
        for _ in range(4):
            lg = s.decode(1).values
        with pytest.raises(DynInferError, match="exceeds session/KV limit"):
            s.decode(1)


def test_k_quant_tensors_in_a_mixed_model(native_lib, oracle, tmp_path):
    """Q4_K, Q5_K and IQ4_XS linears (what Q4_K_M / UD-Q4_K_XL files mix with Q4_0 and Q6_K) through the
    operator path: prompt in chunks (tensor-core GEMM), then single-row steps."""
    path = synth.write_qwen3_gguf(str(tmp_path / "kq.gguf"), synth.TINY, seed=13,
                                  encodings={"attn_q": "gguf.q4_k", "attn_k": "gguf.iq4_xs", "attn_output": "gguf.q5_k",
                                             "ffn_gate": "gguf.q4_k", "ffn_up": "gguf.iq4_xs", "ffn_down": "gguf.q5_k"})
    cat = ck.open_catalog(path)
    prompt = np.random.default_rng(8).integers(0, synth.TINY["vocab"], size=40).tolist()
    want_logits, want_toks, margins = oracle_run(oracle, cat, prompt, 6)
    model = ModelLoader().load(path, max_kv=256, kv_dtype="f32", chunk_size=32)
    with model.create_session(SessionConfig(max_sequence_length=256)) as s:
        assert not s.uses_persistent_kernel()
        lg = s.prefill(prompt).values
        assert np.abs(lg - want_logits[0]).max() <= 1e-2 and helpers.cosine(lg, want_logits[0]) >= 0.9999
        for i in range(6):
            lg = s.decode(want_toks[i]).values
            assert np.abs(lg - want_logits[i + 1]).max() <= 1e-2 and helpers.cosine(lg, want_logits[i + 1]) >= 0.9999


@pytest.mark.parametrize("flavor", ["gguf_q4_0", "gguf_mixed", "mlx_u4"])
@pytest.mark.parametrize("kv", ["f32", "bf16"])
@pytest.mark.parametrize("kernel", ["persistent", "graph"])
def test_tiny_qwen3_logits_and_greedy(native_lib, oracle, tmp_path, flavor, kv, kernel):
    """Seeded Qwen3-shaped model (2 layers): prompt of 16 ids, 32 greedy steps.
    logits max-abs <= 1e-2, cosine >= 0.9999, identical greedy tokens except near-ties."""
    # the persistent kernel needs 1024-wide Q6_K rows: its cases run on the smallest shapes it takes
    cfg = synth.TINY if kernel == "graph" else (synth.SMALL_D64 if kv == "f32" else synth.SMALL_D128)
    if flavor == "mlx_u4":
        path = synth.write_qwen3_mlx(str(tmp_path / "mlx"), cfg, seed=11)
    else:
        encs = {"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"} if flavor == "gguf_mixed" else None
        path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), cfg, seed=11, encodings=encs,
                                      output="gguf.q6_k" if flavor == "gguf_mixed" else None)
    model = ModelLoader().load(path, max_kv=512, kv_dtype=kv, chunk_size=16, decode_kernel=kernel)
    cat = ck.open_catalog(path)
    prompt = np.random.default_rng(5).integers(0, cfg["vocab"], size=16).tolist()
    steps = 32
    want_logits, want_toks, margins = oracle_run(oracle, cat, prompt, steps, kv_round=2 if kv == "bf16" else 0)
    with model.create_session(SessionConfig(max_sequence_length=512)) as s:
        # the path under test is the one that runs (the MLX model's head is its tied bf16 embedding table:
        # plain 16-bit tile steps inside the persistent kernel)
        assert s.uses_persistent_kernel() == (kernel == "persistent")
        lg = s.prefill(prompt).values
        assert np.abs(lg - want_logits[0]).max() <= 1e-2 and helpers.cosine(lg, want_logits[0]) >= 0.9999
        toks = [int(np.argmax(lg))]
        agree = 1
        for i in range(steps):
            # teacher-forced with the oracle's token so that every step is comparable
            lg = s.decode(want_toks[i]).values
            assert np.abs(lg - want_logits[i + 1]).max() <= 1e-2
            assert helpers.cosine(lg, want_logits[i + 1]) >= 0.9999
            toks.append(int(np.argmax(lg)))
        greedy_match(toks, want_toks, margins)
        # free-running greedy through the argmax entry points and the device-side loop
        first = s.prefill_argmax(prompt)
        run = [first]
        for _ in range(8):
            run.append(s.decode_argmax(run[-1]))
        n_ok = greedy_match(run, want_toks[:9], margins[:9])
        first2 = s.prefill_argmax(prompt)
        loop, ms = s.decode_loop(first2, 8)
        assert ms > 0 and [first2] + loop.tolist() == run
        assert n_ok >= 1 and s.launch_count() > 0


def test_chunked_prefill_padding_and_limits(native_lib, oracle, tmp_path):
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=2)
    cat = ck.open_catalog(path)
    prompt = np.random.default_rng(1).integers(0, 512, size=21).tolist()
    want, _, _ = oracle_run(oracle, cat, prompt, 0)
    model = ModelLoader().load(path, max_kv=300, chunk_size=8)       # 21 tokens = chunks 8 + 8 + 5 (right padded)
    with model.create_session(SessionConfig(max_sequence_length=300)) as s:
        lg = s.prefill(prompt).values
        # 8-row chunks of Q4_0 products run on the f16 tensor-core GEMM: the logits tolerance applies
        assert np.abs(lg - want[0]).max() <= 1e-2 and helpers.cosine(lg, want[0]) >= 0.9999
        m = s.kv_cache_metrics()
        assert m.page_count == 2 and m.paged and m.chunk_size == 8 and m.filled_tokens == 21
        assert m.allocated_bytes == 2 * 2 * 2 * 512 * 64 * 4        # K+V x layers x kv heads x cap x d x 4
        a = s.allocator_metrics()
        assert a.device_live_bytes() >= m.allocated_bytes + s.weight_bytes()
        s.reset()
        assert s.position() == 0 and s.kv_cache_metrics().page_count == 2   # reset keeps the pool
        assert np.abs(s.prefill(prompt).values - lg).max() == 0.0            # and is deterministic
        with pytest.raises(DynInferError, match="non-empty"):
            s.prefill([])
        with pytest.raises(DynInferError, match="exceeds session/KV limit"):
            s.prefill([1] * 301)
        with pytest.raises(DynInferError, match="token id"):
            s.prefill([1, 99999])
    with pytest.raises(DynInferError, match="only batch_size=1"):
        model.create_session(SessionConfig(batch_size=2)).prefill([1])


def test_abi_misuse_is_reported(native_lib, tmp_path):
    import ctypes as C
    from dyninfer_b200 import _lib
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=2)
    model = ModelLoader().load(path, max_kv=256, chunk_size=8)
    with model.create_session() as s:
        L, h = _lib.lib(), s._h
        tok = (C.c_int64 * 8)(*range(8))
        out = C.c_int64()
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 8, 0, 0, None, None, C.byref(out), 0) != 0
        assert "no pages" in _lib.last_error()
        assert L.dyninfer_cuda_session_ensure_kv_pages(h, 1) == 0
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 3, 0, 0, None, None, C.byref(out), 0) != 0
        assert "must be 1 or the chunk size" in _lib.last_error()
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 8, 8, 0, None, None, C.byref(out), 0) != 0
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 8, 0, -1, None, None, C.byref(out), 0) != 0
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 8, 7, 250, None, None, C.byref(out), 0) != 0
        assert "exceed the KV capacity" in _lib.last_error()
        # want_logits = 0 with NULL logits pointers still yields the argmax token (wrapper.c:1172-1215)
        assert L.dyninfer_cuda_session_invoke_paged_chunk(h, tok, 8, 7, 0, None, None, C.byref(out), 0) == 0
        assert 0 <= out.value < 512
        # reconfiguring after allocation is an error (wrapper.c:927-930)
        assert L.dyninfer_cuda_session_configure_paged_kv(h, 2, 256, 2, 64, 4, 8, 512) != 0
        assert "cannot be reconfigured" in _lib.last_error()
    bad = ck.open_catalog(path)
    plan = ck.build_runtime_provider_plan(bad)
    plan.parameters[0].length -= 18                                   # short byte range
    model.plan = plan
    with pytest.raises(DynInferError, match="byte range"):
        model.create_session()


def test_generate_and_perf_report(native_lib, tmp_path):
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=4)
    model = ModelLoader().load(path, max_kv=256, chunk_size=16)
    ids, stats = generate_greedy(model, [3, 1, 4, 1, 5], GenerateConfig(max_new_tokens=12), SessionConfig(256))
    assert len(ids) == 17 and stats.generated_tokens == 12 and stats.decode_tps() > 0
    ids2, _ = generate_greedy(model, [3, 1, 4, 1, 5], GenerateConfig(max_new_tokens=12, repetition_penalty=1.0 + 1e-9),
                              SessionConfig(256))
    assert ids2 == ids
    stop = ids[7]
    ids3, st3 = generate_greedy(model, [3, 1, 4, 1, 5], GenerateConfig(max_new_tokens=12, eos_token_id=stop), SessionConfig(256))
    assert stop not in ids3[5:] and st3.generated_tokens <= 2 + ids[5:].index(stop)
    rep = run_perf(model, PerfConfig(prefill_tokens=20, tg=4, warmup=1, iters=2, weight_bytes=1000), SessionConfig(256))
    assert rep["decode"]["tokens"] == 4 and rep["decode"]["eff_weight_bw_gbs"] > 0 and rep["prefill"]["tps"] > 0


@pytest.mark.parametrize("kv", ["f32", "bf16", "f16"])
def test_persistent_kernel_long_context_split_kv(native_lib, oracle, tmp_path, kv):
    """Context past 256 keys makes the persistent kernel split each head's keys over several
    CTAs; its logits must track both the oracle and the per-operator graph path."""
    cfg = synth.SMALL_D64 if kv == "f16" else synth.SMALL_D128
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), cfg, seed=21)
    cat = ck.open_catalog(path)
    prompt = np.random.default_rng(2).integers(0, 512, size=600).tolist()
    rnd = {"f32": 0, "f16": 1, "bf16": 2}[kv]
    want, toks, margins = oracle_run(oracle, cat, prompt, 3, kv_round=rnd, kv_cap=1024)
    outs = {}
    for kernel in ("persistent", "graph"):
        model = ModelLoader().load(path, max_kv=1024, kv_dtype=kv, chunk_size=128, decode_kernel=kernel)
        with model.create_session(SessionConfig(max_sequence_length=1024)) as s:
            assert s.uses_persistent_kernel() == (kernel == "persistent")
            lg = [s.prefill(prompt).values]
            for i in range(3):
                lg.append(s.decode(toks[i]).values)
            outs[kernel] = lg
    for i in range(4):
        for kernel in outs:
            assert np.abs(outs[kernel][i] - want[i]).max() <= 1e-2
            assert helpers.cosine(outs[kernel][i], want[i]) >= 0.9999
        assert np.abs(outs["persistent"][i] - outs["graph"][i]).max() <= 1e-3


@pytest.mark.parametrize("flavor,batch", [("gguf_q4_0", 3), ("mlx_u4", 5), ("gguf_mixed", 20)])
def test_batched_decode_matches_per_sequence_oracle(native_lib, oracle, tmp_path, flavor, batch):
    """`batch` sequences with different prompts and lengths share one session: every step decodes
    all of them in one pass (20 rows go through the tensor-core GEMM where the shapes allow).
    Each sequence must track its own single-sequence oracle run: logits max-abs <= 1e-2,
    cosine >= 0.9999 (teacher-forced), and slots must not disturb each other."""
    if flavor == "mlx_u4":
        path = synth.write_qwen3_mlx(str(tmp_path / "mlx"), synth.TINY, seed=3)
    else:
        encs = {"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"} if flavor == "gguf_mixed" else None
        path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=3, encodings=encs)
    model = ModelLoader().load(path, max_kv=256, kv_dtype="f32", chunk_size=16)
    cat = ck.open_catalog(path)
    rng = np.random.default_rng(batch)
    prompts = [rng.integers(0, synth.TINY["vocab"], size=int(rng.integers(1, 40))).tolist() for _ in range(batch)]
    steps = 6
    want = [oracle_run(oracle, cat, p, steps, kv_cap=256) for p in prompts]
    with model.create_batched_session(SessionConfig(max_sequence_length=256, batch_size=batch)) as s:
        feed = {}
        for b, p in enumerate(prompts):
            lg, tok = s.prefill_slot(b, p, want_logits=True)
            assert np.abs(lg - want[b][0][0]).max() <= 1e-2 and helpers.cosine(lg, want[b][0][0]) >= 0.9999
            feed[b] = want[b][1][0]
        for i in range(steps):
            nxt, logits = s.step(feed, want_logits=True)
            for b in range(batch):
                ref = want[b][0][i + 1]
                assert np.abs(logits[b] - ref).max() <= 1e-2 and helpers.cosine(logits[b], ref) >= 0.9999
                if nxt[b] != want[b][1][i + 1]:
                    assert want[b][2][i + 1] < 1e-3            # only a near-tie may differ
            feed = {b: want[b][1][i + 1] for b in range(batch)}
        # a subset of the slots may step on its own; the others keep their state
        sub = {0: want[0][1][steps], batch - 1: want[batch - 1][1][steps]}
        assert set(s.step(sub)) == {0, batch - 1}
        assert s.positions[0] == len(prompts[0]) + steps + 1 and s.positions[1] == len(prompts[1]) + steps
        with pytest.raises(DynInferError):
            s.step({batch: 1})


@pytest.mark.parametrize("kv", ["bf16", "f16"])
def test_long_prompt_prefill_tensor_core_path(native_lib, oracle, tmp_path, kv):
    """A 150-token prompt in chunks of 64 on a head-dim-128 model: the linears run on the tcgen05
    GEMM and attention on the tensor-core prefill kernel. The logits after the prompt and over the
    following greedy steps must match the oracle (logits max-abs <= 1e-2, cosine >= 0.9999)."""
    cfg = dict(layers=2, hidden=256, heads=2, kv_heads=1, head_dim=128, intermediate=512, vocab=512, eps=1e-6,
               theta=1e6)
    path = synth.write_qwen3_gguf(str(tmp_path / "d128.gguf"), cfg, seed=21)
    model = ModelLoader().load(path, max_kv=512, kv_dtype=kv, chunk_size=64)
    cat = ck.open_catalog(path)
    prompt = np.random.default_rng(9).integers(0, cfg["vocab"], size=150).tolist()
    steps = 4
    want_logits, want_toks, margins = oracle_run(oracle, cat, prompt, steps, kv_round=2 if kv == "bf16" else 1)
    with model.create_session(SessionConfig(max_sequence_length=512)) as s:
        lg = s.prefill(prompt).values
        assert np.abs(lg - want_logits[0]).max() <= 1e-2 and helpers.cosine(lg, want_logits[0]) >= 0.9999
        for i in range(steps):
            lg = s.decode(want_toks[i]).values
            assert np.abs(lg - want_logits[i + 1]).max() <= 1e-2 and helpers.cosine(lg, want_logits[i + 1]) >= 0.9999


def test_logit_drift_traces_cuda_vs_oracle(native_lib, oracle, tmp_path):
    """The drift harness end to end: the cuda target and the oracle write logit traces of the same
    forced trajectory (prompt of 12 ids, 10 forced decode inputs) and the per-row metric set stays
    inside the logits tolerance (max-abs 1e-2, cosine 0.9999)."""
    from dyninfer_b200 import drift
    path = synth.write_qwen3_gguf(str(tmp_path / "q.gguf"), synth.TINY, seed=23,
                                  encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"})
    cat = ck.open_catalog(path)
    rng = np.random.default_rng(9)
    prompt = rng.integers(0, synth.TINY["vocab"], size=12).tolist()
    want_logits, want_toks, _ = oracle_run(oracle, cat, prompt, 10)
    forced = want_toks[:10]                       # the oracle's own greedy trajectory
    sha = drift.sha256_of(path)
    with drift.TraceWriter(str(tmp_path / "ref"), "oracle-cpu", sha, synth.TINY["vocab"], prompt, forced) as w:
        for row in want_logits:
            w.write_row(row)
        ref_dir = w.finish()
    model = ModelLoader().load(path, max_kv=256, kv_dtype="f32", chunk_size=16)
    with model.create_session(SessionConfig(max_sequence_length=256)) as s:
        dyn_dir = drift.record(s, str(tmp_path / "dyn"), "dyninfer-cuda-sm_100a", sha, prompt, forced)
    rep = drift.compare_traces(ref_dir, dyn_dir, top_k=5)
    sm = rep["summary"]
    assert sm["row_count"] == 11 and sm["max_absolute_error"] <= 1e-2 and sm["min_cosine_similarity"] >= 0.9999
    assert sm["max_softmax_kl"] < 1e-4 and sm["min_top_k_overlap_fraction"] >= 0.8
    assert rep["reference_engine"] == "oracle-cpu" and rep["dyninfer_engine"] == "dyninfer-cuda-sm_100a"
