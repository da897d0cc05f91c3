"""Host side of the session on CPU: chunking, right padding, positions, limits, greedy generation and
the perf runner, against a recording stand-in for the native library.

What is held here is the behaviour of the reference's `IreeSession` / `generate_greedy` / `run_perf`
(crates/dyninfer-runtime/src/session.rs:88-389, generate.rs:117-232, perf.rs:92-172) that the Python
mirror repeats above the C ABI. The stand-in computes nothing: it records every call and answers with
scripted tokens, so the tests see exactly what the native session would be asked to do."""
import ctypes as C
import json

import numpy as np
import pytest

from dyninfer_b200 import _lib, runtime, synth
from dyninfer_b200.runtime import (DynInferError, GenerateConfig, ModelLoader, PerfConfig, SessionConfig,
                                   generate_greedy, run_perf)

VOCAB = 96


class RecordingLibrary:
    """Answers the session's native calls; `script` maps (position of the answered row) -> token."""

    def __init__(self):
        self.calls = []
        self.invokes = []          # (tokens, last, start_pos, want_logits)
        self.pages = 0
        self.script = lambda pos: (pos * 7 + 3) % VOCAB
        self._logits = (C.c_float * VOCAB)()
        self.descriptor = None
        self.keys = None
        self.fail_next_invoke = None
        self.slot_invokes = []     # (slot, tokens, last, start_pos, want_logits)
        self.batch_steps = []      # ([(slot, token, position)], want_logits)

    def dyninfer_cuda_last_error(self):
        return (self.fail_next_invoke or "").encode()

    def dyninfer_cuda_session_create_with_file_params(self, device, desc, files, nfiles, params, nparams, out):
        self.calls.append("create")
        self.device = device.decode()
        self.descriptor = json.loads(desc.decode())
        self.files = [files[i].path.decode() for i in range(nfiles)]
        self.keys = [(params[i].key.decode(), params[i].source_file_index, params[i].offset, params[i].length)
                     for i in range(nparams)]
        out._obj.value = 0x5E55
        return 0

    def dyninfer_cuda_session_destroy(self, h):
        self.calls.append("destroy")

    def dyninfer_cuda_session_configure_paged_kv(self, h, layers, page, kv_heads, head_dim, elem, chunk, vocab):
        self.calls.append("configure")
        self.kv_config = (layers, page, kv_heads, head_dim, elem, chunk, vocab)
        return 0

    def dyninfer_cuda_session_ensure_kv_pages(self, h, pages):
        self.calls.append("ensure")
        self.pages = max(self.pages, pages)
        return 0

    def dyninfer_cuda_session_reset_paged_kv(self, h):
        self.calls.append("reset")
        return 0

    def dyninfer_cuda_session_kv_page_count(self, h):
        return self.pages

    def dyninfer_cuda_session_kv_allocated_bytes(self, h):
        return self.pages * 1000

    def dyninfer_cuda_session_allocator_statistics(self, h, out):
        st = out._obj
        st.device_bytes_allocated, st.device_bytes_freed, st.device_bytes_peak = 900, 100, 950
        return 0

    def dyninfer_cuda_session_invoke_paged_chunk(self, h, tokens, n, last, start, out_logits, out_count, out_token,
                                                 want_logits):
        if self.fail_next_invoke:
            return 1
        self.calls.append("invoke")
        self.invokes.append(([int(tokens[i]) for i in range(n)], int(last), int(start), int(want_logits)))
        token = self.script(start + last)
        if want_logits:
            for i in range(VOCAB):
                self._logits[i] = 1.0 if i == token else 0.0
            out_logits._obj.contents = self._logits
            out_count._obj.value = VOCAB
        out_token._obj.value = token
        return 0


    def dyninfer_cuda_session_invoke_paged_chunk_slot(self, h, tokens, n, last, start, slot, out_logits, out_count,
                                                      out_token, want_logits):
        self.slot_invokes.append((int(slot), [int(tokens[i]) for i in range(n)], int(last), int(start),
                                  int(want_logits)))
        out_token._obj.value = self.script(start + last) + int(slot)
        if want_logits:
            out_logits._obj.contents = self._logits
            out_count._obj.value = VOCAB
        return 0

    def dyninfer_cuda_session_decode_batch(self, h, tokens, positions, slots, n, out_tokens, out_logits, want_logits):
        rows = [(int(slots[i]), int(tokens[i]), int(positions[i])) for i in range(n)]
        self.batch_steps.append((rows, int(want_logits)))
        for i, (slot, _, pos) in enumerate(rows):
            out_tokens[i] = self.script(pos) + slot
        if want_logits:
            self._batch_logits = (C.c_float * (n * VOCAB))(*[float(i // VOCAB) for i in range(n * VOCAB)])
            out_logits._obj.contents = self._batch_logits
        return 0


@pytest.fixture
def fake(monkeypatch):
    f = RecordingLibrary()
    monkeypatch.setattr(runtime, "lib", lambda: f)
    monkeypatch.setattr(_lib, "lib", lambda: f)
    monkeypatch.setattr(_lib, "_lib", f)
    return f


@pytest.fixture
def model(tmp_path, fake):
    path = str(tmp_path / "tiny.gguf")
    synth.write_qwen3_gguf(path, dict(vocab=VOCAB, hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=64,
                                      layers=2, eps=1e-6, theta=1e6), seed=5)
    return ModelLoader().load(path, target="cuda:0", max_kv=2048, kv_dtype="bf16")


def test_session_creation_hands_over_the_plan_unchanged(model, fake):
    with model.create_session(SessionConfig(max_sequence_length=2048)) as s:
        assert fake.calls[:2] == ["create", "configure"]
        assert fake.device == "cuda:0" and fake.files == model.plan.file_paths
        assert fake.keys == [(p.external_key, p.source_file_index, p.offset, p.length)
                             for p in model.plan.parameters]
        assert all(k.startswith("weights::") for k, *_ in fake.keys)
        layers, page, kv_heads, head_dim, elem, chunk, vocab = fake.kv_config
        assert (layers, page, kv_heads, head_dim, elem, chunk, vocab) == (2, 256, 2, 64, 2, 512, VOCAB)
        assert fake.descriptor["kv_dtype"] == "bf16"
        assert s.position() == 0
    assert fake.calls[-1] == "destroy"


def test_prefill_is_chunked_and_right_padded(model, fake):
    prompt = [(3 * i + 1) % VOCAB for i in range(1100)]
    with model.create_session(SessionConfig(max_sequence_length=2048)) as s:
        tok = s.prefill_argmax(prompt)
        assert [(len(t), last, start, want) for t, last, start, want in fake.invokes] == \
            [(512, 511, 0, 0), (512, 511, 512, 0), (512, 75, 1024, 0)]
        assert fake.invokes[0][0] == prompt[:512] and fake.invokes[1][0] == prompt[512:1024]
        tail = fake.invokes[2][0]
        assert tail[:76] == prompt[1024:] and set(tail[76:]) == {s.pad_token_id}
        assert tok == fake.script(1099) and s.position() == 1100
        assert fake.pages == 8                      # ceil(2048 / 256): the whole session limit up front
        # logits are asked for on the final chunk only
        fake.invokes.clear()
        lg = s.prefill(prompt[:600])
        assert [want for *_, want in fake.invokes] == [0, 1]
        assert lg.values.shape == (VOCAB,) and int(np.argmax(lg.values)) == fake.script(599)
        assert s.position() == 600                  # a new prefill starts the sequence again
        assert fake.calls.count("reset") == 2


def test_decode_tracks_the_position_and_stops_at_the_limit(model, fake):
    with model.create_session(SessionConfig(max_sequence_length=20)) as s:
        nxt = s.prefill_argmax([1, 2, 3, 4])
        fake.invokes.clear()
        for step in range(16):
            nxt = s.decode_argmax(nxt)
            tokens, last, start, want = fake.invokes[-1]
            assert (len(tokens), last, start, want) == (1, 0, 4 + step, 0)
            assert nxt == fake.script(4 + step)
        assert s.position() == 20
        with pytest.raises(DynInferError, match="decode position 20 exceeds session/KV limit 20"):
            s.decode_argmax(nxt)
        with pytest.raises(DynInferError, match="prefill length 21 exceeds session/KV limit 20"):
            s.prefill_argmax(list(range(21)))
        with pytest.raises(DynInferError, match="non-empty"):
            s.prefill_argmax([])
        s.reset()
        assert s.position() == 0 and s.history == []
        lg = s.decode(5)                             # decode with logits goes through the array form
        assert fake.invokes[-1] == ([5], 0, 0, 1) and lg.values.shape == (VOCAB,)


def test_session_limits_and_native_errors(model, fake):
    with model.create_session(SessionConfig(max_sequence_length=4096)) as s:
        assert s._max_seq() == 2048                  # the smaller of the session and the KV limit
    with model.create_session(SessionConfig(max_sequence_length=64, batch_size=2)) as s:
        with pytest.raises(DynInferError, match="only batch_size=1"):
            s.prefill_argmax([1, 2])
    with model.create_session(SessionConfig(max_sequence_length=64)) as s:
        fake.fail_next_invoke = "device says no"
        with pytest.raises(DynInferError, match="device says no"):
            s.prefill_argmax([1, 2, 3])
        fake.fail_next_invoke = None
        fake.script = lambda pos: -1
        with pytest.raises(DynInferError, match="invalid token -1"):
            s.prefill_argmax([1, 2, 3])


def test_metrics_follow_the_reference_arithmetic(model, fake):
    with model.create_session(SessionConfig(max_sequence_length=512)) as s:
        s.prefill_argmax([1] * 10)
        kv = s.kv_cache_metrics()
        assert kv.paged and kv.page_count == 2 and kv.allocated_bytes == 2000 and kv.filled_tokens == 10
        assert kv.capacity_bytes == 2 * 2 * 64 * 2 * 2 * 2048 and kv.chunk_size == 512
        assert kv.key_dtype == kv.value_dtype == "bf16"
        a = s.allocator_metrics()
        assert a.device_live_bytes() == 800 and a.device_bytes_peak == 950 and a.host_live_bytes() == 0


def test_generate_greedy_stops_and_counts(model, fake):
    ids, stats = generate_greedy(model, [4, 5, 6], GenerateConfig(max_new_tokens=5))
    want = [fake.script(2 + i) for i in range(5)]
    assert ids == [4, 5, 6] + want and stats.prompt_tokens == 3 and stats.generated_tokens == 5
    # an end-of-sequence token is not emitted and ends the run
    ids, stats = generate_greedy(model, [4, 5, 6], GenerateConfig(max_new_tokens=5, eos_token_id=want[2]))
    assert ids == [4, 5, 6] + want[:2] and stats.generated_tokens == 2
    ids, _ = generate_greedy(model, [4, 5, 6], GenerateConfig(max_new_tokens=5, stop_token_ids=[want[0]]))
    assert ids == [4, 5, 6]
    with pytest.raises(DynInferError, match="no tokens"):
        generate_greedy(model, [])


def test_generate_with_repetition_penalty_takes_the_logits_path(model, fake):
    fake.script = lambda pos: 9                      # the model always proposes token 9 (logit 1, the rest 0)
    fake.invokes.clear()
    ids, stats = generate_greedy(model, [1, 2], GenerateConfig(max_new_tokens=3, repetition_penalty=2.0))
    # every call asked for logits; the first step takes 9, after which its halved logit still wins over zeros
    assert all(want == 1 for *_, want in fake.invokes) and ids == [1, 2, 9, 9, 9] and stats.generated_tokens == 3
    logits = np.array([-1.0, 2.0, 0.5], dtype=np.float32)
    runtime.apply_repetition_penalty(logits, {0: 1, 1: 2}, 2.0)
    assert logits.tolist() == [-2.0, 1.0, 0.5]      # negative logits are multiplied, positive ones divided


def test_argmax_is_the_first_strict_maximum():
    assert runtime.argmax([1.0, 3.0, 3.0, 2.0]) == 1
    assert runtime.argmax([float("nan"), -1.0, float("nan")]) == 1
    assert runtime.argmax([float("-inf")] * 3) == 0 and runtime.argmax([]) == 0
    assert runtime.argmax([float("nan")] * 2) == 0


def test_run_perf_repeats_reset_prefill_decode(model, fake):
    rep = run_perf(model, PerfConfig(prefill_tokens=600, tg=4, warmup=1, iters=3, weight_bytes=10**9),
                   SessionConfig(max_sequence_length=1024))
    # (1 warm-up + 3 iterations) x (two prefill chunks + four decode steps)
    assert len(fake.invokes) == 4 * (2 + 4)
    per_iter = fake.invokes[:6]
    assert [(len(t), start) for t, _, start, _ in per_iter] == [(512, 0), (512, 512), (1, 600), (1, 601), (1, 602),
                                                                (1, 603)]
    assert fake.invokes[6:12] == per_iter            # every iteration starts from a reset session
    assert rep["prefill"]["tokens"] == 600 and rep["decode"]["tokens"] == 4 and rep["iters"] == 3
    # a prefill streams the weights once per chunk, a decode phase once per token
    assert rep["prefill"]["eff_weight_bw_gbs"] == pytest.approx(2 / rep["prefill"]["secs"])
    assert rep["decode"]["eff_weight_bw_gbs"] == pytest.approx(4 / rep["decode"]["secs"])
    with pytest.raises(DynInferError, match="--prefill must be > 0"):
        run_perf(model, PerfConfig(prefill_tokens=0))
    with pytest.raises(DynInferError, match="--iters must be > 0"):
        run_perf(model, PerfConfig(iters=0))


def test_target_resolution_never_reaches_a_cpu():
    profile, uri = ModelLoader.resolve_target("cuda")
    assert uri == "cuda:0" and profile.driver == "cuda"
    assert ModelLoader.resolve_target("cuda:3")[1] == "cuda:3"
    assert ModelLoader.resolve_target("cuda:sm_100")[1] == "cuda:0"
    for bad in ("cpu", "local-task", "hip", "rocm:gfx1151"):
        with pytest.raises(DynInferError, match="no CPU fallback"):
            ModelLoader.resolve_target(bad)


def test_batched_session_places_sequences_in_slots(model, fake):
    with model.create_batched_session(SessionConfig(max_sequence_length=1024, batch_size=4)) as s:
        assert fake.descriptor["batch"] == 4 and s.slots == 4
        first = {slot: s.prefill_slot(slot, [slot + 1] * (600 if slot == 2 else 5)) for slot in range(4)}
        assert s.positions == [5, 5, 600, 5]
        # slot 2's prompt spans two chunk calls; every chunk is right padded to the chunk size
        assert [(slot, len(t), last, start) for slot, t, last, start, _ in fake.slot_invokes] == \
            [(0, 512, 4, 0), (1, 512, 4, 0), (2, 512, 511, 0), (2, 512, 87, 512), (3, 512, 4, 0)]
        assert first == {0: fake.script(4), 1: fake.script(4) + 1, 2: fake.script(599) + 2, 3: fake.script(4) + 3}
        # one step over a subset of the slots: rows in ascending slot order, each at its own position
        nxt = s.step({3: 30, 0: 10, 2: 20})
        rows, want = fake.batch_steps[-1]
        assert rows == [(0, 10, 5), (2, 20, 600), (3, 30, 5)] and want == 0
        assert nxt == {0: fake.script(5), 2: fake.script(600) + 2, 3: fake.script(5) + 3}
        assert s.positions == [6, 5, 601, 6]
        nxt, logits = s.step({1: 7}, want_logits=True)
        assert fake.batch_steps[-1] == ([(1, 7, 5)], 1) and logits[1].shape == (VOCAB,) and set(nxt) == {1}
        assert s.step({}) == {} and s.step({}, want_logits=True) == ({}, {})
        with pytest.raises(DynInferError, match=r"slot 4 outside \[0, 4\)"):
            s.prefill_slot(4, [1])
        with pytest.raises(DynInferError, match=r"slot 9 outside \[0, 4\)"):
            s.step({9: 1})
        with pytest.raises(DynInferError, match=r"prefill length 0 outside \[1, 1024\]"):
            s.prefill_slot(0, [])
        s.positions[1] = 1024
        with pytest.raises(DynInferError, match="slot 1: decode position 1024 exceeds session/KV limit 1024"):
            s.step({1: 3})
        s.reset()
        assert s.positions == [0, 0, 0, 0]
    with pytest.raises(DynInferError, match="batch_size must be >= 1"):
        model.create_batched_session(SessionConfig(batch_size=0))
