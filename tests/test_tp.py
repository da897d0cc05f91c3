"""Tensor-parallel shard plan (host logic of the large configuration) on CPU.

The plan only selects verbatim byte ranges. Two gloo ranks each read their shard of a seeded GGUF
model, run one attention-output + feed-forward style chain with the CPU oracle (column-parallel
products, row-parallel products, all-reduce after each row-parallel product) and must reproduce the
unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as mp

CFG = dict(layers=1, hidden=512, heads=8, kv_heads=4, head_dim=64, intermediate=1024, vocab=512, eps=1e-6,
           theta=1e4)


def _write_model(path):
    from dyninfer_b200 import synth
    synth.write_qwen3_gguf(path, CFG, seed=5, encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"})


def _oracle_weight(orc, files, sp):
    from dyninfer_b200 import tp
    return orc.Weight(sp.encoding, sp.shape[0], sp.shape[1], tp.read_shard(files, sp)["data"])


def _chain(orc, weights, x, reduce_fn):
    """x [1, H] -> column q -> row o (+reduce) -> column gate, up -> row down (+reduce)."""
    q = orc.linear(weights["blk.0.attn_q.weight"], x)                      # [1, qd / W]
    o = reduce_fn(orc.linear(weights["blk.0.attn_output.weight"], q))      # partial over this rank's K
    h = x + o
    g = orc.linear(weights["blk.0.ffn_gate.weight"], h)
    u = orc.linear(weights["blk.0.ffn_up.weight"], h)
    act = (g / (1.0 + np.exp(-g))) * u
    d = reduce_fn(orc.linear(weights["blk.0.ffn_down.weight"], act))
    return h + d, orc.linear(weights["output.weight"], h + d)              # lm_head rows of this rank


def _rank_main(rank, world, port, path, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    from dyninfer_b200 import checkpoint as ck, replicas, tp
    from oracle import oracle as orc
    orc.build()
    replicas.init("gloo")
    cat = ck.open_catalog(path)
    plan = tp.plan(cat, rank, world)
    names = [n for n in plan if n.startswith("blk.0.") and plan[n].kind != "replicated"] + ["output.weight"]
    weights = {n: _oracle_weight(orc, cat.files, plan[n]) for n in names}

    def all_reduce(v):
        t = torch.from_numpy(np.ascontiguousarray(v))
        dist.all_reduce(t)
        return t.numpy()

    x = np.random.default_rng(1).normal(size=(1, CFG["hidden"])).astype(np.float32)
    hidden, logits_rows = _chain(orc, weights, x, all_reduce)
    gathered = [torch.zeros(logits_rows.shape, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(logits_rows))
    out.put((rank, hidden, np.concatenate([g.numpy() for g in gathered], axis=1),
             {n: (plan[n].kind, plan[n].shape) for n in names}))
    replicas.shutdown()


def test_two_rank_plan_matches_unsharded(tmp_path, oracle):
    from dyninfer_b200 import checkpoint as ck, tp
    path = str(tmp_path / "tp.gguf")
    _write_model(path)
    cat = ck.open_catalog(path)
    full = tp.plan(cat, 0, 1)
    names = [n for n in full if n.startswith("blk.0.") and full[n].kind != "replicated"] + ["output.weight"]
    weights = {n: _oracle_weight(oracle, cat.files, full[n]) for n in names}
    x = np.random.default_rng(1).normal(size=(1, CFG["hidden"])).astype(np.float32)
    want_hidden, want_logits = _chain(oracle, weights, x, lambda v: v)

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, path, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted((out.get(timeout=180) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, hidden, logits, shapes in results:
        assert np.abs(hidden - want_hidden).max() < 1e-4 * max(1.0, np.abs(want_hidden).max())
        assert np.abs(logits - want_logits).max() < 1e-4 * max(1.0, np.abs(want_logits).max())
        assert shapes["blk.0.attn_q.weight"] == ("column", (CFG["heads"] * CFG["head_dim"] // 2, CFG["hidden"]))
        assert shapes["blk.0.attn_output.weight"] == ("row", (CFG["hidden"], CFG["heads"] * CFG["head_dim"] // 2))
        assert shapes["blk.0.ffn_down.weight"] == ("row", (CFG["hidden"], CFG["intermediate"] // 2))
        assert shapes["output.weight"] == ("column", (CFG["vocab"] // 2, CFG["hidden"]))


def test_plan_ranges_and_rejections(tmp_path):
    from dyninfer_b200 import checkpoint as ck, tp
    path = str(tmp_path / "tp.gguf")
    _write_model(path)
    cat = ck.open_catalog(path)
    p0, p1 = tp.plan(cat, 0, 2), tp.plan(cat, 1, 2)
    q = cat.parameters["blk.0.attn_q.weight"]
    r0, r1 = p0[q.canonical].ranges[0], p1[q.canonical].ranges[0]
    assert r0.rows == 1 and r0.offset == q.components[0].offset and r1.offset == r0.offset + r0.seg_bytes
    assert r0.seg_bytes + r1.seg_bytes == q.components[0].length            # column split: two halves
    dn = cat.parameters["blk.0.ffn_down.weight"]                            # Q8_0, K = 1024 -> 512 per rank
    s0, s1 = p0[dn.canonical].ranges[0], p1[dn.canonical].ranges[0]
    assert s0.rows == CFG["hidden"] and s0.row_stride == 1024 // 32 * 34 and s0.seg_bytes == 512 // 32 * 34
    assert s1.offset == s0.offset + s0.seg_bytes and s0.nbytes + s1.nbytes == dn.components[0].length
    assert p0["blk.0.attn_norm.weight"].kind == "replicated"
    assert p0["token_embd.weight"].kind == "replicated" and p0["output.weight"].kind == "column"
    with pytest.raises(ck.CheckpointError):
        tp.plan(cat, 0, 3)                                                  # must divide the kv head count
    with pytest.raises(ck.CheckpointError):
        tp.plan(cat, 2, 2)
    with pytest.raises(ck.CheckpointError):                                 # K/8 = 64 is not a Q6_K block multiple
        tp.shard_parameter(cat.parameters["token_embd.weight"], 0, 8, "row")


def test_session_inputs_describe_the_rank(tmp_path):
    """The descriptor of a rank carries its share of the geometry; the uploaded bytes of all ranks add
    up to every sharded tensor once (replicated ones once per rank)."""
    from dyninfer_b200 import checkpoint as ck, tp
    path = str(tmp_path / "tp.gguf")
    _write_model(path)
    cat = ck.open_catalog(path)
    d0, r0 = tp.session_inputs(cat, 0, 2, kv_dtype="f32")
    d1, r1 = tp.session_inputs(cat, 1, 2, kv_dtype="f32")
    for d, rank in ((d0, 0), (d1, 1)):
        assert (d["tp_rank"], d["tp_world"]) == (rank, 2) and d["decode_kernel"] == "graph"
        assert d["heads"] == CFG["heads"] // 2 and d["kv_heads"] == CFG["kv_heads"] // 2
        assert d["intermediate"] == CFG["intermediate"] // 2 and d["lm_head_rows"] == CFG["vocab"] // 2
        assert d["head_dim"] == CFG["head_dim"] and d["hidden"] == CFG["hidden"] and d["vocab"] == CFG["vocab"]
        assert d["params"]["blk.0.attn_output.weight"]["strided"]["data"][0] == CFG["hidden"]
        assert "strided" not in d["params"]["blk.0.attn_q.weight"]
    by_key0, by_key1 = {r[0]: r for r in r0}, {r[0]: r for r in r1}
    assert by_key0.keys() == by_key1.keys() and "weights::output.weight::data" in by_key0
    for name, p in cat.parameters.items():
        key = f"weights::{name}::data"
        total = by_key0[key][3] + by_key1[key][3]
        want = p.components[0].length * (2 if tp.plan(cat, 0, 2)[name].kind == "replicated" else 1)
        assert total == want, name


def test_strided_range_is_validated_before_any_device_work(tmp_path):
    """A strided span that is inconsistent with its byte count or leaves the file is refused by the
    session constructor (no GPU is needed to get that far)."""
    import ctypes as C
    import json
    from dyninfer_b200 import _lib, checkpoint as ck, tp
    path = str(tmp_path / "tp.gguf")
    _write_model(path)
    cat = ck.open_catalog(path)
    desc, ranges = tp.session_inputs(cat, 1, 2, kv_dtype="f32")
    lib = _lib.lib()
    lib.dyninfer_cuda_last_error.restype = C.c_char_p

    def create(desc, ranges):
        files = (_lib.ParameterFile * 1)(_lib.ParameterFile(path.encode()))
        keys = [r[0].encode() for r in ranges]
        params = (_lib.FileParam * len(keys))(*[_lib.FileParam(k, r[1], r[2], r[3]) for k, r in zip(keys, ranges)])
        h = C.c_void_p()
        rc = lib.dyninfer_cuda_session_create_with_file_params(b"cuda:0", json.dumps(desc).encode(), files, 1,
                                                               params, len(keys), C.byref(h))
        msg = lib.dyninfer_cuda_last_error().decode() if rc else ""
        if not rc:
            lib.dyninfer_cuda_session_destroy(h)
        return rc, msg

    bad = json.loads(json.dumps(desc))
    bad["params"]["blk.0.ffn_down.weight"]["strided"]["data"][0] += 1        # rows x segment != byte count
    rc, msg = create(bad, ranges)
    assert rc != 0 and "strided range" in msg and "ffn_down" in msg
    far = json.loads(json.dumps(desc))
    far["params"]["blk.0.ffn_down.weight"]["strided"]["data"][2] = 1 << 40    # last row far beyond the file
    rc, msg = create(far, ranges)
    assert rc != 0 and "exceeds file size" in msg
    wrong = json.loads(json.dumps(desc))
    wrong["lm_head_rows"] = CFG["vocab"]                                      # not vocab / tp_world
    rc, msg = create(wrong, ranges)
    assert rc != 0 and "lm_head_rows" in msg
