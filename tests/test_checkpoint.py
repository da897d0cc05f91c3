"""Containers, conventions and the direct byte-range provider plan (CPU only)."""
import json
import os
import struct

import numpy as np
import pytest

import fixtures_ref as fx
import helpers
from dyninfer_b200 import checkpoint as ck, synth


def test_gguf_roundtrip_and_third_party_reader(tmp_path):
    path = str(tmp_path / "tiny.gguf")
    synth.write_qwen3_gguf(path, synth.TINY, seed=3, encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"})
    idx = ck.index_gguf(path)
    assert idx.metadata["general.architecture"] == "qwen3"
    e = idx.entries["blk.1.attn_q.weight"]
    assert e.shape == (256, 256) and e.type_name == "gguf.q4_0" and e.nbytes == 256 * 8 * 18
    assert e.offset % 32 == 0
    assert idx.entries["token_embd.weight"].type_name == "gguf.q6_k"
    gguf = pytest.importorskip("gguf")
    rd = gguf.GGUFReader(path)
    theirs = {t.name: t for t in rd.tensors}
    assert set(theirs) == set(idx.entries)
    raw = np.fromfile(path, dtype=np.uint8)
    for name, ent in idx.entries.items():
        t = theirs[name]
        assert int(t.data_offset) == ent.offset and int(t.n_bytes) == ent.nbytes
        assert tuple(int(d) for d in reversed(t.shape)) == ent.shape     # on-disk dims are reversed
        assert np.array_equal(np.asarray(t.data).view(np.uint8).reshape(-1), raw[ent.offset:ent.offset + ent.nbytes])


def test_gguf_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(ck.CheckpointError, match="not a GGUF"):
        ck.index_gguf(str(p))
    p.write_bytes(b"GGUF" + struct.pack("<I", 1) + b"\0" * 64)
    with pytest.raises(ck.CheckpointError, match="version"):
        ck.index_gguf(str(p))
    good = str(tmp_path / "t.gguf")
    synth.write_qwen3_gguf(good, synth.TINY, seed=1)
    data = open(good, "rb").read()
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(data[:len(data) - 100])
    with pytest.raises(ck.CheckpointError, match="past end of file"):
        ck.index_gguf(str(trunc))


def test_gguf_catalog_and_plan(tmp_path):
    path = str(tmp_path / "tiny.gguf")
    synth.write_qwen3_gguf(path, synth.TINY, seed=3)
    cat = ck.open_catalog(path)
    c = cat.config
    assert (c["layers"], c["hidden"], c["heads"], c["kv_heads"], c["head_dim"], c["intermediate"], c["vocab"]) == \
        (2, 256, 4, 2, 64, 512, 512)
    assert c["tied"] and c["qk_norm"] and abs(c["theta"] - 1e6) < 1 and abs(c["eps"] - 1e-6) < 1e-12
    plan = ck.build_runtime_provider_plan(cat)
    assert plan.kind == "direct-file-ranges-v1" and plan.scope == "weights"
    keys = [p.external_key for p in plan.parameters]
    assert keys == sorted(keys) and "weights::blk.0.attn_q.weight::data" in keys
    idx = ck.index_gguf(path)
    for p in plan.parameters:                 # provider offset/length == catalog range (e2e.rs:309-361)
        name = p.external_key.split("::")[1]
        assert (p.offset, p.length) == (idx.entries[name].offset, idx.entries[name].nbytes)
    assert sorted(os.listdir(tmp_path)) == ["tiny.gguf"]   # nothing is written next to the file
    cat.parameters["x"] = ck.Parameter("x", "plain.f32", (1,), [ck.Component("data", "x", "plain.f32", (1,), 0, 10 ** 12, 4)])
    with pytest.raises(ck.CheckpointError, match="exceeds source size"):
        ck.build_runtime_provider_plan(cat)


def test_safetensors_mlx_convention(tmp_path):
    d = str(tmp_path / "mlx")
    synth.write_qwen3_mlx(d, synth.TINY, seed=5)
    st = pytest.importorskip("safetensors")
    from safetensors import safe_open
    idx = ck.index_safetensors(os.path.join(d, "model.safetensors"))
    assert idx.metadata.get("format") == "mlx"
    with safe_open(os.path.join(d, "model.safetensors"), "np") as f:
        assert set(f.keys()) == set(idx.entries)
        raw = np.fromfile(os.path.join(d, "model.safetensors"), dtype=np.uint8)
        k = "model.layers.0.self_attn.q_proj.weight"
        e = idx.entries[k]
        assert np.array_equal(f.get_tensor(k).view(np.uint8).reshape(-1), raw[e.offset:e.offset + e.nbytes])
    cat = ck.open_catalog(d)
    p = cat.parameters["blk.0.attn_q.weight"]
    assert p.encoding == "mlx.affine.u4" and p.shape == (256, 256) and p.group == 64
    assert [c.name for c in p.components] == ["packed", "scales", "biases"]
    assert cat.parameters["token_embd.weight"].encoding == "plain.bf16" and cat.config["tied"]
    keys = [q.external_key for q in ck.build_runtime_provider_plan(cat).parameters]
    assert "weights::blk.1.ffn_down.weight::scales" in keys
    # bits != 4 has no kernel (mlx_affine.rs:157-160)
    cj = os.path.join(d, "config.json")
    hf = json.load(open(cj))
    hf["quantization"]["bits"] = 8
    json.dump(hf, open(cj, "w"))
    with pytest.raises(ck.CheckpointError, match="bits=8"):
        ck.open_catalog(d)


def test_fixture_files_feed_the_oracle(tmp_path, oracle):
    """GGUF / SafeTensors files of the reference's tiny fixtures reproduce its logits when read back."""
    for kind in ("gguf_mixed", "mlx_u4"):
        tens = fx.encoded_tensors(fx.TINY, kind)
        if kind == "mlx_u4":
            path = helpers.write_fixture_mlx(str(tmp_path / "m"), fx.TINY, tens)
        else:
            path = helpers.write_fixture_gguf(str(tmp_path / "t.gguf"), fx.TINY, tens, arch="llama")
        cat = ck.open_catalog(path)
        cfg = dict(cat.config, qk_norm=False, rope=False)
        m = oracle.Model(cfg, helpers.catalog_weights(oracle, cat), kv_cap=8)
        logits, _ = m.forward([1, 2, 3, 0])
        want = fx.reference_rs_forward(fx.roundtrip_weights(fx.TINY, kind), [1, 2, 3, 0])
        assert np.abs(logits - want).max() < 1e-4
