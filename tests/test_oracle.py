"""Pins the CPU oracle: golden vectors, the reference's fixture formulas, its test forward."""
import os

import numpy as np
import pytest

import fixtures_ref as fx
import helpers
import np_ref
from dyninfer_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dequant_golden.npz")
GGUF_ENCS = ["gguf.q4_0", "gguf.q4_1", "gguf.q8_0", "gguf.q6_k", "gguf.q4_k", "gguf.q5_k", "gguf.iq4_xs"]


@pytest.mark.parametrize("enc", GGUF_ENCS)
def test_dequant_matches_golden_bit_exact(oracle, enc):
    g = np.load(GOLD)
    raw, want = g[enc + ":raw"], g[enc + ":f32"]
    w = oracle.Weight(enc, want.shape[0], want.shape[1], raw)
    got = oracle.dequant(w)
    assert helpers.bits_equal(got, want)
    assert helpers.bits_equal(np_ref.dequant(enc, raw, *want.shape), want)


@pytest.mark.parametrize("enc", GGUF_ENCS)
def test_dequant_matches_gguf_package_live(oracle, enc):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    qt = getattr(gguf.GGMLQuantizationType, enc.split(".")[1].upper())
    raw = synth.random_weight(enc, 16, 1024, 99)["data"]
    want = quants.dequantize(raw.reshape(16, -1), qt).astype(np.float32)
    got = oracle.dequant(oracle.Weight(enc, 16, 1024, raw))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("enc,rt", [("gguf.q4_0", fx.q4_0_roundtrip), ("gguf.q4_1", fx.q4_1_roundtrip),
                                    ("gguf.q8_0", fx.q8_0_roundtrip)])
def test_reference_packers_roundtrip(oracle, enc, rt):
    """pack (q4.rs:16-98) then decode == the reference's round-trip formula (reference.rs:106-175)."""
    w = synth.fill_f32(64 * 128, 7).reshape(64, 128)
    pack = {"gguf.q4_0": synth.pack_q4_0, "gguf.q4_1": synth.pack_q4_1, "gguf.q8_0": synth.pack_q8_0}[enc]
    got = oracle.dequant(oracle.Weight(enc, 64, 128, pack(w)))
    assert np.array_equal(got, rt(w))  # value equality: the formula keeps -0.0 where blocks decode +0.0


def test_q4_0_pack_known_answer(oracle):
    """q4.rs test pack_dequant_roundtrip_rough: w_i = 0.01*i - 0.3, 64 values."""
    w = (np.arange(64, dtype=np.float32) * np.float32(0.01) - np.float32(0.3)).astype(np.float32)
    raw = synth.pack_q4_0(w)
    assert len(raw) == 36
    got = oracle.dequant(oracle.Weight("gguf.q4_0", 1, 64, raw))[0]
    assert np.abs(got - w).max() < 0.05


def test_mlx_u4_matches_reference_formula(oracle):
    w = synth.fill_f32(32 * 128, 3).reshape(32, 128)
    p, s, b = synth.quantize_affine_u4(w, 32, 128, 64)
    got = oracle.dequant(oracle.Weight("mlx.affine.u4", 32, 128, p.tobytes(), s, b, "plain.f32", 64))
    assert np.array_equal(got, fx.affine_u4_roundtrip(w))
    assert np.array_equal(got, np_ref.dequant("mlx.affine.u4", p.tobytes(), 32, 128, s, b, 64))
    # lane k of a packed word is bits [4k, 4k+4)
    word = np.array([[0x76543210] + [0] * 7], dtype=np.uint32)
    one, zero = np.ones((1, 1), np.float32), np.zeros((1, 1), np.float32)
    lanes = oracle.dequant(oracle.Weight("mlx.affine.u4", 1, 64, word.tobytes(), one, zero, "plain.f32", 64))
    assert lanes[0, :8].tolist() == [0, 1, 2, 3, 4, 5, 6, 7]


def test_mlx_bf16_aux_and_plain_types(oracle):
    t = synth.random_weight("mlx.affine.u4", 8, 256, 5)
    s32, b32 = synth.bf16_bits_to_f32(t["scales"]), synth.bf16_bits_to_f32(t["biases"])
    got = oracle.dequant(oracle.Weight("mlx.affine.u4", 8, 256, t["packed"], t["scales"], t["biases"], "plain.bf16", 64))
    assert np.array_equal(got, np_ref.dequant("mlx.affine.u4", t["packed"], 8, 256, s32, b32, 64))
    for enc in ("plain.bf16", "plain.f16", "plain.f32"):
        raw = synth.random_weight(enc, 4, 64, 1)["data"]
        assert np.array_equal(oracle.dequant(oracle.Weight(enc, 4, 64, raw)), np_ref.dequant(enc, raw, 4, 64))


def test_byte_size_table(oracle):
    """crates/dyninfer-checkpoint-gguf/src/types.rs:284-321."""
    L = oracle.lib()
    assert L.orc_row_bytes(oracle.Q4_0, 64) == 36
    assert L.orc_row_bytes(oracle.Q4_1, 32) == 20
    assert L.orc_row_bytes(oracle.Q8_0, 1024) == 34 * 32
    assert L.orc_row_bytes(oracle.Q6_K, 1024) == 840
    assert L.orc_row_bytes(oracle.MLX_U4, 1024) == 512


def test_linear_modes_and_torch(oracle):
    torch = pytest.importorskip("torch")
    raw = synth.random_weight("gguf.q4_0", 48, 256, 11)["data"]
    w = oracle.Weight("gguf.q4_0", 48, 256, raw)
    x = np.random.default_rng(0).normal(size=(3, 256)).astype(np.float32)
    y0, y1 = oracle.linear(w, x), oracle.linear(w, x, fast=True)
    ref = (torch.from_numpy(x).double() @ torch.from_numpy(oracle.dequant(w)).double().T).numpy()
    assert helpers.rel_err(y0, ref) < 1e-5 and helpers.rel_err(y1, ref) < 1e-5


@pytest.mark.parametrize("kind", ["f32", "gguf_mixed", "mlx_u4"])
def test_tiny_llama_forward_matches_reference_rs(oracle, kind):
    """The reference's own bar: logits within 1e-3 of reference.rs
    (crates/dyninfer-runtime/src/e2e.rs:93-100,298-305,401-408), tokens [1,2,3,0]."""
    tens = fx.encoded_tensors(fx.TINY, kind)
    m = oracle.Model(fx.TINY, helpers.oracle_weights(oracle, tens), kv_cap=16)
    logits, tok = m.forward([1, 2, 3, 0])
    want = fx.reference_rs_forward(fx.roundtrip_weights(fx.TINY, kind), [1, 2, 3, 0])
    assert np.abs(logits - want).max() < 1e-4
    assert tok == int(np.argmax(want))
    # prefill(4) == prefill(3) + decode(1)   (e2e.rs:111-132)
    m.reset()
    m.forward([1, 2, 3])
    step, _ = m.forward([0])
    assert np.abs(step - logits).max() < 1e-5


def test_gqa_rope_qknorm_prefill_equals_stepwise(oracle):
    """e2e.rs:412-464: prefill vs token-by-token decode on the GQA+RoPE+QK-norm fixture."""
    tens = fx.encoded_tensors(fx.GQA, "f32")
    w = helpers.oracle_weights(oracle, tens)
    a = oracle.Model(fx.GQA, w, kv_cap=8)
    full, _ = a.forward([5, 17, 3, 41])
    b = oracle.Model(fx.GQA, w, kv_cap=8)
    for t in [5, 17, 3, 41]:
        step, _ = b.forward([t])
    assert np.abs(full - step).max() < 1e-5
    assert np.isfinite(full).all() and full.shape == (48,)
    # RoPE and QK-norm are live: switching either off changes the logits
    for knob in ("rope", "qk_norm"):
        cfg = dict(fx.GQA, **{knob: False})
        other, _ = oracle.Model(cfg, w, kv_cap=8).forward([5, 17, 3, 41])
        assert np.abs(other - full).max() > 1e-4


@pytest.mark.parametrize("length", [255, 256, 257, 1100])
def test_online_softmax_page_walk_equals_direct(oracle, length):
    """kernels.rs:512-591,724-737: the paged online merge equals a direct softmax."""
    rng = np.random.default_rng(length)
    nh, nkv, d = 4, 2, 16
    q = rng.normal(size=(1, nh, d)).astype(np.float32)
    k = rng.normal(size=(nkv, length, d)).astype(np.float32)
    v = rng.normal(size=(nkv, length, d)).astype(np.float32)
    got = oracle.attention(q, k, v, start=length - 1, valid=1, page=256).reshape(nh, d)
    for h in range(nh):
        s = (k[h // 2].astype(np.float64) @ q[0, h].astype(np.float64)) / np.sqrt(d)
        p = np.exp(s - s.max())
        want = (p / p.sum()) @ v[h // 2].astype(np.float64)
        assert np.abs(got[h] - want).max() < 2e-6


def test_rope_and_argmax_semantics(oracle):
    x = np.random.default_rng(1).normal(size=(3, 2, 8)).astype(np.float32)
    y = oracle.rope(x, start_pos=5, theta=10000.0)
    i = np.arange(4, dtype=np.float32)
    freq = np.float32(1.0) / np.power(np.float32(10000.0), (np.float32(2.0) * i) / np.float32(8.0), dtype=np.float32)
    for p in range(3):
        ang = np.float32(5 + p) * freq
        lo = x[p, :, :4] * np.cos(ang) - x[p, :, 4:] * np.sin(ang)
        hi = x[p, :, :4] * np.sin(ang) + x[p, :, 4:] * np.cos(ang)
        assert np.abs(y[p, :, :4] - lo).max() < 1e-6 and np.abs(y[p, :, 4:] - hi).max() < 1e-6
    assert oracle.argmax(np.array([1, 3, 3, 2], np.float32)) == 1          # first maximum
    assert oracle.argmax(np.array([np.nan, -np.inf], np.float32)) == 0     # nothing beats -inf
    assert oracle.argmax(np.array([np.nan, 2, np.nan], np.float32)) == 1
