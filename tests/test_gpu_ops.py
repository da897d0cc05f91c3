"""Parity of every single operator against the CPU oracle, through the C ABI, on a GPU."""
import os

import numpy as np
import pytest

import helpers
from dyninfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GGUF_ENCS = ["gguf.q4_0", "gguf.q4_1", "gguf.q8_0", "gguf.q6_k", "gguf.q4_k", "gguf.q5_k", "gguf.iq4_xs"]
ENCS = GGUF_ENCS + ["mlx.affine.u4", "plain.bf16", "plain.f16", "plain.f32"]
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dequant_golden.npz")


def make_pair(oracle, enc, rows, cols, seed, aux="plain.bf16"):
    from dyninfer_b200 import ops
    t = synth.random_weight(enc, rows, cols, seed)
    if enc == "mlx.affine.u4":
        sc, bi = t["scales"], t["biases"]
        if aux == "plain.f32":
            sc, bi = synth.bf16_bits_to_f32(sc), synth.bf16_bits_to_f32(bi)
        dw = ops.DeviceWeight(enc, rows, cols, t["packed"], sc, bi, aux, 64)
        ow = oracle.Weight(enc, rows, cols, t["packed"], sc, bi, aux, 64)
    else:
        dw = ops.DeviceWeight(enc, rows, cols, t["data"])
        ow = oracle.Weight(enc, rows, cols, t["data"])
    return dw, ow


@pytest.mark.parametrize("enc", ENCS)
@pytest.mark.parametrize("shape", [(1, 256), (33, 512), (257, 1024)])
def test_dequant_bit_exact(native_lib, oracle, enc, shape):
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, enc, *shape, seed=shape[0])
    got = ops.dequant(dw).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.dequant(ow).view(np.uint32))


def test_dequant_golden_and_mlx_f32_aux(native_lib, oracle):
    from dyninfer_b200 import ops
    g = np.load(GOLD)
    for enc in GGUF_ENCS:
        want = g[enc + ":f32"]
        dw = ops.DeviceWeight(enc, want.shape[0], want.shape[1], g[enc + ":raw"])
        assert helpers.bits_equal(ops.dequant(dw).cpu().numpy(), want), enc
    dw, ow = make_pair(oracle, "mlx.affine.u4", 17, 512, 3, aux="plain.f32")
    assert np.array_equal(ops.dequant(dw).cpu().numpy().view(np.uint32), oracle.dequant(ow).view(np.uint32))


def test_dequant_full_size_q4_0_checksum(native_lib, oracle):
    """Full-size tensor (3072 x 1024): a sampled-row comparison plus a linearity property
    (sum over the tensor equals the sum of block scale x integer sums)."""
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, "gguf.q4_0", 3072, 1024, 7)
    got = ops.dequant(dw).cpu().numpy()
    for r in (0, 1, 1535, 3071):
        assert np.array_equal(got[r].view(np.uint32), oracle.dequant_row(ow, r).view(np.uint32))
    blk = ow.data.reshape(-1, 18)
    d = blk[:, :2].copy().view(np.float16).astype(np.float64)[:, 0]
    q = blk[:, 2:]
    isum = ((q & 15).astype(np.int64) - 8).sum(axis=1) + ((q >> 4).astype(np.int64) - 8).sum(axis=1)
    assert abs(got.astype(np.float64).sum() - float((d * isum).sum())) < 1e-6 * max(1.0, np.abs(d * isum).sum())


@pytest.mark.parametrize("enc", ENCS)
def test_embedding_gather(native_lib, oracle, enc):
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, enc, 64, 512, 9)
    ids = np.array([0, 63, 5, 5, 31], dtype=np.int64)
    got = ops.embedding_gather(dw, torch.from_numpy(ids)).cpu().numpy()
    for i, t in enumerate(ids):
        assert np.array_equal(got[i].view(np.uint32), oracle.dequant_row(ow, int(t)).view(np.uint32))
    assert ops.embedding_gather(dw, torch.zeros(0, dtype=torch.int64)).shape == (0, 512)


@pytest.mark.parametrize("enc", ENCS)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 17])
def test_linear_vs_oracle(native_lib, oracle, enc, m):
    """GEMV / skinny GEMM: rel <= 1e-3 with f32 accumulation (bf16 activations ~N(0,1))."""
    from dyninfer_b200 import ops
    n, k = 96, 1024
    dw, ow = make_pair(oracle, enc, n, k, seed=m)
    xb = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).to(torch.bfloat16)
    want = oracle.linear(ow, xb.float().numpy())
    got_bf16 = ops.linear(dw, xb.cuda()).cpu().numpy()
    got_f32 = ops.linear(dw, xb.float().cuda()).cpu().numpy()
    assert helpers.rel_err(got_bf16, want) < 1e-3 and helpers.rel_err(got_f32, want) < 1e-3
    if m <= 4:                                             # exact weights, f32 sums: only the order differs
        assert helpers.rel_err(got_f32, want) < 2e-5      # (more rows use the f16 tensor-core GEMM)


@pytest.mark.parametrize("enc,n,k", [("gguf.q4_0", 1, 32), ("gguf.q4_0", 5, 64), ("gguf.q8_0", 33, 96),
                                     ("gguf.q6_k", 3, 256), ("mlx.affine.u4", 7, 64), ("plain.f32", 2, 4),
                                     ("gguf.q4_1", 1024, 3072), ("gguf.q4_0", 3072, 1024)])
def test_linear_ragged_and_full_shapes(native_lib, oracle, enc, n, k):
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, enc, n, k, seed=n + k)
    x = np.random.default_rng(n).normal(size=(2, k)).astype(np.float32)
    got = ops.linear(dw, torch.from_numpy(x).cuda()).cpu().numpy()
    assert helpers.rel_err(got, oracle.linear(ow, x, fast=True)) < 1e-4


@pytest.mark.parametrize("enc", ["gguf.q4_0", "gguf.q4_1", "gguf.q8_0", "gguf.q6_k", "gguf.q4_k", "mlx.affine.u4"])
@pytest.mark.parametrize("n,k", [(33, 512), (1000, 3072), (4096, 12288), (12288, 4096), (40, 768), (5120, 6400)])
def test_linear_single_row_column_split(native_lib, oracle, enc, n, k):
    """One activation row (the decode shape) on the column-split tensor-core kernels: ragged last
    tile, split-K shapes, rows that end half way through a 512-element stage (the shard widths of
    a down projection split four ways), f32 and bf16 activations, against the oracle's pairwise sums."""
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, enc, n, k, seed=n ^ k)
    x = np.random.default_rng(k).normal(size=(1, k)).astype(np.float32)
    want = oracle.linear(ow, x, fast=True)
    got = ops.linear(dw, torch.from_numpy(x).cuda()).cpu().numpy()
    assert helpers.rel_err(got, want) < 2e-5
    xb = torch.from_numpy(x).to(torch.bfloat16)
    got = ops.linear(dw, xb.cuda()).cpu().numpy()
    assert helpers.rel_err(got, oracle.linear(ow, xb.float().numpy(), fast=True)) < 2e-5
    x[0, ::7] = 0.0                                    # zeros and a huge dynamic range in one row
    x[0, 5] = 3.0e4
    x[0, 6] = 1.0e-6
    got = ops.linear(dw, torch.from_numpy(x).cuda()).cpu().numpy()
    assert helpers.rel_err(got, oracle.linear(ow, x, fast=True)) < 2e-5


@pytest.mark.parametrize("group,aux", [(32, "bf16"), (64, "f16"), (128, "bf16")])
def test_linear_single_row_mlx_groups_and_f16_aux(native_lib, oracle, group, aux):
    """MLX-U4 single rows with groups of 32 (one scale per block), f16 scales and biases, and groups of
    128 (outside the column-split kernel's rules: another kernel takes it), against the oracle."""
    from dyninfer_b200 import ops
    n, k = 520, 2048
    t = synth.random_weight("mlx.affine.u4", n, k, 77, group=group)
    sc, bi, aux_name = t["scales"], t["biases"], "plain.bf16"
    if aux == "f16":
        sc = synth.bf16_bits_to_f32(sc).astype(np.float16)
        bi = synth.bf16_bits_to_f32(bi).astype(np.float16)
        aux_name = "plain.f16"
    dw = ops.DeviceWeight("mlx.affine.u4", n, k, t["packed"], sc, bi, aux_name, group)
    ow = oracle.Weight("mlx.affine.u4", n, k, t["packed"], sc, bi, aux_name, group)
    x = np.random.default_rng(group).normal(size=(1, k)).astype(np.float32)
    got = ops.linear(dw, torch.from_numpy(x).cuda()).cpu().numpy()
    assert helpers.rel_err(got, oracle.linear(ow, x, fast=True)) < 2e-5


@pytest.mark.parametrize("enc", ENCS)
@pytest.mark.parametrize("m,n,k", [(17, 128, 256), (64, 200, 1024), (300, 131, 512)])
def test_linear_many_rows_tensor_core(native_lib, oracle, enc, m, n, k):
    """More than 16 activation rows go through the tcgen05 dequant-GEMM (f16 operands, f32
    accumulation in tensor memory): ragged N tiles, several M tiles, bf16 and f32 activations,
    rows of very different magnitude. Tolerance: the path's stated rel 1e-3."""
    from dyninfer_b200 import ops
    dw, ow = make_pair(oracle, enc, n, k, seed=m + n)
    g = torch.Generator().manual_seed(m)
    xb = torch.randn(m, k, generator=g).to(torch.bfloat16)
    want = oracle.linear(ow, xb.float().numpy(), fast=True)
    got = ops.linear(dw, xb.cuda()).cpu().numpy()
    assert helpers.rel_err(got, want) < 1e-3
    xf = torch.randn(m, k, generator=g)
    xf[1] *= 1.0e5                                     # would overflow f16 without the per-row scale
    xf[2] *= 1.0e-6
    want = oracle.linear(ow, xf.numpy(), fast=True)
    got = ops.linear(dw, xf.cuda()).cpu().numpy()
    for r in (0, 1, 2, m - 1):                         # per row: each has its own magnitude
        assert helpers.rel_err(got[r], want[r]) < 1e-3


@pytest.mark.parametrize("enc", ["gguf.q4_0", "gguf.q4_1", "gguf.q8_0", "gguf.q6_k", "gguf.q4_k", "gguf.q5_k",
                                 "gguf.iq4_xs", "mlx.affine.u4"])
def test_tensor_core_operand_is_the_rounded_weight(native_lib, oracle, enc):
    """Identity activations read the dequant-GEMM's A operand back: y[k, n] = f16(w[n, k]). Every
    element of every 64-wide chunk and both halves of a 256-element block must land in its place.
    Q4_0, Q8_0, Q6_K, Q4_K, Q5_K and IQ4_XS round the decoder's f32 value once (bit-exact); Q4_1 rounds q*d + m once where
    the decoder rounds twice (one f16 unit); MLX-U4 takes its scale and bias as f16 (2^-10 relative)."""
    from dyninfer_b200 import ops
    n, k = 200, 512
    dw, ow = make_pair(oracle, enc, n, k, seed=91)
    got = ops.linear(dw, torch.eye(k).cuda()).cpu().numpy().T            # [n, k]
    w = oracle.dequant(ow)
    want = w.astype(np.float16).astype(np.float32)
    if enc in ("gguf.q4_0", "gguf.q8_0", "gguf.q6_k", "gguf.q4_k", "gguf.q5_k", "gguf.iq4_xs"):
        assert np.array_equal(got, want)                                  # -0.0 == +0.0
    elif enc == "gguf.q4_1":
        ulp = np.spacing(np.abs(want).astype(np.float16)).astype(np.float32)
        assert np.all(np.abs(got - want) <= ulp)
    else:
        assert np.all(np.abs(got - w) <= np.abs(w) * 2.0 ** -9 + 1e-6)


def test_linear_linearity_full_size_lm_head(native_lib, oracle):
    """Size-independent property at the lm_head's full size (151936 x 1024, Q6_K):
    W(a*x + y) == a*W(x) + W(y), and sampled rows against the oracle."""
    from dyninfer_b200 import ops
    n, k = 151936, 1024
    dw, ow = make_pair(oracle, "gguf.q6_k", n, k, seed=2)
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(1, k, generator=g).cuda(), torch.randn(1, k, generator=g).cuda()
    wx, wy, wxy = ops.linear(dw, x), ops.linear(dw, y), ops.linear(dw, 2.0 * x + y)
    assert helpers.rel_err((2.0 * wx + wy).cpu().numpy(), wxy.cpu().numpy()) < 1e-5
    xr = x.cpu().numpy()[0]
    for r in (0, 77777, n - 1):
        want = float(oracle.dequant_row(ow, r).astype(np.float64) @ xr.astype(np.float64))
        assert abs(float(wx[0, r]) - want) < 1e-4 * max(1.0, abs(want))


def test_rms_norm_rope_silu(native_lib, oracle):
    from dyninfer_b200 import ops
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 1024)).astype(np.float32) * 3
    w = rng.normal(size=1024).astype(np.float32)
    got = ops.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-6).cpu().numpy()
    assert np.abs(got - oracle.rms_norm(x, w, 1e-6)).max() < 1e-5
    wb = torch.from_numpy(w).to(torch.bfloat16)
    got = ops.rms_norm(torch.from_numpy(x).cuda(), wb.cuda(), 1e-6).cpu().numpy()
    assert np.abs(got - oracle.rms_norm(x, wb.float().numpy(), 1e-6)).max() < 1e-5
    h = rng.normal(size=(3 * 16, 128)).astype(np.float32)      # per-head norm over d = 128
    wd = rng.normal(size=128).astype(np.float32)
    got = ops.rms_norm(torch.from_numpy(h).cuda(), torch.from_numpy(wd).cuda(), 1e-6).cpu().numpy()
    assert np.abs(got - oracle.rms_norm(h, wd, 1e-6)).max() < 1e-5
    for d, theta, start in ((128, 1e6, 0), (128, 1e6, 4090), (8, 1e4, 3)):
        q = rng.normal(size=(4, 6, d)).astype(np.float32)
        got = ops.rope(torch.from_numpy(q).cuda(), start, theta).cpu().numpy()
        assert np.abs(got - oracle.rope(q, start, theta)).max() < 2e-5
    g, u = rng.normal(size=4096).astype(np.float32) * 4, rng.normal(size=4096).astype(np.float32)
    got = ops.silu_mul(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda()).cpu().numpy()
    assert np.abs(got - oracle.silu_mul(g, u)).max() < 1e-5


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("s,start,d,nh,nkv", [(1, 0, 128, 16, 8), (1, 300, 128, 16, 8), (5, 7, 128, 4, 2),
                                              (4, 0, 8, 4, 2), (3, 255, 64, 4, 4)])
def test_attention_vs_oracle(native_lib, oracle, dtype, s, start, d, nh, nkv):
    from dyninfer_b200 import ops
    rng = np.random.default_rng(start + s)
    cap = 512
    q = rng.normal(size=(s, nh, d)).astype(np.float32)
    k = rng.normal(size=(nkv, cap, d)).astype(np.float32)
    v = rng.normal(size=(nkv, cap, d)).astype(np.float32)
    tt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    kt, vt = torch.from_numpy(k).to(tt), torch.from_numpy(v).to(tt)
    want = oracle.attention(q, kt.float().numpy(), vt.float().numpy(), start, s)
    got = ops.attention(torch.from_numpy(q).cuda(), kt.cuda(), vt.cuda(), start).cpu().numpy()
    assert np.abs(got - want).max() < 2e-5


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("s,start,nh,nkv", [(100, 37, 4, 2), (64, 0, 2, 2), (130, 500, 4, 1), (200, 100, 40, 8)])
def test_attention_prefill_tensor_core(native_lib, oracle, dtype, s, start, nh, nkv):
    """32 or more consecutive rows of one sequence on a 2-byte cache take the tensor-core
    flash-attention kernel (head dim 128): ragged row blocks, GQA, a start position in the middle
    of a key block. Q and P enter as hi+lo pairs, so the result stays within 1e-3 relative of the
    f32 oracle (typically 1e-4)."""
    from dyninfer_b200 import ops
    d, cap = 128, 768
    rng = np.random.default_rng(s + start)
    q = rng.normal(size=(s, nh, d)).astype(np.float32)
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    kc = torch.from_numpy(rng.normal(size=(nkv, cap, d)).astype(np.float32)).to(tdt)
    vc = torch.from_numpy(rng.normal(size=(nkv, cap, d)).astype(np.float32)).to(tdt)
    kc[:, start + s:] = float("nan")                 # never-written rows must not leak into the result
    vc[:, start + s:] = float("nan")
    got = ops.attention(torch.from_numpy(q).cuda(), kc.cuda(), vc.cuda(), start).cpu().numpy()
    kf, vf = kc.float().numpy(), vc.float().numpy()
    kf[:, start + s:] = 0.0
    vf[:, start + s:] = 0.0
    want = oracle.attention(q, kf, vf, start, s)
    assert np.isfinite(got).all()
    assert helpers.rel_err(got, want) < 1e-3


def test_argmax_first_maximum(native_lib, oracle):
    from dyninfer_b200 import ops
    rng = np.random.default_rng(3)
    v = rng.normal(size=151936).astype(np.float32)
    assert ops.argmax(torch.from_numpy(v).cuda()) == oracle.argmax(v)
    v[[1000, 90000, 151935]] = 50.0                        # ties: the lowest index wins
    assert ops.argmax(torch.from_numpy(v).cuda()) == 1000
    v[:] = -np.inf
    assert ops.argmax(torch.from_numpy(v).cuda()) == 0
    v[7] = np.nan
    v[9] = -3.0
    assert ops.argmax(torch.from_numpy(v).cuda()) == 9
    assert ops.argmax(torch.tensor([2.0]).cuda()) == 0
