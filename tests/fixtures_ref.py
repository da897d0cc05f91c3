"""The reference's generator fixtures and its test-only forward, restated in numpy.

The reference stores no golden logits; what pins its numeric path are seeded
generator fixtures compared against a small f32 forward:
  * fill_f32 LCG, seeds 1..9 per tensor: crates/dyninfer-checkpoint-gguf/src/q4.rs:212-223,274-291
  * tiny llama dims V=32 H=64 I=128 nh=4 d=16 S=4 eps=1e-5, no RoPE, no QK-norm:
    crates/dyninfer-runtime/src/reference.rs:6-12,195-227
  * mixed encodings of tiny_llama_q4_0 (attn_q Q4_1, attn_v Q8_0, others Q4_0, F32
    embedding): q4.rs:285-289
  * tiny_llama_mlx_affine_u4 (group 64, F32 scales/biases, every matrix incl. embedding):
    crates/dyninfer-checkpoint-safetensors/src/fixture.rs:208-285, reference.rs:49-60
  * tiny_gqa_rope_f32 (V=48 H=32 nh=4 nkv=2 d=8 I=64 theta 1e4 eps 1e-5): fixture.rs:323-432
"""
import numpy as np

from dyninfer_b200 import synth

TINY = dict(layers=1, hidden=64, heads=4, kv_heads=4, head_dim=16, intermediate=128, vocab=32,
            eps=1e-5, theta=10000.0, qk_norm=False, rope=False)
GQA = dict(layers=1, hidden=32, heads=4, kv_heads=2, head_dim=8, intermediate=64, vocab=48,
           eps=1e-5, theta=10000.0, qk_norm=True, rope=True)

_SEEDS = {"token_embd": 1, "attn_q": 2, "attn_k": 3, "attn_v": 4, "attn_output": 5,
          "ffn_gate": 6, "ffn_up": 7, "ffn_down": 8, "output": 9}


def shapes(cfg):
    H, I, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    qd, kvd = cfg["heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    return {"token_embd": (V, H), "attn_q": (qd, H), "attn_k": (kvd, H), "attn_v": (kvd, H),
            "attn_output": (H, qd), "ffn_gate": (I, H), "ffn_up": (I, H), "ffn_down": (H, I),
            "output": (V, H)}


def dense_weights(cfg):
    """name -> f32 [N, K] filled by the reference LCG."""
    return {n: synth.fill_f32(r * c, _SEEDS[n]).reshape(r, c) for n, (r, c) in shapes(cfg).items()}


def _canon(name):
    return f"{name}.weight" if name in ("token_embd", "output") else f"blk.0.{name}.weight"


def encoded_tensors(cfg, kind):
    """Raw checkpoint tensors of a tiny fixture. kind: 'f32' | 'gguf_mixed' | 'mlx_u4'.
    Returns canonical name -> dict(enc, shape, data[, scales, biases, aux, group])."""
    out = {}
    for n, w in dense_weights(cfg).items():
        r, c = w.shape
        if kind == "f32" or (kind == "gguf_mixed" and n == "token_embd"):
            t = dict(enc="plain.f32", data=w.astype(np.float32).tobytes())
        elif kind == "gguf_mixed":
            if n == "attn_q":
                t = dict(enc="gguf.q4_1", data=synth.pack_q4_1(w))
            elif n == "attn_v":
                t = dict(enc="gguf.q8_0", data=synth.pack_q8_0(w))
            else:
                t = dict(enc="gguf.q4_0", data=synth.pack_q4_0(w))
        elif kind == "mlx_u4":
            p, s, b = synth.quantize_affine_u4(w, r, c, 64)
            t = dict(enc="mlx.affine.u4", data=p.tobytes(), scales=s, biases=b, aux="plain.f32", group=64)
        else:
            raise ValueError(kind)
        t["shape"] = (r, c)
        out[_canon(n)] = t
    ones_h = np.ones(cfg["hidden"], np.float32)
    for n in ("blk.0.attn_norm.weight", "blk.0.ffn_norm.weight", "output_norm.weight"):
        out[n] = dict(enc="plain.f32", shape=(cfg["hidden"],), data=ones_h.tobytes())
    if cfg.get("qk_norm"):
        ones_d = np.ones(cfg["head_dim"], np.float32)
        for n in ("blk.0.attn_q_norm.weight", "blk.0.attn_k_norm.weight"):
            out[n] = dict(enc="plain.f32", shape=(cfg["head_dim"],), data=ones_d.tobytes())
    return out


# ---- the reference's round-trip formulas (reference.rs:106-193), used to dequantise
# ---- independently of any block decoder

def _rha(x):
    return np.sign(x) * np.floor(np.abs(x) + np.float32(0.5))


def q4_0_roundtrip(w):
    b = w.reshape(-1, 32).astype(np.float32)
    amax = np.abs(b).max(axis=1, keepdims=True)
    ps = np.where(amax > 0, amax / np.float32(7.0), 0).astype(np.float32)
    stored = ps.astype(np.float16).astype(np.float32)
    inv = np.where(ps > 0, np.float32(1.0) / np.where(ps > 0, ps, 1), 0).astype(np.float32)
    return (np.clip(_rha(b * inv), -8, 7).astype(np.float32) * stored).reshape(w.shape)


def q4_1_roundtrip(w):
    b = w.reshape(-1, 32).astype(np.float32)
    mn, mx = b.min(axis=1, keepdims=True), b.max(axis=1, keepdims=True)
    ps = np.where(mx > mn, (mx - mn) / np.float32(15.0), 0).astype(np.float32)
    ss, sm = ps.astype(np.float16).astype(np.float32), mn.astype(np.float16).astype(np.float32)
    inv = np.where(ps > 0, np.float32(1.0) / np.where(ps > 0, ps, 1), 0).astype(np.float32)
    q = np.clip(_rha((b - mn) * inv), 0, 15).astype(np.float32)
    return (q * ss + sm).astype(np.float32).reshape(w.shape)


def q8_0_roundtrip(w):
    b = w.reshape(-1, 32).astype(np.float32)
    amax = np.abs(b).max(axis=1, keepdims=True)
    ps = np.where(amax > 0, amax / np.float32(127.0), 0).astype(np.float32)
    stored = ps.astype(np.float16).astype(np.float32)
    inv = np.where(ps > 0, np.float32(1.0) / np.where(ps > 0, ps, 1), 0).astype(np.float32)
    return (np.clip(_rha(b * inv), -127, 127).astype(np.float32) * stored).reshape(w.shape)


def affine_u4_roundtrip(w, group=64):
    g = w.reshape(w.shape[0], -1, group).astype(np.float32)
    mn, mx = g.min(axis=2, keepdims=True), g.max(axis=2, keepdims=True)
    sc = np.maximum((mx - mn) / np.float32(15.0), np.float32(1e-7)).astype(np.float32)
    q = np.clip(_rha((g - mn) / sc), 0, 15).astype(np.float32)
    return (q * sc + mn).astype(np.float32).reshape(w.shape)


def roundtrip_weights(cfg, kind):
    w = dense_weights(cfg)
    if kind == "gguf_mixed":
        for n in w:
            if n == "token_embd":
                continue
            w[n] = {"attn_q": q4_1_roundtrip, "attn_v": q8_0_roundtrip}.get(n, q4_0_roundtrip)(w[n])
    elif kind == "mlx_u4":
        w = {n: affine_u4_roundtrip(v) for n, v in w.items()}
    return w


# ---- reference.rs:195-304 forward (one layer, no RoPE, MHA, -1e30 mask), numpy f32

def _rms(x, eps):
    ms = (x * x).sum(axis=-1, keepdims=True, dtype=np.float32) / np.float32(x.shape[-1])
    return x * (np.float32(1.0) / np.sqrt(ms + np.float32(eps)))


def reference_rs_forward(w, tokens, cfg=TINY):
    """Logits of the last row of the padded window `tokens`, as reference.rs computes them."""
    S, H, nh, d = len(tokens), cfg["hidden"], cfg["heads"], cfg["head_dim"]
    h = w["token_embd"][np.asarray(tokens)].astype(np.float32)
    xn = _rms(h, cfg["eps"])
    q, k, v = xn @ w["attn_q"].T, xn @ w["attn_k"].T, xn @ w["attn_v"].T
    ctx = np.zeros((S, H), np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(d)))
    for hd in range(nh):
        sl = slice(hd * d, (hd + 1) * d)
        s = (q[:, sl] @ k[:, sl].T) * scale
        s = np.where(np.triu(np.ones((S, S), bool), 1), np.float32(-1.0e30), s)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p = p / p.sum(axis=1, keepdims=True)
        ctx[:, sl] = p @ v[:, sl]
    h2 = h + ctx @ w["attn_output"].T
    fn = _rms(h2, cfg["eps"])
    g, u = fn @ w["ffn_gate"].T, fn @ w["ffn_up"].T
    ff = (g / (np.float32(1.0) + np.exp(-g))) * u
    h3 = h2 + ff @ w["ffn_down"].T
    ln = _rms(h3[-1:], cfg["eps"])
    return (ln @ w["output"].T)[0].astype(np.float32)
