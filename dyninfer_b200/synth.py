"""Seeded synthetic checkpoints in the on-disk formats the path consumes.

Two kinds of generator live here:

* the reference's own fixture packers, restated with numpy, which quantise a
  given f32 matrix (crates/dyninfer-checkpoint-gguf/src/q4.rs:16-98 for
  Q4_0 / Q4_1 / Q8_0, crates/dyninfer-checkpoint-safetensors/src/fixture.rs
  :287-317 for MLX affine U4);
* random raw-block generators with the value distributions the benchmark
  configurations state (uniform nibbles, f16 scale 0.0043*U(0.5,1.5), ...),
  which never build an f32 matrix and therefore scale to full-size models.

Everything is a pure function of a seed.
"""
from __future__ import annotations

import json
import os
import zlib

import numpy as np

from . import checkpoint as ck


# ------------------------------------------------------------ reference packers

def fill_f32(n: int, seed: int) -> np.ndarray:
    """The reference's fixture LCG: x = x*1664525 + 1013904223 + i (u32 wrap);
    v = (x % 1000)/1000 - 0.5. crates/dyninfer-checkpoint-gguf/src/q4.rs:212-223."""
    out = np.empty(n, dtype=np.float32)
    x = seed & 0xFFFFFFFF
    for i in range(n):
        x = (x * 1664525 + 1013904223 + i) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(x % 1000) / np.float32(1000.0)) - np.float32(0.5)
    return out


def _round_half_away(x):
    # Rust f32::round: half away from zero
    return np.sign(x) * np.floor(np.abs(x) + np.float32(0.5))


def pack_q4_0(w: np.ndarray) -> bytes:
    b = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(b).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(7.0), np.float32(0)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, 1), np.float32(0)).astype(np.float32)
    q = np.clip(_round_half_away(b * inv[:, None]).astype(np.int32), -8, 7) + 8
    out = np.empty((b.shape[0], 18), dtype=np.uint8)
    out[:, :2] = scale.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = (q[:, :16] | (q[:, 16:] << 4)).astype(np.uint8)
    return out.tobytes()


def pack_q4_1(w: np.ndarray) -> bytes:
    b = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    mn, mx = b.min(axis=1), b.max(axis=1)
    scale = np.where(mx > mn, (mx - mn) / np.float32(15.0), np.float32(0)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, 1), np.float32(0)).astype(np.float32)
    q = np.clip(_round_half_away((b - mn[:, None]) * inv[:, None]), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 20), dtype=np.uint8)
    out[:, 0:2] = scale.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = mn.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 4:] = q[:, :16] | (q[:, 16:] << 4)
    return out.tobytes()


def pack_q8_0(w: np.ndarray) -> bytes:
    b = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(b).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(0)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1.0) / np.where(scale > 0, scale, 1), np.float32(0)).astype(np.float32)
    q = np.clip(_round_half_away(b * inv[:, None]).astype(np.int32), -127, 127).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, :2] = scale.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def quantize_affine_u4(w: np.ndarray, rows: int, cols: int, group: int = 64):
    """-> (packed u32 [rows, cols/8], scales f32 [rows, cols/group], biases f32)."""
    g = np.asarray(w, dtype=np.float32).reshape(rows, cols // group, group)
    mn, mx = g.min(axis=2), g.max(axis=2)
    scale = np.maximum((mx - mn) / np.float32(15.0), np.float32(1.0e-7)).astype(np.float32)
    q = np.clip(_round_half_away((g - mn[..., None]) / scale[..., None]), 0, 15).astype(np.uint32)
    q = q.reshape(rows, cols // 8, 8)
    packed = np.zeros((rows, cols // 8), dtype=np.uint32)
    for lane in range(8):
        packed |= q[:, :, lane] << np.uint32(4 * lane)
    return packed, scale, mn.astype(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ------------------------------------------------------- random raw-block tensors

def tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0xFFFFFFFFFFFF


def random_weight(enc: str, rows: int, cols: int, seed: int, group: int = 64):
    """Random verbatim bytes for one [rows, cols] tensor with the stated distributions;
    dequantised values have std ~= 0.02. Returns dict component -> ndarray."""
    rng = np.random.default_rng(seed)
    if enc in ("gguf.q4_0", "gguf.q4_1", "gguf.q8_0"):
        nb = rows * cols // 32
        u = rng.uniform(0.5, 1.5, size=nb).astype(np.float32)
        if enc == "gguf.q4_0":
            blk = np.empty((nb, 18), dtype=np.uint8)
            d = (np.float32(0.0043) * u).astype(np.float16)
            blk[:, :2] = d.view(np.uint8).reshape(-1, 2)
            blk[:, 2:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
        elif enc == "gguf.q4_1":
            blk = np.empty((nb, 20), dtype=np.uint8)
            d = (np.float32(0.0043) * u).astype(np.float16)
            m = (np.float32(-8.0) * d.astype(np.float32)).astype(np.float16)
            blk[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
            blk[:, 2:4] = m.view(np.uint8).reshape(-1, 2)
            blk[:, 4:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
        else:
            blk = np.empty((nb, 34), dtype=np.uint8)
            d = (np.float32(0.02 / 73.3) * u).astype(np.float16)
            blk[:, :2] = d.view(np.uint8).reshape(-1, 2)
            blk[:, 2:] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
        return {"data": blk.reshape(-1)}
    if enc == "gguf.q6_k":
        nb = rows * cols // 256
        blk = np.empty((nb, 210), dtype=np.uint8)
        blk[:, :192] = rng.integers(0, 256, size=(nb, 192), dtype=np.uint8)
        blk[:, 192:208] = rng.integers(1, 64, size=(nb, 16), dtype=np.int8).view(np.uint8)
        # std(q-32) ~= 18.47, rms(sc) ~= 36.8 -> d ~= 0.02 / 680
        d = (np.float32(0.02 / 680.0) * rng.uniform(0.5, 1.5, size=nb).astype(np.float32)).astype(np.float16)
        blk[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
        return {"data": blk.reshape(-1)}
    if enc in ("gguf.q4_k", "gguf.q5_k"):
        # uniform nibble / high-bit / 6-bit scale and min bytes; f16 d, dmin sized for std ~= 0.02:
        # w = d*sc*q - dmin*m with sc, m ~ U[0,63], q ~ U[0,15] (U[0,31] for Q5_K)
        nb, bsz = rows * cols // 256, (144 if enc == "gguf.q4_k" else 176)
        blk = np.empty((nb, bsz), dtype=np.uint8)
        blk[:, 4:] = rng.integers(0, 256, size=(nb, bsz - 4), dtype=np.uint8)
        qmax = 15.0 if enc == "gguf.q4_k" else 31.0
        d = (np.float32(0.02 / (31.5 * qmax * 0.35)) * rng.uniform(0.5, 1.5, size=nb).astype(np.float32)).astype(np.float16)
        dmin = (d.astype(np.float32) * np.float32(qmax / 2)).astype(np.float16)     # centres the values near zero
        blk[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        blk[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
        return {"data": blk.reshape(-1)}
    if enc == "gguf.iq4_xs":
        # uniform 4-bit table indices and 6-bit sub-block scales; f16 d sized for std ~= 0.02:
        # w = d * (ls - 32) * table[q], rms(ls - 32) ~= 18.5, rms(table) ~= 69 (d lands among the f16
        # subnormals, as it does in real files)
        nb = rows * cols // 256
        blk = np.empty((nb, 136), dtype=np.uint8)
        blk[:, 2:] = rng.integers(0, 256, size=(nb, 134), dtype=np.uint8)
        d = (np.float32(0.02 / (18.5 * 69.0)) * rng.uniform(0.5, 1.5, size=nb).astype(np.float32)).astype(np.float16)
        blk[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        return {"data": blk.reshape(-1)}
    if enc == "mlx.affine.u4":
        packed = rng.integers(0, 2 ** 32, size=(rows, cols // 8), dtype=np.uint32)
        s = (np.float32(0.0043) * rng.uniform(0.5, 1.5, size=(rows, cols // group)).astype(np.float32))
        sb = f32_to_bf16_bits(s)
        bb = f32_to_bf16_bits(np.float32(-7.5) * bf16_bits_to_f32(sb))
        return {"packed": packed, "scales": sb, "biases": bb}
    if enc == "plain.bf16":
        return {"data": f32_to_bf16_bits(rng.normal(0.0, 0.02, size=(rows, cols)).astype(np.float32))}
    if enc == "plain.f16":
        return {"data": rng.normal(0.0, 0.02, size=(rows, cols)).astype(np.float16)}
    if enc == "plain.f32":
        return {"data": rng.normal(0.0, 0.02, size=(rows, cols)).astype(np.float32)}
    raise ValueError(f"no generator for {enc}")


# ----------------------------------------------------------------- whole models

QWEN3_0_6B = dict(layers=28, hidden=1024, heads=16, kv_heads=8, head_dim=128, intermediate=3072,
                  vocab=151936, eps=1e-6, theta=1e6)
QWEN3_8B = dict(layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128, intermediate=12288,
                vocab=151936, eps=1e-6, theta=1e6)
QWEN3_32B = dict(layers=64, hidden=5120, heads=64, kv_heads=8, head_dim=128, intermediate=25600,
                 vocab=151936, eps=1e-6, theta=1e6)
TINY = dict(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=512,
            vocab=512, eps=1e-6, theta=1e6)
# The smallest shapes the persistent decode kernel takes (a Q6_K table needs 1024-wide rows):
# two layers, head dim 128 / 64, a vocabulary that leaves some CTAs without lm_head rows.
SMALL_D128 = dict(layers=2, hidden=1024, heads=4, kv_heads=2, head_dim=128, intermediate=1536,
                  vocab=2048, eps=1e-6, theta=1e6)
SMALL_D64 = dict(layers=3, hidden=1024, heads=8, kv_heads=2, head_dim=64, intermediate=1024,
                 vocab=1000, eps=1e-6, theta=1e6)


def linear_shapes(cfg: dict) -> dict:
    H, I = cfg["hidden"], cfg["intermediate"]
    qd, kvd = cfg["heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    return {"attn_q": (qd, H), "attn_k": (kvd, H), "attn_v": (kvd, H), "attn_output": (H, qd),
            "ffn_gate": (I, H), "ffn_up": (I, H), "ffn_down": (H, I)}


def write_qwen3_gguf(path: str, cfg: dict, seed: int = 0, encodings: dict | None = None,
                     embd: str = "gguf.q6_k", output: str | None = None,
                     default: str = "gguf.q4_0", repeat_layers: bool = False) -> str:
    """Seeded Qwen3-shaped GGUF. `encodings` overrides the encoding per linear slot
    (e.g. {"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"}); `output`=None ties the
    lm_head to token_embd (no output.weight tensor). `repeat_layers` writes layer 0's bytes
    for every layer (each layer still has its own tensors and file ranges): the file is as large
    and is read exactly like one with distinct layers, but is generated in a fraction of the time,
    for throughput runs of the largest shapes."""
    enc = dict.fromkeys(linear_shapes(cfg), default)
    enc.update(encodings or {})
    a = "qwen3"
    meta = {
        "general.architecture": a, f"{a}.block_count": cfg["layers"],
        f"{a}.embedding_length": cfg["hidden"], f"{a}.feed_forward_length": cfg["intermediate"],
        f"{a}.attention.head_count": cfg["heads"], f"{a}.attention.head_count_kv": cfg["kv_heads"],
        f"{a}.attention.key_length": cfg["head_dim"], f"{a}.vocab_size": cfg["vocab"],
        f"{a}.attention.layer_norm_rms_epsilon": float(cfg["eps"]),
        f"{a}.rope.freq_base": float(cfg["theta"]), f"{a}.context_length": 40960,
    }
    t = {}

    def add(name, e, rows, cols):
        w = random_weight(e, rows, cols, tensor_seed(seed, name))["data"]
        t[name] = ((rows, cols), ck.GGML_CODE[e], w)

    add("token_embd.weight", embd, cfg["vocab"], cfg["hidden"])
    if output:
        add("output.weight", output, cfg["vocab"], cfg["hidden"])
    ones_h = np.ones(cfg["hidden"], np.float32)
    ones_d = np.ones(cfg["head_dim"], np.float32)
    t["output_norm.weight"] = ((cfg["hidden"],), 0, ones_h)
    for l in range(cfg["layers"]):
        for slot, (n, k) in linear_shapes(cfg).items():
            if repeat_layers and l > 0:
                t[f"blk.{l}.{slot}.weight"] = t[f"blk.0.{slot}.weight"]
            else:
                add(f"blk.{l}.{slot}.weight", enc[slot], n, k)
        t[f"blk.{l}.attn_norm.weight"] = ((cfg["hidden"],), 0, ones_h)
        t[f"blk.{l}.ffn_norm.weight"] = ((cfg["hidden"],), 0, ones_h)
        t[f"blk.{l}.attn_q_norm.weight"] = ((cfg["head_dim"],), 0, ones_d)
        t[f"blk.{l}.attn_k_norm.weight"] = ((cfg["head_dim"],), 0, ones_d)
    ck.write_gguf(path, meta, t)
    return path


_CANON_TO_HF = {v: k for k, v in ck._HF_LAYER.items()}


def write_qwen3_mlx(dirpath: str, cfg: dict, seed: int = 0, group: int = 64,
                    embed: str = "plain.bf16") -> str:
    """Seeded Qwen3-shaped MLX affine-U4 SafeTensors directory (model.safetensors +
    config.json), HF tensor names, bf16 scales/biases, tied bf16 embeddings."""
    os.makedirs(dirpath, exist_ok=True)
    t = {}
    dt = {"plain.bf16": "BF16", "plain.f16": "F16", "plain.f32": "F32"}
    e = random_weight(embed, cfg["vocab"], cfg["hidden"], tensor_seed(seed, "token_embd.weight"))
    t["model.embed_tokens.weight"] = (dt[embed], (cfg["vocab"], cfg["hidden"]), e["data"])
    ones_h = f32_to_bf16_bits(np.ones(cfg["hidden"], np.float32))
    ones_d = f32_to_bf16_bits(np.ones(cfg["head_dim"], np.float32))
    t["model.norm.weight"] = ("BF16", (cfg["hidden"],), ones_h)
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}."
        for slot, (n, k) in linear_shapes(cfg).items():
            w = random_weight("mlx.affine.u4", n, k, tensor_seed(seed, f"blk.{l}.{slot}.weight"), group)
            hf = p + _CANON_TO_HF[slot]
            t[hf + ".weight"] = ("U32", (n, k // 8), w["packed"])
            t[hf + ".scales"] = ("BF16", (n, k // group), w["scales"])
            t[hf + ".biases"] = ("BF16", (n, k // group), w["biases"])
        t[p + "input_layernorm.weight"] = ("BF16", (cfg["hidden"],), ones_h)
        t[p + "post_attention_layernorm.weight"] = ("BF16", (cfg["hidden"],), ones_h)
        t[p + "self_attn.q_norm.weight"] = ("BF16", (cfg["head_dim"],), ones_d)
        t[p + "self_attn.k_norm.weight"] = ("BF16", (cfg["head_dim"],), ones_d)
    ck.write_safetensors(os.path.join(dirpath, "model.safetensors"), t, {"format": "mlx"})
    hf_cfg = {
        "model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"],
        "num_hidden_layers": cfg["layers"], "hidden_size": cfg["hidden"],
        "intermediate_size": cfg["intermediate"], "num_attention_heads": cfg["heads"],
        "num_key_value_heads": cfg["kv_heads"], "head_dim": cfg["head_dim"],
        "vocab_size": cfg["vocab"], "rms_norm_eps": cfg["eps"], "rope_theta": cfg["theta"],
        "max_position_embeddings": 40960, "tie_word_embeddings": True,
        "quantization": {"group_size": group, "bits": 4},
    }
    with open(os.path.join(dirpath, "config.json"), "w") as f:
        json.dump(hf_cfg, f)
    return dirpath
