"""Independent numpy restatement of the block decoders (second opinion for the C oracle).

Follows crates/dyninfer-quantization/src/quantizations/gguf_codegen.rs:382-526 and
mlx_affine.rs:284-290,590-600 of the reference."""
import numpy as np


def _f16(b):  # uint8[..., 2] -> f32
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)[..., 0]


def dequant(enc, raw, rows, cols, scales=None, biases=None, group=64):
    raw = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.view(np.uint8).reshape(-1)
    if enc == "gguf.q4_0":
        b = raw.reshape(-1, 18)
        d = _f16(b[:, :2])[:, None]
        q = b[:, 2:]
        lo = (q & 15).astype(np.int32) - 8
        hi = (q >> 4).astype(np.int32) - 8
        w = np.concatenate([lo, hi], axis=1).astype(np.float32) * d
    elif enc == "gguf.q4_1":
        b = raw.reshape(-1, 20)
        d = _f16(b[:, :2])[:, None]
        m = _f16(b[:, 2:4])[:, None]
        q = b[:, 4:]
        w = np.concatenate([q & 15, q >> 4], axis=1).astype(np.float32) * d
        w = w + m
    elif enc == "gguf.q8_0":
        b = raw.reshape(-1, 34)
        d = _f16(b[:, :2])[:, None]
        w = b[:, 2:].view(np.int8).astype(np.float32) * d
    elif enc == "gguf.q6_k":
        b = raw.reshape(-1, 210)
        nb = b.shape[0]
        ql, qh = b[:, :128].reshape(nb, 2, 2, 32), b[:, 128:192].reshape(nb, 2, 32)
        sc = b[:, 192:208].view(np.int8).reshape(nb, 2, 2, 2, 2).astype(np.float32)  # n h p s
        d = _f16(b[:, 208:210])
        w = np.empty((nb, 2, 2, 2, 32), dtype=np.float32)  # n h p j
        for h in range(2):
            for p in range(2):
                lo = (ql[:, :, p, :] >> (4 * h)) & 15
                hi = (qh >> (2 * (h * 2 + p))) & 3
                q = lo.astype(np.int32) + 16 * hi.astype(np.int32) - 32
                s = np.repeat(sc[:, :, h, p, :], 16, axis=-1)
                w[:, :, h, p, :] = (q.astype(np.float32) * s) * d[:, None, None]
        w = w.reshape(nb, 256)
    elif enc in ("gguf.q4_k", "gguf.q5_k"):
        # GGML's published K-quant layout (schema-only in the reference): d, dmin f16; 12 bytes of
        # 6-bit scales / mins; Q5_K: 32 high-bit bytes; 128 nibble bytes
        five = enc == "gguf.q5_k"
        b = raw.reshape(-1, 176 if five else 144)
        nb = b.shape[0]
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        s = b[:, 4:16].astype(np.uint32)
        sc = np.empty((nb, 8), np.uint32)
        mn = np.empty((nb, 8), np.uint32)
        for j in range(8):
            if j < 4:
                sc[:, j], mn[:, j] = s[:, j] & 63, s[:, j + 4] & 63
            else:
                sc[:, j] = (s[:, j + 4] & 15) | ((s[:, j - 4] >> 6) << 4)
                mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
        qs = b[:, 48:176] if five else b[:, 16:144]
        qh = b[:, 16:48] if five else None
        w = np.empty((nb, 8, 32), np.float32)
        for j in range(8):
            q = (qs[:, 32 * (j // 2):32 * (j // 2) + 32] >> (4 * (j % 2))) & 15
            if five:
                q = q | (((qh >> j) & 1) << 4)
            ds = d * sc[:, j].astype(np.float32)
            dm = dmin * mn[:, j].astype(np.float32)
            w[:, j, :] = ds[:, None] * q.astype(np.float32) - dm[:, None]
        w = w.reshape(nb, 256)
    elif enc == "gguf.iq4_xs":
        # GGML's published layout (schema-only in the reference): d f16, scales_h u16, 4 bytes scales_l,
        # 128 index bytes; sub-block scale = 6 bits - 32, value = 16-entry table
        table = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
        b = raw.reshape(-1, 136)
        nb = b.shape[0]
        d = _f16(b[:, 0:2])
        sh = b[:, 2:4].copy().view(np.uint16).reshape(nb).astype(np.uint32)
        sl = b[:, 4:8].astype(np.uint32)
        qs = b[:, 8:136]
        w = np.empty((nb, 8, 32), np.float32)
        for ib in range(8):
            ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 15) | (((sh >> (2 * ib)) & 3) << 4)
            dl = d * (ls.astype(np.int32) - 32).astype(np.float32)
            q = qs[:, 16 * ib:16 * ib + 16]
            w[:, ib, :16] = dl[:, None] * table[q & 15]
            w[:, ib, 16:] = dl[:, None] * table[q >> 4]
        w = w.reshape(nb, 256)
    elif enc == "mlx.affine.u4":
        words = raw.view(np.uint32).reshape(rows, cols // 8)
        q = np.stack([(words >> np.uint32(4 * k)) & np.uint32(15) for k in range(8)], axis=-1)
        q = q.reshape(rows, cols // group, group).astype(np.float32)
        w = q * np.asarray(scales, np.float32).reshape(rows, -1, 1)
        w = w + np.asarray(biases, np.float32).reshape(rows, -1, 1)
    elif enc == "plain.f32":
        w = raw.view(np.float32)
    elif enc == "plain.f16":
        w = raw.view(np.float16).astype(np.float32)
    elif enc == "plain.bf16":
        w = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    else:
        raise ValueError(enc)
    return np.ascontiguousarray(w, dtype=np.float32).reshape(rows, cols)
