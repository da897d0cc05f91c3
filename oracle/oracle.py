"""ctypes binding of the CPU oracle (oracle/dyninfer_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py. The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

F32, F16, BF16, Q4_0, Q4_1, Q8_0, Q6_K, MLX_U4, Q4_K, Q5_K, IQ4_XS = range(11)
ENC_BY_NAME = {
    "plain.f32": F32, "plain.f16": F16, "plain.bf16": BF16,
    "gguf.q4_0": Q4_0, "gguf.q4_1": Q4_1, "gguf.q8_0": Q8_0, "gguf.q6_k": Q6_K,
    "mlx.affine.u4": MLX_U4, "gguf.q4_k": Q4_K, "gguf.q5_k": Q5_K, "gguf.iq4_xs": IQ4_XS,
}


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc + OpenMP)."""
    src = os.path.join(_HERE, "dyninfer_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


class Tensor(C.Structure):
    _fields_ = [
        ("enc", C.c_int32), ("aux_enc", C.c_int32), ("group", C.c_int32), ("pad_", C.c_int32),
        ("rows", C.c_int64), ("cols", C.c_int64),
        ("data", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
    ]


class Config(C.Structure):
    _fields_ = [
        ("layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32),
        ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("inter", C.c_int32),
        ("vocab", C.c_int32), ("has_qk_norm", C.c_int32), ("has_rope", C.c_int32),
        ("kv_round", C.c_int32), ("linear_mode", C.c_int32), ("page", C.c_int32),
        ("eps", C.c_float), ("theta", C.c_float), ("kv_cap", C.c_int64),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.orc_row_bytes.restype = C.c_int64
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.orc_dequant.argtypes = [C.POINTER(Tensor), C.c_void_p]
        L.orc_dequant_row.argtypes = [C.POINTER(Tensor), C.c_int64, C.c_void_p]
        L.orc_linear.argtypes = [C.POINTER(Tensor), C.c_void_p, C.c_int64, C.c_void_p, C.c_int]
        L.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]
        L.orc_rope.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float]
        L.orc_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_argmax.restype = C.c_int64
        L.orc_argmax.argtypes = [C.c_void_p, C.c_int64]
        L.orc_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int64] * 8 + [C.c_void_p]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.POINTER(Config), C.POINTER(Tensor)]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_model_reset.argtypes = [C.c_void_p]
        L.orc_model_forward.restype = C.c_int64
        L.orc_model_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_void_p, C.c_void_p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Weight:
    """One [rows, cols] parameter held as its verbatim checkpoint bytes."""

    def __init__(self, enc, rows, cols, data, scales=None, biases=None, aux_enc=BF16, group=64):
        self.enc = ENC_BY_NAME[enc] if isinstance(enc, str) else int(enc)
        self.rows, self.cols = int(rows), int(cols)
        self.data = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1))
        self.scales = None if scales is None else np.ascontiguousarray(scales).view(np.uint8).reshape(-1)
        self.biases = None if biases is None else np.ascontiguousarray(biases).view(np.uint8).reshape(-1)
        self.aux_enc = ENC_BY_NAME[aux_enc] if isinstance(aux_enc, str) else int(aux_enc)
        self.group = int(group)
        expect = lib().orc_row_bytes(self.enc, self.cols) * self.rows
        if self.data.size != expect:
            raise ValueError(f"weight bytes {self.data.size} != expected {expect}")

    def c(self) -> Tensor:
        return Tensor(self.enc, self.aux_enc, self.group, 0, self.rows, self.cols,
                      _ptr(self.data), _ptr(self.scales), _ptr(self.biases))


def dequant(w: Weight) -> np.ndarray:
    out = np.empty((w.rows, w.cols), dtype=np.float32)
    t = w.c()
    lib().orc_dequant(C.byref(t), _ptr(out))
    return out


def dequant_row(w: Weight, row: int) -> np.ndarray:
    out = np.empty((w.cols,), dtype=np.float32)
    t = w.c()
    lib().orc_dequant_row(C.byref(t), int(row), _ptr(out))
    return out


def linear(w: Weight, x: np.ndarray, fast: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, w.cols)
    y = np.empty((x.shape[0], w.rows), dtype=np.float32)
    t = w.c()
    lib().orc_linear(C.byref(t), _ptr(x), x.shape[0], _ptr(y), 1 if fast else 0)
    return y


def rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    H = w.shape[0]
    y = np.empty_like(x)
    lib().orc_rms_norm(_ptr(x), _ptr(w), x.size // H, H, float(eps), _ptr(y))
    return y


def rope(x, start_pos, theta):
    """x: [s, heads, d] -> rotated copy."""
    y = np.array(x, dtype=np.float32, order="C", copy=True)
    s, h, d = y.shape
    lib().orc_rope(_ptr(y), s, h, d, int(start_pos), float(theta))
    return y


def silu_mul(gate, up):
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    y = np.empty_like(gate)
    lib().orc_silu_mul(_ptr(gate), _ptr(up), gate.size, _ptr(y))
    return y


def argmax(v) -> int:
    v = np.ascontiguousarray(v, dtype=np.float32)
    return int(lib().orc_argmax(_ptr(v), v.size))


def attention(q, kcache, vcache, start, valid, page=256):
    """q [s, nh, d]; caches [nkv, kv_cap, d] (already holding rows < start+valid)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kcache = np.ascontiguousarray(kcache, dtype=np.float32)
    vcache = np.ascontiguousarray(vcache, dtype=np.float32)
    s, nh, d = q.shape
    nkv, cap, _ = kcache.shape
    ctx = np.empty((s, nh * d), dtype=np.float32)
    lib().orc_attention(_ptr(q), _ptr(kcache), _ptr(vcache), s, nh, nkv, d, cap, int(start),
                        int(valid), int(page), _ptr(ctx))
    return ctx


LAYER_SLOTS = ["attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "attn_q_norm",
               "attn_k_norm", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"]


class Model:
    """Whole decoder on the CPU. `weights` maps GGUF-style names to Weight."""

    def __init__(self, cfg: dict, weights: dict, kv_cap: int, kv_round: int = 0,
                 fast: bool = False, page: int = 256):
        self.cfg = cfg
        self._keep = weights
        L = cfg["layers"]
        tens = (Tensor * (3 + 11 * L))()
        head = weights.get("output.weight", weights["token_embd.weight"])  # tied: naming.rs:70-96
        tens[0] = weights["token_embd.weight"].c()
        tens[1] = weights["output_norm.weight"].c()
        tens[2] = head.c()
        ones = None
        for l in range(L):
            for j, slot in enumerate(LAYER_SLOTS):
                w = weights.get(f"blk.{l}.{slot}.weight")
                if w is None:
                    if ones is None:
                        ones = Weight(F32, 1, cfg["head_dim"], np.ones(cfg["head_dim"], np.float32))
                        self._ones = ones
                    w = ones
                tens[3 + l * 11 + j] = w.c()
        self.c = Config(L, cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"],
                        cfg["intermediate"], cfg["vocab"], int(cfg.get("qk_norm", True)),
                        int(cfg.get("rope", True)), int(kv_round), 1 if fast else 0, int(page),
                        float(cfg["eps"]), float(cfg.get("theta", 10000.0)), int(kv_cap))
        self._tens = tens
        self.h = lib().orc_model_create(C.byref(self.c), tens)
        self.position = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_model_destroy(self.h)
            self.h = None

    def reset(self):
        lib().orc_model_reset(self.h)
        self.position = 0

    def forward(self, tokens, start_pos=None, last=None, want_hidden=False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        n = tokens.size
        start = self.position if start_pos is None else int(start_pos)
        last = n - 1 if last is None else int(last)
        logits = np.empty((self.cfg["vocab"],), dtype=np.float32)
        hid = np.empty((n, self.cfg["hidden"]), dtype=np.float32) if want_hidden else None
        tok = lib().orc_model_forward(self.h, _ptr(tokens), n, start, last, _ptr(logits), _ptr(hid))
        self.position = start + n
        if want_hidden:
            return logits, int(tok), hid
        return logits, int(tok)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """Use `n` OpenMP threads from now on, whatever OMP_NUM_THREADS said when the runtime loaded."""
    lib().orc_set_num_threads(int(n))
    return num_threads()


def weights_from_catalog(cat) -> dict:
    """Oracle weights built from a checkpoint catalog's byte ranges — the same bytes the
    GPU session uploads. Norm vectors are widened exactly to f32."""
    blobs = [np.fromfile(p, dtype=np.uint8) for p in cat.files]
    out = {}
    for name, p in cat.parameters.items():
        comp = {c.name: blobs[c.source_file_index][c.offset:c.offset + c.length] for c in p.components}
        shape = p.shape
        rows, cols = (shape if len(shape) == 2 else (1, shape[0]))
        if p.encoding == "mlx.affine.u4":
            out[name] = Weight(p.encoding, rows, cols, comp["packed"], comp["scales"], comp["biases"],
                               p.components[1].type_name, p.group)
            continue
        enc, data = p.encoding, comp["data"]
        if len(shape) == 1 and enc != "plain.f32":
            if enc == "plain.bf16":
                data = (data.view(np.uint16).astype(np.uint32) << 16).view(np.float32).view(np.uint8)
            else:
                data = data.view(np.float16).astype(np.float32).view(np.uint8)
            enc = "plain.f32"
        out[name] = Weight(enc, rows, cols, data)
    return out
