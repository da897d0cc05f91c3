"""Single operators of the path, called through the C ABI on torch CUDA tensors.

torch is used only to own device memory and the stream; every computation is a
call into libdyninfer_cuda. There is no eager/PyTorch implementation behind
these functions: without the library or without a GPU they raise.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import ENC, check, lib


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _dev(a, device="cuda"):
    if isinstance(a, torch.Tensor):
        return a.to(device).contiguous()
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


class DeviceWeight:
    """One [rows, cols] parameter resident on the GPU as its verbatim checkpoint bytes."""

    def __init__(self, encoding: str, rows: int, cols: int, data, scales=None, biases=None,
                 aux: str = "plain.bf16", group: int = 64, device="cuda"):
        self.encoding, self.rows, self.cols, self.group, self.aux = encoding, int(rows), int(cols), int(group), aux
        raw = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray, memoryview)) \
            else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        need = lib().dyninfer_cuda_row_bytes(ENC[encoding], cols) * rows
        if raw.size != need:
            raise ValueError(f"{encoding} [{rows},{cols}] needs {need} bytes, got {raw.size}")
        # 64 bytes of readable slack behind the range, as the session arena provides
        buf = torch.zeros(raw.size + 64, dtype=torch.uint8, device=device)
        buf[:raw.size] = torch.from_numpy(raw.copy())
        self.data = buf
        self.scales = _dev(np.ascontiguousarray(scales).view(np.uint8).reshape(-1), device) if scales is not None else None
        self.biases = _dev(np.ascontiguousarray(biases).view(np.uint8).reshape(-1), device) if biases is not None else None
        self.nbytes = raw.size + (self.scales.numel() if self.scales is not None else 0) + \
            (self.biases.numel() if self.biases is not None else 0)

    def c(self) -> _lib.Weight:
        return _lib.Weight(ENC[self.encoding], ENC.get(self.aux, 2), self.group, 0, self.rows,
                           self.cols, _p(self.data), _p(self.scales), _p(self.biases))


def dequant(w: DeviceWeight) -> torch.Tensor:
    out = torch.empty((w.rows, w.cols), dtype=torch.float32, device=w.data.device)
    cw = w.c()
    check(lib().dyninfer_cuda_dequant(C.byref(cw), _p(out), _stream()))
    return out


def embedding_gather(w: DeviceWeight, tokens: torch.Tensor) -> torch.Tensor:
    tokens = tokens.to(device=w.data.device, dtype=torch.int64).contiguous()
    out = torch.empty((tokens.numel(), w.cols), dtype=torch.float32, device=w.data.device)
    cw = w.c()
    check(lib().dyninfer_cuda_embedding_gather(C.byref(cw), _p(tokens), tokens.numel(), _p(out), _stream()))
    return out


def linear(w: DeviceWeight, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("x must be float32 or bfloat16")
    x = x.contiguous().view(-1, w.cols)
    m = x.shape[0]
    if out is None:
        out = torch.empty((m, w.rows), dtype=torch.float32, device=x.device)
    cw = w.c()
    xt = ENC["plain.f32"] if x.dtype == torch.float32 else ENC["plain.bf16"]
    check(lib().dyninfer_cuda_linear(C.byref(cw), _p(x), xt, m, _p(out), _stream()))
    return out


_WT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.contiguous()
    width = w.numel()
    y = torch.empty_like(x)
    check(lib().dyninfer_cuda_rms_norm(_p(x), _p(w.contiguous()), _WT[w.dtype], x.numel() // width,
                                       width, float(eps), _p(y), _stream()))
    return y


def rope(x: torch.Tensor, start_pos: int, theta: float) -> torch.Tensor:
    y = x.contiguous().clone()
    s, h, d = y.shape
    check(lib().dyninfer_cuda_rope(_p(y), s, h, d, int(start_pos), float(theta), _stream()))
    return y


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    gate, up = gate.contiguous(), up.contiguous()
    y = torch.empty_like(gate)
    check(lib().dyninfer_cuda_silu_mul(_p(gate), _p(up), gate.numel(), _p(y), _stream()))
    return y


def attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, start_pos: int) -> torch.Tensor:
    """q [s, heads, d] f32; caches [kv_heads, cap, d] (f32/f16/bf16) holding rows < start_pos + s."""
    q = q.contiguous()
    s, nh, d = q.shape
    nkv, cap, _ = kcache.shape
    ctx = torch.empty((s, nh * d), dtype=torch.float32, device=q.device)
    check(lib().dyninfer_cuda_attention(_p(q), _p(kcache.contiguous()), _p(vcache.contiguous()),
                                        _WT[kcache.dtype], s, nh, nkv, d, cap, int(start_pos),
                                        _p(ctx), _stream()))
    return ctx


def argmax(v: torch.Tensor) -> int:
    v = v.contiguous().view(-1)
    out = torch.empty(1, dtype=torch.int64, device=v.device)
    scratch = torch.empty(lib().dyninfer_cuda_argmax_scratch_bytes(v.numel()), dtype=torch.uint8,
                          device=v.device)
    check(lib().dyninfer_cuda_argmax(_p(v), v.numel(), _p(out), _p(scratch), _stream()))
    return int(out.item())


def check_device_error():
    """Call after synchronising: raises when a kernel's bounded wait (weight ring, GEMM pipeline)
    expired since the last check, in which case the results produced since then are invalid."""
    check(lib().dyninfer_cuda_check_device_error())
