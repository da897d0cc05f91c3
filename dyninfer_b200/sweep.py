"""Single-operator sweep of the fused dequant products (the reference has no equivalent tool; the
shapes, encodings and value distributions are the ones the direct path meets in Qwen3-class models).

    python -m dyninfer_b200.sweep [--enc gguf.q4_0,...] [--m 1,8,64,512] [--shapes 151936x1024,...]

For every (encoding, N x K, M) it times `ops.linear` (C ABI `dyninfer_cuda_linear`) with bf16
activations ~N(0,1) on seeded synthetic weights and prints one JSON line:
weight GB/s (weight bytes / time, against the HBM roofline) and, for M >= 64, TFLOP/s (2*M*N*K).
Timing: CUDA events around `reps` back-to-back calls after warm-up; a 512 MB buffer is rewritten
before each timed batch so that weights smaller than L2 do not stay cached between batches.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import ops, synth

SHAPES = [(3072, 1024), (1024, 3072), (151936, 1024), (12288, 4096), (4096, 12288)]
ENCODINGS = ["gguf.q4_0", "gguf.q4_1", "gguf.q8_0", "gguf.q6_k", "mlx.affine.u4"]


def make_weight(enc: str, n: int, k: int, seed: int = 1) -> ops.DeviceWeight:
    t = synth.random_weight(enc, n, k, seed)
    if enc == "mlx.affine.u4":
        return ops.DeviceWeight(enc, n, k, t["packed"], t["scales"], t["biases"], "plain.bf16", 64)
    return ops.DeviceWeight(enc, n, k, t["data"])


def time_linear(w: ops.DeviceWeight, m: int, batches: int = 5, reps: int = 4, flush=None) -> float:
    """Median over `batches` of the mean time (ms) of `reps` back-to-back products."""
    x = torch.randn(m, w.cols, device="cuda").to(torch.bfloat16)
    y = torch.empty(m, w.rows, device="cuda")
    for _ in range(3):
        ops.linear(w, x, out=y)
    times = []
    for _ in range(batches):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            ops.linear(w, x, out=y)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return statistics.median(times)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--enc", default=",".join(ENCODINGS))
    ap.add_argument("--m", default="1,8,64,512")
    ap.add_argument("--shapes", default=",".join(f"{n}x{k}" for n, k in SHAPES))
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device: the cuda target has no CPU fallback")
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    shapes = [tuple(int(v) for v in s.split("x")) for s in args.shapes.split(",")]
    for enc in args.enc.split(","):
        for n, k in shapes:
            w = make_weight(enc, n, k)
            for m in (int(v) for v in args.m.split(",")):
                ms = time_linear(w, m, flush=flush)
                line = {"enc": enc, "N": n, "K": k, "M": m, "us": round(ms * 1e3, 2),
                        "weight_gbs": round(w.nbytes / ms / 1e6, 1)}
                if m >= 64:
                    line["tflops"] = round(2.0 * m * n * k / ms / 1e9, 1)
                print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
