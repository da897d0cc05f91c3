"""Batched prefill + greedy decode benchmark on seeded synthetic checkpoints, bf16 KV cache.

    python -m dyninfer_b200.batched_decode [--model 0.6b-mlx|8b-mixed|0.6b-q4_0] [--batch 1,8,32,64]
                                           [--prompt 512] [--steps 256] [--chunk 512]

Models: `0.6b-mlx` = Qwen3-0.6B shape, MLX affine-U4 linears (group 64, bf16 scales and biases), tied
bf16 embeddings, SafeTensors; `8b-mixed` = Qwen3-8B shape GGUF with q/k/o/gate/up Q4_0, attn_v Q4_1,
ffn_down Q8_0, token_embd and output Q6_K (untied); `0.6b-q4_0` = the headline decode model.

For every batch size B: B sequences are prefilled with `--prompt` random token ids each (timed, one
sequence after the other, in chunks of `--chunk` rows),
then `--steps` greedy steps decode all of them together (`dyninfer_cuda_session_decode_batch`: one
pass over the weights per step, attention per sequence). Prints one JSON line per batch size:
tokens/s over all sequences, ms per step, and the weight bytes one step reads per second
(weight GB/s; the KV cache traffic, which grows with batch x context, is reported next to it).
All inputs are synthetic and seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import numpy as np

from . import synth
from .runtime import ModelLoader, SessionConfig

SEED = 20242


def checkpoint(model: str):
    """(path, config) of the seeded checkpoint for `model`, written on first use."""
    d = os.environ.get("DYNINFER_BENCH_DIR") or os.path.join(tempfile.gettempdir(), "dyninfer_b200_bench")
    os.makedirs(d, exist_ok=True)
    if model == "0.6b-mlx":
        path = os.path.join(d, f"qwen3_0_6b_mlx_u4_seed{SEED}")
        if not os.path.exists(os.path.join(path, "model.safetensors")):
            tmp = path + f".tmp{os.getpid()}"
            synth.write_qwen3_mlx(tmp, synth.QWEN3_0_6B, seed=SEED)
            os.replace(tmp, path)
        return path, synth.QWEN3_0_6B
    if model == "8b-mixed":
        path = os.path.join(d, f"qwen3_8b_mixed_seed{SEED}.gguf")
        if not os.path.exists(path):
            tmp = path + f".tmp{os.getpid()}"
            synth.write_qwen3_gguf(tmp, synth.QWEN3_8B, seed=SEED,
                                   encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"},
                                   embd="gguf.q6_k", output="gguf.q6_k")
            os.replace(tmp, path)
        return path, synth.QWEN3_8B
    if model == "0.6b-q4_0":
        path = os.path.join(d, f"qwen3_0_6b_q4_0_seed{SEED}.gguf")
        if not os.path.exists(path):
            tmp = path + f".tmp{os.getpid()}"
            synth.write_qwen3_gguf(tmp, synth.QWEN3_0_6B, seed=SEED)
            os.replace(tmp, path)
        return path, synth.QWEN3_0_6B
    raise SystemExit(f"unknown model {model!r}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="0.6b-mlx", choices=["0.6b-mlx", "8b-mixed", "0.6b-q4_0"])
    ap.add_argument("--chunk", type=int, default=512, help="prefill chunk size (rows per forward call)")
    ap.add_argument("--batch", default="1,8,32,64")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("the benchmark needs a CUDA device: the cuda target has no CPU fallback")
    path, cfg = checkpoint(args.model)
    max_seq = args.prompt + args.steps + args.warmup + 8
    for b in (int(v) for v in args.batch.split(",")):
        model = ModelLoader().load(path, max_kv=max_seq, kv_dtype="bf16", chunk_size=args.chunk)
        rng = np.random.default_rng(SEED + b)
        with model.create_batched_session(SessionConfig(max_sequence_length=max_seq, batch_size=b)) as s:
            feed = {}
            prompts = [rng.integers(0, cfg["vocab"], size=args.prompt).tolist() for _ in range(b)]
            s.prefill_slot(0, prompts[0])                      # untimed: first-use set-up
            torch.cuda.synchronize()
            tp0 = time.perf_counter()
            for slot in range(b):
                feed[slot] = s.prefill_slot(slot, prompts[slot])
            torch.cuda.synchronize()
            prefill_s = time.perf_counter() - tp0
            for _ in range(args.warmup):
                feed = s.step(feed)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                feed = s.step(feed)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            wbytes = s.decode_weight_bytes()
            ctx = args.prompt + args.warmup + args.steps / 2
            kv_bytes = 2 * cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * 2 * ctx * b   # K and V, bf16
            print(json.dumps({
                "workload": f"{args.model}: prefill of batch x prompt tokens, then batched greedy decode",
                "batch": b, "prompt": args.prompt, "steps": args.steps, "chunk": args.chunk,
                "prefill_tokens_per_s": round(b * args.prompt / prefill_s, 1),
                "tokens_per_s": round(b * args.steps / dt, 1), "ms_per_step": round(1e3 * dt / args.steps, 3),
                "weight_bytes_per_step": int(wbytes), "weight_gbs": round(wbytes * args.steps / dt / 1e9, 1),
                "kv_bytes_per_step_mid_run": int(kv_bytes),
                "timing": "host clock around the C-ABI calls, tokens in and out through host memory every step",
            }), flush=True)


if __name__ == "__main__":
    main()
