"""Tensor-parallel prefill + greedy decode on a seeded synthetic checkpoint, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        --master-port P -m dyninfer_b200.tp_decode [--model tiny|0.6b-q4_0|8b-mixed|32b-q4_0]
        [--layers N] [--prompt 512] [--steps 64] [--batch 1] [--check]

Every rank opens the same checkpoint and uploads its own slices (consecutive rows of q/k/v, gate,
up and the lm_head; one span of every row of o_proj and down), then all ranks make the same calls:
the prompt is prefilled in chunks and `--steps` greedy steps follow. Each step sums the partial
o_proj / down products over the ranks (two all-reduces per layer) and gathers the logits slices.
`--layers` keeps the model's shapes but writes fewer layers (stated in the output).
`--check` also runs the unsharded model on rank 0's GPU and compares logits and tokens.
Rank 0 prints one JSON line; times are device-independent host clocks around synchronised calls,
the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import numpy as np

from . import replicas, synth
from .runtime import ModelLoader, SessionConfig

SEED = 4242


def _checkpoint(model: str, layers: int | None):
    d = os.environ.get("DYNINFER_BENCH_DIR") or os.path.join(tempfile.gettempdir(), "dyninfer_b200_bench")
    os.makedirs(d, exist_ok=True)
    base = {"tiny": synth.TINY, "0.6b-q4_0": synth.QWEN3_0_6B, "8b-mixed": synth.QWEN3_8B,
            "32b-q4_0": synth.QWEN3_32B}[model]
    cfg = dict(base)
    if layers:
        cfg["layers"] = layers
    path = os.path.join(d, f"tp_{model}_L{cfg['layers']}_seed{SEED}.gguf")
    kw = {}
    if model == "8b-mixed":
        kw = dict(encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"}, embd="gguf.q6_k", output="gguf.q6_k")
    elif model == "32b-q4_0":
        # every layer carries layer 0's bytes: 18 GB of distinct random blocks take minutes to draw
        kw = dict(embd="gguf.q6_k", output="gguf.q6_k", repeat_layers=True)
    return path, cfg, kw


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="0.6b-q4_0", choices=["tiny", "0.6b-q4_0", "8b-mixed", "32b-q4_0"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--kv-dtype", default="bf16")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="sum of the partial products: own peer-memory kernel, or NCCL all-reduce")
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("tensor-parallel decode needs CUDA devices: the cuda target has no CPU fallback")
    rank, local, world = replicas.world()
    torch.cuda.set_device(local)
    replicas.init("gloo")
    path, cfg, kw = _checkpoint(args.model, args.layers or None)
    if rank == 0 and not os.path.exists(path):
        tmp = path + f".tmp{os.getpid()}"
        synth.write_qwen3_gguf(tmp, cfg, seed=SEED, **kw)
        os.replace(tmp, path)
    replicas.barrier()
    max_seq = args.prompt + args.steps + args.warmup + 8
    t_load = time.perf_counter()
    model = ModelLoader().load(path, target=f"cuda:{local}", max_kv=max_seq, kv_dtype=args.kv_dtype,
                               chunk_size=args.chunk, tp=(rank, world), tp_exchange=args.exchange)
    rng = np.random.default_rng(SEED)
    prompts = [rng.integers(0, cfg["vocab"], size=args.prompt).tolist() for _ in range(args.batch)]
    result = {}
    with model.create_batched_session(SessionConfig(max_sequence_length=max_seq, batch_size=args.batch)) as s:
        torch.cuda.synchronize()
        load_s = time.perf_counter() - t_load
        s.prefill_slot(0, prompts[0])                      # untimed: first-use set-up
        replicas.barrier()
        t0 = time.perf_counter()
        feed = {slot: s.prefill_slot(slot, prompts[slot]) for slot in range(args.batch)}
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        first = dict(feed)
        produced = [[] for _ in range(args.batch)]
        for _ in range(args.warmup):
            feed = s.step(feed)
            for k, v in feed.items():
                produced[k].append(v)
        replicas.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            feed = s.step(feed)
            for k, v in feed.items():
                produced[k].append(v)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        wbytes = s.decode_weight_bytes()
        if args.check:   # logits of the prompt's last row and of one batched step, all ranks in step
            tp_lg, tp_tok = s.prefill_slot(0, prompts[0], want_logits=True)
            _, tp_step_lg = s.step({0: tp_tok}, want_logits=True)
    prefill_s, dt = replicas.max_over_ranks([prefill_s, dt])
    result.update({
        "workload": f"{args.model} ({cfg['layers']} layers), tensor parallel over {world} GPUs, prompt "
                    f"{args.prompt}, batch {args.batch}, greedy decode",
        "tp": world, "exchange": args.exchange, "batch": args.batch, "steps": args.steps,
        "prefill_tokens_per_s": round(args.batch * args.prompt / prefill_s, 1),
        "tokens_per_s": round(args.batch * args.steps / dt, 1), "ms_per_step": round(1e3 * dt / args.steps, 3),
        "weight_bytes_per_step_per_rank": int(wbytes),
        "weight_gbs_all_ranks": round(world * wbytes * args.steps / dt / 1e9, 1),
        "load_s": round(load_s, 1),
        "timing": "host clock around synchronised C-ABI calls, maximum over ranks",
    })
    if args.check:
        # every rank must have produced the same tokens; rank 0 compares with the unsharded model
        import torch.distributed as dist
        mine = torch.tensor([first[k] for k in sorted(first)] + [t for p in produced for t in p], dtype=torch.int64)
        theirs = [torch.zeros_like(mine) for _ in range(world)]
        if world > 1:
            dist.all_gather(theirs, mine)
        else:
            theirs = [mine]
        result["ranks_agree"] = bool(all(torch.equal(t, mine) for t in theirs))
        if rank == 0:
            ref = ModelLoader().load(path, target=f"cuda:{local}", max_kv=max_seq, kv_dtype=args.kv_dtype,
                                     chunk_size=args.chunk, decode_kernel="graph")
            with ref.create_batched_session(SessionConfig(max_sequence_length=max_seq,
                                                          batch_size=args.batch)) as r:
                rfeed = {slot: r.prefill_slot(slot, prompts[slot]) for slot in range(args.batch)}
                rfirst = dict(rfeed)
                rprod = [[] for _ in range(args.batch)]
                for _ in range(args.warmup + args.steps):
                    rfeed = r.step(rfeed)
                    for k, v in rfeed.items():
                        rprod[k].append(v)
                ref_lg, ref_tok = r.prefill_slot(0, prompts[0], want_logits=True)
                _, ref_step_lg = r.step({0: ref_tok}, want_logits=True)
            same = sum(int(a == b) for p, q in zip(produced, rprod) for a, b in zip(p, q))
            total = sum(len(p) for p in produced)
            # greedy paths may part at a near-tie; count the common prefix per sequence
            prefix = []
            for p, q in zip(produced, rprod):
                n = 0
                while n < len(p) and p[n] == q[n]:
                    n += 1
                prefix.append(n)
            result["check"] = {"first_tokens_equal": first == rfirst, "tokens_equal": same, "tokens": total,
                               "common_prefix_per_sequence": prefix,
                               "prefill_logits_max_abs_diff": float(np.abs(tp_lg - ref_lg).max()),
                               "step_logits_max_abs_diff": float(np.abs(tp_step_lg[0] - ref_step_lg[0]).max()),
                               "logits_max_abs": float(np.abs(ref_lg).max())}
    if rank == 0:
        print(json.dumps(result), flush=True)
    replicas.shutdown()


if __name__ == "__main__":
    main()
