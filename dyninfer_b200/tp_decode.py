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


def run(model: str = "0.6b-q4_0", layers: int = 0, prompt: int = 512, steps: int = 64, warmup: int = 3,
        batch: int = 1, chunk: int = 512, kv_dtype: str = "bf16", exchange: str = "peer", check: bool = False,
        dump_logits: str = "", solo: bool = False) -> dict:
    """One tensor-parallel run over the ranks of the default process group (any backend that can move
    Python objects; the data path uses this library's own communicator). Every rank calls it with the
    same arguments (`check` and `dump_logits` add collective calls: a rank that leaves them out
    leaves the others waiting in the exchange); the returned dict is complete on rank 0. `solo`: this process alone runs the
    unsharded model on its own GPU, whatever the process group is (no collective is issued)."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("tensor-parallel decode needs CUDA devices: the cuda target has no CPU fallback")
    rank, local, world = replicas.world()
    if solo:
        rank, world = 0, 1
    sync = (lambda: None) if solo else replicas.barrier
    torch.cuda.set_device(local)
    path, cfg, kw = _checkpoint(model, layers or None)
    if rank == 0 and not os.path.exists(path):
        tmp = path + f".tmp{os.getpid()}"
        synth.write_qwen3_gguf(tmp, cfg, seed=SEED, **kw)
        os.replace(tmp, path)
    sync()
    max_seq = prompt + steps + warmup + 8
    t_load = time.perf_counter()
    tp = (rank, world) if world > 1 else None
    loaded = ModelLoader().load(path, target=f"cuda:{local}", max_kv=max_seq, kv_dtype=kv_dtype,
                                chunk_size=chunk, tp=tp, tp_exchange=exchange,
                                decode_kernel="graph")
    rng = np.random.default_rng(SEED)
    prompts = [rng.integers(0, cfg["vocab"], size=prompt).tolist() for _ in range(batch)]
    result = {}
    with loaded.create_batched_session(SessionConfig(max_sequence_length=max_seq, batch_size=batch)) as s:
        torch.cuda.synchronize()
        load_s = time.perf_counter() - t_load
        s.prefill_slot(0, prompts[0])                      # untimed: first-use set-up
        sync()
        s.timer_start()
        feed = {slot: s.prefill_slot(slot, prompts[slot]) for slot in range(batch)}
        prefill_s = s.timer_stop() / 1e3
        first = dict(feed)
        produced = [[] for _ in range(batch)]
        for _ in range(warmup):
            feed = s.step(feed)
            for k, v in feed.items():
                produced[k].append(v)
        sync()
        torch.cuda.synchronize()
        s.timer_start()
        for _ in range(steps):
            feed = s.step(feed)
            for k, v in feed.items():
                produced[k].append(v)
        dt = s.timer_stop() / 1e3
        wbytes = s.decode_weight_bytes()
        if check or dump_logits:   # logits of the prompt's last row and of one batched step, all ranks in step
            tp_lg, tp_tok = s.prefill_slot(0, prompts[0], want_logits=True)
            _, tp_step_lg = s.step({0: tp_tok}, want_logits=True)
            if dump_logits and rank == 0:
                np.savez(dump_logits, prompt=np.array(prompts[0], dtype=np.int64), prefill_logits=tp_lg,
                         first_token=np.int64(tp_tok), step_logits=tp_step_lg[0], checkpoint=np.array(path))
    dev = "cuda" if world > 1 else "cpu"
    if not solo:
        prefill_s, dt = replicas.max_over_ranks([prefill_s, dt], device=dev)
    result.update({
        "workload": f"{model} ({cfg['layers']} layers), tensor parallel over {world} GPUs, prompt "
                    f"{prompt}, batch {batch}, greedy decode",
        "tp": world, "exchange": exchange if world > 1 else "none", "batch": batch, "steps": steps,
        "prefill_tokens_per_s": round(batch * prompt / prefill_s, 1),
        "tokens_per_s": round(batch * steps / dt, 1), "ms_per_step": round(1e3 * dt / steps, 3),
        "weight_bytes_per_step_per_rank": int(wbytes),
        "weight_gbs_per_gpu": round(wbytes * steps / dt / 1e9, 1),
        "weight_gbs_all_ranks": round(world * wbytes * steps / dt / 1e9, 1),
        "load_s": round(load_s, 1),
        "timing": "CUDA events on each rank's session stream around the timed calls, maximum over ranks",
    })
    if check:
        # every rank must have produced the same tokens; rank 0 compares with the unsharded model
        import torch.distributed as dist
        mine = torch.tensor([first[k] for k in sorted(first)] + [t for p in produced for t in p], dtype=torch.int64,
                            device=dev)
        theirs = [torch.zeros_like(mine) for _ in range(world)]
        if world > 1:
            dist.all_gather(theirs, mine)
        else:
            theirs = [mine]
        result["ranks_agree"] = bool(all(torch.equal(t, mine) for t in theirs))
        if rank == 0:
            ref = ModelLoader().load(path, target=f"cuda:{local}", max_kv=max_seq, kv_dtype=kv_dtype,
                                     chunk_size=chunk, decode_kernel="graph")
            with ref.create_batched_session(SessionConfig(max_sequence_length=max_seq,
                                                          batch_size=batch)) as r:
                rfeed = {slot: r.prefill_slot(slot, prompts[slot]) for slot in range(batch)}
                rfirst = dict(rfeed)
                rprod = [[] for _ in range(batch)]
                for _ in range(warmup + steps):
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
    return result


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
    ap.add_argument("--dump-logits", default="",
                    help="rank 0 writes the prompt, the logits of its last row and of one step to this .npz")
    args = ap.parse_args()
    replicas.init("gloo")
    result = run(args.model, args.layers, args.prompt, args.steps, args.warmup, args.batch, args.chunk,
                 args.kv_dtype, args.exchange, args.check, args.dump_logits)
    if replicas.world()[0] == 0:
        print(json.dumps(result), flush=True)
    replicas.shutdown()


if __name__ == "__main__":
    main()
