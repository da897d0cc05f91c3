#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode of the Qwen3-0.6B-shape Q4_0 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one decode step (one generated token) of the seeded synthetic
checkpoint (all linears Q4_0, tied Q6_K embedding / lm_head, GGUF v3). The K timed
steps are laid out the way the reference's perf runner lays out its iterations
(crates/dyninfer-runtime/src/perf.rs:92-172): reset, prefill of the 16-token
prompt (untimed), 32 greedy steps (timed), again until K steps are timed, so every
timed step runs at the contexts of the named configuration (16 .. 48).
Prints ONE JSON line on rank 0.

  value     decode tok/s with everything resident in HBM: the persistent decode kernel
            with the argmax fed back on the device (16 tokens per launch), timed with
            CUDA events on the session stream, summed over the decode phases (max over
            ranks).
  e2e       the same K steps through the public session call `decode_argmax`
            (C ABI `dyninfer_cuda_session_invoke_paged_chunk`): host token in from
            pinned memory, argmax token out, every step; host clock around each decode
            phase with a device synchronisation on both sides.
  roofline  the persistent decode kernel (the only kernel in the timed region): the
            weight bytes one token reads / its average launch time, against the
            measured HBM copy bandwidth. `roofline_lm_head_gemv` adds the largest
            single product (151936 x 1024 Q6_K) as a stand-alone fused dequant-GEMV
            launch, timed alone with CUDA events over back-to-back launches (its 127.6 MB
            of weights exceed L2).
  cpu_baseline  the CPU restatement of the reference's direct path (oracle/) on the
            host cores, on a bounded sample of the same workload (one-GPU run only; the same
            sample checks the timed loop's first tokens, key `parity`).

With N > 1 every rank runs an independent replica of the model on its own GPU
(the 0.6B path does not shard; there is no data-path collective), so the value is
N x the per-replica rate over the slowest rank: weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "qwen3-0.6b-shape q4_0 (tied q6_k lm_head), batch 1, prompt 16, greedy decode"
PROMPT_LEN = 16
GEN_STEPS = 32           # greedy steps per generation of the named configuration
SEED = 20240


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6),
                              ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_mega_kernel launch on this workload,
# recorded from an ncu capture of this kernel (a profiler cannot run inside the timed region); the
# bench line labels it as recorded, not measured in this run
MEGA_DRAM_TRAFFIC = 381_600_640 + 4_658_560


def phases(n):
    """n decode steps as decode phases of at most GEN_STEPS steps, each after its own prompt."""
    return [GEN_STEPS] * (n // GEN_STEPS) + ([n % GEN_STEPS] if n % GEN_STEPS else [])


def checkpoint_path():
    d = os.environ.get("DYNINFER_BENCH_DIR") or os.path.join(tempfile.gettempdir(), "dyninfer_b200_bench")
    os.makedirs(d, exist_ok=True)
    return os.path.join(d, f"qwen3_0_6b_q4_0_seed{SEED}.gguf")


def ensure_checkpoint():
    from dyninfer_b200 import synth
    path = checkpoint_path()
    if not os.path.exists(path):
        tmp = path + f".tmp{os.getpid()}"
        synth.write_qwen3_gguf(tmp, synth.QWEN3_0_6B, seed=SEED)
        os.replace(tmp, path)
    return path


def prompt_ids():
    from dyninfer_b200 import synth
    return np.random.default_rng(SEED).integers(0, synth.QWEN3_0_6B["vocab"], size=PROMPT_LEN).tolist()


# ------------------------------------------------------------------ CPU restatement

def use_all_host_threads():
    """The CPU restatement runs on every core this process may use, whatever OMP_NUM_THREADS the
    launcher exported (torch.distributed.run sets it to 1). Must run before the library loads."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    # a container's CPU quota can be smaller than its affinity mask; threads beyond the quota only
    # spin against the throttle
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()[:2]
        if quota != "max":
            n = min(n, max(1, int(quota) // int(period)))
    except (OSError, ValueError):
        pass
    os.environ["OMP_NUM_THREADS"] = str(max(1, n))
    return n


def cpu_decode(path, steps, warm=1, kv_round=2):
    """The CPU restatement (all host threads) on the bench workload: the same 16-token prompt, then
    greedy steps. Returns (decode tok/s over `steps` timed steps, threads, seconds, tokens, margins):
    tokens[0] follows the prompt, tokens[1 + i] follows decode step i (warm-up steps included);
    margins[i] is the top-2 logit gap behind tokens[i]."""
    cores = use_all_host_threads()
    from oracle import oracle as orc
    from dyninfer_b200 import checkpoint as ck
    orc.build()
    orc.set_num_threads(cores)                     # the OpenMP runtime may have loaded before the env change
    cat = ck.open_catalog(path)
    m = orc.Model(cat.config, orc.weights_from_catalog(cat), kv_cap=PROMPT_LEN + steps + warm + 2,
                  kv_round=kv_round, fast=True)

    def margin(lg):
        top2 = np.partition(lg, -2)[-2:]
        return float(top2[1] - top2[0])

    lg, tok = m.forward(prompt_ids())
    toks, margins = [tok], [margin(lg)]
    for _ in range(max(1, warm)):                  # untimed steps
        lg, tok = m.forward([tok])
        toks.append(tok)
        margins.append(margin(lg))
    t0 = time.perf_counter()
    for _ in range(steps):
        lg, tok = m.forward([tok])
        toks.append(tok)
        margins.append(margin(lg))
    dt = time.perf_counter() - t0
    return steps / dt, orc.num_threads(), dt, toks, margins


def parity_against(cpu_toks, cpu_margins, gpu_toks, tie=1e-3):
    """Greedy tokens of the device loop against the CPU restatement's: identical except where the
    restatement's own top-2 margin is a near-tie (< 1e-3), after which the paths legitimately part."""
    n = min(len(cpu_toks), len(gpu_toks))
    prefix = 0
    while prefix < n and int(cpu_toks[prefix]) == int(gpu_toks[prefix]):
        prefix += 1
    out = {"tokens_compared": n, "common_prefix": prefix, "equal": prefix == n, "near_ties": 0,
           "reference": "CPU restatement, bf16-rounded KV like the device cache"}
    if prefix < n:
        out["margin_at_divergence"] = cpu_margins[prefix]
        out["near_ties"] = int(cpu_margins[prefix] < tie)
        out["ok"] = bool(cpu_margins[prefix] < tie)
    else:
        out["ok"] = True
    return out


def run_reference_arm(args, rank):
    if rank != 0:
        return
    path = ensure_checkpoint()
    warm = max(1, min(args.warmup, 3))
    steps = max(1, min(args.steps, GEN_STEPS - warm))     # one generation of the named configuration
    tps, cores, dt, _, _ = cpu_decode(path, steps, warm=warm)
    sample = (f"{steps} greedy decode steps of the full 28-layer model after the {PROMPT_LEN}-token prompt, "
              f"CPU restatement of the reference's direct path (the reference's own IREE llvm-cpu "
              f"build cannot run here), {cores} OpenMP threads")
    print(json.dumps({
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": 1e3 * dt / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ------------------------------------------------------------------------- GPU arm

def time_lm_head(path, batches=5, reps=8):
    """Average device time of the stand-alone lm_head product (CUDA events on the launching stream
    around `reps` back-to-back launches, median over `batches`). The 127.6 MB of weights exceed L2,
    so consecutive launches cannot reuse cached weights."""
    import torch
    from dyninfer_b200 import checkpoint as ck, ops
    cat = ck.open_catalog(path)
    p = cat.parameters["token_embd.weight"]
    c = p.components[0]
    raw = np.fromfile(path, dtype=np.uint8, count=c.length, offset=c.offset)
    w = ops.DeviceWeight(p.encoding, p.shape[0], p.shape[1], raw)
    x = torch.randn(1, p.shape[1], device="cuda")
    y = torch.empty(1, p.shape[0], device="cuda")
    for _ in range(3):
        ops.linear(w, x, out=y)
    times = []
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            ops.linear(w, x, out=y)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return statistics.median(times), c.length, p.encoding


def time_prefill(model, n=2048, reps=3):
    """Prefill tok/s of an `n`-token random prompt through the public session call (host clock
    around `prefill_argmax`, which ends with the argmax token back on the host)."""
    import torch
    from dyninfer_b200 import synth
    from dyninfer_b200.runtime import SessionConfig
    ids = np.random.default_rng(SEED + 1).integers(0, synth.QWEN3_0_6B["vocab"], size=n).tolist()
    old_max = model.max_kv
    model.max_kv = max(model.max_kv, n + 8)
    times = []
    with model.create_session(SessionConfig(max_sequence_length=n + 8)) as s:
        s.prefill_argmax(ids)                      # first use: allocations, tensor maps
        for _ in range(reps):
            s.reset()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            s.prefill_argmax(ids)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
    model.max_kv = old_max
    return n / statistics.median(times)


# ------------------------------------------------------------- tensor-parallel section

TP_MODEL, TP_LAYERS, TP_FULL_LAYERS = "32b-q4_0", 8, 64


def tp_section(rank, world, local_rank, no_check=False):
    """The configuration that shards: Qwen3-32B shape (hidden 5120, 64/8 heads of 128, intermediate
    25600, Q4_0 linears, Q6_K embeddings and head), tensor parallel over the N ranks of this run with
    one exchange after o_proj and one after down. The file holds TP_LAYERS of the 64 layers (every
    layer carries layer 0's random bytes) so that writing and loading it stays within seconds; times
    per step are therefore those of an 8-layer model of the full width. Batch 1 and batch 32,
    4096-token random prompts, 256 greedy steps. At N > 1 rank 0 afterwards times the unsharded
    model alone (the N = 1 point of the strong-scaling curve), and a short run's logits are compared
    with the CPU restatement."""
    import torch
    from dyninfer_b200 import replicas, tp_decode
    out = {"model": f"qwen3-32b-shape q4_0, q6_k embeddings and head, {TP_LAYERS} of {TP_FULL_LAYERS} layers written "
                    "(each carries layer 0's bytes)", "n_gpus": world, "prompt": 4096, "steps": 256,
           "scaling": "strong", "timing": "CUDA events on each rank's session stream, maximum over ranks"}
    runs = {}
    for batch in (1, 32):
        r = tp_decode.run(TP_MODEL, TP_LAYERS, prompt=4096, steps=256, warmup=3, batch=batch, chunk=512,
                          kv_dtype="bf16", exchange="peer")
        runs[batch] = r
        out[f"batch{batch}"] = {k: r[k] for k in ("tokens_per_s", "ms_per_step", "prefill_tokens_per_s",
                                                  "weight_bytes_per_step_per_rank", "weight_gbs_per_gpu",
                                                  "weight_gbs_all_ranks", "exchange")}
    # short run for the parity check: prompt of 8 ids, the logits of its last row and of one step
    # every rank passes the same (non-empty) name: the extra calls that produce the logits are
    # collective, only rank 0 writes the file
    dump = os.path.join(os.path.dirname(checkpoint_path()), f"tp_logits_w{world}.npz")
    tp_decode.run(TP_MODEL, TP_LAYERS, prompt=8, steps=2, warmup=1, batch=1, chunk=512, kv_dtype="bf16",
                  exchange="peer", dump_logits=dump)
    replicas.barrier()
    if rank != 0:
        replicas.barrier()          # rank 0 is timing the unsharded model
        return None
    if world > 1:
        # the N = 1 point, measured in this run on rank 0's GPU while the other ranks wait
        for batch in (1, 32):
            r1 = tp_decode.run(TP_MODEL, TP_LAYERS, prompt=4096, steps=256, warmup=3, batch=batch, chunk=512,
                               kv_dtype="bf16", solo=True)
            out[f"batch{batch}"]["n1_ms_per_step"] = r1["ms_per_step"]
            out[f"batch{batch}"]["strong_scaling_efficiency"] = round(
                r1["ms_per_step"] / (world * runs[batch]["ms_per_step"]), 3)
        replicas.barrier()
    if not no_check:
        cores = use_all_host_threads()
        if world > 1:
            cores = min(cores, 8)      # the other ranks' runtime threads keep spinning on the same cores
        from oracle import oracle as orc
        from dyninfer_b200 import checkpoint as ck
        orc.build()
        orc.set_num_threads(cores)
        d = np.load(dump)
        cat = ck.open_catalog(str(d["checkpoint"]))
        m = orc.Model(cat.config, orc.weights_from_catalog(cat), kv_cap=32, kv_round=2, fast=True)
        lg0, tok0 = m.forward(d["prompt"].tolist())
        par = {"reference": "CPU restatement on the same file and prompt, bf16-rounded KV",
               "prefill_logits_max_abs_diff": float(np.abs(d["prefill_logits"] - lg0).max()),
               "first_token_equal": bool(int(d["first_token"]) == int(tok0))}
        if par["first_token_equal"]:
            lg1, _ = m.forward([tok0])
            par["step_logits_max_abs_diff"] = float(np.abs(d["step_logits"] - lg1).max())
        par["ok"] = bool(par["prefill_logits_max_abs_diff"] <= 1e-2 and par.get("step_logits_max_abs_diff", 0.0) <= 1e-2)
        out["parity"] = par
    try:
        os.remove(dump)
    except OSError:
        pass
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "f16", "f32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel section (32B shape)")
    ap.add_argument("--decode-only", action="store_true",
                    help="prompt + W + K device-loop decode steps and nothing else (small case for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # in-switch reduction off in every library used: a rank that dies while its memory is bound
    # to the switch's shared mapping can fault its peers
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    from dyninfer_b200 import replicas
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the cuda target has no CPU fallback")
    torch.cuda.set_device(local_rank)
    replicas.init("nccl", torch.device("cuda", local_rank))

    from dyninfer_b200 import build
    from dyninfer_b200.runtime import ModelLoader, SessionConfig
    build.build()
    if rank == 0:
        ensure_checkpoint()
    replicas.barrier()
    path = checkpoint_path()
    model = ModelLoader().load(path, target=f"cuda:{local_rank}", max_kv=2048, kv_dtype=args.kv_dtype)
    prompt = prompt_ids()
    K, W = args.steps, args.warmup
    max_seq = max(2048, PROMPT_LEN + 2 * (K + W) + 8)
    model.max_kv = max_seq
    session = model.create_session(SessionConfig(max_sequence_length=max_seq))
    first = session.prefill_argmax(prompt)

    def barrier():
        replicas.barrier()
        torch.cuda.synchronize()

    def begin_generation():
        session.reset()
        return session.prefill_argmax(prompt)

    # ---- device-resident arm
    if args.decode_only:
        toks_w, _ = session.decode_loop(first, W)
        _, ms = session.decode_loop(int(toks_w[-1]), K)
        print(json.dumps({"decode_only": True, "steps": K, "ms_per_step": ms / K}), flush=True)
        session.close()
        return
    for n in phases(max(W, GEN_STEPS)):               # warm-up: at least one whole generation
        session.decode_loop(begin_generation(), n)
    barrier()
    ms, gpu_launches, generations = 0.0, 0, []
    with ClockSampler(local_rank) as clocks:
        for n in phases(K):
            tok0 = begin_generation()
            torch.cuda.synchronize()
            launches0 = session.launch_count()
            toks, ms_phase = session.decode_loop(tok0, n)
            gpu_launches += session.launch_count() - launches0
            ms += ms_phase
            generations.append([int(tok0)] + [int(t) for t in toks])
        barrier()
        # ---- end-to-end arm through the public per-token call
        for n in phases(max(W, GEN_STEPS)):
            nxt = begin_generation()
            for _ in range(n):
                nxt = session.decode_argmax(nxt)
        barrier()
        e2e_s, e2e_same = 0.0, True
        for n in phases(K):
            nxt = begin_generation()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n):
                nxt = session.decode_argmax(nxt)
            torch.cuda.synchronize()
            e2e_s += time.perf_counter() - t0
            if n == len(generations[0]) - 1:            # the per-token call must end where the device loop did
                e2e_same = e2e_same and int(nxt) == generations[0][-1]
    ms, e2e_ms = replicas.max_over_ranks([ms, e2e_s * 1e3], device="cuda")   # slowest rank decides
    e2e_s = e2e_ms / 1e3
    weight_bytes = session.decode_weight_bytes()
    session.close()
    session = None
    tp = None if args.no_tp else tp_section(rank, world, local_rank, no_check=args.no_cpu_baseline)

    if rank == 0:
        hbm_peak, peak_kind = peaks()
        lm_ms, lm_bytes, lm_enc = time_lm_head(path)
        achieved = lm_bytes / (lm_ms * 1e-3) / 1e9
        out = {
            "metric": "decode_tokens_per_s", "value": replicas.whole_job_rate(K, ms, world), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "kv_dtype": args.kv_dtype, "parallelism": f"replicas x{world}",
                       "protocol": f"the reference perf runner's iterations: reset, prefill {PROMPT_LEN} (untimed), "
                                   f"{GEN_STEPS} greedy steps (timed); {len(generations)} decode phases",
                       "l2": "inputs larger than L2: each step streams %.1f MB of weights" % (weight_bytes / 1e6),
                       "weight_bytes_per_step": weight_bytes},
            "weight_gbs": world * weight_bytes * K / (ms * 1e-3) / 1e9,
            "weight_hbm_frac_of_%s" % peak_kind: weight_bytes * K / (ms * 1e-3) / 1e9 / hbm_peak,
            "e2e": {"value": world * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 24,
                    "d2h_bytes_per_step": 8, "last_token_equals_device_loop": bool(e2e_same)},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks.summary(),
            # dominant kernel: the persistent decode kernel, the only kernel of the timed region; one
            # launch decodes K / gpu_launches tokens. Algorithmic bytes per launch = the weight bytes
            # one token reads x the tokens of a launch; traffic likewise from a one-token capture.
            "roofline": {"bound": "hbm", "kernel": "decode_mega_kernel",
                         "tokens_per_launch": K / max(1, gpu_launches),
                         "achieved": weight_bytes / (ms / K * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": weight_bytes / (ms / K * 1e-3) / 1e9 / hbm_peak, "peak_source": peak_kind,
                         "bytes_per_launch": weight_bytes * K / max(1, gpu_launches),
                         "ms_per_launch": ms / max(1, gpu_launches),
                         "traffic": MEGA_DRAM_TRAFFIC * K / max(1, gpu_launches),
                         "traffic_source": "ncu capture of a one-token launch of this kernel, times the tokens of a launch"},
            # the largest single product of the step as its own launch (fused dequant-GEMV, M=1)
            "roofline_lm_head_gemv": {"bound": "hbm", "kernel": f"gemv_cs_q6k_kernel ({lm_enc}) 151936x1024, M=1",
                                      "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                                      "frac": achieved / hbm_peak, "bytes_per_launch": lm_bytes,
                                      "ms_per_launch": lm_ms},
        }
        out["prefill"] = {"tokens": 2048, "chunk": model.chunk_size, "tokens_per_s": time_prefill(model),
                          "note": "tcgen05 dequant GEMM + tensor-core flash attention, bf16 KV"}
        if not args.no_cpu_baseline and world == 1:
            # the CPU baseline belongs to the one-GPU run: under a multi-rank launch the host cores are
            # shared with the other ranks' runtime threads and the number would describe that contention
            steps, warm = 28, 4
            tps, cores, dt, cpu_toks, cpu_margins = cpu_decode(path, steps, warm=warm,
                                                               kv_round={"bf16": 2, "f16": 1, "f32": 0}[args.kv_dtype])
            out["cpu_baseline"] = {
                "value": tps, "unit": "tok/s", "cores": cores, "kind": "port",
                "sample": f"{steps} decode steps of the same model after the same {PROMPT_LEN}-token prompt "
                          f"({dt:.1f} s), CPU restatement of the reference's direct path"}
            # the same run checks the timed loop: its first tokens against the restatement's
            out["parity"] = parity_against(cpu_toks, cpu_margins, generations[0])
            # every timed generation repeats the first one token for token
            full = [g for g in generations if len(g) == len(generations[0])]
            out["parity"]["generations_identical"] = all(g == full[0] for g in full)
            out["parity"]["ok"] = bool(out["parity"]["ok"] and out["parity"]["generations_identical"])
        if tp is not None:
            out["tp"] = tp
        print(json.dumps(out), flush=True)
    replicas.shutdown()


if __name__ == "__main__":
    # A rank that fails must take the job down at once: left to normal interpreter shutdown it can
    # block in the teardown of its communicators while the other ranks wait for it in a collective.
    try:
        main()
    except SystemExit:
        raise
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)
