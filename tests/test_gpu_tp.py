"""Tensor-parallel session on two GPUs against the unsharded session on one (needs >= 2 GPUs).

Both ranks upload their slices of a small seeded GGUF model (mixed Q4_0 / Q4_1 / Q8_0 linears, Q6_K
lm_head), prefill a prompt in chunks and decode greedily; rank 0 then runs the unsharded model and
compares. The sums over ranks change the f32 summation order, so logits agree to a tolerance and
greedy tokens agree until a near-tie. Both exchange paths run: the NCCL all-reduce and the fused
peer-memory kernel (arrival flags + peer loads + residual + RMSNorm)."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("model,layers,extra", [("tiny", 0, ["--prompt", "40", "--chunk", "32", "--steps", "12"]),
                                                ("8b-mixed", 2, ["--prompt", "96", "--chunk", "64", "--steps", "8",
                                                                 "--batch", "3"])])
@pytest.mark.parametrize("exchange", ["nccl", "peer"])
def test_two_gpu_tensor_parallel_matches_unsharded(tmp_path, oracle, model, layers, extra, exchange):
    import numpy as np
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, DYNINFER_BENCH_DIR=str(tmp_path), NCCL_NVLS_ENABLE="0")
    dump = str(tmp_path / "rank0_logits.npz")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m", "dyninfer_b200.tp_decode",
           "--model", model, "--check", "--kv-dtype", "f32", "--exchange", exchange, "--dump-logits", dump] + extra
    if layers:
        cmd += ["--layers", str(layers)]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    r = json.loads(line)
    assert r["tp"] == 2 and r["exchange"] == exchange and r["ranks_agree"]
    c = r["check"]
    assert c["prefill_logits_max_abs_diff"] <= 1e-2 * max(1.0, c["logits_max_abs"]), c
    assert c["step_logits_max_abs_diff"] <= 1e-2 * max(1.0, c["logits_max_abs"]), c
    assert c["first_tokens_equal"], c
    assert min(c["common_prefix_per_sequence"]) >= 4, c
    # rank 0's logits against the CPU oracle on the same checkpoint and prompt (not only against
    # the unsharded CUDA session): max-abs <= 1e-2, cosine >= 0.9999
    import helpers
    from dyninfer_b200 import checkpoint as ck
    from test_gpu_model import oracle_run
    d = np.load(dump)
    cat = ck.open_catalog(str(d["checkpoint"]))
    want_logits, want_toks, _ = oracle_run(oracle, cat, d["prompt"].tolist(), 1, kv_cap=256)
    assert np.abs(d["prefill_logits"] - want_logits[0]).max() <= 1e-2
    assert helpers.cosine(d["prefill_logits"], want_logits[0]) >= 0.9999
    if int(d["first_token"]) == want_toks[0]:
        assert np.abs(d["step_logits"] - want_logits[1]).max() <= 1e-2
        assert helpers.cosine(d["step_logits"], want_logits[1]) >= 0.9999
