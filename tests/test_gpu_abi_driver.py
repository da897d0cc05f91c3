"""The C ABI driven by a C program (tests/abi_driver.c) with no Python in the process.

The driver is compiled with gcc against include/dyninfer_cuda.h, linked with
libdyninfer_cuda.so, and walks the session the way the reference's Rust `IreeSession`
walks its native handle (crates/dyninfer-runtime/src/session.rs:89-330 over
crates/iree-runtime/src/lib.rs:495-537): create -> configure -> ensure -> chunked prefill ->
one invoke per token -> statistics -> reset -> destroy. Its tokens and logits must equal
the Python host's (same library, same calls) and match the CPU oracle.
"""
import json
import os
import subprocess

import numpy as np
import pytest

from dyninfer_b200 import _lib, checkpoint as ck, synth
from dyninfer_b200.runtime import ModelLoader, SessionConfig
from test_gpu_model import greedy_match, oracle_run

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_driver(tmp_path):
    exe = str(tmp_path / "abi_driver")
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.check_call(["gcc", "-O1", "-Wall", "-Wextra", "-std=c11", "-D_POSIX_C_SOURCE=200809L",
                           os.path.join(ROOT, "tests", "abi_driver.c"), "-I", os.path.join(ROOT, "include"),
                           "-L", libdir, "-ldyninfer_cuda", f"-Wl,-rpath,{libdir}", "-o", exe])
    return exe


@pytest.mark.parametrize("cfg_name,kernel", [("SMALL_D128", "persistent"), ("TINY", "graph")])
def test_c_host_matches_python_host_and_oracle(native_lib, oracle, tmp_path, cfg_name, kernel):
    cfg = getattr(synth, cfg_name)
    path = synth.write_qwen3_gguf(str(tmp_path / "m.gguf"), cfg, seed=77,
                                  encodings={"attn_v": "gguf.q4_1", "ffn_down": "gguf.q8_0"})
    cat = ck.open_catalog(path)
    plan = ck.build_runtime_provider_plan(cat)
    desc = ck.model_descriptor(cat, kv_dtype="f32", decode_kernel=kernel, batch=1)
    (tmp_path / "desc.json").write_text(json.dumps(desc))
    lines = [str(len(plan.file_paths))] + list(plan.file_paths)
    lines += [f"{p.external_key} {p.source_file_index} {p.offset} {p.length}" for p in plan.parameters]
    (tmp_path / "params.txt").write_text("\n".join(lines) + "\n")
    prompt = np.random.default_rng(3).integers(1, cfg["vocab"], size=21).tolist()   # chunks 8 + 8 + 5
    steps = 12
    exe = build_driver(tmp_path)
    out = subprocess.run([exe, str(tmp_path / "desc.json"), str(tmp_path / "params.txt"), "8",
                          ",".join(map(str, prompt)), str(steps)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    rows = dict(ln.split(": ", 1) for ln in out.stdout.strip().splitlines())
    c_tokens = [int(t) for t in rows["tokens"].split()]
    c_logits = np.array([float(v) for v in rows["logits0"].split()], dtype=np.float32)
    assert f"persistent: {int(kernel == 'persistent')}" in rows["pages"] and rows["pages"].startswith("1 ")

    # the Python host makes the same calls through the same library: identical results
    model = ModelLoader().load(path, max_kv=256, kv_dtype="f32", chunk_size=8, decode_kernel=kernel)
    with model.create_session(SessionConfig(max_sequence_length=256)) as s:
        lg = s.prefill(prompt).values
        py = [int(np.argmax(lg))]
        for _ in range(steps):
            py.append(s.decode_argmax(py[-1]))
    assert c_tokens == py
    assert np.array_equal(c_logits, lg[:4])
    # and both follow the oracle
    want_logits, want_toks, margins = oracle_run(oracle, cat, prompt, steps)
    assert np.abs(lg - want_logits[0]).max() <= 1e-2
    assert greedy_match(c_tokens, want_toks, margins) >= 1
