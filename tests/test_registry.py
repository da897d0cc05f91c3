"""Kernel registry: selection, strict rejection and whole-model coverage on the cuda target."""
import pytest

from dyninfer_b200 import checkpoint as ck, registry as reg, synth
from dyninfer_b200.runtime import ModelLoader
from dyninfer_b200 import DynInferError


def _params(cfg, enc="gguf.q4_0", embd="gguf.q6_k"):
    p = {"token_embd.weight": (embd, (cfg["vocab"], cfg["hidden"]))}
    for l in range(cfg["layers"]):
        for slot, shape in synth.linear_shapes(cfg).items():
            p[f"blk.{l}.{slot}.weight"] = (enc, shape)
    return p


def test_qwen3_0_6b_coverage_counts():
    """620 ops x 2 modes = 1240 requests, all covered (crates/dyninfer-runtime/src/qwen_e2e.rs:159)."""
    cfg = dict(synth.QWEN3_0_6B, qk_norm=True, rope=True)
    rep = reg.dry_run_coverage(cfg, _params(cfg), reg.TargetProfile.cuda())
    assert rep.requests == 1240 and not rep.missing
    ids = {k for _, _, k in rep.selected}
    assert "gguf.q4_0.matmul.cuda_sm100" in ids and "gguf.q6_k.gather.cuda_sm100" in ids
    assert "gguf.q6_k.lm_head.cuda_sm100" in ids and "attention.gqa.cuda_sm100" in ids
    rep.require_complete()


def test_k_quant_and_iq4_xs_files_are_covered():
    """A file that mixes Q4_K, Q5_K, IQ4_XS and Q6_K linears (the Q4_K_M / UD-Q4_K_XL kind) is fully covered on
    the cuda target; the container knows their block geometry."""
    cfg = dict(synth.QWEN3_0_6B, qk_norm=True, rope=True)
    p = _params(cfg, enc="gguf.q4_k")
    for l in range(cfg["layers"]):
        p[f"blk.{l}.attn_k.weight"] = ("gguf.iq4_xs", p[f"blk.{l}.attn_k.weight"][1])
        p[f"blk.{l}.ffn_down.weight"] = ("gguf.q5_k", p[f"blk.{l}.ffn_down.weight"][1])
    rep = reg.dry_run_coverage(cfg, p, reg.TargetProfile.cuda())
    assert rep.requests == 1240 and not rep.missing
    ids = {k for _, _, k in rep.selected}
    assert {"gguf.q4_k.matmul.cuda_sm100", "gguf.q5_k.matmul.cuda_sm100", "gguf.iq4_xs.matmul.cuda_sm100"} <= ids
    assert ck.GGML_TYPES[23] == ("gguf.iq4_xs", 256, 136) and ck.GGML_TYPES[12] == ("gguf.q4_k", 256, 144)
    assert ck.GGML_CODE["gguf.iq4_xs"] == 23 and 23 not in ck.GGML_SCHEMA_ONLY


def test_exact_backend_bonus_and_tie_break():
    r = reg.default_registry()
    rep = r.select(reg.KernelRequest("x", "RmsNorm"), reg.TargetProfile.cuda())
    assert rep.selected.id == "rms_norm.cuda_sm100.f32" and rep.score == 1200   # 200 + 1000
    r2 = reg.KernelRegistry()
    for i in ("b.k", "a.k"):
        r2.register(reg.KernelCandidate(i, "Silu", None, reg.TargetConstraint()))
    assert r2.select(reg.KernelRequest("x", "Silu"), reg.TargetProfile.cuda()).selected.id == "a.k"
    with pytest.raises(ValueError, match="duplicate"):
        r2.register(reg.KernelCandidate("a.k", "Silu", None, reg.TargetConstraint()))


def test_strict_rejection_reasons():
    r = reg.default_registry()
    cuda = reg.TargetProfile.cuda()
    # unregistered encoding -> E_KERNEL_COVERAGE, never a fallback
    with pytest.raises(reg.KernelCoverageError, match="E_KERNEL_COVERAGE.*gguf.q3_k"):
        r.require(reg.KernelRequest("blk.0.attn_q", "Linear", "gguf.q3_k", (1024, 1024)), cuda)
    # exact architecture match (kernel-registry lib.rs:627-740 `cuda.sm100`)
    rep = r.select(reg.KernelRequest("q", "Linear", "gguf.q4_0", (1024, 1024)), reg.TargetProfile.cuda("sm_90a"))
    assert rep.selected is None and any("architecture_mismatch" in w for _, ws in rep.rejected for w in ws)
    # wrong backend
    rep = r.select(reg.KernelRequest("q", "Linear", "gguf.q4_0", (1024, 1024)), reg.TargetProfile.llvm_cpu_host())
    assert rep.selected is None and any("backend_mismatch" in w for _, ws in rep.rejected for w in ws)
    # axis 1 must be a whole number of blocks; rank must be 2
    rep = r.select(reg.KernelRequest("q", "Linear", "gguf.q6_k", (64, 128)), cuda)
    assert rep.selected is None and any("axis_not_divisible" in w for _, ws in rep.rejected for w in ws)
    rep = r.select(reg.KernelRequest("q", "Linear", "gguf.q4_0", (64,)), cuda)
    assert rep.selected is None and any("rank_mismatch" in w for _, ws in rep.rejected for w in ws)
    # encoding-free generic candidates still match a cpu profile, cuda-specific ones do not
    assert r.select(reg.KernelRequest("n", "Rope"), reg.TargetProfile.llvm_cpu_host()).selected.id == "rope.generated.f32"


def test_loader_rejects_uncovered_model_and_cpu_target(tmp_path):
    path = str(tmp_path / "m.gguf")
    synth.write_qwen3_gguf(path, synth.TINY, seed=1)
    ld = ModelLoader()
    with pytest.raises(DynInferError, match="no CPU fallback"):
        ld.load(path, target="cpu")
    cat = ld.bind(path)
    cat.parameters["blk.0.attn_q.weight"].encoding = "gguf.q3_k"
    rep = ld.kernel_coverage(cat, reg.TargetProfile.cuda())
    assert len(rep.missing) == 2          # prefill + decode
    with pytest.raises(reg.KernelCoverageError, match="E_KERNEL_COVERAGE"):
        rep.require_complete()
    model = ld.load(path, target="cuda:sm_100a")
    assert model.coverage.requests == (2 * 22 + 4) * 2 and model.target_profile().driver == "cuda"
