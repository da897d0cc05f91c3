"""Kernel candidates for the `cuda` sm_100a target and strict coverage checking.

Same contract as the reference's registry (crates/dyninfer-kernel-registry/src/lib.rs):
candidates are described per (operation x encoding x target x mode); `select`
filters by rejection reasons (:499-581), scores with the deterministic cost model
(+1000 when the candidate names the target's driver, :252-268), ties break by id
(:330-335); `require` raises E_KERNEL_COVERAGE when nothing qualifies (:350-402).
`dry_run_coverage` walks every operation of the decoder in both execution modes
like crates/dyninfer-quantization/src/lib.rs:311-426. Nothing ever falls back to
another target.
"""
from __future__ import annotations

from dataclasses import dataclass, field

OPERATIONS = ("Input", "Embedding", "Linear", "RmsNorm", "PerHeadRmsNorm", "Rope", "KvCacheWrite",
              "KvCacheRead", "Attention", "ShortConv", "Silu", "Multiply", "Residual",
              "OutputProjection")
MODES = ("prefill", "decode")


class KernelCoverageError(RuntimeError):
    code = "E_KERNEL_COVERAGE"


@dataclass(frozen=True)
class TargetProfile:
    """crates/dyninfer-core/src/types.rs:274-379 (TargetProfile::cuda)."""
    driver: str
    architecture: str | None = None
    features: tuple = ()

    @staticmethod
    def cuda(arch: str = "sm_100a") -> "TargetProfile":
        return TargetProfile("cuda", arch, ("native_bf16", "tensor_cores", "nvfp4"))

    @staticmethod
    def llvm_cpu_host() -> "TargetProfile":
        return TargetProfile("local-task", None, ("avx2",))


@dataclass(frozen=True)
class TargetConstraint:
    backends: tuple = ("any",)
    exact_architectures: tuple = ()
    required_features: tuple = ()


@dataclass(frozen=True)
class KernelCandidate:
    id: str
    operation: str
    encoding: str | None
    target: TargetConstraint
    modes: tuple = MODES
    logical_rank: int | None = None
    axis_multiples: tuple = ()      # ((axis, multiple_of), ...)
    deterministic_score: int = 100
    production: bool = True
    lowering: str = ""
    notes: str = ""


@dataclass
class KernelRequest:
    operation_id: str
    operation: str
    encoding: str | None = None
    logical_shape: tuple | None = None
    mode: str = "decode"


@dataclass
class SelectionReport:
    selected: KernelCandidate | None
    score: int | None
    rejected: list = field(default_factory=list)   # [(candidate id, [reasons])]


def rejection_reasons(c: KernelCandidate, r: KernelRequest, t: TargetProfile) -> list:
    reasons = []
    if c.encoding != r.encoding:
        reasons.append("encoding_mismatch")
    if not c.production:
        reasons.append("not_production_ready")
    if r.mode not in c.modes:
        reasons.append("mode_mismatch")
    if "any" not in c.target.backends and t.driver not in c.target.backends:
        reasons.append(f"backend_mismatch(selected={t.driver})")
    if c.target.exact_architectures and t.architecture not in c.target.exact_architectures:
        reasons.append(f"architecture_mismatch(selected={t.architecture})")
    for f in c.target.required_features:
        if f not in t.features:
            reasons.append(f"missing_target_feature({f})")
    if r.logical_shape is not None:
        if c.logical_rank is not None and len(r.logical_shape) != c.logical_rank:
            reasons.append(f"rank_mismatch(expected={c.logical_rank}, actual={len(r.logical_shape)})")
        else:
            for axis, mult in c.axis_multiples:
                if axis < len(r.logical_shape) and r.logical_shape[axis] % mult:
                    reasons.append(f"axis_not_divisible(axis={axis}, dimension={r.logical_shape[axis]}, multiple_of={mult})")
    return reasons


class KernelRegistry:
    VERSION = "5+cuda1"

    def __init__(self):
        self.candidates: list[KernelCandidate] = []

    def register(self, c: KernelCandidate):
        if any(e.id == c.id for e in self.candidates):
            raise ValueError(f"duplicate kernel candidate `{c.id}`")
        self.candidates.append(c)

    def select(self, r: KernelRequest, t: TargetProfile) -> SelectionReport:
        accepted, rejected = [], []
        for c in self.candidates:
            if c.operation != r.operation:
                continue
            why = rejection_reasons(c, r, t)
            if why:
                rejected.append((c.id, why))
            else:
                score = c.deterministic_score + (1000 if t.driver in c.target.backends else 0)
                accepted.append((score, c))
        accepted.sort(key=lambda sc: (-sc[0], sc[1].id))
        if accepted:
            return SelectionReport(accepted[0][1], accepted[0][0], rejected)
        return SelectionReport(None, None, rejected)

    def require(self, r: KernelRequest, t: TargetProfile) -> KernelCandidate:
        rep = self.select(r, t)
        if rep.selected is not None:
            return rep.selected
        rej = "; ".join(f"{i}: {w}" for i, w in rep.rejected) or "none registered"
        raise KernelCoverageError(
            f"E_KERNEL_COVERAGE: no production kernel for {r.operation} with encoding "
            f"{r.encoding or 'none'} in {r.mode} mode (op {r.operation_id}; target={t.driver} "
            f"architecture={t.architecture}); rejected candidates: {rej}")


CUDA_SM100 = TargetConstraint(("cuda",), ("sm_100a", "sm_100"), ())
# (encoding, elements per block along the input axis)
CUDA_ENCODINGS = (("gguf.q4_0", 32), ("gguf.q4_1", 32), ("gguf.q8_0", 32), ("gguf.q6_k", 256),
                  ("gguf.q4_k", 256), ("gguf.q5_k", 256), ("gguf.iq4_xs", 256),
                  ("mlx.affine.u4", 64), ("plain.bf16", 4), ("plain.f16", 4), ("plain.f32", 4))


def register_cuda_candidates(reg: KernelRegistry) -> KernelRegistry:
    """The kernels libdyninfer_cuda implements, one candidate per (op x encoding)."""
    for enc, block in CUDA_ENCODINGS:
        short = enc.replace(".", "_")
        for op, tag in (("Linear", "matmul"), ("OutputProjection", "lm_head"), ("Embedding", "gather")):
            reg.register(KernelCandidate(
                id=f"{enc}.{tag}.cuda_sm100", operation=op, encoding=enc, target=CUDA_SM100,
                logical_rank=2, axis_multiples=((1, block),), deterministic_score=300,
                lowering=f"cuda.{short}.{tag}",
                notes="fused dequant on the verbatim checkpoint bytes, f32 accumulation"))
    for op, kid in (("Input", "model.input.cuda"), ("RmsNorm", "rms_norm.cuda_sm100.f32"),
                    ("PerHeadRmsNorm", "per_head_rms_norm.cuda_sm100.f32"),
                    ("Rope", "rope.cuda_sm100.f32"), ("KvCacheWrite", "kv_cache.write.cuda_sm100"),
                    ("KvCacheRead", "kv_cache.read.cuda_sm100"),
                    ("Attention", "attention.gqa.cuda_sm100"), ("Silu", "silu.cuda_sm100.f32"),
                    ("Multiply", "multiply.cuda_sm100.f32"), ("Residual", "residual.cuda_sm100.f32")):
        reg.register(KernelCandidate(id=kid, operation=op, encoding=None, target=CUDA_SM100,
                                     deterministic_score=200, lowering=kid))
    return reg


def register_builtin_semantic_candidates(reg: KernelRegistry) -> KernelRegistry:
    """Encoding-free candidates valid on any target
    (crates/dyninfer-kernel-registry/src/lib.rs:404-497)."""
    for op, kid in (("Input", "model.input.abi"), ("Rope", "rope.generated.f32"),
                    ("RmsNorm", "rms_norm.generated.f32"),
                    ("PerHeadRmsNorm", "per_head_rms_norm.generated.f32"),
                    ("KvCacheWrite", "kv_cache.write.generated"),
                    ("KvCacheRead", "kv_cache.read.generated"),
                    ("Attention", "attention.generated.f32"), ("Silu", "silu.generated.f32"),
                    ("Multiply", "multiply.generated.f32"), ("Residual", "residual.generated.f32")):
        reg.register(KernelCandidate(id=kid, operation=op, encoding=None, target=TargetConstraint()))
    return reg


def default_registry() -> KernelRegistry:
    return register_cuda_candidates(register_builtin_semantic_candidates(KernelRegistry()))


def decoder_operations(config: dict, parameters: dict):
    """(operation id, kind, encoding, logical shape) for every op of the decoder graph in the
    order fixed by crates/dyninfer-architecture/src/builder.rs:491-614,664-718.
    `parameters` maps canonical name -> (encoding, shape)."""
    def par(name):
        enc, shape = parameters[name]
        return enc, tuple(shape)

    ops = [("input.tokens", "Input", None, None),
           ("embed", "Embedding", *par("token_embd.weight"))]
    for l in range(config["layers"]):
        p = f"blk.{l}."
        ops.append((p + "attn_norm", "RmsNorm", None, None))
        for s in ("attn_q", "attn_k", "attn_v"):
            ops.append((p + s, "Linear", *par(p + s + ".weight")))
        if config.get("qk_norm", True):
            ops += [(p + "attn_q_norm", "PerHeadRmsNorm", None, None),
                    (p + "attn_k_norm", "PerHeadRmsNorm", None, None)]
        if config.get("rope", True):
            ops += [(p + "rope_q", "Rope", None, None), (p + "rope_k", "Rope", None, None)]
        ops += [(p + "kv_write_k", "KvCacheWrite", None, None),
                (p + "kv_write_v", "KvCacheWrite", None, None),
                (p + "kv_read_k", "KvCacheRead", None, None),
                (p + "kv_read_v", "KvCacheRead", None, None),
                (p + "attention", "Attention", None, None),
                (p + "attn_output", "Linear", *par(p + "attn_output.weight")),
                (p + "attn_residual", "Residual", None, None),
                (p + "ffn_norm", "RmsNorm", None, None),
                (p + "ffn_gate", "Linear", *par(p + "ffn_gate.weight")),
                (p + "ffn_up", "Linear", *par(p + "ffn_up.weight")),
                (p + "ffn_silu", "Silu", None, None), (p + "ffn_mul", "Multiply", None, None),
                (p + "ffn_down", "Linear", *par(p + "ffn_down.weight")),
                (p + "ffn_residual", "Residual", None, None)]
    head = "output.weight" if "output.weight" in parameters else "token_embd.weight"
    ops += [("output_norm", "RmsNorm", None, None), ("lm_head", "OutputProjection", *par(head))]
    return ops


@dataclass
class CoverageReport:
    target: TargetProfile
    selected: list = field(default_factory=list)   # [(op id, mode, kernel id)]
    missing: list = field(default_factory=list)    # [(op id, mode, message)]

    @property
    def requests(self) -> int:
        return len(self.selected) + len(self.missing)

    def require_complete(self):
        """crates/dyninfer-quantization/src/lib.rs:255-306."""
        if self.missing:
            op, mode, msg = self.missing[0]
            raise KernelCoverageError(f"{msg} ({len(self.missing)} of {self.requests} requests uncovered)")
        return self


def dry_run_coverage(config: dict, parameters: dict, target: TargetProfile,
                     registry: KernelRegistry | None = None) -> CoverageReport:
    reg = registry or default_registry()
    rep = CoverageReport(target)
    for op_id, kind, enc, shape in decoder_operations(config, parameters):
        for mode in MODES:
            req = KernelRequest(op_id, kind, enc, shape, mode)
            try:
                rep.selected.append((op_id, mode, reg.require(req, target).id))
            except KernelCoverageError as e:
                rep.missing.append((op_id, mode, str(e)))
    return rep
