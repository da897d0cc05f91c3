"""Host-side runtime for the `cuda` target: loader, session, greedy generation, perf.

Mirrors the reference's runtime interface for this path — same names, argument
meaning and error behaviour — on top of libdyninfer_cuda:

  * `CausalLanguageModel` / `ModelSession`: crates/dyninfer-runtime/src/lib.rs:44-138
  * session logic (chunking, right padding, position, limits):
    crates/dyninfer-runtime/src/session.rs:15-389
  * `ModelLoader.bind / kernel_coverage / load`: crates/dyninfer-runtime/src/model.rs:231-557
  * `argmax`, `generate_greedy`: crates/dyninfer-runtime/src/generate.rs:16-26,117-232
    (token ids in, token ids out: the tokenizer is outside this path)
  * `run_perf`, `eff_weight_bw_gbs`: crates/dyninfer-runtime/src/perf.rs:92-172,298-305

Paged-KV constants: page 256, chunk 512
(crates/dyninfer-compiler/src/lowering/dense_decoder.rs:52-56).
"""
from __future__ import annotations

import ctypes as C
import json
import time
from dataclasses import dataclass, field

import numpy as np

from . import _lib, checkpoint as ck, registry as reg
from ._lib import DynInferError, check, lib

PAGE_SIZE = 256
CHUNK_SIZE = 512


@dataclass
class SessionConfig:
    max_sequence_length: int = 2048
    batch_size: int = 1
    seed: int | None = None


@dataclass
class KvCacheMetrics:
    page_count: int = 0
    allocated_bytes: int = 0
    capacity_bytes: int = 0
    used_bytes: int = 0
    filled_tokens: int = 0
    layers: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    max_sequence_length: int = 0
    key_dtype: str = "f32"
    value_dtype: str = "f32"
    paged: bool = False
    chunk_size: int = 0


@dataclass
class AllocatorMetrics:
    host_bytes_peak: int = 0
    host_bytes_allocated: int = 0
    host_bytes_freed: int = 0
    device_bytes_peak: int = 0
    device_bytes_allocated: int = 0
    device_bytes_freed: int = 0

    def host_live_bytes(self):
        return max(0, self.host_bytes_allocated - self.host_bytes_freed)

    def device_live_bytes(self):
        return max(0, self.device_bytes_allocated - self.device_bytes_freed)


@dataclass
class Logits:
    values: np.ndarray


def argmax(logits) -> int:
    """First strict maximum; 0 when nothing exceeds -inf (NaNs never win)."""
    v = np.asarray(logits)
    if v.size == 0:
        return 0
    m = np.where(np.isnan(v), -np.inf, v)
    i = int(np.argmax(m))  # numpy returns the first maximum
    return i if m[i] > -np.inf else 0


class CudaSession:
    """One KV cache = one native handle; sessions are independent."""

    def __init__(self, model: "LoadedModel", config: SessionConfig):
        self.model, self.config = model, config
        self.metadata = model.metadata
        self.position_ = 0
        self.history: list[int] = []
        self.pad_token_id = int(model.metadata.get("pad_token_id", model.metadata.get("bos_token_id", 0)) or 0)
        self._h = C.c_void_p()
        cfg = model.catalog.config
        self.kv_dtype = model.kv_dtype
        self.kv_elem = 4 if self.kv_dtype == "f32" else 2
        self.max_kv = int(model.max_kv)
        files = (_lib.ParameterFile * len(model.plan.file_paths))(
            *[_lib.ParameterFile(p.encode()) for p in model.plan.file_paths])
        kv_heads = cfg["kv_heads"]
        if model.tp:
            # one rank of a tensor-parallel group: this rank's slices and share of the geometry
            from . import tp as _tp
            rank, world = model.tp
            desc, ranges = _tp.session_inputs(model.catalog, rank, world, kv_dtype=self.kv_dtype,
                                              batch=max(1, int(config.batch_size)))
            kv_heads = desc["kv_heads"]
        else:
            desc = ck.model_descriptor(model.catalog, kv_dtype=self.kv_dtype, decode_kernel=model.decode_kernel,
                                       batch=max(1, int(config.batch_size)))
            ranges = [(p.external_key, p.source_file_index, p.offset, p.length) for p in model.plan.parameters]
        self._keys = [r[0].encode() for r in ranges]
        params = (_lib.FileParam * len(self._keys))(
            *[_lib.FileParam(k, r[1], r[2], r[3]) for k, r in zip(self._keys, ranges)])
        check(lib().dyninfer_cuda_session_create_with_file_params(
            model.device_uri.encode(), json.dumps(desc).encode(), files, len(files), params,
            len(self._keys), C.byref(self._h)))
        if model.tp:
            from . import tp as _tp
            n = lib().dyninfer_cuda_tp_unique_id_bytes()

            def make_id():
                buf = C.create_string_buffer(n)
                check(lib().dyninfer_cuda_tp_unique_id(buf, n))
                return buf.raw
            uid = _tp.exchange_unique_id(make_id)
            check(lib().dyninfer_cuda_session_tp_init(self._h, uid, len(uid)))
        check(lib().dyninfer_cuda_session_configure_paged_kv(
            self._h, cfg["layers"], PAGE_SIZE, kv_heads, cfg["head_dim"], self.kv_elem,
            model.chunk_size, cfg["vocab"]))
        if model.tp and model.tp_exchange == "peer":
            # partial products are summed by this library's own kernel over peer memory
            import torch.distributed as dist
            n = lib().dyninfer_cuda_tp_peer_handle_bytes()
            buf = C.create_string_buffer(n)
            check(lib().dyninfer_cuda_session_tp_peer_handle(self._h, buf, n))
            handles = [None] * model.tp[1]
            dist.all_gather_object(handles, buf.raw)
            blob = b"".join(handles)
            check(lib().dyninfer_cuda_session_tp_peer_attach(self._h, blob, len(blob)))
            dist.barrier()
        self._pages_ready = False
        self._tok1 = (C.c_int64 * 1)()
        self._out1 = C.c_int64(-1)
        self._invoke_fn = lib().dyninfer_cuda_session_invoke_paged_chunk

    # -- lifetime
    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            native = _lib._lib          # already loaded; at interpreter shutdown modules may be half torn down
            if native is not None:
                native.dyninfer_cuda_session_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- helpers
    def _max_seq(self) -> int:
        return min(max(1, self.config.max_sequence_length), max(1, self.max_kv))

    def _require_batch_1(self):
        if self.config.batch_size != 1:
            raise DynInferError(f"batch_size {self.config.batch_size} is not supported (only batch_size=1)")

    def _ensure_pages(self):
        pages = max(1, -(-self._max_seq() // PAGE_SIZE))
        check(lib().dyninfer_cuda_session_ensure_kv_pages(self._h, pages))
        self._pages_ready = True

    def _window(self, tokens):
        w = self.model.chunk_size
        window = np.full(w, self.pad_token_id, dtype=np.int64)
        n = min(len(tokens), w)
        if n == 0:
            return window, 0
        window[:n] = tokens[:n]
        return window, n - 1

    def _invoke(self, tokens: np.ndarray, last: int, start: int, want_logits: bool):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        ptr = C.POINTER(C.c_float)()
        count = C.c_size_t(0)
        tok = C.c_int64(-1)
        check(lib().dyninfer_cuda_session_invoke_paged_chunk(
            self._h, tokens.ctypes.data_as(C.POINTER(C.c_int64)), tokens.size, int(last), int(start),
            C.byref(ptr), C.byref(count), C.byref(tok), 1 if want_logits else 0))
        logits = None
        if want_logits:
            # session-owned scratch, valid until the next invoke: copy immediately
            logits = np.ctypeslib.as_array(ptr, shape=(count.value,)).copy()
        return logits, int(tok.value)

    def _prefill(self, tokens, want_logits: bool):
        self._require_batch_1()
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise DynInferError("prefill requires a non-empty token list")
        if len(tokens) > self._max_seq():
            raise DynInferError(f"prefill length {len(tokens)} exceeds session/KV limit {self._max_seq()}")
        self.history = list(tokens)
        check(lib().dyninfer_cuda_session_reset_paged_kv(self._h))
        self._ensure_pages()
        cs = self.model.chunk_size
        chunks = [tokens[i:i + cs] for i in range(0, len(tokens), cs)]
        logits, token = None, -1
        for ci, chunk in enumerate(chunks):
            window, last = self._window(chunk)
            final = ci + 1 == len(chunks)
            lg, token = self._invoke(window, last, ci * cs, want_logits and final)
            if final:
                logits = lg
        self.position_ = len(tokens)
        return logits, token

    def _decode(self, token: int, want_logits: bool):
        self._require_batch_1()
        if self.position_ >= self._max_seq():
            raise DynInferError(f"decode position {self.position_} exceeds session/KV limit {self._max_seq()}")
        if not self._pages_ready:
            self._ensure_pages()
        if want_logits:
            lg, nxt = self._invoke(np.array([int(token)], dtype=np.int64), 0, self.position_, True)
        else:
            # the per-token hot call: reuse the argument objects instead of building arrays every step
            self._tok1[0] = int(token)
            check(self._invoke_fn(self._h, self._tok1, 1, 0, self.position_, None, None, C.byref(self._out1), 0))
            lg, nxt = None, int(self._out1.value)
        self.history.append(int(token))
        self.position_ += 1
        return lg, nxt

    # -- ModelSession
    def prefill(self, tokens) -> Logits:
        lg, _ = self._prefill(tokens, True)
        if lg.size != self.metadata["vocabulary_size"]:
            raise DynInferError(f"prefill returned {lg.size} logits, expected vocab {self.metadata['vocabulary_size']}")
        return Logits(lg)

    def decode(self, token: int) -> Logits:
        lg, _ = self._decode(token, True)
        return Logits(lg)

    def prefill_argmax(self, tokens) -> int:
        _, tok = self._prefill(tokens, False)
        if tok < 0:
            raise DynInferError(f"prefill_argmax returned invalid token {tok}")
        return tok

    def decode_argmax(self, token: int) -> int:
        _, tok = self._decode(token, False)
        if tok < 0:
            raise DynInferError(f"decode_argmax returned invalid token {tok}")
        return tok

    def position(self) -> int:
        return self.position_

    def reset(self):
        check(lib().dyninfer_cuda_session_reset_paged_kv(self._h))
        self.position_ = 0
        self.history = []

    def kv_cache_metrics(self) -> KvCacheMetrics:
        cfg = self.model.catalog.config
        per_token = cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * self.kv_elem * 2
        pages = lib().dyninfer_cuda_session_kv_page_count(self._h)
        alloc = lib().dyninfer_cuda_session_kv_allocated_bytes(self._h)
        return KvCacheMetrics(page_count=pages, allocated_bytes=alloc,
                              capacity_bytes=per_token * self.max_kv, used_bytes=alloc,
                              filled_tokens=self.position_, layers=cfg["layers"],
                              kv_heads=cfg["kv_heads"], head_dim=cfg["head_dim"],
                              max_sequence_length=self.max_kv, key_dtype=self.kv_dtype,
                              value_dtype=self.kv_dtype, paged=True, chunk_size=self.model.chunk_size)

    def allocator_metrics(self) -> AllocatorMetrics:
        st = _lib.AllocatorStatistics()
        check(lib().dyninfer_cuda_session_allocator_statistics(self._h, C.byref(st)))
        return AllocatorMetrics(*[getattr(st, f[0]) for f in st._fields_])

    # -- extensions of the cuda target
    def decode_loop(self, first_token: int, steps: int):
        """Device-resident greedy loop starting at the current position.
        Returns (tokens produced, device milliseconds)."""
        self._require_batch_1()
        if self.position_ + steps > self._max_seq():
            raise DynInferError(f"decode loop of {steps} steps from {self.position_} exceeds session/KV limit {self._max_seq()}")
        self._ensure_pages()
        out = np.empty(steps, dtype=np.int64)
        ms = C.c_float(0)
        check(lib().dyninfer_cuda_session_decode_loop(
            self._h, int(first_token), self.position_, steps,
            out.ctypes.data_as(C.POINTER(C.c_int64)), C.byref(ms)))
        self.history.append(int(first_token))
        self.history.extend(int(t) for t in out[:-1])
        self.position_ += steps
        return out, float(ms.value)

    def decode_phase_profile(self) -> dict:
        """Microseconds per phase kind in the last persistent-kernel launch (CTA 0's view)."""
        out = (C.c_double * 24)()
        check(lib().dyninfer_cuda_session_decode_phase_profile(self._h, out, 24))
        names = ("embed", "qkv", "attention", "o_proj", "gate_up", "down", "lm_head", "argmax", "total",
                 "t_stage", "t_wait_weights", "t_rows", "t_round_reduce", "t_attn_prepare", "t_attn_scores",
                 "t_attn_merge", "t_stage_arrive", "t_stage_convert")
        return dict(zip(names, [float(v) for v in out]))

    def timer_start(self) -> None:
        """Starts the device-side stopwatch of the session's stream (CUDA events)."""
        check(lib().dyninfer_cuda_session_timer(self._h, 0, None))

    def timer_stop(self) -> float:
        """Milliseconds the session's stream spent since `timer_start` (waits for the work)."""
        ms = C.c_float()
        check(lib().dyninfer_cuda_session_timer(self._h, 1, C.byref(ms)))
        return float(ms.value)

    def decode_trace(self):
        """[CTAs, layers + 1, 16] global-timer stamps (ns) of the last persistent-kernel launch, or None
        when the session was not created with DYNINFER_CUDA_TRACE=1."""
        need = C.c_size_t(0)
        check(lib().dyninfer_cuda_session_decode_trace(self._h, None, 0, C.byref(need)))
        if not need.value:
            return None
        out = np.zeros(need.value, dtype=np.uint64)
        check(lib().dyninfer_cuda_session_decode_trace(self._h, out.ctypes.data_as(C.POINTER(C.c_uint64)), need.value,
                                                       C.byref(need)))
        layers = self.model.catalog.config["layers"]
        return out.reshape(-1, layers + 1, 16)

    def uses_persistent_kernel(self) -> bool:
        """Whether single-row steps run as the one-launch-per-token persistent kernel (decided when
        the KV geometry is configured; False: a captured graph of per-operator kernels)."""
        return bool(lib().dyninfer_cuda_session_uses_persistent_kernel(self._h))

    def weight_bytes(self) -> int:
        return int(lib().dyninfer_cuda_session_weight_bytes(self._h))

    def decode_weight_bytes(self) -> int:
        return int(lib().dyninfer_cuda_session_decode_weight_bytes(self._h))

    def launch_count(self) -> int:
        return int(lib().dyninfer_cuda_session_launch_count(self._h))


class LoadedModel:
    """CausalLanguageModel for the cuda target."""

    def __init__(self, catalog: ck.Catalog, plan: ck.ProviderPlan, target: reg.TargetProfile,
                 device_uri: str, coverage: reg.CoverageReport, max_kv: int, kv_dtype: str,
                 chunk_size: int, decode_kernel: str = "persistent", tp: tuple | None = None,
                 tp_exchange: str = "peer"):
        self.catalog, self.plan, self.target, self.device_uri = catalog, plan, target, device_uri
        # (rank, world) of a tensor-parallel group: one process per GPU, every process loads the
        # same checkpoint and uploads its own slices; torch.distributed must be initialised
        self.tp = tp if tp and tp[1] > 1 else None
        # "peer": o_proj / down partial sums through the fused peer-memory kernel; "nccl": all-reduce
        if tp_exchange not in ("peer", "nccl"):
            raise DynInferError(f"tp_exchange `{tp_exchange}` unknown (peer | nccl)")
        self.tp_exchange = tp_exchange
        self.coverage, self.max_kv, self.kv_dtype, self.chunk_size = coverage, max_kv, kv_dtype, chunk_size
        # "persistent": one cooperative kernel per decoded token; "graph": a captured graph of
        # per-operator kernels (the path multi-row chunks always take)
        self.decode_kernel = decode_kernel
        c = catalog.config
        self.metadata = {"architecture": c.get("model_type", "qwen3"), "vocabulary_size": c["vocab"],
                         "context_length": c.get("context_length", 0), "pad_token_id": 0}

    def target_profile(self) -> reg.TargetProfile:
        return self.target

    def create_session(self, config: SessionConfig | None = None) -> CudaSession:
        return CudaSession(self, config or SessionConfig())

    def create_batched_session(self, config: SessionConfig) -> "BatchedCudaSession":
        return BatchedCudaSession(self, config)


class BatchedCudaSession(CudaSession):
    """`config.batch_size` independent sequences sharing one weight upload and one KV pool (one
    slot each). Extension of the cuda target: the reference session is batch 1. Prefill runs per
    slot through the chunk call; `step` decodes every active slot in one pass over the weights."""

    def __init__(self, model: "LoadedModel", config: SessionConfig):
        if config.batch_size < 1:
            raise DynInferError("batch_size must be >= 1")
        super().__init__(model, config)
        self.slots = int(config.batch_size)
        self.positions = [0] * self.slots

    def _require_batch_1(self):      # the single-sequence calls keep working on slot 0 only
        return None

    def prefill_slot(self, slot: int, tokens, want_logits: bool = False):
        """Greedy first token (and optionally logits) of `tokens` placed in KV slot `slot` from position 0."""
        tokens = [int(t) for t in tokens]
        if not 0 <= slot < self.slots:
            raise DynInferError(f"slot {slot} outside [0, {self.slots})")
        if not tokens or len(tokens) > self._max_seq():
            raise DynInferError(f"prefill length {len(tokens)} outside [1, {self._max_seq()}]")
        self._ensure_pages()
        cs = self.model.chunk_size
        logits, token = None, -1
        for ci in range(0, len(tokens), cs):
            window, last = self._window(tokens[ci:ci + cs])
            final = ci + cs >= len(tokens)
            ptr, count, tok = C.POINTER(C.c_float)(), C.c_size_t(0), C.c_int64(-1)
            check(lib().dyninfer_cuda_session_invoke_paged_chunk_slot(
                self._h, window.ctypes.data_as(C.POINTER(C.c_int64)), window.size, int(last), ci, int(slot),
                C.byref(ptr), C.byref(count), C.byref(tok), 1 if (want_logits and final) else 0))
            token = int(tok.value)
            if want_logits and final:
                logits = np.ctypeslib.as_array(ptr, shape=(count.value,)).copy()
        self.positions[slot] = len(tokens)
        return (logits, token) if want_logits else token

    def step(self, tokens: dict, want_logits: bool = False):
        """One decode step: `tokens` maps slot -> token to feed. Returns slot -> next token
        (and slot -> logits when asked)."""
        slots = sorted(int(s) for s in tokens)
        if not slots:
            return ({}, {}) if want_logits else {}
        for s in slots:
            if not 0 <= s < self.slots:
                raise DynInferError(f"slot {s} outside [0, {self.slots})")
            if self.positions[s] >= self._max_seq():
                raise DynInferError(f"slot {s}: decode position {self.positions[s]} exceeds session/KV limit {self._max_seq()}")
        self._ensure_pages()
        n = len(slots)
        tok = np.array([int(tokens[s]) for s in slots], dtype=np.int64)
        pos = np.array([self.positions[s] for s in slots], dtype=np.int64)
        sl = np.array(slots, dtype=np.int64)
        out = np.empty(n, dtype=np.int64)
        ptr = C.POINTER(C.c_float)()
        i64p = C.POINTER(C.c_int64)
        check(lib().dyninfer_cuda_session_decode_batch(
            self._h, tok.ctypes.data_as(i64p), pos.ctypes.data_as(i64p), sl.ctypes.data_as(i64p), n,
            out.ctypes.data_as(i64p), C.byref(ptr), 1 if want_logits else 0))
        for s in slots:
            self.positions[s] += 1
        nxt = {s: int(out[i]) for i, s in enumerate(slots)}
        if not want_logits:
            return nxt
        vocab = self.metadata["vocabulary_size"]
        lg = np.ctypeslib.as_array(ptr, shape=(n, vocab)).copy()
        return nxt, {s: lg[i] for i, s in enumerate(slots)}

    def reset(self):
        super().reset()
        self.positions = [0] * self.slots


class ModelLoader:
    """bind -> kernel_coverage (strict) -> provider plan -> LoadedModel."""

    def __init__(self, registry: reg.KernelRegistry | None = None):
        self.registry = registry or reg.default_registry()

    @staticmethod
    def resolve_target(spec: str):
        """`cuda`, `cuda:<ordinal>`, `cuda:sm_100a`. Never resolves to a CPU target
        (crates/dyninfer-target/src/lib.rs:73-111)."""
        if not spec.startswith("cuda"):
            raise DynInferError(f"target `{spec}` is not served by this library (cuda only, no CPU fallback)")
        rest = spec[5:] if spec.startswith("cuda:") else ""
        if rest.startswith("sm_"):
            return reg.TargetProfile.cuda(rest), "cuda:0"
        return reg.TargetProfile.cuda("sm_100a"), f"cuda:{rest or 0}"

    def bind(self, path: str) -> ck.Catalog:
        return ck.open_catalog(path)

    def kernel_coverage(self, catalog: ck.Catalog, target: reg.TargetProfile) -> reg.CoverageReport:
        params = {n: (p.encoding, p.shape) for n, p in catalog.parameters.items()}
        return reg.dry_run_coverage(catalog.config, params, target, self.registry)

    def load(self, path: str, target: str = "cuda", max_kv: int = 2048, kv_dtype: str = "f32",
             chunk_size: int = CHUNK_SIZE, decode_kernel: str = "persistent",
             tp: tuple | None = None, tp_exchange: str = "peer") -> LoadedModel:
        profile, uri = self.resolve_target(target)
        catalog = self.bind(path)
        coverage = self.kernel_coverage(catalog, profile).require_complete()
        plan = ck.build_runtime_provider_plan(catalog)
        return LoadedModel(catalog, plan, profile, uri, coverage, max_kv, kv_dtype, chunk_size, decode_kernel, tp,
                           tp_exchange)


# ----------------------------------------------------------------------- generation

@dataclass
class GenerateConfig:
    max_new_tokens: int = 48
    eos_token_id: int | None = None
    stop_token_ids: list = field(default_factory=list)
    repetition_penalty: float = 1.0


@dataclass
class GenerateStats:
    prompt_tokens: int
    generated_tokens: int
    prefill_secs: float
    decode_secs: float
    kv: KvCacheMetrics

    def prefill_tps(self):
        return self.prompt_tokens / self.prefill_secs if self.prefill_secs > 0 else 0.0

    def decode_tps(self):
        return self.generated_tokens / self.decode_secs if self.decode_secs > 0 else 0.0


def apply_repetition_penalty(logits: np.ndarray, seen: dict, penalty: float):
    if abs(penalty - 1.0) < np.finfo(np.float32).eps or not seen:
        return
    for t in seen:
        if t < logits.size:
            logits[t] = logits[t] * penalty if logits[t] < 0 else logits[t] / penalty


def generate_greedy(model: LoadedModel, prompt_ids, config: GenerateConfig | None = None,
                    session_cfg: SessionConfig | None = None):
    """Greedy continuation of `prompt_ids`; returns (all token ids, GenerateStats)."""
    config = config or GenerateConfig()
    ids = [int(t) for t in prompt_ids]
    if not ids:
        raise DynInferError("prompt produced no tokens")
    stop = list(config.stop_token_ids)
    if config.eos_token_id is not None and config.eos_token_id not in stop:
        stop.append(config.eos_token_id)
    seen: dict = {}
    for t in ids:
        seen[t] = seen.get(t, 0) + 1
    n_prompt = len(ids)
    generated = []
    with model.create_session(session_cfg) as session:
        t0 = time.perf_counter()
        if abs(config.repetition_penalty - 1.0) < np.finfo(np.float32).eps:
            nxt = session.prefill_argmax(ids)
            prefill_secs = time.perf_counter() - t0
            t1 = time.perf_counter()
            for _ in range(config.max_new_tokens):
                if nxt in stop:
                    break
                generated.append(nxt)
                ids.append(nxt)
                nxt = session.decode_argmax(nxt)
            decode_secs = time.perf_counter() - t1
        else:
            logits = session.prefill(ids).values
            prefill_secs = time.perf_counter() - t0
            t1 = time.perf_counter()
            for _ in range(config.max_new_tokens):
                apply_repetition_penalty(logits, seen, config.repetition_penalty)
                nxt = argmax(logits)
                if nxt in stop:
                    break
                generated.append(nxt)
                ids.append(nxt)
                seen[nxt] = seen.get(nxt, 0) + 1
                logits = session.decode(nxt).values
            decode_secs = time.perf_counter() - t1
        kv = session.kv_cache_metrics()
    return ids, GenerateStats(n_prompt, len(generated), prefill_secs, decode_secs, kv)


# ------------------------------------------------------------------------------ perf

@dataclass
class PerfConfig:
    prefill_tokens: int = 128
    tg: int = 32
    warmup: int = 1
    iters: int = 1
    weight_bytes: int = 0
    fill_token: int = 1


def run_perf(model: LoadedModel, config: PerfConfig, session_cfg: SessionConfig | None = None) -> dict:
    """Synthetic-token prefill + decode through the public session calls, wall-clock timed
    like the reference; eff_weight_bw_gbs = weight_bytes * weight_passes / secs / 1e9."""
    if config.prefill_tokens == 0:
        raise DynInferError("perf --prefill must be > 0")
    if config.iters == 0:
        raise DynInferError("perf --iters must be > 0")
    prompt = [config.fill_token] * config.prefill_tokens
    pre, dec = [], []
    with model.create_session(session_cfg) as s:
        for _ in range(config.warmup):
            s.reset()
            nxt = s.prefill_argmax(prompt)
            for _ in range(config.tg):
                nxt = s.decode_argmax(nxt)
        for _ in range(config.iters):
            s.reset()
            t0 = time.perf_counter()
            nxt = s.prefill_argmax(prompt)
            pre.append(time.perf_counter() - t0)
            t0 = time.perf_counter()
            for _ in range(config.tg):
                nxt = s.decode_argmax(nxt)
            dec.append(time.perf_counter() - t0)
        kv, alloc = s.kv_cache_metrics(), s.allocator_metrics()
    wb = config.weight_bytes

    def phase(tokens, secs, passes):
        mean = sum(secs) / len(secs)
        return {"tokens": tokens, "secs": mean, "tps": tokens / mean if mean > 0 else 0.0,
                "eff_weight_bw_gbs": (wb * passes / mean / 1e9) if wb and mean > 0 else None,
                "kv_page_count": kv.page_count, "kv_allocated_bytes": kv.allocated_bytes,
                "device_live_bytes": alloc.device_live_bytes(), "device_bytes_peak": alloc.device_bytes_peak}

    chunks = -(-config.prefill_tokens // model.chunk_size)
    return {"prefill": phase(config.prefill_tokens, pre, chunks), "decode": phase(config.tg, dec, config.tg),
            "warmup": config.warmup, "iters": config.iters, "weight_bytes": wb}
