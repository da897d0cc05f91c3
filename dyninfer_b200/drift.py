"""Logit drift between two engines: per-row metrics and the versioned logit-trace files.

Mirrors the reference's drift tooling for the cuda target: the metric set of
`crates/dyninfer-cli/src/drift.rs:22-41` (computed in f64, stable softmax) and the trace layout of
`crates/dyninfer-cli/src/logit_trace.rs` (a directory with `trace.json` + one little-endian f32
row of `vocab_size` logits per step: row 0 is the last prompt position, row i >= 1 feeds
`decode_inputs[i-1]` at position `len(prompt) + i - 1`; `forced_token` of row i is the token fed
next, so both engines walk the same trajectory).

    python -m dyninfer_b200.drift record  --model M.gguf --prompt 1,2,3 --decode 7,8,9 --out DIR
    python -m dyninfer_b200.drift compare --reference DIR_A --dyninfer DIR_B [--top-k 10]

`record` runs the cuda target; any other engine that writes the same layout can be the other side.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import shutil

import numpy as np

TRACE_FORMAT = "dyninfer.logit-trace"
TRACE_VERSION = 1


class DriftError(ValueError):
    pass


# ------------------------------------------------------------------------------ row metrics

def _descending(values: np.ndarray) -> np.ndarray:
    """Indices by descending value, ties by ascending index (drift.rs:186-193)."""
    return np.lexsort((np.arange(values.size), -values.astype(np.float64)))


def _logsumexp(v64: np.ndarray) -> float:
    m = float(v64.max())
    return m + math.log(float(np.exp(v64 - m).sum()))


def compare(reference, dyninfer, top_k: int = 10) -> dict:
    """Drift of one logit row, field for field the reference's `RowMetrics` (drift.rs:44-184)."""
    ref = np.asarray(reference, dtype=np.float32).reshape(-1)
    dyn = np.asarray(dyninfer, dtype=np.float32).reshape(-1)
    if ref.size == 0:
        raise DriftError("cannot compare empty logit rows")
    if ref.size != dyn.size:
        raise DriftError(f"logit row width mismatch: reference {ref.size}, dyninfer {dyn.size}")
    if top_k <= 0:
        raise DriftError("top-k must be greater than zero")
    for engine, values in (("reference", ref), ("dyninfer", dyn)):
        bad = np.flatnonzero(~np.isfinite(values))
        if bad.size:
            raise DriftError(f"{engine} logit {int(bad[0])} is non-finite: {values[bad[0]]}")
    r, d = ref.astype(np.float64), dyn.astype(np.float64)
    n = float(ref.size)
    delta = d - r
    absd = np.abs(delta)
    sse = float((delta * delta).sum())
    mean_signed = float(delta.sum()) / n
    rn, dn = math.sqrt(float((r * r).sum())), math.sqrt(float((d * d).sum()))
    if rn == 0.0 or dn == 0.0:
        cosine = 1.0 if (rn == 0.0 and dn == 0.0) else 0.0
    else:
        cosine = min(1.0, max(-1.0, float((r * d).sum()) / (rn * dn)))
    k = min(top_k, ref.size)
    ri, di = _descending(ref), _descending(dyn)
    overlap = int(np.intersect1d(ri[:k], di[:k]).size)
    rl, dl = r - _logsumexp(r), d - _logsumexp(d)
    rp, dp = np.exp(rl), np.exp(dl)
    kl = float((rp * (rl - dl)).sum())
    if -1.0e-12 < kl < 0.0:      # roundoff can make a zero KL a few ulps negative
        kl = 0.0
    worst = np.lexsort((np.arange(ref.size), -absd))[:k]
    return {
        "max_absolute_error": float(absd.max()),
        "mean_absolute_error": float(absd.sum()) / n,
        "rmse": math.sqrt(sse / n),
        "mean_signed_delta": mean_signed,
        "relative_l2_error": math.sqrt(sse) / max(rn, np.finfo(np.float64).eps),
        "cosine_similarity": cosine,
        "centered_rmse": math.sqrt(float(((delta - mean_signed) ** 2).sum()) / n),
        "reference_argmax": int(ri[0]),
        "dyninfer_argmax": int(di[0]),
        "argmax_match": bool(ri[0] == di[0]),
        "top_k": k,
        "top_k_overlap": overlap,
        "top_k_overlap_fraction": overlap / k,
        "softmax_kl_reference_dyninfer": kl,
        "max_probability_delta": float(np.abs(rp - dp).max()),
        "largest_deltas": [{"token_id": int(i), "reference": float(ref[i]), "dyninfer": float(dyn[i]),
                            "delta": float(delta[i]), "absolute_delta": float(absd[i])} for i in worst],
        "reference_top": [{"token_id": int(i), "logit": float(ref[i])} for i in ri[:k]],
        "dyninfer_top": [{"token_id": int(i), "logit": float(dyn[i])} for i in di[:k]],
    }


# ------------------------------------------------------------------------------ trace files

def first_strict_argmax(values: np.ndarray) -> int:
    return int(np.argmax(values))        # numpy returns the first maximum, like `value > best`


def _expected_row(prompt, decode, index):
    if index == 0:
        return "prefill", len(prompt) - 1, int(prompt[-1])
    return "decode", len(prompt) + index - 1, int(decode[index - 1])


def validate_header(h: dict) -> None:
    """The reader-side rules of logit_trace.rs:330-398, same wording."""
    if h.get("format") != TRACE_FORMAT:
        raise DriftError(f"unsupported trace format {h.get('format')!r}")
    if h.get("version") != TRACE_VERSION:
        raise DriftError(f"unsupported trace version {h.get('version')}")
    if not str(h.get("engine", "")).strip():
        raise DriftError("trace engine is empty")
    sha = str(h.get("checkpoint_sha256", ""))
    if len(sha) != 64 or any(c not in "0123456789abcdefABCDEF" for c in sha):
        raise DriftError("checkpoint_sha256 must contain 64 hexadecimal characters")
    vocab = int(h.get("vocab_size", 0))
    if vocab <= 0:
        raise DriftError("trace vocabulary is empty")
    if h.get("logits_dtype") != "f32":
        raise DriftError(f"unsupported logits dtype {h.get('logits_dtype')!r}")
    if h.get("logits_byte_order") != "little":
        raise DriftError(f"unsupported logits byte order {h.get('logits_byte_order')!r}")
    lf = str(h.get("logits_file", ""))
    if not lf or lf in (".", "..") or "/" in lf or "\\" in lf:
        raise DriftError("logits_file must be a plain relative file name")
    prompt, decode = list(h.get("prompt_tokens", [])), list(h.get("decode_inputs", []))
    if not prompt:
        raise DriftError("trace prompt token list is empty")
    for kind, toks in (("prompt", prompt), ("decode", decode)):
        for i, t in enumerate(toks):
            if not 0 <= int(t) < vocab:
                raise DriftError(f"{kind} token {i} ({t}) is outside vocabulary {vocab}")
    rows = h.get("rows", [])
    if len(rows) != len(decode) + 1:
        raise DriftError(f"trace row count mismatch: expected {len(decode) + 1}, found {len(rows)}")
    for i, row in enumerate(rows):
        phase, pos, inp = _expected_row(prompt, decode, i)
        if row.get("phase") != phase:
            raise DriftError(f"trace row {i} has inconsistent phase")
        if row.get("position") != pos:
            raise DriftError(f"trace row {i} has discontinuous position {row.get('position')} (expected {pos})")
        if row.get("input_token") != inp:
            raise DriftError(f"trace row {i} input token {row.get('input_token')} does not match trajectory token {inp}")
        if not 0 <= int(row.get("argmax", -1)) < vocab:
            raise DriftError(f"trace row {i} argmax {row.get('argmax')} is outside vocabulary {vocab}")
        forced = decode[i] if i < len(decode) else None
        if row.get("forced_token") != forced:
            raise DriftError(f"trace row {i} forced token is inconsistent with decode_inputs")


class TraceWriter:
    """Writes a trace into `<directory>.tmp-<pid>` and renames it into place on `finish`
    (logit_trace.rs:172-318); an unfinished trace leaves nothing behind."""

    def __init__(self, directory: str, engine: str, checkpoint_sha256: str, vocab_size: int, prompt_tokens,
                 decode_inputs, logits_file: str = "logits.f32", engine_metadata=None):
        self.directory = directory
        self.tmp = f"{directory.rstrip('/')}.tmp-{os.getpid()}"
        self.header = {"format": TRACE_FORMAT, "version": TRACE_VERSION, "engine": engine,
                       "checkpoint_sha256": checkpoint_sha256, "vocab_size": int(vocab_size),
                       "prompt_tokens": [int(t) for t in prompt_tokens],
                       "decode_inputs": [int(t) for t in decode_inputs], "logits_dtype": "f32",
                       "logits_byte_order": "little", "rows": [], "logits_file": logits_file}
        if engine_metadata is not None:
            self.header["engine_metadata"] = engine_metadata
        if os.path.exists(directory):
            raise DriftError(f"trace directory {directory} already exists")
        os.makedirs(self.tmp)
        self._f = open(os.path.join(self.tmp, logits_file), "wb")
        self.finished = False

    def write_row(self, logits) -> int:
        v = np.ascontiguousarray(logits, dtype="<f4").reshape(-1)
        i = len(self.header["rows"])
        if v.size != self.header["vocab_size"]:
            raise DriftError(f"trace row {i} has {v.size} logits, vocabulary is {self.header['vocab_size']}")
        if not np.isfinite(v).all():
            raise DriftError(f"trace row {i} token {int(np.flatnonzero(~np.isfinite(v))[0])} is non-finite")
        if i > len(self.header["decode_inputs"]):
            raise DriftError(f"trace has unexpected row {i}")
        phase, pos, inp = _expected_row(self.header["prompt_tokens"], self.header["decode_inputs"], i)
        row = {"phase": phase, "position": pos, "input_token": inp, "argmax": first_strict_argmax(v)}
        if i < len(self.header["decode_inputs"]):
            row["forced_token"] = self.header["decode_inputs"][i]
        self.header["rows"].append(row)
        self._f.write(v.tobytes())
        return row["argmax"]

    def finish(self) -> str:
        self._f.close()
        validate_header(self.header)
        with open(os.path.join(self.tmp, "trace.json"), "w") as f:
            json.dump(self.header, f, indent=2)
        os.replace(self.tmp, self.directory)
        self.finished = True
        return self.directory

    def abort(self):
        if not self.finished and os.path.isdir(self.tmp):
            self._f.close()
            shutil.rmtree(self.tmp, ignore_errors=True)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, *a):
        if exc_type is not None:
            self.abort()


class TraceReader:
    def __init__(self, directory: str):
        hp = os.path.join(directory, "trace.json")
        with open(hp) as f:
            self.header = json.load(f)
        validate_header(self.header)
        lp = os.path.join(directory, self.header["logits_file"])
        expected = len(self.header["rows"]) * int(self.header["vocab_size"]) * 4
        actual = os.path.getsize(lp)
        if actual != expected:
            raise DriftError(f"trace logits size mismatch: expected {expected} bytes, found {actual} "
                             "(truncated or trailing data)")
        self._f = open(lp, "rb")
        self.next = 0

    def next_row(self) -> np.ndarray:
        if self.next >= len(self.header["rows"]):
            raise DriftError(f"trace has no row {self.next}")
        v = np.frombuffer(self._f.read(int(self.header["vocab_size"]) * 4), dtype="<f4").astype(np.float32)
        bad = np.flatnonzero(~np.isfinite(v))
        if bad.size:
            raise DriftError(f"trace row {self.next} token {int(bad[0])} is non-finite: {v[bad[0]]}")
        got, want = first_strict_argmax(v), self.header["rows"][self.next]["argmax"]
        if got != want:
            raise DriftError(f"trace row {self.next} argmax mismatch: metadata {want}, logits {got}")
        self.next += 1
        return v

    def finish(self):
        left = len(self.header["rows"]) - self.next
        self._f.close()
        if left:
            raise DriftError(f"trace has {left} unread rows")


def sha256_of(path: str) -> str:
    files = [path] if os.path.isfile(path) else sorted(
        os.path.join(path, f) for f in os.listdir(path) if os.path.isfile(os.path.join(path, f)))
    h = hashlib.sha256()
    for p in files:
        with open(p, "rb") as f:
            for blk in iter(lambda: f.read(1 << 22), b""):
                h.update(blk)
    return h.hexdigest()


def record(session, directory: str, engine: str, checkpoint_sha256: str, prompt_tokens, decode_inputs,
           engine_metadata=None) -> str:
    """Walk `session` (prefill / decode returning logits, the `ModelSession` calls) along the given
    trajectory and write its trace."""
    vocab = int(session.metadata["vocabulary_size"])
    with TraceWriter(directory, engine, checkpoint_sha256, vocab, prompt_tokens, decode_inputs,
                     engine_metadata=engine_metadata) as w:
        w.write_row(session.prefill(list(prompt_tokens)).values)
        for t in decode_inputs:
            w.write_row(session.decode(int(t)).values)
        return w.finish()


def compare_traces(reference_dir: str, dyninfer_dir: str, top_k: int = 10) -> dict:
    """Row-by-row drift of two traces of the same trajectory plus a summary (worst row per metric)."""
    a, b = TraceReader(reference_dir), TraceReader(dyninfer_dir)
    for key in ("checkpoint_sha256", "vocab_size", "prompt_tokens", "decode_inputs"):
        if a.header[key] != b.header[key]:
            raise DriftError(f"traces differ in {key}: they do not follow the same trajectory")
    rows = []
    for i, meta in enumerate(a.header["rows"]):
        m = compare(a.next_row(), b.next_row(), top_k)
        m.update(row=i, phase=meta["phase"], position=meta["position"])
        rows.append(m)
    a.finish()
    b.finish()
    return {
        "reference_engine": a.header["engine"], "dyninfer_engine": b.header["engine"], "rows": rows,
        "summary": {
            "row_count": len(rows),
            "max_absolute_error": max(r["max_absolute_error"] for r in rows),
            "max_rmse": max(r["rmse"] for r in rows),
            "min_cosine_similarity": min(r["cosine_similarity"] for r in rows),
            "max_softmax_kl": max(r["softmax_kl_reference_dyninfer"] for r in rows),
            "argmax_mismatches": sum(0 if r["argmax_match"] else 1 for r in rows),
            "min_top_k_overlap_fraction": min(r["top_k_overlap_fraction"] for r in rows),
        },
    }


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("record", help="run the cuda target along a trajectory and write its trace")
    r.add_argument("--model", required=True)
    r.add_argument("--prompt", required=True, help="comma-separated token ids")
    r.add_argument("--decode", default="", help="comma-separated forced decode inputs")
    r.add_argument("--out", required=True)
    r.add_argument("--target", default="cuda")
    r.add_argument("--kv-dtype", default="f32")
    c = sub.add_parser("compare", help="drift metrics of two traces of the same trajectory")
    c.add_argument("--reference", required=True)
    c.add_argument("--dyninfer", required=True)
    c.add_argument("--top-k", type=int, default=10)
    args = ap.parse_args()
    if args.cmd == "compare":
        print(json.dumps(compare_traces(args.reference, args.dyninfer, args.top_k)["summary"]))
        return
    from .runtime import ModelLoader, SessionConfig
    prompt = [int(t) for t in args.prompt.split(",") if t.strip()]
    decode = [int(t) for t in args.decode.split(",") if t.strip()]
    n = len(prompt) + len(decode) + 1
    model = ModelLoader().load(args.model, target=args.target, max_kv=n, kv_dtype=args.kv_dtype)
    with model.create_session(SessionConfig(max_sequence_length=n)) as s:
        print(record(s, args.out, "dyninfer-cuda-sm_100a", sha256_of(args.model), prompt, decode,
                     engine_metadata={"kv_dtype": args.kv_dtype, "target": args.target}))


if __name__ == "__main__":
    main()
