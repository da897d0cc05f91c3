"""Drift metrics and logit-trace files (host logic; the properties the reference's own unit tests pin,
`crates/dyninfer-cli/src/drift.rs` and `logit_trace.rs` test modules)."""
import json
import os

import numpy as np
import pytest

from dyninfer_b200 import drift

SHA = "0123456789abcdef" * 4


def test_identical_rows_have_zero_drift():
    m = drift.compare([1.0, 3.0, -2.0], [1.0, 3.0, -2.0], 2)
    assert m["max_absolute_error"] == 0.0 and m["rmse"] == 0.0 and m["centered_rmse"] == 0.0
    assert m["cosine_similarity"] == 1.0 and m["softmax_kl_reference_dyninfer"] == 0.0
    assert m["argmax_match"] and m["top_k_overlap"] == 2


def test_constant_offset_is_removed_by_centering():
    m = drift.compare([-1.0, 0.0, 2.0], [4.0, 5.0, 7.0], 3)
    assert abs(m["mean_signed_delta"] - 5.0) < 1e-12 and m["centered_rmse"] < 1e-12
    assert m["softmax_kl_reference_dyninfer"] < 1e-12 and m["argmax_match"]


def test_scale_and_argmax_changes_are_detected():
    assert abs(drift.compare([1.0, 2.0, 3.0], [2.0, 4.0, 6.0], 2)["relative_l2_error"] - 1.0) < 1e-12
    c = drift.compare([3.0, 2.0], [1.0, 4.0], 1)
    assert not c["argmax_match"] and (c["reference_argmax"], c["dyninfer_argmax"]) == (0, 1)


def test_large_logits_and_rejections():
    m = drift.compare([3.0e38, 3.0e38 - 1.0e32], [3.0e38, 3.0e38], 2)
    assert np.isfinite(m["softmax_kl_reference_dyninfer"]) and np.isfinite(m["max_probability_delta"])
    with pytest.raises(drift.DriftError, match="non-finite"):
        drift.compare([0.0, float("nan")], [0.0, 1.0], 1)
    with pytest.raises(drift.DriftError, match="width mismatch"):
        drift.compare([0.0, 1.0], [0.0], 1)
    with pytest.raises(drift.DriftError, match="empty"):
        drift.compare([], [], 1)
    with pytest.raises(drift.DriftError, match="top-k"):
        drift.compare([0.0], [0.0], 0)


def test_metrics_against_a_direct_f64_computation():
    rng = np.random.default_rng(3)
    r = rng.normal(size=257).astype(np.float32)
    d = (r + rng.normal(scale=1e-2, size=257)).astype(np.float32)
    m = drift.compare(r, d, 10)
    r64, d64 = r.astype(np.float64), d.astype(np.float64)
    assert abs(m["rmse"] - np.sqrt(np.mean((d64 - r64) ** 2))) < 1e-12
    assert abs(m["cosine_similarity"] - (r64 @ d64) / np.linalg.norm(r64) / np.linalg.norm(d64)) < 1e-12
    p = np.exp(r64 - r64.max()); p /= p.sum()
    q = np.exp(d64 - d64.max()); q /= q.sum()
    assert abs(m["softmax_kl_reference_dyninfer"] - float(np.sum(p * np.log(p / q)))) < 1e-10
    assert m["largest_deltas"][0]["absolute_delta"] == m["max_absolute_error"]
    assert [t["token_id"] for t in m["reference_top"]] == list(np.argsort(-r64, kind="stable")[:10])


def _write(tmp_path, name, rows, prompt=(1, 2, 3), decode=(4, 5), vocab=8, engine="a"):
    w = drift.TraceWriter(str(tmp_path / name), engine, SHA, vocab, prompt, decode)
    for r in rows:
        w.write_row(r)
    return w.finish()


def test_trace_round_trip_and_comparison(tmp_path):
    rng = np.random.default_rng(1)
    rows = rng.normal(size=(3, 8)).astype(np.float32)
    a = _write(tmp_path, "a", rows)
    b = _write(tmp_path, "b", rows + np.float32(1e-3), engine="b")
    h = json.load(open(os.path.join(a, "trace.json")))
    assert h["format"] == "dyninfer.logit-trace" and h["version"] == 1 and h["logits_dtype"] == "f32"
    assert [r["phase"] for r in h["rows"]] == ["prefill", "decode", "decode"]
    assert [r["position"] for r in h["rows"]] == [2, 3, 4] and [r["input_token"] for r in h["rows"]] == [3, 4, 5]
    assert [r.get("forced_token") for r in h["rows"]] == [4, 5, None]
    assert os.path.getsize(os.path.join(a, h["logits_file"])) == 3 * 8 * 4
    rd = drift.TraceReader(a)
    got = [rd.next_row() for _ in range(3)]
    rd.finish()
    assert all(np.array_equal(g, r) for g, r in zip(got, rows))
    rep = drift.compare_traces(a, b, 3)
    assert rep["summary"]["row_count"] == 3 and rep["summary"]["argmax_mismatches"] == 0
    assert abs(rep["summary"]["max_absolute_error"] - 1e-3) < 1e-6
    assert not [p for p in os.listdir(tmp_path) if ".tmp-" in p]


def test_trace_validation(tmp_path):
    rows = np.arange(24, dtype=np.float32).reshape(3, 8)
    a = _write(tmp_path, "a", rows)
    hp = os.path.join(a, "trace.json")
    good = json.load(open(hp))

    def broken(**kw):
        h = json.loads(json.dumps(good))
        h.update(kw)
        json.dump(h, open(hp, "w"))
        return a

    with pytest.raises(drift.DriftError, match="unsupported trace version"):
        drift.TraceReader(broken(version=2))
    with pytest.raises(drift.DriftError, match="64 hexadecimal"):
        drift.TraceReader(broken(checkpoint_sha256="abc"))
    with pytest.raises(drift.DriftError, match="plain relative file name"):
        drift.TraceReader(broken(logits_file="../x"))
    with pytest.raises(drift.DriftError, match="row count mismatch"):
        drift.TraceReader(broken(decode_inputs=[4]))
    rows_bad = json.loads(json.dumps(good["rows"]))
    rows_bad[1]["position"] = 9
    with pytest.raises(drift.DriftError, match="discontinuous position"):
        drift.TraceReader(broken(rows=rows_bad))
    rows_bad = json.loads(json.dumps(good["rows"]))
    rows_bad[0]["argmax"] = 0
    rd = drift.TraceReader(broken(rows=rows_bad))
    with pytest.raises(drift.DriftError, match="argmax mismatch"):
        rd.next_row()
    json.dump(good, open(hp, "w"))
    with open(os.path.join(a, good["logits_file"]), "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(drift.DriftError, match="size mismatch"):
        drift.TraceReader(a)
    # a writer that is abandoned leaves nothing behind; a short trace is refused at finish
    w = drift.TraceWriter(str(tmp_path / "c"), "e", SHA, 8, [1], [2])
    w.write_row(rows[0])
    with pytest.raises(drift.DriftError, match="row count mismatch"):
        w.finish()
    w.abort()
    assert not os.path.exists(tmp_path / "c") and not [p for p in os.listdir(tmp_path) if ".tmp-" in p]
    with pytest.raises(drift.DriftError, match="outside vocabulary"):
        drift.TraceWriter(str(tmp_path / "d"), "e", SHA, 8, [1], [9]).finish()
