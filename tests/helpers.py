"""Shared test plumbing: fixture tensors -> oracle weights / checkpoint files."""
import json
import os

import numpy as np

from dyninfer_b200 import checkpoint as ck

_ST = {"plain.f32": "F32", "plain.f16": "F16", "plain.bf16": "BF16"}


def oracle_weights(orc, tensors):
    out = {}
    for name, t in tensors.items():
        shape = t["shape"]
        rows, cols = (shape if len(shape) == 2 else (1, shape[0]))
        out[name] = orc.Weight(t["enc"], rows, cols, t["data"], t.get("scales"), t.get("biases"),
                               t.get("aux", "plain.bf16"), t.get("group", 64))
    return out


def catalog_weights(orc, cat):
    """Oracle weights straight from a checkpoint file's byte ranges (what the GPU uploads)."""
    return orc.weights_from_catalog(cat)


def write_fixture_gguf(path, cfg, tensors, arch="qwen3"):
    meta = {"general.architecture": arch, f"{arch}.block_count": cfg["layers"],
            f"{arch}.embedding_length": cfg["hidden"], f"{arch}.feed_forward_length": cfg["intermediate"],
            f"{arch}.attention.head_count": cfg["heads"], f"{arch}.attention.head_count_kv": cfg["kv_heads"],
            f"{arch}.attention.key_length": cfg["head_dim"], f"{arch}.vocab_size": cfg["vocab"],
            f"{arch}.attention.layer_norm_rms_epsilon": float(cfg["eps"]),
            f"{arch}.rope.freq_base": float(cfg["theta"]), "dyninfer.rope": int(cfg.get("rope", True))}
    t = {n: (tuple(v["shape"]), ck.GGML_CODE[v["enc"]], v["data"]) for n, v in tensors.items()}
    ck.write_gguf(path, meta, t)
    return path


_HF = {v: k for k, v in ck._HF_LAYER.items()}


def _hf_name(canon):
    stem = canon[:-len(".weight")]
    if stem == "token_embd":
        return "model.embed_tokens"
    if stem == "output_norm":
        return "model.norm"
    if stem == "output":
        return "lm_head"
    _, n, slot = stem.split(".", 2)
    return f"model.layers.{n}.{_HF[slot]}"


def write_fixture_mlx(dirpath, cfg, tensors):
    os.makedirs(dirpath, exist_ok=True)
    t = {}
    for canon, v in tensors.items():
        hf = _hf_name(canon)
        if v["enc"] == "mlx.affine.u4":
            r, c = v["shape"]
            aux = _ST[v.get("aux", "plain.bf16")]
            t[hf + ".weight"] = ("U32", (r, c // 8), v["data"])
            t[hf + ".scales"] = (aux, (r, c // v["group"]), np.ascontiguousarray(v["scales"]))
            t[hf + ".biases"] = (aux, (r, c // v["group"]), np.ascontiguousarray(v["biases"]))
        else:
            t[hf + ".weight"] = (_ST[v["enc"]], tuple(v["shape"]), v["data"])
    ck.write_safetensors(os.path.join(dirpath, "model.safetensors"), t, {"format": "mlx"})
    hf_cfg = {"model_type": "qwen3", "num_hidden_layers": cfg["layers"], "hidden_size": cfg["hidden"],
              "intermediate_size": cfg["intermediate"], "num_attention_heads": cfg["heads"],
              "num_key_value_heads": cfg["kv_heads"], "head_dim": cfg["head_dim"],
              "vocab_size": cfg["vocab"], "rms_norm_eps": cfg["eps"], "rope_theta": cfg["theta"],
              "quantization": {"group_size": 64, "bits": 4}}
    with open(os.path.join(dirpath, "config.json"), "w") as f:
        json.dump(hf_cfg, f)
    return dirpath


def rel_err(a, b):
    """max |a-b| / max |b| — the relative error the GEMV/GEMM tolerance (1e-3) is stated in."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def cosine(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def bits_equal(a, b):
    """Bit-for-bit equality of two f32 arrays; NaNs must sit in the same places but their
    payload bits are not compared (a NaN scale in a block makes x86 and the GPU pick
    different, equally valid, quiet-NaN encodings)."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    na, nb = np.isnan(a), np.isnan(b)
    return a.shape == b.shape and np.array_equal(na, nb) and \
        np.array_equal(a.view(np.uint32)[~na], b.view(np.uint32)[~nb])
