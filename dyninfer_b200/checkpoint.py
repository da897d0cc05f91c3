"""Checkpoint containers and the direct byte-range provider plan.

Mirrors, for the `cuda` target, what the reference does before it hands
weights to its runtime: index an unmodified GGUF or SafeTensors file, decode
each tensor into a logical parameter with a physical encoding, and produce one
`(external_key, file, offset, length)` entry per storage component. Nothing is
repacked: the device receives exactly these byte ranges.

Reference behaviour followed here:
  * GGUF v2/v3 index, reversed dims, data section aligned to
    `general.alignment` (default 32): crates/dyninfer-checkpoint-gguf/src/container.rs:179-343
  * GGUF type table (block sizes / bytes per block): crates/dyninfer-checkpoint-gguf/src/types.rs:137-201
  * metadata normalisation: crates/dyninfer-checkpoint-gguf/src/convention.rs:281-316
  * SafeTensors header: crates/dyninfer-checkpoint-safetensors/src/container.rs:87
  * MLX convention (`.weight` u32 + `.scales` + `.biases`): crates/dyninfer-checkpoint-safetensors/src/mlx.rs:52-261
  * external key "{scope}::{canonical}::{component}": crates/dyninfer-binding/src/lib.rs:247-250
  * provider plan, one contiguous range per component, sorted by key:
    crates/dyninfer-checkpoint/src/provider.rs:9-125
  * HF -> GGUF canonical names, tied lm_head: crates/dyninfer-architecture/src/naming.rs:37-96
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field

# ggml type code -> (encoding id, elements per block, bytes per block)
GGML_TYPES = {
    0: ("plain.f32", 1, 4),
    1: ("plain.f16", 1, 2),
    2: ("gguf.q4_0", 32, 18),
    3: ("gguf.q4_1", 32, 20),
    8: ("gguf.q8_0", 32, 34),
    12: ("gguf.q4_k", 256, 144),
    13: ("gguf.q5_k", 256, 176),
    14: ("gguf.q6_k", 256, 210),
    23: ("gguf.iq4_xs", 256, 136),
    30: ("plain.bf16", 1, 2),
}
GGML_CODE = {v[0]: k for k, v in GGML_TYPES.items()}
# Types the container can describe but for which no kernel is registered on any
# target (schema only): crates/dyninfer-quantization/src/quantizations/gguf_block.rs:184-316
GGML_SCHEMA_ONLY = {
    6: ("gguf.q5_0", 32, 22), 7: ("gguf.q5_1", 32, 24), 9: ("gguf.q8_1", 32, 36),
    10: ("gguf.q2_k", 256, 84), 11: ("gguf.q3_k", 256, 110), 15: ("gguf.q8_k", 256, 292),
    20: ("gguf.iq4_nl", 32, 18),
}

ST_DTYPES = {"F32": ("plain.f32", 4), "F16": ("plain.f16", 2), "BF16": ("plain.bf16", 2),
             "U32": ("u32", 4), "I64": ("i64", 8), "U8": ("u8", 1)}

PARAMETER_SCOPE = "weights"


class CheckpointError(ValueError):
    """Invalid or unsupported checkpoint (the reference's E_CHECKPOINT family)."""


def nbytes_for_shape(code: int, shape) -> int:
    name, block, size = GGML_TYPES.get(code) or GGML_SCHEMA_ONLY[code]
    numel = 1
    for d in shape:
        numel *= int(d)
    inner = int(shape[-1]) if len(shape) else 1
    if inner % block:
        raise CheckpointError(f"{name}: innermost dim {inner} not divisible by block {block}")
    return numel // block * size


# --------------------------------------------------------------------------- GGUF

_GGUF_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?",
                10: "<Q", 11: "<q", 12: "<d"}


def _w_str(buf: bytearray, s: str):
    b = s.encode("utf-8")
    buf += struct.pack("<Q", len(b)) + b


def write_gguf(path: str, metadata: dict, tensors: dict, alignment: int = 32) -> None:
    """Write a GGUF v3 file. tensors: name -> (logical shape, ggml type code, bytes-like).

    Same structure as the reference's fixture writer
    (crates/dyninfer-checkpoint-gguf/src/q4.rs:139-195): sorted names, reversed
    dims, per-tensor and data-section alignment of 32.
    """
    head = bytearray()
    head += b"GGUF" + struct.pack("<I", 3)
    head += struct.pack("<QQ", len(tensors), len(metadata))
    for k in sorted(metadata):
        v = metadata[k]
        _w_str(head, k)
        if isinstance(v, str):
            head += struct.pack("<I", 8)
            _w_str(head, v)
        elif isinstance(v, float):
            head += struct.pack("<If", 6, v)
        elif isinstance(v, int):
            if v < 2 ** 32:
                head += struct.pack("<II", 4, v)
            else:
                head += struct.pack("<IQ", 10, v)
        else:
            raise CheckpointError(f"unsupported metadata value for {k}")
    offsets = {}
    cursor = 0
    for name in sorted(tensors):
        shape, code, data = tensors[name]
        _w_str(head, name)
        head += struct.pack("<I", len(shape))
        for d in reversed(shape):
            head += struct.pack("<Q", int(d))
        head += struct.pack("<I", code)
        cursor = (cursor + alignment - 1) // alignment * alignment
        offsets[name] = cursor
        head += struct.pack("<Q", cursor)
        n = len(memoryview(data).cast("B"))
        if n != nbytes_for_shape(code, shape):
            raise CheckpointError(f"{name}: {n} bytes, expected {nbytes_for_shape(code, shape)}")
        cursor += n
    pad = (-len(head)) % alignment
    head += b"\0" * pad
    with open(path, "wb") as f:
        f.write(head)
        pos = 0
        for name in sorted(tensors):
            data = tensors[name][2]
            if offsets[name] > pos:
                f.write(b"\0" * (offsets[name] - pos))
                pos = offsets[name]
            mv = memoryview(data).cast("B")
            f.write(mv)
            pos += len(mv)


class _Cur:
    def __init__(self, f, size):
        self.f, self.size = f, size

    def read(self, n):
        b = self.f.read(n)
        if len(b) != n:
            raise CheckpointError("unexpected end of GGUF header")
        return b

    def u32(self):
        return struct.unpack("<I", self.read(4))[0]

    def u64(self):
        return struct.unpack("<Q", self.read(8))[0]

    def string(self):
        n = self.u64()
        if n > 1 << 20:
            raise CheckpointError("GGUF string exceeds limit")
        return self.read(n).decode("utf-8")

    def value(self, t):
        if t in _GGUF_SCALAR:
            fmt = _GGUF_SCALAR[t]
            return struct.unpack(fmt, self.read(struct.calcsize(fmt)))[0]
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.u32(), self.u64()
            return [self.value(et) for _ in range(n)]
        raise CheckpointError(f"unknown GGUF metadata value type {t}")


@dataclass
class RawEntry:
    key: str
    shape: tuple
    type_name: str      # "gguf.q4_0", "plain.f32", "u32", ...
    offset: int         # absolute in file
    nbytes: int
    source_file_index: int = 0


@dataclass
class RawIndex:
    format_id: str
    files: list
    metadata: dict
    entries: dict = field(default_factory=dict)


def index_gguf(path: str) -> RawIndex:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        cur = _Cur(f, size)
        if cur.read(4) != b"GGUF":
            raise CheckpointError("not a GGUF file")
        version = cur.u32()
        if version not in (2, 3):
            raise CheckpointError(f"unsupported GGUF version {version} (supported: 2, 3)")
        n_tensors, n_kv = cur.u64(), cur.u64()
        if n_tensors > 1 << 20 or n_kv > 1 << 20:
            raise CheckpointError("GGUF counts exceed limits")
        meta = {}
        for _ in range(n_kv):
            k = cur.string()
            meta[k] = cur.value(cur.u32())
        alignment = int(meta.get("general.alignment", 32))
        dirs = []
        for _ in range(n_tensors):
            name = cur.string()
            nd = cur.u32()
            if nd > 8:
                raise CheckpointError(f"GGUF tensor rank {nd} exceeds limit")
            shape = tuple(reversed([cur.u64() for _ in range(nd)]))
            code = cur.u32()
            if code not in GGML_TYPES and code not in GGML_SCHEMA_ONLY:
                raise CheckpointError(f"unknown GGUF tensor type code {code} for {name}")
            dirs.append((name, shape, code, cur.u64()))
        data_offset = (f.tell() + alignment - 1) // alignment * alignment
    idx = RawIndex("gguf", [path], meta)
    for name, shape, code, rel in dirs:
        nbytes = nbytes_for_shape(code, shape)
        absolute = data_offset + rel
        if absolute + nbytes > size:
            raise CheckpointError(f"tensor data extends past end of file: {name}")
        tname = (GGML_TYPES.get(code) or GGML_SCHEMA_ONLY[code])[0]
        idx.entries[name] = RawEntry(name, shape, tname, absolute, nbytes)
    return idx


# --------------------------------------------------------------------- SafeTensors

def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> (dtype string e.g. "BF16", shape, bytes-like)."""
    header = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    pos = 0
    order = sorted(tensors)
    for name in order:
        dt, shape, data = tensors[name]
        n = len(memoryview(data).cast("B"))
        header[name] = {"dtype": dt, "shape": [int(s) for s in shape], "data_offsets": [pos, pos + n]}
        pos += n
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((-len(hb)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for name in order:
            f.write(memoryview(tensors[name][2]).cast("B"))


def index_safetensors(path: str) -> RawIndex:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen > 100 << 20 or 8 + hlen > size:
            raise CheckpointError("SafeTensors header length out of range")
        header = json.loads(f.read(hlen))
    base = 8 + hlen
    meta = header.pop("__metadata__", {}) or {}
    idx = RawIndex("safetensors", [path], dict(meta))
    for name, e in header.items():
        if e["dtype"] not in ST_DTYPES:
            raise CheckpointError(f"unsupported SafeTensors dtype {e['dtype']} for {name}")
        tname, esz = ST_DTYPES[e["dtype"]]
        b, en = e["data_offsets"]
        numel = 1
        for d in e["shape"]:
            numel *= d
        if en - b != numel * esz or base + en > size:
            raise CheckpointError(f"SafeTensors byte range mismatch for {name}")
        idx.entries[name] = RawEntry(name, tuple(e["shape"]), tname, base + b, en - b)
    return idx


# ------------------------------------------------------------- logical parameters

@dataclass
class Component:
    name: str            # "data" | "packed" | "scales" | "biases"
    checkpoint_key: str
    type_name: str
    shape: tuple
    source_file_index: int
    offset: int
    length: int


@dataclass
class Parameter:
    canonical: str       # GGUF-style canonical name, e.g. blk.0.attn_q.weight
    encoding: str        # "gguf.q4_0", "mlx.affine.u4", "plain.bf16", ...
    shape: tuple         # logical [N, K] (or [H])
    components: list
    group: int = 0       # MLX group size


@dataclass
class Catalog:
    files: list
    config: dict         # normalised model metadata
    parameters: dict     # canonical -> Parameter


_HF_LAYER = {
    "input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
    "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
    "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm",
    "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
    "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down",
}


def hf_to_canonical(name: str):
    """HF tensor name (without trailing .weight/.scales/.biases) -> GGUF canonical stem."""
    if name == "model.embed_tokens":
        return "token_embd"
    if name == "model.norm":
        return "output_norm"
    if name == "lm_head":
        return "output"
    if name.startswith("model.layers."):
        rest = name[len("model.layers."):]
        n, _, sub = rest.partition(".")
        if sub in _HF_LAYER and n.isdigit():
            return f"blk.{n}.{_HF_LAYER[sub]}"
    return None


def _config_from_gguf(meta: dict, entries: dict) -> dict:
    arch = meta.get("general.architecture")
    if not isinstance(arch, str):
        raise CheckpointError("GGUF metadata lacks general.architecture")

    def g(suffix, default=None):
        return meta.get(f"{arch}.{suffix}", default)

    hidden = int(g("embedding_length"))
    heads = int(g("attention.head_count"))
    head_dim = g("attention.key_length") or g("rope.dimension_count") or hidden // heads
    emb = entries.get("token_embd.weight")
    vocab = g("vocab_size") or (emb.shape[0] if emb else None)
    return {
        "model_type": arch, "layers": int(g("block_count")), "hidden": hidden,
        "intermediate": int(g("feed_forward_length")), "heads": heads,
        "kv_heads": int(g("attention.head_count_kv", heads)), "head_dim": int(head_dim),
        "vocab": int(vocab), "eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)),
        "theta": float(g("rope.freq_base", 10000.0)),
        "context_length": int(g("context_length", 0) or 0),
        "qk_norm": "blk.0.attn_q_norm.weight" in entries,
        "rope": bool(meta.get("dyninfer.rope", 1)),
        "tied": "output.weight" not in entries,
    }


def catalog_from_gguf(path: str) -> Catalog:
    idx = index_gguf(path)
    cfg = _config_from_gguf(idx.metadata, idx.entries)
    params = {}
    for name, e in idx.entries.items():
        params[name] = Parameter(name, e.type_name, e.shape,
                                 [Component("data", name, e.type_name, e.shape, 0, e.offset, e.nbytes)])
    return Catalog(idx.files, cfg, params)


def catalog_from_mlx(path: str) -> Catalog:
    """`path` is a model directory holding model.safetensors + config.json, or the file itself."""
    if os.path.isdir(path):
        st, cj = os.path.join(path, "model.safetensors"), os.path.join(path, "config.json")
    else:
        st, cj = path, os.path.join(os.path.dirname(path), "config.json")
    idx = index_safetensors(st)
    with open(cj) as f:
        hf = json.load(f)
    # quantization{,_config}.{bits,group_size}: crates/dyninfer-checkpoint-safetensors/src/config_json.rs:129-140
    q = hf.get("quantization") or hf.get("quantization_config") or {}
    bits, group = int(q.get("bits", 0)), int(q.get("group_size", 0))
    heads = int(hf["num_attention_heads"])
    cfg = {
        "model_type": hf.get("model_type", "qwen3"), "layers": int(hf["num_hidden_layers"]),
        "hidden": int(hf["hidden_size"]), "intermediate": int(hf["intermediate_size"]),
        "heads": heads, "kv_heads": int(hf.get("num_key_value_heads", heads)),
        "head_dim": int(hf.get("head_dim", hf["hidden_size"] // heads)),
        "vocab": int(hf["vocab_size"]), "eps": float(hf.get("rms_norm_eps", 1e-6)),
        "theta": float(hf.get("rope_theta", 10000.0)),
        "context_length": int(hf.get("max_position_embeddings", 0)),
        "rope": True,
    }
    params = {}
    stems = {}
    for name in idx.entries:
        stem, _, suffix = name.rpartition(".")
        stems.setdefault(stem, {})[suffix] = idx.entries[name]
    for stem, parts in stems.items():
        canon = hf_to_canonical(stem)
        if canon is None:
            continue
        canon += ".weight"
        w = parts.get("weight")
        if w is None:
            continue
        if "scales" in parts and "biases" in parts:
            if bits != 4:
                raise CheckpointError(f"MLX affine bits={bits} has no kernel (only 4)")
            if w.type_name != "u32":
                raise CheckpointError(f"MLX packed tensor {stem}.weight must be U32")
            n, kw = w.shape
            k = kw * 8
            s, b = parts["scales"], parts["biases"]
            if s.shape != (n, k // group) or b.shape != s.shape or s.type_name != b.type_name:
                raise CheckpointError(f"MLX scales/biases shape mismatch for {stem}")
            comps = [
                Component("packed", w.key, "u32", w.shape, 0, w.offset, w.nbytes),
                Component("scales", s.key, s.type_name, s.shape, 0, s.offset, s.nbytes),
                Component("biases", b.key, b.type_name, b.shape, 0, b.offset, b.nbytes),
            ]
            params[canon] = Parameter(canon, "mlx.affine.u4", (n, k), comps, group)
        else:
            params[canon] = Parameter(canon, w.type_name, w.shape,
                                      [Component("data", w.key, w.type_name, w.shape, 0, w.offset, w.nbytes)])
    cfg["qk_norm"] = "blk.0.attn_q_norm.weight" in params
    cfg["tied"] = "output.weight" not in params
    return Catalog(idx.files, cfg, params)


def open_catalog(path: str) -> Catalog:
    if os.path.isdir(path) or path.endswith(".safetensors"):
        return catalog_from_mlx(path)
    return catalog_from_gguf(path)


# ---------------------------------------------------------------- provider plan

@dataclass
class ProviderParam:
    external_key: str
    source_file_index: int
    offset: int
    length: int


@dataclass
class ProviderPlan:
    kind: str
    scope: str
    file_paths: list
    parameters: list


def build_runtime_provider_plan(cat: Catalog) -> ProviderPlan:
    """One `(key, file, offset, length)` per component, sorted by key; refuses empty or
    out-of-file ranges and duplicate keys like the reference's plan builder."""
    if not cat.files:
        raise CheckpointError("checkpoint has no source files")
    sizes = [os.path.getsize(p) for p in cat.files]
    out, seen = [], set()
    for p in cat.parameters.values():
        for c in p.components:
            key = f"{PARAMETER_SCOPE}::{p.canonical}::{c.name}"
            if c.source_file_index >= len(sizes):
                raise CheckpointError(f"component source_file_index is out of range: {key}")
            end = c.offset + c.length
            if c.length == 0 or end > sizes[c.source_file_index]:
                raise CheckpointError(f"component byte range [{c.offset}, {end}) exceeds source size: {key}")
            if key in seen:
                raise CheckpointError(f"duplicate stable external parameter key: {key}")
            seen.add(key)
            out.append(ProviderParam(key, c.source_file_index, c.offset, c.length))
    out.sort(key=lambda d: d.external_key)
    return ProviderPlan("direct-file-ranges-v1", PARAMETER_SCOPE, list(cat.files), out)


def model_descriptor(cat: Catalog, **overrides) -> dict:
    """The JSON document handed to the session constructor: model geometry plus, per
    parameter, the encoding, logical shape and component element types. It carries
    what the reference bakes into its compiled module (shapes and selected
    lowerings); weights themselves travel only as byte ranges."""
    desc = dict(cat.config)
    desc.update(overrides)
    desc["params"] = {
        p.canonical: {
            "encoding": p.encoding, "shape": list(p.shape), "group": p.group,
            "aux": (p.components[1].type_name if len(p.components) > 1 else ""),
        }
        for p in cat.parameters.values()
    }
    return desc
