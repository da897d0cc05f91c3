"""Tensor-parallel shard plan for the large configuration (one process per GPU, TP degree 2/4/8).

Host-side planning only: which verbatim byte ranges of the checkpoint every rank uploads, and the
per-rank logical shapes. Nothing is re-encoded.

* column-parallel (split the output rows N): attn_q, attn_k, attn_v, ffn_gate, ffn_up and the
  lm_head (`output.weight`, or the tied `token_embd.weight` when used as lm_head). A rank's rows are
  one contiguous byte range of every component.
* row-parallel (split the reduction dim K on quantisation-block boundaries): attn_output, ffn_down.
  A rank holds, for every row, one contiguous span of that row's blocks: a strided range
  (`rows` segments of `seg_bytes` every `row_stride` bytes) that a 2-D copy uploads unchanged.
  The partial products of the ranks are summed by an all-reduce after o_proj and after down_proj.
* everything else (norm vectors, the embedding table for lookups) is replicated.

Heads follow the shards: rank r owns q heads [r*nh/W, (r+1)*nh/W) and kv heads [r*nkv/W, ...), so
the KV cache and attention need no communication; W must divide the kv head count.
"""
from __future__ import annotations

from dataclasses import dataclass

from .checkpoint import Catalog, CheckpointError, Parameter

COLUMN = ("attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up")
ROW = ("attn_output", "ffn_down")

# (elements per block, bytes per block) of the row-major encodings
_BLOCK = {"gguf.q4_0": (32, 18), "gguf.q4_1": (32, 20), "gguf.q8_0": (32, 34), "gguf.q6_k": (256, 210), "gguf.q4_k": (256, 144), "gguf.q5_k": (256, 176), "gguf.iq4_xs": (256, 136),
          "plain.f32": (1, 4), "plain.f16": (1, 2), "plain.bf16": (1, 2)}


@dataclass(frozen=True)
class ShardRange:
    """`rows` segments of `seg_bytes`, the first at `offset`, `row_stride` bytes apart, of file
    `source_file_index`. A contiguous range has rows == 1."""
    canonical: str
    component: str
    source_file_index: int
    offset: int
    rows: int
    seg_bytes: int
    row_stride: int

    @property
    def nbytes(self) -> int:
        return self.rows * self.seg_bytes


@dataclass(frozen=True)
class ShardedParameter:
    canonical: str
    encoding: str
    kind: str            # "column" | "row" | "replicated"
    shape: tuple         # this rank's logical shape
    ranges: tuple        # ShardRange per component


def _role(canonical: str) -> str:
    stem = canonical.rsplit(".", 1)[0].split(".")[-1]      # blk.3.attn_q.weight -> attn_q
    if stem in COLUMN:
        return "column"
    if stem in ROW:
        return "row"
    if canonical == "output.weight":
        return "column"
    return "replicated"


def _component_row_bytes(p: Parameter, comp) -> int:
    n = p.shape[0]
    if comp.length % n:
        raise CheckpointError(f"{p.canonical}/{comp.name}: {comp.length} bytes do not divide into {n} rows")
    return comp.length // n


def shard_parameter(p: Parameter, rank: int, world: int, role: str | None = None) -> ShardedParameter:
    role = role or _role(p.canonical)
    if role == "replicated" or len(p.shape) != 2:
        rng = tuple(ShardRange(p.canonical, c.name, c.source_file_index, c.offset, 1, c.length, c.length)
                    for c in p.components)
        return ShardedParameter(p.canonical, p.encoding, "replicated", tuple(p.shape), rng)
    n, k = p.shape
    if role == "column":
        if n % world:
            raise CheckpointError(f"{p.canonical}: {n} rows do not split over {world} ranks")
        lo, cnt = rank * (n // world), n // world
        rng = []
        for c in p.components:
            rb = _component_row_bytes(p, c)
            rng.append(ShardRange(p.canonical, c.name, c.source_file_index, c.offset + lo * rb, 1, cnt * rb, cnt * rb))
        return ShardedParameter(p.canonical, p.encoding, "column", (cnt, k), tuple(rng))
    # row-parallel: split K on block (and MLX group) boundaries
    if k % world:
        raise CheckpointError(f"{p.canonical}: K = {k} does not split over {world} ranks")
    kr = k // world
    rng = []
    for c in p.components:
        rb = _component_row_bytes(p, c)
        if p.encoding == "mlx.affine.u4":
            unit = 8 if c.name == "packed" else p.group     # elements covered by one stored item
        else:
            unit = _BLOCK[p.encoding][0]
        if kr % unit:
            raise CheckpointError(f"{p.canonical}/{c.name}: K/{world} = {kr} is not a multiple of {unit}")
        seg = rb // world
        if seg * world != rb:
            raise CheckpointError(f"{p.canonical}/{c.name}: row bytes {rb} do not split over {world} ranks")
        rng.append(ShardRange(p.canonical, c.name, c.source_file_index, c.offset + rank * seg, n, seg, rb))
    return ShardedParameter(p.canonical, p.encoding, "row", (n, kr), tuple(rng))


def plan(cat: Catalog, rank: int, world: int, shard_lm_head: bool = True) -> dict:
    """canonical -> ShardedParameter for `rank` of `world`. With tied embeddings the table is
    replicated for lookups and, when `shard_lm_head`, additionally row-sliced under the name
    `output.weight` (an alias of the same bytes, `naming.rs:70-96`)."""
    cfg = cat.config
    nkv = int(cfg.get("kv_heads", cfg.get("heads", 1)))
    if world < 1 or nkv % world or int(cfg["heads"]) % world:
        raise CheckpointError(f"tensor-parallel degree {world} must divide the head counts ({cfg['heads']}, {nkv})")
    if not 0 <= rank < world:
        raise CheckpointError(f"rank {rank} outside 0..{world - 1}")
    out = {}
    for name, p in cat.parameters.items():
        role = _role(name)
        if name == "output.weight" and not shard_lm_head:
            role = "replicated"
        out[name] = shard_parameter(p, rank, world, role)
    if shard_lm_head and "output.weight" not in cat.parameters and "token_embd.weight" in cat.parameters:
        tied = cat.parameters["token_embd.weight"]
        sp = shard_parameter(tied, rank, world, "column")
        out["output.weight"] = ShardedParameter("output.weight", sp.encoding, "column", sp.shape, sp.ranges)
    return out


def read_shard(files: list, sp: ShardedParameter) -> dict:
    """component name -> bytes of this rank's shard, gathered exactly as a 2-D copy would."""
    out = {}
    for r in sp.ranges:
        with open(files[r.source_file_index], "rb") as f:
            buf = bytearray()
            for i in range(r.rows):
                f.seek(r.offset + i * r.row_stride)
                buf += f.read(r.seg_bytes)
        out[r.component] = bytes(buf)
    return out


def session_inputs(cat: Catalog, rank: int, world: int, **overrides):
    """What rank `rank` hands to the session constructor: the model descriptor with this rank's
    share of the geometry (heads, kv_heads and intermediate divided by `world`, `lm_head_rows`
    = vocab / world, per-parameter local shapes, strided spans for the row-parallel products) and
    the byte ranges as `(key, source_file_index, offset, byte_count)`, sorted by key."""
    from .checkpoint import PARAMETER_SCOPE, model_descriptor
    shards = plan(cat, rank, world)
    cfg = cat.config
    if int(cfg["intermediate"]) % world or int(cfg["vocab"]) % world:
        raise CheckpointError(f"tensor-parallel degree {world} must divide intermediate and vocab")
    desc = model_descriptor(cat, **overrides)
    desc.update(tp_rank=rank, tp_world=world, heads=int(cfg["heads"]) // world,
                kv_heads=int(cfg.get("kv_heads", cfg["heads"])) // world,
                head_dim=int(cfg.get("head_dim", int(cfg["hidden"]) // int(cfg["heads"]))),
                intermediate=int(cfg["intermediate"]) // world, lm_head_rows=int(cfg["vocab"]) // world,
                decode_kernel="graph")
    params, ranges = {}, []
    for name, sp in shards.items():
        src = cat.parameters.get(name) or cat.parameters["token_embd.weight"]    # tied lm_head alias
        entry = {"encoding": sp.encoding, "shape": list(sp.shape), "group": src.group,
                 "aux": (src.components[1].type_name if len(src.components) > 1 else "")}
        strided = {r.component: [r.rows, r.seg_bytes, r.row_stride] for r in sp.ranges if r.rows > 1}
        if strided:
            entry["strided"] = strided
        params[name] = entry
        for r in sp.ranges:
            ranges.append((f"{PARAMETER_SCOPE}::{name}::{r.component}", r.source_file_index, r.offset, r.nbytes))
    desc["params"] = params
    ranges.sort(key=lambda t: t[0])
    return desc, ranges


def exchange_unique_id(make_id):
    """Rank 0 calls `make_id()` (bytes); every rank of the default torch.distributed group returns
    the same bytes. The host-side hand-off the native communicator needs before its first step."""
    import torch.distributed as dist
    box = [make_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]
