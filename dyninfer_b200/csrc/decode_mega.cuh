// Arguments and host-side program of the persistent single-token decode kernel (decode_mega.cu).
#pragma once

#include <vector>

#include "common.cuh"

namespace dyn {

struct MegaLayer {
  WRef q, k, v, o, gate, up, down;
  const void* attn_norm;
  const void* ffn_norm;
  const void* q_norm;
  const void* k_norm;
  int norm_type;     // element type of attn_norm / ffn_norm
  int qk_norm_type;  // element type of q_norm / k_norm
};

// One ring-slot's worth of weights, precomputed on the host: rows [0, n) of a 16-row tile of one
// tensor, `nu` units of K starting at 32-block kb0; its sums go to accumulator `acc` of the round.
// The first 16 bytes are all a consumer warp reads (one vector load).
struct MegaChunk {
  uint16_t pitch, kb0;       // shared-memory bytes per tile row; first 32-block of the slice
  uint8_t n, nu;             // valid rows, units
  uint8_t acc, enc;          // accumulator index within the round; encoding
  uint8_t al, al_step;       // row i starts (al + i * al_step) & 15 bytes into its 16-byte aligned copy
  uint8_t aux, group_shift;  // MLX: aux element type, log2(group / 32)
  uint16_t apitch;           // MLX: shared-memory bytes per aux row
  uint8_t aal, aal_step;     // MLX: the same alignment rule for the scale / bias rows
  // producer side
  const uint8_t* src;  // first byte of (tile row 0, K-slice)
  const uint8_t* sc;   // MLX: scales / biases of (tile row 0, slice's first group)
  const uint8_t* bi;
  uint32_t rb, arb;    // bytes between consecutive rows: data, MLX aux
  uint16_t seg, aseg;  // bytes per row in this chunk: data, MLX aux
  uint32_t contig;     // != 0: the rows are one run in memory, copied by a single bulk copy of this many bytes
  uint32_t tx;         // bytes all per-row copies of the chunk bring (the slot barrier's transaction count)
  int32_t jump16;      // rows 8..15 come from a second matrix: their source is 16 * jump16 bytes further on
};
static_assert(sizeof(MegaChunk) == 64, "MegaChunk must stay 64 bytes");

// What happens to a finished tile of output rows.
// SWIGLU_IL: tile rows 0..7 are gate rows, rows 8..15 the same rows of up (one accumulator).
enum {
  MEGA_EP_QKV = 0,
  MEGA_EP_RESID_O = 1,
  MEGA_EP_SWIGLU = 2,
  MEGA_EP_RESID_DOWN = 3,
  MEGA_EP_LOGITS = 4,
  MEGA_EP_SWIGLU_IL = 5
};
struct MegaTile {
  int32_t out_row;  // index of tile row 0 in the phase's output vector
  uint8_t n;        // valid rows
  uint8_t ep;       // MEGA_EP_*
  uint8_t acc;      // accumulator of the tile's sums
  uint8_t acc2;     // SWIGLU: accumulator of the `up` sums
};
static_assert(sizeof(MegaTile) == 8, "MegaTile must stay 8 bytes");
// A round: chunks whose sums are held in registers (at most MEGA_TA accumulators), then ONE
// cross-warp reduction and the epilogues of its tiles.
constexpr int MEGA_TA = 8;
struct MegaRound {
  uint16_t nchunks;
  uint8_t ntiles;
  uint8_t naccs;  // accumulators in use
};
// Per-CTA program blob in global memory (copied to shared memory by one bulk copy):
//   MegaProgHeader | chunks[max_chunks] | tiles[max_tiles] | rounds[max_rounds] | phase_rounds[nph] |
//   MegaLayerHot[layers]
struct MegaProgHeader {
  uint32_t nchunks, hid_hi, nrounds, hid_lo;  // [hid_lo, hid_hi): the hidden rows this CTA owns
};
// What the kernel needs of a layer besides its weights, kept in shared memory (part of the blob)
// so that no layer begins with a fetch of its descriptor.
struct MegaLayerHot {
  const void* attn_norm;
  const void* ffn_norm;
  const void* q_norm;
  const void* k_norm;
  uint8_t norm_type, qk_norm_type;
  uint8_t enc_q, enc_o, enc_gate, enc_down;  // activation layout of a phase whose tensors differ
  uint8_t pad_[2];
};
static_assert(sizeof(MegaLayerHot) == 40, "MegaLayerHot layout");
struct MegaProgLayout {
  int max_chunks = 0, max_tiles = 0, max_rounds = 0, nph = 0;
  size_t off_tiles = 0, off_rounds = 0, off_phase = 0, off_layers = 0, bytes = 0;  // offsets inside one CTA's blob
};
// phase_rounds[ph]: low byte = rounds of the phase, high byte = the encoding all its chunks share
// (0xff: mixed, the tile steps then select per chunk).

struct MegaArgs {
  int layers, H, I, V, nh, nkv, d;
  float eps;
  int has_norm, has_rope;
  const MegaLayer* L;  // device array [layers]
  WRef embed, lm_head;
  const void* out_norm;
  int out_norm_type;
  float* logits;  // f32 [V], plain
  // Hand-off vectors between the CTAs: arrays of (value, epoch) pairs, 8 bytes each; a reader
  // polls the pairs themselves until they carry the epoch it expects.
  float* ll_hidden[2];  // [H]: after o_proj + residual / after down + residual
  float* ll_qkv;        // [nh*d + 2*nkv*d]
  float* ll_ctx;        // [nh*d]: attention output when one CTA holds all keys of a head
  float* ll_part;       // [nh][max_split][d + 4]: split-KV partial outputs, then (max, sum), two unused
  float* ll_act;        // [I]
  float* ll_amax;       // [grid][4]: (value, row) of each CTA's best logit, two unused (one sector per CTA)
  unsigned epoch_base;  // epochs of the launch's token t are epoch_base + t * (layers + 2) + 1 + layer
  // KV pool
  uint8_t* kcache;
  uint8_t* vcache;
  int64_t cap;
  uint64_t layer_stride;  // bytes between layers in each pool
  int kv_type;
  // step state: io[0] token, io[1] position, io[2] cache slot, io[3] produced token
  int64_t* io;
  int64_t* hist;
  int64_t* hist_count;
  int64_t hist_cap;
  // One-token calls pass the token, position and sequence as launch parameters and get the result
  // written straight into pinned host memory (no copy before or after the launch): inline_io = 1,
  // out_host = device address of two host words (produced token, error code of an expired wait).
  int inline_io;
  int64_t in_token, in_pos, in_seq;
  int64_t* out_host;
  int advance;  // 1: feed the produced token back and advance the position on the device
  int opts;     // bit 1: no L2 prefetch of the next layer's norm vectors (measurement switch)
  int steps;    // tokens decoded by this launch (> 1 needs advance); epochs: steps * (layers + 2)
  int* error;   // set non-zero when a bounded wait gave up
  int max_split;
  unsigned long long* prof;  // nullable: nanoseconds per kind seen by CTA 0 (last launch)
  // nullable: [grid][layers + 1][16] global-timer stamps of thread 0 of every CTA. Per layer: 0 QKV
  // input staged, 1 its tile steps done, 2 its outputs stored; 3 attention has q/k/v, 4 attention
  // stored; 5-7 o_proj, 8-10 gate/up, 11-13 down likewise; row `layers`: 0-2 = lm_head.
  unsigned long long* trace;
  const uint8_t* prog;       // [grid] blobs of lay.bytes
  MegaProgLayout lay;
  int nslot;      // ring slots in shared memory
  int xs_floats;  // activation vector capacity in shared memory
  FreqTable ft;
};

size_t mega_smem_bytes(int nslot, int xs_floats, size_t prog_bytes);
// Chooses the ring depth for the model; returns 0 when the model cannot use this kernel.
int mega_plan(int H, int I, int qd, int d, size_t prog_bytes, int* nslot, int* xs_floats, size_t* smem);
bool mega_supports_weight(const WRef& w);
struct MegaBuildLayer {
  WRef q, k, v, o, gate, up, down;
};
// Builds every CTA's program (host): `blob` receives grid * lay->bytes bytes.
int mega_build_program(const MegaBuildLayer* layers, const MegaLayer* full, int nlayers, const WRef& lm_head, int nh,
                       int nkv, int d, int H, int I, int V, int grid, std::vector<uint8_t>* blob, MegaProgLayout* lay);
int launch_decode_mega(const MegaArgs& a, int grid, size_t smem, cudaStream_t s);
int mega_grid_size(int device, size_t smem, int* grid);

}  // namespace dyn
