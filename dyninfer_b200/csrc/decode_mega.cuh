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
struct MegaChunk {
  const uint8_t* src;  // first byte of (tile row 0, K-slice)
  const uint8_t* sc;   // MLX: scales / biases of (tile row 0, slice's first group)
  const uint8_t* bi;
  uint32_t rb, arb;    // bytes between consecutive rows: data, MLX aux
  uint16_t seg, aseg;  // bytes per row in this chunk: data, MLX aux
  uint16_t pitch, apitch;  // shared-memory bytes per tile row
  uint16_t kb0;        // first 32-block of the slice
  uint8_t n, nu;       // valid rows, units
  uint8_t enc, acc;    // encoding; accumulator index within the round
  uint8_t aux, group_shift;  // MLX: aux element type, log2(group / 32)
  uint32_t pad_[4];
};
static_assert(sizeof(MegaChunk) == 64, "MegaChunk must stay 64 bytes");

// What happens to a finished tile of output rows.
enum { MEGA_EP_QKV = 0, MEGA_EP_RESID_O = 1, MEGA_EP_SWIGLU = 2, MEGA_EP_RESID_DOWN = 3, MEGA_EP_LOGITS = 4 };
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
//   MegaProgHeader | chunks[max_chunks] | tiles[max_tiles] | rounds[max_rounds] | phase_rounds[nph]
struct MegaProgHeader {
  uint32_t nchunks, ntiles, nrounds, hid_lo;  // hid_lo: first hidden row this CTA owns
};
struct MegaProgLayout {
  int max_chunks = 0, max_tiles = 0, max_rounds = 0, nph = 0;
  size_t off_tiles = 0, off_rounds = 0, off_phase = 0, bytes = 0;  // offsets inside one CTA's blob
};

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
  float* ll_part;       // [nh][max_split][d + 2]: split-KV partial outputs, then (max, sum)
  float* ll_act;        // [I]
  float* ll_amax;       // [grid][2]: (value, row) of each CTA's best logit
  unsigned epoch_base;  // epochs of this launch are epoch_base + 1 + layer
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
  int advance;  // 1: feed the produced token back and advance the position on the device
  int* error;   // set non-zero when a bounded wait gave up
  int max_split;
  unsigned long long* prof;  // nullable: nanoseconds per kind seen by CTA 0 (last launch)
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
int mega_build_program(const MegaBuildLayer* layers, int nlayers, const WRef& lm_head, int nh, int nkv,
                       int d, int H, int I, int V, int grid, std::vector<uint8_t>* blob, MegaProgLayout* lay);
int launch_decode_mega(const MegaArgs& a, int grid, size_t smem, cudaStream_t s);
int mega_grid_size(int device, size_t smem, int* grid);

}  // namespace dyn
