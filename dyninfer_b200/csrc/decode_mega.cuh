// Arguments of the persistent single-token decode kernel (decode_mega.cu).
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

// One ring-slot's worth of work, precomputed on the host: rows [0, n) of a 16-row tile of one
// tensor, `nu` units of K starting at 32-block kb0. 64 bytes.
struct MegaChunk {
  const uint8_t* src;  // first byte of (tile row 0, K-slice)
  const uint8_t* sc;   // MLX: scales / biases of (tile row 0, slice's first group)
  const uint8_t* bi;
  float* out;          // output vector the finished rows go to
  uint32_t rb, arb;    // bytes between consecutive rows: data, MLX aux
  uint16_t seg, aseg;  // bytes per row in this chunk: data, MLX aux
  uint16_t pitch, apitch;  // shared-memory bytes per tile row
  uint16_t kb0;        // first 32-block of the slice
  uint8_t n, nu;       // valid rows, units
  uint8_t enc, flags;  // encoding; bit0 closes the tile, bit1 second accumulator, bits 2..3 epilogue
  uint8_t aux, group_shift;  // MLX: aux element type, log2(group / 32)
  int32_t out_row;     // index of tile row 0 in `out`
  uint32_t pad_;
};
static_assert(sizeof(MegaChunk) == 64, "MegaChunk must stay 64 bytes");
enum { MEGA_EP_STORE = 0, MEGA_EP_RESIDUAL = 1, MEGA_EP_SWIGLU = 2, MEGA_EP_LOGITS = 3 };

struct MegaArgs {
  int layers, H, I, V, nh, nkv, d;
  float eps;
  int has_norm, has_rope;
  const MegaLayer* L;  // device array [layers]
  WRef embed, lm_head;
  const void* out_norm;
  int out_norm_type;
  // activations, f32, global
  float *hidden, *q, *k, *v, *ctx, *act, *logits;
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
  // cross-CTA synchronisation and scratch
  unsigned long long* bar;  // [0] arrivals (monotonic), [1] published generation
  int* error;               // set non-zero when a bounded wait gave up
  float* attn_part;         // [nh][max_split][d + 2]
  int max_split;
  float* argmax_val;        // [grid]
  long long* argmax_idx;    // [grid]
  unsigned long long* prof; // nullable: [9] nanoseconds per phase kind seen by CTA 0 (last launch)
  const MegaChunk* prog;     // [grid][max_chunks]
  const uint16_t* counts;    // [grid][4 * layers + 1] chunks per phase
  int max_chunks;
  int prog_in_smem;          // the CTA copies its program into shared memory at start
  int nslot;                // ring slots in shared memory
  int xs_floats;            // activation vector capacity in shared memory
  FreqTable ft;
};

size_t mega_smem_bytes(int nslot, int xs_floats, size_t prog_bytes);
// Chooses ring depth for the model; returns 0 when the model cannot use this kernel.
int mega_plan(int H, int I, int qd, int d, size_t prog_bytes, int* nslot, int* xs_floats, size_t* smem,
              int* prog_in_smem);
bool mega_supports_weight(const WRef& w);
// Builds every CTA's chunk program (host). counts: [grid][4*layers+1]; chunks: [grid][*max_chunks].
struct MegaBuildLayer {
  WRef q, k, v, o, gate, up, down;
};
int mega_build_program(const MegaBuildLayer* layers, int nlayers, const WRef& lm_head, int nh, int nkv,
                       int d, int H, int I, int V, float* q, float* k, float* v, float* hidden,
                       float* act, float* logits, int grid, std::vector<MegaChunk>* chunks,
                       std::vector<uint16_t>* counts, int* max_chunks);
int launch_decode_mega(const MegaArgs& a, int grid, size_t smem, cudaStream_t s);
int mega_grid_size(int device, size_t smem, int* grid);

}  // namespace dyn
