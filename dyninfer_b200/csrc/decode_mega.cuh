// Arguments of the persistent single-token decode kernel (decode_mega.cu).
#pragma once

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
  int nslot;                // ring slots in shared memory
  int xs_floats;            // activation vector capacity in shared memory
  FreqTable ft;
};

size_t mega_smem_bytes(int nslot, int xs_floats);
// Chooses ring depth for the model; returns 0 when the model cannot use this kernel.
int mega_plan(int H, int I, int qd, int d, int* nslot, int* xs_floats, size_t* smem);
int launch_decode_mega(const MegaArgs& a, int grid, size_t smem, cudaStream_t s);
int mega_grid_size(int device, size_t smem, int* grid);

}  // namespace dyn
