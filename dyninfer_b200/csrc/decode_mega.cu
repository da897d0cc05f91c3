// Persistent single-token decode kernel: one launch per generated token.
//
// One CTA per SM, launched cooperatively so that all CTAs are co-resident. Each CTA owns a
// fixed, balanced slice of the rows of every weight matrix, cut into tiles of 16 rows (x
// K-slices). A producer warp streams the tiles — the verbatim checkpoint bytes, one 1-D bulk
// async copy per row segment (cp.async.bulk + mbarrier transaction counts) — from HBM into a
// shared-memory ring, running as far ahead of the math as the ring allows: weight traffic never
// waits for the activation dependency chain. Rows land PITCH bytes apart with PITCH/4 = 4
// (mod 8), so the tensor-core fragment loads are bank-conflict free. Sixteen consumer warps
// split each tile's K range, run the tile steps of gemv_core.cuh against the activation vector
// staged in shared memory in fragment order, and reduce their partial sums in a fixed order.
// CTAs meet at a grid barrier between dependent phases:
//
//   embed | per layer: norm+QKV | qk-norm+RoPE+KV-write+attention | o_proj+res |
//   norm+gate/up+SwiGLU | down+res | final: norm+lm_head+argmax partials | argmax
//
// Every wait (mbarrier, grid barrier) is bounded: when it gives up it raises the error word,
// the remaining phases are skipped in lockstep and the kernel ends.
#include <algorithm>

#include "codec.cuh"
#include "decode_mega.cuh"
#include "gemv_core.cuh"
#include "ring.cuh"

namespace dyn {

namespace {

// Embedding row through the exact scalar decoders (one row per token: not performance relevant).
template <int ENC>
__device__ __forceinline__ void gather_row_t(const WRef& w, int64_t row, float* out, int tid, int nthreads) {
  using C = Codec<ENC>;
  const RowPtr rp = row_ptr(w, row);
  const int nparts = (int)(w.cols / C::BLOCK) * C::PARTS;
  for (int it = tid; it < nparts; it += nthreads) {
    const int blk = it / C::PARTS, part = it - blk * C::PARTS;
    float v[4 * C::G];
    C::decode(rp, blk, part, v);
#pragma unroll
    for (int g = 0; g < C::G; g++)
      *reinterpret_cast<float4*>(out + blk * C::BLOCK + C::xoff(part, g)) =
          make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
  }
}
__device__ __noinline__ void mega_gather_row(const WRef w, int64_t row, float* out, int tid, int nthreads) {
  switch (w.enc) {
    case E_Q4_0: gather_row_t<E_Q4_0>(w, row, out, tid, nthreads); break;
    case E_Q4_1: gather_row_t<E_Q4_1>(w, row, out, tid, nthreads); break;
    case E_Q8_0: gather_row_t<E_Q8_0>(w, row, out, tid, nthreads); break;
    case E_Q6_K: gather_row_t<E_Q6_K>(w, row, out, tid, nthreads); break;
    case E_MLX_U4: gather_row_t<E_MLX_U4>(w, row, out, tid, nthreads); break;
    case E_BF16: gather_row_t<E_BF16>(w, row, out, tid, nthreads); break;
    case E_F16: gather_row_t<E_F16>(w, row, out, tid, nthreads); break;
    default: gather_row_t<E_F32>(w, row, out, tid, nthreads); break;
  }
}

constexpr int MK_CW = 16;               // consumer warps
constexpr int MK_CT = MK_CW * 32;       // consumer threads
constexpr int MK_THREADS = MK_CT + 32;  // + one producer warp
constexpr int MK_SLOT = 18432;          // bytes per ring slot (one 16-row tile x K-slice)
constexpr int MK_MISC_FLOATS = 6400;    // per-CTA scratch (attention state, reductions, partials, RoPE table)
constexpr int MK_ROPE_OFF = 6144;       // misc floats [6144, 6400): cos[128], sin[128] of this token's position
constexpr int MK_PART_OFF = 5120;       // misc floats [5120, 6144): 2 x [16 warps][32] partial sums
constexpr long long MK_MBAR_SPINS = 1LL << 22;
constexpr long long MK_GRID_SPINS = 1LL << 22;


__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CT) : "memory"); }

struct Smem {
  float* xs;      // activation vector, f32
  __half* xf;     // same, hi/lo f16 fragments
  float* sx32;    // per-32 sums of the scaled activation
  float* sx16;    // per-16 sums
  float* misc;
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* part_full;   // [2] partial-sum buffers: 16 warps arrived
  uint64_t* part_empty;  // [2] finalising warp done reading
  uint64_t* prog_bar;    // program copy landed
  const MegaChunk* prog; // this CTA's chunk program (shared memory copy, or global)
  const uint16_t* counts;
  volatile int* abort;
  int nslot;
};

// ---- producer: one bulk copy per tile row (lanes 0..15), MLX aux rows by lanes 16..31 --------
__device__ __forceinline__ void produce_chunk(const MegaChunk* c, const Smem& sm, uint32_t pi, int lane) {
  const int slot = pi % sm.nslot;
  if (pi >= (uint32_t)sm.nslot) {
    int ok = 1;
    if (lane == 0) {
      ok = mbar_wait_bounded(sm.empty + slot, ((pi / sm.nslot) - 1u) & 1u, MK_MBAR_SPINS, sm.abort) ? 1 : 0;
      if (!ok && !*sm.abort) *sm.abort = 4;
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return;
  }
  uint8_t* base = sm.ring + (size_t)slot * MK_SLOT;
  const int i = lane & 15;
  const int n = c->n;
  const uint8_t* g0 = nullptr;
  const uint8_t* g1 = nullptr;
  uint8_t* d0 = nullptr;
  uint8_t* d1 = nullptr;
  uint32_t n0 = 0, n1 = 0;
  if (i < n) {
    if (lane < 16) {
      const uint8_t* s = c->src + (size_t)i * c->rb;
      const uint32_t off = (uint32_t)(reinterpret_cast<uintptr_t>(s) & 15);
      g0 = s - off;
      n0 = (off + c->seg + 15u) & ~15u;
      d0 = base + i * c->pitch;
    } else if (c->aseg) {
      const uint8_t* s = c->sc + (size_t)i * c->arb;
      uint32_t off = (uint32_t)(reinterpret_cast<uintptr_t>(s) & 15);
      g0 = s - off;
      n0 = (off + c->aseg + 15u) & ~15u;
      d0 = base + 16 * c->pitch + i * c->apitch;
      s = c->bi + (size_t)i * c->arb;
      off = (uint32_t)(reinterpret_cast<uintptr_t>(s) & 15);
      g1 = s - off;
      n1 = (off + c->aseg + 15u) & ~15u;
      d1 = base + 16 * c->pitch + (16 + i) * c->apitch;
    }
  }
  uint32_t total = n0 + n1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) mbar_expect_tx(sm.full + slot, total);
  __syncwarp();
  if (n0) bulk_g2s(d0, g0, n0, sm.full + slot);
  if (n1) bulk_g2s(d1, g1, n1, sm.full + slot);
}

// ---- consumer helpers ---------------------------------------------------------------------------
// Stage the activation vector of a phase in one pass. Thread i owns fragment item i = (block kb,
// lane quarter t) and loads exactly the 8 elements that item holds (the items partition the
// vector; n <= 8 * MK_CT), so the sum of squares and the scale come from one combined block
// reduction and the normalised values go straight from registers to hi/lo f16 fragments and
// 16-/32-run sums. Optional RMSNorm: v = (x*inv)*w, inv = 1/sqrt(mean(x^2)+eps).
// Returns 2^24 / scale. `src_smem`: the vector already sits in sm.xs; else it is read from L2.
__device__ __forceinline__ float stage_phase(const float* x, bool src_smem, const void* nw, int nw_type,
                                             int n, float eps, int layout, const Smem& sm, int tid,
                                             int lane, int warp) {
  float* red = sm.misc + MK_PART_OFF - 64;
  const int items = (n >> 5) * 4;
  const int kb = tid >> 2, t = tid & 3;
  const bool live = tid < items;
  // load order: A = 4 elements, B = 4 elements
  const int baseA = kb * 32 + (layout == XL_MLXW ? 8 * t : 4 * t);
  const int baseB = layout == XL_MLXW ? baseA + 4 : kb * 32 + 16 + 4 * t;
  float v[8], w[8];
  float ss = 0.f, mx = 0.f;
  if (live) {
    const float4 a4 = src_smem ? *reinterpret_cast<const float4*>(sm.xs + baseA)
                               : __ldcg(reinterpret_cast<const float4*>(x + baseA));
    const float4 b4 = src_smem ? *reinterpret_cast<const float4*>(sm.xs + baseB)
                               : __ldcg(reinterpret_cast<const float4*>(x + baseB));
    v[0] = a4.x, v[1] = a4.y, v[2] = a4.z, v[3] = a4.w;
    v[4] = b4.x, v[5] = b4.y, v[6] = b4.z, v[7] = b4.w;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      w[i] = nw ? aux_load(reinterpret_cast<const uint8_t*>(nw), nw_type, (i < 4 ? baseA : baseB - 4) + i) : 1.0f;
      ss = fmaf(v[i], v[i], ss);
      mx = fmaxf(mx, fabsf(v[i] * w[i]));
    }
  }
  ss = warp_sum(ss);
  mx = warp_max(mx);
  consumer_sync();
  if (lane == 0) {
    red[warp] = ss;
    red[32 + warp] = mx;
  }
  consumer_sync();
  float tss = 0.f, tmx = 0.f;
#pragma unroll
  for (int i = 0; i < MK_CW; i++) {
    tss += red[i];
    tmx = fmaxf(tmx, red[32 + i]);
  }
  const float inv = nw ? 1.0f / sqrtf(tss / (float)n + eps) : 1.0f;
  float s, is;
  scale_for(tmx * inv * 1.0001f, &s, &is);
  float run0 = 0.f, run1 = 0.f;  // this item's share of the block's two 16-element runs
  if (live) {
    float sv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) sv[i] = (nw ? __fmul_rn(__fmul_rn(v[i], inv), w[i]) : v[i]) * s;
    const float sa = (sv[0] + sv[1]) + (sv[2] + sv[3]), sb = (sv[4] + sv[5]) + (sv[6] + sv[7]);
    float f[8];  // fragment order
    if (layout == XL_NIBBLE) {
      f[0] = sv[0], f[1] = sv[2], f[2] = sv[4] * 0.0625f, f[3] = sv[6] * 0.0625f;
      f[4] = sv[1], f[5] = sv[3], f[6] = sv[5] * 0.0625f, f[7] = sv[7] * 0.0625f;
      run0 = sa, run1 = sb;
    } else if (layout == XL_MLXW) {
      f[0] = sv[0], f[1] = sv[4], f[2] = sv[1] * 0.0625f, f[3] = sv[5] * 0.0625f;
      f[4] = sv[2], f[5] = sv[6], f[6] = sv[3] * 0.0625f, f[7] = sv[7] * 0.0625f;
      if (t < 2) run0 = sa + sb; else run1 = sa + sb;
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] = sv[i];
      run0 = sa, run1 = sb;
    }
    __half hi[8], lo[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const __half h = __float2half_rn(f[i]);
      hi[i] = h;
      lo[i] = __float2half_rn(f[i] - __half2float(h));
    }
    uint4* dst = reinterpret_cast<uint4*>(sm.xf + ((size_t)(kb * 2) * 4 + t) * 8);
    dst[0] = *reinterpret_cast<uint4*>(hi);
    dst[4] = *reinterpret_cast<uint4*>(lo);
  }
  // the four quarters of a block are four consecutive lanes
  run0 += __shfl_xor_sync(0xffffffffu, run0, 1);
  run1 += __shfl_xor_sync(0xffffffffu, run1, 1);
  run0 += __shfl_xor_sync(0xffffffffu, run0, 2);
  run1 += __shfl_xor_sync(0xffffffffu, run1, 2);
  if (live && t == 0) {
    sm.sx16[2 * kb] = run0;
    sm.sx16[2 * kb + 1] = run1;
    sm.sx32[kb] = run0 + run1;
  }
  consumer_sync();
  return GV_2P24 * is;
}

// One unit of a chunk for this warp. p0 / p1: the chunk's bytes in rows g, g+8; a0 / a1: MLX
// scales of those rows (biases 16 * apitch further).
__device__ __forceinline__ void run_unit(int enc, int aux, int group_shift, const uint8_t* p0,
                                         const uint8_t* p1, const uint8_t* a0, const uint8_t* a1,
                                         int apitch16, int u, int kb0, const Smem& sm, int lane,
                                         TileAcc<true>& acc) {
  const int t = lane & 3;
  const int c = (lane >> 2) & 1;
  const __half* xf0 = sm.xf + (size_t)c * 32 + t * 8;  // block kb adds kb * 64 halfs
  if (enc == E_Q4_0) {
    const int kb = kb0 + 2 * u;
    blk_q4<E_Q4_0, 0, true>(p0 + u * 36, p1 + u * 36, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc);
    blk_q4<E_Q4_0, 2, true>(p0 + u * 36 + 18, p1 + u * 36 + 18, xf0 + (size_t)(kb + 1) * 64,
                            sm.sx32[kb + 1], 0.f, t, acc);
  } else if (enc == E_Q4_1) {
    const int kb = kb0 + u;
    blk_q4<E_Q4_1, 0, true>(p0 + u * 20, p1 + u * 20, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc);
  } else if (enc == E_Q8_0) {
    const int kb = kb0 + 2 * u;
    blk_q8_0<0, true>(p0 + u * 68, p1 + u * 68, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc);
    blk_q8_0<2, true>(p0 + u * 68 + 34, p1 + u * 68 + 34, xf0 + (size_t)(kb + 1) * 64, sm.sx32[kb + 1],
                      0.f, t, acc);
  } else if (enc == E_MLX_U4) {
    const int kb = kb0 + u;
    const int gi = u >> group_shift;
    blk_mlx<true>(p0 + u * 16, p1 + u * 16, aux_load(a0, aux, gi), aux_load(a1, aux, gi),
                  aux_load(a0 + apitch16, aux, gi), aux_load(a1 + apitch16, aux, gi),
                  xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc);
  } else {
    // Q6_K quarter: superblock u / 4 of the chunk, half n, sub-block s
    const int sb = u >> 2, n = (u >> 1) & 1, s = u & 1;
    const int kb = kb0 + sb * 8;
    const uint8_t* s0 = p0 + sb * 210;
    const uint8_t* s1 = p1 + sb * 210;
    if (sb & 1)
      q6k_quarter<2, true>(s0, s1, n, s, xf0 + (size_t)kb * 64, 64, sm.sx16 + 2 * kb, sm.sx16 + 2 * kb, t, acc);
    else
      q6k_quarter<0, true>(s0, s1, n, s, xf0 + (size_t)kb * 64, 64, sm.sx16 + 2 * kb, sm.sx16 + 2 * kb, t, acc);
  }
}

__device__ __forceinline__ float round_kv(float v, int kv_type) {
  if (kv_type == E_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (kv_type == E_F16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ void store_kv(uint8_t* base, int kv_type, int64_t idx, float v) {
  if (kv_type == E_F32)
    reinterpret_cast<float*>(base)[idx] = v;
  else if (kv_type == E_F16)
    reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else
    reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ bool arg_better(float v, long long i, float bv, long long bi) {
  return v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Phase timing seen by CTA 0 (optional): kind 0 embed, 1 qkv, 2 attention, 3 o_proj, 4 gate/up,
// 5 down, 6 lm_head, 7 argmax, 8 whole kernel; 9 staging, 10 waiting for weights, 11 tile math,
// 12 grid barrier; attention of CTA 0: 13 q/k/v load + norm + RoPE + first key fetch, 14 scores and
// softmax, 15 merge and write.
struct Prof {
  unsigned long long* out;
  unsigned long long last, start;
  bool on;
  __device__ void begin(unsigned long long* p, bool active) {
    out = p;
    on = active && p != nullptr;
    if (on) {
      for (int i = 0; i < 24; i++) out[i] = 0;
      last = start = gtime();
    }
  }
  __device__ void mark(int kind) {
    if (on) {
      const unsigned long long t = gtime();
      out[kind] += t - last;
      last = t;
    }
  }
  __device__ void end() {
    if (on) out[8] = gtime() - start;
  }
  __device__ unsigned long long tic() const { return on ? gtime() : 0ULL; }
  __device__ void toc(int kind, unsigned long long t0) {
    if (on) out[kind] += gtime() - t0;
  }
};

struct GridBar {
  unsigned long long gen;
};

// Arrival: release-add on a monotonic counter; waiting: acquire-poll the same counter.
__device__ __forceinline__ void grid_sync(const MegaArgs& a, GridBar& gb, int G, int tid,
                                          const Smem& sm) {
  consumer_sync();
  if (tid == 0) {
    gb.gen += 1;
    const unsigned long long target = gb.gen * (unsigned long long)G;
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(a.bar) : "memory");
    if (!*sm.abort) {
      unsigned long long seen = 0;
      long long it = 0;
      do {
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(a.bar) : "memory");
        if (seen >= target) break;
      } while (++it < MK_GRID_SPINS);
      if (seen < target) *sm.abort = 2;
    }
  }
  consumer_sync();
}

// ---- attention for one (head, split); DPL = head-dim slots per lane ------------------------------
// Latency plan: one L2 round trip for q/k/v and the norm weights, one combined block reduction
// for both RMS sums, then every warp fetches all of its keys (K and V rows, up to KB at a time)
// before touching any of them, so a short context costs one more round trip, not one per key.
template <int DPL>
__device__ __forceinline__ void phase_attention(const MegaArgs& a, int l, const MegaLayer* L, int cta,
                                                int64_t pos, int64_t seq, int nsplit, const Smem& sm,
                                                int tid, int lane, int warp, Prof& prof) {
  if (cta >= a.nh * nsplit) return;
  unsigned long long tp = prof.tic();
  constexpr int KB = 4;  // keys in flight per warp
  const int h = cta / nsplit, sp = cta - h * nsplit;
  const int grp = a.nh / a.nkv, kvh = h / grp, gi = h - kvh * grp;
  const int d = a.d, half = d / 2;
  float* qs = sm.misc;           // [256]
  float* kn = sm.misc + 256;     // [256]
  float* vn = sm.misc + 512;     // [256]
  float* wm = sm.misc + 768;     // [16]
  float* wl = sm.misc + 784;     // [16]
  float* red = sm.misc + 800;    // [64]
  float* wacc = sm.misc + 1024;  // [16][256]
  // thread i < d/2 owns the rotation pair (i, i + d/2) of q and of k
  float q1 = 0.f, q2 = 0.f, k1 = 0.f, k2 = 0.f, wq1 = 1.f, wq2 = 1.f, wk1 = 1.f, wk2 = 1.f;
  const bool pair = tid < half;
  if (pair) {
    q1 = __ldcg(a.q + (int64_t)h * d + tid);
    q2 = __ldcg(a.q + (int64_t)h * d + tid + half);
    k1 = __ldcg(a.k + (int64_t)kvh * d + tid);
    k2 = __ldcg(a.k + (int64_t)kvh * d + tid + half);
    if (a.has_norm) {
      const uint8_t* qw = reinterpret_cast<const uint8_t*>(L->q_norm);
      const uint8_t* kw = reinterpret_cast<const uint8_t*>(L->k_norm);
      wq1 = aux_load(qw, L->qk_norm_type, tid), wq2 = aux_load(qw, L->qk_norm_type, tid + half);
      wk1 = aux_load(kw, L->qk_norm_type, tid), wk2 = aux_load(kw, L->qk_norm_type, tid + half);
    }
  }
  for (int i = tid; i < d; i += MK_CT) vn[i] = round_kv(__ldcg(a.v + (int64_t)kvh * d + i), a.kv_type);
  float qinv = 1.f, kinv = 1.f;
  unsigned long long tq_ = prof.tic();
  if (a.has_norm) {
    float sq = warp_sum(fmaf(q1, q1, q2 * q2)), sk = warp_sum(fmaf(k1, k1, k2 * k2));
    prof.toc(16, tp);  // q/k/v and norm weights arrived
    tq_ = prof.tic();
    consumer_sync();
    if (lane == 0) {
      red[warp] = sq;
      red[32 + warp] = sk;
    }
    consumer_sync();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int i = 0; i < MK_CW; i++) {
      tq += red[i];
      tk += red[32 + i];
    }
    qinv = 1.0f / sqrtf(tq / (float)d + a.eps);
    kinv = 1.0f / sqrtf(tk / (float)d + a.eps);
    prof.toc(17, tq_);  // block reduction of the two RMS sums
    tq_ = prof.tic();
  }
  if (pair) {
    if (a.has_norm) {
      q1 = __fmul_rn(__fmul_rn(q1, qinv), wq1);
      q2 = __fmul_rn(__fmul_rn(q2, qinv), wq2);
      k1 = __fmul_rn(__fmul_rn(k1, kinv), wk1);
      k2 = __fmul_rn(__fmul_rn(k2, kinv), wk2);
    }
    if (a.has_rope) {
      const float cv = sm.misc[MK_ROPE_OFF + tid], sv = sm.misc[MK_ROPE_OFF + 128 + tid];  // once per token
      const float ql = __fsub_rn(__fmul_rn(q1, cv), __fmul_rn(q2, sv));
      const float qh = __fadd_rn(__fmul_rn(q1, sv), __fmul_rn(q2, cv));
      const float kl = __fsub_rn(__fmul_rn(k1, cv), __fmul_rn(k2, sv));
      const float kh = __fadd_rn(__fmul_rn(k1, sv), __fmul_rn(k2, cv));
      q1 = ql, q2 = qh, k1 = kl, k2 = kh;
    }
    qs[tid] = q1;
    qs[tid + half] = q2;
    kn[tid] = round_kv(k1, a.kv_type);
    kn[tid + half] = round_kv(k2, a.kv_type);
  }
  uint8_t* kc = a.kcache + (uint64_t)l * a.layer_stride;
  uint8_t* vc = a.vcache + (uint64_t)l * a.layer_stride;
  const int64_t plane = ((seq * a.nkv + kvh) * a.cap) * d;  // element offset of this head's plane
  const int64_t n = pos + 1;
  const int64_t per = (n + nsplit - 1) / nsplit;
  const int64_t k_lo = (int64_t)sp * per;
  const int64_t k_hi = (k_lo + per < n) ? k_lo + per : n;
  // A lane owns DPL consecutive head dims (one 8- or 16-byte piece of every cached row), so a
  // warp reads a key or value row with one coalesced vector load. First batch of this warp's
  // keys: the loads are issued before the barrier that publishes q.
  constexpr int WPL = DPL;  // raw words per lane and row (f32 cache); 2-byte caches use DPL / 2
  const bool wide = a.kv_type == E_F32;
  const int e0 = lane * DPL;  // first head dim of this lane
  const bool lane_live = e0 < d;
  uint32_t kraw[KB][WPL], vraw[KB][WPL];
  auto fetch = [&](int64_t key0) {
#pragma unroll
    for (int b = 0; b < KB; b++) {
      const int64_t key = key0 + (int64_t)b * MK_CW;
#pragma unroll
      for (int w = 0; w < WPL; w++) kraw[b][w] = vraw[b][w] = 0;
      if (key < k_hi && key != pos && lane_live) {
        const int64_t el = plane + key * d + e0;
        if (wide) {
          const uint4* kp = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(kc) + el);
          const uint4* vp = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(vc) + el);
#pragma unroll
          for (int w4 = 0; w4 < WPL / 4; w4++) {
            const uint4 kk = kp[w4], vv = vp[w4];
            kraw[b][4 * w4] = kk.x, kraw[b][4 * w4 + 1] = kk.y, kraw[b][4 * w4 + 2] = kk.z, kraw[b][4 * w4 + 3] = kk.w;
            vraw[b][4 * w4] = vv.x, vraw[b][4 * w4 + 1] = vv.y, vraw[b][4 * w4 + 2] = vv.z, vraw[b][4 * w4 + 3] = vv.w;
          }
        } else {
          const uint2* kp = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(kc) + el);
          const uint2* vp = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(vc) + el);
#pragma unroll
          for (int w2 = 0; w2 < WPL / 4; w2++) {
            const uint2 kk = kp[w2], vv = vp[w2];
            kraw[b][2 * w2] = kk.x, kraw[b][2 * w2 + 1] = kk.y;
            vraw[b][2 * w2] = vv.x, vraw[b][2 * w2 + 1] = vv.y;
          }
        }
      }
    }
  };
  // element j of a raw row piece as f32
  auto elem = [&](const uint32_t (&raw)[WPL], int j) -> float {
    if (wide) return __uint_as_float(raw[j]);
    const uint32_t bits = (raw[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    return a.kv_type == E_F16 ? f16_bits_to_f32(bits) : bf16_bits_to_f32(bits);
  };
  prof.toc(18, tq_);  // norm, RoPE, shared-memory hand-off, cache addresses
  tq_ = prof.tic();
  fetch(k_lo + warp);
  prof.toc(19, tq_);  // issuing the first key / value loads
  consumer_sync();
  prof.toc(13, tp);
  tp = prof.tic();
  if (sp == 0 && gi == 0) {
    for (int i = tid; i < d; i += MK_CT) {
      store_kv(kc, a.kv_type, plane + pos * d + i, kn[i]);
      store_kv(vc, a.kv_type, plane + pos * d + i, vn[i]);
    }
  }
  const float scale = 1.0f / sqrtf((float)d);
  float qreg[DPL], acc[DPL];
#pragma unroll
  for (int j = 0; j < DPL; j++) {
    qreg[j] = lane_live ? qs[e0 + j] : 0.f;
    acc[j] = 0.f;
  }
  float m = -3.40282347e38f, lsum = 0.f;
  for (int64_t key0 = k_lo + warp; key0 < k_hi; key0 += (int64_t)KB * MK_CW) {
    if (key0 != k_lo + warp) fetch(key0);
    float sc[KB];
#pragma unroll
    for (int b = 0; b < KB; b++) {
      const int64_t key = key0 + (int64_t)b * MK_CW;
      float dot = 0.f;
      if (lane_live) {
#pragma unroll
        for (int j = 0; j < DPL; j++) dot = fmaf(qreg[j], key == pos ? kn[e0 + j] : elem(kraw[b], j), dot);
      }
      sc[b] = warp_sum(dot) * scale;
    }
#pragma unroll
    for (int b = 0; b < KB; b++) {
      const int64_t key = key0 + (int64_t)b * MK_CW;
      if (key < k_hi) {
        const float mn = fmaxf(m, sc[b]);
        const float factor = expf(m - mn);
        const float p = expf(sc[b] - mn);
        lsum = lsum * factor + p;
        if (lane_live) {
#pragma unroll
          for (int j = 0; j < DPL; j++)
            acc[j] = acc[j] * factor + p * (key == pos ? vn[e0 + j] : elem(vraw[b], j));
        }
        m = mn;
      }
    }
  }
  prof.toc(14, tp);
  tp = prof.tic();
  if (lane == 0) {
    wm[warp] = m;
    wl[warp] = lsum;
  }
  if (lane_live) {
#pragma unroll
    for (int j = 0; j < DPL; j++) wacc[warp * 256 + e0 + j] = acc[j];
  }
  consumer_sync();
  float gm = wm[0];
#pragma unroll
  for (int w = 1; w < MK_CW; w++) gm = fmaxf(gm, wm[w]);
  // each warp's weight exp(m_w - gm) once, by one lane per warp, instead of per output element
  float* wwt = red;  // [16], free since the RMS reduction
  if (tid < MK_CW) wwt[tid] = expf(wm[tid] - gm);
  consumer_sync();
  float gl = 0.f;
#pragma unroll
  for (int w = 0; w < MK_CW; w++) gl += wl[w] * wwt[w];
  float* part = a.attn_part + ((int64_t)h * a.max_split + sp) * (d + 2);
  for (int idx = tid; idx < d; idx += MK_CT) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < MK_CW; w++) o += wacc[w * 256 + idx] * wwt[w];
    if (nsplit == 1)
      a.ctx[(int64_t)h * d + idx] = o / gl;
    else
      part[idx] = o;
  }
  if (nsplit > 1 && tid == 0) {
    part[d] = gm;
    part[d + 1] = gl;
  }
  prof.toc(15, tp);
}

// ---- the kernel ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(MK_THREADS, 1) decode_mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  __shared__ int s_abort;

  Smem sm;
  sm.nslot = a.nslot;
  sm.xs = reinterpret_cast<float*>(smem_raw);
  sm.xf = reinterpret_cast<__half*>(sm.xs + a.xs_floats);
  sm.sx32 = reinterpret_cast<float*>(sm.xf + (size_t)a.xs_floats * 2);
  sm.sx16 = sm.sx32 + a.xs_floats / 32;
  sm.misc = sm.sx16 + a.xs_floats / 16;
  sm.ring = reinterpret_cast<uint8_t*>(sm.misc + MK_MISC_FLOATS);
  sm.full = reinterpret_cast<uint64_t*>(sm.ring + (size_t)a.nslot * MK_SLOT);
  sm.empty = sm.full + a.nslot;
  sm.part_full = sm.empty + a.nslot;
  sm.part_empty = sm.part_full + 2;
  sm.prog_bar = sm.part_empty + 2;
  uint8_t* prog_area = reinterpret_cast<uint8_t*>(sm.prog_bar + 2);
  const int nph = 4 * a.layers + 1;
  sm.prog = a.prog + (size_t)cta * a.max_chunks;
  sm.counts = a.counts + (size_t)cta * nph;
  sm.abort = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < a.nslot; i++) {
      mbar_init(sm.full + i, 1);
      mbar_init(sm.empty + i, MK_CW);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(sm.part_full + i, MK_CW);
      mbar_init(sm.part_empty + i, 1);
    }
    mbar_init(sm.prog_bar, 1);
    mbar_fence_init();
    if (a.prog_in_smem) {
      // one bulk copy brings this CTA's whole program next to the math
      const unsigned bytes = (unsigned)a.max_chunks * (unsigned)sizeof(MegaChunk);
      mbar_expect_tx(sm.prog_bar, bytes);
      bulk_g2s(prog_area, sm.prog, bytes, sm.prog_bar);
    }
  }
  __syncthreads();
  if (a.prog_in_smem) {
    uint16_t* cdst = reinterpret_cast<uint16_t*>(prog_area + (size_t)a.max_chunks * sizeof(MegaChunk));
    for (int i = tid; i < nph; i += MK_THREADS) cdst[i] = sm.counts[i];
    if (!mbar_wait_bounded(sm.prog_bar, 0, MK_MBAR_SPINS, sm.abort) && !*sm.abort) *sm.abort = 7;
    __syncthreads();
    sm.prog = reinterpret_cast<const MegaChunk*>(prog_area);
    sm.counts = cdst;
  }

  if (warp == MK_CW) {
    // ------------------------------ producer: stream this CTA's weight tiles --------------
    int total = 0;
    for (int i = lane; i < nph; i += 32) total += sm.counts[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    for (int pi = 0; pi < total; pi++) produce_chunk(sm.prog + pi, sm, (uint32_t)pi, lane);
    return;
  }

  // -------------------------------- consumers -------------------------------------------------
  GridBar gb;
  gb.gen = 0;
  if (tid == 0) gb.gen = *reinterpret_cast<const volatile unsigned long long*>(a.bar) / (unsigned long long)G;
  const int64_t token = __ldcg(a.io + 0), pos = __ldcg(a.io + 1), seq = __ldcg(a.io + 2);
  int nsplit = (int)((pos + 1 + 63) / 64);
  if (nsplit > a.max_split) nsplit = a.max_split;
  if (nsplit < 1) nsplit = 1;
  const int64_t qd = (int64_t)a.nh * a.d;
  const int g = lane >> 2;
  uint32_t ci = 0;
  unsigned closes = 0;
  float out_scale = 1.f;
  float bv = -INFINITY;  // running argmax over the rows this thread finalises
  long long bi = 0x7fffffffffffffffLL;
  Prof prof;
  prof.begin(a.prof, cta == 0 && tid == 0);
  TileAcc<true> acc, acc2;

  // One phase's chunks, in program order.
  const MegaChunk* prog = sm.prog;
  const uint16_t* counts = sm.counts;
  auto run_phase = [&](int phase_index) {
    acc.clear();
    acc2.clear();
    const int cnt = counts[phase_index];
    for (int k = 0; k < cnt; k++, ci++) {
      const MegaChunk* c = prog + ci;
      const int slot = ci % sm.nslot;
      // the finalising lanes fetch the residual now so that it is there when the tile closes
      float resid = 0.f;
      if (warp == 0 && lane < 16 && lane < c->n && (c->flags & 1) && ((c->flags >> 2) & 3) == MEGA_EP_RESIDUAL)
        resid = __ldcg(c->out + c->out_row + lane);
      const unsigned long long tw = prof.tic();
      const bool ok = mbar_wait_bounded(sm.full + slot, (ci / sm.nslot) & 1u, MK_MBAR_SPINS, sm.abort);
      if (!ok && !*sm.abort) *sm.abort = 3;
      prof.toc(10, tw);
      const unsigned long long tr = prof.tic();
      const int n = c->n, nu = c->nu, flags = c->flags;
      if (ok) {
        const uint8_t* base = sm.ring + (size_t)slot * MK_SLOT;
        const int i0 = g < n ? g : n - 1, i1 = g + 8 < n ? g + 8 : n - 1;  // clamp to valid rows
        const uint32_t pitch = c->pitch, rb = c->rb;
        const uint8_t* src = c->src;
        const uint8_t* p0 = base + i0 * pitch + (reinterpret_cast<uintptr_t>(src + (size_t)i0 * rb) & 15);
        const uint8_t* p1 = base + i1 * pitch + (reinterpret_cast<uintptr_t>(src + (size_t)i1 * rb) & 15);
        const uint8_t* a0 = nullptr;
        const uint8_t* a1 = nullptr;
        const int apitch = c->apitch;
        if (c->aseg) {
          const uint8_t* ab = base + 16 * pitch;
          a0 = ab + i0 * apitch + (reinterpret_cast<uintptr_t>(c->sc + (size_t)i0 * c->arb) & 15);
          a1 = ab + i1 * apitch + (reinterpret_cast<uintptr_t>(c->sc + (size_t)i1 * c->arb) & 15);
        }
        const int enc = c->enc, aux = c->aux, gs = c->group_shift, kb0 = c->kb0;
        TileAcc<true>& A = (flags & 2) ? acc2 : acc;
        for (int u = warp; u < nu; u += MK_CW) run_unit(enc, aux, gs, p0, p1, a0, a1, 16 * apitch, u, kb0, sm, lane, A);
      }
      prof.toc(11, tr);
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.empty + slot);
      if (!(flags & 1)) continue;
      // tile complete: per-warp partial sums -> warp 0 adds them in a fixed order -> epilogue.
      // The other warps do not wait: they hand their sums over through an mbarrier and go on.
      const int buf = closes & 1;
      const unsigned use = closes >> 1;
      if (use > 0) {
        if (!mbar_wait_bounded(sm.part_empty + buf, (use - 1u) & 1u, MK_MBAR_SPINS, sm.abort) && !*sm.abort)
          *sm.abort = 5;
      }
      float* pw = sm.misc + MK_PART_OFF + ((size_t)buf * MK_CW + warp) * 32;
      if ((lane & 3) == 0) {
        pw[g] = acc.v[0];
        pw[g + 8] = acc.v[1];
        pw[16 + g] = acc2.v[0];
        pw[16 + g + 8] = acc2.v[1];
      }
      acc.clear();
      acc2.clear();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.part_full + buf);
      if (warp == 0) {
        if (!mbar_wait_bounded(sm.part_full + buf, use & 1u, MK_MBAR_SPINS, sm.abort) && !*sm.abort)
          *sm.abort = 6;
        if (lane < 16 && lane < n) {
          const float* pb = sm.misc + MK_PART_OFF + (size_t)buf * MK_CW * 32 + lane;
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int wv = 0; wv < MK_CW; wv++) {
            s0 += pb[wv * 32];
            s1 += pb[wv * 32 + 16];
          }
          s0 *= out_scale;
          s1 *= out_scale;
          const int ep = (flags >> 2) & 3;
          const int64_t row = (int64_t)c->out_row + lane;
          float* out = c->out;
          if (ep == MEGA_EP_STORE) {
            out[row] = s0;
          } else if (ep == MEGA_EP_RESIDUAL) {
            out[row] = resid + s0;
          } else if (ep == MEGA_EP_SWIGLU) {
            out[row] = (s0 / (1.0f + expf(-s0))) * s1;
          } else {
            out[row] = s0;
            if (s0 > -INFINITY && arg_better(s0, row, bv, bi)) bv = s0, bi = row;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.part_empty + buf);
      }
      closes++;
    }
  };

  auto gsync = [&]() {
    const unsigned long long t_ = prof.tic();
    grid_sync(a, gb, G, tid, sm);
    prof.toc(12, t_);
  };

  if (a.has_rope && tid < a.d / 2) {
    // the rotation of this token's position, shared by all layers (kernels.rs:1047-1064)
    float sv, cv;
    sincosf(__fmul_rn((float)pos, a.ft.f[tid]), &sv, &cv);
    sm.misc[MK_ROPE_OFF + tid] = cv;
    sm.misc[MK_ROPE_OFF + 128 + tid] = sv;
  }
  if (cta == 0) mega_gather_row(a.embed, token, a.hidden, tid, MK_CT);
  gsync();
  prof.mark(0);

  for (int l = 0; l < a.layers; l++) {
    const MegaLayer* L = a.L + l;
    unsigned long long ts = prof.tic();
    out_scale = stage_phase(a.hidden, false, L->attn_norm, L->norm_type, a.H, a.eps,
                            xl_for_encoding(L->q.enc), sm, tid, lane, warp);
    prof.toc(9, ts);
    run_phase(4 * l + 0);
    gsync();
    prof.mark(1);
    if (!*sm.abort) {
      if (a.d <= 128)
        phase_attention<4>(a, l, L, cta, pos, seq, nsplit, sm, tid, lane, warp, prof);
      else
        phase_attention<8>(a, l, L, cta, pos, seq, nsplit, sm, tid, lane, warp, prof);
    }
    gsync();
    prof.mark(2);
    ts = prof.tic();
    if (nsplit > 1) {
      for (int e = tid; e < qd; e += MK_CT) {
        const int h = e / a.d, i = e - h * a.d;
        const float* p0 = a.attn_part + (int64_t)h * a.max_split * (a.d + 2);
        float pm[16], pl[16], po[16];
#pragma unroll
        for (int s = 0; s < 16; s++)
          if (s < nsplit) {
            const float* ps = p0 + s * (a.d + 2);
            pm[s] = __ldcg(ps + a.d);
            pl[s] = __ldcg(ps + a.d + 1);
            po[s] = __ldcg(ps + i);
          }
        float gm = -3.40282347e38f;
#pragma unroll
        for (int s = 0; s < 16; s++)
          if (s < nsplit) gm = fmaxf(gm, pm[s]);
        float o = 0.f, gl = 0.f;
#pragma unroll
        for (int s = 0; s < 16; s++)
          if (s < nsplit) {
            const float wgt = expf(pm[s] - gm);
            o += po[s] * wgt;
            gl += pl[s] * wgt;
          }
        sm.xs[e] = o / gl;
      }
      consumer_sync();
    }
    out_scale = stage_phase(a.ctx, nsplit > 1, nullptr, 0, (int)qd, 0.f, xl_for_encoding(L->o.enc), sm,
                            tid, lane, warp);
    prof.toc(9, ts);
    run_phase(4 * l + 1);
    gsync();
    prof.mark(3);
    ts = prof.tic();
    out_scale = stage_phase(a.hidden, false, L->ffn_norm, L->norm_type, a.H, a.eps,
                            xl_for_encoding(L->gate.enc), sm, tid, lane, warp);
    prof.toc(9, ts);
    run_phase(4 * l + 2);
    gsync();
    prof.mark(4);
    ts = prof.tic();
    out_scale = stage_phase(a.act, false, nullptr, 0, a.I, 0.f, xl_for_encoding(L->down.enc), sm, tid,
                            lane, warp);
    prof.toc(9, ts);
    run_phase(4 * l + 3);
    gsync();
    prof.mark(5);
  }

  // ---- final norm + lm_head + argmax partials (first strict maximum)
  {
    const unsigned long long ts = prof.tic();
    out_scale = stage_phase(a.hidden, false, a.out_norm, a.out_norm_type, a.H, a.eps,
                            xl_for_encoding(a.lm_head.enc), sm, tid, lane, warp);
    prof.toc(9, ts);
  }
  run_phase(4 * a.layers);
  if (warp == 0) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {  // the 16 finalising threads are lanes 0..15 of warp 0
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (arg_better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) {
      a.argmax_val[cta] = bv;
      a.argmax_idx[cta] = bi;
    }
  }
  gsync();
  prof.mark(6);
  if (cta == 0 && warp == 0) {
    float v = -INFINITY;
    long long i = 0x7fffffffffffffffLL;
    for (int c = lane; c < G; c += 32) {
      const float cv = __ldcg(a.argmax_val + c);
      const long long cidx = __ldcg(a.argmax_idx + c);
      if (arg_better(cv, cidx, v, i)) v = cv, i = cidx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (arg_better(ov, oi, v, i)) v = ov, i = oi;
    }
    if (lane == 0) {
      const int64_t tok = i == 0x7fffffffffffffffLL ? 0 : (int64_t)i;
      a.io[3] = tok;
      if (a.advance) {
        a.io[0] = tok;
        a.io[1] = pos + 1;
        const int64_t cnt = a.hist_count[0];
        if (cnt < a.hist_cap) a.hist[cnt] = tok;
        a.hist_count[0] = cnt + 1;
      }
    }
  }
  prof.mark(7);
  prof.end();
  if (tid == 0 && *sm.abort) {
    atomicExch(a.error, *sm.abort);
    // let any bulk copy still in flight land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < (1LL << 22)) {
    }
  }
}

}  // namespace

size_t mega_smem_bytes(int nslot, int xs_floats, size_t prog_bytes) {
  return (size_t)xs_floats * 4 * 2 + (size_t)(xs_floats / 32 + xs_floats / 16) * 4 +
         (size_t)MK_MISC_FLOATS * 4 + (size_t)nslot * MK_SLOT + (size_t)nslot * 16 + 128 + prog_bytes;
}

// prog_bytes: bytes of one CTA's program (chunks + counts, 16-byte rounded) to keep in shared
// memory; *prog_in_smem tells whether it fit beside a ring of at least 5 slots.
int mega_plan(int H, int I, int qd, int d, size_t prog_bytes, int* nslot, int* xs_floats, size_t* smem,
              int* prog_in_smem) {
  int xs = H > I ? H : I;
  if (qd > xs) xs = qd;
  xs = (xs + 255) / 256 * 256;
  if (d > 256 || xs > 8 * MK_CT) return 0;  // staging: one 8-element item per consumer thread
  const size_t budget = 225 * 1024;
  size_t fixed = mega_smem_bytes(0, xs, 0) + 512;
  if (fixed + 4 * (size_t)MK_SLOT > budget) return 0;
  *prog_in_smem = 0;
  if (prog_bytes && fixed + prog_bytes + 5 * (size_t)(MK_SLOT + 16) <= budget) {
    *prog_in_smem = 1;
    fixed += prog_bytes;
  }
  int n = (int)((budget - fixed) / (MK_SLOT + 16));
  if (n > 12) n = 12;
  *nslot = n;
  *xs_floats = xs;
  *smem = mega_smem_bytes(n, xs, *prog_in_smem ? prog_bytes : 0);
  return 1;
}

// ---- host: chunk programs ------------------------------------------------------------------------
namespace {
int host_bank_pitch(int bytes) {
  int p = (bytes + 15) / 16 * 16;
  while ((p / 4) % 8 != 4) p += 16;
  return p;
}
struct HostPlan {
  int ubytes, ukb, units_total, unit_q6;
};
HostPlan host_plan(const WRef& w) {
  HostPlan p{0, 1, 0, 0};
  const int K = (int)w.cols;
  switch (w.enc) {
    case E_Q4_0: p.ubytes = 36, p.ukb = 2, p.units_total = K / 64; break;
    case E_Q4_1: p.ubytes = 20, p.ukb = 1, p.units_total = K / 32; break;
    case E_Q8_0: p.ubytes = 68, p.ukb = 2, p.units_total = K / 64; break;
    case E_MLX_U4: p.ubytes = 16, p.ukb = 1, p.units_total = K / 32; break;
    default: p.ubytes = 0, p.ukb = 2, p.units_total = K / 64, p.unit_q6 = 1; break;  // quarters
  }
  return p;
}
int seg_bytes(const HostPlan& p, int nu) { return p.unit_q6 ? (nu / 4) * 210 : nu * p.ubytes; }

// Appends the chunks of rows [lo, hi) of `w`: tiles of 16 rows, each cut into the fewest K-slices
// whose rows fit one ring slot (slices are multiples of 16 units so the 16 consumer warps share
// them evenly; Q6_K slices are whole groups of 4 superblocks, which keeps rows 8-byte aligned).
void add_tensor_chunks(const WRef& w, int64_t lo, int64_t hi, float* out, int ep, bool second,
                       bool closes, std::vector<MegaChunk>* v) {
  const HostPlan p = host_plan(w);
  const int ael = w.aux == E_F32 ? 4 : 2;
  for (int64_t r = lo; r < hi; r += 16) {
    const int n = (int)std::min<int64_t>(16, hi - r);
    // largest slice (multiple of 16 units) whose rows fit one slot; only valid rows are copied
    int su = p.units_total < 16 ? p.units_total : 16;
    for (int cand = 16; cand <= p.units_total && cand <= 240; cand += 16) {
      const int pitch = host_bank_pitch(seg_bytes(p, cand) + 20);
      const int ap = w.enc == E_MLX_U4 ? ((cand * 32 / w.group) * ael + 31) / 16 * 16 : 0;
      const size_t need = ap ? (size_t)16 * pitch + 32 * (size_t)ap : (size_t)n * pitch;
      if (need <= (size_t)MK_SLOT && pitch < 65536) su = cand;
    }
    const int nsl = (p.units_total + su - 1) / su;
    for (int sl = 0; sl < nsl; sl++) {
      const int u0 = sl * su, nu = std::min(su, p.units_total - u0);
      MegaChunk c{};
      const int64_t boff = p.unit_q6 ? (int64_t)(u0 / 4) * 210 : (int64_t)u0 * p.ubytes;
      c.src = w.data + r * w.row_bytes() + boff;
      c.rb = (uint32_t)w.row_bytes();
      c.seg = (uint16_t)seg_bytes(p, nu);
      c.pitch = (uint16_t)host_bank_pitch(seg_bytes(p, su) + 20);
      c.kb0 = (uint16_t)(u0 * p.ukb);
      c.n = (uint8_t)n;
      c.nu = (uint8_t)nu;
      c.enc = (uint8_t)w.enc;
      c.out = out;
      c.out_row = (int32_t)r;
      c.flags = (uint8_t)(((closes && sl == nsl - 1) ? 1 : 0) | (second ? 2 : 0) | (ep << 2));
      if (w.enc == E_MLX_U4) {
        const int64_t arow = (int64_t)(w.cols / w.group) * ael, ao = (int64_t)(u0 * 32 / w.group) * ael;
        c.sc = w.scales + r * arow + ao;
        c.bi = w.biases + r * arow + ao;
        c.arb = (uint32_t)arow;
        c.aseg = (uint16_t)((nu * 32 / w.group) * ael);
        c.apitch = (uint16_t)(((su * 32 / w.group) * ael + 31) / 16 * 16);
        c.aux = (uint8_t)w.aux;
        c.group_shift = (uint8_t)(w.group == 32 ? 0 : (w.group == 64 ? 1 : 2));
      }
      v->push_back(c);
    }
  }
}
}  // namespace

int mega_build_program(const MegaBuildLayer* layers, int nlayers, const WRef& lm_head, int nh, int nkv,
                       int d, int H, int I, int V, float* q, float* k, float* v, float* hidden,
                       float* act, float* logits, int grid, std::vector<MegaChunk>* chunks,
                       std::vector<uint16_t>* counts, int* max_chunks) {
  const int nph = 4 * nlayers + 1;
  std::vector<std::vector<MegaChunk>> per(grid);
  counts->assign((size_t)grid * nph, 0);
  const int64_t qd = (int64_t)nh * d, kvd = (int64_t)nkv * d;
  for (int cta = 0; cta < grid; cta++) {
    std::vector<MegaChunk>& pc = per[cta];
    auto close_phase = [&](int ph, size_t before) {
      (*counts)[(size_t)cta * nph + ph] = (uint16_t)(pc.size() - before);
    };
    for (int l = 0; l < nlayers; l++) {
      const MegaBuildLayer& L = layers[l];
      size_t b0 = pc.size();
      {  // q, k, v share one balanced split of their concatenated rows
        const int64_t R = qd + 2 * kvd, a0 = R * cta / grid, a1 = R * (cta + 1) / grid;
        const int64_t offs[3] = {0, qd, qd + kvd}, lens[3] = {qd, kvd, kvd};
        const WRef* ws[3] = {&L.q, &L.k, &L.v};
        float* outs[3] = {q, k, v};
        for (int t = 0; t < 3; t++) {
          const int64_t lo = std::max(a0, offs[t]) - offs[t], hi = std::min(a1, offs[t] + lens[t]) - offs[t];
          if (hi > lo) add_tensor_chunks(*ws[t], lo, hi, outs[t], MEGA_EP_STORE, false, true, &pc);
        }
      }
      close_phase(4 * l + 0, b0);
      b0 = pc.size();
      add_tensor_chunks(L.o, (int64_t)H * cta / grid, (int64_t)H * (cta + 1) / grid, hidden, MEGA_EP_RESIDUAL,
                        false, true, &pc);
      close_phase(4 * l + 1, b0);
      b0 = pc.size();
      {  // per tile: gate slices, then up slices into the second accumulator; the pair closes after up
        const int64_t lo = (int64_t)I * cta / grid, hi = (int64_t)I * (cta + 1) / grid;
        for (int64_t r = lo; r < hi; r += 16) {
          const int64_t e = std::min(r + 16, hi);
          add_tensor_chunks(L.gate, r, e, act, MEGA_EP_SWIGLU, false, false, &pc);
          add_tensor_chunks(L.up, r, e, act, MEGA_EP_SWIGLU, true, true, &pc);
        }
      }
      close_phase(4 * l + 2, b0);
      b0 = pc.size();
      add_tensor_chunks(L.down, (int64_t)H * cta / grid, (int64_t)H * (cta + 1) / grid, hidden,
                        MEGA_EP_RESIDUAL, false, true, &pc);
      close_phase(4 * l + 3, b0);
    }
    const size_t b0 = pc.size();
    add_tensor_chunks(lm_head, (int64_t)V * cta / grid, (int64_t)V * (cta + 1) / grid, logits, MEGA_EP_LOGITS,
                      false, true, &pc);
    close_phase(4 * nlayers, b0);
  }
  size_t mc = 1;
  for (auto& pc : per) mc = std::max(mc, pc.size());
  DYN_CHECK(mc < 60000, "decode program too long (%zu chunks per CTA)", mc);
  *max_chunks = (int)mc;
  chunks->assign((size_t)grid * mc, MegaChunk{});
  for (int cta = 0; cta < grid; cta++)
    std::copy(per[cta].begin(), per[cta].end(), chunks->begin() + (size_t)cta * mc);
  return 0;
}

// Whether the persistent kernel's tile steps can read this tensor (encoding and row alignment).
bool mega_supports_weight(const WRef& w) {
  switch (w.enc) {
    case E_Q4_0:
    case E_Q8_0: return w.cols % 256 == 0;
    case E_Q4_1: return w.cols % 128 == 0;
    case E_Q6_K: return w.cols % 1024 == 0;
    case E_MLX_U4: return w.cols % 256 == 0 && (w.group == 32 || w.group == 64 || w.group == 128);
    default: return false;
  }
}

int mega_grid_size(int device, size_t smem, int* grid) {
  DYN_CUDA(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)smem));
  int sms = 0, per_sm = 0, coop = 0;
  DYN_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  DYN_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  DYN_CHECK(coop != 0, "device %d does not support cooperative launches", device);
  DYN_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, MK_THREADS,
                                                         smem));
  DYN_CHECK(per_sm >= 1, "the decode kernel does not fit one CTA per SM with %zu bytes of shared memory", smem);
  *grid = sms;
  return 0;
}

int launch_decode_mega(const MegaArgs& a, int grid, size_t smem, cudaStream_t s) {
  void* args[] = {const_cast<MegaArgs*>(&a)};
  DYN_CUDA(cudaLaunchCooperativeKernel((void*)decode_mega_kernel, dim3(grid), dim3(MK_THREADS), args,
                                       smem, s));
  count_launch();
  return 0;
}

}  // namespace dyn
