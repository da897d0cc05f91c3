// Persistent single-token decode kernel: one launch per generated token.
//
// One CTA per SM, launched cooperatively so that all CTAs are co-resident. Each
// CTA owns a fixed, balanced slice of the rows of every weight matrix. A producer
// warp streams that slice — the verbatim checkpoint bytes — from HBM into a
// shared-memory ring with 1-D bulk async copies (cp.async.bulk + mbarrier
// transaction counts), running as far ahead of the math as the ring allows:
// weight traffic never waits for the activation dependency chain. Eight consumer
// warps decode rows straight out of shared memory (exact f32 weights, f32
// accumulation) against the activation vector staged in shared memory, and the
// CTAs meet at a grid barrier between dependent phases:
//
//   embed | per layer: norm+QKV | qk-norm+RoPE+KV-write+attention | o_proj+res |
//   norm+gate/up+SwiGLU | down+res | final: norm+lm_head+argmax partials | argmax
//
// Every wait (mbarrier, grid barrier) is bounded: when it gives up it raises the
// error word, the remaining phases are skipped in lockstep and the kernel ends.
#include <cooperative_groups.h>

#include "codec.cuh"
#include "decode_mega.cuh"

namespace dyn {

namespace {

constexpr int MK_CW = 16;               // consumer warps
constexpr int MK_CT = MK_CW * 32;       // consumer threads
constexpr int MK_THREADS = MK_CT + 32;  // + one producer warp
constexpr int MK_SLOT = 16384;          // bytes per ring slot
constexpr int MK_MISC_FLOATS = 6144;    // per-CTA scratch (attention state, reductions)
constexpr int MK_MAX_COPIES = 6;
constexpr long long MK_MBAR_SPINS = 1LL << 22;
constexpr long long MK_GRID_SPINS = 1LL << 22;

enum { PH_QKV = 0, PH_O, PH_GATEUP, PH_DOWN, PH_HEAD };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CT) : "memory"); }

struct Smem {
  float* xs;
  float* misc;
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  volatile int* abort;
  int nslot;
};

struct Chunk {
  int ncopy;
  const uint8_t* g[MK_MAX_COPIES];
  uint32_t bytes[MK_MAX_COPIES];
  uint32_t soff[MK_MAX_COPIES];  // slot offset of each copy
  uint32_t doff[MK_MAX_COPIES];  // slot offset of the first row's bytes of each component
  int64_t r0;
  int n;
  int tag;
};

__device__ __forceinline__ int aux_row_bytes(const WRef& w) {
  return (int)(w.cols / w.group) * (w.aux == E_F32 ? 4 : 2);
}
__device__ __forceinline__ int rows_per_region(const WRef& w, int region) {
  const int rb = (int)w.row_bytes();
  if (w.enc == E_MLX_U4) return (region - 96) / (rb + 2 * aux_row_bytes(w));
  return (region - 32) / rb;
}
__device__ __forceinline__ void add_copy(Chunk& c, const uint8_t* base, int64_t r0, int n, int rb,
                                         uint32_t& cursor) {
  const uint8_t* start = base + r0 * rb;
  const uintptr_t s = reinterpret_cast<uintptr_t>(start);
  const uint32_t off = (uint32_t)(s & 15);
  const int i = c.ncopy++;
  c.g[i] = start - off;
  c.bytes[i] = (off + (uint32_t)(n * rb) + 15u) & ~15u;
  c.soff[i] = cursor;
  c.doff[i] = cursor + off;
  cursor += c.bytes[i];
}
__device__ __forceinline__ void add_tensor(Chunk& c, const WRef& w, int64_t r0, int n,
                                           uint32_t region_off) {
  uint32_t cursor = region_off;
  add_copy(c, w.data, r0, n, (int)w.row_bytes(), cursor);
  if (w.enc == E_MLX_U4) {
    add_copy(c, w.scales, r0, n, aux_row_bytes(w), cursor);
    add_copy(c, w.biases, r0, n, aux_row_bytes(w), cursor);
  }
}

// Chunks of rows [s0, s1) of one tensor (or of a gate/up pair sharing row indices).
template <typename F>
__device__ __forceinline__ void chunks_of(const WRef& w, const WRef* pair, int64_t s0, int64_t s1,
                                          int tag, F&& f) {
  if (s1 <= s0) return;
  const int region = pair ? MK_SLOT / 2 : MK_SLOT;
  int rpc = rows_per_region(w, region);
  if (pair) {
    const int r2 = rows_per_region(*pair, region);
    rpc = r2 < rpc ? r2 : rpc;
  }
  if (rpc < 1) rpc = 1;  // excluded by mega_plan on the host
  if (rpc > MK_CW) rpc -= rpc % MK_CW;  // whole rounds of the consumer warps
  for (int64_t r = s0; r < s1; r += rpc) {
    Chunk c;
    c.ncopy = 0;
    c.r0 = r;
    c.n = (int)((s1 - r) < rpc ? (s1 - r) : rpc);
    c.tag = tag;
    add_tensor(c, w, r, c.n, 0);
    if (pair) add_tensor(c, *pair, r, c.n, MK_SLOT / 2);
    f(c);
  }
}

// The fixed per-CTA program of one phase: both roles enumerate exactly this sequence.
template <typename F>
__device__ __forceinline__ void enum_phase(const MegaArgs& a, const MegaLayer* L, int phase, int cta,
                                           int G, F&& f) {
  const int64_t qd = (int64_t)a.nh * a.d, kvd = (int64_t)a.nkv * a.d;
  if (phase == PH_QKV) {
    const int64_t R = qd + 2 * kvd;
    const int64_t a0 = R * cta / G, a1 = R * (cta + 1) / G;
    const int64_t offs[3] = {0, qd, qd + kvd};
    const int64_t lens[3] = {qd, kvd, kvd};
    const WRef* ws[3] = {&L->q, &L->k, &L->v};
#pragma unroll
    for (int t = 0; t < 3; t++) {
      const int64_t lo = (a0 > offs[t] ? a0 : offs[t]) - offs[t];
      const int64_t hi = (a1 < offs[t] + lens[t] ? a1 : offs[t] + lens[t]) - offs[t];
      chunks_of(*ws[t], nullptr, lo, hi, t, f);
    }
  } else if (phase == PH_O) {
    chunks_of(L->o, nullptr, (int64_t)a.H * cta / G, (int64_t)a.H * (cta + 1) / G, 0, f);
  } else if (phase == PH_GATEUP) {
    chunks_of(L->gate, &L->up, (int64_t)a.I * cta / G, (int64_t)a.I * (cta + 1) / G, 0, f);
  } else if (phase == PH_DOWN) {
    chunks_of(L->down, nullptr, (int64_t)a.H * cta / G, (int64_t)a.H * (cta + 1) / G, 0, f);
  } else {
    chunks_of(a.lm_head, nullptr, (int64_t)a.V * cta / G, (int64_t)a.V * (cta + 1) / G, 0, f);
  }
}

// ---- math on one row held in shared memory ------------------------------------------
template <int ENC>
__device__ __forceinline__ float dot_row_t(const RowPtr& rp, int64_t K, const float* xs, int lane) {
  using C = Codec<ENC>;
  const int nparts = (int)(K / C::BLOCK) * C::PARTS;
  float acc = 0.f;
#pragma unroll 4
  for (int it = lane; it < nparts; it += 32) {
    const int blk = it / C::PARTS, part = it - blk * C::PARTS;
    float wv[4 * C::G];
    C::decode(rp, blk, part, wv);
#pragma unroll
    for (int g = 0; g < C::G; g++) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + blk * C::BLOCK + C::xoff(part, g));
      acc = fmaf(wv[4 * g + 0], xv.x, acc);
      acc = fmaf(wv[4 * g + 1], xv.y, acc);
      acc = fmaf(wv[4 * g + 2], xv.z, acc);
      acc = fmaf(wv[4 * g + 3], xv.w, acc);
    }
  }
  return warp_sum(acc);
}

__device__ __forceinline__ float dot_row(int enc, const RowPtr& rp, int64_t K, const float* xs,
                                         int lane) {
  switch (enc) {
    case E_Q4_0: return dot_row_t<E_Q4_0>(rp, K, xs, lane);
    case E_Q4_1: return dot_row_t<E_Q4_1>(rp, K, xs, lane);
    case E_Q8_0: return dot_row_t<E_Q8_0>(rp, K, xs, lane);
    case E_Q6_K: return dot_row_t<E_Q6_K>(rp, K, xs, lane);
    case E_MLX_U4: return dot_row_t<E_MLX_U4>(rp, K, xs, lane);
    case E_BF16: return dot_row_t<E_BF16>(rp, K, xs, lane);
    case E_F16: return dot_row_t<E_F16>(rp, K, xs, lane);
    default: return dot_row_t<E_F32>(rp, K, xs, lane);
  }
}

template <int ENC>
__device__ __forceinline__ void gather_row_t(const WRef& w, int64_t row, float* out, int tid) {
  using C = Codec<ENC>;
  const RowPtr rp = row_ptr(w, row);
  const int nparts = (int)(w.cols / C::BLOCK) * C::PARTS;
  for (int it = tid; it < nparts; it += MK_CT) {
    const int blk = it / C::PARTS, part = it - blk * C::PARTS;
    float v[4 * C::G];
    C::decode(rp, blk, part, v);
#pragma unroll
    for (int g = 0; g < C::G; g++)
      *reinterpret_cast<float4*>(out + blk * C::BLOCK + C::xoff(part, g)) =
          make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
  }
}
__device__ __noinline__ void gather_row(const WRef& w, int64_t row, float* out, int tid) {
  switch (w.enc) {
    case E_Q4_0: gather_row_t<E_Q4_0>(w, row, out, tid); break;
    case E_Q4_1: gather_row_t<E_Q4_1>(w, row, out, tid); break;
    case E_Q8_0: gather_row_t<E_Q8_0>(w, row, out, tid); break;
    case E_Q6_K: gather_row_t<E_Q6_K>(w, row, out, tid); break;
    case E_MLX_U4: gather_row_t<E_MLX_U4>(w, row, out, tid); break;
    case E_BF16: gather_row_t<E_BF16>(w, row, out, tid); break;
    case E_F16: gather_row_t<E_F16>(w, row, out, tid); break;
    default: gather_row_t<E_F32>(w, row, out, tid); break;
  }
}

__device__ __forceinline__ RowPtr chunk_row(const WRef& w, const uint8_t* slot, const Chunk& c,
                                            int comp, int j) {
  RowPtr rp;
  rp.data = slot + c.doff[comp] + (int64_t)j * w.row_bytes();
  rp.aux = w.aux;
  rp.group = w.group;
  if (w.enc == E_MLX_U4) {
    const int ab = aux_row_bytes(w);
    rp.sc = slot + c.doff[comp + 1] + j * ab;
    rp.bi = slot + c.doff[comp + 2] + j * ab;
  } else {
    rp.sc = rp.bi = nullptr;
  }
  return rp;
}

// Sum over the consumer threads; every thread gets the total. `red` holds >= 8 floats.
__device__ __forceinline__ float consumer_sum(float v, float* red, int lane, int warp) {
  v = warp_sum(v);
  consumer_sync();
  if (lane == 0) red[warp] = v;
  consumer_sync();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < MK_CW; i++) t += red[i];
  return t;
}

// xs[i] = (x[i] * inv) * w[i]  with inv = 1/sqrt(mean(x^2) + eps); x is read from L2.
__device__ __forceinline__ void stage_norm(const float* x, const void* w, int w_type, int n,
                                           float eps, const Smem& sm, int tid, int lane, int warp) {
  float ss = 0.f;
  for (int i = tid; i < n; i += MK_CT) {
    const float v = __ldcg(x + i);
    sm.xs[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = consumer_sum(ss, sm.misc + MK_MISC_FLOATS - 32, lane, warp);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = tid; i < n; i += MK_CT)
    sm.xs[i] = __fmul_rn(__fmul_rn(sm.xs[i], inv),
                         aux_load(reinterpret_cast<const uint8_t*>(w), w_type, i));
  consumer_sync();
}

__device__ __forceinline__ bool wait_full(const Smem& sm, uint32_t ci) {
  uint64_t* bar = sm.full + (ci % sm.nslot);
  const unsigned parity = (ci / sm.nslot) & 1u;
  for (long long it = 0; it < MK_MBAR_SPINS; it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*sm.abort) return false;
  }
  *sm.abort = 3;
  return false;
}
__device__ __forceinline__ void release_slot(const Smem& sm, uint32_t ci, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(sm.empty + (ci % sm.nslot));
}

__device__ __forceinline__ float round_kv(float v, int kv_type) {
  if (kv_type == E_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (kv_type == E_F16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ float load_kv(const uint8_t* base, int kv_type, int64_t idx) {
  if (kv_type == E_F32) return reinterpret_cast<const float*>(base)[idx];
  const uint32_t b = reinterpret_cast<const uint16_t*>(base)[idx];
  return kv_type == E_F16 ? f16_bits_to_f32(b) : bf16_bits_to_f32(b);
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
// 5 down, 6 lm_head, 7 argmax, 8 whole kernel.
struct Prof {
  unsigned long long* out;
  unsigned long long last, start;
  bool on;
  __device__ void begin(unsigned long long* p, bool active) {
    out = p;
    on = active && p != nullptr;
    if (on) {
      for (int i = 0; i < 16; i++) out[i] = 0;
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
  // fine-grained accumulators: 9 staging, 10 waiting for weights, 11 row math, 12 grid barrier
  __device__ unsigned long long tic() const { return on ? gtime() : 0ULL; }
  __device__ void toc(int kind, unsigned long long t0) {
    if (on) out[kind] += gtime() - t0;
  }
};

struct GridBar {
  unsigned long long gen;
};

__device__ __forceinline__ void grid_sync(const MegaArgs& a, GridBar& gb, int G, int tid,
                                          const Smem& sm) {
  consumer_sync();
  if (tid == 0) {
    gb.gen += 1;
    const unsigned long long target = gb.gen * (unsigned long long)G;
    __threadfence();  // release this CTA's writes before announcing arrival
    const unsigned long long prev = atomicAdd(a.bar, 1ULL);
    if (prev + 1 < target && !*sm.abort) {
      const volatile unsigned long long* cnt = a.bar;
      long long it = 0;
      while (*cnt < target && ++it < MK_GRID_SPINS) {
      }
      if (*cnt < target) *sm.abort = 2;
    }
    __threadfence();  // acquire the other CTAs' writes
  }
  consumer_sync();
}

// ---- attention for one (head, split) ---------------------------------------------------
__device__ __forceinline__ uint32_t load_kv_bits(const uint8_t* base, int kv_type, int64_t idx) {
  if (kv_type == E_F32) return reinterpret_cast<const uint32_t*>(base)[idx];
  return reinterpret_cast<const uint16_t*>(base)[idx];
}
__device__ __forceinline__ float kv_bits_to_f32(uint32_t b, int kv_type) {
  if (kv_type == E_F32) return __uint_as_float(b);
  return kv_type == E_F16 ? f16_bits_to_f32(b) : bf16_bits_to_f32(b);
}

// DPL = head-dim slots per lane (4 covers d <= 128, 8 covers d <= 256).
template <int DPL>
__device__ __forceinline__ void phase_attention(const MegaArgs& a, int l, const MegaLayer* L, int cta,
                                                int64_t pos, int64_t seq, int nsplit, const Smem& sm,
                                                int tid, int lane, int warp) {
  if (cta >= a.nh * nsplit) return;
  const int h = cta / nsplit, sp = cta - h * nsplit;
  const int grp = a.nh / a.nkv, kvh = h / grp, gi = h - kvh * grp;
  const int d = a.d, half = d / 2;
  float* qs = sm.misc;           // [256]
  float* kn = sm.misc + 256;     // [256]
  float* vn = sm.misc + 512;     // [256]
  float* wm = sm.misc + 768;     // [16]
  float* wl = sm.misc + 784;     // [16]
  float* red = sm.misc + 800;    // [32]
  float* wacc = sm.misc + 1024;  // [16][256]
  for (int i = tid; i < d; i += MK_CT) {
    qs[i] = __ldcg(a.q + (int64_t)h * d + i);
    kn[i] = __ldcg(a.k + (int64_t)kvh * d + i);
    vn[i] = round_kv(__ldcg(a.v + (int64_t)kvh * d + i), a.kv_type);
  }
  consumer_sync();
  float qinv = 1.f, kinv = 1.f;
  if (a.has_norm) {
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < d; i += MK_CT) {
      sq = fmaf(qs[i], qs[i], sq);
      sk = fmaf(kn[i], kn[i], sk);
    }
    sq = consumer_sum(sq, red, lane, warp);
    sk = consumer_sum(sk, red + 16, lane, warp);
    qinv = 1.0f / sqrtf(sq / (float)d + a.eps);
    kinv = 1.0f / sqrtf(sk / (float)d + a.eps);
  }
  uint8_t* kc = a.kcache + (uint64_t)l * a.layer_stride;
  uint8_t* vc = a.vcache + (uint64_t)l * a.layer_stride;
  const int64_t plane = ((seq * a.nkv + kvh) * a.cap) * d;  // element offset of this head's plane
  const bool writer = (sp == 0 && gi == 0);
  for (int i = tid; i < half; i += MK_CT) {
    float q1 = qs[i], q2 = qs[i + half], k1 = kn[i], k2 = kn[i + half];
    if (a.has_norm) {
      const uint8_t* qw = reinterpret_cast<const uint8_t*>(L->q_norm);
      const uint8_t* kw = reinterpret_cast<const uint8_t*>(L->k_norm);
      q1 = __fmul_rn(__fmul_rn(q1, qinv), aux_load(qw, L->qk_norm_type, i));
      q2 = __fmul_rn(__fmul_rn(q2, qinv), aux_load(qw, L->qk_norm_type, i + half));
      k1 = __fmul_rn(__fmul_rn(k1, kinv), aux_load(kw, L->qk_norm_type, i));
      k2 = __fmul_rn(__fmul_rn(k2, kinv), aux_load(kw, L->qk_norm_type, i + half));
    }
    if (a.has_rope) {
      const float angle = __fmul_rn((float)pos, a.ft.f[i]);
      float sv, cv;
      sincosf(angle, &sv, &cv);
      const float ql = __fsub_rn(__fmul_rn(q1, cv), __fmul_rn(q2, sv));
      const float qh = __fadd_rn(__fmul_rn(q1, sv), __fmul_rn(q2, cv));
      const float kl = __fsub_rn(__fmul_rn(k1, cv), __fmul_rn(k2, sv));
      const float kh = __fadd_rn(__fmul_rn(k1, sv), __fmul_rn(k2, cv));
      q1 = ql, q2 = qh, k1 = kl, k2 = kh;
    }
    qs[i] = q1;
    qs[i + half] = q2;
    kn[i] = round_kv(k1, a.kv_type);
    kn[i + half] = round_kv(k2, a.kv_type);
  }
  consumer_sync();
  if (writer) {
    for (int i = tid; i < d; i += MK_CT) {
      store_kv(kc, a.kv_type, plane + pos * d + i, kn[i]);
      store_kv(vc, a.kv_type, plane + pos * d + i, vn[i]);
    }
  }
  const int64_t n = pos + 1;
  const int64_t per = (n + nsplit - 1) / nsplit;
  const int64_t k_lo = (int64_t)sp * per;
  const int64_t k_hi = (k_lo + per < n) ? k_lo + per : n;
  const float scale = 1.0f / sqrtf((float)d);
  float qreg[DPL], acc[DPL];
#pragma unroll
  for (int j = 0; j < DPL; j++) {
    const int idx = lane + 32 * j;
    qreg[j] = idx < d ? qs[idx] : 0.f;
    acc[j] = 0.f;
  }
  float m = -3.40282347e38f, lsum = 0.f;
  // Keys round-robin over warps; the next key's K and V rows are fetched while the
  // current one is reduced, so two rows per warp are in flight.
  uint32_t kb[DPL], vb[DPL], kb2[DPL], vb2[DPL];
  auto fetch = [&](int64_t key, uint32_t* kk, uint32_t* vv) {
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      const int idx = lane + 32 * j;
      if (idx < d && key != pos) {
        kk[j] = load_kv_bits(kc, a.kv_type, plane + key * d + idx);
        vv[j] = load_kv_bits(vc, a.kv_type, plane + key * d + idx);
      } else {
        kk[j] = vv[j] = 0;
      }
    }
  };
  int64_t key = k_lo + warp;
  if (key < k_hi) fetch(key, kb, vb);
  for (; key < k_hi; key += MK_CW) {
    const int64_t nxt = key + MK_CW;
    if (nxt < k_hi) fetch(nxt, kb2, vb2);
    const bool fresh = key == pos;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      const int idx = lane + 32 * j;
      if (idx < d) dot = fmaf(qreg[j], fresh ? kn[idx] : kv_bits_to_f32(kb[j], a.kv_type), dot);
    }
    dot = warp_sum(dot);
    const float sc = dot * scale;
    const float mn = fmaxf(m, sc);
    const float factor = expf(m - mn);
    const float p = expf(sc - mn);
    lsum = lsum * factor + p;
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      const int idx = lane + 32 * j;
      if (idx < d)
        acc[j] = acc[j] * factor + p * (fresh ? vn[idx] : kv_bits_to_f32(vb[j], a.kv_type));
    }
    m = mn;
#pragma unroll
    for (int j = 0; j < DPL; j++) kb[j] = kb2[j], vb[j] = vb2[j];
  }
  if (lane == 0) {
    wm[warp] = m;
    wl[warp] = lsum;
  }
#pragma unroll
  for (int j = 0; j < DPL; j++) {
    const int idx = lane + 32 * j;
    if (idx < d) wacc[warp * 256 + idx] = acc[j];
  }
  consumer_sync();
  float gm = wm[0];
#pragma unroll
  for (int w = 1; w < MK_CW; w++) gm = fmaxf(gm, wm[w]);
  float gl = 0.f;
#pragma unroll
  for (int w = 0; w < MK_CW; w++) gl += wl[w] * expf(wm[w] - gm);
  float* part = a.attn_part + ((int64_t)h * a.max_split + sp) * (d + 2);
  for (int idx = tid; idx < d; idx += MK_CT) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < MK_CW; w++) o += wacc[w * 256 + idx] * expf(wm[w] - gm);
    if (nsplit == 1)
      a.ctx[(int64_t)h * d + idx] = o / gl;
    else
      part[idx] = o;
  }
  if (nsplit > 1 && tid == 0) {
    part[d] = gm;
    part[d + 1] = gl;
  }
}

// ---- the kernel --------------------------------------------------------------------------
__global__ void __launch_bounds__(MK_THREADS, 1) decode_mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, G = gridDim.x;
  __shared__ int s_abort;

  Smem sm;
  sm.nslot = a.nslot;
  sm.xs = reinterpret_cast<float*>(smem_raw);
  sm.misc = sm.xs + a.xs_floats;
  sm.ring = reinterpret_cast<uint8_t*>(sm.misc + MK_MISC_FLOATS);
  sm.full = reinterpret_cast<uint64_t*>(sm.ring + (size_t)a.nslot * MK_SLOT);
  sm.empty = sm.full + a.nslot;
  sm.abort = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < a.nslot; i++) {
      mbar_init(sm.full + i, 1);
      mbar_init(sm.empty + i, MK_CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == MK_CW) {
    // ------------------------------ producer: stream this CTA's weight slices ----------
    if (lane != 0) return;
    uint32_t pi = 0;
    auto issue = [&](const Chunk& c) {
      const int slot = pi % sm.nslot;
      bool ok = true;
      if (pi >= (uint32_t)sm.nslot) {
        const unsigned parity = ((pi / sm.nslot) - 1u) & 1u;
        ok = false;
        for (long long it = 0; it < MK_MBAR_SPINS; it++) {
          if (mbar_try_wait(sm.empty + slot, parity)) {
            ok = true;
            break;
          }
          if (*sm.abort) break;
        }
        if (!ok && !*sm.abort) *sm.abort = 4;
      }
      if (ok && !*sm.abort) {
        uint32_t total = 0;
        for (int i = 0; i < c.ncopy; i++) total += c.bytes[i];
        mbar_expect_tx(sm.full + slot, total);
        uint8_t* base = sm.ring + (size_t)slot * MK_SLOT;
        for (int i = 0; i < c.ncopy; i++) bulk_g2s(base + c.soff[i], c.g[i], c.bytes[i], sm.full + slot);
      }
      pi++;
    };
    for (int l = 0; l < a.layers; l++) {
      const MegaLayer* L = a.L + l;
      enum_phase(a, L, PH_QKV, cta, G, issue);
      enum_phase(a, L, PH_O, cta, G, issue);
      enum_phase(a, L, PH_GATEUP, cta, G, issue);
      enum_phase(a, L, PH_DOWN, cta, G, issue);
    }
    enum_phase(a, a.L, PH_HEAD, cta, G, issue);
    return;
  }

  // -------------------------------- consumers ---------------------------------------------
  GridBar gb;
  gb.gen = 0;
  if (tid == 0) gb.gen = *reinterpret_cast<const volatile unsigned long long*>(a.bar) / (unsigned long long)G;
  const int64_t token = __ldcg(a.io + 0), pos = __ldcg(a.io + 1), seq = __ldcg(a.io + 2);
  int nsplit = (int)((pos + 1) / 32);
  if (nsplit > a.max_split) nsplit = a.max_split;
  if (nsplit < 1) nsplit = 1;
  const int64_t qd = (int64_t)a.nh * a.d;
  uint32_t ci = 0;

  Prof prof;
  prof.begin(a.prof, cta == 0 && tid == 0);
  if (cta == 0) gather_row(a.embed, token, a.hidden, tid);
  { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
  prof.mark(0);

  for (int l = 0; l < a.layers; l++) {
    const MegaLayer* L = a.L + l;
    // ---- norm + q/k/v rows
    { const unsigned long long t_ = prof.tic(); stage_norm(a.hidden, L->attn_norm, L->norm_type, a.H, a.eps, sm, tid, lane, warp); prof.toc(9, t_); }
    enum_phase(a, L, PH_QKV, cta, G, [&](const Chunk& c) {
      const unsigned long long tw_ = prof.tic();
      const bool ok = wait_full(sm, ci);
      prof.toc(10, tw_);
      const unsigned long long tr_ = prof.tic();
      const uint8_t* slot = sm.ring + (size_t)(ci % sm.nslot) * MK_SLOT;
      const WRef& w = c.tag == 0 ? L->q : (c.tag == 1 ? L->k : L->v);
      float* out = c.tag == 0 ? a.q : (c.tag == 1 ? a.k : a.v);
      if (ok)
        for (int j = warp; j < c.n; j += MK_CW) {
          const float v = dot_row(w.enc, chunk_row(w, slot, c, 0, j), w.cols, sm.xs, lane);
          if (lane == 0) out[c.r0 + j] = v;
        }
      prof.toc(11, tr_);
      release_slot(sm, ci, lane);
      ci++;
    });
    { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
    prof.mark(1);
    // ---- qk-norm, RoPE, KV write, attention
    if (!*sm.abort) {
      if (a.d <= 128)
        phase_attention<4>(a, l, L, cta, pos, seq, nsplit, sm, tid, lane, warp);
      else
        phase_attention<8>(a, l, L, cta, pos, seq, nsplit, sm, tid, lane, warp);
    }
    { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
    prof.mark(2);
    // ---- o_proj + residual
    if (nsplit == 1) {
      for (int i = tid; i < qd / 4; i += MK_CT)
        reinterpret_cast<float4*>(sm.xs)[i] = __ldcg(reinterpret_cast<const float4*>(a.ctx) + i);
    } else {
      for (int e = tid; e < qd; e += MK_CT) {
        const int h = e / a.d, i = e - h * a.d;
        const float* p0 = a.attn_part + (int64_t)h * a.max_split * (a.d + 2);
        float gm = -3.40282347e38f;
        for (int s = 0; s < nsplit; s++) gm = fmaxf(gm, __ldcg(p0 + s * (a.d + 2) + a.d));
        float o = 0.f, gl = 0.f;
        for (int s = 0; s < nsplit; s++) {
          const float* ps = p0 + s * (a.d + 2);
          const float wgt = expf(__ldcg(ps + a.d) - gm);
          o += __ldcg(ps + i) * wgt;
          gl += __ldcg(ps + a.d + 1) * wgt;
        }
        sm.xs[e] = o / gl;
      }
    }
    consumer_sync();
    enum_phase(a, L, PH_O, cta, G, [&](const Chunk& c) {
      const unsigned long long tw_ = prof.tic();
      const bool ok = wait_full(sm, ci);
      prof.toc(10, tw_);
      const unsigned long long tr_ = prof.tic();
      const uint8_t* slot = sm.ring + (size_t)(ci % sm.nslot) * MK_SLOT;
      if (ok)
        for (int j = warp; j < c.n; j += MK_CW) {
          const float v = dot_row(L->o.enc, chunk_row(L->o, slot, c, 0, j), L->o.cols, sm.xs, lane);
          if (lane == 0) a.hidden[c.r0 + j] = __ldcg(a.hidden + c.r0 + j) + v;
        }
      prof.toc(11, tr_);
      release_slot(sm, ci, lane);
      ci++;
    });
    { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
    prof.mark(3);
    // ---- norm + gate/up + SwiGLU
    { const unsigned long long t_ = prof.tic(); stage_norm(a.hidden, L->ffn_norm, L->norm_type, a.H, a.eps, sm, tid, lane, warp); prof.toc(9, t_); }
    enum_phase(a, L, PH_GATEUP, cta, G, [&](const Chunk& c) {
      const unsigned long long tw_ = prof.tic();
      const bool ok = wait_full(sm, ci);
      prof.toc(10, tw_);
      const unsigned long long tr_ = prof.tic();
      const uint8_t* slot = sm.ring + (size_t)(ci % sm.nslot) * MK_SLOT;
      const int up_comp = L->gate.enc == E_MLX_U4 ? 3 : 1;
      if (ok)
        for (int j = warp; j < c.n; j += MK_CW) {
          const float g = dot_row(L->gate.enc, chunk_row(L->gate, slot, c, 0, j), L->gate.cols, sm.xs, lane);
          const float u = dot_row(L->up.enc, chunk_row(L->up, slot, c, up_comp, j), L->up.cols, sm.xs, lane);
          if (lane == 0) a.act[c.r0 + j] = (g / (1.0f + expf(-g))) * u;
        }
      prof.toc(11, tr_);
      release_slot(sm, ci, lane);
      ci++;
    });
    { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
    prof.mark(4);
    // ---- down + residual
    for (int i = tid; i < a.I / 4; i += MK_CT)
      reinterpret_cast<float4*>(sm.xs)[i] = __ldcg(reinterpret_cast<const float4*>(a.act) + i);
    consumer_sync();
    enum_phase(a, L, PH_DOWN, cta, G, [&](const Chunk& c) {
      const unsigned long long tw_ = prof.tic();
      const bool ok = wait_full(sm, ci);
      prof.toc(10, tw_);
      const unsigned long long tr_ = prof.tic();
      const uint8_t* slot = sm.ring + (size_t)(ci % sm.nslot) * MK_SLOT;
      if (ok)
        for (int j = warp; j < c.n; j += MK_CW) {
          const float v = dot_row(L->down.enc, chunk_row(L->down, slot, c, 0, j), L->down.cols, sm.xs, lane);
          if (lane == 0) a.hidden[c.r0 + j] = __ldcg(a.hidden + c.r0 + j) + v;
        }
      prof.toc(11, tr_);
      release_slot(sm, ci, lane);
      ci++;
    });
    { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
    prof.mark(5);
  }

  // ---- final norm + lm_head + argmax partials (first strict maximum)
  { const unsigned long long t_ = prof.tic(); stage_norm(a.hidden, a.out_norm, a.out_norm_type, a.H, a.eps, sm, tid, lane, warp); prof.toc(9, t_); }
  float bv = -INFINITY;
  long long bi = 0x7fffffffffffffffLL;
  enum_phase(a, a.L, PH_HEAD, cta, G, [&](const Chunk& c) {
    const unsigned long long tw_ = prof.tic();
      const bool ok = wait_full(sm, ci);
      prof.toc(10, tw_);
      const unsigned long long tr_ = prof.tic();
    const uint8_t* slot = sm.ring + (size_t)(ci % sm.nslot) * MK_SLOT;
    if (ok)
      for (int j = warp; j < c.n; j += MK_CW) {
        const float v = dot_row(a.lm_head.enc, chunk_row(a.lm_head, slot, c, 0, j), a.lm_head.cols, sm.xs, lane);
        const long long row = c.r0 + j;
        if (lane == 0) a.logits[row] = v;
        if (v > -INFINITY && arg_better(v, row, bv, bi)) bv = v, bi = row;
      }
    prof.toc(11, tr_);
    release_slot(sm, ci, lane);
    ci++;
  });
  {
    float* rv = sm.misc;
    long long* ri = reinterpret_cast<long long*>(sm.misc + 64);
    consumer_sync();
    if (lane == 0) {
      rv[warp] = bv;
      ri[warp] = bi;
    }
    consumer_sync();
    if (tid == 0) {
      for (int w = 1; w < MK_CW; w++)
        if (arg_better(rv[w], ri[w], bv, bi)) bv = rv[w], bi = ri[w];
      a.argmax_val[cta] = bv;
      a.argmax_idx[cta] = bi;
    }
  }
  { const unsigned long long t_ = prof.tic(); grid_sync(a, gb, G, tid, sm); prof.toc(12, t_); }
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

size_t mega_smem_bytes(int nslot, int xs_floats) {
  return (size_t)xs_floats * 4 + (size_t)MK_MISC_FLOATS * 4 + (size_t)nslot * MK_SLOT +
         (size_t)nslot * 16 + 128;
}

int mega_plan(int H, int I, int qd, int d, int* nslot, int* xs_floats, size_t* smem) {
  int xs = H > I ? H : I;
  if (qd > xs) xs = qd;
  xs = (xs + 31) / 32 * 32;
  if (d > 256) return 0;
  const size_t budget = 225 * 1024;
  const size_t fixed = (size_t)xs * 4 + (size_t)MK_MISC_FLOATS * 4 + 512;
  if (fixed + 3 * (size_t)MK_SLOT > budget) return 0;
  int n = (int)((budget - fixed) / (MK_SLOT + 16));
  if (n > 12) n = 12;
  *nslot = n;
  *xs_floats = xs;
  *smem = mega_smem_bytes(n, xs);
  return 1;
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
