// Persistent decode kernel: one launch decodes one or several consecutive tokens of one sequence.
//
// One CTA per SM, launched cooperatively so that all CTAs are co-resident. Each CTA owns a fixed,
// balanced slice of the rows of every weight matrix, cut into tiles of 16 rows (x K-slices). A
// producer warp streams the tiles -- the verbatim checkpoint bytes, one 1-D bulk async copy per
// row segment (cp.async.bulk + mbarrier transaction counts) -- from HBM into a shared-memory
// ring, running as far ahead of the math as the ring allows: weight traffic never waits for the
// activation dependency chain. Rows land PITCH bytes apart with PITCH/4 = 4 (mod 8), so the
// tensor-core fragment loads are bank-conflict free. Eight consumer warps split each tile's K
// range and run the tile steps of gemv_core.cuh against the activation vector staged in shared
// memory in fragment order.
//
// The step is a chain of dependent phases, and what bounds it is the hand-off between them, not
// bandwidth. Three rules keep a hand-off near one L2 round trip:
//
//   * Vectors travel between CTAs as (value, epoch) pairs of 8 bytes. A producer stores a pair
//     with one store; a consumer polls the pairs themselves until they carry the epoch of this
//     token and layer. Arrival and data are the same round trip: there is no grid barrier and no
//     second load after a flag. Every vector has its own buffer; a buffer is rewritten a full
//     layer later, by which time every reader has passed (each CTA needs all of a phase's outputs
//     before it can produce the next phase's).
//   * A phase's tiles keep their sums in registers ("round": at most MEGA_TA tiles); the eight
//     K-slice partials of a round meet in shared memory once, behind one block barrier, and the
//     first warps finish them (scale, residual / SwiGLU / logits) and store the pairs.
//   * Nothing but the activation vector is fetched on the critical path: norm weights are
//     requested before the poll begins, the cached keys and values of earlier positions are
//     copied into shared memory a layer ahead, and the residual rows a CTA owns stay in its
//     shared memory for the whole token.
//   * Code that runs once per layer is kept small: on this GPU a warp executes straight-line
//     code at about one instruction per cycle while it fits 8 KB, one per 2.7 cycles up to 32 KB
//     and one per 6 cycles beyond (measured), whatever the arithmetic. The 4 * layers + 1 products
//     therefore share ONE copy of the product code (a loop), attention uses rolled loops, and
//     the timers exist only in a twin kernel.
//
//   per layer: norm+QKV | qk-norm+RoPE+KV-write+attention | o_proj+res | norm+gate/up+SwiGLU |
//   down+res ; then: norm+lm_head+argmax partials | argmax
//
// Every wait (mbarrier, pair poll) is bounded: when it gives up it raises the error word, the
// CTA stops waiting for the rest of the launch (it still stores its pairs, so no other CTA is
// held up by it) and the kernel ends; the host fails the call.
#include <algorithm>

#include "codec.cuh"
#include "decode_mega.cuh"
#include "gemv_core.cuh"
#include "ring.cuh"

namespace dyn {

namespace {

#ifndef MK_OPT_CW
#define MK_OPT_CW 8
#endif
constexpr int MK_CW = MK_OPT_CW;   // consumer warps (a power of two)
constexpr int MK_CT = MK_CW * 32;  // consumer threads
// Eight consumer warps and one producer warp: nine warps leave 168 registers per thread (sixteen
// consumers plus a producer would leave 96 and spill; measured alternatives -- 4 or 16 consumers,
// consumers taking turns as producer -- were slower). MK_OPT_LOCAL = 0 forces whole-block staging.
#ifndef MK_OPT_LOCAL
#define MK_OPT_LOCAL 1
#endif
constexpr int MK_THREADS = MK_CT + 32;
constexpr int MK_SLOT = 18432;          // bytes per ring slot (one 16-row tile x K-slice)
constexpr int MK_PART = MEGA_TA * MK_CW * 16;  // floats of one partial-sum buffer
// per-CTA scratch, in floats
constexpr int MK_OFF_PART = 0;                       // 2 x MK_PART
constexpr int MK_OFF_QS = 2 * MK_PART;               // [128] q of this CTA's head
constexpr int MK_OFF_KN = MK_OFF_QS + 128;           // [128] new key (as cached)
constexpr int MK_OFF_VN = MK_OFF_KN + 128;           // [128] new value (as cached)
constexpr int MK_OFF_WM = MK_OFF_VN + 128;           // [16] per-warp running max
constexpr int MK_OFF_WL = MK_OFF_WM + 16;            // [16] per-warp running sum
constexpr int MK_OFF_RED = MK_OFF_WL + 16;           // [64] block reductions; [32, 64): per-warp sums of squares of two phases
constexpr int MK_OFF_WACC = MK_OFF_RED + 64;         // [16][128] per-warp weighted values
constexpr int MK_OFF_ROPE = MK_OFF_WACC + 16 * 128;  // cos[64], sin[64] of this token's position
constexpr int MK_OFF_RES = MK_OFF_ROPE + 128;        // [64] residual rows this CTA owns
constexpr int MK_OFF_AMAX = MK_OFF_RES + 64;         // [2 x 128] argmax candidates
constexpr int MK_OFF_KVK = MK_OFF_AMAX + 256;        // 16 KB: the first batch of cached keys of this CTA's (head, split)
constexpr int MK_OFF_KVV = MK_OFF_KVK + 4096;        // 16 KB: and of cached values
constexpr int MK_MISC_FLOATS = MK_OFF_KVV + 4096;
constexpr int MK_KV_STAGE_BYTES = 16384;             // 64 rows of 128 two-byte elements, or 32 rows of f32
constexpr int MK_MAX_OWNED = 64;  // hidden rows per CTA
constexpr long long MK_MBAR_SPINS = 1LL << 22;
constexpr long long MK_LL_SPINS = 1LL << 21;  // x ~0.5 us per poll round

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(MK_CT) : "memory"); }

// ---- (value, epoch) pairs ----------------------------------------------------------------------
__device__ __forceinline__ void ll_store(float* buf, int64_t idx, float v, unsigned ep) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(buf + 2 * idx), "r"(__float_as_uint(v)), "r"(ep)
               : "memory");
}
// The 16-byte line that holds pairs idx and idx + 1 (idx even).
__device__ __forceinline__ uint4 ll_load(const float* buf, int64_t idx) {
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(buf + 2 * idx)
               : "memory");
  return r;
}
// Polls NL lines until all carry `ep`. v[2i], v[2i+1] = the two values of line i. Gives up when the
// CTA has already given up elsewhere or after MK_LL_SPINS rounds (then *abort = 8).
template <int NL>
__device__ __forceinline__ void ll_poll(const float* buf, const int64_t (&idx)[NL], unsigned ep, float (&v)[2 * NL],
                                        volatile int* abort) {
  uint4 r[NL];
  long long it = 0;
  for (;;) {
    bool ok = true;
#pragma unroll
    for (int i = 0; i < NL; i++) r[i] = ll_load(buf, idx[i]);
#pragma unroll
    for (int i = 0; i < NL; i++) ok = ok && r[i].y == ep && r[i].w == ep;
    if (ok) break;
    if (*abort) break;
    if (++it >= MK_LL_SPINS) {
      *abort = 8;
      break;
    }
  }
#pragma unroll
  for (int i = 0; i < NL; i++) {
    v[2 * i] = __uint_as_float(r[i].x);
    v[2 * i + 1] = __uint_as_float(r[i].z);
  }
}

// Ask L2 for a line that will be read later (norm vectors and cached keys / values of the NEXT
// layer: the weight stream pushes everything a token wrote out of L2 before the next token reads it,
// and a miss on the dependency chain costs a DRAM round trip).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_span(const void* p, size_t bytes, int tid, int nthreads) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(p);
  for (size_t off = (size_t)tid * 128; off < bytes; off += (size_t)nthreads * 128) prefetch_l2(b + off);
}

struct Smem {
  float* xs;      // activation vector, f32
  __half* xf;     // same, hi/lo f16 fragments
  float* sx32;    // per-32 sums of the scaled activation
  float* sx16;    // per-16 sums
  float* isx;     // per 32-block: 2^24 / the power-of-two scale its activations were staged with
  float* misc;
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* prog_bar;  // program copy landed
  const MegaChunk* chunks;
  const MegaTile* tiles;
  const MegaRound* rounds;
  const uint16_t* phase_rounds;
  const MegaLayerHot* hot;
  volatile int* abort;
  uint32_t nchunks;  // chunks of one token's program
  int nslot;
};

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

// ---- producer: one bulk copy per tile row (lanes 0..15), MLX aux rows by lanes 16..31 --------
// slot / lap: ring position of the chunk and how many times the ring has gone round before it.
__device__ __forceinline__ void produce_chunk(const MegaChunk* c, const Smem& sm, int slot, uint32_t lap, int lane) {
  if (lap > 0) {
    int ok = 1;
    if (lane == 0) {
      ok = mbar_wait_bounded(sm.empty + slot, (lap - 1u) & 1u, MK_MBAR_SPINS, sm.abort) ? 1 : 0;
      if (!ok && !*sm.abort) *sm.abort = 4;
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return;
  }
  uint8_t* base = sm.ring + (size_t)slot * MK_SLOT;
  if (c->contig) {
    // the tile's rows follow each other in memory: one copy, rows rb bytes apart in the slot
    if (lane == 0) {
      mbar_expect_tx(sm.full + slot, c->contig);
      bulk_g2s(base, c->src - c->al, c->contig, sm.full + slot);
    }
    return;
  }
  // the byte count of all copies is known on the host (tx): no reduction over the lanes
  if (lane == 0) mbar_expect_tx(sm.full + slot, c->tx);
  __syncwarp();
  const int i = lane & 15;
  if (i >= (int)c->n) return;
  if (lane < 16) {
    const uint32_t off = ((uint32_t)c->al + (uint32_t)i * c->al_step) & 15u;
    const uint8_t* row = c->src + (size_t)i * c->rb + (i >= 8 ? (int64_t)c->jump16 * 16 : 0);
    bulk_g2s(base + i * c->pitch, row - off, (off + c->seg + 15u) & ~15u, sm.full + slot);
  } else if (c->aseg) {
    // scales and biases share their alignment (both tensors start 256-byte aligned in the arena)
    const uint32_t off = ((uint32_t)c->aal + (uint32_t)i * c->aal_step) & 15u;
    const uint32_t nb = (off + c->aseg + 15u) & ~15u;
    uint8_t* d = base + 16 * c->pitch + i * c->apitch;
    bulk_g2s(d, c->sc + (size_t)i * c->arb - off, nb, sm.full + slot);
    bulk_g2s(d + 16 * c->apitch, c->bi + (size_t)i * c->arb - off, nb, sm.full + slot);
  }
}

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Timing seen by CTA 0, thread 0 (optional). By phase: 0 embed, 1 qkv, 2 attention, 3 o_proj,
// 4 gate/up, 5 down, 6 lm_head, 7 argmax, 8 whole kernel. Across phases: 9 staging (poll +
// conversion), 10 waiting for weights, 11 tile math, 12 round reduction + epilogue; attention of
// CTA 0: 13 until q/k/v are in place, 14 scores and softmax, 15 merge and write; staging split: 16 until
// the vector has arrived, 17 reduction + conversion.
// INSTR = false compiles every method to nothing: the kernel that serves requests carries no timer
// code (the instrumented twin is launched when a profile or a trace was asked for).
template <bool INSTR>
struct ProfT {
  unsigned long long* out;
  unsigned long long* trace;  // this CTA's [layers + 1][16] stamps (thread 0), or nullptr
  int layer;
  unsigned long long last, start;
  bool on;
  __device__ void stamp(int id) {
    if constexpr (!INSTR) return;
#ifdef MK_DEBUG_ATT_STAMPS
    if (id >= 9 && id <= 13) return;
#endif
    if (trace) trace[layer * 16 + id] = gtime();
  }
  __device__ void stamp_dbg(int id) {
    if constexpr (!INSTR) return;
#ifdef MK_DEBUG_ATT_STAMPS
    if (trace) trace[layer * 16 + id] = gtime();
#endif
  }
  __device__ void begin(unsigned long long* p, bool active) {
    if constexpr (!INSTR) return;
    out = p;
    on = active && p != nullptr;
    if (on) {
      for (int i = 0; i < 24; i++) out[i] = 0;
      last = start = gtime();
    }
  }
  __device__ void mark(int kind) {
    if constexpr (!INSTR) return;
    if (on) {
      const unsigned long long t = gtime();
      out[kind] += t - last;
      last = t;
    }
  }
  __device__ void end() {
    if constexpr (!INSTR) return;
    if (on) out[8] = gtime() - start;
  }
  __device__ unsigned long long tic() const {
    if constexpr (!INSTR) return 0ULL;
    return on ? gtime() : 0ULL;
  }
  __device__ void toc(int kind, unsigned long long t0) {
    if constexpr (!INSTR) return;
    if (on) out[kind] += gtime() - t0;
  }
};

// ---- staging the activation vector of a phase ---------------------------------------------------
// Item i = (block kb = i / 4, lane quarter t = i % 4) holds 8 elements of the vector: A = 4
// elements at baseA, B = 4 elements at baseB (the items partition the vector). An item's elements
// come from polled pairs, from the split-KV partials, or from xs (the embedding row).
//
// Two ways of staging:
//   * per warp (stage_local): a warp stages exactly the 32-blocks its own K-slice of the phase's
//     tiles reads, each block with a power-of-two scale of its own (the tile steps multiply the
//     block's contribution by 2^24 / scale, isx[kb]), and goes straight on to its tile steps: no
//     block barrier between the arrival of the vector and the math, and a warp whose slice has
//     arrived does not wait for the others. RMSNorm is split: the weights are applied here, the
//     factor 1/sqrt(mean(x^2)+eps) -- a scalar, the product is linear in it -- is applied to the
//     finished sums; each warp leaves its sum of squares in `red` for the finishing threads.
//   * whole block (stage_phase): one scale for the vector, RMSNorm applied here; for encodings whose
//     units share 32-blocks between warps (Q6_K quarters) and for phases of mixed encodings.
enum { SRC_XS = 0, SRC_LL = 1, SRC_PARTIALS = 2 };

struct StageSrc {
  int kind;
  const float* ll;  // SRC_LL: the pair buffer; SRC_PARTIALS: a.ll_part
  unsigned ep;
  int nsplit, max_split, d;  // SRC_PARTIALS
};

__device__ __forceinline__ void item_bases(int layout, int kb, int t, int* baseA, int* baseB) {
  *baseA = kb * 32 + (layout == XL_MLXW ? 8 * t : 4 * t);
  *baseB = layout == XL_MLXW ? *baseA + 4 : kb * 32 + 16 + 4 * t;
}

// The 8 elements of one item.
__device__ __forceinline__ void item_fetch(const StageSrc& src, int baseA, int baseB, const Smem& sm, float (&v)[8]) {
  if (src.kind == SRC_LL) {
    const int64_t idx[4] = {baseA, baseA + 2, baseB, baseB + 2};
    ll_poll<4>(src.ll, idx, src.ep, v, sm.abort);
  } else if (src.kind == SRC_PARTIALS) {
    // merge the split-KV partial outputs of this item's head in split order (online softmax merge)
    const int head = baseA / src.d, ia = baseA - head * src.d, ib = baseB - head * src.d;
    float M = -3.40282347e38f, Lsum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = 0.f;
    for (int s = 0; s < src.nsplit; s++) {
      const int64_t pb = ((int64_t)head * src.max_split + s) * (src.d + 4);
      const int64_t idx[5] = {pb + ia, pb + ia + 2, pb + ib, pb + ib + 2, pb + src.d};
      float p[10];
      ll_poll<5>(src.ll, idx, src.ep, p, sm.abort);
      const float ms = p[8], ls = p[9];
      const float mn = fmaxf(M, ms);
      const float f = expf(M - mn), wgt = expf(ms - mn);
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] = v[j] * f + p[j] * wgt;
      Lsum = Lsum * f + ls * wgt;
      M = mn;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = v[j] / Lsum;
  } else {
    const float4 a4 = *reinterpret_cast<const float4*>(sm.xs + baseA);
    const float4 b4 = *reinterpret_cast<const float4*>(sm.xs + baseB);
    v[0] = a4.x, v[1] = a4.y, v[2] = a4.z, v[3] = a4.w;
    v[4] = b4.x, v[5] = b4.y, v[6] = b4.z, v[7] = b4.w;
  }
}

// Writes one item's hi/lo f16 fragments from its 8 scaled values sv and returns its share of the
// block's two 16-element runs.
__device__ __forceinline__ void item_store(const float (&sv)[8], int layout, int kb, int t, const Smem& sm, float* run0,
                                           float* run1) {
  const float sa = (sv[0] + sv[1]) + (sv[2] + sv[3]), sb = (sv[4] + sv[5]) + (sv[6] + sv[7]);
  float f[8];  // fragment order
  if (layout == XL_NIBBLE) {
    f[0] = sv[0], f[1] = sv[2], f[2] = sv[4] * 0.0625f, f[3] = sv[6] * 0.0625f;
    f[4] = sv[1], f[5] = sv[3], f[6] = sv[5] * 0.0625f, f[7] = sv[7] * 0.0625f;
    *run0 = sa, *run1 = sb;
  } else if (layout == XL_MLXW) {
    f[0] = sv[0], f[1] = sv[4], f[2] = sv[1] * 0.0625f, f[3] = sv[5] * 0.0625f;
    f[4] = sv[2], f[5] = sv[6], f[6] = sv[3] * 0.0625f, f[7] = sv[7] * 0.0625f;
    if (t < 2) *run0 = sa + sb, *run1 = 0.f; else *run0 = 0.f, *run1 = sa + sb;
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = sv[j];
    *run0 = sa, *run1 = sb;
  }
  __half hi[8], lo[8];  // 16-bit storage: f16, or bf16 bit patterns for the plain-bf16 layout
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if (layout == XL_BF16N) {
      const __nv_bfloat16 h = __float2bfloat16_rn(f[j]);
      const __nv_bfloat16 l = __float2bfloat16_rn(f[j] - __bfloat162float(h));
      hi[j] = __ushort_as_half(__bfloat16_as_ushort(h));
      lo[j] = __ushort_as_half(__bfloat16_as_ushort(l));
    } else {
      const __half h = __float2half_rn(f[j]);
      hi[j] = h;
      lo[j] = __float2half_rn(f[j] - __half2float(h));
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(sm.xf + ((size_t)(kb * 2) * 4 + t) * 8);
  dst[0] = *reinterpret_cast<uint4*>(hi);
  dst[4] = *reinterpret_cast<uint4*>(lo);
}

// Per-warp staging. ukb: 32-blocks per unit of the phase's encoding; the warp owns the units
// U = warp, warp + 16, ... of the K range (n / 32 blocks), as its tile steps do. `ssq` receives the
// warp's sum of squares of the raw vector elements it staged.
__device__ __forceinline__ void stage_local(const StageSrc& src, const void* nw, int nw_type, int n, int ukb,
                                            int layout, const Smem& sm, float* ssq, int lane, int warp) {
  const int units = (n >> 5) / ukb;                      // units over the whole K range
  const int mine = units > warp ? (units - warp + MK_CW - 1) / MK_CW : 0;  // units of this warp
  const int ipu = 4 * ukb;                               // items per unit
  float ss = 0.f;
  for (int i0 = 0; i0 < mine * ipu; i0 += 32) {          // whole warps enter, for the shuffles below
    const int i = i0 + lane;
    const bool live = i < mine * ipu;
    const int j = i / ipu, r = i - j * ipu;
    const int kb = (warp + MK_CW * j) * ukb + (r >> 2), t = r & 3;
    int baseA, baseB;
    item_bases(layout, kb, t, &baseA, &baseB);
    float run0 = 0.f, run1 = 0.f, mx = 0.f;
    float v[8];
    if (live) {
      // norm weights first: their loads are in flight while the pairs are polled
      float w[8];
#pragma unroll
      for (int q = 0; q < 8; q++)
        w[q] = nw ? aux_load(reinterpret_cast<const uint8_t*>(nw), nw_type, (q < 4 ? baseA : baseB - 4) + q) : 1.0f;
      item_fetch(src, baseA, baseB, sm, v);
#pragma unroll
      for (int q = 0; q < 8; q++) {
        ss = fmaf(v[q], v[q], ss);
        v[q] = __fmul_rn(v[q], w[q]);
        mx = fmaxf(mx, fabsf(v[q]));
      }
    }
    // the block's own scale: its four items are four consecutive lanes
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float s, is;
    scale_for(mx * 1.0001f, &s, &is);
    if (live) {
      float sv[8];
#pragma unroll
      for (int q = 0; q < 8; q++) sv[q] = v[q] * s;
      item_store(sv, layout, kb, t, sm, &run0, &run1);
    }
    run0 += __shfl_xor_sync(0xffffffffu, run0, 1);
    run1 += __shfl_xor_sync(0xffffffffu, run1, 1);
    run0 += __shfl_xor_sync(0xffffffffu, run0, 2);
    run1 += __shfl_xor_sync(0xffffffffu, run1, 2);
    if (live && t == 0) {
      sm.sx16[2 * kb] = run0;
      sm.sx16[2 * kb + 1] = run1;
      sm.sx32[kb] = run0 + run1;
      sm.isx[kb] = GV_2P24 * is;
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) *ssq = ss;
  __syncwarp();
}

// Whole-block staging: pass 1 brings each item's elements in, stores them to xs and accumulates
// the sum of squares and the largest magnitude; one block reduction gives the RMSNorm factor and
// the power-of-two scale; pass 2 writes the fragments and sums.
__device__ __forceinline__ void stage_phase(const StageSrc& src, const void* nw, int nw_type, int n, float eps,
                                            int layout, const Smem& sm, int tid, int lane, int warp) {
  float* red = sm.misc + MK_OFF_RED;
  const int items = n >> 3;
  float ss = 0.f, mx = 0.f;
  for (int i = tid; i < items; i += MK_CT) {
    const int kb = i >> 2, t = i & 3;
    int baseA, baseB;
    item_bases(layout, kb, t, &baseA, &baseB);
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
      w[j] = nw ? aux_load(reinterpret_cast<const uint8_t*>(nw), nw_type, (j < 4 ? baseA : baseB - 4) + j) : 1.0f;
    float v[8];
    item_fetch(src, baseA, baseB, sm, v);
    if (src.kind != SRC_XS) {
      *reinterpret_cast<float4*>(sm.xs + baseA) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(sm.xs + baseB) = make_float4(v[4], v[5], v[6], v[7]);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      ss = fmaf(v[j], v[j], ss);
      mx = fmaxf(mx, fabsf(v[j] * w[j]));
    }
  }
  ss = warp_sum(ss);
  mx = warp_max(mx);
  consumer_sync();  // red is free (earlier readers are past their last use)
  if (lane == 0) {
    red[warp] = ss;
    red[16 + warp] = mx;
  }
  consumer_sync();
  float tss = 0.f, tmx = 0.f;
#pragma unroll
  for (int i = 0; i < MK_CW; i++) {
    tss += red[i];
    tmx = fmaxf(tmx, red[16 + i]);
  }
  const float inv = nw ? 1.0f / sqrtf(tss / (float)n + eps) : 1.0f;
  float s, is;
  scale_for(tmx * inv * 1.0001f, &s, &is);
  for (int iw = warp * 32; iw < items; iw += MK_CT) {  // whole warps enter, for the shuffles below
    const int i = iw + lane;
    const bool live = i < items;
    const int kb = i >> 2, t = i & 3;
    int baseA, baseB;
    item_bases(layout, kb, t, &baseA, &baseB);
    float run0 = 0.f, run1 = 0.f;
    if (live) {
      const float4 a4 = *reinterpret_cast<const float4*>(sm.xs + baseA);  // written by this thread
      const float4 b4 = *reinterpret_cast<const float4*>(sm.xs + baseB);
      const float v[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
      float sv[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float wj = nw ? aux_load(reinterpret_cast<const uint8_t*>(nw), nw_type, (j < 4 ? baseA : baseB - 4) + j) : 1.0f;
        sv[j] = (nw ? __fmul_rn(__fmul_rn(v[j], inv), wj) : v[j]) * s;
      }
      item_store(sv, layout, kb, t, sm, &run0, &run1);
    }
    run0 += __shfl_xor_sync(0xffffffffu, run0, 1);
    run1 += __shfl_xor_sync(0xffffffffu, run1, 1);
    run0 += __shfl_xor_sync(0xffffffffu, run0, 2);
    run1 += __shfl_xor_sync(0xffffffffu, run1, 2);
    if (live && t == 0) {
      sm.sx16[2 * kb] = run0;
      sm.sx16[2 * kb + 1] = run1;
      sm.sx32[kb] = run0 + run1;
      sm.isx[kb] = GV_2P24 * is;
    }
  }
  consumer_sync();
}

// One unit of a chunk for this warp. p0 / p1: the chunk's bytes in rows g, g+8; a0 / a1: MLX
// scales of those rows (biases 16 * apitch further).
template <int ENC>
__device__ __forceinline__ void run_unit_t(int aux, int group_shift, const uint8_t* p0, const uint8_t* p1,
                                           const uint8_t* a0, const uint8_t* a1, int apitch16, int u, int kb0,
                                           const Smem& sm, int lane, TileAcc<true>& acc) {
  const int t = lane & 3;
  const int c = (lane >> 2) & 1;
  const __half* xf0 = sm.xf + (size_t)c * 32 + t * 8;  // block kb adds kb * 64 halfs
  if (ENC == E_Q4_0) {
    const int kb = kb0 + 2 * u;
    blk_q4<E_Q4_0, 0, true>(p0 + u * 36, p1 + u * 36, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc, sm.isx[kb]);
    blk_q4<E_Q4_0, 2, true>(p0 + u * 36 + 18, p1 + u * 36 + 18, xf0 + (size_t)(kb + 1) * 64,
                            sm.sx32[kb + 1], 0.f, t, acc, sm.isx[kb + 1]);
  } else if (ENC == E_Q4_1) {
    const int kb = kb0 + u;
    blk_q4<E_Q4_1, 0, true>(p0 + u * 20, p1 + u * 20, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc, sm.isx[kb]);
  } else if (ENC == E_Q8_0) {
    const int kb = kb0 + 2 * u;
    blk_q8_0<0, true>(p0 + u * 68, p1 + u * 68, xf0 + (size_t)kb * 64, sm.sx32[kb], 0.f, t, acc, sm.isx[kb]);
    blk_q8_0<2, true>(p0 + u * 68 + 34, p1 + u * 68 + 34, xf0 + (size_t)(kb + 1) * 64, sm.sx32[kb + 1],
                      0.f, t, acc, sm.isx[kb + 1]);
  } else if (ENC == E_BF16 || ENC == E_F16) {
    // a unit is one block of 32 plain weights; the activations carry the block's own power-of-two
    // scale (isx = 2^24 / scale), the weights are true values
    const int kb = kb0 + u;
    blk_plain16<ENC == E_BF16, true>(p0 + u * 64, p1 + u * 64, xf0 + (size_t)kb * 64, t, acc, sm.isx[kb] * GV_2M24);
  } else if (ENC == E_MLX_U4) {
    // a unit is two 32-blocks (32 bytes per row); with groups of 64 or 128 they share scale and bias
    const int kb = kb0 + 2 * u;
    const int gi = (2 * u) >> group_shift, gj = (2 * u + 1) >> group_shift;
    const float s0 = aux_load(a0, aux, gi), s1 = aux_load(a1, aux, gi);
    const float b0 = aux_load(a0 + apitch16, aux, gi), b1 = aux_load(a1 + apitch16, aux, gi);
    const float bs = sm.isx[kb], bt = sm.isx[kb + 1];
    blk_mlx<true>(p0 + u * 32, p1 + u * 32, s0 * bs, s1 * bs, b0 * bs, b1 * bs, xf0 + (size_t)kb * 64, sm.sx32[kb],
                  0.f, t, acc);
    if (gj == gi) {
      blk_mlx<true>(p0 + u * 32 + 16, p1 + u * 32 + 16, s0 * bt, s1 * bt, b0 * bt, b1 * bt,
                    xf0 + (size_t)(kb + 1) * 64, sm.sx32[kb + 1], 0.f, t, acc);
    } else {
      blk_mlx<true>(p0 + u * 32 + 16, p1 + u * 32 + 16, aux_load(a0, aux, gj) * bt, aux_load(a1, aux, gj) * bt,
                    aux_load(a0 + apitch16, aux, gj) * bt, aux_load(a1 + apitch16, aux, gj) * bt,
                    xf0 + (size_t)(kb + 1) * 64, sm.sx32[kb + 1], 0.f, t, acc);
    }
  } else {
    // Q6_K quarter: superblock u / 4 of the chunk, half n, sub-block s
    const int sb = u >> 2, n = (u >> 1) & 1, s = u & 1;
    const int kb = kb0 + sb * 8;
    const uint8_t* s0 = p0 + sb * 210;
    const uint8_t* s1 = p1 + sb * 210;
    // the quarter spans four 32-blocks: Q6_K phases stage the whole vector with one scale
    const float bs = sm.isx[kb];
    if (sb & 1)
      q6k_quarter<2, true>(s0, s1, n, s, xf0 + (size_t)kb * 64, 64, sm.sx16 + 2 * kb, sm.sx16 + 2 * kb, t, acc, bs);
    else
      q6k_quarter<0, true>(s0, s1, n, s, xf0 + (size_t)kb * 64, 64, sm.sx16 + 2 * kb, sm.sx16 + 2 * kb, t, acc, bs);
  }
}
// ENC < 0: the chunk says which encoding it holds (phases whose tensors differ).
template <int ENC>
__device__ __forceinline__ void run_unit(int enc, int aux, int group_shift, const uint8_t* p0, const uint8_t* p1,
                                         const uint8_t* a0, const uint8_t* a1, int apitch16, int u, int kb0,
                                         const Smem& sm, int lane, TileAcc<true>& acc) {
  if (ENC >= 0) {
    run_unit_t<ENC < 0 ? E_Q4_0 : ENC>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc);
    return;
  }
  switch (enc) {
    case E_Q4_0: run_unit_t<E_Q4_0>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    case E_Q4_1: run_unit_t<E_Q4_1>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    case E_Q8_0: run_unit_t<E_Q8_0>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    case E_MLX_U4: run_unit_t<E_MLX_U4>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    case E_BF16: run_unit_t<E_BF16>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    case E_F16: run_unit_t<E_F16>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
    default: run_unit_t<E_Q6_K>(aux, group_shift, p0, p1, a0, a1, apitch16, u, kb0, sm, lane, acc); break;
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

// ---- attention for one (head, split); head dim 64 or 128, a lane owns 4 head dims ----------------
// Latency plan: the cached keys and values of earlier positions and the norm weights are requested
// first; then warps 0 / 1 / 2 poll this token's q / k / v of the head (one or two lines per lane),
// normalise and rotate them inside the warp (no block reduction) and leave them in shared memory.
// The cached rows [k_lo, min(k_hi, pos)) of this CTA's (head, split) in layer l are one run per pool.
// Its first batch (64 rows of a 2-byte cache, 32 of an f32 cache) is copied into shared memory with
// 16-byte asynchronous copies a layer ahead: a load issued when attention begins would queue behind
// the weight copies that refill the ring at that moment (measured: ~1 us until the rows arrived).
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Byte offset of byte `b` of staged row `row`: 16-byte pieces of odd rows of a 2-byte cache are
// exchanged in groups of four (piece ^ 4), which makes the score loop's 16-byte reads (two rows per
// quarter warp, four threads per row) free of bank conflicts. Rows of an f32 cache need no exchange.
__device__ __forceinline__ int kv_stage_off(int row, int b, int rowbytes, bool wide) {
  const int piece = (b >> 4) ^ ((!wide && (row & 1)) ? 4 : 0);
  return row * rowbytes + (piece << 4) + (b & 15);
}

// Where this CTA's (head, split) sits for the token being decoded: worked out once per token (the
// divisions are not cheap and this code is cold every time it runs), used by every layer.
struct AttGeo {
  int h;             // head; >= the number of heads when this CTA has no (head, split)
  int sp, kvh, gi;
  int k_lo, k_hi;    // keys [k_lo, k_hi) of positions 0 .. pos
  size_t plane_bytes;  // byte offset of (sequence, kv head, position 0) inside a layer of the pool
};
__device__ __forceinline__ AttGeo att_geometry(const MegaArgs& a, int cta, int pos, int seq, int nsplit) {
  AttGeo g;
  g.h = cta / nsplit, g.sp = cta - g.h * nsplit;
  const int grp = a.nh / a.nkv;
  g.kvh = g.h / grp, g.gi = g.h - g.kvh * grp;
  const int n = pos + 1, per = (n + nsplit - 1) / nsplit;
  g.k_lo = g.sp * per;
  g.k_hi = g.k_lo + per < n ? g.k_lo + per : n;
  const int rshift = 31 - __clz(a.d * (a.kv_type == E_F32 ? 4 : 2));  // rows are 128, 256 or 512 bytes
  g.plane_bytes = ((size_t)((int64_t)seq * a.nkv + g.kvh) * (size_t)a.cap) << rshift;
  return g;
}

// Copies the cached rows [k_first, k_first + batch) of this CTA's (head, split) that exist already
// (positions below pos) from layer l of the pool into the staging buffers: asynchronous, one
// commit group.
__device__ __forceinline__ void stage_kv(const MegaArgs& a, const AttGeo& g, int l, int pos, const Smem& sm, int tid,
                                         int batch_index = 0) {
  if (g.h >= a.nh || l >= a.layers) return;
  const bool wide = a.kv_type == E_F32;
  const int rowbytes = a.d * (wide ? 4 : 2), rshift = 31 - __clz(rowbytes);
  const int k_first = g.k_lo + batch_index * (wide ? 32 : 64);
  const int k_end = g.k_hi < pos ? g.k_hi : pos;
  if (k_end <= k_first) return;
  int bytes = (k_end - k_first) << rshift;  // a multiple of 128
  if (bytes > MK_KV_STAGE_BYTES) bytes = MK_KV_STAGE_BYTES;
  const size_t start = (size_t)l * a.layer_stride + g.plane_bytes + ((size_t)k_first << rshift);
  const uint8_t* ksrc = a.kcache + start;
  const uint8_t* vsrc = a.vcache + start;
  uint8_t* kdst = reinterpret_cast<uint8_t*>(sm.misc + MK_OFF_KVK);
  uint8_t* vdst = reinterpret_cast<uint8_t*>(sm.misc + MK_OFF_KVV);
  for (int off = tid * 16; off < bytes; off += MK_CT * 16) {
    const int row = off >> rshift;
    const int o = kv_stage_off(row, off - (row << rshift), rowbytes, wide);
    cp_async16(kdst + o, ksrc + off);
    cp_async16(vdst + o, vsrc + off);
  }
  cp_async_commit();
}

// Attention of one (head, split) over the keys [k_lo, k_hi), in batches of 64 (32 for an f32 cache)
// staged in shared memory. The code is deliberately compact (rolled loops, no per-key unrolling): it
// runs once per layer, and instructions that are not in the instruction cache cost more than the
// arithmetic they encode.
//   scores : thread (key = tid / TPK, part = tid % TPK) multiplies q with 16-byte pieces part,
//            part + TPK, ... of its key's row; TPK lanes add up by shuffle
//   softmax: batch maximum and sum through shared memory (two block barriers), running maximum and
//            sum across batches
//   values : thread (pair = tid % (d/2), group = tid / (d/2)) accumulates two head dims over the
//            keys of its group; groups are added in a fixed order at the end
template <int KVT, class Prof>
__device__ __forceinline__ void phase_attention_t(const MegaArgs& a, int l, const MegaLayerHot* L, const AttGeo& G,
                                                int64_t pos, int nsplit, unsigned ep, const Smem& sm, int tid,
                                                int lane, int warp, Prof& prof) {
  if (G.h >= a.nh) return;
  constexpr bool WIDE = KVT == E_F32;
  constexpr int EL = WIDE ? 4 : 2;
  constexpr int BK = WIDE ? 32 : 64;    // keys per batch
  constexpr int TPK = MK_CT / BK;       // threads per key
  constexpr int EPP = 16 / EL;          // elements per 16-byte piece
  unsigned long long tp = prof.tic();
  const int h = G.h, sp = G.sp, kvh = G.kvh, gi = G.gi;
  const int d = a.d, half = d / 2, rowbytes = d * EL;
  float* qs = sm.misc + MK_OFF_QS;
  float* kn = sm.misc + MK_OFF_KN;
  float* vn = sm.misc + MK_OFF_VN;
  float* wm = sm.misc + MK_OFF_WM;
  float* wl = sm.misc + MK_OFF_WL;
  float* ps = sm.misc + MK_OFF_RED;     // [64] the batch's softmax numerators
  float* wacc = sm.misc + MK_OFF_WACC;
  uint8_t* kbuf = reinterpret_cast<uint8_t*>(sm.misc + MK_OFF_KVK);
  uint8_t* vbuf = reinterpret_cast<uint8_t*>(sm.misc + MK_OFF_KVV);
  uint8_t* kc = a.kcache + (uint64_t)l * a.layer_stride;
  uint8_t* vc = a.vcache + (uint64_t)l * a.layer_stride;
  const int64_t plane = (int64_t)(G.plane_bytes / EL);  // element offset of this head's plane
  const int pos32 = (int)pos;  // positions are below the cache capacity, which fits 31 bits
  const int k_lo = G.k_lo, k_hi = G.k_hi;
  // this token's own key / value row goes into the staged batch that holds position pos
  auto put_own = [&](uint8_t* buf, int row, int e, float v) {
    const int o = kv_stage_off(row, e * EL, rowbytes, WIDE);
    if constexpr (WIDE)
      *reinterpret_cast<float*>(buf + o) = v;
    else if constexpr (KVT == E_BF16)
      *reinterpret_cast<__nv_bfloat16*>(buf + o) = __float2bfloat16_rn(v);
    else
      *reinterpret_cast<__half*>(buf + o) = __float2half_rn(v);
  };
  const bool own_here = pos32 >= k_lo && pos32 < k_hi;  // the last split
  const int own_row0 = pos32 - k_lo;                      // its row if it falls into the first batch

  if (warp < 3) {
    // lane j < d/4 holds elements i = 2j, 2j+1 and their rotation partners i + d/2
    const int64_t qd = (int64_t)a.nh * d, kvd = (int64_t)a.nkv * d;
    const int64_t base = warp == 0 ? (int64_t)h * d : (warp == 1 ? qd + (int64_t)kvh * d : qd + kvd + (int64_t)kvh * d);
    const bool act = lane < d / 4;
    const int i0 = 2 * lane;
    float w1a = 1.f, w1b = 1.f, w2a = 1.f, w2b = 1.f;
    if (act && a.has_norm && warp < 2) {
      const uint8_t* nw = reinterpret_cast<const uint8_t*>(warp == 0 ? L->q_norm : L->k_norm);
      w1a = aux_load(nw, L->qk_norm_type, i0), w1b = aux_load(nw, L->qk_norm_type, i0 + 1);
      w2a = aux_load(nw, L->qk_norm_type, i0 + half), w2b = aux_load(nw, L->qk_norm_type, i0 + half + 1);
    }
    float x[4] = {0.f, 0.f, 0.f, 0.f};  // x1a x1b x2a x2b
    if (act) {
      const int64_t idx[2] = {base + i0, base + i0 + half};
      ll_poll<2>(a.ll_qkv, idx, ep, x, sm.abort);
    }
    if (warp < 2) {
      if (a.has_norm) {
        const float ssq = warp_sum(fmaf(x[0], x[0], x[1] * x[1]) + fmaf(x[2], x[2], x[3] * x[3]));
        const float inv = 1.0f / sqrtf(ssq / (float)d + a.eps);
        x[0] = __fmul_rn(__fmul_rn(x[0], inv), w1a);
        x[1] = __fmul_rn(__fmul_rn(x[1], inv), w1b);
        x[2] = __fmul_rn(__fmul_rn(x[2], inv), w2a);
        x[3] = __fmul_rn(__fmul_rn(x[3], inv), w2b);
      }
      if (a.has_rope && act) {
        const float* cs = sm.misc + MK_OFF_ROPE;
        const float ca = cs[i0], cb = cs[i0 + 1], sa = cs[64 + i0], sb = cs[64 + i0 + 1];
        const float la = __fsub_rn(__fmul_rn(x[0], ca), __fmul_rn(x[2], sa));
        const float ha = __fadd_rn(__fmul_rn(x[0], sa), __fmul_rn(x[2], ca));
        const float lb = __fsub_rn(__fmul_rn(x[1], cb), __fmul_rn(x[3], sb));
        const float hb = __fadd_rn(__fmul_rn(x[1], sb), __fmul_rn(x[3], cb));
        x[0] = la, x[1] = lb, x[2] = ha, x[3] = hb;
      }
    }
    if (act) {
      float* dst = warp == 0 ? qs : (warp == 1 ? kn : vn);
      const int e[4] = {i0, i0 + 1, i0 + half, i0 + half + 1};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        dst[e[j]] = warp == 0 ? x[j] : round_kv(x[j], KVT);
        if (warp != 0 && own_here && own_row0 < BK) put_own(warp == 1 ? kbuf : vbuf, own_row0, e[j], x[j]);
      }
    }
  }
  cp_async_wait_all();  // this thread's share of the staged rows; the barrier covers the others'
  consumer_sync();
  prof.stamp(3);
  prof.toc(13, tp);
  tp = prof.tic();
  if (sp == 0 && gi == 0) {
    for (int i = tid; i < d; i += MK_CT) {
      store_kv(kc, KVT, plane + pos * d + i, kn[i]);
      store_kv(vc, KVT, plane + pos * d + i, vn[i]);
    }
  }
  const float scale = 1.0f / sqrtf((float)d);
  static_assert(MK_CT == 256, "the thread maps below assume 256 consumer threads");
  const int kl = tid / TPK, part = tid - kl * TPK;  // key within the batch, piece phase
  // value pass: dim pair and key group (head dim 128 or 64: shifts, not divisions -- this code is cold
  // every time it runs)
  const int lognp = d == 128 ? 6 : 5;
  const int npair = 1 << lognp, kg = tid >> lognp, dp = tid & (npair - 1);
  const int ngroups = MK_CT >> lognp;   // 4 or 8 key groups
  const int kpg = BK >> (8 - lognp);    // keys per group
  const int npiece = rowbytes >> 4;
  float m_run = -3.40282347e38f, l_run = 0.f, acc0 = 0.f, acc1 = 0.f;
  int bi = 0;
  for (int k0 = k_lo; k0 < k_hi; k0 += BK, bi++) {
    if (bi > 0) {  // long contexts: the later batches are brought in when their turn comes
      consumer_sync();  // everyone is done with the previous batch
      stage_kv(a, G, l, pos32, sm, tid, bi);
      if (own_here && pos32 >= k0 && pos32 < k0 + BK && tid < d) {
        put_own(kbuf, pos32 - k0, tid, kn[tid]);
        put_own(vbuf, pos32 - k0, tid, vn[tid]);
      }
      cp_async_wait_all();
      consumer_sync();
    }
    const int nvalid = k_hi - k0 < BK ? k_hi - k0 : BK;
    // ---- scores
    float dot = 0.f;
    if (kl < nvalid) {
#pragma unroll 2
      for (int pc = part; pc < npiece; pc += TPK) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kbuf + kv_stage_off(kl, pc << 4, rowbytes, WIDE));
        const float* q = qs + pc * EPP;
        const float4 q0 = *reinterpret_cast<const float4*>(q);
        if constexpr (WIDE) {
          dot = fmaf(q0.x, __uint_as_float(raw.x), dot), dot = fmaf(q0.y, __uint_as_float(raw.y), dot);
          dot = fmaf(q0.z, __uint_as_float(raw.z), dot), dot = fmaf(q0.w, __uint_as_float(raw.w), dot);
        } else {
          const float4 q1 = *reinterpret_cast<const float4*>(q + 4);
          const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
          const float qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float lo = KVT == E_BF16 ? __uint_as_float(r[j] << 16) : f16_bits_to_f32(r[j] & 0xffffu);
            const float hi = KVT == E_BF16 ? __uint_as_float(r[j] & 0xffff0000u) : f16_bits_to_f32(r[j] >> 16);
            dot = fmaf(qq[2 * j], lo, dot);
            dot = fmaf(qq[2 * j + 1], hi, dot);
          }
        }
      }
    }
#pragma unroll
    for (int o = 1; o < TPK; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float sc = kl < nvalid ? dot * scale : -INFINITY;
    prof.stamp_dbg(9);
    const float wmax = warp_max(sc);
    if (lane == 0) wm[warp] = wmax;
    consumer_sync();
    float m_new = m_run;
#pragma unroll
    for (int w = 0; w < MK_CW; w++) m_new = fmaxf(m_new, wm[w]);
    const float pr = expf(sc - m_new);  // a key past the range: exp(-inf) = 0
    if (part == 0) ps[kl] = pr;
    const float wsum = warp_sum(part == 0 ? pr : 0.f);
    if (lane == 0) wl[warp] = wsum;
    consumer_sync();
    float l_batch = 0.f;
#pragma unroll
    for (int w = 0; w < MK_CW; w++) l_batch += wl[w];
    prof.stamp_dbg(10);
    const float factor = expf(m_run - m_new);
    l_run = l_run * factor + l_batch;
    acc0 *= factor, acc1 *= factor;
    m_run = m_new;
    // ---- values
    const int kq_end = (kg + 1) * kpg < nvalid ? (kg + 1) * kpg : nvalid;
#pragma unroll 4
    for (int kq = kg * kpg; kq < kq_end; kq++) {
      const float pk = ps[kq];
      const uint8_t* vp = vbuf + kv_stage_off(kq, dp * 2 * EL, rowbytes, WIDE);
      float v0, v1;
      if constexpr (WIDE) {
        const float2 vv = *reinterpret_cast<const float2*>(vp);
        v0 = vv.x, v1 = vv.y;
      } else {
        const uint32_t r = *reinterpret_cast<const uint32_t*>(vp);
        v0 = KVT == E_BF16 ? __uint_as_float(r << 16) : f16_bits_to_f32(r & 0xffffu);
        v1 = KVT == E_BF16 ? __uint_as_float(r & 0xffff0000u) : f16_bits_to_f32(r >> 16);
      }
      acc0 = fmaf(pk, v0, acc0);
      acc1 = fmaf(pk, v1, acc1);
    }
  }
  prof.stamp_dbg(11);
  prof.toc(14, tp);
  prof.stamp(14);
  tp = prof.tic();
  // the key groups' sums meet in shared memory and are added in group order
  wacc[kg * 128 + 2 * dp] = acc0;
  wacc[kg * 128 + 2 * dp + 1] = acc1;
  consumer_sync();
  prof.stamp(15);
  const int64_t pbase = ((int64_t)h * a.max_split + sp) * (d + 4);
  if (tid < d) {
    float o = 0.f;
    for (int g = 0; g < ngroups; g++) o += wacc[g * 128 + tid];
    if (nsplit == 1)
      ll_store(a.ll_ctx, (int64_t)h * d + tid, o / l_run, ep);
    else
      ll_store(a.ll_part, pbase + tid, o, ep);
  }
  if (nsplit > 1 && tid == 0) {
    ll_store(a.ll_part, pbase + d, m_run, ep);
    ll_store(a.ll_part, pbase + d + 1, l_run, ep);
  }
  prof.stamp(4);
  prof.toc(15, tp);
  // the next layer's first batch: every warp is past its reads of the staging buffers (barrier above)
  stage_kv(a, G, l + 1, pos32, sm, tid);
}

template <class Prof>
__device__ __forceinline__ void phase_attention(const MegaArgs& a, int l, const MegaLayerHot* L, const AttGeo& G,
                                                int64_t pos, int nsplit, unsigned ep, const Smem& sm, int tid,
                                                int lane, int warp, Prof& prof) {
#ifndef MK_SIZE_PROBE
  if (a.kv_type == E_F32)
    phase_attention_t<E_F32>(a, l, L, G, pos, nsplit, ep, sm, tid, lane, warp, prof);
  else
#endif
#if !defined(MK_SIZE_PROBE) || MK_SIZE_PROBE < 3
  if (a.kv_type == E_BF16)
#else
  if (false)
#endif
    phase_attention_t<E_BF16>(a, l, L, G, pos, nsplit, ep, sm, tid, lane, warp, prof);
#ifndef MK_SIZE_PROBE
  else
    phase_attention_t<E_F16>(a, l, L, G, pos, nsplit, ep, sm, tid, lane, warp, prof);
#endif
}

// ---- one phase's rounds, in program order ---------------------------------------------------------
struct Walk {
  uint32_t ci, ri, ti;    // next chunk, round, tile of this CTA's program
  uint32_t slot, parity;  // ring position of chunk ci
  unsigned nround;        // rounds so far (selects the partial-sum buffer)
  unsigned nlocal;        // per-warp stagings so far (selects the sum-of-squares buffer)
  float bv;               // running argmax over the rows this thread finishes
  long long bi;
};

template <int ENC, class Prof>
__device__ __forceinline__ void run_phase_t(const MegaArgs& a, const Smem& sm, Walk& w, int nr, unsigned ep,
                                            const float* ssq, int n_in, float* res, int hid_lo, int tid, int lane,
                                            int warp, Prof& prof, int sid) {
  const int g = lane >> 2;
  for (int r = 0; r < nr; r++, w.ri++) {
    const MegaRound R = sm.rounds[w.ri];
    float* pb = sm.misc + MK_OFF_PART + (w.nround & 1u) * MK_PART;
    w.nround++;
    // chunks of one tile follow each other: a tile's sums stay in registers until the next tile begins
    TileAcc<true> t;
    t.clear();
    int cur = -1;
    auto flush = [&]() {
      if (cur >= 0 && (lane & 3) == 0) {
        pb[(cur * MK_CW + warp) * 16 + g] = t.v[0];
        pb[(cur * MK_CW + warp) * 16 + g + 8] = t.v[1];
      }
    };
    // Geometry of one chunk for this lane, from the 16 bytes a consumer reads.
    struct Geo {
      const uint8_t *p0, *p1, *a0, *a1;
      int nu, enc, aux, gs, kb0, apitch16;
    };
    auto geometry = [&](const uint4& hot, int slot) {
      Geo q;
      const int pitch = (int)(hot.x & 0xffffu);
      const int n = (int)(hot.y & 0xffu);
      const int al = (int)(hot.z & 0xffu), al_step = (int)((hot.z >> 8) & 0xffu);
      const int apitch = (int)(hot.w & 0xffffu);
      q.kb0 = (int)(hot.x >> 16), q.nu = (int)((hot.y >> 8) & 0xffu), q.enc = (int)(hot.y >> 24);
      q.aux = (int)((hot.z >> 16) & 0xffu), q.gs = (int)(hot.z >> 24), q.apitch16 = 16 * apitch;
      const uint8_t* base = sm.ring + (size_t)slot * MK_SLOT;
      const int i0 = g < n ? g : n - 1, i1 = g + 8 < n ? g + 8 : n - 1;  // clamp to valid rows
      q.p0 = base + i0 * pitch + ((al + i0 * al_step) & 15);
      q.p1 = base + i1 * pitch + ((al + i1 * al_step) & 15);
      q.a0 = q.a1 = nullptr;
      if (apitch) {
        const int aal = (int)((hot.w >> 16) & 0xffu), aal_step = (int)(hot.w >> 24);
        const uint8_t* ab = base + 16 * pitch;
        q.a0 = ab + i0 * apitch + ((aal + i0 * aal_step) & 15);
        q.a1 = ab + i1 * apitch + ((aal + i1 * aal_step) & 15);
      }
      return q;
    };
    auto release = [&](int slot) {
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.empty + slot);
      if (++w.slot == (uint32_t)sm.nslot) w.slot = 0, w.parity ^= 1u;
    };
    for (int k = 0; k < (int)R.nchunks; k++, w.ci++) {
      const uint4 hot = *reinterpret_cast<const uint4*>(sm.chunks + w.ci);
      const int which = (int)((hot.y >> 16) & 0xffu);
      const int slot = (int)w.slot;
      const unsigned long long tw = prof.tic();
      const bool ok = mbar_wait_bounded(sm.full + slot, w.parity, MK_MBAR_SPINS, sm.abort);
      if (!ok && !*sm.abort) *sm.abort = 3;
      prof.toc(10, tw);
      const unsigned long long tr = prof.tic();
      if (which != cur) {
        flush();
        t.clear();
        cur = which;
      }
      if (ok) {
        const Geo q = geometry(hot, slot);
        int u = warp;
        for (; u < q.nu; u += MK_CW)
          run_unit<ENC>(q.enc, q.aux, q.gs, q.p0, q.p1, q.a0, q.a1, q.apitch16, u, q.kb0, sm, lane, t);
      }
      prof.toc(11, tr);
      release(slot);
    }
    flush();
    prof.stamp(sid + 1);
    // the K-slice partials of every tile of the round meet here, once
    const unsigned long long tc = prof.tic();
    consumer_sync();
    const int nt = R.ntiles;
    if (tid < nt * 16) {
      const MegaTile T = sm.tiles[w.ti + (tid >> 4)];
      const int row = tid & 15;
      if (row < (int)T.n) {
        // per-warp staging leaves RMSNorm's scalar factor to be applied here
        float out_scale = 1.0f;
        if (ssq) {
          float tss = 0.f;
#pragma unroll
          for (int wv = 0; wv < MK_CW; wv++) tss += ssq[wv];
          out_scale = 1.0f / sqrtf(tss / (float)n_in + a.eps);
        }
        const float* p1 = pb + (int)T.acc * MK_CW * 16 + row;
        float s0 = 0.f;
#pragma unroll
        for (int wv = 0; wv < MK_CW; wv++) s0 += p1[wv * 16];
        s0 *= out_scale;
        const int64_t orow = (int64_t)T.out_row + row;
        if (T.ep == MEGA_EP_QKV) {
          ll_store(a.ll_qkv, orow, s0, ep);
        } else if (T.ep == MEGA_EP_RESID_O || T.ep == MEGA_EP_RESID_DOWN) {
          const float hnew = res[orow - hid_lo] + s0;
          res[orow - hid_lo] = hnew;
          ll_store(a.ll_hidden[T.ep == MEGA_EP_RESID_O ? 0 : 1], orow, hnew, ep);
        } else if (T.ep == MEGA_EP_SWIGLU) {
          const float* p2 = pb + (int)T.acc2 * MK_CW * 16 + row;
          float s1 = 0.f;
#pragma unroll
          for (int wv = 0; wv < MK_CW; wv++) s1 += p2[wv * 16];
          s1 *= out_scale;
          ll_store(a.ll_act, orow, (s0 / (1.0f + expf(-s0))) * s1, ep);
        } else if (T.ep == MEGA_EP_SWIGLU_IL) {
          float s1 = 0.f;  // the same row of `up`: tile row + 8 of the same accumulator
#pragma unroll
          for (int wv = 0; wv < MK_CW; wv++) s1 += p1[wv * 16 + 8];
          s1 *= out_scale;
          ll_store(a.ll_act, orow, (s0 / (1.0f + expf(-s0))) * s1, ep);
        } else {
          a.logits[orow] = s0;
          if (s0 > -INFINITY && arg_better(s0, orow, w.bv, w.bi)) w.bv = s0, w.bi = orow;
        }
      }
    }
    w.ti += nt;
    prof.stamp(sid + 2);
    prof.toc(12, tc);
  }
}

// phase word: low byte = rounds, high byte = the phase's common encoding (0xff: per chunk)
// Stages the phase's input vector (per warp where the encoding allows) and runs its rounds. A CTA
// without rows in the phase neither waits for the vector nor stages it.
template <class Prof>
__device__ __forceinline__ void run_phase(const MegaArgs& a, const Smem& sm, Walk& w, int phase_index, unsigned ep,
                                          const StageSrc& src, const void* nw, int nw_type, int n_in, int layout_enc,
                                          float* res, int hid_lo, int tid, int lane, int warp, Prof& prof) {
  const unsigned word = sm.phase_rounds[phase_index];
  const int nr = (int)(word & 0xffu), enc = (int)(word >> 8);
  if (nr == 0) return;
  const unsigned long long ts = prof.tic();
  const float* ssq = nullptr;
  if (MK_OPT_LOCAL && (enc == E_Q4_0 || enc == E_Q4_1 || enc == E_Q8_0 || enc == E_MLX_U4)) {
    float* mine = sm.misc + MK_OFF_RED + 32 + (w.nlocal & 1u) * MK_CW;  // consecutive per-warp stages alternate
    w.nlocal++;
    stage_local(src, nw, nw_type, n_in, (enc == E_Q4_0 || enc == E_Q8_0 || enc == E_MLX_U4) ? 2 : 1, xl_for_encoding(enc), sm, mine + warp,
                lane, warp);
    if (nw) ssq = mine;
  } else {
#if !defined(MK_SIZE_PROBE) || MK_SIZE_PROBE < 4
    stage_phase(src, nw, nw_type, n_in, a.eps, xl_for_encoding(layout_enc), sm, tid, lane, warp);
#endif
  }
  prof.toc(9, ts);
  const int sid = (phase_index & 3) == 0 ? 0 : 2 + 3 * (phase_index & 3);  // 0, 5, 8, 11
  prof.stamp(sid);
  if (enc == E_Q4_0)
    run_phase_t<E_Q4_0>(a, sm, w, nr, ep, ssq, n_in, res, hid_lo, tid, lane, warp, prof, sid);
#if !defined(MK_SIZE_PROBE) || MK_SIZE_PROBE < 2
  else if (enc == E_Q6_K)
    run_phase_t<E_Q6_K>(a, sm, w, nr, ep, ssq, n_in, res, hid_lo, tid, lane, warp, prof, sid);
  else if (enc == E_MLX_U4)  // MLX models: every layer product is of this kind
    run_phase_t<E_MLX_U4>(a, sm, w, nr, ep, ssq, n_in, res, hid_lo, tid, lane, warp, prof, sid);
#endif
#ifndef MK_SIZE_PROBE
  else
    run_phase_t<-1>(a, sm, w, nr, ep, ssq, n_in, res, hid_lo, tid, lane, warp, prof, sid);
#endif
}

// ---- the kernel ------------------------------------------------------------------------------------
template <bool INSTR>
__device__ __forceinline__ void decode_mega_body(const MegaArgs& a) {
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
  sm.isx = sm.sx16 + a.xs_floats / 16;
  sm.misc = sm.isx + a.xs_floats / 32;
  sm.ring = reinterpret_cast<uint8_t*>(sm.misc + MK_MISC_FLOATS);
  sm.full = reinterpret_cast<uint64_t*>(sm.ring + (size_t)a.nslot * MK_SLOT);
  sm.empty = sm.full + a.nslot;
  sm.prog_bar = sm.empty + a.nslot;
  uint8_t* prog_area = reinterpret_cast<uint8_t*>(sm.prog_bar + 2);
  sm.abort = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < a.nslot; i++) {
      mbar_init(sm.full + i, 1);
      mbar_init(sm.empty + i, MK_CW);
    }
    mbar_init(sm.prog_bar, 1);
    mbar_fence_init();
    // one bulk copy brings this CTA's whole program next to the math
    mbar_expect_tx(sm.prog_bar, (unsigned)a.lay.bytes);
    bulk_g2s(prog_area, a.prog + (size_t)cta * a.lay.bytes, (unsigned)a.lay.bytes, sm.prog_bar);
  }
  __syncthreads();
  if (!mbar_wait_bounded(sm.prog_bar, 0, MK_MBAR_SPINS, sm.abort) && !*sm.abort) *sm.abort = 7;
  const MegaProgHeader* hdr = reinterpret_cast<const MegaProgHeader*>(prog_area);
  sm.chunks = reinterpret_cast<const MegaChunk*>(prog_area + sizeof(MegaProgHeader));
  sm.tiles = reinterpret_cast<const MegaTile*>(prog_area + a.lay.off_tiles);
  sm.rounds = reinterpret_cast<const MegaRound*>(prog_area + a.lay.off_rounds);
  sm.phase_rounds = reinterpret_cast<const uint16_t*>(prog_area + a.lay.off_phase);
  sm.hot = reinterpret_cast<const MegaLayerHot*>(prog_area + a.lay.off_layers);

  sm.nchunks = hdr->nchunks;
  if (warp == MK_CW) {
    // ------------------------------ producer: stream this CTA's weight tiles --------------
    const int total = *sm.abort ? 0 : (int)hdr->nchunks;
    int slot = 0;
    uint32_t lap = 0;
    for (int step = 0; step < a.steps; step++)  // the same program for every token of the launch
      for (int pi = 0; pi < total; pi++) {
        produce_chunk(sm.chunks + pi, sm, slot, lap, lane);
        if (++slot == sm.nslot) slot = 0, lap++;
      }
    return;
  }
  // -------------------------------- consumers -------------------------------------------------
  int64_t token = a.inline_io ? a.in_token : __ldcg(a.io + 0), pos = a.inline_io ? a.in_pos : __ldcg(a.io + 1);
  const int64_t seq = a.inline_io ? a.in_seq : __ldcg(a.io + 2);
  const int64_t qd = (int64_t)a.nh * a.d;
  const int hid_lo = (int)hdr->hid_lo;
  float* res = sm.misc + MK_OFF_RES;
  Walk wk;
  wk.ci = wk.ri = wk.ti = 0, wk.slot = 0, wk.parity = 0, wk.nround = 0, wk.nlocal = 0;
  wk.bv = -INFINITY, wk.bi = 0x7fffffffffffffffLL;
  ProfT<INSTR> prof;
  // One launch decodes a.steps tokens: every CTA learns each token from the argmax hand-off and goes
  // on with the next position; the weight ring and its barriers simply keep running.
  for (int step = 0; step < a.steps; step++) {
  const unsigned epoch_base = a.epoch_base + (unsigned)step * (unsigned)(a.layers + 2);
  int nsplit = (int)((pos + 1 + 63) / 64);
  if (nsplit > a.max_split) nsplit = a.max_split;
  if (nsplit < 1) nsplit = 1;
  wk.ci = wk.ri = wk.ti = 0;
  wk.bv = -INFINITY, wk.bi = 0x7fffffffffffffffLL;
  prof.begin(a.prof, cta == 0 && tid == 0);
  if constexpr (INSTR) prof.trace = (a.trace && tid == 0) ? a.trace + (size_t)cta * (a.layers + 1) * 16 : nullptr;
  prof.layer = 0;

  if (a.has_rope && tid < a.d / 2) {
    // the rotation of this token's position, shared by all layers (kernels.rs:1047-1064)
    float sv, cv;
    sincosf(__fmul_rn((float)pos, a.ft.f[tid]), &sv, &cv);
    sm.misc[MK_OFF_ROPE + tid] = cv;
    sm.misc[MK_OFF_ROPE + 64 + tid] = sv;
  }
  const AttGeo AG = att_geometry(a, cta, (int)pos, (int)seq, nsplit);
  stage_kv(a, AG, 0, (int)pos, sm, tid);
  // every CTA decodes the token's embedding row for itself: no hand-off before the first product
  mega_gather_row(a.embed, token, sm.xs, tid, MK_CT);
  consumer_sync();
  {
    const int hid_hi = (int)hdr->hid_hi;
    for (int i = hid_lo + tid; i < hid_hi; i += MK_CT) res[i - hid_lo] = sm.xs[i];
  }
  prof.mark(0);

  StageSrc src;
  src.nsplit = nsplit, src.max_split = a.max_split, src.d = a.d;
  // One loop over the 4 * layers + 1 products (q/k/v, o, gate/up, down per layer, then the head) so
  // that the product code exists once in the kernel: the five products of a layer run the same
  // instructions, which then stay in the instruction cache from layer to layer.
  const int nprod = 4 * a.layers;
  const MegaLayerHot* L = sm.hot;
  unsigned ep = epoch_base;
  for (int ph = 0; ph <= nprod; ph++) {
    const int l = ph >> 2, k = ph & 3;
    const bool head = ph == nprod;
    const void* nw = nullptr;
    int nw_type = 0, n_in, lenc;
    if (k == 0) {
      // layer l begins (l == layers: the final norm and the head, which follow the same hand-off rule)
      ep = epoch_base + 1u + (unsigned)l;
      prof.layer = l;
      if (!head) {
        L = sm.hot + l;
        if (!(a.opts & 2)) {  // the next layer's norm vectors (the final one behind the last layer)
          const size_t nel = L->norm_type == E_F32 ? 4 : 2, qel = L->qk_norm_type == E_F32 ? 4 : 2;
          if (l + 1 < a.layers) {
            prefetch_span(L[1].attn_norm, (size_t)a.H * nel, tid, MK_CT);
            prefetch_span(L[1].ffn_norm, (size_t)a.H * nel, tid, MK_CT);
            if (a.has_norm && cta < a.nh * nsplit && tid < 2)
              prefetch_span(tid == 0 ? L[1].q_norm : L[1].k_norm, (size_t)a.d * qel, 0, 1);
          } else {
            prefetch_span(a.out_norm, (size_t)a.H * (a.out_norm_type == E_F32 ? 4 : 2), tid, MK_CT);
          }
        }
      }
      src.kind = l == 0 ? SRC_XS : SRC_LL, src.ll = a.ll_hidden[1], src.ep = ep - 1u;
      nw = head ? a.out_norm : L->attn_norm, nw_type = head ? a.out_norm_type : L->norm_type;
      n_in = a.H, lenc = head ? a.lm_head.enc : L->enc_q;
    } else if (k == 1) {
      phase_attention(a, l, L, AG, pos, nsplit, ep, sm, tid, lane, warp, prof);
      prof.mark(2);
      src.kind = nsplit > 1 ? SRC_PARTIALS : SRC_LL, src.ll = nsplit > 1 ? a.ll_part : a.ll_ctx, src.ep = ep;
      n_in = (int)qd, lenc = L->enc_o;
    } else if (k == 2) {
      src.kind = SRC_LL, src.ll = a.ll_hidden[0], src.ep = ep;
      nw = L->ffn_norm, nw_type = L->norm_type, n_in = a.H, lenc = L->enc_gate;
    } else {
      src.kind = SRC_LL, src.ll = a.ll_act, src.ep = ep;
      n_in = a.I, lenc = L->enc_down;
    }
    run_phase(a, sm, wk, ph, ep, src, nw, nw_type, n_in, lenc, res, hid_lo, tid, lane, warp, prof);
    prof.mark(head ? 6 : (k == 0 ? 1 : 2 + k));
  }
  const unsigned ep_last = epoch_base + (unsigned)a.layers;
  {
    // the (at most 128) finishing threads hold this CTA's candidates
    float* cv = sm.misc + MK_OFF_AMAX;
    if (tid < MEGA_TA * 16) {
      cv[tid] = wk.bv;
      cv[128 + tid] = __int_as_float((int)(wk.bi == 0x7fffffffffffffffLL ? 0x7fffffff : wk.bi));
    }
    consumer_sync();
    if (warp == 0) {
      float v = -INFINITY;
      long long i = 0x7fffffffffffffffLL;
      for (int c = lane; c < MEGA_TA * 16; c += 32) {
        const float ov = cv[c];
        const int oi = __float_as_int(cv[128 + c]);
        if (oi != 0x7fffffff && arg_better(ov, oi, v, i)) v = ov, i = oi;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (arg_better(ov, oi, v, i)) v = ov, i = oi;
      }
      if (lane == 0) {
        // this CTA's cache rows of the token (stored by other threads, before block barriers this
        // thread has passed) are ordered before the pair that lets the next token begin
        __threadfence();
        // one 32-byte sector per CTA: (value, epoch), (row, epoch), unused
        ll_store(a.ll_amax, 4 * (int64_t)cta, v, ep_last + 1u);
        ll_store(a.ll_amax, 4 * (int64_t)cta + 1, __int_as_float((int)(i == 0x7fffffffffffffffLL ? 0x7fffffff : i)),
                 ep_last + 1u);
      }
    }
  }
  prof.mark(6);
  // every CTA reads all candidates and arrives at the same token (first strict maximum)
  int* next_tok = reinterpret_cast<int*>(sm.misc + MK_OFF_AMAX);
  if (warp == 0) {
    float v = -INFINITY;
    long long i = 0x7fffffffffffffffLL;
    for (int c = lane; c < G; c += 32) {
      const int64_t idx[1] = {4 * (int64_t)c};
      float p[2];
      ll_poll<1>(a.ll_amax, idx, ep_last + 1u, p, sm.abort);
      const int oi = __float_as_int(p[1]);
      if (oi != 0x7fffffff && arg_better(p[0], oi, v, i)) v = p[0], i = oi;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (arg_better(ov, oi, v, i)) v = ov, i = oi;
    }
    __threadfence();  // the cache rows other CTAs stored for this token are visible to what follows
    if (lane == 0) {
      const int64_t tok = i == 0x7fffffffffffffffLL ? 0 : (int64_t)i;
      *next_tok = (int)tok;
      if (cta == 0) {
        a.io[3] = tok;
        if (a.out_host) a.out_host[0] = tok;
        if (a.advance) {
          a.io[0] = tok;
          a.io[1] = pos + 1;
          const int64_t cnt = a.hist_count[0];
          if (cnt < a.hist_cap) a.hist[cnt] = tok;
          a.hist_count[0] = cnt + 1;
        }
      }
    }
  }
  prof.mark(7);
  prof.end();
  consumer_sync();
  token = *next_tok;
  pos += 1;
  if (*sm.abort) break;
  consumer_sync();  // next_tok shares its words with the candidates of the next token
  }  // tokens of the launch
  if (tid == 0 && *sm.abort) {
    atomicExch(a.error, *sm.abort);
    if (a.out_host) a.out_host[1] = *sm.abort;
    // let any bulk copy still in flight land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < (1LL << 22)) {
    }
  }
}

__global__ void __launch_bounds__(MK_THREADS, 1) decode_mega_kernel(const MegaArgs a) { decode_mega_body<false>(a); }
// the same kernel with the per-phase timers and the event trace compiled in
__global__ void __launch_bounds__(MK_THREADS, 1) decode_mega_kernel_timed(const MegaArgs a) {
  decode_mega_body<true>(a);
}

}  // namespace

size_t mega_smem_bytes(int nslot, int xs_floats, size_t prog_bytes) {
  return (size_t)xs_floats * 4 * 2 + (size_t)(xs_floats / 32 + xs_floats / 16 + xs_floats / 32) * 4 +
         (size_t)MK_MISC_FLOATS * 4 + (size_t)nslot * MK_SLOT + (size_t)nslot * 16 + 128 + prog_bytes;
}

// prog_bytes: bytes of one CTA's program blob, which lives in shared memory beside the ring.
int mega_plan(int H, int I, int qd, int d, size_t prog_bytes, int* nslot, int* xs_floats, size_t* smem) {
  int xs = H > I ? H : I;
  if (qd > xs) xs = qd;
  xs = (xs + 255) / 256 * 256;
  if ((d != 64 && d != 128) || H % 32 || I % 32 || qd % 32) return 0;
  const size_t budget = 225 * 1024;
  const size_t fixed = mega_smem_bytes(0, xs, prog_bytes) + 512;
  if (fixed + 4 * (size_t)(MK_SLOT + 16) > budget) return 0;
  int n = (int)((budget - fixed) / (MK_SLOT + 16));
  if (n > 12) n = 12;
  *nslot = n;
  *xs_floats = xs;
  *smem = mega_smem_bytes(n, xs, prog_bytes);
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
    case E_MLX_U4: p.ubytes = 32, p.ukb = 2, p.units_total = K / 64; break;
    case E_BF16:
    case E_F16: p.ubytes = 64, p.ukb = 1, p.units_total = K / 32; break;
    default: p.ubytes = 0, p.ukb = 2, p.units_total = K / 64, p.unit_q6 = 1; break;  // quarters
  }
  return p;
}
int seg_bytes(const HostPlan& p, int nu) { return p.unit_q6 ? (nu / 4) * 210 : nu * p.ubytes; }

// Appends the chunks of rows [r, r + n) (n <= 16) of `w`, summed into accumulator `acc`: the
// fewest K-slices whose rows fit one ring slot (slices are multiples of 16 units so the 16
// consumer warps share them evenly; Q6_K slices are whole groups of 4 superblocks, which keeps
// rows 8-byte aligned).
void add_tile_chunks(const WRef& w, int64_t r, int n, int acc, std::vector<MegaChunk>* v, int64_t jump = 0) {
  const HostPlan p = host_plan(w);
  const int ael = w.aux == E_F32 ? 4 : 2;
  // largest slice (multiple of 16 units) whose rows fit one slot; only valid rows are copied
  int su = p.units_total < 16 ? p.units_total : 16;
  for (int cand = 16; cand <= p.units_total && cand <= 240; cand += 16) {
    const int pitch = host_bank_pitch(seg_bytes(p, cand) + 20);
    const int ap = w.enc == E_MLX_U4 ? ((cand * p.ukb * 32 / w.group) * ael + 31) / 16 * 16 : 0;
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
    c.acc = (uint8_t)acc;
    c.al = (uint8_t)(reinterpret_cast<uintptr_t>(c.src) & 15);
    c.al_step = (uint8_t)(c.rb & 15u);
    c.jump16 = (int32_t)(jump / 16);
    // Q6_K rows over the full K are copied as one run: their natural pitch (840 bytes for K = 1024)
    // spreads the eight row pairs over the banks almost as well as a padded pitch does, and one copy
    // replaces sixteen
    for (int i = 0; i < n; i++) c.tx += ((((uint32_t)c.al + (uint32_t)i * c.al_step) & 15u) + c.seg + 15u) & ~15u;
    if (w.enc == E_Q6_K && jump == 0 && nsl == 1 && (size_t)n * c.rb + 16 <= (size_t)MK_SLOT && c.rb % 4 == 0 && ((c.rb / 4) & 1) == 0) {
      c.pitch = (uint16_t)c.rb;
      c.al_step = 0;
      c.contig = (uint32_t)((c.al + (size_t)n * c.rb + 15) / 16 * 16);
    }
    if (w.enc == E_MLX_U4) {
      const int64_t arow = (int64_t)(w.cols / w.group) * ael, ao = (int64_t)(u0 * p.ukb * 32 / w.group) * ael;
      c.sc = w.scales + r * arow + ao;
      c.bi = w.biases + r * arow + ao;
      c.arb = (uint32_t)arow;
      c.aseg = (uint16_t)((nu * p.ukb * 32 / w.group) * ael);
      c.apitch = (uint16_t)(((su * p.ukb * 32 / w.group) * ael + 31) / 16 * 16);
      c.aal = (uint8_t)(reinterpret_cast<uintptr_t>(c.sc) & 15);
      c.aal_step = (uint8_t)(c.arb & 15u);
      for (int i = 0; i < n; i++) c.tx += 2u * (((((uint32_t)c.aal + (uint32_t)i * c.aal_step) & 15u) + c.aseg + 15u) & ~15u);
      c.aux = (uint8_t)w.aux;
      c.group_shift = (uint8_t)(w.group == 32 ? 0 : (w.group == 64 ? 1 : 2));
    }
    v->push_back(c);
  }
}

struct CtaProgram {
  std::vector<MegaChunk> chunks;
  std::vector<MegaTile> tiles;
  std::vector<MegaRound> rounds;
  std::vector<uint16_t> phase_rounds;
  // the round being filled
  int accs = 0;
  bool open = false;
  void begin_phase() {
    phase_rounds.push_back(0);
    open = false;
  }
  void need(int naccs) {
    if (!open || accs + naccs > MEGA_TA) {
      rounds.push_back(MegaRound{0, 0, 0});
      phase_rounds.back()++;
      accs = 0;
      open = true;
    }
  }
  // gate and up rows [lo, hi), eight of each per tile (rows 0..7 gate, 8..15 up): three tiles where
  // separate gate and up tiles would take four for 24 rows. (hi - lo) % 8 == 0.
  void add_rows_interleaved(const WRef& gate, const WRef& up, int64_t lo, int64_t hi) {
    const int64_t rb = (int64_t)gate.row_bytes();
    const int64_t jump = (up.data - gate.data) - 8 * rb;
    for (int64_t r = lo; r < hi; r += 8) {
      need(1);
      MegaTile t{};
      t.out_row = (int32_t)r, t.n = 8, t.ep = (uint8_t)MEGA_EP_SWIGLU_IL, t.acc = (uint8_t)accs, t.acc2 = 0;
      const size_t before = chunks.size();
      add_tile_chunks(gate, r, 16, accs, &chunks, jump);
      accs += 1;
      rounds.back().naccs = (uint8_t)accs;
      tiles.push_back(t);
      rounds.back().nchunks = (uint16_t)(rounds.back().nchunks + (chunks.size() - before));
      rounds.back().ntiles++;
    }
  }
  // rows [lo, hi) of w (and of w2 for SwiGLU pairs), output rows out_off + row
  void add_rows(const WRef& w, const WRef* w2, int64_t lo, int64_t hi, int64_t out_off, int ep) {
    for (int64_t r = lo; r < hi; r += 16) {
      const int n = (int)std::min<int64_t>(16, hi - r);
      need(w2 ? 2 : 1);
      MegaTile t{};
      t.out_row = (int32_t)(out_off + r), t.n = (uint8_t)n, t.ep = (uint8_t)ep;
      t.acc = (uint8_t)accs, t.acc2 = (uint8_t)(w2 ? accs + 1 : 0);
      const size_t before = chunks.size();
      add_tile_chunks(w, r, n, accs, &chunks);
      if (w2) add_tile_chunks(*w2, r, n, accs + 1, &chunks);
      accs += w2 ? 2 : 1;
      rounds.back().naccs = (uint8_t)accs;
      tiles.push_back(t);
      rounds.back().nchunks = (uint16_t)(rounds.back().nchunks + (chunks.size() - before));
      rounds.back().ntiles++;
    }
  }
};
}  // namespace

// First row of CTA `cta` when `n` rows are dealt to `grid` CTAs in units of 4 rows. Four pairs are
// one 32-byte sector of a hand-off vector: when two CTAs store into the same sector the hand-off
// takes more than twice as long (2.46 us against 1.10 us for a 1024-element vector between 148
// CTAs), so no sector has two writers. Needs n % 4 == 0.
static int64_t split4(int64_t n, int cta, int grid) { return 4 * ((n / 4) * cta / grid); }
static int64_t split8(int64_t n, int cta, int grid) { return 8 * ((n / 8) * cta / grid); }
// gate and up can share tiles when they are the same kind of matrix and 16-byte congruent
static bool can_interleave(const WRef& g, const WRef& u, int I) {
  return (g.enc == E_Q4_0 || g.enc == E_Q4_1 || g.enc == E_Q8_0) && u.enc == g.enc && u.cols == g.cols && I % 8 == 0 &&
         ((u.data - g.data) - 8 * (int64_t)g.row_bytes()) % 16 == 0 &&
         std::llabs(((u.data - g.data) - 8 * (int64_t)g.row_bytes()) / 16) < (1LL << 31);
}

int mega_build_program(const MegaBuildLayer* layers, const MegaLayer* full, int nlayers, const WRef& lm_head, int nh,
                       int nkv, int d, int H, int I, int V, int grid, std::vector<uint8_t>* blob, MegaProgLayout* lay) {
  DYN_CHECK(H % 4 == 0 && I % 4 == 0 && (nh * d) % 4 == 0 && (nkv * d) % 4 == 0,
            "persistent decode kernel: widths must be multiples of 4");
  const int nph = 4 * nlayers + 1;
  std::vector<CtaProgram> per(grid);
  const int64_t qd = (int64_t)nh * d, kvd = (int64_t)nkv * d;
  for (int cta = 0; cta < grid; cta++) {
    CtaProgram& pc = per[cta];
    const int64_t h0 = split4(H, cta, grid), h1 = split4(H, cta + 1, grid);
    DYN_CHECK(h1 - h0 <= MK_MAX_OWNED, "persistent decode kernel: %lld hidden rows per CTA exceed %d",
              (long long)(h1 - h0), MK_MAX_OWNED);
    for (int l = 0; l < nlayers; l++) {
      const MegaBuildLayer& L = layers[l];
      pc.begin_phase();
      {  // q, k, v share one balanced split of their concatenated rows
        const int64_t R = qd + 2 * kvd, a0 = split4(R, cta, grid), a1 = split4(R, cta + 1, grid);
        const int64_t offs[3] = {0, qd, qd + kvd}, lens[3] = {qd, kvd, kvd};
        const WRef* ws[3] = {&L.q, &L.k, &L.v};
        for (int t = 0; t < 3; t++) {
          const int64_t lo = std::max(a0, offs[t]) - offs[t], hi = std::min(a1, offs[t] + lens[t]) - offs[t];
          if (hi > lo) pc.add_rows(*ws[t], nullptr, lo, hi, offs[t], MEGA_EP_QKV);
        }
      }
      pc.begin_phase();
      pc.add_rows(L.o, nullptr, h0, h1, 0, MEGA_EP_RESID_O);
      pc.begin_phase();
      if (can_interleave(L.gate, L.up, I))
        pc.add_rows_interleaved(L.gate, L.up, split8(I, cta, grid), split8(I, cta + 1, grid));
      else
        pc.add_rows(L.gate, &L.up, split4(I, cta, grid), split4(I, cta + 1, grid), 0, MEGA_EP_SWIGLU);
      pc.begin_phase();
      pc.add_rows(L.down, nullptr, h0, h1, 0, MEGA_EP_RESID_DOWN);
    }
    pc.begin_phase();
    pc.add_rows(lm_head, nullptr, (int64_t)V * cta / grid, (int64_t)V * (cta + 1) / grid, 0, MEGA_EP_LOGITS);
  }
  // every output row of every phase is produced exactly once, by a tile of at most 16 rows
  {
    std::vector<int64_t> rows((size_t)nph, 0);
    for (auto& pc : per) {
      size_t ti = 0, ri = 0;
      DYN_CHECK((int)pc.phase_rounds.size() == nph, "decode program: phase count mismatch");
      for (int ph = 0; ph < nph; ph++)
        for (int r = 0; r < pc.phase_rounds[ph]; r++, ri++) {
          DYN_CHECK(pc.rounds[ri].naccs <= MEGA_TA && pc.rounds[ri].ntiles <= MEGA_TA, "decode program: round too wide");
          DYN_CHECK(pc.phase_rounds[ph] <= 255, "decode program: more than 255 rounds in a phase");
          for (int t = 0; t < pc.rounds[ri].ntiles; t++, ti++) {
            DYN_CHECK(pc.tiles[ti].n >= 1 && pc.tiles[ti].n <= 16, "decode program: bad tile");
            rows[ph] += pc.tiles[ti].n;
          }
        }
    }
    for (int l = 0; l < nlayers; l++)
      DYN_CHECK(rows[4 * l] == qd + 2 * kvd && rows[4 * l + 1] == H && rows[4 * l + 2] == I && rows[4 * l + 3] == H,
                "decode program: layer %d rows are not covered exactly once", l);
    DYN_CHECK(rows[4 * nlayers] == V, "decode program: lm_head rows are not covered exactly once");
  }
  size_t mc = 1, mt = 1, mr = 1;
  for (auto& pc : per) {
    mc = std::max(mc, pc.chunks.size());
    mt = std::max(mt, pc.tiles.size());
    mr = std::max(mr, pc.rounds.size());
  }
  DYN_CHECK(mc < 60000 && mr < 60000, "decode program too long (%zu chunks per CTA)", mc);
  lay->max_chunks = (int)mc, lay->max_tiles = (int)mt, lay->max_rounds = (int)mr, lay->nph = nph;
  lay->off_tiles = sizeof(MegaProgHeader) + mc * sizeof(MegaChunk);
  lay->off_rounds = lay->off_tiles + mt * sizeof(MegaTile);
  lay->off_phase = lay->off_rounds + mr * sizeof(MegaRound);
  lay->off_layers = (lay->off_phase + (size_t)nph * 2 + 7) / 8 * 8;
  lay->bytes = (lay->off_layers + (size_t)nlayers * sizeof(MegaLayerHot) + 15) / 16 * 16;
  blob->assign((size_t)grid * lay->bytes, 0);
  std::vector<MegaLayerHot> hot(nlayers);
  for (int l = 0; l < nlayers; l++) {
    MegaLayerHot& t = hot[l];
    memset(&t, 0, sizeof t);
    t.attn_norm = full[l].attn_norm, t.ffn_norm = full[l].ffn_norm, t.q_norm = full[l].q_norm, t.k_norm = full[l].k_norm;
    t.norm_type = (uint8_t)full[l].norm_type, t.qk_norm_type = (uint8_t)full[l].qk_norm_type;
    t.enc_q = (uint8_t)full[l].q.enc, t.enc_o = (uint8_t)full[l].o.enc;
    t.enc_gate = (uint8_t)full[l].gate.enc, t.enc_down = (uint8_t)full[l].down.enc;
  }
  for (int cta = 0; cta < grid; cta++) {
    const CtaProgram& pc = per[cta];
    uint8_t* b = blob->data() + (size_t)cta * lay->bytes;
    MegaProgHeader h{(uint32_t)pc.chunks.size(), (uint32_t)split4(H, cta + 1, grid), (uint32_t)pc.rounds.size(),
                     (uint32_t)split4(H, cta, grid)};
    memcpy(b, &h, sizeof h);
    if (!pc.chunks.empty()) memcpy(b + sizeof h, pc.chunks.data(), pc.chunks.size() * sizeof(MegaChunk));
    if (!pc.tiles.empty()) memcpy(b + lay->off_tiles, pc.tiles.data(), pc.tiles.size() * sizeof(MegaTile));
    if (!pc.rounds.empty()) memcpy(b + lay->off_rounds, pc.rounds.data(), pc.rounds.size() * sizeof(MegaRound));
    // phase word: rounds in the low byte, the encoding every chunk of the phase shares in the high byte
    std::vector<uint16_t> words(pc.phase_rounds.size());
    size_t ci = 0, ri = 0;
    for (size_t ph = 0; ph < pc.phase_rounds.size(); ph++) {
      int enc = -1;
      for (int r = 0; r < pc.phase_rounds[ph]; r++, ri++)
        for (int k = 0; k < pc.rounds[ri].nchunks; k++, ci++)
          enc = enc == -1 ? pc.chunks[ci].enc : (enc == pc.chunks[ci].enc ? enc : 0xff);
      words[ph] = (uint16_t)(pc.phase_rounds[ph] | ((enc < 0 ? 0xff : enc) << 8));
    }
    memcpy(b + lay->off_phase, words.data(), words.size() * 2);
    if (nlayers) memcpy(b + lay->off_layers, hot.data(), hot.size() * sizeof(MegaLayerHot));
  }
  return 0;
}

// Whether the persistent kernel's tile steps can read this tensor (encoding and row alignment).
bool mega_supports_weight(const WRef& w) {
  switch (w.enc) {
    case E_Q4_0:
    case E_Q8_0: return w.cols % 256 == 0;
    case E_Q4_1: return w.cols % 128 == 0;
    case E_Q6_K: return w.cols % 1024 == 0;
    case E_BF16:  // plain 16-bit matrices (a tied bf16 embedding table as the head)
    case E_F16: return w.cols % 512 == 0;
    case E_MLX_U4:  // scales and biases are copied with one alignment rule: they must agree modulo 16
      return w.cols % 256 == 0 && (w.group == 32 || w.group == 64 || w.group == 128) &&
             ((reinterpret_cast<uintptr_t>(w.scales) ^ reinterpret_cast<uintptr_t>(w.biases)) & 15) == 0;
    default: return false;
  }
}

int mega_grid_size(int device, size_t smem, int* grid) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(decode_mega_kernel), (int)smem)) return 1;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(decode_mega_kernel_timed), (int)smem)) return 1;
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
  const bool timed = a.prof != nullptr || a.trace != nullptr;
  DYN_CUDA(cudaLaunchCooperativeKernel(timed ? (void*)decode_mega_kernel_timed : (void*)decode_mega_kernel, dim3(grid),
                                       dim3(MK_THREADS), args, smem, s));
  count_launch();
  return 0;
}

}  // namespace dyn
