// Dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for prefill and every product
// with many activation rows: y[m, n] = sum_k x[m, k] * w[n, k], f32 accumulate.
//
// One CTA computes a 128 (weight rows) x BN (activation rows, <= 256) tile of y^T:
//   * sixteen warps dequantise (four groups of four, one pipeline stage each): for every 64-wide K chunk
//     they decode the raw checkpoint blocks of the tile's 128 rows (every quantised encoding with word
//     fetches issued a step ahead and packed f16 / f32 arithmetic that rounds like the decoders of
//     codec.cuh; plain f32 / f16 / bf16 weights through those decoders) and round to f16. Q4_0, Q4_1,
//     Q8_0, MLX-U4, Q4_K, Q5_K and IQ4_XS write the A operand into tensor memory (tcgen05.st, thread =
//     weight row, column = two consecutive K elements); Q6_K and the plain types store it in shared
//     memory in the canonical K-major 128-byte-swizzled layout (8-row groups of 1024 bytes, 16-byte
//     chunk c of row r at position c ^ (r & 7));
//   * one thread of another warp fetches the matching activation chunk (f16, prepared once per call, or
//     by the caller's norm / SwiGLU kernel: TgIo) as the B operand with a 2-D TMA tile copy
//     (cp.async.bulk.tensor, hardware 128-byte swizzle);
//   * one thread of a third issues tcgen05.mma (kind::f16, M = 128, N = BN, K = 16, four per
//     chunk) with the accumulator in tensor memory, and releases each stage with tcgen05.commit;
//   * all warps (after their pipeline roles) read the accumulator back with tcgen05.ld (lane = weight row,
//     a warp reads the lanes of its own SM partition) and write y with coalesced stores.
// Stages hand over through mbarriers; every wait is bounded and reports through an error word, and
// the tensor memory is always released before the CTA exits.
//
// Precision: weights enter as f16(exact dequantised value) (relative rounding 2^-12; plain f32 / bf16
// weights are rounded the same way and must lie inside the f16 range), activations
// as f16 (bf16 inputs of ordinary magnitude convert exactly), products accumulate in f32.
#include <cuda.h>

#include <algorithm>

#include "codec.cuh"
#include "ring.cuh"

namespace dyn {

namespace {

constexpr int TG_BM = 128;          // weight rows per CTA (MMA M)
constexpr int TG_BK = 64;           // K elements per stage: 128 bytes of f16 per row
constexpr int TG_GROUPS = 4;         // producer groups; group g fills stage g with chunks g, g + 4, ...
constexpr int TG_GWARPS = 4;         // warps per group
constexpr int TG_A_WARPS = TG_GROUPS * TG_GWARPS, TG_B_WARPS = 1;
// Warp roles: warps 0..15 convert (group = warp / 4; with the A operand in tensor memory a warp converts
// the 32 weight rows of its own TMEM lane quarter, warp mod 4), warp 16 issues the activation copies,
// warp 17 the MMAs. (Moving the two service warps to an SM partition of their own changed nothing measurable.)
constexpr int TG_B_WARP = TG_A_WARPS, TG_MMA_WARP = TG_A_WARPS + 1;
constexpr int TG_WARPS = TG_A_WARPS + 2;
constexpr int TG_THREADS = TG_WARPS * 32;
__host__ __device__ constexpr bool tg_converts(int warp) { return warp < TG_A_WARPS; }
__host__ __device__ constexpr int tg_conversion_index(int warp) { return warp; }
// Encodings whose converted A operand goes to tensor memory instead of shared memory: the MMA then reads
// only B from shared memory. With both operands there a 128 x 256 x 64 chunk moves 96 KB through the
// shared-memory port (A stored + B copied in + both read by the MMAs) = 768 cycles at 128 bytes per
// cycle, more than the chunk's 512 tensor-pipe cycles.
__host__ __device__ constexpr bool tg_a_in_tmem(int enc) {
  return enc == E_Q4_0 || enc == E_Q4_1 || enc == E_Q8_0 || enc == E_MLX_U4 || enc == E_Q4_K || enc == E_Q5_K ||
         enc == E_IQ4_XS;
}
__host__ __device__ constexpr bool tg_kquant(int enc) { return enc == E_Q4_K || enc == E_Q5_K || enc == E_IQ4_XS; }
constexpr int TG_TMEM_A_COL = 256;        // first column of the A ring (32 columns per slot) behind the accumulator
constexpr int TG_RAW_WORDS = 32 * 21;     // per-warp staging of raw row words (Q5_K: 20 words per row and chunk, odd stride)
constexpr int TG_MAX_SLOTS = 2 * TG_GROUPS;  // a group owns one pipeline slot, or two when they fit
constexpr int TG_A_BYTES = TG_BM * 128;
constexpr long long TG_SPINS = 1LL << 24;

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major, 128-byte swizzle: start >> 4, LBO = 1 (unused for swizzled K-major), SBO = 1024 bytes
// between 8-row groups, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// kind::f16: D = f32, A = B = f16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TG_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory: lane = row, a 32-bit column holds two consecutive K elements.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// ---- activations -> f16 [Mpad, K] (rows >= M are zero) ------------------------------------------
// Every row is scaled by a power of two that puts its largest magnitude in [2^12, 2^13), so the
// conversion can neither overflow nor push ordinary entries into the f16 subnormals; inv_s[m]
// undoes the scale in the epilogue (exact). One block per row.
__global__ void __launch_bounds__(256)
tg_prepare_x_kernel(const void* __restrict__ x, int x_bf16, int64_t M, int64_t K, __half* xh, float* inv_s) {
  __shared__ float red[8];
  const int64_t m = blockIdx.x;
  const int tid = threadIdx.x;
  __half* dst = xh + m * K;
  if (m >= M) {
    for (int64_t i = tid * 8; i < K; i += 256 * 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
    if (tid == 0) inv_s[m] = 0.f;
    return;
  }
  auto ld = [&](int64_t i) -> float {
    return x_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(x)[m * K + i])
                  : reinterpret_cast<const float*>(x)[m * K + i];
  };
  float mx = 0.f;
  for (int64_t i = tid; i < K; i += 256) mx = fmaxf(mx, fabsf(ld(i)));
  mx = warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) mx = fmaxf(mx, red[i]);
  int e = 0;
  if (mx > 0.f && mx < 3.0e38f) frexpf(mx, &e);
  const float sc = ldexpf(1.0f, 13 - e);
  if (tid == 0) inv_s[m] = ldexpf(1.0f, e - 13);
  for (int64_t i = tid * 2; i < K; i += 512) {
    const __half2 h = __floats2half2_rn(ld(i) * sc, ld(i + 1) * sc);
    *reinterpret_cast<__half2*>(dst + i) = h;
  }
}

struct TgArgs {
  WRef w;
  const __half* xh;  // [Mpad, K]
  const float* inv_s; // [Mpad]
  int64_t M;
  int bn;            // activation rows per CTA (multiple of 16, <= 256)
  int tmem_cols;     // power of two >= bn, >= 32
  int nslot;         // pipeline slots: 4, or 8 when the stages are small enough
  float* y;          // [M, N]
  const float* residual;
  int* error;
  // K split over gridDim.z CTAs per tile (few weight-row tiles would leave most SMs idle): CTA z takes
  // chunks [z * nk_split, ...) and writes its scaled sums to partial[z][M][N]; a second pass adds them
  int nk_split;      // chunks per split (all of them when gridDim.z == 1)
  float* partial;
};

// Items of one row in a K chunk: every item is one decoder part; its groups that fall inside the
// chunk are stored.
template <int ENC>
struct ChunkItems {
  using C = Codec<ENC>;
  static constexpr int IPR = C::BLOCK <= TG_BK ? (TG_BK / C::BLOCK) * C::PARTS : 8;  // 256-element blocks: 8 parts per chunk
  __device__ static __forceinline__ void locate(int64_t k0, int it, int64_t* blk, int* part) {
    if (C::BLOCK <= TG_BK) {
      *blk = k0 / C::BLOCK + it / C::PARTS;
      *part = it % C::PARTS;
    } else {
      *blk = k0 / C::BLOCK;
      *part = (int)((k0 % C::BLOCK) / C::CHUNK_DIV) * 8 + it;
    }
  }
};

// The A producers' chunk loop for the encodings below: group `grp` converts chunks grp, grp + 4, ...
// Each chunk is converted in SUB steps; the raw words of the next step (of the group's next chunk
// after the last one) are fetched before the current step is converted, so global loads stay in
// flight during the conversion and while the group waits for its stage to drain. fetch(kc, sub, buf)
// loads, convert(kc, sub, buf, abase) stores the step's f16 weights into the stage.
template <int NR, int SUB, class Fetch, class Convert>
__device__ __forceinline__ void tg_produce_chunks(int grp, int nk, int nslot, uint8_t* smem, uint32_t stage_bytes,
                                                  uint64_t* empty_bar, uint64_t* full_bar, int* s_abort, int lane,
                                                  Fetch fetch, Convert convert) {
  constexpr int U = SUB == 1 ? 2 : 1;  // chunks per loop body, so that the buffer index is static
  static_assert(SUB == 1 || SUB % 2 == 0, "steps per chunk: one or an even number");
  const int slot_shift = nslot == TG_GROUPS ? 2 : 3;
  uint32_t buf[2][NR];
  if (grp < nk) fetch(grp, 0, buf[0]);
  bool live = true;
  for (int kc0 = grp; kc0 < nk && live; kc0 += U * TG_GROUPS) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int kc = kc0 + u * TG_GROUPS;
      if (kc >= nk) break;
      const int slot = (kc & (nslot - 1));
      uint8_t* abase = smem + (size_t)slot * stage_bytes;
#pragma unroll
      for (int sub = 0; sub < SUB; sub++) {
        const int b = (u * SUB + sub) & 1;
        if (sub + 1 < SUB)
          fetch(kc, sub + 1, buf[b ^ 1]);
        else if (kc + TG_GROUPS < nk)
          fetch(kc + TG_GROUPS, 0, buf[b ^ 1]);
        if (sub == 0 && kc >= nslot &&
            !mbar_wait_bounded(empty_bar + slot, (unsigned)((kc >> slot_shift) - 1) & 1u, TG_SPINS, s_abort)) {
          if (!*s_abort) *s_abort = 1;
          live = false;
          break;
        }
        convert(kc, sub, buf[b], abase);
      }
      if (!live) break;
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar + slot);
    }
  }
}

template <int ENC>
__global__ void __launch_bounds__(TG_THREADS, 1)
dqgemm_tc_kernel(const TgArgs a, const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ __align__(1024) uint8_t tg_smem[];
  __shared__ uint64_t full_bar[TG_MAX_SLOTS], empty_bar[TG_MAX_SLOTS], accum_bar;
  const int nslot = a.nslot;  // TG_GROUPS or 2 * TG_GROUPS (powers of two); chunk kc uses slot kc mod nslot and belongs to group kc mod TG_GROUPS
  const int slot_shift = nslot == TG_GROUPS ? 2 : 3;
  static_assert(TG_GROUPS == 4, "slot_shift assumes four or eight slots");
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;
  __shared__ float s_inv[256];  // inverse activation-row scales of this tile
  using C = Codec<ENC>;
  using CI = ChunkItems<ENC>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bn = a.bn;
  const int64_t N = a.w.rows, K = a.w.cols;
  const int64_t n0 = (int64_t)blockIdx.x * TG_BM, m0 = (int64_t)blockIdx.y * bn;
  const int kbase = (int)blockIdx.z * a.nk_split;  // first chunk of this CTA's share of K
  const int nk = min(a.nk_split, (int)(K / TG_BK) - kbase);
  constexpr bool AT = tg_a_in_tmem(ENC);
  constexpr uint32_t A_BYTES = AT ? 0u : (uint32_t)TG_A_BYTES;  // shared-memory bytes of a stage's A operand
  const uint32_t stage_bytes = A_BYTES + (uint32_t)bn * 128;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tg_smem) + 1023) & ~uintptr_t(1023));

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < TG_MAX_SLOTS; i++) {
      mbar_init(full_bar + i, TG_GWARPS + TG_B_WARPS);
      mbar_init(empty_bar + i, 1);
    }
    mbar_init(&accum_bar, 1);
    mbar_fence_init();
  }
  if (warp == TG_MMA_WARP) {  // the MMA warp owns the tensor memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)a.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base_s;

  if (tg_converts(warp)) {
    // ---------------- A producers: dequantise 128 rows x 64 k per stage --------------------------
    // Four groups of four warps; group g produces chunks g, g + 4, ... into stage g, so the fixed
    // costs of a hand-over (proxy fence, barrier round trip) of up to four chunks overlap.
    const int pw = tg_conversion_index(warp);
    const int grp = pw / TG_GWARPS, wg = pw % TG_GWARPS;
    if constexpr (AT && tg_kquant(ENC)) {
      // 256-weight blocks (Q4_K, Q5_K, IQ4_XS) with the A operand in tensor memory, thread = row as below.
      // A 64-wide chunk is one quarter of a block: the block's header words (d, dmin / scales) plus the
      // quarter's 32 index bytes (Q5_K: plus the block's 32 high-bit bytes):
      //   Q4_K   12 words: 4 header + quant words 4 + 8 jj ..; Q5_K 20 words: 4 header + 8 high-bit + 12 + 8 jj ..
      //   IQ4_XS 10 words: 2 header + index words 2 + 8 c ..
      // The values are computed in f32 exactly as the decoders of codec.cuh do (each product and the
      // difference rounded on its own; index -> f32 through 0x4B000000 | q), then rounded to f16.
      constexpr int HW = ENC == E_Q4_K ? 4 : ENC == E_Q5_K ? 12 : 2;      // words taken from the block's start
      constexpr int WPR = HW + 8, RS = WPR | 1, BW = Codec<ENC>::BYTES / 4;
      static_assert(32 * RS <= TG_RAW_WORDS, "per-warp scratch");
      const int quarter = warp & 3;
      const int64_t rw = a.w.row_bytes() / 4;
      const uint32_t* wbase = reinterpret_cast<const uint32_t*>(a.w.data);
      uint32_t* raw = reinterpret_cast<uint32_t*>(smem + (size_t)nslot * stage_bytes) + warp * TG_RAW_WORDS;
      const int64_t last = N - 1 - (n0 + quarter * 32);
      auto fetch = [&](int kc, int, uint32_t (&q)[WPR]) {
        const int64_t k0 = (int64_t)(kbase + kc) * TG_BK;
        const uint32_t* cb = wbase + (k0 >> 8) * BW;
        const int qoff = HW + 8 * (int)((k0 >> 6) & 3) - HW;  // quarter's index words start HW + 8 * quarter words in
#pragma unroll
        for (int it = 0; it < WPR; it++) {
          const int idx = it * 32 + lane, r = idx / WPR, w = idx - r * WPR;
          q[it] = cb[(n0 + quarter * 32 + (r < last ? r : last)) * rw + (w < HW ? w : w + qoff)];
        }
      };
      auto h2u = [](__half2 v) { return *reinterpret_cast<uint32_t*>(&v); };
      auto convert = [&](int kc, int, uint32_t (&q)[WPR], uint8_t*) {
#pragma unroll
        for (int it = 0; it < WPR; it++) {
          const int idx = it * 32 + lane, r = idx / WPR;
          raw[r * RS + (idx - r * WPR)] = q[it];
        }
        __syncwarp();
        const uint32_t* me = raw + lane * RS;
        const int jj = (kbase + kc) & 3;  // which quarter of the block
        const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + TG_TMEM_A_COL + (uint32_t)(kc & (nslot - 1)) * 32u;
        const uint32_t h0 = me[0];
        const float d = f16_bits_to_f32(h0 & 0xffffu);
#pragma unroll
        for (int h = 0; h < 2; h++) {
          uint32_t out[16];
          if constexpr (ENC == E_IQ4_XS) {
            const int ib = 2 * jj + h;
            const uint32_t ls = ((me[1] >> (4 * ib)) & 15u) | ((((h0 >> 16) >> (2 * ib)) & 3u) << 4);
            const float dl = __fmul_rn(d, (float)((int)ls - 32));
#pragma unroll
            for (int wq = 0; wq < 4; wq++) {
              const uint32_t x = me[HW + 4 * h + wq];
              float lo[4], hi[4];
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint32_t byte = (x >> (8 * i)) & 0xffu;
                lo[i] = __fmul_rn(dl, iq4_value(byte & 15u));
                hi[i] = __fmul_rn(dl, iq4_value(byte >> 4));
              }
              out[2 * wq] = h2u(__floats2half2_rn(lo[0], lo[1])), out[2 * wq + 1] = h2u(__floats2half2_rn(lo[2], lo[3]));
              out[8 + 2 * wq] = h2u(__floats2half2_rn(hi[0], hi[1])), out[8 + 2 * wq + 1] = h2u(__floats2half2_rn(hi[2], hi[3]));
            }
          } else {
            // sub-block j = 2 jj + h: 6-bit scale and minimum out of the 12 packed bytes (words 1..3)
            const int j = 2 * jj + h;
            auto sb = [&](int i) { return (me[1 + (i >> 2)] >> (8 * (i & 3))) & 0xffu; };
            uint32_t sc, mn;
            if (j < 4) {
              sc = sb(j) & 63u, mn = sb(j + 4) & 63u;
            } else {
              sc = (sb(j + 4) & 15u) | ((sb(j - 4) >> 6) << 4);
              mn = (sb(j + 4) >> 4) | ((sb(j) >> 6) << 4);
            }
            const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(f16_bits_to_f32(h0 >> 16), (float)mn);
#pragma unroll
            for (int wq = 0; wq < 8; wq++) {
              uint32_t v = (me[HW + wq] >> (4 * h)) & 0x0F0F0F0Fu;
              if constexpr (ENC == E_Q5_K) v |= ((me[4 + wq] >> j) & 0x01010101u) << 4;
              float f[4];
              f[0] = __fsub_rn(__fmul_rn(ds, __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440)) - 8388608.f), dm);
              f[1] = __fsub_rn(__fmul_rn(ds, __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7441)) - 8388608.f), dm);
              f[2] = __fsub_rn(__fmul_rn(ds, __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7442)) - 8388608.f), dm);
              f[3] = __fsub_rn(__fmul_rn(ds, __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7443)) - 8388608.f), dm);
              out[2 * wq] = h2u(__floats2half2_rn(f[0], f[1])), out[2 * wq + 1] = h2u(__floats2half2_rn(f[2], f[3]));
            }
          }
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
              ::"r"(taddr + 16u * h), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]),
                "r"(out[7]), "r"(out[8]), "r"(out[9]), "r"(out[10]), "r"(out[11]), "r"(out[12]), "r"(out[13]), "r"(out[14]), "r"(out[15])
              : "memory");
        }
        __syncwarp();  // the scratch is read; the next chunk may overwrite it
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
      };
      tg_produce_chunks<WPR, 1>(grp, nk, nslot, smem, stage_bytes, empty_bar, full_bar, &s_abort, lane, fetch, convert);
    } else if constexpr (AT) {
      // A operand in tensor memory. A warp converts the 32 rows of its lane quarter: thread = row, the
      // chunk's 64 weights of a row = 32 packed columns (column c = weights 2c, 2c + 1), written with one
      // tcgen05.st. The raw words of the next chunk are fetched a step ahead with coalesced loads (lane i
      // of pass p holds word 32 p + i of the warp's 32 rows x WPR words) and turned to "thread = row"
      // through a per-warp scratch in shared memory (odd row stride: conflict-free both ways).
      //   Q4_0  9 words: d | 16 quant bytes from byte 2; second block from byte 18 (d = high half of word 4)
      //   Q4_1 10 words: (d, m), 4 quant words, twice
      //   Q8_0 17 words: d | 32 int8 from byte 2; second block from byte 34 (d = high half of word 8)
      //   MLX-U4 8 words (word j = weights 8j..8j+7, nibble k = bits [4k, 4k+4)) + the scale and bias of
      //          the chunk's two 32-weight halves (groups are powers of two >= 32)
      // The arithmetic is that of the shared-memory producers: q | 0x6400 = 1024 + q in f16, reduced to q
      // exactly, then one rounding for q * d (+ m) or q * scale + bias.
      constexpr int WPR = ENC == E_Q4_0 ? 9 : ENC == E_Q4_1 ? 10 : ENC == E_Q8_0 ? 17 : 8;
      constexpr int RS = WPR | 1;
      constexpr int NX = ENC == E_MLX_U4 ? 4 : 0;
      static_assert(32 * RS <= TG_RAW_WORDS, "per-warp scratch");
      const int quarter = warp & 3;
      const int64_t rw = ENC == E_MLX_U4 ? K / 8 : a.w.row_bytes() / 4;
      const uint32_t* wbase = reinterpret_cast<const uint32_t*>(a.w.data);
      uint32_t* raw = reinterpret_cast<uint32_t*>(smem + (size_t)nslot * stage_bytes) + warp * TG_RAW_WORDS;
      const int64_t last = N - 1 - (n0 + quarter * 32);  // rows past the matrix repeat its last row (never stored)
      // MLX: this thread's own row of scales and biases
      const int ael = a.w.aux == E_F32 ? 4 : 2;
      int gshift = 5;
      const uint8_t *scp = nullptr, *bip = nullptr;
      if constexpr (ENC == E_MLX_U4) {
        while ((1 << gshift) < a.w.group) gshift++;
        const int64_t row = n0 + quarter * 32 + (lane < last ? lane : last);
        scp = a.w.scales + row * (K >> gshift) * ael;
        bip = a.w.biases + row * (K >> gshift) * ael;
      }
      auto fetch = [&](int kc, int, uint32_t (&q)[WPR + NX]) {
        const uint32_t* cb = wbase + (int64_t)(kbase + kc) * WPR;
#pragma unroll
        for (int it = 0; it < WPR; it++) {
          const int idx = it * 32 + lane, r = idx / WPR;
          q[it] = cb[(n0 + quarter * 32 + (r < last ? r : last)) * rw + (idx - r * WPR)];
        }
        if constexpr (ENC == E_MLX_U4) {
          const int64_t k0 = (int64_t)(kbase + kc) * TG_BK;
          q[WPR] = __float_as_uint(aux_load(scp, a.w.aux, k0 >> gshift));
          q[WPR + 1] = __float_as_uint(aux_load(bip, a.w.aux, k0 >> gshift));
          if (gshift > 5) {  // one group covers the whole chunk
            q[WPR + 2] = q[WPR], q[WPR + 3] = q[WPR + 1];
          } else {
            q[WPR + 2] = __float_as_uint(aux_load(scp, a.w.aux, (k0 + 32) >> gshift));
            q[WPR + 3] = __float_as_uint(aux_load(bip, a.w.aux, (k0 + 32) >> gshift));
          }
        }
      };
      const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f), c72 = __floats2half2_rn(72.f, 72.f);
      const __half2 c16th = __floats2half2_rn(0.0625f, 0.0625f), c1024 = __floats2half2_rn(1024.f, 1024.f);
      const __half2 c64n = __floats2half2_rn(-64.f, -64.f), c1152 = __floats2half2_rn(1152.f, 1152.f);
      auto h2u = [](__half2 v) { return *reinterpret_cast<uint32_t*>(&v); };
      auto u2h = [](uint32_t v) { return *reinterpret_cast<__half2*>(&v); };
      auto convert = [&](int kc, int, uint32_t (&q)[WPR + NX], uint8_t*) {
#pragma unroll
        for (int it = 0; it < WPR; it++) {
          const int idx = it * 32 + lane, r = idx / WPR;
          raw[r * RS + (idx - r * WPR)] = q[it];
        }
        __syncwarp();
        // one 32-weight half of the chunk at a time (its words w[0..NW) of the row): 16 columns per tcgen05.st
        constexpr int NW = ENC == E_Q8_0 ? 9 : ENC == E_MLX_U4 ? 4 : 5, WSTEP = ENC == E_Q4_1 ? 5 : NW - (ENC == E_MLX_U4 ? 0 : 1);
        const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + TG_TMEM_A_COL + (uint32_t)(kc & (nslot - 1)) * 32u;
#pragma unroll
        for (int b = 0; b < 2; b++) {
          uint32_t w[NW];
#pragma unroll
          for (int i = 0; i < NW; i++) w[i] = raw[lane * RS + b * WSTEP + i];
          uint32_t out[16];
          if constexpr (ENC == E_Q4_0 || ENC == E_Q4_1) {
            const uint32_t dm = ENC == E_Q4_1 ? w[0] : (b ? w[0] >> 16 : w[0] & 0xffffu);
            const __half dh = __ushort_as_half((unsigned short)(dm & 0xffffu));
            const __half mh = __ushort_as_half((unsigned short)(dm >> 16));
            const __half2 d2 = __halves2half2(dh, dh), m2 = __halves2half2(mh, mh);
#pragma unroll
            for (int t = 0; t < 4; t++) {
              const uint32_t x = ENC == E_Q4_1 || b ? w[1 + t] : __funnelshift_r(w[t], w[t + 1], 16);
              uint32_t l02 = (x & 0x000F000Fu) | 0x64006400u, l13 = ((x >> 8) & 0x000F000Fu) | 0x64006400u;
              uint32_t h02 = (x & 0x00F000F0u) | 0x64006400u, h13 = ((x >> 8) & 0x00F000F0u) | 0x64006400u;
              if constexpr (ENC == E_Q4_0) {  // (q - 8) * d
                l02 = h2u(__hmul2(__hsub2(u2h(l02), c1032), d2));
                l13 = h2u(__hmul2(__hsub2(u2h(l13), c1032), d2));
                h02 = h2u(__hmul2(__hsub2(__hmul2(u2h(h02), c16th), c72), d2));
                h13 = h2u(__hmul2(__hsub2(__hmul2(u2h(h13), c16th), c72), d2));
              } else {  // q * d + m
                l02 = h2u(__hfma2(__hsub2(u2h(l02), c1024), d2, m2));
                l13 = h2u(__hfma2(__hsub2(u2h(l13), c1024), d2, m2));
                h02 = h2u(__hfma2(__hfma2(u2h(h02), c16th, c64n), d2, m2));
                h13 = h2u(__hfma2(__hfma2(u2h(h13), c16th, c64n), d2, m2));
              }
              // weights 4t..4t+3 (low nibbles) and 16+4t..16+4t+3 (high nibbles) of the block
              out[2 * t] = __byte_perm(l02, l13, 0x5410);
              out[2 * t + 1] = __byte_perm(l02, l13, 0x7632);
              out[8 + 2 * t] = __byte_perm(h02, h13, 0x5410);
              out[8 + 2 * t + 1] = __byte_perm(h02, h13, 0x7632);
            }
          } else if constexpr (ENC == E_Q8_0) {
            const __half dh = __ushort_as_half((unsigned short)(b ? w[0] >> 16 : w[0] & 0xffffu));
            const __half2 d2 = __halves2half2(dh, dh);
#pragma unroll
            for (int t = 0; t < 8; t++) {
              const uint32_t x = (b ? w[1 + t] : __funnelshift_r(w[t], w[t + 1], 16)) ^ 0x80808080u;
              out[2 * t] = h2u(__hmul2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4140)), c1152), d2));
              out[2 * t + 1] = h2u(__hmul2(__hsub2(u2h(__byte_perm(x, 0x64646464u, 0x4342)), c1152), d2));
            }
          } else {
            const __half2 s2 = __float2half2_rn(__uint_as_float(q[WPR + 2 * b]));
            const __half2 b2 = __float2half2_rn(__uint_as_float(q[WPR + 2 * b + 1]));
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t x = w[j];
              const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;  // nibbles 0,2,4,6 / 1,3,5,7
#pragma unroll
              for (int e = 0; e < 4; e++) {
                const uint32_t pr = (__byte_perm(lo, hi, 0x0400 + 0x0101 * e) & 0x00FF00FFu) | 0x64006400u;  // (n 2e, n 2e+1)
                out[4 * j + e] = h2u(__hfma2(__hsub2(u2h(pr), c1024), s2, b2));
              }
            }
          }
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
              ::"r"(taddr + 16u * b), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]),
                "r"(out[7]), "r"(out[8]), "r"(out[9]), "r"(out[10]), "r"(out[11]), "r"(out[12]), "r"(out[13]), "r"(out[14]), "r"(out[15])
              : "memory");
        }
        __syncwarp();  // the scratch is read; the next chunk may overwrite it
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
      };
      tg_produce_chunks<WPR + NX, 1>(grp, nk, nslot, smem, stage_bytes, empty_bar, full_bar, &s_abort, lane, fetch, convert);
    } else if constexpr (ENC == E_Q6_K) {
      // Q6_K: a 64-wide chunk is one quarter (n, h) of a 210-byte block: nibble h of ql bytes
      // 64 n .. 64 n + 63 and bit field 2 h + p of qh bytes 32 n .. 32 n + 31 (p = 0: the chunk's first 32
      // weights, p = 1: the last 32). Lane = (row sub-index, j4): 4 ql bytes at 4 j4 and at 32 + 4 j4,
      // 4 qh bytes, the two sub-block scales and d -> weights 4 j4..+3 and 32 + 4 j4..+3. Blocks are only
      // 2-byte aligned, so every word is fetched as two halves. A chunk is converted two rows at a
      // time. q - 32 is made exact in f32 (byte under 0x4B000000 = 2^23 + q) and multiplied by the exact
      // f32 product scale * d: one f32 rounding of (q - 32) * scale * d, the value the decoder defines.
      constexpr int NJ = TG_BM / (TG_GWARPS * 4), RB = 2, SUB = NJ / RB;
      const int j4 = lane & 7, rsub = lane >> 3;
      const int64_t rb = a.w.row_bytes();
      auto row_of = [&](int j) {
        int64_t row = n0 + wg * 4 + rsub + 16 * j;
        return row > N - 1 ? N - 1 : row;
      };
      auto fetch = [&](int kc, int sub, uint32_t (&q)[9 * RB]) {
        const int64_t k0 = (int64_t)(kbase + kc) * TG_BK;
        const int64_t blk = k0 >> 8;
        const int n = (int)(k0 >> 7) & 1, h = (int)(k0 >> 6) & 1;
#pragma unroll
        for (int i = 0; i < RB; i++) {
          const uint8_t* b = a.w.data + row_of(sub * RB + i) * rb + blk * 210;
          const unsigned short* ql = reinterpret_cast<const unsigned short*>(b + n * 64 + 4 * j4);
          const unsigned short* qh = reinterpret_cast<const unsigned short*>(b + 128 + n * 32 + 4 * j4);
          const uint8_t* sc = b + 192 + n * 8 + h * 4 + (j4 >> 2);
          q[9 * i] = ql[0], q[9 * i + 1] = ql[1];
          q[9 * i + 2] = ql[16], q[9 * i + 3] = ql[17];
          q[9 * i + 4] = qh[0], q[9 * i + 5] = qh[1];
          q[9 * i + 6] = sc[0], q[9 * i + 7] = sc[2];
          q[9 * i + 8] = *reinterpret_cast<const unsigned short*>(b + 208);
        }
      };
      auto convert = [&](int kc, int sub, uint32_t (&q)[9 * RB], uint8_t* abase) {
        const int h = (kbase + kc) & 1;
#pragma unroll
        for (int i = 0; i < RB; i++) {
          const int r = wg * 4 + rsub + 16 * (sub * RB + i);
          const uint32_t ql0 = q[9 * i] | (q[9 * i + 1] << 16), ql1 = q[9 * i + 2] | (q[9 * i + 3] << 16);
          const uint32_t qh = (q[9 * i + 4] | (q[9 * i + 5] << 16)) >> (4 * h);
          const float d = __half2float(__ushort_as_half((unsigned short)q[9 * i + 8]));
          const float sd0 = __fmul_rn((float)(int)(int8_t)q[9 * i + 6], d);
          const float sd1 = __fmul_rn((float)(int)(int8_t)q[9 * i + 7], d);
          const uint32_t v0 = ((ql0 >> (4 * h)) & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4);
          const uint32_t v1 = ((ql1 >> (4 * h)) & 0x0F0F0F0Fu) | (((qh >> 2) & 0x03030303u) << 4);
          auto four = [&](uint32_t v, float sd) {
            float f[4];
            f[0] = __fmul_rn(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440)) - 8388640.f, sd);
            f[1] = __fmul_rn(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7441)) - 8388640.f, sd);
            f[2] = __fmul_rn(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7442)) - 8388640.f, sd);
            f[3] = __fmul_rn(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7443)) - 8388640.f, sd);
            const __half2 a01 = __floats2half2_rn(f[0], f[1]), a23 = __floats2half2_rn(f[2], f[3]);
            return make_uint2(*reinterpret_cast<const uint32_t*>(&a01), *reinterpret_cast<const uint32_t*>(&a23));
          };
          const int klo = 4 * j4, khi = 32 + 4 * j4;
          uint8_t* rowbase = abase + r * 128;
          *reinterpret_cast<uint2*>(rowbase + (((klo >> 3) ^ (r & 7)) << 4) + (klo & 7) * 2) = four(v0, sd0);
          *reinterpret_cast<uint2*>(rowbase + (((khi >> 3) ^ (r & 7)) << 4) + (khi & 7) * 2) = four(v1, sd1);
        }
      };
      tg_produce_chunks<9 * RB, SUB>(grp, nk, nslot, smem, stage_bytes, empty_bar, full_bar, &s_abort, lane, fetch, convert);
    } else {
      constexpr int RPP = 32 / CI::IPR;  // rows per warp pass
      const int it = lane % CI::IPR, rsub = lane / CI::IPR;
      for (int kc = grp; kc < nk; kc += TG_GROUPS) {
        const int slot = (kc & (nslot - 1));
        uint8_t* abase = smem + (size_t)slot * stage_bytes;
        if (kc >= nslot && !mbar_wait_bounded(empty_bar + slot, (unsigned)((kc >> slot_shift) - 1) & 1u, TG_SPINS, &s_abort)) {
          if (!s_abort) s_abort = 1;
          break;
        }
        const int64_t k0 = (int64_t)(kbase + kc) * TG_BK;
        int64_t blk;
        int part;
        CI::locate(k0, it, &blk, &part);
        for (int r = wg * RPP + rsub; r < TG_BM; r += TG_GWARPS * RPP) {
          int64_t row = n0 + r;
          if (row > N - 1) row = N - 1;
          const RowPtr rp = row_ptr(a.w, row);
          float wv[4 * C::G];
          C::decode(rp, blk, part, wv);
#pragma unroll
          for (int g = 0; g < C::G; g++) {
            const int koff = (int)(blk * C::BLOCK + C::xoff(part, g) - k0);
            if (koff >= 0 && koff < TG_BK) {
              const __half2 h0 = __floats2half2_rn(wv[4 * g], wv[4 * g + 1]);
              const __half2 h1 = __floats2half2_rn(wv[4 * g + 2], wv[4 * g + 3]);
              const int c = koff >> 3;
              uint8_t* dst = abase + r * 128 + ((c ^ (r & 7)) << 4) + (koff & 7) * 2;
              *reinterpret_cast<uint2*>(dst) =
                  make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
            }
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar + slot);
      }
    }
  } else if (warp == TG_B_WARP) {
    // ---------------- B producer: one TMA tile (bn rows x 64 k, swizzled by the hardware) per stage -----
    if (lane == 0) {
      int slot = 0;
      unsigned phase = 1;  // parity of the drain that frees a slot for its next chunk; the first round waits for none
      uint8_t* dst = smem + A_BYTES;
      for (int kc = 0; kc < nk; kc++) {
        if (kc >= nslot && !mbar_wait_bounded(empty_bar + slot, phase, TG_SPINS, &s_abort)) {
          if (!s_abort) s_abort = 1;
          break;
        }
        mbar_expect_tx(full_bar + slot, (unsigned)bn * 128u);
        tma_load_2d(dst, &xmap, (kbase + kc) * TG_BK, (int)m0, full_bar + slot);
        slot++, dst += stage_bytes;
        if (slot == nslot) slot = 0, dst = smem + A_BYTES, phase ^= 1u;
      }
    }
  } else if (warp == TG_MMA_WARP) {
    // ---------------- MMA issue: one thread ---------------------------------------------------------
    if (lane == 0) {
      // This one thread is the pipeline's serial section: every instruction between two chunks' MMAs
      // delays all of them, so slot, phase and the operand descriptors advance by additions only (no
      // division by the runtime slot count, no descriptor rebuilt per MMA: 16 K elements further along
      // a swizzled K-major row is +32 bytes = +2 in the descriptor's address field).
      const uint32_t idesc = umma_idesc(bn);
      const uint32_t smem0 = smem_u32(smem);
      uint32_t aaddr = smem0, accumulate = 0u;
      int slot = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int kc = 0; kc < nk && ok; kc++) {
        ok = mbar_wait_bounded(full_bar + slot, phase, TG_SPINS, &s_abort);
        if (!ok) {
          if (!s_abort) s_abort = 2;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = umma_desc(aaddr), bdesc = umma_desc(aaddr + A_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < TG_BK / 16; k4++) {
          if constexpr (AT)
            umma_f16_ts(tmem_d, tmem_d + TG_TMEM_A_COL + (uint32_t)slot * 32u + 8u * k4, bdesc + 2 * k4, idesc, accumulate);
          else
            umma_f16(tmem_d, adesc + 2 * k4, bdesc + 2 * k4, idesc, accumulate);
          accumulate = 1u;
        }
        umma_commit(empty_bar + slot);  // frees the stage once these MMAs have read it
        slot++, aaddr += stage_bytes;
        if (slot == nslot) slot = 0, aaddr = smem0, phase ^= 1u;
      }
      umma_commit(&accum_bar);  // accumulator complete (also reached after a failed wait)
    }
  }

  // ---------------- epilogue: every warp, TMEM lane = weight row ---------------------------------------
  // A warp reads the 32 accumulator lanes of its SM partition (warp index mod 4), sixteen columns
  // (activation rows) per tcgen05.ld, and stores them scaled: one store = 32 consecutive weight rows of
  // one activation row = 128 bytes. The four or five warps of a partition take the sixteen-column blocks in
  // turn: with one warp per partition every instruction of the store loop paid its full issue latency
  // (measured ~150 cycles per column, 40 % of the kernel on a 256-column tile). Addresses advance by
  // additions; the rows' inverse scales wait in shared memory; a block's residual values are all loaded
  // before its first store (y may be the residual's own buffer).
  {
    __syncwarp();  // the issuing lanes of the MMA and copy warps rejoin here
    for (int j = tid; j < bn; j += TG_THREADS) s_inv[j] = m0 + j < a.M ? __ldg(a.inv_s + m0 + j) : 0.f;
    __syncthreads();
    const bool ok = mbar_wait_bounded(&accum_bar, 0, TG_SPINS, &s_abort);
    if (!ok && !s_abort) s_abort = 3;
    tc_fence_after();
    const int quarter = warp & 3;
    const int64_t n = n0 + quarter * 32 + lane;
    if (ok && !s_abort) {
      const uint32_t tbase = tmem_d + ((uint32_t)(quarter * 32) << 16);
      const bool split = gridDim.z > 1;
      float* const out = (split ? a.partial + (int64_t)blockIdx.z * a.M * N : a.y) + m0 * N + n;
      const float* const res = split || !a.residual ? nullptr : a.residual + m0 * N + n;
      const int mleft = (int)min((int64_t)bn, a.M - m0);  // live activation rows of this tile
      const int quarter_warps = (TG_WARPS - quarter + 3) / 4;
      for (int j0 = (warp >> 2) * 16; j0 < mleft; j0 += quarter_warps * 16) {
        uint32_t v[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(tbase + (uint32_t)j0));
        float r[16];
        if (res && n < N) {
          const float* rp = res + (int64_t)j0 * N;
#pragma unroll
          for (int j = 0; j < 16; j++) {
            r[j] = j0 + j < mleft ? *rp : 0.f;
            rp += N;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; j++) r[j] = 0.f;
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < N) {
          float* p = out + (int64_t)j0 * N;
#pragma unroll
          for (int j = 0; j < 16; j++) {
            if (j0 + j < mleft) *p = __fadd_rn(__fmul_rn(__uint_as_float(v[j]), s_inv[j0 + j]), r[j]);
            p += N;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == TG_MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)a.tmem_cols)
                 : "memory");
  }
  if (tid == 0 && s_abort) report_wait_expired(a.error, DEV_ERR_GEMM_PIPE);
}

bool tg_shape_ok(const WRef& w, int64_t M) {
  switch (w.enc) {
    case E_Q4_0:
    case E_Q4_1:
    case E_Q8_0:
    case E_MLX_U4:
    case E_Q6_K:
    case E_Q4_K:
    case E_Q5_K:
    case E_IQ4_XS:
    case E_F32:
    case E_F16:
    case E_BF16: break;
    default: return false;
  }
  // MLX-U4: a 64-wide chunk takes one scale and bias per 32-weight half
  if (w.enc == E_MLX_U4 && (w.group < 32 || (w.group & (w.group - 1)) || w.cols % w.group)) return false;
  // the word-fetching producers read aligned 32-bit words (Q6_K: 16-bit halves)
  const uintptr_t addr = reinterpret_cast<uintptr_t>(w.data);
  if ((w.enc == E_Q4_0 || w.enc == E_Q4_1 || w.enc == E_Q8_0 || w.enc == E_MLX_U4 || tg_kquant(w.enc)) && (addr & 3))
    return false;
  if (w.enc == E_Q6_K && (addr & 1)) return false;
  return M >= 1 && w.rows >= 1 && w.cols >= TG_BK && w.cols % (enc_block_elems(w.enc) == 256 ? 256 : TG_BK) == 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D map over the f16 activations [rows, K]: boxes of 64 k x bn rows, 128-byte swizzle.
int tg_make_xmap(__half* xh, int64_t rows, int64_t K, int bn, CUtensorMap* map) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    DYN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    DYN_CHECK(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TG_BK, (cuuint32_t)bn};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DYN_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

// y = sum over the K splits (fixed order) + residual
__global__ void __launch_bounds__(256)
tg_split_reduce_kernel(const float* __restrict__ partial, int splits, int64_t count, float* y, const float* residual) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= count) return;
  float v = 0.f;
  for (int z = 0; z < splits; z++) v += partial[(int64_t)z * count + i];
  if (residual) v += residual[i];
  y[i] = v;
}

template <int ENC>
int tg_launch(const TgArgs& a, const CUtensorMap& xmap, dim3 grid, size_t smem, cudaStream_t s) {
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(dqgemm_tc_kernel<ENC>), 200 * 1024)) return 1;
  dqgemm_tc_kernel<ENC><<<grid, TG_THREADS, smem, s>>>(a, xmap);
  return 0;
}

// Scratch of one product: the caller's region when it is large enough (a session's own scratch:
// no allocation nodes inside a captured step), else the stream-ordered allocator. Freed on every
// path by the destructor.
struct TgScratch {
  uint8_t* ptr = nullptr;
  bool pooled = false;
  cudaStream_t s;
  explicit TgScratch(cudaStream_t st) : s(st) {}
  int take(size_t bytes) {
    ptr = reinterpret_cast<uint8_t*>(thread_scratch(bytes));
    if (ptr) return 0;
    if (keep_scratch_pool_cached()) return 1;
    DYN_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&ptr), bytes, s));
    pooled = true;
    return 0;
  }
  ~TgScratch() {
    if (pooled && ptr) cudaFreeAsync(ptr, s);
  }
};

}  // namespace

namespace {
struct TgPlan {
  int64_t mtiles, Mpad;
  int bn, cols, splits, nk_split;
};
// activation rows per CTA: as many as fit one accumulator (256), rounded up to the MMA granule.
// Few weight-row tiles would leave most SMs idle: K is split first (at least 4 chunks = 256 elements
// per CTA, at most 8 ways; the CTAs of a split dequantise disjoint parts of the tile, a second pass
// adds their sums), and only a product whose K cannot be split gets narrower activation tiles, down
// to 32 rows (each of those re-dequantises the whole weight tile: measured 116 us against 91 us with
// the K split on 4096 x 12288 x 512)
TgPlan tg_plan(const WRef& w, int64_t M) {
  const int sms = std::max(1, sm_count());
  const int64_t ntiles = (w.rows + TG_BM - 1) / TG_BM;
  const int nk_all = (int)(w.cols / TG_BK);
  auto k_splits = [&](int64_t ctas) {
    int sp = 1;
    while (sp < 8 && ctas * (sp * 2) <= sms && nk_all / (sp * 2) >= 4) sp *= 2;
    return sp;
  };
  int64_t cap_rows = 256;
  if (k_splits(ntiles * ((M + 255) / 256)) == 1)
    while (cap_rows > 32 && ntiles * ((M + cap_rows / 2 - 1) / (cap_rows / 2)) <= sms) cap_rows /= 2;  // stay within one wave
  TgPlan p;
  p.mtiles = (M + cap_rows - 1) / cap_rows;
  p.bn = (int)((M + p.mtiles - 1) / p.mtiles);
  p.bn = (p.bn + 15) / 16 * 16;
  p.Mpad = p.mtiles * p.bn;
  p.cols = 32;
  while (p.cols < p.bn) p.cols *= 2;
  p.splits = k_splits(ntiles * p.mtiles);
  p.nk_split = (nk_all + p.splits - 1) / p.splits;
  p.splits = (nk_all + p.nk_split - 1) / p.nk_split;
  return p;
}
}  // namespace

bool dqgemm_tc_takes(const WRef& w, int64_t M) { return tg_shape_ok(w, M); }
int64_t dqgemm_tc_padded_rows(const WRef& w, int64_t M) { return tg_shape_ok(w, M) ? tg_plan(w, M).Mpad : 0; }

// Tensor-core dequant GEMM. *handled = false when the encoding or shape does not qualify.
int launch_dqgemm_tc(const WRef& w, const void* x, int x_type, int64_t M, float* y, const float* residual,
                     cudaStream_t s, bool* handled, TgIo* io) {
  *handled = false;
  if (io) io->splits = 0;
  if (!tg_shape_ok(w, M)) return 0;
  const int64_t K = w.cols;
  const TgPlan pl = tg_plan(w, M);
  const int64_t mtiles = pl.mtiles, Mpad = pl.Mpad;
  const int bn = pl.bn, cols = pl.cols, nk_split = pl.nk_split;
  int splits = pl.splits;
  const bool prepared = io && io->xh;
  DYN_CHECK(!prepared || Mpad <= io->rows_alloc, "dequant GEMM: %lld prepared rows, %lld needed", (long long)(io ? io->rows_alloc : 0),
            (long long)Mpad);
  const size_t part_need = splits > 1 ? (size_t)splits * M * w.rows * 4 : 0;
  const bool part_out = io && io->partial && part_need && part_need <= io->partial_bytes;  // the caller adds the sums
  const size_t xh_bytes = prepared ? 0 : ((size_t)Mpad * K * 2 + 255) / 256 * 256;
  const size_t inv_bytes = prepared ? 0 : ((size_t)Mpad * 4 + 255) / 256 * 256;
  const size_t part_bytes = part_out ? 0 : part_need;
  TgScratch ws(s);
  if (xh_bytes + inv_bytes + part_bytes && ws.take(xh_bytes + inv_bytes + part_bytes)) return 1;
  const __half* xh = prepared ? io->xh : reinterpret_cast<__half*>(ws.ptr);
  const float* inv_s = prepared ? io->inv_s : reinterpret_cast<float*>(ws.ptr + xh_bytes);
  float* partial = part_out ? io->partial : (splits > 1 ? reinterpret_cast<float*>(ws.ptr + xh_bytes + inv_bytes) : nullptr);
  int* err = device_error_word();
  if (!err) return 1;
  if (!prepared)
    tg_prepare_x_kernel<<<(unsigned)Mpad, 256, 0, s>>>(x, x_type == E_BF16 ? 1 : 0, M, K, reinterpret_cast<__half*>(ws.ptr),
                                                       reinterpret_cast<float*>(ws.ptr + xh_bytes));
  TgArgs a;
  a.w = w, a.xh = xh, a.inv_s = inv_s, a.M = M, a.bn = bn, a.tmem_cols = cols, a.y = y, a.residual = residual, a.error = err;
  CUtensorMap xmap;
  if (tg_make_xmap(const_cast<__half*>(xh), Mpad, K, bn, &xmap)) return 1;
  a.nk_split = nk_split, a.partial = partial;
  const dim3 grid((unsigned)((w.rows + TG_BM - 1) / TG_BM), (unsigned)mtiles, (unsigned)splits);
  const bool a_tmem = tg_a_in_tmem(w.enc);
  const size_t stage_b = (a_tmem ? 0 : TG_A_BYTES) + (size_t)bn * 128;
  const size_t raw_b = a_tmem ? (size_t)TG_A_WARPS * TG_RAW_WORDS * 4 : 0;  // per-warp scratch behind the stages
  const int nslot = 2 * TG_GROUPS * stage_b + raw_b + 1024 <= 200 * 1024 ? 2 * TG_GROUPS : TG_GROUPS;
  a.nslot = nslot;
  if (a_tmem) a.tmem_cols = 512;  // accumulator (<= 256 columns) + the A ring (32 columns per slot)
  const size_t smem = (size_t)nslot * stage_b + raw_b + 1024;
  int rc = 1;
  switch (w.enc) {
    case E_Q4_0: rc = tg_launch<E_Q4_0>(a, xmap, grid, smem, s); break;
    case E_Q4_1: rc = tg_launch<E_Q4_1>(a, xmap, grid, smem, s); break;
    case E_Q8_0: rc = tg_launch<E_Q8_0>(a, xmap, grid, smem, s); break;
    case E_Q6_K: rc = tg_launch<E_Q6_K>(a, xmap, grid, smem, s); break;
    case E_Q4_K: rc = tg_launch<E_Q4_K>(a, xmap, grid, smem, s); break;
    case E_Q5_K: rc = tg_launch<E_Q5_K>(a, xmap, grid, smem, s); break;
    case E_IQ4_XS: rc = tg_launch<E_IQ4_XS>(a, xmap, grid, smem, s); break;
    case E_MLX_U4: rc = tg_launch<E_MLX_U4>(a, xmap, grid, smem, s); break;
    case E_F32: rc = tg_launch<E_F32>(a, xmap, grid, smem, s); break;
    case E_F16: rc = tg_launch<E_F16>(a, xmap, grid, smem, s); break;
    case E_BF16: rc = tg_launch<E_BF16>(a, xmap, grid, smem, s); break;
    default: break;
  }
  if (rc) return rc;
  count_launch(prepared ? 1 : 2);
  if (part_out) {
    io->splits = splits;
  } else if (splits > 1) {
    const int64_t count = M * w.rows;
    tg_split_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(partial, splits, count, y, residual);
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  *handled = true;
  return 0;
}

}  // namespace dyn
