// Fused dequant-GEMV for ONE activation row, "column-split" tensor-core scheme.
//
// mma.sync.m16n8k16 has 8 output columns but a matrix-vector product needs one (two with the
// hi/lo f16 split of an f32 activation). This kernel uses the other columns to keep FOUR
// quantisation blocks apart inside one instruction: lane quarter t (lane & 3) feeds the A operand
// with the nibbles of block t of its two rows, and the B operand holds block t's activations only
// in columns 2t (hi) and 2t+1 (lo), zeros elsewhere. The accumulator fragment of lane (g, t) is
// then exactly (row g | row g+8) x (block t hi, lo): every lane applies one block scale per row
// per 8 mma steps instead of one per block per step, and reads its 16 quant bytes + scale as one
// contiguous run. Instruction cost drops to ~1.3 per weight, which is what it takes for the
// product to be bound by HBM instead of by instruction issue.
//
// Q4_0 (18-byte blocks, crates/dyninfer-kernel-registry/src/gguf_codegen.rs:268-330 for the
// decode rule w = (q - 8) * d): a unit is 8 blocks = 144 bytes per row = 36 words; lane t reads
// words 9t .. 9t+8 of its rows, which hold blocks 2t (scale in the low half of word 0, quants
// straddling words 0..4) and 2t+1 (scale in the high half of word 4, quants = words 5..8).
// Even blocks form one mma group, odd blocks the next, so the alignment case is uniform per
// group.
//
// Data movement: every warp owns a ring of CS_NST stages in shared memory; a stage is 16 rows x
// 288 bytes (two units, K-span 512), brought by FOUR 2-D tensor copies (cp.async.bulk.tensor over a
// map of the matrix as [rows][row bytes / 4] words) of 8 rows x one unit each, completing on the
// stage's mbarrier. (One 1-D bulk copy per row, sixteen per stage, is what this kernel used before:
// with 288-byte copies the copy engine's request rate, not HBM, set the pace -- the copies alone
// ran at 69 % of the measured HBM peak.) A box lands densely, 144 bytes per row = 36 words, so the
// eight rows of a fragment load start 4 banks apart and the four lane quarters 9 words apart: 32
// lanes, 32 banks. Box bytes past the end of a row or of the matrix arrive as zeros, which is how a
// row that ends half way through a stage (K % 512 == 256) and the ragged last tile are handled. A
// stage is read into registers in one go and its slot refilled before the math starts. A warp
// walks a contiguous range of (tile, K-slice) items and keeps the ring running across item
// boundaries.
// All waits are bounded; a wait that runs out sets the error word in the workspace and the warp
// leaves (its rows are then not written).
#include <algorithm>

#include "gemv_core.cuh"
#include "ring.cuh"
#include "tensor_map.cuh"

namespace dyn {

namespace {

constexpr int CS_WARPS = 16;
constexpr int CS_NST = 2;            // stages per warp
constexpr int CS_PAIRS = 1;          // unit pairs (512 elements) per stage
constexpr int CS_KSTAGE = 512 * CS_PAIRS; // K elements per stage
// Per encoding: words a lane reads per unit and row (two blocks incl. their scales), bytes of one
// row in a stage, and the row pitch in shared memory (bytes of a stage row + 16).
//   Q4_0: 18-byte blocks, 9 words per lane, 144-byte unit rows (36 words: conflict-free)
//   Q4_1: 20-byte blocks (f16 d, f16 m, 16 quant bytes), 10 words, 160-byte unit rows (two-way conflicts)
// A stage holds, for each of its two units, a box of rows 0..7 and a box of rows 8..15.
template <int ENC>
struct CsGeo {
  static constexpr int LW = ENC == E_Q4_0 ? 9 : 10;          // words per lane, unit and row
  static constexpr int UW = 4 * LW;                          // words per unit and row
  static constexpr int ROWB = UW * 4 * 2 * CS_PAIRS;         // bytes of one row in a stage
  static constexpr int BOX = 8 * UW * 4;                     // bytes of one box (8 rows of one unit): 1152 / 1280
  static constexpr int STAGE = 4 * CS_PAIRS * BOX;           // a multiple of 128
  static constexpr int RING_BYTES = CS_WARPS * CS_NST * STAGE + CS_WARPS * CS_NST * 8;  // rings + barriers
};
constexpr long long CS_SPINS = 1LL << 22;
constexpr int CS_MAX_SMEM = 226 * 1024;  // dynamic shared memory the kernel may ask for (static: 128 bytes)


// ---- activation staging (every CTA, into its own shared memory) ---------------------------------
// xq: per (unit U of 256 elements, parity e, word i, quarter t, hi/lo) one uint4 holding the B
// registers of mma steps 2i (x, y) and 2i+1 (z, w) of block 8U + 2t + e:
//   step 2i+o: b0 = (x[4i+o], x[4i+o+2]), b1 = (x[16+4i+o], x[16+4i+o+2]) / 16,
// scaled so the row's largest magnitude sits in [2^12, 2^13); index ((U*2+e)*4+i)*8 + 2t + hl, so
// the eight lanes that feed one step read 128 contiguous bytes.
// sx8[b] = sum_factor * sum(block b of the scaled row) in accumulator units (8 = the Q4_0 zero point;
// 1 for Q4_1, whose minimum multiplies the plain sum).
// Returns 2^24 / scale (what turns accumulator units back into the product).
// K may end half way through a stage (K % 512 == 256): elements past K read as zeros.
// Only the span [k0, k0 + kspan) of the row is arranged (the K-slices this CTA's items touch: items
// are numbered slice-major, so a CTA works inside one or two slices and the arrangement costs
// 1/S of the row instead of all of it); the scale comes from the whole row, so that every CTA
// uses the same one. xq and sx8 are indexed from the start of the span.
// order 1 (MLX-U4): a block's 32-bit word i holds elements 8i .. 8i+7, nibble k = element 8i + k, so step
//   2i+o pairs b0 = (x[8i+2o], x[8i+2o+4]), b1 = (x[8i+2o+1], x[8i+2o+5]) / 16.
// order 2 (Q4_K): a 32-element sub-block is one nibble plane of 32 bytes; step s = 2i+o takes the plane's
//   elements of word s: b0 = (x[4s], x[4s+2]), b1 = (x[4s+1], x[4s+3]), all of them / 16 for the odd
//   sub-blocks (the high-nibble plane).
__device__ __forceinline__ float cs_stage_x(const void* __restrict__ x, int x_bf16, int K, int k0, int kspan, uint2* xq,
                                            float* sx8, float* red, float sum_factor, int order = 0) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto ld = [&](int i) -> float {
    if (i >= K) return 0.f;
    return x_bf16 ? bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(x) + i))
                  : __ldg(reinterpret_cast<const float*>(x) + i);
  };
  float mx = 0.f;
  for (int i = tid; i < K; i += CS_WARPS * 32) mx = fmaxf(mx, fabsf(ld(i)));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = 0.f;
#pragma unroll
  for (int i = 0; i < CS_WARPS; i++) mx = fmaxf(mx, red[i]);
  float s, is;
  scale_for(mx, &s, &is);
  for (int j = tid; j < (kspan >> 2); j += CS_WARPS * 32) {  // item j: block j / 8 of the span, mma step j % 8
    const int b = j >> 3, st = j & 7, i = st >> 1, o = st & 1;
    const int U = b >> 3, r = b & 7, t = r >> 1, e = r & 1;
    const int kb = k0 + b * 32;
    const int ia = order == 1 ? 8 * i + 2 * o : (order == 2 ? 4 * st : 4 * i + o), da = order == 1 ? 4 : 2;
    const int ib = order == 0 ? ia + 16 : ia + 1;
    const float e0 = ld(kb + ia) * s, e1 = ld(kb + ia + da) * s;
    const float g0 = ld(kb + ib) * s, g1 = ld(kb + ib + da) * s;
    float sum = (e0 + e1) + (g0 + g1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (st == 0) sx8[b] = sum_factor * GV_2M24 * sum;
    const float m0 = order == 2 && e ? 0.0625f : 1.0f, m1 = order == 2 && !e ? 1.0f : 0.0625f;
    const float f0 = g0 * m1, f1 = g1 * m1, d0 = e0 * m0, d1 = e1 * m0;
    const __half h0 = __float2half_rn(d0), h1 = __float2half_rn(d1);
    const __half h2 = __float2half_rn(f0), h3 = __float2half_rn(f1);
    const __half2 hi0 = __halves2half2(h0, h1), hi1 = __halves2half2(h2, h3);
    const __half2 lo0 = __halves2half2(__float2half_rn(d0 - __half2float(h0)), __float2half_rn(d1 - __half2float(h1)));
    const __half2 lo1 = __halves2half2(__float2half_rn(f0 - __half2float(h2)), __float2half_rn(f1 - __half2float(h3)));
    uint2* dst = xq + ((size_t)(((U * 2 + e) * 4 + i) * 8 + 2 * t) * 2 + o);  // uint2 units; hl adds 2
    dst[0] = make_uint2(*reinterpret_cast<const uint32_t*>(&hi0), *reinterpret_cast<const uint32_t*>(&hi1));
    dst[2] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo0), *reinterpret_cast<const uint32_t*>(&lo1));
  }
  return GV_2P24 * is;
}

// ---- tiles -------------------------------------------------------------------------------------
struct CsArgs {
  int64_t N;
  int K;
  int S;                 // K-slices per tile
  int nst;               // stages per item (ceil(K / 512) / S)
  int ntiles;
  int span_units;        // 256-element units of the activation row a CTA arranges at most
  const void* x;         // the activation row
  int x_bf16;
  float* misc;           // [0] = 2^24 / scale, for the K-slice reduction
  float* y;
  const float* residual;
  float* partial;        // [S][N] when S > 1
  int* error;
  // MLX-U4 only: aux element type is f16 (else bf16); bytes of scales (= of biases) per row and stage;
  // group of 32 (else 64) weights per scale
  int aux_f16, sb, group32;
};

template <int ENC>
__global__ void __launch_bounds__(CS_WARPS * 32, 1)
gemv_cs_q4_kernel(const CsArgs a, const __grid_constant__ CUtensorMap wmap) {
  using G = CsGeo<ENC>;
  constexpr int LW = G::LW;
  extern __shared__ __align__(128) uint8_t cs_smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = cs_smem + (size_t)warp * CS_NST * G::STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(cs_smem + (size_t)CS_WARPS * CS_NST * G::STAGE) + warp * CS_NST;
  uint4* xq = reinterpret_cast<uint4*>(cs_smem + G::RING_BYTES);
  float* sx8 = reinterpret_cast<float*>(xq + (size_t)a.span_units * 64);
  float* red = sx8 + a.span_units * 8;
  pdl_trigger();  // the next kernel of the stream may start its own weight fetch
  if (threadIdx.x == 0) s_abort = 0;
  if (lane == 0) {
    for (int i = 0; i < CS_NST; i++) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  __syncthreads();

  // item = slice * ntiles + tile (slice-major): consecutive items share their K-slice
  const int64_t nitems = (int64_t)a.ntiles * a.S;
  const int64_t gw = (int64_t)blockIdx.x * CS_WARPS + warp;
  const int64_t nwarps = (int64_t)gridDim.x * CS_WARPS;
  const int64_t item_lo = nitems * gw / nwarps, item_hi = nitems * (gw + 1) / nwarps;  // balanced split
  const int nst = a.nst;
  const int total = item_lo < item_hi ? (int)(item_hi - item_lo) * nst : 0;
  // the slices this CTA's sixteen warps touch, and the units of the activation row they cover
  const int64_t cta_lo = nitems * ((int64_t)blockIdx.x * CS_WARPS) / nwarps;
  const int64_t cta_hi = nitems * ((int64_t)(blockIdx.x + 1) * CS_WARPS) / nwarps;
  const int sl_first = (int)(cta_lo / a.ntiles), sl_last = cta_hi > cta_lo ? (int)((cta_hi - 1) / a.ntiles) : sl_first;
  const int U_base = sl_first * nst * 2;

  // copy role: lanes 0..3 each fetch one box (unit lane >> 1, rows 8 * (lane & 1) ..) of the stage.
  // The copy cursor (tile, slice, stage, slot) runs CS_NST stages ahead of the math and advances
  // without divisions.
  const int sl_lo = (int)(item_lo / a.ntiles), tile_lo = (int)(item_lo - (int64_t)sl_lo * a.ntiles);
  int c_left = total, c_tile = tile_lo, c_sl = sl_lo, c_st = 0, c_slot = 0;
  auto issue = [&]() {
    if (c_left <= 0) return;
    c_left--;
    if (lane == 0) mbar_expect_tx(bars + c_slot, G::STAGE);  // boxes count in full, zeros included
    __syncwarp();
    if (lane < 4) {
      const int u = lane >> 1, hf = lane & 1;
      const int x = ((c_sl * nst + c_st) * 2 + u) * G::UW;  // words into the row: a multiple of 4
      const int y = c_tile * 16 + hf * 8;
      tma_box_g2s(ring + c_slot * G::STAGE + lane * G::BOX, &wmap, x, y, bars + c_slot);
    }
    if (++c_slot == CS_NST) c_slot = 0;
    if (++c_st == nst) {
      c_st = 0;
      if (++c_tile == a.ntiles) c_tile = 0, c_sl++;
    }
  };
#pragma unroll
  for (int q = 0; q < CS_NST; q++) issue();

  // The weights do not depend on the kernels before this one: the first stages are already in
  // flight. Everything else (the activation row, the scratch words) does.
  pdl_wait();
  // while the first stages are in flight: arrange the activation row in shared memory
  const float out_scale = cs_stage_x(a.x, a.x_bf16, a.K, U_base * 256, (sl_last - sl_first + 1) * nst * 512,
                                     reinterpret_cast<uint2*>(xq), sx8, red, ENC == E_Q4_0 ? 8.0f : 1.0f);
  if (blockIdx.x == 0 && threadIdx.x == 0) a.misc[0] = out_scale;
  __syncthreads();
  if (total == 0) return;
  // only the lanes with g >> 1 == t feed non-zero B columns (hi for even g, lo for odd g)
  const bool active = (g >> 1) == t;
  float acc0 = 0.f, acc1 = 0.f;
  int tile = tile_lo, sl = sl_lo, slot = 0;
  unsigned parity = 0;
  for (int64_t item = item_lo; item < item_hi; item++) {
    for (int st = 0; st < nst; st++) {
      if (!mbar_wait_bounded_sleepy(bars + slot, parity, CS_SPINS, &s_abort, 2000u)) {
        if (!s_abort) {
          s_abort = 1;
          report_wait_expired(a.error, DEV_ERR_GEMV_RING);
        }
        return;  // warp-uniform: every lane polls the same barrier
      }
      // box (unit u, rows 8 hf ..) sits at (2 u + hf) * BOX; row g of a box at g * UW words
      const uint8_t* base = ring + slot * G::STAGE;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(base) + g * G::UW + LW * t;
      const uint32_t* r1 = r0 + G::BOX / 4;
#pragma unroll
      for (int pr = 0; pr < CS_PAIRS; pr++) {
      const int U0 = ((sl * nst + st) * CS_PAIRS + pr) * 2 - U_base;  // first unit of this pair within the arranged span
      // the pair goes to registers first; after the last pair the slot can be refilled before the math
      uint32_t w0[2][LW], w1[2][LW];
#pragma unroll
      for (int u = 0; u < 2; u++)
#pragma unroll
        for (int i = 0; i < LW; i++) {
          w0[u][i] = r0[(pr * 2 + u) * (G::BOX / 2) + i];
          w1[u][i] = r1[(pr * 2 + u) * (G::BOX / 2) + i];
        }
      if (pr == CS_PAIRS - 1) {
        __syncwarp();
        issue();
        if (++slot == CS_NST) slot = 0, parity ^= 1u;
      }
      // four independent groups (unit u, parity e), their mma steps interleaved so that
      // consecutive tensor instructions never depend on each other
      const uint4* bp = xq + (size_t)U0 * 64 + g;   // group gi, word i: + gi * 32 + i * 8
      const float* sxp = sx8 + U0 * 8 + 2 * t;
      float c[4][4];
#pragma unroll
      for (int gi = 0; gi < 4; gi++) c[gi][0] = c[gi][1] = c[gi][2] = c[gi][3] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        uint32_t q0[4], q1[4];
        uint4 bf[4];
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
          const int u = gi >> 1;
          if (ENC == E_Q4_1) {  // both blocks word aligned: (d, m) then four quant words
            q0[gi] = w0[u][5 * (gi & 1) + 1 + i];
            q1[gi] = w1[u][5 * (gi & 1) + 1 + i];
          } else if (gi & 1) {  // Q4_0 odd block: words 5..8
            q0[gi] = w0[u][5 + i];
            q1[gi] = w1[u][5 + i];
          } else {       // Q4_0 even block: quants start 2 bytes into word 0
            q0[gi] = __funnelshift_r(w0[u][i], w0[u][i + 1], 16);
            q1[gi] = __funnelshift_r(w1[u][i], w1[u][i + 1], 16);
          }
          bf[gi] = active ? bp[gi * 32 + i * 8] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int gi = 0; gi < 4; gi++)
          mma_f16_16816(c[gi], q0[gi] & 0x000F000Fu, q1[gi] & 0x000F000Fu, q0[gi] & 0x00F000F0u,
                        q1[gi] & 0x00F000F0u, bf[gi].x, bf[gi].y);
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
          const uint32_t s0 = q0[gi] >> 8, s1 = q1[gi] >> 8;
          mma_f16_16816(c[gi], s0 & 0x000F000Fu, s1 & 0x000F000Fu, s0 & 0x00F000F0u, s1 & 0x00F000F0u,
                        bf[gi].z, bf[gi].w);
        }
      }
#pragma unroll
      for (int gi = 0; gi < 4; gi++) {
        const int u = gi >> 1;
        const float sx = sxp[u * 8 + (gi & 1)];
        if (ENC == E_Q4_1) {  // w = q * d + m: scale the tile sums, add the minimum times the plain sum
          const __half2 h0 = *reinterpret_cast<const __half2*>(&w0[u][5 * (gi & 1)]);
          const __half2 h1 = *reinterpret_cast<const __half2*>(&w1[u][5 * (gi & 1)]);
          acc0 = fmaf(__low2float(h0), c[gi][0] + c[gi][1], fmaf(__high2float(h0), sx, acc0));
          acc1 = fmaf(__low2float(h1), c[gi][2] + c[gi][3], fmaf(__high2float(h1), sx, acc1));
        } else {
          const __half2 h0 = *reinterpret_cast<const __half2*>(&w0[u][(gi & 1) ? 4 : 0]);
          const __half2 h1 = *reinterpret_cast<const __half2*>(&w1[u][(gi & 1) ? 4 : 0]);
          const float d0 = (gi & 1) ? __high2float(h0) : __low2float(h0);
          const float d1 = (gi & 1) ? __high2float(h1) : __low2float(h1);
          acc0 = fmaf(d0, (c[gi][0] + c[gi][1]) - sx, acc0);
          acc1 = fmaf(d1, (c[gi][2] + c[gi][3]) - sx, acc1);
        }
      }
      }
    }
    // the four quarters of a row hold disjoint blocks: add them in a fixed order
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) {
      const int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
      if (a.S == 1) {
        if (row0 < a.N) a.y[row0] = acc0 * out_scale + (a.residual ? a.residual[row0] : 0.f);
        if (row1 < a.N) a.y[row1] = acc1 * out_scale + (a.residual ? a.residual[row1] : 0.f);
      } else {
        if (row0 < a.N) a.partial[(int64_t)sl * a.N + row0] = acc0;
        if (row1 < a.N) a.partial[(int64_t)sl * a.N + row1] = acc1;
      }
    }
    acc0 = acc1 = 0.f;
    if (++tile == a.ntiles) tile = 0, sl++;
  }
}

// ---- MLX affine U4 ---------------------------------------------------------------------------
// The same scheme for MLX-U4 rows (ui32[N, K/8], word j = weights 8j..8j+7, nibble k = bits [4k, 4k+4);
// bf16 / f16 scales and biases per group of 64 or 32 weights, w = q * scale + bias,
// mlx_affine.rs:284-290,590-600). A 32-weight block is four words; lane quarter t takes blocks 2t and
// 2t + 1 of a 256-weight unit = words 8t .. 8t+7 = two 16-byte pieces of the row's 128 bytes. A stage is
// two units x 16 rows: four tensor copies of 8 rows x 128 bytes, 128-byte swizzled so that the lanes'
// 16-byte loads of one piece from eight rows fall into different banks, plus one box of the stage's
// scales and one of its biases (16 rows x 16 or 32 bytes). The row's product is
// sum_groups scale * sum(q x) + bias * sum(x): the second term uses the per-block sums of the arranged row.
constexpr int CM_WSTAGE = 4096;  // weight bytes of a stage: 4 boxes of 8 rows x 128 bytes

__global__ void __launch_bounds__(CS_WARPS * 32, 1)
gemv_cs_mlx_kernel(const CsArgs a, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                   const __grid_constant__ CUtensorMap bmap) {
  extern __shared__ __align__(128) uint8_t cs_smem_mlx[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cs_smem_mlx) + 1023) & ~uintptr_t(1023));
  const int aux_stage = 2 * 16 * a.sb;  // scales then biases
  uint8_t* ring = smem + (size_t)warp * CS_NST * CM_WSTAGE;
  uint8_t* aring = smem + (size_t)CS_WARPS * CS_NST * CM_WSTAGE + (size_t)warp * CS_NST * aux_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)CS_WARPS * CS_NST * (CM_WSTAGE + aux_stage)) + warp * CS_NST;
  uint4* xq = reinterpret_cast<uint4*>(smem + (size_t)CS_WARPS * CS_NST * (CM_WSTAGE + aux_stage + 8));
  float* sx8 = reinterpret_cast<float*>(xq + (size_t)a.span_units * 64);
  float* red = sx8 + a.span_units * 8;
  pdl_trigger();  // the next kernel of the stream may start its own weight fetch
  if (threadIdx.x == 0) s_abort = 0;
  if (lane == 0) {
    for (int i = 0; i < CS_NST; i++) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int64_t nitems = (int64_t)a.ntiles * a.S;
  const int64_t gw = (int64_t)blockIdx.x * CS_WARPS + warp;
  const int64_t nwarps = (int64_t)gridDim.x * CS_WARPS;
  const int64_t item_lo = nitems * gw / nwarps, item_hi = nitems * (gw + 1) / nwarps;
  const int nst = a.nst;
  const int total = item_lo < item_hi ? (int)(item_hi - item_lo) * nst : 0;
  const int64_t cta_lo = nitems * ((int64_t)blockIdx.x * CS_WARPS) / nwarps;
  const int64_t cta_hi = nitems * ((int64_t)(blockIdx.x + 1) * CS_WARPS) / nwarps;
  const int sl_first = (int)(cta_lo / a.ntiles), sl_last = cta_hi > cta_lo ? (int)((cta_hi - 1) / a.ntiles) : sl_first;
  const int U_base = sl_first * nst * 2;

  const int sl_lo = (int)(item_lo / a.ntiles), tile_lo = (int)(item_lo - (int64_t)sl_lo * a.ntiles);
  int c_left = total, c_tile = tile_lo, c_sl = sl_lo, c_st = 0, c_slot = 0;
  auto issue = [&]() {
    if (c_left <= 0) return;
    c_left--;
    if (lane == 0) mbar_expect_tx(bars + c_slot, CM_WSTAGE + aux_stage);  // boxes count in full, zeros included
    __syncwarp();
    const int stage = c_sl * nst + c_st;
    if (lane < 4) {  // weights: unit lane >> 1, rows 8 * (lane & 1) ..
      tma_box_g2s(ring + c_slot * CM_WSTAGE + lane * 1024, &wmap, (stage * 2 + (lane >> 1)) * 32, c_tile * 16 + (lane & 1) * 8,
                  bars + c_slot);
    } else if (lane < 6) {  // the stage's scales / biases of the tile's 16 rows
      tma_box_g2s(aring + c_slot * aux_stage + (lane - 4) * 16 * a.sb, lane == 4 ? &smap : &bmap, stage * (a.sb / 4),
                  c_tile * 16, bars + c_slot);
    }
    if (++c_slot == CS_NST) c_slot = 0;
    if (++c_st == nst) {
      c_st = 0;
      if (++c_tile == a.ntiles) c_tile = 0, c_sl++;
    }
  };
#pragma unroll
  for (int q = 0; q < CS_NST; q++) issue();

  pdl_wait();
  const float out_scale = cs_stage_x(a.x, a.x_bf16, a.K, U_base * 256, (sl_last - sl_first + 1) * nst * 512,
                                     reinterpret_cast<uint2*>(xq), sx8, red, 1.0f, 1);
  if (blockIdx.x == 0 && threadIdx.x == 0) a.misc[0] = out_scale;
  __syncthreads();
  if (total == 0) return;
  const bool active = (g >> 1) == t;
  auto aux_f32 = [&](const uint8_t* p) -> float {
    const uint32_t bits = *reinterpret_cast<const uint16_t*>(p);
    return a.aux_f16 ? __half2float(__ushort_as_half((unsigned short)bits)) : __uint_as_float(bits << 16);
  };
  float acc0 = 0.f, acc1 = 0.f;
  int tile = tile_lo, sl = sl_lo, slot = 0;
  unsigned parity = 0;
  for (int64_t item = item_lo; item < item_hi; item++) {
    for (int st = 0; st < nst; st++) {
      if (!mbar_wait_bounded_sleepy(bars + slot, parity, CS_SPINS, &s_abort, 2000u)) {
        if (!s_abort) {
          s_abort = 1;
          report_wait_expired(a.error, DEV_ERR_GEMV_RING);
        }
        return;  // warp-uniform: every lane polls the same barrier
      }
      const uint8_t* base = ring + slot * CM_WSTAGE;
      const uint8_t* ab = aring + slot * aux_stage;
      const int U0 = (sl * nst + st) * 2 - U_base;
      // words 8t .. 8t+7 of rows g (box rows 0..7) and g + 8 (the next box) of both units; and the
      // lane's scales and biases (rows g, g + 8; group of blocks 2t, 2t+1 or one per block)
      uint32_t w0[2][8], w1[2][8];
      float sc0[4], sc1[4], bi0[4], bi1[4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int piece = ((2 * t + h) ^ g) << 4;
          const uint4 v0 = *reinterpret_cast<const uint4*>(base + (2 * u) * 1024 + g * 128 + piece);
          const uint4 v1 = *reinterpret_cast<const uint4*>(base + (2 * u + 1) * 1024 + g * 128 + piece);
          w0[u][4 * h] = v0.x, w0[u][4 * h + 1] = v0.y, w0[u][4 * h + 2] = v0.z, w0[u][4 * h + 3] = v0.w;
          w1[u][4 * h] = v1.x, w1[u][4 * h + 1] = v1.y, w1[u][4 * h + 2] = v1.z, w1[u][4 * h + 3] = v1.w;
          const int si = a.group32 ? u * 8 + 2 * t + h : u * 4 + t;
          sc0[2 * u + h] = aux_f32(ab + g * a.sb + 2 * si);
          sc1[2 * u + h] = aux_f32(ab + (g + 8) * a.sb + 2 * si);
          bi0[2 * u + h] = aux_f32(ab + 16 * a.sb + g * a.sb + 2 * si);
          bi1[2 * u + h] = aux_f32(ab + 16 * a.sb + (g + 8) * a.sb + 2 * si);
        }
      }
      __syncwarp();
      issue();
      if (++slot == CS_NST) slot = 0, parity ^= 1u;
      const uint4* bp = xq + (size_t)U0 * 64 + g;   // group gi, word i: + gi * 32 + i * 8
      const float* sxp = sx8 + U0 * 8 + 2 * t;
      float c[4][4];
#pragma unroll
      for (int gi = 0; gi < 4; gi++) c[gi][0] = c[gi][1] = c[gi][2] = c[gi][3] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        uint32_t q0[4], q1[4];
        uint4 bf[4];
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
          q0[gi] = w0[gi >> 1][4 * (gi & 1) + i];
          q1[gi] = w1[gi >> 1][4 * (gi & 1) + i];
          bf[gi] = active ? bp[gi * 32 + i * 8] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int gi = 0; gi < 4; gi++)
          mma_f16_16816(c[gi], q0[gi] & 0x000F000Fu, q1[gi] & 0x000F000Fu, q0[gi] & 0x00F000F0u,
                        q1[gi] & 0x00F000F0u, bf[gi].x, bf[gi].y);
#pragma unroll
        for (int gi = 0; gi < 4; gi++) {
          const uint32_t s0 = q0[gi] >> 8, s1 = q1[gi] >> 8;
          mma_f16_16816(c[gi], s0 & 0x000F000Fu, s1 & 0x000F000Fu, s0 & 0x00F000F0u, s1 & 0x00F000F0u,
                        bf[gi].z, bf[gi].w);
        }
      }
#pragma unroll
      for (int gi = 0; gi < 4; gi++) {
        const float sx = sxp[(gi >> 1) * 8 + (gi & 1)];
        acc0 = fmaf(sc0[gi], c[gi][0] + c[gi][1], fmaf(bi0[gi], sx, acc0));
        acc1 = fmaf(sc1[gi], c[gi][2] + c[gi][3], fmaf(bi1[gi], sx, acc1));
      }
    }
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) {
      const int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
      if (a.S == 1) {
        if (row0 < a.N) a.y[row0] = acc0 * out_scale + (a.residual ? a.residual[row0] : 0.f);
        if (row1 < a.N) a.y[row1] = acc1 * out_scale + (a.residual ? a.residual[row1] : 0.f);
      } else {
        if (row0 < a.N) a.partial[(int64_t)sl * a.N + row0] = acc0;
        if (row1 < a.N) a.partial[(int64_t)sl * a.N + row1] = acc1;
      }
    }
    acc0 = acc1 = 0.f;
    if (++tile == a.ntiles) tile = 0, sl++;
  }
}

// ---- Q4_K ------------------------------------------------------------------------------------
// The same scheme for Q4_K (256-weight blocks of 144 bytes: f16 d, f16 dmin, 12 bytes of 6-bit scales and
// minimums, 128 nibble bytes; weight 64 jj + 32 h + l = nibble h of byte 32 jj + l, sub-block j = 2 jj + h,
// w = (d sc_j) q - dmin m_j; arithmetic after GGML's published dequantisation, see codec.cuh). A block is one
// 256-weight unit of 36 words, the box geometry is Q4_0's. Lane quarter t takes the 32 nibble bytes jj = t
// (two 16-byte loads) and the block's four header words: the low-nibble plane is sub-block 2t, the high
// plane sub-block 2t + 1, each with its own accumulator; one mma covers four weights of ONE plane
// (a0/a1 = bytes 0 and 2 of a word, a2/a3 = bytes 1 and 3), so both planes together issue as many mma as a
// Q4_0 unit. The row's product is sum_j (d sc_j) sum(q x) - (dmin m_j) sum(x).
__global__ void __launch_bounds__(CS_WARPS * 32, 1)
gemv_cs_q4k_kernel(const CsArgs a, const __grid_constant__ CUtensorMap wmap) {
  using G = CsGeo<E_Q4_0>;
  extern __shared__ __align__(128) uint8_t cs_smem_q4k[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = cs_smem_q4k + (size_t)warp * CS_NST * G::STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(cs_smem_q4k + (size_t)CS_WARPS * CS_NST * G::STAGE) + warp * CS_NST;
  uint4* xq = reinterpret_cast<uint4*>(cs_smem_q4k + G::RING_BYTES);
  float* sx8 = reinterpret_cast<float*>(xq + (size_t)a.span_units * 64);
  float* red = sx8 + a.span_units * 8;
  pdl_trigger();  // the next kernel of the stream may start its own weight fetch
  if (threadIdx.x == 0) s_abort = 0;
  if (lane == 0) {
    for (int i = 0; i < CS_NST; i++) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int64_t nitems = (int64_t)a.ntiles * a.S;
  const int64_t gw = (int64_t)blockIdx.x * CS_WARPS + warp;
  const int64_t nwarps = (int64_t)gridDim.x * CS_WARPS;
  const int64_t item_lo = nitems * gw / nwarps, item_hi = nitems * (gw + 1) / nwarps;
  const int nst = a.nst;
  const int total = item_lo < item_hi ? (int)(item_hi - item_lo) * nst : 0;
  const int64_t cta_lo = nitems * ((int64_t)blockIdx.x * CS_WARPS) / nwarps;
  const int64_t cta_hi = nitems * ((int64_t)(blockIdx.x + 1) * CS_WARPS) / nwarps;
  const int sl_first = (int)(cta_lo / a.ntiles), sl_last = cta_hi > cta_lo ? (int)((cta_hi - 1) / a.ntiles) : sl_first;
  const int U_base = sl_first * nst * 2;

  const int sl_lo = (int)(item_lo / a.ntiles), tile_lo = (int)(item_lo - (int64_t)sl_lo * a.ntiles);
  int c_left = total, c_tile = tile_lo, c_sl = sl_lo, c_st = 0, c_slot = 0;
  auto issue = [&]() {
    if (c_left <= 0) return;
    c_left--;
    if (lane == 0) mbar_expect_tx(bars + c_slot, G::STAGE);  // boxes count in full, zeros included
    __syncwarp();
    if (lane < 4) {
      const int u = lane >> 1, hf = lane & 1;
      tma_box_g2s(ring + c_slot * G::STAGE + lane * G::BOX, &wmap, ((c_sl * nst + c_st) * 2 + u) * G::UW, c_tile * 16 + hf * 8,
                  bars + c_slot);
    }
    if (++c_slot == CS_NST) c_slot = 0;
    if (++c_st == nst) {
      c_st = 0;
      if (++c_tile == a.ntiles) c_tile = 0, c_sl++;
    }
  };
#pragma unroll
  for (int q = 0; q < CS_NST; q++) issue();

  pdl_wait();
  const float out_scale = cs_stage_x(a.x, a.x_bf16, a.K, U_base * 256, (sl_last - sl_first + 1) * nst * 512,
                                     reinterpret_cast<uint2*>(xq), sx8, red, 1.0f, 2);
  if (blockIdx.x == 0 && threadIdx.x == 0) a.misc[0] = out_scale;
  __syncthreads();
  if (total == 0) return;
  const bool active = (g >> 1) == t;
  // d * sc_j and dmin * m_j of sub-block j out of a block's four header words
  auto scale_min = [](const uint4& h, int j, float* ds, float* dm) {
    const uint32_t sw[3] = {h.y, h.z, h.w};
    auto sb = [&](int i) { return (sw[i >> 2] >> (8 * (i & 3))) & 0xffu; };
    uint32_t sc, mn;
    if (j < 4) {
      sc = sb(j) & 63u, mn = sb(j + 4) & 63u;
    } else {
      sc = (sb(j + 4) & 15u) | ((sb(j - 4) >> 6) << 4);
      mn = (sb(j + 4) >> 4) | ((sb(j) >> 6) << 4);
    }
    const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
    *ds = __low2float(dd) * (float)sc;
    *dm = __high2float(dd) * (float)mn;
  };
  float acc0 = 0.f, acc1 = 0.f;
  int tile = tile_lo, sl = sl_lo, slot = 0;
  unsigned parity = 0;
  for (int64_t item = item_lo; item < item_hi; item++) {
    for (int st = 0; st < nst; st++) {
      if (!mbar_wait_bounded_sleepy(bars + slot, parity, CS_SPINS, &s_abort, 2000u)) {
        if (!s_abort) {
          s_abort = 1;
          report_wait_expired(a.error, DEV_ERR_GEMV_RING);
        }
        return;  // warp-uniform: every lane polls the same barrier
      }
      // box (unit u, rows 8 hf ..) sits at (2 u + hf) * BOX; row g of a box at g * 144 bytes
      const uint8_t* base = ring + slot * G::STAGE;
      const int U0 = (sl * nst + st) * 2 - U_base;
      uint4 hd0[2], hd1[2], qa0[2], qb0[2], qa1[2], qb1[2];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const uint8_t* r0 = base + (2 * u) * G::BOX + g * 144;
        const uint8_t* r1 = base + (2 * u + 1) * G::BOX + g * 144;
        hd0[u] = *reinterpret_cast<const uint4*>(r0), hd1[u] = *reinterpret_cast<const uint4*>(r1);
        qa0[u] = *reinterpret_cast<const uint4*>(r0 + 16 + 32 * t), qb0[u] = *reinterpret_cast<const uint4*>(r0 + 32 + 32 * t);
        qa1[u] = *reinterpret_cast<const uint4*>(r1 + 16 + 32 * t), qb1[u] = *reinterpret_cast<const uint4*>(r1 + 32 + 32 * t);
      }
      __syncwarp();
      issue();
      if (++slot == CS_NST) slot = 0, parity ^= 1u;
      const uint4* bp = xq + (size_t)U0 * 64 + g;   // (unit u, plane e), step pair m: + (2 u + e) * 32 + m * 8
      const float* sxp = sx8 + U0 * 8 + 2 * t;
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const uint32_t w0[8] = {qa0[u].x, qa0[u].y, qa0[u].z, qa0[u].w, qb0[u].x, qb0[u].y, qb0[u].z, qb0[u].w};
        const uint32_t w1[8] = {qa1[u].x, qa1[u].y, qa1[u].z, qa1[u].w, qb1[u].x, qb1[u].y, qb1[u].z, qb1[u].w};
        float c[2][4];
#pragma unroll
        for (int e = 0; e < 2; e++) c[e][0] = c[e][1] = c[e][2] = c[e][3] = 0.f;
#pragma unroll
        for (int m = 0; m < 4; m++) {
          uint4 bf[2];
#pragma unroll
          for (int e = 0; e < 2; e++) bf[e] = active ? bp[(2 * u + e) * 32 + m * 8] : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int o = 0; o < 2; o++) {
            const uint32_t x0 = w0[2 * m + o], x1 = w1[2 * m + o];
            mma_f16_16816(c[0], x0 & 0x000F000Fu, x1 & 0x000F000Fu, (x0 >> 8) & 0x000F000Fu, (x1 >> 8) & 0x000F000Fu,
                          o ? bf[0].z : bf[0].x, o ? bf[0].w : bf[0].y);
            mma_f16_16816(c[1], x0 & 0x00F000F0u, x1 & 0x00F000F0u, (x0 >> 8) & 0x00F000F0u, (x1 >> 8) & 0x00F000F0u,
                          o ? bf[1].z : bf[1].x, o ? bf[1].w : bf[1].y);
          }
        }
#pragma unroll
        for (int e = 0; e < 2; e++) {
          float ds0, dm0, ds1, dm1;
          scale_min(hd0[u], 2 * t + e, &ds0, &dm0);
          scale_min(hd1[u], 2 * t + e, &ds1, &dm1);
          const float sx = sxp[u * 8 + e];
          acc0 = fmaf(ds0, c[e][0] + c[e][1], fmaf(-dm0, sx, acc0));
          acc1 = fmaf(ds1, c[e][2] + c[e][3], fmaf(-dm1, sx, acc1));
        }
      }
    }
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) {
      const int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
      if (a.S == 1) {
        if (row0 < a.N) a.y[row0] = acc0 * out_scale + (a.residual ? a.residual[row0] : 0.f);
        if (row1 < a.N) a.y[row1] = acc1 * out_scale + (a.residual ? a.residual[row1] : 0.f);
      } else {
        if (row0 < a.N) a.partial[(int64_t)sl * a.N + row0] = acc0;
        if (row1 < a.N) a.partial[(int64_t)sl * a.N + row1] = acc1;
      }
    }
    acc0 = acc1 = 0.f;
    if (++tile == a.ntiles) tile = 0, sl++;
  }
}

// partial sums over the K-slices, fixed order
__global__ void __launch_bounds__(256)
cs_reduce_kernel(const float* __restrict__ partial, int S, int64_t N, const float* __restrict__ misc,
                 float* y, const float* residual) {
  pdl_trigger();
  pdl_wait();  // the partial sums come from the kernel before this one
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= N) return;
  float v = 0.f;
  for (int j = 0; j < S; j++) v += partial[(int64_t)j * N + i];
  v *= misc[0];
  if (residual) v += residual[i];
  y[i] = v;
}

struct CsPlan {
  int S, nst, ntiles, grid, span_units;
  size_t smem, off_err, off_part, bytes;
};

bool cs_basic_ok(const WRef& w, int M) {
  if (w.enc == E_MLX_U4)  // whole stages; groups of 64 or 32; 2-byte scales and biases; 16-byte aligned arrays
    return M == 1 && w.rows >= 1 && w.cols >= CS_KSTAGE && w.cols % CS_KSTAGE == 0 && (w.group == 64 || w.group == 32) &&
           (w.aux == E_BF16 || w.aux == E_F16) && w.scales && w.biases &&
           ((reinterpret_cast<uintptr_t>(w.data) | reinterpret_cast<uintptr_t>(w.scales) |
             reinterpret_cast<uintptr_t>(w.biases)) & 15) == 0;
  return M == 1 && (w.enc == E_Q4_0 || w.enc == E_Q4_1 || w.enc == E_Q4_K) && w.rows >= 1 && w.cols >= CS_KSTAGE &&
         w.cols % (CS_KSTAGE / 2) == 0 && (reinterpret_cast<uintptr_t>(w.data) & 15) == 0;
}
int cs_mlx_sb(const WRef& w) { return w.group == 32 ? 32 : 16; }  // bytes of scales per row and stage

void cs_plan(const WRef& w, CsPlan* p) {
  const int K = (int)w.cols, stages = (K + CS_KSTAGE - 1) / CS_KSTAGE;
  p->ntiles = (int)((w.rows + 15) / 16);
  const int sms = std::max(1, sm_count());
  const int64_t warps = (int64_t)sms * CS_WARPS;
  // split K while there are fewer than ~8 items per warp and slices keep >= 1 stage
  int S = 1;
  for (int cand = 1; cand <= stages; cand++) {
    if (stages % cand) continue;
    S = cand;
    if ((int64_t)p->ntiles * cand >= 8 * warps) break;
  }
  p->S = S;
  p->nst = stages / S;
  const int64_t items = (int64_t)p->ntiles * S;
  p->grid = (int)std::min<int64_t>(sms, (items + CS_WARPS - 1) / CS_WARPS);
  // the widest span of K-slices one CTA's items touch (items are slice-major)
  const int64_t nwarps = (int64_t)p->grid * CS_WARPS;
  int span = 1;
  for (int b = 0; b < p->grid; b++) {
    const int64_t lo = items * ((int64_t)b * CS_WARPS) / nwarps, hi = items * ((int64_t)(b + 1) * CS_WARPS) / nwarps;
    if (hi > lo) span = std::max(span, (int)((hi - 1) / p->ntiles - lo / p->ntiles) + 1);
  }
  p->span_units = span * p->nst * 2;
  const size_t ring = w.enc == E_MLX_U4
                          ? 1024 + (size_t)CS_WARPS * CS_NST * (CM_WSTAGE + 2 * 16 * cs_mlx_sb(w) + 8)  // 1024: alignment slack
                          : (w.enc == E_Q4_1 ? CsGeo<E_Q4_1>::RING_BYTES : CsGeo<E_Q4_0>::RING_BYTES);  // Q4_K: Q4_0's boxes
  p->smem = ring + (size_t)p->span_units * (1024 + 32) + 128;
  p->off_err = 0;       // [64] 2^24 / scale
  p->off_part = 256;
  p->bytes = 256 + (S > 1 ? (size_t)S * w.rows * 4 : 0);
}

bool cs_shape_ok(const WRef& w, int M) {
  if (!cs_basic_ok(w, M)) return false;
  CsPlan p;
  cs_plan(w, &p);
  return p.smem <= (size_t)CS_MAX_SMEM;
}

}  // namespace

size_t gemv_cs_workspace_bytes(const WRef& w, int M) {
  if (w.enc == E_Q6_K) return gemv_cs_q6k_workspace_bytes(w, M);
  if (w.enc == E_Q8_0) return gemv_cs_q8_0_workspace_bytes(w, M);
  if (!cs_shape_ok(w, M)) return 0;
  CsPlan p;
  cs_plan(w, &p);
  return p.bytes;
}

// Column-split GEMV for one activation row (f32 or bf16). *handled = false when the shape does
// not qualify; the caller then uses another kernel. `ws` must hold gemv_cs_workspace_bytes.
int launch_gemv_cs(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                   uint8_t* ws, cudaStream_t s, bool* handled) {
  *handled = false;
  if (w.enc == E_Q6_K) {
    if (!gemv_cs_q6k_shape_ok(w, M)) return 0;
    if (launch_gemv_cs_q6k(w, x, x_type, y, residual, ws, s)) return 1;
    *handled = true;
    return 0;
  }
  if (w.enc == E_Q8_0) {
    if (!gemv_cs_q8_0_shape_ok(w, M)) return 0;
    if (launch_gemv_cs_q8_0(w, x, x_type, y, residual, ws, s)) return 1;
    *handled = true;
    return 0;
  }
  if (!cs_shape_ok(w, M)) return 0;
  CsPlan p;
  cs_plan(w, &p);
  CsArgs a;
  a.N = w.rows, a.K = (int)w.cols;
  a.aux_f16 = 0, a.sb = 0, a.group32 = 0;
  if (w.enc == E_MLX_U4) {
    // weights as [rows][K / 8] words in boxes of 8 rows x 128 bytes (swizzled); scales and biases as
    // [rows][K / group] 2-byte values in boxes of 16 rows x one stage's worth
    CUtensorMap wm, sm, bm;
    const int sb = cs_mlx_sb(w);
    const size_t aux_row = (size_t)(w.cols / w.group) * 2;
    if (make_row_box_map(w.data, (size_t)w.cols / 2, w.rows, 32, 8, &wm, true) ||
        make_row_box_map(w.scales, aux_row, w.rows, sb / 4, 16, &sm) || make_row_box_map(w.biases, aux_row, w.rows, sb / 4, 16, &bm))
      return 1;
    a.S = p.S, a.nst = p.nst, a.ntiles = p.ntiles, a.span_units = p.span_units;
    a.x = x, a.x_bf16 = x_type == E_BF16 ? 1 : 0;
    a.aux_f16 = w.aux == E_F16 ? 1 : 0, a.sb = sb, a.group32 = w.group == 32 ? 1 : 0;
    a.error = device_error_word();
    if (!a.error) return 1;
    a.misc = reinterpret_cast<float*>(ws + p.off_err + 64);
    a.partial = reinterpret_cast<float*>(ws + p.off_part);
    a.y = y, a.residual = residual;
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_cs_mlx_kernel), CS_MAX_SMEM)) return 1;
    DYN_CUDA(launch_pdl(gemv_cs_mlx_kernel, dim3(p.grid), dim3(CS_WARPS * 32), p.smem, s, a, wm, sm, bm));
    count_launch(1);
    Deferred* defer = p.S > 1 && !residual ? defer_take() : nullptr;
    if (defer) {
      defer->partial = a.partial, defer->scale = a.misc, defer->S = p.S, defer->N = w.rows, defer->ws_bytes = p.bytes;
    } else if (p.S > 1) {
      DYN_CUDA(launch_pdl(cs_reduce_kernel, dim3((unsigned)((w.rows + 255) / 256)), dim3(256), 0, s,
                          (const float*)a.partial, p.S, (int64_t)w.rows, (const float*)a.misc, y, residual));
      count_launch();
    }
    DYN_CUDA(cudaGetLastError());
    *handled = true;
    return 0;
  }
  // the matrix as [rows][row bytes / 4] words; boxes of 8 rows x one unit
  CUtensorMap wmap;
  if (make_row_box_map(w.data, w.row_bytes(), w.rows, w.enc == E_Q4_1 ? CsGeo<E_Q4_1>::UW : CsGeo<E_Q4_0>::UW, 8, &wmap))
    return 1;
  a.S = p.S, a.nst = p.nst, a.ntiles = p.ntiles, a.span_units = p.span_units;
  a.x = x, a.x_bf16 = x_type == E_BF16 ? 1 : 0;
  a.error = device_error_word();
  if (!a.error) return 1;
  a.misc = reinterpret_cast<float*>(ws + p.off_err + 64);
  a.partial = reinterpret_cast<float*>(ws + p.off_part);
  a.y = y, a.residual = residual;
  if (ensure_dynamic_smem(w.enc == E_Q4_K   ? reinterpret_cast<const void*>(gemv_cs_q4k_kernel)
                          : w.enc == E_Q4_0 ? reinterpret_cast<const void*>(gemv_cs_q4_kernel<E_Q4_0>)
                                            : reinterpret_cast<const void*>(gemv_cs_q4_kernel<E_Q4_1>),
                          CS_MAX_SMEM))
    return 1;
  if (w.enc == E_Q4_K)
    DYN_CUDA(launch_pdl(gemv_cs_q4k_kernel, dim3(p.grid), dim3(CS_WARPS * 32), p.smem, s, a, wmap));
  else if (w.enc == E_Q4_0)
    DYN_CUDA(launch_pdl(gemv_cs_q4_kernel<E_Q4_0>, dim3(p.grid), dim3(CS_WARPS * 32), p.smem, s, a, wmap));
  else
    DYN_CUDA(launch_pdl(gemv_cs_q4_kernel<E_Q4_1>, dim3(p.grid), dim3(CS_WARPS * 32), p.smem, s, a, wmap));
  count_launch(1);
  Deferred* defer = p.S > 1 && !residual ? defer_take() : nullptr;
  if (defer) {
    defer->partial = a.partial, defer->scale = a.misc, defer->S = p.S, defer->N = w.rows, defer->ws_bytes = p.bytes;
  } else if (p.S > 1) {
    DYN_CUDA(launch_pdl(cs_reduce_kernel, dim3((unsigned)((w.rows + 255) / 256)), dim3(256), 0, s,
                        (const float*)a.partial, p.S, (int64_t)w.rows, (const float*)a.misc, y, residual));
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  *handled = true;
  return 0;
}

}  // namespace dyn
