// Column-split tensor-core GEMV for ONE activation row on Q8_0 rows (34-byte blocks: f16 d, 32 int8;
// w = d * q, crates/dyninfer-kernel-registry/src/gguf_codegen.rs:382-410).
//
// Same scheme as gemv_colsplit.cu: the 8 output columns of mma.sync.m16n8k16 keep four blocks apart.
// A unit is 8 blocks = 272 bytes per row = 68 words; lane quarter t reads words 17t .. 17t+16 of
// its two rows, which hold block 2t (scale in the low half of word 0, the 32 quant bytes straddling
// words 0..8) and block 2t+1 (scale in the high half of word 8, quants = words 9..16). Bytes are
// biased to unsigned (q + 128, exact zero point) and widened to f16 subnormals with byte permutes;
// one quant word = one mma step. Activations stay in natural order as two f16 arrays (hi, lo) in
// shared memory; every block's sum times 128 undoes the bias. Per warp a ring of two stages of
// 16 rows x 272 bytes, brought by two 2-D tensor copies of 8 rows each (dense rows of 68 words: the
// eight rows of a fragment load start 4 banks apart, the lane quarters 17 words apart, so the 32
// lanes hit 32 banks; rows past the end of the matrix arrive as zeros); a stage is read into
// registers and its slot refilled before the math. All waits are bounded.
#include <algorithm>

#include "gemv_core.cuh"
#include "ring.cuh"
#include "tensor_map.cuh"

namespace dyn {

namespace {

constexpr int Q8_WARPS = 16;
constexpr int Q8_NST = 2;
constexpr int Q8_ROWB = 272;     // one unit of 8 blocks
constexpr int Q8_BOX = 8 * Q8_ROWB;   // one box: rows 0..7 or 8..15 of the unit (2176 bytes = 17 x 128)
constexpr int Q8_STAGE = 2 * Q8_BOX;
constexpr int Q8_KSTAGE = 256;
constexpr long long Q8_SPINS = 1LL << 22;
constexpr int Q8_MAX_SMEM = 226 * 1024;
constexpr int Q8_RING_BYTES = Q8_WARPS * Q8_NST * Q8_STAGE + Q8_WARPS * Q8_NST * 8;

struct Q8Args {
  int64_t N;
  int K, S, nst, ntiles;
  const void* x;
  int x_bf16;
  float* misc;  // [0] = 2^24 / scale
  float* y;
  const float* residual;
  float* partial;
  int* error;
};

// Activation row -> shared memory: xhi[K], 16 bytes of padding, xlo[K] (f16, natural order, scaled
// so the largest magnitude sits in [2^12, 2^13)); sx[K/32] = 128 * 2^-24 * sum of each block.
// Returns 2^24 / scale.
__device__ __forceinline__ float q8_stage_x(const void* __restrict__ x, int x_bf16, int K, __half* xhi,
                                            __half* xlo, float* sx, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto ld = [&](int i) -> float {
    return x_bf16 ? bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(x) + i))
                  : __ldg(reinterpret_cast<const float*>(x) + i);
  };
  float mx = 0.f;
  for (int i = tid; i < K; i += Q8_WARPS * 32) mx = fmaxf(mx, fabsf(ld(i)));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = 0.f;
#pragma unroll
  for (int i = 0; i < Q8_WARPS; i++) mx = fmaxf(mx, red[i]);
  float s, is;
  scale_for(mx, &s, &is);
  for (int j = tid; j < (K >> 2); j += Q8_WARPS * 32) {  // 4 elements per item, 8 items per block
    float v[4], sum = 0.f;
    __half h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      v[e] = ld(4 * j + e) * s;
      sum += v[e];
      h[e] = __float2half_rn(v[e]);
      l[e] = __float2half_rn(v[e] - __half2float(h[e]));
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if ((j & 7) == 0) sx[j >> 3] = 128.0f * GV_2M24 * sum;
    *reinterpret_cast<uint2*>(xhi + 4 * j) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(xlo + 4 * j) = *reinterpret_cast<const uint2*>(l);
  }
  return GV_2P24 * is;
}

__global__ void __launch_bounds__(Q8_WARPS * 32, 1)
gemv_cs_q8_0_kernel(const Q8Args a, const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(128) uint8_t q8_smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = q8_smem + (size_t)warp * Q8_NST * Q8_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(q8_smem + (size_t)Q8_WARPS * Q8_NST * Q8_STAGE) + warp * Q8_NST;
  __half* xhi = reinterpret_cast<__half*>(q8_smem + Q8_RING_BYTES);
  __half* xlo = xhi + a.K + 8;  // 16 bytes off a multiple of 128: hi and lo lanes hit different banks
  float* sx = reinterpret_cast<float*>(xlo + a.K + 8);
  float* red = sx + (a.K >> 5);
  pdl_trigger();  // the next kernel of the stream may start its own weight fetch
  if (threadIdx.x == 0) s_abort = 0;
  if (lane == 0) {
    for (int i = 0; i < Q8_NST; i++) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int64_t nitems = (int64_t)a.ntiles * a.S;
  const int64_t gw = (int64_t)blockIdx.x * Q8_WARPS + warp;
  const int64_t nwarps = (int64_t)gridDim.x * Q8_WARPS;
  const int64_t item_lo = nitems * gw / nwarps, item_hi = nitems * (gw + 1) / nwarps;
  const int nst = a.nst;
  const int total = item_lo < item_hi ? (int)(item_hi - item_lo) * nst : 0;
  const int S = a.S;
  const int tile_lo = (int)(item_lo / S), sl_lo = (int)(item_lo - (int64_t)tile_lo * S);
  int c_left = total, c_tile = tile_lo, c_sl = sl_lo, c_st = 0, c_slot = 0;
  auto issue = [&]() {
    if (c_left <= 0) return;
    c_left--;
    if (lane == 0) mbar_expect_tx(bars + c_slot, Q8_STAGE);
    __syncwarp();
    if (lane < 2)  // box `lane`: rows 8 * lane .. of the tile, words of unit (c_sl * nst + c_st)
      tma_box_g2s(ring + c_slot * Q8_STAGE + lane * Q8_BOX, &wmap, (c_sl * nst + c_st) * (Q8_ROWB / 4),
                  c_tile * 16 + lane * 8, bars + c_slot);
    if (++c_slot == Q8_NST) c_slot = 0;
    if (++c_st == nst) {
      c_st = 0;
      if (++c_sl == S) c_sl = 0, c_tile++;
    }
  };
#pragma unroll
  for (int q = 0; q < Q8_NST; q++) issue();

  // the weights do not depend on the kernels before this one (their first stages are in flight);
  // the activation row and the scratch words do
  pdl_wait();
  const float out_scale = q8_stage_x(a.x, a.x_bf16, a.K, xhi, xlo, sx, red);
  if (blockIdx.x == 0 && threadIdx.x == 0) a.misc[0] = out_scale;
  __syncthreads();
  if (total == 0) return;
  const bool active = (g >> 1) == t;
  const __half* xsel = (g & 1) ? xlo : xhi;
  float acc0 = 0.f, acc1 = 0.f;
  int tile = tile_lo, sl = sl_lo, slot = 0;
  unsigned parity = 0;
  for (int64_t item = item_lo; item < item_hi; item++) {
    for (int st = 0; st < nst; st++) {
      if (!mbar_wait_bounded_sleepy(bars + slot, parity, Q8_SPINS, &s_abort, 2000u)) {
        if (!s_abort) {
          s_abort = 1;
          report_wait_expired(a.error, DEV_ERR_GEMV_RING);
        }
        return;
      }
      const uint8_t* base = ring + slot * Q8_STAGE;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(base + g * Q8_ROWB) + 17 * t;
      const uint32_t* r1 = r0 + Q8_BOX / 4;
      uint32_t w0[17], w1[17];
#pragma unroll
      for (int i = 0; i < 17; i++) {
        w0[i] = r0[i];
        w1[i] = r1[i];
      }
      __syncwarp();
      issue();
      if (++slot == Q8_NST) slot = 0, parity ^= 1u;
      const int U = sl * nst + st;                       // unit index along K
      const int blk0 = U * 8 + 2 * t;                    // the lane's even block; the odd one follows
      // two blocks x two accumulators (even / odd steps): four independent mma chains
      float c[2][2][4];
#pragma unroll
      for (int e = 0; e < 2; e++)
#pragma unroll
        for (int k = 0; k < 2; k++) c[e][k][0] = c[e][k][1] = c[e][k][2] = c[e][k][3] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {  // uint4 j of a block = elements 8j .. 8j+7 = steps 2j, 2j+1
        uint4 bf[2];
#pragma unroll
        for (int e = 0; e < 2; e++)
          bf[e] = active ? *reinterpret_cast<const uint4*>(xsel + (size_t)(blk0 + e) * 32 + 8 * j)
                         : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < 2; k++) {
          const int i = 2 * j + k;  // quant word = mma step
#pragma unroll
          for (int e = 0; e < 2; e++) {
            uint32_t q0, q1;
            if (e == 0) {  // even block: quants start 2 bytes into word 0
              q0 = __funnelshift_r(w0[i], w0[i + 1], 16);
              q1 = __funnelshift_r(w1[i], w1[i + 1], 16);
            } else {       // odd block: words 9..16
              q0 = w0[9 + i];
              q1 = w1[9 + i];
            }
            q0 ^= 0x80808080u;  // int8 -> biased unsigned byte
            q1 ^= 0x80808080u;
            mma_f16_16816(c[e][k], __byte_perm(q0, 0, 0x4140), __byte_perm(q1, 0, 0x4140),
                          __byte_perm(q0, 0, 0x4342), __byte_perm(q1, 0, 0x4342), k ? bf[e].z : bf[e].x,
                          k ? bf[e].w : bf[e].y);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const __half2 h0 = *reinterpret_cast<const __half2*>(&w0[e ? 8 : 0]);
        const __half2 h1 = *reinterpret_cast<const __half2*>(&w1[e ? 8 : 0]);
        const float d0 = e ? __high2float(h0) : __low2float(h0);
        const float d1 = e ? __high2float(h1) : __low2float(h1);
        const float sxv = sx[blk0 + e];
        acc0 = fmaf(d0, ((c[e][0][0] + c[e][0][1]) + (c[e][1][0] + c[e][1][1])) - sxv, acc0);
        acc1 = fmaf(d1, ((c[e][0][2] + c[e][0][3]) + (c[e][1][2] + c[e][1][3])) - sxv, acc1);
      }
    }
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) {
      const int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
      if (S == 1) {
        if (row0 < a.N) a.y[row0] = acc0 * out_scale + (a.residual ? a.residual[row0] : 0.f);
        if (row1 < a.N) a.y[row1] = acc1 * out_scale + (a.residual ? a.residual[row1] : 0.f);
      } else {
        if (row0 < a.N) a.partial[(int64_t)sl * a.N + row0] = acc0;
        if (row1 < a.N) a.partial[(int64_t)sl * a.N + row1] = acc1;
      }
    }
    acc0 = acc1 = 0.f;
    if (++sl == S) sl = 0, tile++;
  }
}

__global__ void __launch_bounds__(256)
q8_reduce_kernel(const float* __restrict__ partial, int S, int64_t N, const float* __restrict__ misc, float* y,
                 const float* residual) {
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

size_t q8_smem_bytes(int K) {
  return (size_t)Q8_RING_BYTES + 2 * ((size_t)K + 8) * 2 + (size_t)(K >> 5) * 4 + 128;
}

struct Q8Plan {
  int S, nst, ntiles, grid;
  size_t smem, bytes;
};

void q8_plan(const WRef& w, Q8Plan* p) {
  const int K = (int)w.cols, stages = K / Q8_KSTAGE;
  p->ntiles = (int)((w.rows + 15) / 16);
  const int sms = std::max(1, sm_count());
  const int64_t warps = (int64_t)sms * Q8_WARPS;
  int S = 1;
  for (int cand = 1; cand <= stages; cand++) {
    if (stages % cand) continue;
    S = cand;
    if ((int64_t)p->ntiles * cand >= 8 * warps) break;
  }
  p->S = S;
  p->nst = stages / S;
  const int64_t items = (int64_t)p->ntiles * S;
  p->grid = (int)std::min<int64_t>(sms, (items + Q8_WARPS - 1) / Q8_WARPS);
  p->smem = q8_smem_bytes(K);
  p->bytes = 256 + (S > 1 ? (size_t)S * w.rows * 4 : 0);
}

}  // namespace

bool gemv_cs_q8_0_shape_ok(const WRef& w, int M) {
  return M == 1 && w.enc == E_Q8_0 && w.rows >= 1 && w.cols >= Q8_KSTAGE && w.cols % Q8_KSTAGE == 0 &&
         q8_smem_bytes((int)w.cols) <= (size_t)Q8_MAX_SMEM && (reinterpret_cast<uintptr_t>(w.data) & 15) == 0;
}

size_t gemv_cs_q8_0_workspace_bytes(const WRef& w, int M) {
  if (!gemv_cs_q8_0_shape_ok(w, M)) return 0;
  Q8Plan p;
  q8_plan(w, &p);
  return p.bytes;
}

int launch_gemv_cs_q8_0(const WRef& w, const void* x, int x_type, float* y, const float* residual, uint8_t* ws,
                        cudaStream_t s) {
  Q8Plan p;
  q8_plan(w, &p);
  Q8Args a;
  a.N = w.rows, a.K = (int)w.cols;
  CUtensorMap wmap;
  if (make_row_box_map(w.data, w.row_bytes(), w.rows, Q8_ROWB / 4, 8, &wmap)) return 1;
  a.S = p.S, a.nst = p.nst, a.ntiles = p.ntiles;
  a.x = x, a.x_bf16 = x_type == E_BF16 ? 1 : 0;
  a.error = device_error_word();
  if (!a.error) return 1;
  a.misc = reinterpret_cast<float*>(ws + 64);
  a.partial = reinterpret_cast<float*>(ws + 256);
  a.y = y, a.residual = residual;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_cs_q8_0_kernel), Q8_MAX_SMEM)) return 1;
  DYN_CUDA(launch_pdl(gemv_cs_q8_0_kernel, dim3(p.grid), dim3(Q8_WARPS * 32), p.smem, s, a, wmap));
  count_launch(1);
  Deferred* defer = p.S > 1 && !residual ? defer_take() : nullptr;
  if (defer) {
    defer->partial = a.partial, defer->scale = a.misc, defer->S = p.S, defer->N = w.rows, defer->ws_bytes = p.bytes;
  } else if (p.S > 1) {
    DYN_CUDA(launch_pdl(q8_reduce_kernel, dim3((unsigned)((w.rows + 255) / 256)), dim3(256), 0, s, (const float*)a.partial,
                        p.S, (int64_t)w.rows, (const float*)a.misc, y, residual));
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace dyn
