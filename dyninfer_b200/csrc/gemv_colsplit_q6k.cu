// Column-split tensor-core GEMV for ONE activation row on Q6_K rows (the tied lm_head of the
// Qwen3-shape models is Q6_K; decode rule crates/dyninfer-kernel-registry/src/gguf_codegen.rs:474-526:
// element n*128 + h*64 + p*32 + j has low nibble in ql byte n*64 + p*32 + j (nibble h), two high
// bits in qh byte n*32 + j (field h*2 + p), int8 scale n*8 + h*4 + p*2 + j/16, w = d * sc * (q - 32)).
//
// Same idea as the Q4_0 kernel (gemv_colsplit.cu): the 8 output columns of mma.sync.m16n8k16
// keep four 16-element sub-blocks apart, so a lane owns whole sub-blocks. Lane quarter t = (p, s)
// reads, for each half n of a superblock, the 16 ql bytes n*64 + 16t .. +15 (they hold sub-blocks
// (n, h=0, p, s) in the low and (n, h=1, p, s) in the high nibbles) and the 16 qh bytes
// n*32 + 16s .. +15; it merges nibble and 2-bit field into bytes 0..63, widens them to f16
// subnormals (exact) with byte permutes and feeds four mma steps per sub-block; its accumulator
// columns 2t / 2t+1 (hi / lo part of the activation) then hold exactly that sub-block, whose scale
// index is n*8 + h*4 + t. The activations stay in natural order (sub-block = 16 consecutive
// elements), as two f16 arrays hi and lo in shared memory.
//
// Data movement: per warp a ring of two stages of 16 rows x 2 superblocks (420 bytes). A stage's
// 420 bytes of a row start anywhere on the 4-byte grid, so every copy starts at the 16-byte boundary
// below the first byte (432 bytes per row) and the lane adds the remainder when it reads; the second
// superblock of a stage sits 2 bytes off the word grid and is read with funnel shifts. The copies are
// 2-D tensor copies where the layout allows a tensor map (row strides must be multiples of 16 bytes):
// rows of a multiple of 16 bytes (K a multiple of 2048) as one box of 16 rows per stage; rows of
// 8 mod 16 bytes (K = 1024, 5120: the lm_head) with an even row count as a matrix of ROW PAIRS, one box
// of 8 pairs for the stage's even rows and one for its odd rows (in shared memory: even rows first) --
// two requests to the copy engine instead of sixteen. Otherwise one cp.async.bulk per row. All waits are
// bounded.
#include <algorithm>

#include "gemv_core.cuh"
#include "ring.cuh"
#include "tensor_map.cuh"

namespace dyn {

namespace {

constexpr int Q6_WARPS = 12;
constexpr int Q6_NST = 2;
constexpr int Q6_ROWB = 420;     // two superblocks
constexpr int Q6_COPYB = 432;    // bytes copied per row: 420 + up to 12 of misalignment, rounded to 16
constexpr int Q6_PITCH = 432;
constexpr int Q6_STAGE = 16 * Q6_PITCH;
constexpr int Q6_KSTAGE = 512;
constexpr long long Q6_SPINS = 1LL << 22;
constexpr int Q6_MAX_SMEM = 226 * 1024;
constexpr int Q6_RING_BYTES = Q6_WARPS * Q6_NST * Q6_STAGE + Q6_WARPS * Q6_NST * 8;

struct Q6Args {
  const uint8_t* data;
  int64_t N, rb;
  int K, S, nst, ntiles;
  const void* x;
  int x_bf16;
  float* misc;  // [0] = 2^24 / scale
  float* y;
  const float* residual;
  float* partial;
  int* error;
  int mode;  // how a stage is copied: 0 one bulk copy per row, 1 one box of 16 rows, 2 two boxes of 8 row pairs
};

// Activation row -> shared memory: xhi[K], 16 bytes of padding, xlo[K] (f16, natural order, scaled
// so the largest magnitude sits in [2^12, 2^13)); sx[K/16] = 32 * 2^-24 * sum of each 16-run.
// Returns 2^24 / scale.
__device__ __forceinline__ float q6_stage_x(const void* __restrict__ x, int x_bf16, int K, __half* xhi,
                                            __half* xlo, float* sx, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto ld = [&](int i) -> float {
    return x_bf16 ? bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(x) + i))
                  : __ldg(reinterpret_cast<const float*>(x) + i);
  };
  float mx = 0.f;
  for (int i = tid; i < K; i += Q6_WARPS * 32) mx = fmaxf(mx, fabsf(ld(i)));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = 0.f;
#pragma unroll
  for (int i = 0; i < Q6_WARPS; i++) mx = fmaxf(mx, red[i]);
  float s, is;
  scale_for(mx, &s, &is);
  for (int j = tid; j < (K >> 2); j += Q6_WARPS * 32) {  // 4 elements per item, 4 items per 16-run
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
    if ((j & 3) == 0) sx[j >> 2] = 32.0f * GV_2M24 * sum;
    *reinterpret_cast<uint2*>(xhi + 4 * j) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(xlo + 4 * j) = *reinterpret_cast<const uint2*>(l);
  }
  return GV_2P24 * is;
}

// 16 bytes at `p` (p 4-byte aligned, MIS = 0) or at p + 2 with p 4-byte aligned... the caller
// passes the address of the first wanted byte; MIS = (address & 3) known at compile time.
template <int MIS>
__device__ __forceinline__ void ld16(const uint8_t* q, uint32_t (&w)[4]) {
  if (MIS == 0) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(q);
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = p[i];
  } else {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(q - 2);
    uint32_t r[5];
#pragma unroll
    for (int i = 0; i < 5; i++) r[i] = p[i];
#pragma unroll
    for (int i = 0; i < 4; i++) w[i] = __funnelshift_r(r[i], r[i + 1], 16);
  }
}

// One superblock of the lane's two rows (b0, b1: first byte of the superblock in each row).
template <int MIS>
__device__ __forceinline__ void q6_superblock(const uint8_t* b0, const uint8_t* b1, int t, bool active, int g,
                                              const __half* xhi, const __half* xlo, const float* sx, int kbase,
                                              float& acc0, float& acc1) {
  const int p = t >> 1, s = t & 1;
  const float d0 = __half2float(*reinterpret_cast<const __half*>(b0 + 208));
  const float d1 = __half2float(*reinterpret_cast<const __half*>(b1 + 208));
#pragma unroll
  for (int n = 0; n < 2; n++) {
    uint32_t ql0[4], ql1[4], qh0[4], qh1[4];
    ld16<MIS>(b0 + n * 64 + 16 * t, ql0);
    ld16<MIS>(b1 + n * 64 + 16 * t, ql1);
    ld16<MIS>(b0 + 128 + n * 32 + 16 * s, qh0);
    ld16<MIS>(b1 + 128 + n * 32 + 16 * s, qh1);
    float c[2][4];
#pragma unroll
    for (int h = 0; h < 2; h++) c[h][0] = c[h][1] = c[h][2] = c[h][3] = 0.f;
    // the lane's 16 activations of sub-block (n, h, p, s): elements kbase + n*128 + h*64 + 16t ..
    uint4 bf[2][2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const __half* xs = ((g & 1) ? xlo : xhi) + kbase + n * 128 + h * 64 + 16 * t;
#pragma unroll
      for (int ip = 0; ip < 2; ip++)
        bf[h][ip] = active ? *reinterpret_cast<const uint4*>(xs + 8 * ip) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int shq = 4 * h + 2 * p;  // qh field of (h, p)
        const uint32_t v0 = ((ql0[i] >> (4 * h)) & 0x0F0F0F0Fu) | (((qh0[i] >> shq) & 0x03030303u) << 4);
        const uint32_t v1 = ((ql1[i] >> (4 * h)) & 0x0F0F0F0Fu) | (((qh1[i] >> shq) & 0x03030303u) << 4);
        const uint4 b = bf[h][i >> 1];
        mma_f16_16816(c[h], __byte_perm(v0, 0, 0x4140), __byte_perm(v1, 0, 0x4140), __byte_perm(v0, 0, 0x4342),
                      __byte_perm(v1, 0, 0x4342), (i & 1) ? b.z : b.x, (i & 1) ? b.w : b.y);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int si = n * 8 + h * 4 + t;
      const float f0 = d0 * (float)*reinterpret_cast<const int8_t*>(b0 + 192 + si);
      const float f1 = d1 * (float)*reinterpret_cast<const int8_t*>(b1 + 192 + si);
      const float sxv = sx[(kbase >> 4) + si];
      acc0 = fmaf(f0, (c[h][0] + c[h][1]) - sxv, acc0);
      acc1 = fmaf(f1, (c[h][2] + c[h][3]) - sxv, acc1);
    }
  }
}

__global__ void __launch_bounds__(Q6_WARPS * 32, 1)
gemv_cs_q6k_kernel(const Q6Args a, const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(128) uint8_t q6_smem[];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = q6_smem + (size_t)warp * Q6_NST * Q6_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(q6_smem + (size_t)Q6_WARPS * Q6_NST * Q6_STAGE) + warp * Q6_NST;
  __half* xhi = reinterpret_cast<__half*>(q6_smem + Q6_RING_BYTES);
  __half* xlo = xhi + a.K + 8;  // 16 bytes apart from a multiple of 128: hi and lo lanes hit different banks
  float* sx = reinterpret_cast<float*>(xlo + a.K + 8);
  float* red = sx + (a.K >> 4);
  pdl_trigger();  // the next kernel of the stream may start its own weight fetch
  if (threadIdx.x == 0) s_abort = 0;
  if (lane == 0) {
    for (int i = 0; i < Q6_NST; i++) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int64_t nitems = (int64_t)a.ntiles * a.S;
  const int64_t gw = (int64_t)blockIdx.x * Q6_WARPS + warp;
  const int64_t nwarps = (int64_t)gridDim.x * Q6_WARPS;
  const int64_t item_lo = nitems * gw / nwarps, item_hi = nitems * (gw + 1) / nwarps;
  const int nst = a.nst;
  const int total = item_lo < item_hi ? (int)(item_hi - item_lo) * nst : 0;
  const int S = a.S;
  const int tile_lo = (int)(item_lo / S), sl_lo = (int)(item_lo - (int64_t)tile_lo * S);
  int c_left = total, c_tile = tile_lo, c_sl = sl_lo, c_st = 0, c_slot = 0;
  const int64_t last_row = a.N - 1;
  auto issue = [&]() {
    if (c_left <= 0) return;
    c_left--;
    if (lane == 0) mbar_expect_tx(bars + c_slot, 16 * Q6_COPYB);
    __syncwarp();
    if (a.mode) {
      if (lane == 0) {
        const int64_t coff = (int64_t)(c_sl * nst + c_st) * Q6_ROWB;
        uint8_t* dst = ring + c_slot * Q6_STAGE;
        if (a.mode == 1) {
          tma_box_g2s(dst, &wmap, (int)((coff >> 4) << 2), c_tile * 16, bars + c_slot);
        } else {
          tma_box_g2s(dst, &wmap, (int)((coff >> 4) << 2), c_tile * 8, bars + c_slot);
          tma_box_g2s(dst + 8 * Q6_PITCH, &wmap, (int)(((a.rb + coff) >> 4) << 2), c_tile * 8, bars + c_slot);
        }
      }
    } else if (lane < 16) {
      int64_t row = (int64_t)c_tile * 16 + lane;
      if (row > last_row) row = last_row;
      const uint8_t* src = a.data + row * a.rb + (int64_t)(c_sl * nst + c_st) * Q6_ROWB;
      src -= reinterpret_cast<uintptr_t>(src) & 15;
      bulk_g2s(ring + c_slot * Q6_STAGE + lane * Q6_PITCH, src, Q6_COPYB, bars + c_slot);
    }
    if (++c_slot == Q6_NST) c_slot = 0;
    if (++c_st == nst) {
      c_st = 0;
      if (++c_sl == S) c_sl = 0, c_tile++;
    }
  };
#pragma unroll
  for (int q = 0; q < Q6_NST; q++) issue();

  // the weights do not depend on the kernels before this one (their first stages are in flight);
  // the activation row and the scratch words do
  pdl_wait();
  const float out_scale = q6_stage_x(a.x, a.x_bf16, a.K, xhi, xlo, sx, red);
  if (blockIdx.x == 0 && threadIdx.x == 0) a.misc[0] = out_scale;
  __syncthreads();
  if (total == 0) return;
  const bool active = (g >> 1) == t;
  float acc0 = 0.f, acc1 = 0.f;
  int tile = tile_lo, sl = sl_lo, slot = 0;
  unsigned parity = 0;
  for (int64_t item = item_lo; item < item_hi; item++) {
    // where the lane's two rows start inside their 16-byte aligned copies (same for every stage of
    // the item only if 420 * stage keeps the remainder; recomputed per stage below)
    int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
    const int64_t r0c = row0 > last_row ? last_row : row0, r1c = row1 > last_row ? last_row : row1;
    for (int st = 0; st < nst; st++) {
      if (!mbar_wait_bounded_sleepy(bars + slot, parity, Q6_SPINS, &s_abort, 2000u)) {
        if (!s_abort) {
          s_abort = 1;
          report_wait_expired(a.error, DEV_ERR_GEMV_RING);
        }
        return;
      }
      const int64_t coff = (int64_t)(sl * nst + st) * Q6_ROWB;
      const uint32_t off0 = (uint32_t)(reinterpret_cast<uintptr_t>(a.data + r0c * a.rb + coff) & 15);
      const uint32_t off1 = (uint32_t)(reinterpret_cast<uintptr_t>(a.data + r1c * a.rb + coff) & 15);
      const uint8_t* base = ring + slot * Q6_STAGE;
      // rows g and g + 8 of the tile; pair mode keeps the tile's even rows in the first eight slots
      const int sr0 = a.mode == 2 ? (g & 1) * 8 + (g >> 1) : g;
      const int sr1 = a.mode == 2 ? sr0 + 4 : g + 8;
      const uint8_t* b0 = base + sr0 * Q6_PITCH + off0;
      const uint8_t* b1 = base + sr1 * Q6_PITCH + off1;
      const int kbase = (sl * nst + st) * Q6_KSTAGE;
      q6_superblock<0>(b0, b1, t, active, g, xhi, xlo, sx, kbase, acc0, acc1);
      q6_superblock<2>(b0 + 210, b1 + 210, t, active, g, xhi, xlo, sx, kbase + 256, acc0, acc1);
      __syncwarp();
      issue();
      if (++slot == Q6_NST) slot = 0, parity ^= 1u;
    }
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) {
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
q6_reduce_kernel(const float* __restrict__ partial, int S, int64_t N, const float* __restrict__ misc, float* y,
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

size_t q6_smem_bytes(int K) {
  return (size_t)Q6_RING_BYTES + 2 * ((size_t)K + 8) * 2 + (size_t)(K >> 4) * 4 + 128;
}

struct Q6Plan {
  int S, nst, ntiles, grid;
  size_t smem, bytes;
};

void q6_plan(const WRef& w, Q6Plan* p) {
  const int K = (int)w.cols, stages = K / Q6_KSTAGE;
  p->ntiles = (int)((w.rows + 15) / 16);
  const int sms = std::max(1, sm_count());
  const int64_t warps = (int64_t)sms * Q6_WARPS;
  int S = 1;
  for (int cand = 1; cand <= stages; cand++) {
    if (stages % cand) continue;
    S = cand;
    if ((int64_t)p->ntiles * cand >= 8 * warps) break;
  }
  p->S = S;
  p->nst = stages / S;
  const int64_t items = (int64_t)p->ntiles * S;
  p->grid = (int)std::min<int64_t>(sms, (items + Q6_WARPS - 1) / Q6_WARPS);
  p->smem = q6_smem_bytes(K);
  p->bytes = 256 + (S > 1 ? (size_t)S * w.rows * 4 : 0);
}

}  // namespace

bool gemv_cs_q6k_shape_ok(const WRef& w, int M) {
  return M == 1 && w.enc == E_Q6_K && w.rows >= 1 && w.cols >= Q6_KSTAGE && w.cols % Q6_KSTAGE == 0 &&
         q6_smem_bytes((int)w.cols) <= (size_t)Q6_MAX_SMEM && (reinterpret_cast<uintptr_t>(w.data) & 15) == 0;
}

size_t gemv_cs_q6k_workspace_bytes(const WRef& w, int M) {
  if (!gemv_cs_q6k_shape_ok(w, M)) return 0;
  Q6Plan p;
  q6_plan(w, &p);
  return p.bytes;
}

// The weight buffer must stay readable for 12 bytes past its last row (row copies are rounded up
// to 16 bytes); session arenas and the operator API's device weights keep 64 bytes of slack.
int launch_gemv_cs_q6k(const WRef& w, const void* x, int x_type, float* y, const float* residual, uint8_t* ws,
                       cudaStream_t s) {
  Q6Plan p;
  q6_plan(w, &p);
  Q6Args a;
  a.data = w.data, a.N = w.rows, a.rb = w.row_bytes(), a.K = (int)w.cols;
  a.S = p.S, a.nst = p.nst, a.ntiles = p.ntiles;
  a.x = x, a.x_bf16 = x_type == E_BF16 ? 1 : 0;
  a.error = device_error_word();
  if (!a.error) return 1;
  a.misc = reinterpret_cast<float*>(ws + 64);
  a.partial = reinterpret_cast<float*>(ws + 256);
  a.y = y, a.residual = residual;
  CUtensorMap wmap;
  memset(&wmap, 0, sizeof wmap);
  a.mode = 0;
  static_assert(Q6_COPYB % 16 == 0 && Q6_PITCH == Q6_COPYB && (8 * Q6_PITCH) % 128 == 0, "boxes land row after row");
  if (a.rb % 16 == 0) {
    if (make_row_box_map(w.data, (size_t)a.rb, w.rows, Q6_COPYB / 4, 16, &wmap)) return 1;
    a.mode = 1;
  } else if (a.rb % 8 == 0 && w.rows % 2 == 0) {
    if (make_row_box_map(w.data, (size_t)a.rb * 2, w.rows / 2, Q6_COPYB / 4, 8, &wmap)) return 1;
    a.mode = 2;
  }
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_cs_q6k_kernel), Q6_MAX_SMEM)) return 1;
  DYN_CUDA(launch_pdl(gemv_cs_q6k_kernel, dim3(p.grid), dim3(Q6_WARPS * 32), p.smem, s, a, wmap));
  count_launch(1);
  Deferred* defer = p.S > 1 && !residual ? defer_take() : nullptr;
  if (defer) {
    defer->partial = a.partial, defer->scale = a.misc, defer->S = p.S, defer->N = w.rows, defer->ws_bytes = p.bytes;
  } else if (p.S > 1) {
    DYN_CUDA(launch_pdl(q6_reduce_kernel, dim3((unsigned)((w.rows + 255) / 256)), dim3(256), 0, s, (const float*)a.partial,
                        p.S, (int64_t)w.rows, (const float*)a.misc, y, residual));
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace dyn
