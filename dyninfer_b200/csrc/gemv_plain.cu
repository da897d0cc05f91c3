// Streaming GEMV for plain bf16 / f16 weights and one to four activation rows (f32 accumulate).
//
// The dense path of the reference widens bf16 / f16 to f32 exactly and multiplies in f32
// (crates/dyninfer-compiler/src/lowering/kernels.rs:741-772,1157-1173); the only such matrix on the
// decode path is a tied bf16 embedding table used as lm_head (151936 x 1024 = 311 MB per step), so
// this kernel is HBM-bound: 2 bytes per weight, one widening and one FMA per weight and row.
//
// A warp owns whole weight rows; a lane reads 16 bytes (8 weights) of a row at a time, four rows
// in flight (64 bytes per lane outstanding, 8 KB per warp), widens them with one shift or mask
// each, multiplies by the activation row held in shared memory as f32 and reduces over the warp
// with shuffles. Rows are dealt to warps in blocks so that the grid is one CTA per SM and every
// warp streams one contiguous run of the matrix.
#include <algorithm>

#include "common.cuh"

namespace dyn {
namespace {

constexpr int GP_WARPS = 16;
constexpr int GP_UNROLL = 4;  // weight rows in flight per warp

template <bool BF16>
__device__ __forceinline__ void widen8(const uint4& w, float (&f)[8]) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    if (BF16) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    } else {
      f[2 * i] = __half2float(__ushort_as_half((unsigned short)(u[i] & 0xffffu)));
      f[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(u[i] >> 16)));
    }
  }
}

// y[m][n] = sum_k x[m][k] * w[n][k] (+ residual). K % 256 == 0, M <= 4.
template <bool BF16, int M>
__global__ void __launch_bounds__(GP_WARPS * 32) gemv_plain_kernel(const uint8_t* __restrict__ w, int64_t N, int K,
                                                                   const void* __restrict__ x, int x_bf16,
                                                                   float* __restrict__ y,
                                                                   const float* __restrict__ residual) {
  extern __shared__ __align__(16) float gp_xs[];  // [M][K]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();
  // the weights do not depend on earlier kernels of the stream; the activations do
  pdl_wait();
  for (int i = tid; i < M * K; i += GP_WARPS * 32)
    gp_xs[i] = x_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i])
                      : reinterpret_cast<const float*>(x)[i];
  __syncthreads();
  const int64_t warps = (int64_t)gridDim.x * GP_WARPS, wid = (int64_t)blockIdx.x * GP_WARPS + warp;
  const int64_t lo = N * wid / warps, hi = N * (wid + 1) / warps;
  const size_t rb = (size_t)K * 2;
  for (int64_t r0 = lo; r0 < hi; r0 += GP_UNROLL) {
    float acc[GP_UNROLL][M];
#pragma unroll
    for (int j = 0; j < GP_UNROLL; j++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[j][m] = 0.f;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
      uint4 wv[GP_UNROLL];
#pragma unroll
      for (int j = 0; j < GP_UNROLL; j++) {
        const int64_t r = r0 + j < hi ? r0 + j : hi - 1;  // clamp: the last block repeats a row it owns
        wv[j] = __ldcs(reinterpret_cast<const uint4*>(w + r * rb + (size_t)k0 * 2));  // streamed once
      }
      float xv[M][8];
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float4 a = *reinterpret_cast<const float4*>(gp_xs + m * K + k0);
        const float4 b = *reinterpret_cast<const float4*>(gp_xs + m * K + k0 + 4);
        xv[m][0] = a.x, xv[m][1] = a.y, xv[m][2] = a.z, xv[m][3] = a.w;
        xv[m][4] = b.x, xv[m][5] = b.y, xv[m][6] = b.z, xv[m][7] = b.w;
      }
#pragma unroll
      for (int j = 0; j < GP_UNROLL; j++) {
        float f[8];
        widen8<BF16>(wv[j], f);
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
          for (int i = 0; i < 8; i++) acc[j][m] = fmaf(xv[m][i], f[i], acc[j][m]);
      }
    }
#pragma unroll
    for (int j = 0; j < GP_UNROLL; j++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float v = warp_sum(acc[j][m]);
        const int64_t r = r0 + j;
        if (lane == 0 && r < hi) y[(int64_t)m * N + r] = residual ? v + residual[(int64_t)m * N + r] : v;
      }
  }
}

template <bool BF16, int M>
int run_plain(const WRef& w, const void* x, int x_type, float* y, const float* residual, cudaStream_t s) {
  const int K = (int)w.cols;
  const size_t smem = (size_t)M * K * 4;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_plain_kernel<BF16, M>), (int)std::max<size_t>(smem, 48 * 1024)))
    return 1;
  const int sms = std::max(1, sm_count());
  const int grid = (int)std::min<int64_t>(sms, (w.rows + GP_WARPS - 1) / GP_WARPS);
  DYN_CUDA(launch_pdl(gemv_plain_kernel<BF16, M>, dim3(grid), dim3(GP_WARPS * 32), smem, s, w.data, (int64_t)w.rows, K,
                      x, x_type == E_BF16 ? 1 : 0, y, residual));
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

// *handled = false when the encoding or shape does not qualify (the caller uses another kernel).
int launch_gemv_plain(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                      cudaStream_t s, bool* handled) {
  *handled = false;
  if ((w.enc != E_BF16 && w.enc != E_F16) || M < 1 || M > 4 || w.cols % 256 != 0 || w.rows < 1 ||
      (size_t)M * w.cols * 4 > 160 * 1024 || (reinterpret_cast<uintptr_t>(w.data) & 15))
    return 0;
  int rc;
  const bool bf = w.enc == E_BF16;
  switch (M) {
    case 1: rc = bf ? run_plain<true, 1>(w, x, x_type, y, residual, s) : run_plain<false, 1>(w, x, x_type, y, residual, s); break;
    case 2: rc = bf ? run_plain<true, 2>(w, x, x_type, y, residual, s) : run_plain<false, 2>(w, x, x_type, y, residual, s); break;
    case 3: rc = bf ? run_plain<true, 3>(w, x, x_type, y, residual, s) : run_plain<false, 3>(w, x, x_type, y, residual, s); break;
    default: rc = bf ? run_plain<true, 4>(w, x, x_type, y, residual, s) : run_plain<false, 4>(w, x, x_type, y, residual, s); break;
  }
  if (rc) return rc;
  *handled = true;
  return 0;
}

}  // namespace dyn
