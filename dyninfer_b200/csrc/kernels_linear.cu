// Fused dequant + matrix-vector / skinny-matrix product on the raw checkpoint
// bytes: y[m, n] = sum_k x[m, k] * w[n, k], f32 accumulation.
//
// Row-per-warp kernel: a warp walks one weight row, consecutive lanes decode
// consecutive parts (so the warp reads a contiguous byte span), every decoded
// weight is the exact f32 value the reference dequantises to, and the partial
// sums are combined with warp shuffles. Up to MT activation rows share one
// pass over the weights.
#include "codec.cuh"

namespace dyn {

constexpr int LIN_WARPS = 4;

template <bool XBF16>
__device__ __forceinline__ float4 load_x4(const void* x, int64_t idx) {
  if constexpr (XBF16) {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + idx);
    return make_float4(bf16_bits_to_f32(v.x & 0xffffu), bf16_bits_to_f32(v.x >> 16),
                       bf16_bits_to_f32(v.y & 0xffffu), bf16_bits_to_f32(v.y >> 16));
  } else {
    return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx);
  }
}

template <int ENC, int MT, bool XBF16>
__device__ __forceinline__ void row_dot(const WRef& w, int64_t row, const void* x, int m_valid,
                                        int lane, float* acc) {
  using C = Codec<ENC>;
  const RowPtr rp = row_ptr(w, row);
  const int64_t K = w.cols;
  const int64_t nparts = (K / C::BLOCK) * C::PARTS;
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int64_t it = lane; it < nparts; it += 32) {
    const int64_t blk = it / C::PARTS;
    const int part = (int)(it - blk * C::PARTS);
    float wv[4 * C::G];
    C::decode(rp, blk, part, wv);
#pragma unroll
    for (int g = 0; g < C::G; g++) {
      const int64_t k0 = blk * C::BLOCK + C::xoff(part, g);
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const int mm = m < m_valid ? m : m_valid - 1;
        const float4 xv = load_x4<XBF16>(x, (int64_t)mm * K + k0);
        acc[m] = fmaf(wv[4 * g + 0], xv.x, acc[m]);
        acc[m] = fmaf(wv[4 * g + 1], xv.y, acc[m]);
        acc[m] = fmaf(wv[4 * g + 2], xv.z, acc[m]);
        acc[m] = fmaf(wv[4 * g + 3], xv.w, acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = warp_sum(acc[m]);
}

template <int ENC, int MT, bool XBF16>
__global__ void __launch_bounds__(LIN_WARPS * 32)
linear_rows_kernel(WRef w, const void* __restrict__ x, int m_valid, float* y,
                   const float* residual) {  // residual may alias y
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * LIN_WARPS + warp;
  if (row >= w.rows) return;
  float acc[MT];
  row_dot<ENC, MT, XBF16>(w, row, x, m_valid, lane, acc);
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; m++)
      if (m < m_valid) {
        float v = acc[m];
        if (residual) v += residual[(int64_t)m * w.rows + row];
        y[(int64_t)m * w.rows + row] = v;
      }
  }
}

// gate and up share the activation pass; y = silu(g) * u with
// silu(g) = g / (1 + exp(-g)) (crates/dyninfer-compiler/src/lowering/dense_decoder.rs:1379-1385).
template <int ENC, int MT>
__global__ void __launch_bounds__(LIN_WARPS * 32)
linear_swiglu_kernel(WRef wg, WRef wu, const float* __restrict__ x, int m_valid,
                     float* __restrict__ y) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * LIN_WARPS + warp;
  if (row >= wg.rows) return;
  float g[MT], u[MT];
  row_dot<ENC, MT, false>(wg, row, x, m_valid, lane, g);
  row_dot<ENC, MT, false>(wu, row, x, m_valid, lane, u);
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; m++)
      if (m < m_valid) y[(int64_t)m * wg.rows + row] = (g[m] / (1.0f + expf(-g[m]))) * u[m];
  }
}

template <int ENC, bool XBF16>
static int run_linear(const WRef& w, const void* x, int64_t m, float* y, const float* residual,
                      cudaStream_t s) {
  const unsigned grid = (unsigned)((w.rows + LIN_WARPS - 1) / LIN_WARPS);
  const size_t xe = XBF16 ? 2 : 4;
  for (int64_t m0 = 0; m0 < m; m0 += 8) {
    const int mv = (int)((m - m0) < 8 ? (m - m0) : 8);
    const void* xp = reinterpret_cast<const uint8_t*>(x) + (size_t)m0 * w.cols * xe;
    float* yp = y + m0 * w.rows;
    const float* rp = residual ? residual + m0 * w.rows : nullptr;
    if (mv == 1)
      linear_rows_kernel<ENC, 1, XBF16><<<grid, LIN_WARPS * 32, 0, s>>>(w, xp, mv, yp, rp);
    else if (mv == 2)
      linear_rows_kernel<ENC, 2, XBF16><<<grid, LIN_WARPS * 32, 0, s>>>(w, xp, mv, yp, rp);
    else if (mv <= 4)
      linear_rows_kernel<ENC, 4, XBF16><<<grid, LIN_WARPS * 32, 0, s>>>(w, xp, mv, yp, rp);
    else
      linear_rows_kernel<ENC, 8, XBF16><<<grid, LIN_WARPS * 32, 0, s>>>(w, xp, mv, yp, rp);
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  return 0;
}

int launch_linear(const WRef& w, const void* x, int x_type, int64_t m, float* y,
                  const float* residual, cudaStream_t s) {
  DYN_CHECK(x_type == E_F32 || x_type == E_BF16, "linear: x_type must be f32 or bf16, got %d",
            x_type);
  DYN_CHECK(m >= 1, "linear: m must be >= 1");
  // more rows than one pass of the tensor-core GEMV takes (4 with f32 activations, 8 with bf16):
  // dequant-in-shared-memory tensor-core GEMM, one pass over the weights for all rows
  // (below 17 rows only for the encodings with a word-fetching GEMM producer, which beats repeated GEMV
  // passes: the GEMM's dequantisation cost does not shrink with the row count)
  const bool cheap_producer = w.enc == E_Q4_0 || w.enc == E_Q4_1 || w.enc == E_Q8_0 || w.enc == E_Q6_K ||
                              w.enc == E_Q4_K || w.enc == E_Q5_K || w.enc == E_IQ4_XS || w.enc == E_MLX_U4;
  if (m > 16 || (cheap_producer && m > (x_type == E_BF16 ? 8 : 4))) {
    bool handled = false;
    if (launch_dqgemm_tc(w, x, x_type, m, y, residual, s, &handled)) return 1;
    if (handled) return 0;
  }
  if (m <= 4 && (w.enc == E_BF16 || w.enc == E_F16)) {
    // plain 2-byte weights (a tied bf16 embedding table as lm_head): streaming kernel
    bool handled = false;
    if (launch_gemv_plain(w, x, x_type, (int)m, y, residual, s, &handled)) return 1;
    if (handled) return 0;
  }
  {
    // few rows: tensor-core GEMV, 4 (f32) or 8 (bf16) activation rows per pass over the weights
    const int64_t step = x_type == E_BF16 ? 8 : 4;
    const size_t xe = x_type == E_BF16 ? 2 : 4;
    int64_t m0 = 0;
    for (; m0 < m && m <= 16; m0 += step) {
      const int mv = (int)((m - m0) < step ? (m - m0) : step);
      bool handled = false;
      if (launch_gemv_mma(w, reinterpret_cast<const uint8_t*>(x) + (size_t)m0 * w.cols * xe, x_type, mv,
                          y + m0 * w.rows, residual ? residual + m0 * w.rows : nullptr, nullptr, s,
                          &handled))
        return 1;
      if (!handled) break;
    }
    if (m0 >= m) return 0;
    if (m0 > 0) {  // cannot happen: the first chunk decides for the whole shape
      x = reinterpret_cast<const uint8_t*>(x) + (size_t)m0 * w.cols * xe;
      y += m0 * w.rows;
      if (residual) residual += m0 * w.rows;
      m -= m0;
    }
  }
  if (x_type == E_BF16) {
    DYN_ENC_SWITCH(w.enc, return (run_linear<ENC, true>(w, x, m, y, residual, s)));
  } else {
    DYN_ENC_SWITCH(w.enc, return (run_linear<ENC, false>(w, x, m, y, residual, s)));
  }
  return 0;
}

template <int ENC>
static int run_swiglu(const WRef& wg, const WRef& wu, const float* x, int64_t m, float* y,
                      cudaStream_t s) {
  const unsigned grid = (unsigned)((wg.rows + LIN_WARPS - 1) / LIN_WARPS);
  for (int64_t m0 = 0; m0 < m; m0 += 4) {
    const int mv = (int)((m - m0) < 4 ? (m - m0) : 4);
    const float* xp = x + m0 * wg.cols;
    float* yp = y + m0 * wg.rows;
    if (mv == 1)
      linear_swiglu_kernel<ENC, 1><<<grid, LIN_WARPS * 32, 0, s>>>(wg, wu, xp, mv, yp);
    else if (mv == 2)
      linear_swiglu_kernel<ENC, 2><<<grid, LIN_WARPS * 32, 0, s>>>(wg, wu, xp, mv, yp);
    else
      linear_swiglu_kernel<ENC, 4><<<grid, LIN_WARPS * 32, 0, s>>>(wg, wu, xp, mv, yp);
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  return 0;
}

int launch_linear_swiglu(const WRef& wg, const WRef& wu, const float* x, int64_t m, float* y,
                         cudaStream_t s) {
  DYN_CHECK(wg.enc == wu.enc && wg.rows == wu.rows && wg.cols == wu.cols,
            "swiglu: gate and up must share encoding and shape");
  DYN_ENC_SWITCH(wg.enc, return run_swiglu<ENC>(wg, wu, x, m, y, s));
  return 0;
}

}  // namespace dyn
