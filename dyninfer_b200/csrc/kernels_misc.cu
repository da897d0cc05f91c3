// RMSNorm, RoPE, QK-norm + RoPE + KV write, GQA attention, SiLU*up, argmax.
#include <math.h>

#include "common.cuh"

namespace dyn {

void fill_freq_table(FreqTable* t, int64_t d, float theta) {
  // den = powf(theta, (2*i)/d); freq = 1/den, all in f32
  // (crates/dyninfer-compiler/src/lowering/kernels.rs:1047-1052). Computed on the host
  // once per call, like the reference's static variants which bake the table
  // at compile time (kernels.rs:936-960).
  const int64_t half = d / 2;
  for (int64_t i = 0; i < 128; i++) {
    if (i < half) {
      float exponent = (2.0f * (float)i) / (float)d;
      float den = powf(theta, exponent);
      t->f[i] = 1.0f / den;
    } else {
      t->f[i] = 0.f;
    }
  }
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; i++) t += smem[i];
  return t;
}

// y = (x * inv) * w with inv = 1 / sqrt(sum(x^2)/H + eps)  (kernels.rs:817-829)
// PER > 0: the row fits PER elements per thread; they are loaded once, all loads in flight
// together, and stay in registers for the second pass (the loop form waits for one load after the
// other because x and y may alias). Element-to-thread assignment and summation order are the same
// in both forms.
template <int PER>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float* x, const void* __restrict__ w, int w_type, int64_t width, float eps,
                float* y) {
  __shared__ float red[32];
  pdl_trigger();  // a product launched next may begin fetching its weights
  const float* xr = x + (int64_t)blockIdx.x * width;
  float* yr = y + (int64_t)blockIdx.x * width;
  float ss = 0.f;
  if (PER > 0) {
    float v[PER > 0 ? PER : 1], wv[PER > 0 ? PER : 1];
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
      v[k] = i < width ? xr[i] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
      wv[k] = i < width ? aux_load(reinterpret_cast<const uint8_t*>(w), w_type, i) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < PER; k++) ss = fmaf(v[k], v[k], ss);  // absent elements add +0
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
      if (i < width) yr[i] = __fmul_rn(__fmul_rn(v[k], inv), wv[k]);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, red);
  const float ms = ss / (float)width;
  const float inv = 1.0f / sqrtf(ms + eps);
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
    const float wv = aux_load(reinterpret_cast<const uint8_t*>(w), w_type, i);
    yr[i] = __fmul_rn(__fmul_rn(xr[i], inv), wv);
  }
}

int launch_rms_norm(const float* x, const void* w, int w_type, int64_t rows, int64_t width,
                    float eps, float* y, cudaStream_t s) {
  if (rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 32);
  if (width <= 8 * threads) {
    rms_norm_kernel<8><<<(unsigned)rows, threads, 0, s>>>(x, w, w_type, width, eps, y);
  } else if (width <= 16 * threads) {
    rms_norm_kernel<16><<<(unsigned)rows, threads, 0, s>>>(x, w, w_type, width, eps, y);
  } else if (width <= 32 * threads) {
    rms_norm_kernel<32><<<(unsigned)rows, threads, 0, s>>>(x, w, w_type, width, eps, y);
  } else {
    rms_norm_kernel<0><<<(unsigned)rows, threads, 0, s>>>(x, w, w_type, width, eps, y);
  }
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// out[e] = sum over the S K-slices of partial[j][idx[e]], j ascending (the order of the products' own
// reduction kernels), four slices' loads in flight at a time for all NE elements: a plain loop would wait
// for one L2 round trip per slice and element.
template <int NE>
__device__ __forceinline__ void deferred_sums(const float* __restrict__ partial, int S, int64_t N,  // N: floats between slices
                                              const int64_t (&idx)[NE], const bool (&live)[NE], float (&out)[NE]) {
#pragma unroll
  for (int e = 0; e < NE; e++) out[e] = 0.f;
  for (int j0 = 0; j0 < S; j0 += 4) {
    float t[4][NE];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
      for (int e = 0; e < NE; e++)
        t[u][e] = (j0 + u < S && live[e]) ? partial[(int64_t)(j0 + u) * N + idx[e]] : 0.f;
#pragma unroll
    for (int u = 0; u < 4; u++)
      if (j0 + u < S) {
#pragma unroll
        for (int e = 0; e < NE; e++) out[e] += t[u][e];
      }
  }
}

// ---- producers of the dequant GEMM's activation operand ------------------------------------------
// max |v| over the block -> the power-of-two scale that puts it in [2^12, 2^13) (the GEMM's activation
// pass: no overflow, ordinary entries stay out of the f16 subnormals) and its inverse
__device__ __forceinline__ void f16_row_scale(float mx, float* red, float* sc, float* inv) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  mx = warp_max(mx);
  __syncthreads();
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = 0.f;
  for (int i = 0; i < nw; i++) mx = fmaxf(mx, red[i]);
  int e = 0;
  if (mx > 0.f && mx < 3.0e38f) frexpf(mx, &e);
  *sc = ldexpf(1.0f, 13 - e);
  *inv = ldexpf(1.0f, e - 13);
}

template <int PER>
__global__ void __launch_bounds__(256)
norm_prepare_kernel(const float* __restrict__ x, const float* __restrict__ partial, int S, int64_t rows,
                    const float* residual, float* hidden, const void* __restrict__ w, int w_type, int64_t width,
                    float eps, __half* __restrict__ xh, float* __restrict__ inv_s) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  float v[PER], wv[PER];
#pragma unroll
  for (int k = 0; k < PER; k++) {
    const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
    float t = 0.f;
    if (i < width) {
      if (S) {
        for (int z = 0; z < S; z++) t += partial[((int64_t)z * rows + row) * width + i];
      } else {
        t = x[row * width + i];
      }
    }
    v[k] = t;
  }
  if (residual) {
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
      if (i < width) v[k] += residual[row * width + i];
    }
  }
#pragma unroll
  for (int k = 0; k < PER; k++) {
    const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
    wv[k] = i < width ? aux_load(reinterpret_cast<const uint8_t*>(w), w_type, i) : 0.f;
    if (hidden && i < width) hidden[row * width + i] = v[k];
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; k++) ss = fmaf(v[k], v[k], ss);  // absent elements add +0
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  float mx = 0.f;
#pragma unroll
  for (int k = 0; k < PER; k++) {
    v[k] = __fmul_rn(__fmul_rn(v[k], inv), wv[k]);
    mx = fmaxf(mx, fabsf(v[k]));
  }
  float sc, is;
  f16_row_scale(mx, red, &sc, &is);
  if (threadIdx.x == 0) inv_s[row] = is;
#pragma unroll
  for (int k = 0; k < PER; k++) {
    const int64_t i = threadIdx.x + (int64_t)k * blockDim.x;
    if (i < width) xh[row * width + i] = __float2half_rn(v[k] * sc);
  }
}

int launch_norm_prepare(const float* x, const float* partial, int splits, const float* residual, float* hidden,
                        const void* w, int w_type, int64_t rows, int64_t width, float eps, __half* xh, float* inv_s,
                        cudaStream_t s) {
  if (rows == 0) return 0;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 32);  // rms_norm_kernel's: same summation order
  DYN_CHECK(width <= 32 * threads, "row of %lld elements is too wide for the fused RMSNorm", (long long)width);
  const int S = splits > 1 ? splits : 0;
  if (width <= 8 * threads)
    norm_prepare_kernel<8><<<(unsigned)rows, threads, 0, s>>>(x, partial, S, rows, residual, hidden, w, w_type, width, eps, xh, inv_s);
  else if (width <= 16 * threads)
    norm_prepare_kernel<16><<<(unsigned)rows, threads, 0, s>>>(x, partial, S, rows, residual, hidden, w, w_type, width, eps, xh, inv_s);
  else
    norm_prepare_kernel<32><<<(unsigned)rows, threads, 0, s>>>(x, partial, S, rows, residual, hidden, w, w_type, width, eps, xh, inv_s);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

__global__ void __launch_bounds__(256)
silu_prepare_kernel(const float* __restrict__ gu, int64_t I, __half* __restrict__ xh, float* __restrict__ inv_s) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const float* g = gu + row * 2 * I;
  auto val = [&](int64_t i) {
    const float gv = g[i];
    return (gv / (1.0f + expf(-gv))) * g[I + i];
  };
  float mx = 0.f;
  for (int64_t i = threadIdx.x; i < I; i += blockDim.x) mx = fmaxf(mx, fabsf(val(i)));
  float sc, is;
  f16_row_scale(mx, red, &sc, &is);
  if (threadIdx.x == 0) inv_s[row] = is;
  for (int64_t i = threadIdx.x; i < I; i += blockDim.x) xh[row * I + i] = __float2half_rn(val(i) * sc);
}

int launch_silu_prepare(const float* gate_up, int64_t rows, int64_t inter, __half* xh, float* inv_s, cudaStream_t s) {
  if (rows == 0 || inter == 0) return 0;
  silu_prepare_kernel<<<(unsigned)rows, 256, 0, s>>>(gate_up, inter, xh, inv_s);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// Rotate-half RoPE (kernels.rs:1053-1064): pair (i, i + d/2).
__device__ __forceinline__ void rope_pair(float x1, float x2, float pos, float freq, float* lo,
                                          float* hi) {
  const float angle = __fmul_rn(pos, freq);
  float sv, cv;
  sincosf(angle, &sv, &cv);
  *lo = __fsub_rn(__fmul_rn(x1, cv), __fmul_rn(x2, sv));
  *hi = __fadd_rn(__fmul_rn(x1, sv), __fmul_rn(x2, cv));
}

__global__ void rope_kernel(float* x, int64_t heads, int64_t d, int64_t start_pos, FreqTable ft) {
  const int64_t p = blockIdx.x, h = blockIdx.y, half = d / 2;
  float* v = x + (p * heads + h) * d;
  const float pos = (float)(start_pos + p);
  for (int64_t i = threadIdx.x; i < half; i += blockDim.x) {
    float lo, hi;
    rope_pair(v[i], v[i + half], pos, ft.f[i], &lo, &hi);
    v[i] = lo;
    v[i + half] = hi;
  }
}

int launch_rope(float* x, int64_t s_rows, int64_t heads, int64_t d, int64_t start_pos,
                const FreqTable& ft, cudaStream_t s) {
  if (s_rows == 0) return 0;
  dim3 grid((unsigned)s_rows, (unsigned)heads);
  rope_kernel<<<grid, 64, 0, s>>>(x, heads, d, start_pos, ft);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, int64_t n,
                                float* __restrict__ y) {
  pdl_trigger();  // a product launched next may begin fetching its weights
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float gv = g[i];
    y[i] = (gv / (1.0f + expf(-gv))) * u[i];
  }
}

// y[r, i] = silu(gu[r, i]) * gu[r, I + i] for the rows of a fused [gate; up] product ([rows, 2 I])
__global__ void silu_mul_rows_kernel(const float* __restrict__ gu, int64_t rows, int64_t I, float* __restrict__ y) {
  pdl_trigger();
  const int64_t n = rows * I;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / I, c = i - r * I;
    const float gv = gu[r * 2 * I + c];
    y[i] = (gv / (1.0f + expf(-gv))) * gu[r * 2 * I + I + c];
  }
}

int launch_silu_mul_rows(const float* gu, int64_t rows, int64_t I, float* y, cudaStream_t s) {
  if (rows * I == 0) return 0;
  int64_t blocks = (rows * I + 255) / 256;
  const int64_t cap = (int64_t)std::max(1, sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  silu_mul_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>(gu, rows, I, y);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// One row of [gate | up] still lying as K-slice sums (or in gate_up when S == 0)
__global__ void silu_mul_deferred_kernel(const float* __restrict__ partial, const float* __restrict__ scale, int S,
                                         int64_t N, const float* __restrict__ gate_up, int64_t I, float* __restrict__ y) {
  pdl_trigger();
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= I) return;
  float g, u;
  if (S) {
    const int64_t idx[2] = {i, I + i};
    const bool live[2] = {true, true};
    float t[2];
    deferred_sums<2>(partial, S, N, idx, live, t);
    g = t[0] * scale[0], u = t[1] * scale[0];
  } else {
    g = gate_up[i], u = gate_up[I + i];
  }
  y[i] = (g / (1.0f + expf(-g))) * u;
}

int launch_silu_mul_deferred(const Deferred& d, const float* gate_up, int64_t inter, float* y, cudaStream_t s) {
  if (inter == 0) return 0;
  DYN_CHECK(!d.S || d.N == 2 * inter, "deferred sums of %lld rows against [gate | up] of %lld", (long long)d.N,
            (long long)(2 * inter));
  silu_mul_deferred_kernel<<<(unsigned)((inter + 255) / 256), 256, 0, s>>>(d.partial, d.scale, d.S, d.N, gate_up, inter, y);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

int launch_silu_mul(const float* gate, const float* up, int64_t n, float* y, cudaStream_t s) {
  if (n == 0) return 0;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, s>>>(gate, up, n, y);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// ---- KV element store / load ---------------------------------------------------
template <int KV>
struct KvT;
template <>
struct KvT<E_F32> {
  using T = float;
  __device__ static __forceinline__ T enc(float v) { return v; }
  __device__ static __forceinline__ float dec(T v) { return v; }
};
template <>
struct KvT<E_F16> {
  using T = __half;
  __device__ static __forceinline__ T enc(float v) { return __float2half_rn(v); }
  __device__ static __forceinline__ float dec(T v) { return __half2float(v); }
};
template <>
struct KvT<E_BF16> {
  using T = __nv_bfloat16;
  __device__ static __forceinline__ T enc(float v) { return __float2bfloat16_rn(v); }
  __device__ static __forceinline__ float dec(T v) { return __bfloat162float(v); }
};

// One block per (row, head). Heads [0, nh) are query heads (per-head RMSNorm then
// RoPE, written back in place); [nh, nh+nkv) key heads (norm, RoPE, stored into the
// cache at the row's position); [nh+nkv, nh+2nkv) value heads (stored unchanged).
// Order norm -> rope follows crates/dyninfer-compiler/src/lowering/dense_decoder.rs:2431-2452,
// the write follows dense_decoder.rs:1115-1197.
template <int KV>
__global__ void __launch_bounds__(128) qkv_prepare_kernel(QkvPrepArgs a, FreqTable ft) {
  using T = typename KvT<KV>::T;
  __shared__ float red[32];
  const int64_t r = blockIdx.x, hh = blockIdx.y, d = a.d, half = d / 2;
  const int64_t pos = a.row_pos ? a.row_pos[r] : a.base_pos + r;
  const int64_t seq = a.row_seq ? a.row_seq[r] : 0;
  const int kind = hh < a.nh ? 0 : (hh < a.nh + a.nkv ? 1 : 2);
  const int64_t head = kind == 0 ? hh : (kind == 1 ? hh - a.nh : hh - a.nh - a.nkv);
  // the head's values: from the product's output, or (one row) added up here from its K-slice sums
  __shared__ float hv[256];
  float* qv = a.q + r * (a.ldq ? a.ldq : a.nh * d) + head * d;
  const float* src;
  {
    const DeferredCols& dc = kind == 0 ? a.dq : (kind == 1 ? a.dk : a.dv);
    const float* in = kind == 0 ? qv
                                : (kind == 1 ? a.k + r * (a.ldk ? a.ldk : a.nkv * d) + head * d
                                             : a.v + r * (a.ldv ? a.ldv : a.nkv * d) + head * d);
    if (dc.S) {
      // up to four elements per thread (d <= 256, at least 32 or 64 threads)
      int64_t idx[4];
      bool live[4];
      float t[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int64_t i = threadIdx.x + (int64_t)e * blockDim.x;
        live[e] = i < d, idx[e] = dc.col + head * d + i;
      }
      deferred_sums<4>(dc.partial + r * dc.N, dc.S, dc.rows * dc.N, idx, live, t);
      const float sc = dc.scale ? dc.scale[0] : 1.0f;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int64_t i = threadIdx.x + (int64_t)e * blockDim.x;
        if (i < d) hv[i] = t[e] * sc;
      }
      __syncthreads();
      src = hv;
    } else {
      src = in;  // read in place, as the multi-row steps always do
    }
  }
  if (kind == 2) {
    T* dst = reinterpret_cast<T*>(a.vcache) + ((seq * a.nkv + head) * a.cap + pos) * d;
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) dst[i] = KvT<KV>::enc(src[i]);
    return;
  }
  const void* nw = kind == 0 ? a.q_norm_w : a.k_norm_w;
  float inv = 1.f;
  if (a.has_norm) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, red);
    inv = 1.0f / sqrtf(ss / (float)d + a.eps);
  }
  T* kdst = kind == 1 ? reinterpret_cast<T*>(a.kcache) + ((seq * a.nkv + head) * a.cap + pos) * d
                      : nullptr;
  for (int64_t i = threadIdx.x; i < half; i += blockDim.x) {
    float x1 = src[i], x2 = src[i + half];
    if (a.has_norm) {
      const uint8_t* nwb = reinterpret_cast<const uint8_t*>(nw);
      x1 = __fmul_rn(__fmul_rn(x1, inv), aux_load(nwb, a.norm_w_type, i));
      x2 = __fmul_rn(__fmul_rn(x2, inv), aux_load(nwb, a.norm_w_type, i + half));
    }
    float lo = x1, hi = x2;
    if (a.has_rope) rope_pair(x1, x2, (float)pos, ft.f[i], &lo, &hi);
    if (kind == 0) {
      qv[i] = lo;
      qv[i + half] = hi;
    } else {
      kdst[i] = KvT<KV>::enc(lo);
      kdst[i + half] = KvT<KV>::enc(hi);
    }
  }
}

int launch_qkv_prepare(const QkvPrepArgs& a, const FreqTable& ft, cudaStream_t s) {
  if (a.rows == 0) return 0;
  DYN_CHECK(a.d % 2 == 0 && a.d <= 256, "head_dim %lld unsupported (even, <= 256)", (long long)a.d);
  dim3 grid((unsigned)a.rows, (unsigned)(a.nh + 2 * a.nkv));
  const int threads = a.d >= 128 ? 64 : 32;
  if (a.kv_type == E_F32) {
    qkv_prepare_kernel<E_F32><<<grid, threads, 0, s>>>(a, ft);
  } else if (a.kv_type == E_F16) {
    qkv_prepare_kernel<E_F16><<<grid, threads, 0, s>>>(a, ft);
  } else if (a.kv_type == E_BF16) {
    qkv_prepare_kernel<E_BF16><<<grid, threads, 0, s>>>(a, ft);
  } else
    DYN_CHECK(false, "kv_type %d unsupported", a.kv_type);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// ---- attention -------------------------------------------------------------------
// One block per (query head, row). Keys 0..pos of the row's sequence are visible
// (causal mask kernels.rs:460-506; every key <= pos has been written). Warps take
// keys round-robin, keep an online (max, sum, acc) state (merge rule kernels.rs
// :375-454), and the four states are merged through shared memory; the result is
// acc / sum (dense_decoder.rs:1317-1328). scale = 1/sqrt(d).
constexpr int ATT_WARPS = 4;
constexpr int ATT_DPL = 8;  // dims per lane, head_dim <= 256

template <int KV>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_kernel(AttnArgs a) {
  using T = typename KvT<KV>::T;
  __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
  __shared__ float s_acc[ATT_WARPS][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t h = blockIdx.x, r = blockIdx.y, d = a.d;
  const int64_t kvh = h / (a.nh / a.nkv);
  const int64_t pos = a.row_pos ? a.row_pos[r] : a.base_pos + r;
  const int64_t seq = a.row_seq ? a.row_seq[r] : 0;
  const float scale = 1.0f / sqrtf((float)d);
  const float* qv = a.q + r * (a.ldq ? a.ldq : a.nh * d) + h * d;
  const T* kb = reinterpret_cast<const T*>(a.kcache) + (seq * a.nkv + kvh) * a.cap * d;
  const T* vb = reinterpret_cast<const T*>(a.vcache) + (seq * a.nkv + kvh) * a.cap * d;
  float qreg[ATT_DPL], acc[ATT_DPL];
#pragma unroll
  for (int j = 0; j < ATT_DPL; j++) {
    const int64_t idx = lane + 32 * j;
    qreg[j] = idx < d ? qv[idx] : 0.f;
    acc[j] = 0.f;
  }
  float m = -3.40282347e38f, l = 0.f;
  for (int64_t key = warp; key <= pos; key += ATT_WARPS) {
    const T* kr = kb + key * d;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < ATT_DPL; j++) {
      const int64_t idx = lane + 32 * j;
      if (idx < d) dot = fmaf(qreg[j], KvT<KV>::dec(kr[idx]), dot);
    }
    dot = warp_sum(dot);
    const float sc = dot * scale;
    const float mn = fmaxf(m, sc);
    const float factor = expf(m - mn);
    const float p = expf(sc - mn);
    l = l * factor + p;
    const T* vr = vb + key * d;
#pragma unroll
    for (int j = 0; j < ATT_DPL; j++) {
      const int64_t idx = lane + 32 * j;
      if (idx < d) acc[j] = acc[j] * factor + p * KvT<KV>::dec(vr[idx]);
    }
    m = mn;
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
#pragma unroll
  for (int j = 0; j < ATT_DPL; j++) {
    const int idx = lane + 32 * j;
    if (idx < d) s_acc[warp][idx] = acc[j];
  }
  __syncthreads();
  float gm = s_m[0];
  for (int w = 1; w < ATT_WARPS; w++) gm = fmaxf(gm, s_m[w]);
  float gl = 0.f;
  for (int w = 0; w < ATT_WARPS; w++) gl += s_l[w] * expf(s_m[w] - gm);
  for (int64_t idx = threadIdx.x; idx < d; idx += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < ATT_WARPS; w++) o += s_acc[w][idx] * expf(s_m[w] - gm);
    a.ctx[r * a.nh * d + h * d + idx] = o / gl;
  }
}

// ---- decode attention with split keys (long contexts, batched decode) ------------------------
// Grid (head, row, split): every CTA walks one slice of the row's keys; a lane owns DPL consecutive
// head dims, so a warp reads a cached key or value row with one coalesced vector load, and four
// keys per warp are in flight before any is used. Each CTA leaves (unnormalised output, max, sum)
// for its slice; attention_merge_kernel combines the slices in a fixed order.
template <int KV, int DPL>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_split_kernel(AttnArgs a, float* __restrict__ part, int nsplit) {
  using T = typename KvT<KV>::T;
  constexpr int KB = 4;
  __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
  __shared__ float s_acc[ATT_WARPS][32 * DPL];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t h = blockIdx.x, r = blockIdx.y, sp = blockIdx.z, d = a.d;
  const int64_t kvh = h / (a.nh / a.nkv);
  const int64_t pos = a.row_pos ? a.row_pos[r] : a.base_pos + r;
  const int64_t seq = a.row_seq ? a.row_seq[r] : 0;
  const int64_t n = pos + 1, per = (n + nsplit - 1) / nsplit;
  const int64_t k_lo = sp * per, k_hi = k_lo + per < n ? k_lo + per : n;
  const float scale = 1.0f / sqrtf((float)d);
  const int e0 = lane * DPL;
  const bool live = e0 < d;
  const T* kb = reinterpret_cast<const T*>(a.kcache) + (seq * a.nkv + kvh) * a.cap * d + e0;
  const T* vb = reinterpret_cast<const T*>(a.vcache) + (seq * a.nkv + kvh) * a.cap * d + e0;
  float qreg[DPL], acc[DPL];
#pragma unroll
  for (int j = 0; j < DPL; j++) {
    qreg[j] = live ? a.q[r * (a.ldq ? a.ldq : a.nh * d) + h * d + e0 + j] : 0.f;
    acc[j] = 0.f;
  }
  struct __align__(sizeof(T) * DPL) Row {  // one vector load per lane and cached row
    T v[DPL];
  };
  float m = -3.40282347e38f, l = 0.f;
  for (int64_t key0 = k_lo + warp; key0 < k_hi; key0 += (int64_t)KB * ATT_WARPS) {
    Row kr[KB], vr[KB];
#pragma unroll
    for (int b = 0; b < KB; b++) {
      const int64_t key = key0 + (int64_t)b * ATT_WARPS;
      if (key < k_hi && live) {
        kr[b] = *reinterpret_cast<const Row*>(kb + key * d);
        vr[b] = *reinterpret_cast<const Row*>(vb + key * d);
      }
    }
#pragma unroll
    for (int b = 0; b < KB; b++) {
      const int64_t key = key0 + (int64_t)b * ATT_WARPS;
      if (key >= k_hi) break;  // warp-uniform
      float dot = 0.f;
      if (live) {
#pragma unroll
        for (int j = 0; j < DPL; j++) dot = fmaf(qreg[j], KvT<KV>::dec(kr[b].v[j]), dot);
      }
      const float sc = warp_sum(dot) * scale;
      const float mn = fmaxf(m, sc);
      const float factor = expf(m - mn), p = expf(sc - mn);
      l = l * factor + p;
      if (live) {
#pragma unroll
        for (int j = 0; j < DPL; j++) acc[j] = acc[j] * factor + p * KvT<KV>::dec(vr[b].v[j]);
      }
      m = mn;
    }
  }
  if (lane == 0) s_m[warp] = m, s_l[warp] = l;
  if (live) {
#pragma unroll
    for (int j = 0; j < DPL; j++) s_acc[warp][e0 + j] = acc[j];
  }
  __syncthreads();
  float gm = s_m[0];
#pragma unroll
  for (int w = 1; w < ATT_WARPS; w++) gm = fmaxf(gm, s_m[w]);
  float wgt[ATT_WARPS], gl = 0.f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; w++) {
    wgt[w] = expf(s_m[w] - gm);
    gl += s_l[w] * wgt[w];
  }
  float* out = part + (((r * a.nh + h) * nsplit) + sp) * (d + 2);
  for (int64_t idx = threadIdx.x; idx < d; idx += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) o += s_acc[w][idx] * wgt[w];
    out[idx] = o;
  }
  if (threadIdx.x == 0) out[d] = gm, out[d + 1] = gl;
}

__global__ void __launch_bounds__(256)
attention_merge_kernel(const float* __restrict__ part, int nsplit, float* ctx, int64_t nh, int64_t d) {
  pdl_trigger();  // a product launched next may begin fetching its weights
  const int64_t h = blockIdx.x, r = blockIdx.y;
  const float* p0 = part + ((r * nh + h) * nsplit) * (d + 2);
  float gm = -3.40282347e38f;
  for (int s = 0; s < nsplit; s++) gm = fmaxf(gm, p0[s * (d + 2) + d]);
  for (int64_t idx = threadIdx.x; idx < d; idx += blockDim.x) {
    float o = 0.f, gl = 0.f;
    for (int s = 0; s < nsplit; s++) {
      const float* ps = p0 + s * (d + 2);
      const float w = expf(ps[d] - gm);  // an empty slice has sum 0 and contributes nothing
      o += ps[idx] * w;
      gl += ps[d + 1] * w;
    }
    ctx[r * nh * d + h * d + idx] = o / gl;
  }
}

template <int KV>
static int run_attention_split(const AttnArgs& a, float* part, int nsplit, cudaStream_t s) {
  const dim3 grid((unsigned)a.nh, (unsigned)a.rows, (unsigned)nsplit);
  if (a.d == 64) {
    attention_split_kernel<KV, 2><<<grid, ATT_WARPS * 32, 0, s>>>(a, part, nsplit);
  } else if (a.d == 128) {
    attention_split_kernel<KV, 4><<<grid, ATT_WARPS * 32, 0, s>>>(a, part, nsplit);
  } else {
    attention_split_kernel<KV, 8><<<grid, ATT_WARPS * 32, 0, s>>>(a, part, nsplit);
  }
  attention_merge_kernel<<<dim3((unsigned)a.nh, (unsigned)a.rows), 256, 0, s>>>(part, nsplit, a.ctx, a.nh, a.d);
  count_launch(2);
  DYN_CUDA(cudaGetLastError());
  return 0;
}

size_t attention_split_scratch_bytes(int64_t rows, int64_t nh, int64_t d, int nsplit) {
  return (size_t)rows * nh * nsplit * (d + 2) * sizeof(float);
}

// Split-key decode attention into caller scratch (attention_split_scratch_bytes). Head dims 64,
// 128 and 256 only; *handled = false otherwise.
int launch_attention_split(const AttnArgs& a, float* part, int nsplit, cudaStream_t s, bool* handled) {
  *handled = false;
  if (a.rows == 0 || (a.d != 64 && a.d != 128 && a.d != 256) || nsplit < 1) return 0;
  DYN_CHECK(a.nkv > 0 && a.nh % a.nkv == 0, "heads %lld not a multiple of kv heads %lld", (long long)a.nh,
            (long long)a.nkv);
  int rc;
  if (a.kv_type == E_F32)
    rc = run_attention_split<E_F32>(a, part, nsplit, s);
  else if (a.kv_type == E_F16)
    rc = run_attention_split<E_F16>(a, part, nsplit, s);
  else if (a.kv_type == E_BF16)
    rc = run_attention_split<E_BF16>(a, part, nsplit, s);
  else
    return 0;
  if (!rc) *handled = true;
  return rc;
}

int launch_attention(const AttnArgs& a, cudaStream_t s) {
  if (a.rows == 0) return 0;
  DYN_CHECK(a.d <= 256, "head_dim %lld unsupported (<= 256)", (long long)a.d);
  DYN_CHECK(a.nkv > 0 && a.nh % a.nkv == 0, "heads %lld not a multiple of kv heads %lld",
            (long long)a.nh, (long long)a.nkv);
  if (!a.row_pos || a.uniform_base >= 0) {  // one sequence, consecutive positions: tensor-core kernel
    bool handled = false;
    if (launch_attention_prefill(a, a.row_pos ? a.uniform_base : a.base_pos, a.row_pos ? a.uniform_seq : 0, s,
                                 &handled))
      return 1;
    if (handled) return 0;
  }
  if (a.d == 64 || a.d == 128 || a.d == 256) {
    // decode / batched decode: slice every row's keys over enough CTAs to fill the GPU. The slice
    // count depends only on shapes and capacity, so a captured graph stays valid as positions grow.
    int nsplit = (int)(592 / (a.rows * a.nh));
    const int by_cap = (int)(a.cap / 128);
    if (nsplit > by_cap) nsplit = by_cap;
    if (nsplit > 32) nsplit = 32;
    if (nsplit < 1) nsplit = 1;
    // the slices' partial results: the caller's scratch region when it is large enough (a session's:
    // no allocation nodes in a captured step), else the stream-ordered allocator
    const size_t part_bytes = attention_split_scratch_bytes(a.rows, a.nh, a.d, nsplit);
    float* part = reinterpret_cast<float*>(thread_scratch(part_bytes));
    const bool pooled = part == nullptr;
    if (pooled) {
      if (keep_scratch_pool_cached()) return 1;
      DYN_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), part_bytes, s));
    }
    bool handled = false;
    const int rc = launch_attention_split(a, part, nsplit, s, &handled);
    const cudaError_t fe = pooled ? cudaFreeAsync(part, s) : cudaSuccess;
    if (rc) return rc;
    if (fe != cudaSuccess) return cuda_fail(fe, "cudaFreeAsync", __FILE__, __LINE__);
    if (handled) return 0;
  }
  dim3 grid((unsigned)a.nh, (unsigned)a.rows);
  if (a.kv_type == E_F32)
    attention_kernel<E_F32><<<grid, ATT_WARPS * 32, 0, s>>>(a);
  else if (a.kv_type == E_F16)
    attention_kernel<E_F16><<<grid, ATT_WARPS * 32, 0, s>>>(a);
  else if (a.kv_type == E_BF16)
    attention_kernel<E_BF16><<<grid, ATT_WARPS * 32, 0, s>>>(a);
  else
    DYN_CHECK(false, "kv_type %d unsupported", a.kv_type);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

// ---- argmax: first strict maximum (dense_decoder.rs:885-893) ---------------------
struct ArgPair {
  float v;
  int pad;
  long long i;
};
__device__ __forceinline__ bool arg_better(float v, long long i, float bv, long long bi) {
  return v > bv || (v == bv && i < bi);
}
constexpr int ARGMAX_BLOCKS = 296;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ v, int64_t n, ArgPair* part) {
  __shared__ float sv[256];
  __shared__ long long si[256];
  float bv = -INFINITY;
  long long bi = 0x7fffffffffffffffLL;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float x = v[i];
    if (x > -INFINITY && arg_better(x, i, bv, bi)) bv = x, bi = i;
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o && arg_better(sv[threadIdx.x + o], si[threadIdx.x + o],
                                           sv[threadIdx.x], si[threadIdx.x])) {
      sv[threadIdx.x] = sv[threadIdx.x + o];
      si[threadIdx.x] = si[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    part[blockIdx.x].v = sv[0];
    part[blockIdx.x].i = si[0];
  }
}

__global__ void __launch_bounds__(512)
argmax_final_kernel(const ArgPair* part, int count, int64_t* out) {
  __shared__ float sv[512];
  __shared__ long long si[512];
  float bv = -INFINITY;
  long long bi = 0x7fffffffffffffffLL;
  if ((int)threadIdx.x < count) bv = part[threadIdx.x].v, bi = part[threadIdx.x].i;
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = 256; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o && arg_better(sv[threadIdx.x + o], si[threadIdx.x + o],
                                           sv[threadIdx.x], si[threadIdx.x])) {
      sv[threadIdx.x] = sv[threadIdx.x + o];
      si[threadIdx.x] = si[threadIdx.x + o];
    }
    __syncthreads();
  }
  // all values NaN or -inf: the scan never moves off index 0 (generate.rs:16-26)
  if (threadIdx.x == 0) out[0] = si[0] == 0x7fffffffffffffffLL ? 0 : si[0];
}

// One block per row of v [rows, n]: first strict maximum of every row (batched decode).
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float* __restrict__ v, int64_t n, int shards, int64_t* out) {
  __shared__ float sv[32];
  __shared__ long long si[32];
  float bv = -INFINITY;
  long long bi = 0x7fffffffffffffffLL;
  // slice w of this row sits at [w][row][n]; its elements are indices w * n + j
  for (int w = 0; w < shards; w++) {
    const float* row = v + ((int64_t)w * gridDim.x + blockIdx.x) * n;
    for (int64_t i = threadIdx.x; i < n; i += 1024) {
      const float x = row[i];
      if (x > -INFINITY && arg_better(x, (int64_t)w * n + i, bv, bi)) bv = x, bi = (int64_t)w * n + i;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (arg_better(ov, oi, bv, bi)) bv = ov, bi = oi;
  }
  if (lane == 0) sv[warp] = bv, si[warp] = bi;
  __syncthreads();
  if (warp == 0) {
    bv = sv[lane], bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (arg_better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffffffffffffLL ? 0 : bi;
  }
}

int launch_argmax_rows(const float* v, int64_t rows, int64_t n, int64_t* out, cudaStream_t s) {
  DYN_CHECK(rows >= 1 && n >= 1, "argmax_rows: rows and n must be >= 1");
  argmax_rows_kernel<<<(unsigned)rows, 1024, 0, s>>>(v, n, 1, out);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

int launch_argmax_rows_sharded(const float* v, int64_t rows, int64_t n_local, int shards, int64_t* out,
                               cudaStream_t s) {
  DYN_CHECK(rows >= 1 && n_local >= 1 && shards >= 1, "argmax_rows: rows, n and shards must be >= 1");
  argmax_rows_kernel<<<(unsigned)rows, 1024, 0, s>>>(v, n_local, shards, out);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

size_t argmax_scratch_bytes(int64_t) { return sizeof(ArgPair) * ARGMAX_BLOCKS; }

int launch_argmax(const float* v, int64_t n, int64_t* out, void* scratch, cudaStream_t s) {
  DYN_CHECK(n >= 1, "argmax: n must be >= 1");
  int blocks = (int)((n + 255) / 256);
  if (blocks > ARGMAX_BLOCKS) blocks = ARGMAX_BLOCKS;
  argmax_partial_kernel<<<blocks, 256, 0, s>>>(v, n, reinterpret_cast<ArgPair*>(scratch));
  argmax_final_kernel<<<1, 512, 0, s>>>(reinterpret_cast<const ArgPair*>(scratch), blocks, out);
  count_launch(2);
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace dyn
