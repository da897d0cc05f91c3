// Fused dequant-GEMV for 1..8 activation rows on the raw checkpoint bytes.
//
// Two launches per product:
//   1. stage_x_kernel arranges the activations once, in global scratch, in the register
//      order the tensor-core tile steps consume (gemv_core.cuh), with per-row power-of-two
//      scales and per-16-element sums.
//   2. gemv_tile_kernel: every warp owns one (16-row tile, K-chunk) of the weight matrix and
//      walks its 32-element blocks straight from global memory — the 18/20/34/210-byte
//      blocks are read with aligned 32-bit loads and a funnel shift, consecutive blocks of a
//      row share cache lines so each line leaves HBM once — and issues the tile steps.
//      No shared memory, no block-level synchronisation. When the matrix has too few tiles
//      to fill the GPU, K is split over several warps and a third, tiny launch adds the
//      partial sums in a fixed order (results stay deterministic).
#include "gemv_core.cuh"

namespace dyn {

namespace {

constexpr int GT_WARPS = 8;

struct XView {
  const __half* xf;   // [K/32][ncol][4][8]
  const float* sx16;  // [xrows][K/16]
  const float* sx32;  // [xrows][K/32]
  const float* inv_s; // [8] inverse scales, then [8] scales
};

// ---- 1. activation staging ------------------------------------------------------------
template <int NCOL, bool HILO>
__global__ void __launch_bounds__(256)
stage_x_kernel(const void* __restrict__ x, int x_bf16, int M, int xrows, int K, int layout,
               __half* xf, float* sx16, float* sx32, float* inv_s) {
  __shared__ float red[8][8];
  __shared__ float s_scale[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto ld = [&](int m, int i) -> float {
    return x_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(x)[(size_t)m * K + i])
                  : reinterpret_cast<const float*>(x)[(size_t)m * K + i];
  };
  for (int m = 0; m < M; m++) {
    float mx = 0.f;
    for (int i = tid; i < K; i += 256) mx = fmaxf(mx, fabsf(ld(m, i)));
    mx = warp_max(mx);
    if (lane == 0) red[m][warp] = mx;
  }
  __syncthreads();
  if (tid < 8) {
    float mx = 0.f;
    if (tid < M)
      for (int i = 0; i < 8; i++) mx = fmaxf(mx, red[tid][i]);
    float s, is;
    scale_for(mx, &s, &is);
    s_scale[tid] = s;
    if (blockIdx.x == 0) {
      inv_s[tid] = is;
      inv_s[8 + tid] = s;
    }
  }
  __syncthreads();
  const int per_row = (K >> 5) * 4;
  const int stride = gridDim.x * 256;
  for (int it = blockIdx.x * 256 + tid; it < per_row * xrows; it += stride) {
    const int m = it / per_row, r = it - m * per_row;
    const int kb = r >> 2, t = r & 3;
    if (m < M) {
      float tmp[32];
#pragma unroll
      for (int j = 0; j < 32; j++) tmp[j] = ld(m, kb * 32 + j);
      stage_item<NCOL, HILO>(tmp - kb * 32, layout, xf, kb, t, m, s_scale[m]);
    } else if (HILO ? (2 * m + 1 < NCOL) : (m < NCOL)) {
      const uint4 z = make_uint4(0, 0, 0, 0);  // unused columns must be finite
      if (HILO) {
        uint4* dst = reinterpret_cast<uint4*>(xf + ((size_t)(kb * NCOL + 2 * m) * 4 + t) * 8);
        dst[0] = z;
        dst[4] = z;
      } else {
        *reinterpret_cast<uint4*>(xf + ((size_t)(kb * NCOL + m) * 4 + t) * 8) = z;
      }
    }
  }
  const int runs = K >> 4;
  for (int it = blockIdx.x * 256 + tid; it < runs * xrows; it += stride) {
    const int m = it / runs, r = it - m * runs;
    float a = 0.f;
    if (m < M) {
#pragma unroll
      for (int j = 0; j < 16; j++) a += ld(m, r * 16 + j);
      a *= s_scale[m];
    }
    sx16[it] = a;
  }
  const int blocks = K >> 5;
  for (int it = blockIdx.x * 256 + tid; it < blocks * xrows; it += stride) {
    const int m = it / blocks, r = it - m * blocks;
    float a = 0.f;
    if (m < M) {
#pragma unroll
      for (int j = 0; j < 32; j++) a += ld(m, r * 32 + j);
      a *= s_scale[m];
    }
    sx32[it] = a;
  }
}

// ---- 2. tiles ---------------------------------------------------------------------------
// Each warp streams its 16 row segments through a private byte ring in shared memory with
// cp.async copies that run several 32-byte stages ahead of the math, so every SM keeps tens of
// kilobytes of HBM reads in flight without any block-level synchronisation. The ring holds a
// whole number of units, so a unit never straddles the wrap and all addresses inside a unit
// are compile-time offsets from one pointer. Rows sit PITCH bytes apart with PITCH/4 = 4
// (mod 8): the 8 rows x 4 consecutive words a fragment load touches hit 32 distinct banks.
constexpr int STAGE = 32;

template <int ENC>
struct UG;
template <>
struct UG<E_Q4_0> { static constexpr int UBYTES = 36, UKB = 2, RING_UNITS = 8, PITCH = 304, CPB = 16, OVER = 2; };
template <>
struct UG<E_Q4_1> { static constexpr int UBYTES = 20, UKB = 1, RING_UNITS = 16, PITCH = 336, CPB = 16, OVER = 0; };
template <>
struct UG<E_Q8_0> { static constexpr int UBYTES = 68, UKB = 2, RING_UNITS = 4, PITCH = 304, CPB = 16, OVER = 2; };
template <>
struct UG<E_MLX_U4> { static constexpr int UBYTES = 16, UKB = 1, RING_UNITS = 16, PITCH = 272, CPB = 16, OVER = 0; };
template <>
struct UG<E_Q6_K> { static constexpr int UBYTES = 210, UKB = 8, RING_UNITS = 4, PITCH = 848, CPB = 8, OVER = 2; };

template <int ENC>
struct UGD {
  static constexpr int RINGB = UG<ENC>::UBYTES * UG<ENC>::RING_UNITS;
  static constexpr int D0 = (RINGB - UG<ENC>::UBYTES - UG<ENC>::OVER) / STAGE;
  static constexpr int DEPTH = D0 > 7 ? 7 : D0;  // stages in flight
  static_assert(RINGB % UG<ENC>::CPB == 0 && UG<ENC>::PITCH >= RINGB + 4 && (UG<ENC>::PITCH / 4) % 8 == 4, "ring geometry");
  static_assert(DEPTH >= 2, "ring too small");
};

template <int CPB>
__device__ __forceinline__ void cp_async(void* dst, const void* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (CPB == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int ENC, int NCOL, bool HILO>
__global__ void __launch_bounds__(GT_WARPS * 32, 3)
gemv_tile_kernel(const WRef w, const XView xv, const int M, float* y, const float* residual,
                 float* partial, const int S, const int kb_per, const int ntiles) {
  extern __shared__ __align__(128) uint8_t gt_smem[];
  using G = UG<ENC>;
  constexpr int RINGB = UGD<ENC>::RINGB, DEPTH = UGD<ENC>::DEPTH;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t unit_id = (int64_t)blockIdx.x * GT_WARPS + warp;
  if (unit_id >= (int64_t)ntiles * S) return;
  const int tile = (int)(unit_id / S), j = (int)(unit_id - (int64_t)tile * S);
  const int K = (int)w.cols, kb_total = K >> 5;
  const int kb0 = j * kb_per;
  int nkb = kb_total - kb0;
  if (nkb > kb_per) nkb = kb_per;
  const int64_t N = w.rows, rb = w.row_bytes();
  const int g = lane >> 2, t = lane & 3;
  int64_t row0 = (int64_t)tile * 16 + g, row1 = row0 + 8;
  const bool v0 = row0 < N, v1 = row1 < N;
  if (!v0) row0 = N - 1;
  if (!v1) row1 = N - 1;
  const int64_t boff = (int64_t)(kb0 / G::UKB) * G::UBYTES;
  uint8_t* ring = gt_smem + (size_t)warp * 16 * G::PITCH;
  const uint8_t* q0 = ring + g * G::PITCH;        // this lane's two rows inside the ring
  const uint8_t* q1 = ring + (g + 8) * G::PITCH;
  // copy role: row cr of the tile, 16-byte half `ch` of every 32-byte stage
  const int cr = lane >> 1, ch = lane & 1;
  int64_t crow = (int64_t)tile * 16 + cr;
  if (crow > N - 1) crow = N - 1;
  const uint8_t* csrc = w.data + crow * rb + boff + ch * 16;
  uint8_t* cdst = ring + cr * G::PITCH;
  const uint8_t* tensor_end = w.data + N * rb;
  const int nunits = nkb / G::UKB;
  const int nstages = (nunits * G::UBYTES + G::OVER + STAGE - 1) / STAGE;
  int cpos = ch * 16;  // ring position of this lane's next copy
  auto issue = [&](int st) {
    if (st < nstages) {
#pragma unroll
      for (int i = 0; i < 16 / G::CPB; i++) {
        const uint8_t* src = csrc + (int64_t)st * STAGE + i * G::CPB;
        const int64_t left = tensor_end - src;
        int pos = cpos + i * G::CPB;
        if (pos >= RINGB) pos -= RINGB;
        if (left > 0) cp_async<G::CPB>(cdst + pos, src, left >= G::CPB ? G::CPB : (int)left);
      }
      cpos += STAGE;
      if (cpos >= RINGB) cpos -= RINGB;
    }
    cp_async_commit();
  };
  const int c = (lane >> 2) & (NCOL - 1);
  const __half* xfp = xv.xf + ((size_t)kb0 * NCOL + c) * 32 + t * 8;  // + NCOL*32 halfs per block
  const int ma = HILO ? t : 2 * t, mb = HILO ? t : 2 * t + 1;
  const float* sa32 = xv.sx32 + (size_t)ma * kb_total + kb0;
  const float* sb32 = xv.sx32 + (size_t)mb * kb_total + kb0;
  const float* sa16 = xv.sx16 + (size_t)ma * (kb_total * 2) + 2 * kb0;
  const float* sb16 = xv.sx16 + (size_t)mb * (kb_total * 2) + 2 * kb0;
  const uint8_t* asc0 = nullptr;
  const uint8_t* abi0 = nullptr;
  const uint8_t* asc1 = nullptr;
  const uint8_t* abi1 = nullptr;
  int gshift = 0;
  if (ENC == E_MLX_U4) {
    const int ael = w.aux == E_F32 ? 4 : 2;
    const int64_t arow = (int64_t)(K / w.group) * ael, a0 = (int64_t)(kb0 * 32 / w.group) * ael;
    asc0 = w.scales + row0 * arow + a0;
    abi0 = w.biases + row0 * arow + a0;
    asc1 = w.scales + row1 * arow + a0;
    abi1 = w.biases + row1 * arow + a0;
    gshift = w.group == 32 ? 0 : (w.group == 64 ? 1 : (w.group == 128 ? 2 : 3));
  }
  TileAcc<HILO> acc;
  acc.clear();
#pragma unroll
  for (int st = 0; st < DEPTH; st++) issue(st);
  int u = 0, ro = 0, need = G::UBYTES + G::OVER;
  for (int st = 0; st < nstages; st++) {
    cp_async_wait<DEPTH - 1>();
    __syncwarp();
    const int arrived = (st + 1) * STAGE;
    while (u < nunits && need <= arrived) {
      const uint8_t* p0 = q0 + ro;
      const uint8_t* p1 = q1 + ro;
      const int kl = u * G::UKB;
      if constexpr (ENC == E_Q4_0) {
        blk_q4<E_Q4_0, 0, HILO>(p0, p1, xfp, sa32[kl], sb32[kl], t, acc);
        blk_q4<E_Q4_0, 2, HILO>(p0 + 18, p1 + 18, xfp + NCOL * 32, sa32[kl + 1], sb32[kl + 1], t, acc);
      } else if constexpr (ENC == E_Q4_1) {
        blk_q4<E_Q4_1, 0, HILO>(p0, p1, xfp, sa32[kl], sb32[kl], t, acc);
      } else if constexpr (ENC == E_Q8_0) {
        blk_q8_0<0, HILO>(p0, p1, xfp, sa32[kl], sb32[kl], t, acc);
        blk_q8_0<2, HILO>(p0 + 34, p1 + 34, xfp + NCOL * 32, sa32[kl + 1], sb32[kl + 1], t, acc);
      } else if constexpr (ENC == E_MLX_U4) {
        const int gi = kl >> gshift;
        blk_mlx<HILO>(p0, p1, aux_load(asc0, w.aux, gi), aux_load(asc1, w.aux, gi),
                      aux_load(abi0, w.aux, gi), aux_load(abi1, w.aux, gi), xfp, sa32[kl], sb32[kl], t, acc);
      } else {
        if (u & 1)
          sblk_q6_k<2, HILO>(p0, p1, xfp, NCOL * 32, sa16 + 2 * kl, sb16 + 2 * kl, t, acc);
        else
          sblk_q6_k<0, HILO>(p0, p1, xfp, NCOL * 32, sa16 + 2 * kl, sb16 + 2 * kl, t, acc);
      }
      xfp += G::UKB * NCOL * 32;
      ro += G::UBYTES;
      if (ro == RINGB) ro = 0;
      need += G::UBYTES;
      u++;
    }
    issue(st + DEPTH);
  }
  cp_async_wait<0>();

  // lane (g, t): rows g / g+8; HILO: activation row t; plain: activation rows 2t, 2t+1
  auto emit = [&](int m, int64_t row, bool valid, float v) {
    if (!valid || m >= M) return;
    if (S == 1) {
      v *= GV_2P24 * xv.inv_s[m];
      if (residual) v += residual[(int64_t)m * N + row];
      y[(int64_t)m * N + row] = v;
    } else {
      partial[((int64_t)j * M + m) * N + row] = v;
    }
  };
  if (HILO) {
    emit(t, row0, v0, acc.v[0]);
    emit(t, row1, v1, acc.v[1]);
  } else {
    emit(2 * t, row0, v0, acc.v[0]);
    emit(2 * t + 1, row0, v0, acc.v[1]);
    emit(2 * t, row1, v1, acc.v[2]);
    emit(2 * t + 1, row1, v1, acc.v[3]);
  }
}

// ---- 3. partial sums over the K-chunks, fixed order --------------------------------------
__global__ void __launch_bounds__(256)
gemv_reduce_kernel(const float* __restrict__ partial, int S, int M, int64_t N,
                   const float* __restrict__ inv_s, float* y, const float* residual) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= (int64_t)M * N) return;
  float a = 0.f;
  for (int j = 0; j < S; j++) a += partial[(int64_t)j * M * N + i];
  a *= GV_2P24 * inv_s[i / N];
  if (residual) a += residual[i];
  y[i] = a;
}

struct Shape {
  int ncol, xrows, S, kb_per, ntiles;
  bool hilo;
  size_t off_sx, off_sx32, off_inv, off_part, bytes;
};

void plan_shape(const WRef& w, int M, bool bf16, Shape* sh) {
  const int K = (int)w.cols, kb_total = K / 32;
  sh->hilo = !bf16;
  sh->ncol = (M == 1 && !bf16) ? 2 : 8;
  sh->xrows = sh->hilo ? (sh->ncol / 2 < 4 ? 4 : sh->ncol / 2) : 8;
  sh->ntiles = (int)((w.rows + 15) / 16);
  // split K until there are enough warp-sized work items to fill the GPU
  // chunks start on copy-aligned, phase-0 unit boundaries
  int unit = 8;
  if (w.enc == E_Q4_1) unit = 4;
  if (w.enc == E_Q6_K) unit = 32;
  if (w.enc == E_MLX_U4) unit = w.group / 32;
  int S = 1;
  const int sms = std::max(1, sm_count());
  while (S < 16 && (int64_t)sh->ntiles * S < (int64_t)sms * 16 && kb_total / (S * 2) >= 8 * unit) S *= 2;
  int per = (kb_total + S - 1) / S;
  per = (per + unit - 1) / unit * unit;
  sh->kb_per = per;
  sh->S = (kb_total + per - 1) / per;
  size_t off = xstage_xf_bytes(K, sh->ncol);
  off = (off + 255) / 256 * 256;
  sh->off_sx = off;
  off += xstage_sx_bytes(K, sh->xrows);
  off = (off + 255) / 256 * 256;
  sh->off_sx32 = off;
  off += xstage_sx_bytes(K, sh->xrows) / 2;
  off = (off + 255) / 256 * 256;
  sh->off_inv = off;
  off += 256;
  sh->off_part = off;
  if (sh->S > 1) off += (size_t)sh->S * M * w.rows * 4;
  sh->bytes = off;
}

template <int ENC, int NCOL, bool HILO>
int run_gemv(const WRef& w, const void* x, int x_bf16, int M, float* y, const float* residual,
             const Shape& sh, uint8_t* ws, cudaStream_t s) {
  const int K = (int)w.cols;
  __half* xf = reinterpret_cast<__half*>(ws);
  float* sx16 = reinterpret_cast<float*>(ws + sh.off_sx);
  float* sx32 = reinterpret_cast<float*>(ws + sh.off_sx32);
  float* inv_s = reinterpret_cast<float*>(ws + sh.off_inv);
  float* partial = reinterpret_cast<float*>(ws + sh.off_part);
  int sgrid = (K / 32 * 4 * sh.xrows + 255) / 256;
  if (sgrid > 64) sgrid = 64;
  stage_x_kernel<NCOL, HILO><<<sgrid, 256, 0, s>>>(x, x_bf16, M, sh.xrows, K, xl_for_encoding(ENC), xf,
                                                   sx16, sx32, inv_s);
  XView xv{xf, sx16, sx32, inv_s};
  const int64_t units = (int64_t)sh.ntiles * sh.S;
  constexpr int tile_smem = GT_WARPS * 16 * UG<ENC>::PITCH;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(gemv_tile_kernel<ENC, NCOL, HILO>), tile_smem)) return 1;
  gemv_tile_kernel<ENC, NCOL, HILO><<<(unsigned)((units + GT_WARPS - 1) / GT_WARPS), GT_WARPS * 32, tile_smem, s>>>(
      w, xv, M, y, residual, partial, sh.S, sh.kb_per, sh.ntiles);
  count_launch(2);
  if (sh.S > 1) {
    gemv_reduce_kernel<<<(unsigned)(((int64_t)M * w.rows + 255) / 256), 256, 0, s>>>(
        partial, sh.S, M, w.rows, inv_s, y, residual);
    count_launch();
  }
  DYN_CUDA(cudaGetLastError());
  return 0;
}

template <int ENC>
int run_gemv_enc(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                 const Shape& sh, uint8_t* ws, cudaStream_t s) {
  if (x_type == E_BF16) return run_gemv<ENC, 8, false>(w, x, 1, M, y, residual, sh, ws, s);
  if (M == 1) return run_gemv<ENC, 2, true>(w, x, 0, M, y, residual, sh, ws, s);
  return run_gemv<ENC, 8, true>(w, x, 0, M, y, residual, sh, ws, s);
}

bool shape_ok(const WRef& w, int x_type, int M) {
  if (!gemv_mma_supports(w.enc) || w.rows < 1) return false;
  if (w.cols > (1 << 20)) return false;
  // rows must start on the copy granule (16 bytes; Q6_K 8) and hold whole units
  if ((w.enc == E_Q4_0 || w.enc == E_Q8_0) && w.cols % 256) return false;
  if (w.enc == E_Q4_1 && w.cols % 128) return false;
  if (w.enc == E_Q6_K && w.cols % 1024) return false;
  if (w.enc == E_MLX_U4 && (w.cols % 32 || (w.group != 32 && w.group != 64 && w.group != 128 && w.group != 256) || w.cols % w.group)) return false;
  return M >= 1 && M <= (x_type == E_BF16 ? 8 : 4);
}

}  // namespace

// Scratch bytes the product needs (0 when the shape does not qualify for this kernel).
size_t gemv_mma_workspace_bytes(const WRef& w, int x_type, int M) {
  if (const size_t cs = gemv_cs_workspace_bytes(w, M)) return cs;
  if (!shape_ok(w, x_type, M)) return 0;
  Shape sh;
  plan_shape(w, M, x_type == E_BF16, &sh);
  return sh.bytes;
}

// Runs the tensor-core GEMV when the shape qualifies (*handled = true): f32 activations
// M <= 4 (hi/lo pairs), bf16 activations M <= 8. `workspace` may be NULL: the scratch is
// then taken from and returned to the stream-ordered allocator around the launches.
int launch_gemv_mma(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                    void* workspace, cudaStream_t s, bool* handled) {
  *handled = false;
  const size_t cs_bytes = gemv_cs_workspace_bytes(w, M);  // one row, Q4_0: column-split kernel
  if (!cs_bytes && !shape_ok(w, x_type, M)) return 0;
  Shape sh;
  if (cs_bytes)
    sh.bytes = cs_bytes;
  else
    plan_shape(w, M, x_type == E_BF16, &sh);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  if (!ws) ws = reinterpret_cast<uint8_t*>(workspace = thread_scratch(sh.bytes));  // the caller's region
  if (!ws) {
    if (keep_scratch_pool_cached()) return 1;
    DYN_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&ws), sh.bytes, s));
  }
  int rc = 1;
  if (cs_bytes) {
    bool did = false;
    rc = launch_gemv_cs(w, x, x_type, M, y, residual, ws, s, &did);
    if (!rc && !did) rc = 1;
  } else
  switch (w.enc) {
    case E_Q4_0: rc = run_gemv_enc<E_Q4_0>(w, x, x_type, M, y, residual, sh, ws, s); break;
    case E_Q4_1: rc = run_gemv_enc<E_Q4_1>(w, x, x_type, M, y, residual, sh, ws, s); break;
    case E_Q8_0: rc = run_gemv_enc<E_Q8_0>(w, x, x_type, M, y, residual, sh, ws, s); break;
    case E_Q6_K: rc = run_gemv_enc<E_Q6_K>(w, x, x_type, M, y, residual, sh, ws, s); break;
    case E_MLX_U4: rc = run_gemv_enc<E_MLX_U4>(w, x, x_type, M, y, residual, sh, ws, s); break;
    default: break;
  }
  if (!workspace) {
    cudaError_t e = cudaFreeAsync(ws, s);
    if (!rc && e != cudaSuccess) return cuda_fail(e, "cudaFreeAsync", __FILE__, __LINE__);
  }
  if (!rc) *handled = true;
  return rc;
}

}  // namespace dyn
