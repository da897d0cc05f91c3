// Causal GQA attention for prefill chunks: many query rows of ONE sequence at consecutive
// positions against a 2-byte (bf16 / f16) KV cache, on the tensor cores.
//
// Same mathematics as the per-row kernel (kernels.rs:310-458: s = (q.k) * 1/sqrt(d), keys beyond the
// row's position masked, online max / sum merge, out / sum at the end), restructured the usual
// flash-attention way: one CTA = one query head x 64 consecutive rows. The 64-key blocks stream through
// shared memory with cp.async, the next group of blocks in flight while the current one is used.
// Two shapes of CTA: when the grid is no larger than the GPU (a 512-row chunk of a 16-head model: 128
// CTAs), eight warps -- warp w takes the 16 rows of group w mod 4 and, of every PAIR of blocks, block
// w / 4, so two blocks are worked on at once and the two halves' running (max, sum, out) are merged at
// the end (four K + V tiles resident, one CTA per SM); for larger grids four warps and one block at a
// time (two tiles resident, two CTAs per SM). S = Q K^T and O += P V run on mma.sync.m16n8k16 with f32
// accumulators. The cache entries are used
// in their stored type (exact); the f32 operands Q and P enter as hi + lo pairs of that type
// (two mma per tile), so the products carry ~16 significant bits of Q / P and the result stays
// within ~1e-4 of the f32 evaluation.
#include <algorithm>

#include "common.cuh"

namespace dyn {

namespace {

constexpr int FA_D = 128;      // head dim handled by this kernel
constexpr int FA_BR = 64;      // query rows per CTA
constexpr int FA_BC = 64;      // keys per step
constexpr int FA_PITCH = FA_D + 8;  // elements per shared-memory row (272 bytes: conflict-free fragment loads)
constexpr int FA_TILE = FA_BC * FA_PITCH;            // elements of one K (or V) tile
constexpr int fa_threads(int halves) { return 128 * halves; }
constexpr int fa_smem_bytes(int halves) { return 2 * halves * 2 * FA_TILE * 2; }  // buffers x blocks of a group x (K, V) x 2 bytes

__device__ __forceinline__ void fa_cp16(void* dst, const void* src, bool live) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = live ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

template <int KV>
struct Mma;
template <>
struct Mma<E_BF16> {
  using T = __nv_bfloat16;
  __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  // (hi, lo) packed pairs of two f32 values
  __device__ static __forceinline__ void split2(float x, float y, uint32_t* hi, uint32_t* lo) {
    const __nv_bfloat16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
    const __nv_bfloat16 lx = __float2bfloat16_rn(x - __bfloat162float(hx));
    const __nv_bfloat16 ly = __float2bfloat16_rn(y - __bfloat162float(hy));
    *hi = (uint32_t)__bfloat16_as_ushort(hx) | ((uint32_t)__bfloat16_as_ushort(hy) << 16);
    *lo = (uint32_t)__bfloat16_as_ushort(lx) | ((uint32_t)__bfloat16_as_ushort(ly) << 16);
  }
};
template <>
struct Mma<E_F16> {
  using T = __half;
  __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ static __forceinline__ void split2(float x, float y, uint32_t* hi, uint32_t* lo) {
    const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
    const __half lx = __float2half_rn(x - __half2float(hx)), ly = __float2half_rn(y - __half2float(hy));
    *hi = (uint32_t)__half_as_ushort(hx) | ((uint32_t)__half_as_ushort(hy) << 16);
    *lo = (uint32_t)__half_as_ushort(lx) | ((uint32_t)__half_as_ushort(ly) << 16);
  }
};

struct FaArgs {
  const float* q;     // [rows, nh, d]
  const void* kcache; // plane of (seq, kv head): [cap, d]
  const void* vcache;
  float* ctx;         // [rows, nh * d]
  int64_t rows, nh, nkv, cap, base_pos, seq;
  int64_t ldq;        // floats between consecutive rows of q
};

template <int KV, int HALVES>
__global__ void __launch_bounds__(fa_threads(HALVES)) attention_prefill_kernel(const FaArgs a) {
  constexpr int FA_THREADS = fa_threads(HALVES);
  using M = Mma<KV>;
  using T = typename M::T;
  extern __shared__ __align__(16) uint8_t fa_smem[];
  T* const tiles = reinterpret_cast<T*>(fa_smem);  // [buffer][block of the pair][K, V][FA_BC][FA_PITCH]
  const int tid = threadIdx.x, lane = tid & 31, warp8 = tid >> 5;
  const int warp = warp8 & 3, half = warp8 >> 2;   // row group; which block of a group
  const int g = lane >> 2, t = lane & 3;
  const int64_t h = blockIdx.x, rb = gridDim.y - 1 - blockIdx.y;  // the longest row blocks start first
  const int64_t kvh = h / (a.nh / a.nkv);
  const T* kplane = reinterpret_cast<const T*>(a.kcache) + (a.seq * a.nkv + kvh) * a.cap * FA_D;
  const T* vplane = reinterpret_cast<const T*>(a.vcache) + (a.seq * a.nkv + kvh) * a.cap * FA_D;
  const int64_t row_lo = rb * FA_BR + warp * 16;   // this warp's first query row
  const int64_t r0 = row_lo + g, r1 = r0 + 8;      // the lane's two rows
  const int64_t r0c = r0 < a.rows ? r0 : a.rows - 1, r1c = r1 < a.rows ? r1 : a.rows - 1;
  const int64_t pos0 = a.base_pos + r0, pos1 = a.base_pos + r1;
  const float scale = 1.0f / sqrtf((float)FA_D);

  // Q fragments (hi, lo) for the 8 k-steps over the head dim
  uint32_t qh[8][4], ql[8][4];
  {
    const float* q0 = a.q + r0c * a.ldq + h * FA_D;
    const float* q1 = a.q + r1c * a.ldq + h * FA_D;
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
      const float2 a0 = *reinterpret_cast<const float2*>(q0 + 16 * kk + 2 * t);
      const float2 a1 = *reinterpret_cast<const float2*>(q1 + 16 * kk + 2 * t);
      const float2 a2 = *reinterpret_cast<const float2*>(q0 + 16 * kk + 8 + 2 * t);
      const float2 a3 = *reinterpret_cast<const float2*>(q1 + 16 * kk + 8 + 2 * t);
      M::split2(a0.x, a0.y, &qh[kk][0], &ql[kk][0]);
      M::split2(a1.x, a1.y, &qh[kk][1], &ql[kk][1]);
      M::split2(a2.x, a2.y, &qh[kk][2], &ql[kk][2]);
      M::split2(a3.x, a3.y, &qh[kk][3], &ql[kk][3]);
    }
  }
  float o[16][4];
#pragma unroll
  for (int dt = 0; dt < 16; dt++) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
  float m0 = -3.40282347e38f, m1 = -3.40282347e38f, l0 = 0.f, l1 = 0.f;

  // keys 0 .. last position of the CTA's rows
  int64_t cta_last = a.base_pos + rb * FA_BR + FA_BR - 1;
  if (cta_last > a.base_pos + a.rows - 1) cta_last = a.base_pos + a.rows - 1;
  const int64_t warp_last = a.base_pos + (row_lo + 15 < a.rows ? row_lo + 15 : a.rows - 1);
  const int64_t nkb = cta_last / FA_BC + 1, npairs = (nkb + HALVES - 1) / HALVES;
  // HALVES blocks x (K, V) x 64 keys x 16 pieces of 16 bytes per group, coalesced; rows past the last written
  // position may hold anything: they are masked, but 0 * NaN must not happen, so they arrive as zeros
  auto load_pair = [&](int64_t pr) {
    T* dst = tiles + (pr & 1) * 2 * HALVES * FA_TILE;
    for (int i = tid; i < HALVES * FA_BC * (FA_D / 8); i += FA_THREADS) {
      const int blk = i / (FA_BC * (FA_D / 8)), key = (i / (FA_D / 8)) % FA_BC, c = i % (FA_D / 8);
      const int64_t gk = (HALVES * pr + blk) * FA_BC + key;  // < cap for every written key
      const bool written = gk <= cta_last;
      const int64_t src = (written ? gk : 0) * FA_D + c * 8;
      fa_cp16(dst + (blk * 2) * FA_TILE + key * FA_PITCH + c * 8, kplane + src, written);
      fa_cp16(dst + (blk * 2 + 1) * FA_TILE + key * FA_PITCH + c * 8, vplane + src, written);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_pair(0);
  for (int64_t pr = 0; pr < npairs; pr++) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // pair pr has arrived for everyone, and nobody still reads the buffer the next pair goes to
    if (pr + 1 < npairs) load_pair(pr + 1);
    const int64_t kb = HALVES * pr + half;
    if (kb >= nkb) continue;
    const T(*ks)[FA_PITCH] = reinterpret_cast<const T(*)[FA_PITCH]>(tiles + ((pr & 1) * 2 * HALVES + half * 2) * FA_TILE);
    const T(*vs)[FA_PITCH] = reinterpret_cast<const T(*)[FA_PITCH]>(tiles + ((pr & 1) * 2 * HALVES + half * 2 + 1) * FA_TILE);
    if (kb * FA_BC > warp_last) continue;  // every key of the block lies after this warp's rows
    // ---- S = Q K^T for 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const T* krow = &ks[nt * 8 + g][0];
#pragma unroll
      for (int kk = 0; kk < 8; kk++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + 16 * kk + 2 * t);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + 16 * kk + 8 + 2 * t);
        M::mma(s[nt], qh[kk], b0, b1);
        M::mma(s[nt], ql[kk], b0, b1);
      }
    }
    // ---- scale, causal mask, running maximum
    float bm0 = -3.40282347e38f, bm1 = -3.40282347e38f;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int64_t key = kb * FA_BC + nt * 8 + 2 * t + e;
        s[nt][e] = key <= pos0 ? s[nt][e] * scale : -3.40282347e38f;
        s[nt][2 + e] = key <= pos1 ? s[nt][2 + e] * scale : -3.40282347e38f;
        bm0 = fmaxf(bm0, s[nt][e]);
        bm1 = fmaxf(bm1, s[nt][2 + e]);
      }
    }
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
    bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
    bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
    const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
    const float f0 = expf(m0 - mn0), f1 = expf(m1 - mn1);
    m0 = mn0, m1 = mn1;
    l0 *= f0, l1 *= f1;
#pragma unroll
    for (int dt = 0; dt < 16; dt++) {
      o[dt][0] *= f0, o[dt][1] *= f0;
      o[dt][2] *= f1, o[dt][3] *= f1;
    }
    // ---- P = exp(S - m) (masked keys give exactly 0 once a real key has been seen), hi/lo fragments
    uint32_t ph[4][4], pl[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int64_t key = kb * FA_BC + nt * 8 + 2 * t + e;
        p[e] = key <= pos0 ? expf(s[nt][e] - m0) : 0.f;
        p[2 + e] = key <= pos1 ? expf(s[nt][2 + e] - m1) : 0.f;
      }
      l0 += p[0] + p[1];
      l1 += p[2] + p[3];
      // accumulator tiles 2j, 2j+1 are the A fragment of k-step j of P V
      const int j = nt >> 1, half = nt & 1;
      M::split2(p[0], p[1], &ph[j][2 * half], &pl[j][2 * half]);          // row g
      M::split2(p[2], p[3], &ph[j][2 * half + 1], &pl[j][2 * half + 1]);  // row g + 8
    }
    // ---- O += P V: B fragments come transposed out of the [key][dim] tile
#pragma unroll
    for (int dt = 0; dt < 16; dt++) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        uint32_t b0, b1;
        const T* vrow = &vs[16 * j + (lane & 15)][dt * 8];  // lanes 0..7: keys 16j.., 8..15: keys 16j+8..
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
                     : "=r"(b0), "=r"(b1)
                     : "r"((uint32_t)__cvta_generic_to_shared(vrow)));
        M::mma(o[dt], ph[j], b0, b1);
        M::mma(o[dt], pl[j], b0, b1);
      }
    }
  }
  // ---- merge the two halves' running states (thread for thread: both cover the same rows and columns)
  if constexpr (HALVES == 2) {
  __syncthreads();  // the tiles are no longer read
  float* const mg = reinterpret_cast<float*>(fa_smem) + (size_t)(warp * 32 + lane) * 68;
  if (half == 1) {
    mg[0] = m0, mg[1] = m1, mg[2] = l0, mg[3] = l1;
#pragma unroll
    for (int dt = 0; dt < 16; dt++)
      *reinterpret_cast<float4*>(mg + 4 + 4 * dt) = make_float4(o[dt][0], o[dt][1], o[dt][2], o[dt][3]);
  }
  __syncthreads();
  if (half == 1) return;
  {
    const float mb0 = mg[0], mb1 = mg[1];
    const float mn0 = fmaxf(m0, mb0), mn1 = fmaxf(m1, mb1);
    const float fa0 = expf(m0 - mn0), fb0 = expf(mb0 - mn0), fa1 = expf(m1 - mn1), fb1 = expf(mb1 - mn1);
    l0 = l0 * fa0 + mg[2] * fb0;
    l1 = l1 * fa1 + mg[3] * fb1;
#pragma unroll
    for (int dt = 0; dt < 16; dt++) {
      const float4 ob = *reinterpret_cast<const float4*>(mg + 4 + 4 * dt);
      o[dt][0] = o[dt][0] * fa0 + ob.x * fb0, o[dt][1] = o[dt][1] * fa0 + ob.y * fb0;
      o[dt][2] = o[dt][2] * fa1 + ob.z * fb1, o[dt][3] = o[dt][3] * fa1 + ob.w * fb1;
    }
  }
  }
  // ---- out / sum
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
  for (int dt = 0; dt < 16; dt++) {
    if (r0 < a.rows)
      *reinterpret_cast<float2*>(a.ctx + r0 * a.nh * FA_D + h * FA_D + dt * 8 + 2 * t) =
          make_float2(o[dt][0] * i0, o[dt][1] * i0);
    if (r1 < a.rows)
      *reinterpret_cast<float2*>(a.ctx + r1 * a.nh * FA_D + h * FA_D + dt * 8 + 2 * t) =
          make_float2(o[dt][2] * i1, o[dt][3] * i1);
  }
}

}  // namespace

// Tensor-core attention for `a.rows` query rows of sequence `seq` at positions base_pos + row.
// *handled = false when the shape does not qualify (f32 cache, head dim != 128, few rows).
int launch_attention_prefill(const AttnArgs& a, int64_t base_pos, int64_t seq, cudaStream_t s, bool* handled) {
  *handled = false;
  if (a.d != FA_D || a.rows < 32 || (a.kv_type != E_BF16 && a.kv_type != E_F16)) return 0;
  if (a.nkv <= 0 || a.nh % a.nkv || a.cap % FA_BC) return 0;
  FaArgs f;
  f.q = a.q, f.kcache = a.kcache, f.vcache = a.vcache, f.ctx = a.ctx;
  f.rows = a.rows, f.nh = a.nh, f.nkv = a.nkv, f.cap = a.cap, f.base_pos = base_pos, f.seq = seq;
  f.ldq = a.ldq ? a.ldq : a.nh * FA_D;
  const dim3 grid((unsigned)a.nh, (unsigned)((a.rows + FA_BR - 1) / FA_BR));
  // a grid that fits the GPU in one round: eight warps and pairs of key blocks; larger: four warps, two CTAs per SM
  const bool pairs = (int64_t)grid.x * grid.y <= std::max(1, sm_count());
  auto run = [&](auto kernel, int halves) -> int {
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), fa_smem_bytes(halves))) return 1;
    kernel<<<grid, fa_threads(halves), fa_smem_bytes(halves), s>>>(f);
    return 0;
  };
  int rc;
  if (a.kv_type == E_BF16)
    rc = pairs ? run(attention_prefill_kernel<E_BF16, 2>, 2) : run(attention_prefill_kernel<E_BF16, 1>, 1);
  else
    rc = pairs ? run(attention_prefill_kernel<E_F16, 2>, 2) : run(attention_prefill_kernel<E_F16, 1>, 1);
  if (rc) return 1;
  count_launch();
  DYN_CUDA(cudaGetLastError());
  *handled = true;
  return 0;
}

}  // namespace dyn
