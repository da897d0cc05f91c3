// Causal GQA attention for prefill chunks: many query rows of ONE sequence at consecutive
// positions against a 2-byte (bf16 / f16) KV cache, on the tensor cores.
//
// Same mathematics as the per-row kernel (kernels.rs:310-458: s = (q.k) * 1/sqrt(d), keys beyond the
// row's position masked, online max / sum merge, out / sum at the end), restructured the usual
// flash-attention way: one CTA = one query head x 64 consecutive rows, four warps x 16 rows; the
// key / value rows of the head's KV plane stream through shared memory 64 keys at a time;
// S = Q K^T and O += P V run on mma.sync.m16n8k16 with f32 accumulators. The cache entries are used
// in their stored type (exact); the f32 operands Q and P enter as hi + lo pairs of that type
// (two mma per tile), so the products carry ~16 significant bits of Q / P and the result stays
// within ~1e-4 of the f32 evaluation.
#include "common.cuh"

namespace dyn {

namespace {

constexpr int FA_D = 128;      // head dim handled by this kernel
constexpr int FA_BR = 64;      // query rows per CTA
constexpr int FA_BC = 64;      // keys per step
constexpr int FA_PITCH = FA_D + 8;  // elements per shared-memory row (272 bytes: conflict-free fragment loads)

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

template <int KV>
__global__ void __launch_bounds__(128) attention_prefill_kernel(const FaArgs a) {
  using M = Mma<KV>;
  using T = typename M::T;
  __shared__ __align__(16) T ks[FA_BC][FA_PITCH];
  __shared__ __align__(16) T vs[FA_BC][FA_PITCH];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int64_t h = blockIdx.x, rb = blockIdx.y;
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
  for (int64_t kb = 0; kb * FA_BC <= cta_last; kb++) {
    __syncthreads();  // the previous block is no longer read
    // 64 keys x 256 bytes each for K and V: 16-byte pieces, coalesced
    for (int i = tid; i < FA_BC * (FA_D / 8); i += 128) {
      const int key = i / (FA_D / 8), c = i % (FA_D / 8);
      const int64_t gk = kb * FA_BC + key;   // < cap: the capacity is a multiple of the page size
      // rows past the last written position may hold anything: they are masked, but 0 * NaN must not happen
      const bool written = gk <= cta_last;
      const uint4 z = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(&ks[key][c * 8]) =
          written ? *reinterpret_cast<const uint4*>(kplane + gk * FA_D + c * 8) : z;
      *reinterpret_cast<uint4*>(&vs[key][c * 8]) =
          written ? *reinterpret_cast<const uint4*>(vplane + gk * FA_D + c * 8) : z;
    }
    __syncthreads();
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
  if (a.kv_type == E_BF16)
    attention_prefill_kernel<E_BF16><<<grid, 128, 0, s>>>(f);
  else
    attention_prefill_kernel<E_F16><<<grid, 128, 0, s>>>(f);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  *handled = true;
  return 0;
}

}  // namespace dyn
