// Warp-level building blocks of the fused dequant-GEMV (1..8 activation rows).
//
// The matrix-vector products of decode are HBM-bound, but decoding 4/6/8-bit
// blocks on the scalar pipes costs 8-9 instructions per weight and becomes the
// limiter long before HBM does. These routines cut that to ~2 per weight:
//
//   * quantised integers are never converted: the raw nibble / byte / 6-bit value
//     q is placed in the low mantissa bits of an f16, which is the subnormal
//     number q * 2^-24 — exact, one logic op per two weights;
//   * a 16-row x 16-k tile of such values is the A operand of
//     mma.sync.m16n8k16 (f16 in, f32 accumulate); the B operand holds the
//     activations, pre-arranged once per vector in shared memory in the exact
//     register order the unpacking produces ("fragment order");
//   * block scales, zero points and minima are applied to the f32 tile sums:
//     sum_k x_k*(q_k*d + m) = d * sum_k x_k q_k + m * sum_k x_k, with the
//     per-block activation sums computed once per vector.
//
// The products q*x are exact (integer x f16) and accumulation is f32. An f32
// activation row enters as an f16 pair hi + lo (22 significant bits) in two
// B columns, scaled by a power of two so that its largest entry sits near 2^13;
// the result tracks the f32 reference to ~1e-6 relative. bf16 activation rows
// are exact in one f16 column each. The tensor pipe is used for instruction
// economy, not for FLOPs: the kernel stays HBM-bound.
#pragma once

#include "common.cuh"

namespace dyn {

constexpr float GV_2P24 = 16777216.0f;

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- activation staging ---------------------------------------------------------------
// Fragment layouts (per 32-element block kb, column c, lane quarter t = lane & 3), 8 halfs:
//   NIBBLE (Q4_0, Q4_1): x[4t] x[4t+2] x[16+4t]/16 x[16+4t+2]/16 x[4t+1] x[4t+3]
//                        x[16+4t+1]/16 x[16+4t+3]/16
//   MLXW   (MLX u4)    : x[8t] x[8t+4] x[8t+1]/16 x[8t+5]/16 x[8t+2] x[8t+6] x[8t+3]/16 x[8t+7]/16
//   BYTES  (Q8_0, Q6_K): x[4t] x[4t+1] x[4t+2] x[4t+3] x[16+4t] ... x[16+4t+3]
//   BF16N  (plain bf16): the order of BYTES, the fragments held as bf16 (hi + lo) instead of f16
// The /16 compensates high nibbles that are used in place (as 16*q).
enum { XL_NIBBLE = 0, XL_MLXW = 1, XL_BYTES = 2, XL_BF16N = 3 };

__host__ __device__ inline int xl_for_encoding(int enc) {
  return (enc == E_Q4_0 || enc == E_Q4_1) ? XL_NIBBLE
                                         : (enc == E_MLX_U4 ? XL_MLXW : (enc == E_BF16 ? XL_BF16N : XL_BYTES));
}

__device__ __forceinline__ int xl_index(int layout, int t, int i) {
  // element offset (within the 32-block) of half i of lane quarter t; bit 8 set = divide by 16
  if (layout == XL_NIBBLE) {
    const int hi = (i >> 1) & 1, odd = (i >> 2) & 1, second = i & 1;
    return (hi ? 16 : 0) + 4 * t + odd + 2 * second + (hi ? 256 : 0);
  }
  if (layout == XL_MLXW) {
    const int pair = i >> 1, second = i & 1;  // pair p holds nibbles p and p+4
    return 8 * t + pair + 4 * second + ((pair & 1) ? 256 : 0);
  }
  return (i >> 2) * 16 + 4 * t + (i & 3);
}

// Shared-memory footprint of the staged activations.
__host__ __device__ inline size_t xstage_xf_bytes(int K, int ncol) { return (size_t)(K / 32) * ncol * 64; }
__host__ __device__ inline size_t xstage_sx_bytes(int K, int rows) { return (size_t)(K / 16) * rows * 4; }

// Power-of-two scale for one activation row whose largest magnitude is `mx`:
// mx * s lies in [2^12, 2^13).
__device__ __forceinline__ void scale_for(float mx, float* s, float* inv_s) {
  int e = 0;
  if (mx > 0.f && mx < 3.0e38f) frexpf(mx, &e);
  *s = ldexpf(1.0f, 13 - e);
  *inv_s = ldexpf(1.0f, e - 13);
}

// Writes the fragments of one (block, lane-quarter) of one activation row.
//   HILO: two columns (2*m, 2*m+1) hold hi and lo; else one column m holds the f16 value.
template <int NCOL, bool HILO>
__device__ __forceinline__ void stage_item(const float* src, int layout, __half* xf, int kb, int t,
                                           int m, float s) {
  __half hi[8], lo[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int code = xl_index(layout, t, i);
    float v = src[kb * 32 + (code & 255)] * s;
    if (code & 256) v *= 0.0625f;
    const __half h = __float2half_rn(v);
    hi[i] = h;
    lo[i] = __float2half_rn(v - __half2float(h));
  }
  if (HILO) {
    uint4* dst = reinterpret_cast<uint4*>(xf + ((size_t)(kb * NCOL + 2 * m) * 4 + t) * 8);
    dst[0] = *reinterpret_cast<uint4*>(hi);
    dst[4] = *reinterpret_cast<uint4*>(lo);  // the next column starts 4 lane-quarters further
  } else {
    *reinterpret_cast<uint4*>(xf + ((size_t)(kb * NCOL + m) * 4 + t) * 8) =
        *reinterpret_cast<uint4*>(hi);
  }
}

// ---- accumulators ------------------------------------------------------------------------
// A lane (g = lane >> 2, t = lane & 3) owns weight rows g and g + 8 of the tile.
//   HILO : activation row t (columns 2t = hi, 2t+1 = lo): v[0] = row g, v[1] = row g + 8
//   plain: activation rows 2t and 2t+1: v[0],v[1] = row g; v[2],v[3] = row g + 8
template <bool HILO>
struct TileAcc {
  float v[HILO ? 2 : 4];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < (HILO ? 2 : 4); i++) v[i] = 0.f;
  }
};

// ---- fast unit steps (static addressing) --------------------------------------------------
// A "unit" is the smallest run of blocks whose 4-byte phase is known at compile time: block
// sizes 18 / 34 / 210 are 2 (mod 4), so the phase flips every block and a unit is a pair (the
// caller guarantees units start 4-byte aligned); 20- and 16-byte blocks are always aligned.
// p0 / p1 point at the unit in rows g and g + 8 (any memory space). Accumulators are kept in
// units of 2^-24 (the caller multiplies the final sums by 2^24 / scale once).
template <int MIS>  // MIS = address mod 4 of q (0 or 2)
__device__ __forceinline__ uint32_t ld32_ph(const uint8_t* q) {
  if (MIS == 0) return *reinterpret_cast<const uint32_t*>(q);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(q - 2);
  return __funnelshift_r(w[0], w[1], 16);
}
__device__ __forceinline__ float ldh_f32(const uint8_t* q) {
  return __half2float(*reinterpret_cast<const __half*>(q));
}

constexpr float GV_2M24 = 5.9604644775390625e-08f;  // 2^-24

// acc (in 2^-24 units) += sc * (S - z * sx) with S the tile sums, for the lane's two rows.
template <bool HILO>
__device__ __forceinline__ void unit_apply(TileAcc<HILO>& a, const float (&c)[4], float sc0, float sc1,
                                           float z24, float sxa, float sxb) {
  if (HILO) {
    a.v[0] = fmaf(sc0, fmaf(-z24, sxa, c[0] + c[1]), a.v[0]);
    a.v[1] = fmaf(sc1, fmaf(-z24, sxa, c[2] + c[3]), a.v[1]);
  } else {
    a.v[0] = fmaf(sc0, fmaf(-z24, sxa, c[0]), a.v[0]);
    a.v[1] = fmaf(sc0, fmaf(-z24, sxb, c[1]), a.v[1]);
    a.v[2] = fmaf(sc1, fmaf(-z24, sxa, c[2]), a.v[2]);
    a.v[3] = fmaf(sc1, fmaf(-z24, sxb, c[3]), a.v[3]);
  }
}
// acc += sc * S + ad * (2^-24 sx)
template <bool HILO>
__device__ __forceinline__ void unit_apply_add(TileAcc<HILO>& a, const float (&c)[4], float sc0, float sc1,
                                               float ad0, float ad1, float sxa24, float sxb24) {
  if (HILO) {
    a.v[0] = fmaf(sc0, c[0] + c[1], fmaf(ad0, sxa24, a.v[0]));
    a.v[1] = fmaf(sc1, c[2] + c[3], fmaf(ad1, sxa24, a.v[1]));
  } else {
    a.v[0] = fmaf(sc0, c[0], fmaf(ad0, sxa24, a.v[0]));
    a.v[1] = fmaf(sc0, c[1], fmaf(ad0, sxb24, a.v[1]));
    a.v[2] = fmaf(sc1, c[2], fmaf(ad1, sxa24, a.v[2]));
    a.v[3] = fmaf(sc1, c[3], fmaf(ad1, sxb24, a.v[3]));
  }
}

// One Q4_0 / Q4_1 block. PH: phase (0 / 2) of the block base. xfp: this lane's fragment
// pointer for the block; sxa/sxb: 32-block activation sums of the lane's row(s). bs: an extra
// factor on the block's contribution (callers that scale every activation block by its own power
// of two pass 2^24 / that scale and keep their accumulators in true units).
template <int ENC, int PH, bool HILO>
__device__ __forceinline__ void blk_q4(const uint8_t* p0, const uint8_t* p1, const __half* xfp,
                                       float sxa, float sxb, int t, TileAcc<HILO>& acc, float bs = 1.0f) {
  constexpr int QO = ENC == E_Q4_0 ? 2 : 4;
  const uint32_t w0 = ld32_ph<(PH + QO) & 3>(p0 + QO + 4 * t);
  const uint32_t w1 = ld32_ph<(PH + QO) & 3>(p1 + QO + 4 * t);
  const uint4 b = *reinterpret_cast<const uint4*>(xfp);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  mma_f16_16816(c, w0 & 0x000F000Fu, w1 & 0x000F000Fu, w0 & 0x00F000F0u, w1 & 0x00F000F0u, b.x, b.y);
  const uint32_t s0 = w0 >> 8, s1 = w1 >> 8;
  mma_f16_16816(c, s0 & 0x000F000Fu, s1 & 0x000F000Fu, s0 & 0x00F000F0u, s1 & 0x00F000F0u, b.z, b.w);
  const float d0 = ldh_f32(p0) * bs, d1 = ldh_f32(p1) * bs;
  if (ENC == E_Q4_0)
    unit_apply<HILO>(acc, c, d0, d1, 8.0f * GV_2M24, sxa, sxb);
  else
    unit_apply_add<HILO>(acc, c, d0, d1, ldh_f32(p0 + 2) * bs, ldh_f32(p1 + 2) * bs, sxa * GV_2M24, sxb * GV_2M24);
}

template <int PH, bool HILO>
__device__ __forceinline__ void blk_q8_0(const uint8_t* p0, const uint8_t* p1, const __half* xfp,
                                         float sxa, float sxb, int t, TileAcc<HILO>& acc, float bs = 1.0f) {
  const uint4 b = *reinterpret_cast<const uint4*>(xfp);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int hlf = 0; hlf < 2; hlf++) {
    const uint32_t w0 = ld32_ph<(PH + 2) & 3>(p0 + 2 + 16 * hlf + 4 * t) ^ 0x80808080u;
    const uint32_t w1 = ld32_ph<(PH + 2) & 3>(p1 + 2 + 16 * hlf + 4 * t) ^ 0x80808080u;
    mma_f16_16816(c, __byte_perm(w0, 0, 0x4140), __byte_perm(w1, 0, 0x4140), __byte_perm(w0, 0, 0x4342),
                  __byte_perm(w1, 0, 0x4342), hlf ? b.z : b.x, hlf ? b.w : b.y);
  }
  unit_apply<HILO>(acc, c, ldh_f32(p0) * bs, ldh_f32(p1) * bs, 128.0f * GV_2M24, sxa, sxb);
}

// One block of 32 plain 16-bit weights (64 bytes, 4-byte aligned): bf16 weights against bf16
// activation fragments (layout BF16N), f16 weights against f16 fragments (layout BYTES). The
// weights are the A operand as they lie in memory: lane quarter t owns elements 4t .. 4t+3 of
// each half of the block. scale: what turns the tile sums back into true units.
template <bool BF16, bool HILO>
__device__ __forceinline__ void blk_plain16(const uint8_t* p0, const uint8_t* p1, const __half* xfp, int t,
                                            TileAcc<HILO>& acc, float scale) {
  const uint4 b = *reinterpret_cast<const uint4*>(xfp);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int hlf = 0; hlf < 2; hlf++) {
    const uint2 w0 = *reinterpret_cast<const uint2*>(p0 + 32 * hlf + 8 * t);
    const uint2 w1 = *reinterpret_cast<const uint2*>(p1 + 32 * hlf + 8 * t);
    if (BF16)
      mma_bf16_16816(c, w0.x, w1.x, w0.y, w1.y, hlf ? b.z : b.x, hlf ? b.w : b.y);
    else
      mma_f16_16816(c, w0.x, w1.x, w0.y, w1.y, hlf ? b.z : b.x, hlf ? b.w : b.y);
  }
  if (HILO) {
    acc.v[0] = fmaf(scale, c[0] + c[1], acc.v[0]);
    acc.v[1] = fmaf(scale, c[2] + c[3], acc.v[1]);
  } else {
    acc.v[0] = fmaf(scale, c[0], acc.v[0]);
    acc.v[1] = fmaf(scale, c[1], acc.v[1]);
    acc.v[2] = fmaf(scale, c[2], acc.v[2]);
    acc.v[3] = fmaf(scale, c[3], acc.v[3]);
  }
}

template <bool HILO>
__device__ __forceinline__ void blk_mlx(const uint8_t* p0, const uint8_t* p1, float s0, float s1,
                                        float b0, float b1, const __half* xfp, float sxa, float sxb,
                                        int t, TileAcc<HILO>& acc) {
  const uint32_t w0 = *reinterpret_cast<const uint32_t*>(p0 + 4 * t);
  const uint32_t w1 = *reinterpret_cast<const uint32_t*>(p1 + 4 * t);
  const uint4 b = *reinterpret_cast<const uint4*>(xfp);
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  mma_f16_16816(c, w0 & 0x000F000Fu, w1 & 0x000F000Fu, w0 & 0x00F000F0u, w1 & 0x00F000F0u, b.x, b.y);
  const uint32_t h0 = w0 >> 8, h1 = w1 >> 8;
  mma_f16_16816(c, h0 & 0x000F000Fu, h1 & 0x000F000Fu, h0 & 0x00F000F0u, h1 & 0x00F000F0u, b.z, b.w);
  unit_apply_add<HILO>(acc, c, s0, s1, b0, b1, sxa * GV_2M24, sxb * GV_2M24);
}

// One Q6_K superblock (8 blocks of 32). PH: phase of the superblock base. xfp points at the
// lane's fragments of the superblock's first 32-block, consecutive blocks XSTRIDE halfs apart;
// sxa/sxb point at the 16-run sums of that first block (two per block).
template <int PH, bool HILO>
__device__ __forceinline__ void sblk_q6_k(const uint8_t* p0, const uint8_t* p1, const __half* xfp,
                                          int xstride, const float* sxa, const float* sxb, int t,
                                          TileAcc<HILO>& acc) {
  const float d0 = ldh_f32(p0 + 208), d1 = ldh_f32(p1 + 208);
#pragma unroll
  for (int e32 = 0; e32 < 8; e32++) {
    const int n = e32 >> 2, h = (e32 >> 1) & 1, p = e32 & 1;
    const uint4 b = *reinterpret_cast<const uint4*>(xfp + (size_t)e32 * xstride);
#pragma unroll
    for (int s = 0; s < 2; s++) {
      const int j0 = 16 * s + 4 * t;
      const uint32_t l0 = ld32_ph<PH>(p0 + n * 64 + p * 32 + j0) >> (4 * h);
      const uint32_t l1 = ld32_ph<PH>(p1 + n * 64 + p * 32 + j0) >> (4 * h);
      const uint32_t q0 = ld32_ph<PH>(p0 + 128 + n * 32 + j0) >> (2 * (h * 2 + p));
      const uint32_t q1 = ld32_ph<PH>(p1 + 128 + n * 32 + j0) >> (2 * (h * 2 + p));
      const uint32_t v0 = (l0 & 0x0F0F0F0Fu) | ((q0 & 0x03030303u) << 4);
      const uint32_t v1 = (l1 & 0x0F0F0F0Fu) | ((q1 & 0x03030303u) << 4);
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      mma_f16_16816(c, __byte_perm(v0, 0, 0x4140), __byte_perm(v1, 0, 0x4140), __byte_perm(v0, 0, 0x4342),
                    __byte_perm(v1, 0, 0x4342), s ? b.z : b.x, s ? b.w : b.y);
      const int sci = 192 + n * 8 + h * 4 + p * 2 + s;
      const float f0 = d0 * (float)*reinterpret_cast<const int8_t*>(p0 + sci);
      const float f1 = d1 * (float)*reinterpret_cast<const int8_t*>(p1 + sci);
      unit_apply<HILO>(acc, c, f0, f1, 32.0f * GV_2M24, sxa[2 * e32 + s], HILO ? 0.f : sxb[2 * e32 + s]);
    }
  }
}

// One quarter of a Q6_K superblock: half n (128 elements), 16-element sub-block s of each of
// its four 32-element slices (h, p). Loads the qh word once and each ql word once.
// xfp: the lane's fragments of the superblock's first 32-block (xstride halfs per block);
// sxa/sxb: 16-run sums of that first block.
template <int PH, bool HILO>
__device__ __forceinline__ void q6k_quarter(const uint8_t* p0, const uint8_t* p1, int n, int s,
                                            const __half* xfp, int xstride, const float* sxa,
                                            const float* sxb, int t, TileAcc<HILO>& acc, float bs = 1.0f) {
  const int j0 = 16 * s + 4 * t;
  const float d0 = ldh_f32(p0 + 208) * bs, d1 = ldh_f32(p1 + 208) * bs;
  const uint32_t qh0 = ld32_ph<PH>(p0 + 128 + n * 32 + j0), qh1 = ld32_ph<PH>(p1 + 128 + n * 32 + j0);
#pragma unroll
  for (int p = 0; p < 2; p++) {
    const uint32_t ql0 = ld32_ph<PH>(p0 + n * 64 + p * 32 + j0), ql1 = ld32_ph<PH>(p1 + n * 64 + p * 32 + j0);
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int e32 = n * 4 + h * 2 + p;
      const uint4 b = *reinterpret_cast<const uint4*>(xfp + (size_t)e32 * xstride);
      const uint32_t v0 = ((ql0 >> (4 * h)) & 0x0F0F0F0Fu) | (((qh0 >> (2 * (h * 2 + p))) & 0x03030303u) << 4);
      const uint32_t v1 = ((ql1 >> (4 * h)) & 0x0F0F0F0Fu) | (((qh1 >> (2 * (h * 2 + p))) & 0x03030303u) << 4);
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      mma_f16_16816(c, __byte_perm(v0, 0, 0x4140), __byte_perm(v1, 0, 0x4140), __byte_perm(v0, 0, 0x4342),
                    __byte_perm(v1, 0, 0x4342), s ? b.z : b.x, s ? b.w : b.y);
      const int sci = 192 + n * 8 + h * 4 + p * 2 + s;
      const float f0 = d0 * (float)*reinterpret_cast<const int8_t*>(p0 + sci);
      const float f1 = d1 * (float)*reinterpret_cast<const int8_t*>(p1 + sci);
      unit_apply<HILO>(acc, c, f0, f1, 32.0f * GV_2M24, sxa[2 * e32 + s], HILO ? 0.f : sxb[2 * e32 + s]);
    }
  }
}

__host__ __device__ inline bool gemv_mma_supports(int enc) {
  return enc == E_Q4_0 || enc == E_Q4_1 || enc == E_Q8_0 || enc == E_Q6_K || enc == E_MLX_U4;
}
// Bytes of one 32-element block inside a row (Q6_K: handled per 256-element superblock).
__host__ __device__ inline int gemv_block32_bytes(int enc) {
  switch (enc) {
    case E_Q4_0: return 18;
    case E_Q4_1: return 20;
    case E_Q8_0: return 34;
    case E_MLX_U4: return 16;
    default: return 0;
  }
}

}  // namespace dyn
