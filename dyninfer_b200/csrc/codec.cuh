// Exact (bit-for-bit) decoders for the raw checkpoint encodings.
//
// Every encoding is cut into "parts": the unit one thread decodes at a time.
// A part yields 4*G consecutive-in-groups weights: group g covers the four
// logical elements [xoff(part, g), xoff(part, g) + 4) of its block. Products
// and sums are formed with __fmul_rn / __fadd_rn so that the compiler cannot
// contract them into an FMA: the reference rounds the multiply and the add
// separately (arith.mulf then arith.addf,
// crates/dyninfer-quantization/src/quantizations/gguf_codegen.rs:464-465,
// mlx_affine.rs:596-597).
#pragma once

#include "common.cuh"

namespace dyn {

struct RowPtr {  // one weight row
  const uint8_t* data;
  const uint8_t* sc;  // MLX: this row's scales
  const uint8_t* bi;  // MLX: this row's biases
  int aux, group;
};

__device__ __forceinline__ RowPtr row_ptr(const WRef& w, int64_t row) {
  RowPtr r;
  r.data = w.data + row * w.row_bytes();
  r.aux = w.aux;
  r.group = w.group;
  if (w.enc == E_MLX_U4) {
    int64_t per_row = (w.cols / w.group) * (w.aux == E_F32 ? 4 : 2);
    r.sc = w.scales + row * per_row;
    r.bi = w.biases + row * per_row;
  } else {
    r.sc = r.bi = nullptr;
  }
  return r;
}

template <int ENC>
struct Codec;

// Q4_0: f16 d @0, 16 bytes @2; byte l: low nibble = element l, high = l+16;
// w = f32(q - 8) * f32(d). gguf_codegen.rs:412-472.
template <>
struct Codec<E_Q4_0> {
  static constexpr int BLOCK = 32, BYTES = 18, PARTS = 4, G = 2, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int part, int g) { return g * 16 + 4 * part; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t q = ld_u32_a2(b + 2 + 4 * part);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t byte = (q >> (8 * i)) & 0xffu;
      w[i] = __fmul_rn((float)((int)(byte & 15u) - 8), d);
      w[4 + i] = __fmul_rn((float)((int)(byte >> 4) - 8), d);
    }
  }
};

// Q4_1: f16 d @0, f16 m @2, 16 bytes @4; w = f32(q)*d + m. gguf_codegen.rs:373-375,425-465.
template <>
struct Codec<E_Q4_1> {
  static constexpr int BLOCK = 32, BYTES = 20, PARTS = 4, G = 2, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int part, int g) { return g * 16 + 4 * part; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;
    const float d = f16_bits_to_f32(ld_u16(b));
    const float m = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t q = *reinterpret_cast<const uint32_t*>(b + 4 + 4 * part);  // 20*blk is 4-aligned
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t byte = (q >> (8 * i)) & 0xffu;
      w[i] = __fadd_rn(__fmul_rn((float)(byte & 15u), d), m);
      w[4 + i] = __fadd_rn(__fmul_rn((float)(byte >> 4), d), m);
    }
  }
};

// Q8_0: f16 d @0, 32 int8 @2; w = f32(q) * d. gguf_codegen.rs:382-410.
template <>
struct Codec<E_Q8_0> {
  static constexpr int BLOCK = 32, BYTES = 34, PARTS = 8, G = 1, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int part, int) { return 4 * part; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t q = ld_u32_a2(b + 2 + 4 * part);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int v = (int)(int8_t)((q >> (8 * i)) & 0xffu);
      w[i] = __fmul_rn((float)v, d);
    }
  }
};

// Q6_K: ql 128 B @0, qh 64 B @128, 16 int8 scales @192, f16 d @208.
// element e = n*128 + h*64 + p*32 + j: ql byte n*64+p*32+j nibble h, qh byte
// n*32+j field h*2+p, scale n*8+h*4+p*2+j/16; w = (f32(q-32)*f32(sc))*f32(d).
// gguf_codegen.rs:474-526. A part is (n, 4 consecutive j); group g = (h, p).
template <>
struct Codec<E_Q6_K> {
  // CHUNK_DIV: the 8 parts that cover a 64-element K chunk starting koff elements into the block are
  // parts (koff / CHUNK_DIV) * 8 .. + 7 (a Q6_K part spans a 128-element half)
  static constexpr int BLOCK = 256, BYTES = 210, PARTS = 16, G = 4, CHUNK_DIV = 128;
  __device__ static __forceinline__ int xoff(int part, int g) {
    return (part >> 3) * 128 + (g >> 1) * 64 + (g & 1) * 32 + 4 * (part & 7);
  }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;
    const int n = part >> 3, j4 = part & 7;
    const float d = f16_bits_to_f32(ld_u16(b + 208));
    const uint32_t ql0 = ld_u32_a2(b + n * 64 + 4 * j4);
    const uint32_t ql1 = ld_u32_a2(b + n * 64 + 32 + 4 * j4);
    const uint32_t qh = ld_u32_a2(b + 128 + n * 32 + 4 * j4);
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + n * 8 + (j4 >> 2);
#pragma unroll
    for (int g = 0; g < 4; g++) {
      const int h = g >> 1, p = g & 1;
      const uint32_t ql = p ? ql1 : ql0;
      const float s = (float)sc[h * 4 + p * 2];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int lo = (int)((ql >> (8 * i + 4 * h)) & 15u);
        const int hi = (int)((qh >> (8 * i + 2 * (h * 2 + p))) & 3u);
        w[4 * g + i] = __fmul_rn(__fmul_rn((float)(lo + 16 * hi - 32), s), d);
      }
    }
  }
};

// Q4_K / Q5_K (the K-quants real Q4_K_M / UD-Q4_K_XL files mix in; schema-only in the reference,
// crates/dyninfer-checkpoint-gguf/src/types.rs:21-22,137-201, so the arithmetic follows GGML's
// published dequantisation as the `gguf` Python package evaluates it in f32):
//   f16 d @0, f16 dmin @2, 12 bytes of 6-bit scales / mins @4 for 8 sub-blocks of 32,
//   Q4_K: 128 nibble bytes @16; Q5_K: 32 high-bit bytes @16, 128 nibble bytes @48.
//   element 64*jj + 32*h + l (jj < 4, h < 2, l < 32): sub-block j = 2*jj + h, nibble h of byte
//   32*jj + l (Q5_K: plus 16 * bit j of high byte l);
//   sc_j, m_j: j < 4: s[j] & 63, s[j+4] & 63; j >= 4: (s[j+4] & 15) | ((s[j-4] >> 6) << 4),
//   (s[j+4] >> 4) | ((s[j] >> 6) << 4);  w = (f32(d) * sc_j) * q - (f32(dmin) * m_j), each
//   product and the difference rounded on its own.
// A part is (jj, 4 consecutive l); group g = h.
__device__ __forceinline__ void kquant_scale_min(const uint8_t* s, int j, float* sc, float* mn) {
  uint32_t a, b;
  if (j < 4) {
    a = s[j] & 63u;
    b = s[j + 4] & 63u;
  } else {
    a = (s[j + 4] & 15u) | ((uint32_t)(s[j - 4] >> 6) << 4);
    b = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
  }
  *sc = (float)a;
  *mn = (float)b;
}
template <int ENC>
struct KQuant45 {
  static constexpr bool Q5 = ENC == E_Q5_K;
  static constexpr int BLOCK = 256, BYTES = Q5 ? 176 : 144, PARTS = 32, G = 2, CHUNK_DIV = 64;
  __device__ static __forceinline__ int xoff(int part, int g) { return (part >> 3) * 64 + g * 32 + 4 * (part & 7); }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;  // 144 and 176 are multiples of 16: blocks stay word aligned
    const int jj = part >> 3, l4 = part & 7;
    const float d = f16_bits_to_f32(ld_u16(b)), dmin = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t ql = *reinterpret_cast<const uint32_t*>(b + (Q5 ? 48 : 16) + 32 * jj + 4 * l4);
    uint32_t qh = 0;
    if (Q5) qh = *reinterpret_cast<const uint32_t*>(b + 16 + 4 * l4);
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int j = 2 * jj + h;
      float sc, mn;
      kquant_scale_min(b + 4, j, &sc, &mn);
      const float ds = __fmul_rn(d, sc), dm = __fmul_rn(dmin, mn);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        uint32_t q = (ql >> (8 * i + 4 * h)) & 15u;
        if (Q5) q |= ((qh >> (8 * i + j)) & 1u) << 4;
        w[4 * h + i] = __fsub_rn(__fmul_rn(ds, (float)q), dm);
      }
    }
  }
};
template <>
struct Codec<E_Q4_K> : KQuant45<E_Q4_K> {};
template <>
struct Codec<E_Q5_K> : KQuant45<E_Q5_K> {};

// IQ4_XS (a non-linear 4-bit K-quant of UD-Q4_K_XL files; schema-only in the reference,
// crates/dyninfer-checkpoint-gguf/src/types.rs, so the arithmetic follows GGML's published
// dequantisation as the `gguf` Python package evaluates it in f32): 256 weights in 136 bytes:
//   f16 d @0, u16 scales_h @2, 4 bytes scales_l @4, 128 index bytes @8.
//   sub-block ib (32 weights, ib < 8): 6-bit scale ls = nibble (ib & 1) of scales_l[ib / 2] | bits
//   [2 ib, 2 ib + 2) of scales_h << 4; weight 32 ib + j (j < 16) = low nibble of byte 16 ib + j,
//   weight 32 ib + 16 + j its high nibble; w = (f32(d) * f32(ls - 32)) * f32(table[index]), each
//   product rounded on its own.
// A part is (ib, 4 consecutive j); group g = nibble.
__device__ __forceinline__ float iq4_value(uint32_t idx) {
  // -127 -104 -83 -65 -49 -35 -22 -10 | 1 13 25 38 53 69 89 113 as two's-complement bytes
  const uint64_t lo = 0xF6EADDCFBFAD9881ull, hi = 0x7159453526190D01ull;
  return (float)(int)(int8_t)(((idx & 8u) ? hi : lo) >> (8u * (idx & 7u)));
}
template <>
struct Codec<E_IQ4_XS> {
  static constexpr int BLOCK = 256, BYTES = 136, PARTS = 32, G = 2, CHUNK_DIV = 64;
  __device__ static __forceinline__ int xoff(int part, int g) { return (part >> 2) * 32 + g * 16 + 4 * (part & 3); }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int part, float* w) {
    const uint8_t* b = r.data + blk * BYTES;  // 136 is a multiple of 8: blocks stay word aligned
    const int ib = part >> 2, j4 = part & 3;
    const uint32_t head = *reinterpret_cast<const uint32_t*>(b);       // d | scales_h << 16
    const uint32_t sl = *reinterpret_cast<const uint32_t*>(b + 4);
    const uint32_t q = *reinterpret_cast<const uint32_t*>(b + 8 + 16 * ib + 4 * j4);
    const uint32_t ls = ((sl >> (4 * ib)) & 15u) | ((((head >> 16) >> (2 * ib)) & 3u) << 4);
    const float dl = __fmul_rn(f16_bits_to_f32(head & 0xffffu), (float)((int)ls - 32));
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t byte = (q >> (8 * i)) & 0xffu;
      w[i] = __fmul_rn(dl, iq4_value(byte & 15u));
      w[4 + i] = __fmul_rn(dl, iq4_value(byte >> 4));
    }
  }
};

// MLX affine U4: ui32[N, K/8], lane k of a word = bits [4k, 4k+4); per group:
// w = f32(q)*scale + bias. mlx_affine.rs:284-290,590-600. One word is one "block".
template <>
struct Codec<E_MLX_U4> {
  static constexpr int BLOCK = 8, BYTES = 4, PARTS = 1, G = 2, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int, int g) { return 4 * g; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int, float* w) {
    const uint32_t q = reinterpret_cast<const uint32_t*>(r.data)[blk];
    const int64_t gi = (blk * 8) / r.group;
    const float s = aux_load(r.sc, r.aux, gi);
    const float bb = aux_load(r.bi, r.aux, gi);
#pragma unroll
    for (int i = 0; i < 8; i++)
      w[i] = __fadd_rn(__fmul_rn((float)((q >> (4 * i)) & 15u), s), bb);
  }
};

// Plain element types: exact widening (arith.extf,
// crates/dyninfer-compiler/src/lowering/kernels.rs:1157-1173). Block = 4 elements.
template <>
struct Codec<E_F32> {
  static constexpr int BLOCK = 4, BYTES = 16, PARTS = 1, G = 1, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int, int) { return 0; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int, float* w) {
    const float4 v = reinterpret_cast<const float4*>(r.data)[blk];
    w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
  }
};
template <>
struct Codec<E_F16> {
  static constexpr int BLOCK = 4, BYTES = 8, PARTS = 1, G = 1, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int, int) { return 0; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int, float* w) {
    const uint2 v = reinterpret_cast<const uint2*>(r.data)[blk];
    w[0] = f16_bits_to_f32(v.x & 0xffffu), w[1] = f16_bits_to_f32(v.x >> 16);
    w[2] = f16_bits_to_f32(v.y & 0xffffu), w[3] = f16_bits_to_f32(v.y >> 16);
  }
};
template <>
struct Codec<E_BF16> {
  static constexpr int BLOCK = 4, BYTES = 8, PARTS = 1, G = 1, CHUNK_DIV = 1;
  __device__ static __forceinline__ int xoff(int, int) { return 0; }
  __device__ static __forceinline__ void decode(const RowPtr& r, int64_t blk, int, float* w) {
    const uint2 v = reinterpret_cast<const uint2*>(r.data)[blk];
    w[0] = bf16_bits_to_f32(v.x & 0xffffu), w[1] = bf16_bits_to_f32(v.x >> 16);
    w[2] = bf16_bits_to_f32(v.y & 0xffffu), w[3] = bf16_bits_to_f32(v.y >> 16);
  }
};

// Dispatch a functor templated on the encoding.
#define DYN_ENC_SWITCH(enc, ...)                        \
  switch (enc) {                                        \
    case E_F32: { constexpr int ENC = E_F32; __VA_ARGS__; } break;       \
    case E_F16: { constexpr int ENC = E_F16; __VA_ARGS__; } break;       \
    case E_BF16: { constexpr int ENC = E_BF16; __VA_ARGS__; } break;     \
    case E_Q4_0: { constexpr int ENC = E_Q4_0; __VA_ARGS__; } break;     \
    case E_Q4_1: { constexpr int ENC = E_Q4_1; __VA_ARGS__; } break;     \
    case E_Q8_0: { constexpr int ENC = E_Q8_0; __VA_ARGS__; } break;     \
    case E_Q6_K: { constexpr int ENC = E_Q6_K; __VA_ARGS__; } break;     \
    case E_MLX_U4: { constexpr int ENC = E_MLX_U4; __VA_ARGS__; } break; \
    case E_Q4_K: { constexpr int ENC = E_Q4_K; __VA_ARGS__; } break;     \
    case E_Q5_K: { constexpr int ENC = E_Q5_K; __VA_ARGS__; } break;     \
    case E_IQ4_XS: { constexpr int ENC = E_IQ4_XS; __VA_ARGS__; } break; \
    default:                                            \
      dyn::set_error("unknown encoding %d", (int)(enc)); \
      return 1;                                         \
  }

}  // namespace dyn
