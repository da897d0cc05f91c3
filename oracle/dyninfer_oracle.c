/*
 * CPU restatement of dyninfer's direct quantized decoder path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the parity checker and the timed CPU
 * baseline; no product code path may call it. The reference executes this
 * math as MLIR compiled by IREE (a third-party engine that is not vendored
 * with it, pinned at IREE 3.11.0), so it cannot be run beside this file; the
 * functions below restate the reference's emitters one by one, each citing the
 * reference file:line it follows.
 *
 * Pin status:
 *   - dequantisation of Q4_0 / Q4_1 / Q8_0 / Q6_K / Q4_K / Q5_K / IQ4_XS: pinned, bit for bit,
 *     against the third-party `gguf` Python package and against the
 *     reference's own fixture packers restated in tests/fixtures_ref.py
 *     (crates/dyninfer-checkpoint-gguf/src/q4.rs:16-128).
 *   - MLX affine U4: pinned against the reference's quantize/round-trip
 *     formulas (crates/dyninfer-checkpoint-safetensors/src/fixture.rs:287-317,
 *     crates/dyninfer-runtime/src/reference.rs:177-193).
 *   - whole-model forward: pinned only against a restatement of the
 *     reference's tiny test forward (crates/dyninfer-runtime/src/reference.rs
 *     :195-304) on the reference's generator fixtures; no stored logits exist
 *     in the reference, so forward parity is otherwise UNPINNED.
 *
 * All arithmetic is f32 with separate multiply and add (build with
 * -ffp-contract=off) exactly as the reference's arith.mulf / arith.addf ops.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

enum {
  ORC_F32 = 0,
  ORC_F16 = 1,
  ORC_BF16 = 2,
  ORC_Q4_0 = 3,
  ORC_Q4_1 = 4,
  ORC_Q8_0 = 5,
  ORC_Q6_K = 6,
  ORC_MLX_U4 = 7,
  ORC_Q4_K = 8,
  ORC_Q5_K = 9,
  ORC_IQ4_XS = 10
};

typedef struct {
  int32_t enc;      /* ORC_* */
  int32_t aux_enc;  /* element type of scales/biases for ORC_MLX_U4 */
  int32_t group;    /* MLX group size (64) */
  int32_t pad_;
  int64_t rows;     /* N: output features; weights are [N, K] row-major */
  int64_t cols;     /* K: input features */
  const uint8_t* data;
  const uint8_t* scales; /* MLX only: [N, K/group] */
  const uint8_t* biases; /* MLX only */
} orc_tensor;

/* ---- exact widening conversions (arith.extf) ---------------------------- */

static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

static inline float aux_to_f32(const uint8_t* base, int enc, int64_t idx) {
  if (enc == ORC_F32) {
    float f;
    memcpy(&f, base + idx * 4, 4);
    return f;
  }
  if (enc == ORC_F16) return f16_to_f32(rd16(base + idx * 2));
  return bf16_to_f32(rd16(base + idx * 2));
}

/* round-to-nearest-even narrowing, used only by the optional KV rounding knob */
static inline float round_bf16(float f) {
  uint32_t b;
  memcpy(&b, &f, 4);
  if ((b & 0x7f800000u) == 0x7f800000u) return f;
  b += 0x7fffu + ((b >> 16) & 1u);
  b &= 0xffff0000u;
  memcpy(&f, &b, 4);
  return f;
}
static inline float round_f16(float f) { return (float)(_Float16)f; }

ORC_API float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
ORC_API float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* ---- block geometry (crates/dyninfer-checkpoint-gguf/src/types.rs:137-201) */

ORC_API int64_t orc_block_elems(int enc) {
  switch (enc) {
    case ORC_Q4_0:
    case ORC_Q4_1:
    case ORC_Q8_0:
      return 32;
    case ORC_Q6_K:
    case ORC_Q4_K:
    case ORC_Q5_K:
    case ORC_IQ4_XS:
      return 256;
    case ORC_MLX_U4:
      return 8;
    default:
      return 1;
  }
}
ORC_API int64_t orc_block_bytes(int enc) {
  switch (enc) {
    case ORC_F32:
      return 4;
    case ORC_F16:
    case ORC_BF16:
      return 2;
    case ORC_Q4_0:
      return 18;
    case ORC_Q4_1:
      return 20;
    case ORC_Q8_0:
      return 34;
    case ORC_Q6_K:
      return 210;
    case ORC_Q4_K:
      return 144;
    case ORC_Q5_K:
      return 176;
    case ORC_IQ4_XS:
      return 136;
    case ORC_MLX_U4:
      return 4;
    default:
      return 0;
  }
}
ORC_API int64_t orc_row_bytes(int enc, int64_t cols) {
  return cols / orc_block_elems(enc) * orc_block_bytes(enc);
}

/* ---- dequantisation ----------------------------------------------------- */

/* Q4_0: f16 d at byte 0, 16 quant bytes at 2; byte l low nibble is element l,
 * high nibble element l+16; w = f32(q-8) * f32(d).
 * crates/dyninfer-quantization/src/quantizations/gguf_codegen.rs:412-472 (zero
 * point 8 at :470, lane map at :452). */
static void dq_q4_0(const uint8_t* blk, float* out) {
  float d = f16_to_f32(rd16(blk));
  const uint8_t* qs = blk + 2;
  for (int l = 0; l < 16; l++) {
    out[l] = (float)((int)(qs[l] & 0x0f) - 8) * d;
    out[l + 16] = (float)((int)(qs[l] >> 4) - 8) * d;
  }
}

/* Q4_1: f16 d at 0, f16 m at 2, 16 quant bytes at 4; w = f32(q)*d + m, with
 * the multiply and the add rounded separately. gguf_codegen.rs:373-375,
 * 425-445,464-465. */
static void dq_q4_1(const uint8_t* blk, float* out) {
  float d = f16_to_f32(rd16(blk));
  float m = f16_to_f32(rd16(blk + 2));
  const uint8_t* qs = blk + 4;
  for (int l = 0; l < 16; l++) {
    float lo = (float)(qs[l] & 0x0f) * d;
    float hi = (float)(qs[l] >> 4) * d;
    out[l] = lo + m;
    out[l + 16] = hi + m;
  }
}

/* Q8_0: f16 d at 0, 32 int8 at 2; w = f32(q) * d. gguf_codegen.rs:382-410. */
static void dq_q8_0(const uint8_t* blk, float* out) {
  float d = f16_to_f32(rd16(blk));
  const int8_t* qs = (const int8_t*)(blk + 2);
  for (int l = 0; l < 32; l++) out[l] = (float)qs[l] * d;
}

/* Q6_K: ql 128 B at 0, qh 64 B at 128, 16 int8 scales at 192, f16 d at 208.
 * Element e = n*128 + h*64 + p*32 + j: ql byte n*64+p*32+j nibble h; qh byte
 * n*32+j two-bit field h*2+p; scale index n*8+h*4+p*2+j/16;
 * w = (f32(q-32) * f32(sc)) * f32(d). gguf_codegen.rs:474-526 (maps :499-503,
 * order :519-520). */
static void dq_q6_k(const uint8_t* blk, float* out) {
  const uint8_t* ql = blk;
  const uint8_t* qh = blk + 128;
  const int8_t* sc = (const int8_t*)(blk + 192);
  float d = f16_to_f32(rd16(blk + 208));
  for (int n = 0; n < 2; n++)
    for (int h = 0; h < 2; h++)
      for (int p = 0; p < 2; p++)
        for (int j = 0; j < 32; j++) {
          int lo = (ql[n * 64 + p * 32 + j] >> (4 * h)) & 0x0f;
          int hi = (qh[n * 32 + j] >> (2 * (h * 2 + p))) & 0x03;
          int q = lo + 16 * hi - 32;
          float s = (float)sc[n * 8 + h * 4 + p * 2 + (j >> 4)];
          float local = (float)q * s;
          out[n * 128 + h * 64 + p * 32 + j] = local * d;
        }
}

/* Q4_K / Q5_K: schema-only in the reference
 * (crates/dyninfer-checkpoint-gguf/src/types.rs:21-22,137-201), so this restates GGML's published
 * dequantisation as the third-party `gguf` package (0.19) evaluates it, in f32:
 * f16 d at 0, f16 dmin at 2, 12 bytes of 6-bit scales/mins at 4 (8 sub-blocks of 32); Q4_K: 128
 * nibble bytes at 16; Q5_K: 32 high-bit bytes at 16 and 128 nibble bytes at 48. Element
 * 64*jj + 32*h + l uses sub-block j = 2*jj + h, nibble h of byte 32*jj + l (Q5_K: + 16 * bit j of high
 * byte l); w = (d * sc_j) * q - (dmin * m_j), each product and the difference rounded on its own.
 * Pinned by tests/golden/dequant_golden.npz. */
static void kq_scale_min(const uint8_t* s, int j, float* sc, float* mn) {
  unsigned a, b;
  if (j < 4) {
    a = s[j] & 63u;
    b = s[j + 4] & 63u;
  } else {
    a = (s[j + 4] & 15u) | ((unsigned)(s[j - 4] >> 6) << 4);
    b = (unsigned)(s[j + 4] >> 4) | ((unsigned)(s[j] >> 6) << 4);
  }
  *sc = (float)a;
  *mn = (float)b;
}
static void dq_q45_k(const uint8_t* blk, float* out, int five) {
  const float d = f16_to_f32(rd16(blk)), dmin = f16_to_f32(rd16(blk + 2));
  const uint8_t* qh = blk + 16;
  const uint8_t* qs = blk + (five ? 48 : 16);
  for (int j = 0; j < 8; j++) {
    float sc, mn;
    kq_scale_min(blk + 4, j, &sc, &mn);
    const float ds = d * sc;
    const float dm = dmin * mn;
    const int jj = j >> 1, h = j & 1;
    for (int l = 0; l < 32; l++) {
      unsigned q = (qs[32 * jj + l] >> (4 * h)) & 15u;
      if (five) q |= ((unsigned)(qh[l] >> j) & 1u) << 4;
      const float scaled = ds * (float)q;
      out[64 * jj + 32 * h + l] = scaled - dm;
    }
  }
}

/* IQ4_XS: schema-only in the reference (crates/dyninfer-checkpoint-gguf/src/types.rs), so this restates
 * GGML's published dequantisation as the third-party `gguf` package evaluates it, in f32: f16 d at 0,
 * u16 scales_h at 2, 4 bytes scales_l at 4, 128 index bytes at 8. Sub-block ib (32 weights): 6-bit scale
 * ls = nibble (ib & 1) of scales_l[ib / 2] | bits [2 ib, 2 ib + 2) of scales_h << 4; weight 32 ib + j
 * (j < 16) takes the low nibble of byte 16 ib + j, weight 32 ib + 16 + j its high nibble, as an index
 * into the 16-entry table below; w = (d * (ls - 32)) * table[index], each product rounded on its own.
 * Pinned by tests/golden/dequant_golden.npz. */
static const int8_t iq4_table[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static void dq_iq4_xs(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const unsigned sh = rd16(blk + 2);
  const uint8_t* sl = blk + 4;
  const uint8_t* qs = blk + 8;
  for (int ib = 0; ib < 8; ib++) {
    const int ls = (int)(((sl[ib >> 1] >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
    const float dl = d * (float)(ls - 32);
    for (int j = 0; j < 16; j++) {
      out[32 * ib + j] = dl * (float)iq4_table[qs[16 * ib + j] & 15u];
      out[32 * ib + 16 + j] = dl * (float)iq4_table[qs[16 * ib + j] >> 4];
    }
  }
}

ORC_API void orc_dequant_row(const orc_tensor* t, int64_t row, float* out) {
  const int64_t K = t->cols;
  switch (t->enc) {
    case ORC_F32:
      memcpy(out, t->data + row * K * 4, (size_t)K * 4);
      break;
    case ORC_F16:
      for (int64_t k = 0; k < K; k++) out[k] = f16_to_f32(rd16(t->data + (row * K + k) * 2));
      break;
    case ORC_BF16:
      for (int64_t k = 0; k < K; k++) out[k] = bf16_to_f32(rd16(t->data + (row * K + k) * 2));
      break;
    case ORC_Q4_0: {
      const uint8_t* p = t->data + row * (K / 32) * 18;
      for (int64_t b = 0; b < K / 32; b++) dq_q4_0(p + b * 18, out + b * 32);
    } break;
    case ORC_Q4_1: {
      const uint8_t* p = t->data + row * (K / 32) * 20;
      for (int64_t b = 0; b < K / 32; b++) dq_q4_1(p + b * 20, out + b * 32);
    } break;
    case ORC_Q8_0: {
      const uint8_t* p = t->data + row * (K / 32) * 34;
      for (int64_t b = 0; b < K / 32; b++) dq_q8_0(p + b * 34, out + b * 32);
    } break;
    case ORC_Q6_K: {
      const uint8_t* p = t->data + row * (K / 256) * 210;
      for (int64_t b = 0; b < K / 256; b++) dq_q6_k(p + b * 210, out + b * 256);
    } break;
    case ORC_Q4_K: {
      const uint8_t* p = t->data + row * (K / 256) * 144;
      for (int64_t b = 0; b < K / 256; b++) dq_q45_k(p + b * 144, out + b * 256, 0);
    } break;
    case ORC_Q5_K: {
      const uint8_t* p = t->data + row * (K / 256) * 176;
      for (int64_t b = 0; b < K / 256; b++) dq_q45_k(p + b * 176, out + b * 256, 1);
    } break;
    case ORC_IQ4_XS: {
      const uint8_t* p = t->data + row * (K / 256) * 136;
      for (int64_t b = 0; b < K / 256; b++) dq_iq4_xs(p + b * 136, out + b * 256);
    } break;
    case ORC_MLX_U4: {
      /* packed ui32[N, K/8], lane k of a word is bits [4k, 4k+4); per group of
       * `group` inputs: w = f32(q) * scale + bias (mulf then addf).
       * crates/dyninfer-quantization/src/quantizations/mlx_affine.rs:284-290,
       * 517-537,590-600. */
      const int g = t->group;
      const uint8_t* p = t->data + row * (K / 8) * 4;
      for (int64_t k = 0; k < K; k++) {
        uint32_t word;
        memcpy(&word, p + (k / 8) * 4, 4);
        uint32_t q = (word >> (4 * (k % 8))) & 0x0fu;
        int64_t gi = row * (K / g) + k / g;
        float s = aux_to_f32(t->scales, t->aux_enc, gi);
        float b = aux_to_f32(t->biases, t->aux_enc, gi);
        float scaled = (float)q * s;
        out[k] = scaled + b;
      }
    } break;
    default:
      break;
  }
}

ORC_API void orc_dequant(const orc_tensor* t, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < t->rows; r++) orc_dequant_row(t, r, out + r * t->cols);
}

/* ---- linear: y[b,o] = sum_k x[b,k] * w[o,k] ------------------------------ */
/* gguf_codegen.rs:268-314 and mlx_affine.rs:601-616 leave the reduction order
 * to the compiler; mode 0 follows crates/dyninfer-runtime/src/reference.rs
 * :229-242 (one accumulator, k ascending). mode 1 keeps 8 interleaved partial
 * sums so the loop vectorises: same products, different association; it is
 * what the timed CPU baseline uses. */
static float dot_seq(const float* x, const float* w, int64_t K) {
  float acc = 0.0f;
  for (int64_t k = 0; k < K; k++) acc += x[k] * w[k];
  return acc;
}
static float dot_fast(const float* x, const float* w, int64_t K) {
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int64_t k = 0;
  for (; k + 8 <= K; k += 8)
    for (int j = 0; j < 8; j++) a[j] += x[k + j] * w[k + j];
  float acc = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
  for (; k < K; k++) acc += x[k] * w[k];
  return acc;
}

ORC_API void orc_linear(const orc_tensor* w, const float* x, int64_t M, float* y, int mode) {
  const int64_t N = w->rows, K = w->cols;
#pragma omp parallel
  {
    float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t o = 0; o < N; o++) {
      orc_dequant_row(w, o, row);
      for (int64_t b = 0; b < M; b++)
        y[b * N + o] = mode ? dot_fast(x + b * K, row, K) : dot_seq(x + b * K, row, K);
    }
    free(row);
  }
}

/* ---- RMSNorm: ms = sum(x*x)/H; inv = 1/sqrt(ms+eps); y = (x*inv)*w -------- */
/* crates/dyninfer-compiler/src/lowering/kernels.rs:774-835 (:817-829) and
 * reference.rs:254-258. Also used per head over head_dim (kernels.rs:837-903),
 * where the weight [d] is shared by all heads. */
ORC_API void orc_rms_norm(const float* x, const float* w, int64_t rows, int64_t H, float eps,
                          float* y) {
  for (int64_t r = 0; r < rows; r++) {
    const float* xr = x + r * H;
    float s = 0.0f;
    for (int64_t i = 0; i < H; i++) s += xr[i] * xr[i];
    float ms = s / (float)H;
    float inv = 1.0f / sqrtf(ms + eps);
    for (int64_t i = 0; i < H; i++) y[r * H + i] = (xr[i] * inv) * w[i];
  }
}

/* ---- RoPE, rotate-half: kernels.rs:1007-1070 ------------------------------ */
/* x is [s, heads, d]; pair (i, i+d/2); den = powf(theta, (2*i)/d);
 * freq = 1/den; angle = f32(pos)*freq; lo = x1*c - x2*s; hi = x1*s + x2*c. */
ORC_API void orc_rope(float* x, int64_t s, int64_t heads, int64_t d, int64_t start_pos,
                      float theta) {
  const int64_t half = d / 2;
  for (int64_t p = 0; p < s; p++)
    for (int64_t h = 0; h < heads; h++) {
      float* v = x + (p * heads + h) * d;
      for (int64_t i = 0; i < half; i++) {
        float exponent = (2.0f * (float)i) / (float)d;
        float den = powf(theta, exponent);
        float freq = 1.0f / den;
        float angle = (float)(start_pos + p) * freq;
        float c = cosf(angle), sn = sinf(angle);
        float x1 = v[i], x2 = v[i + half];
        float x1c = x1 * c, x2s = x2 * sn, x1s = x1 * sn, x2c = x2 * c;
        v[i] = x1c - x2s;
        v[i + half] = x1s + x2c;
      }
    }
}

/* ---- SiLU * up: silu(g) = g / (1 + exp(-g)) ------------------------------ */
/* crates/dyninfer-compiler/src/lowering/dense_decoder.rs:1379-1385,
 * reference.rs:260-262. */
ORC_API void orc_silu_mul(const float* gate, const float* up, int64_t n, float* y) {
  for (int64_t i = 0; i < n; i++) {
    float g = gate[i];
    y[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

/* ---- argmax = first strict maximum: dense_decoder.rs:885-893,
 * crates/dyninfer-runtime/src/generate.rs:16-26 -------------------------- */
ORC_API int64_t orc_argmax(const float* v, int64_t n) {
  int64_t best = 0;
  float bv = -INFINITY;
  for (int64_t i = 0; i < n; i++)
    if (v[i] > bv) {
      bv = v[i];
      best = i;
    }
  return best;
}

/* ---- GQA causal attention over a [nkv, kv_cap, d] cache ------------------ */
/* Online-softmax walk over 256-key pages, kernels.rs:310-458, mask
 * kernels.rs:460-506 (0 where k <= start+q and k < start+valid, else
 * -3.40282347e38), page loop dense_decoder.rs:549-560,734-742, final
 * out / row_sum dense_decoder.rs:1317-1328. q is [s, nh, d] with head
 * h = kvh*g + gi (dense_decoder.rs:2454-2456); ctx is [s, nh*d]. */
ORC_API void orc_attention(const float* q, const float* kc, const float* vc, int64_t s,
                           int64_t nh, int64_t nkv, int64_t d, int64_t kv_cap, int64_t start,
                           int64_t valid, int64_t page, float* ctx) {
  const float NEG = -3.40282347e38f;
  const float scale = 1.0f / sqrtf((float)d);
  const int64_t g = nh / nkv;
  const int64_t seq_end = start + valid;
  const int64_t pages = (seq_end + page - 1) / page;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t h = 0; h < nh; h++)
    for (int64_t qi = 0; qi < s; qi++) {
      const int64_t kvh = h / g;
      const float* qv = q + (qi * nh + h) * d;
      float* out = (float*)calloc((size_t)d, sizeof(float));
      float* pout = (float*)malloc((size_t)d * sizeof(float));
      float* wts = (float*)malloc((size_t)page * sizeof(float));
      float row_max = NEG, row_sum = 0.0f;
      for (int64_t pg = 0; pg < pages; pg++) {
        float pmax = NEG;
        for (int64_t k = 0; k < page; k++) {
          int64_t ak = pg * page + k;
          float dot = 0.0f;
          if (ak < kv_cap) {
            const float* kv = kc + (kvh * kv_cap + ak) * d;
            for (int64_t t = 0; t < d; t++) dot += qv[t] * kv[t];
          }
          int visible = (ak <= start + qi) && (ak < seq_end);
          float sc = dot * scale + (visible ? 0.0f : NEG);
          wts[k] = sc;
          if (sc > pmax) pmax = sc;
        }
        float new_max = row_max > pmax ? row_max : pmax;
        float psum = 0.0f;
        for (int64_t k = 0; k < page; k++) {
          wts[k] = expf(wts[k] - new_max);
          psum += wts[k];
        }
        for (int64_t t = 0; t < d; t++) pout[t] = 0.0f;
        for (int64_t k = 0; k < page; k++) {
          int64_t ak = pg * page + k;
          if (ak >= kv_cap || wts[k] == 0.0f) continue; /* adds of +0 products */
          const float* vv = vc + (kvh * kv_cap + ak) * d;
          for (int64_t t = 0; t < d; t++) pout[t] += wts[k] * vv[t];
        }
        float factor = expf(row_max - new_max);
        row_sum = row_sum * factor + psum;
        for (int64_t t = 0; t < d; t++) out[t] = out[t] * factor + pout[t];
        row_max = new_max;
      }
      for (int64_t t = 0; t < d; t++) ctx[qi * nh * d + h * d + t] = out[t] / row_sum;
      free(out);
      free(pout);
      free(wts);
    }
}

/* ---- whole decoder ------------------------------------------------------- */
/* Op order per layer follows crates/dyninfer-architecture/src/builder.rs
 * :491-614,664-718: norm -> q,k,v -> [q-norm,k-norm] -> [rope q,k] -> kv write
 * -> attention -> o -> +res -> norm -> gate,up -> silu*up -> down -> +res.
 * Chunk begin / logits / argmax: dense_decoder.rs:902-970,1573-1615,787-900. */

typedef struct {
  int32_t layers, hidden, heads, kv_heads, head_dim, inter, vocab;
  int32_t has_qk_norm, has_rope;
  int32_t kv_round; /* 0 keep f32, 1 round K/V to f16, 2 to bf16 (mirrors a 2-byte KV cache) */
  int32_t linear_mode;
  int32_t page;
  float eps, theta;
  int64_t kv_cap;
} orc_config;

enum { T_EMBED = 0, T_OUT_NORM = 1, T_LM_HEAD = 2, T_LAYER0 = 3 };
enum {
  L_ATTN_NORM = 0,
  L_Q,
  L_K,
  L_V,
  L_O,
  L_Q_NORM,
  L_K_NORM,
  L_FFN_NORM,
  L_GATE,
  L_UP,
  L_DOWN,
  L_COUNT
};

typedef struct {
  orc_config cfg;
  orc_tensor* t;
  float* kcache; /* [layers][nkv][kv_cap][d] */
  float* vcache;
} orc_model;

ORC_API orc_model* orc_model_create(const orc_config* cfg, const orc_tensor* tensors) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->cfg = *cfg;
  int nt = T_LAYER0 + cfg->layers * L_COUNT;
  m->t = (orc_tensor*)malloc(sizeof(orc_tensor) * (size_t)nt);
  memcpy(m->t, tensors, sizeof(orc_tensor) * (size_t)nt);
  size_t n = (size_t)cfg->layers * cfg->kv_heads * (size_t)cfg->kv_cap * cfg->head_dim;
  m->kcache = (float*)calloc(n, sizeof(float));
  m->vcache = (float*)calloc(n, sizeof(float));
  return m;
}
ORC_API void orc_model_destroy(orc_model* m) {
  if (!m) return;
  free(m->t);
  free(m->kcache);
  free(m->vcache);
  free(m);
}
ORC_API void orc_model_reset(orc_model* m) {
  size_t n = (size_t)m->cfg.layers * m->cfg.kv_heads * (size_t)m->cfg.kv_cap * m->cfg.head_dim;
  memset(m->kcache, 0, n * sizeof(float));
  memset(m->vcache, 0, n * sizeof(float));
}

static const float* f32_weight(const orc_tensor* t) { return (const float*)t->data; }

/* Runs rows [0, n) of one chunk starting at absolute position start_pos, writes
 * K/V, and returns logits (vocab floats) of row `last`. If hidden_out is not
 * NULL it receives the final residual stream [n, hidden]. Returns the argmax. */
ORC_API int64_t orc_model_forward(orc_model* m, const int64_t* tokens, int64_t n,
                                  int64_t start_pos, int64_t last, float* logits,
                                  float* hidden_out) {
  const orc_config* c = &m->cfg;
  const int64_t H = c->hidden, nh = c->heads, nkv = c->kv_heads, d = c->head_dim, I = c->inter;
  const int64_t qd = nh * d, kvd = nkv * d;
  float* hid = (float*)malloc(sizeof(float) * (size_t)(n * H));
  float* xn = (float*)malloc(sizeof(float) * (size_t)(n * H));
  float* q = (float*)malloc(sizeof(float) * (size_t)(n * qd));
  float* k = (float*)malloc(sizeof(float) * (size_t)(n * kvd));
  float* v = (float*)malloc(sizeof(float) * (size_t)(n * kvd));
  float* ctx = (float*)malloc(sizeof(float) * (size_t)(n * qd));
  float* o = (float*)malloc(sizeof(float) * (size_t)(n * H));
  float* gate = (float*)malloc(sizeof(float) * (size_t)(n * I));
  float* up = (float*)malloc(sizeof(float) * (size_t)(n * I));
  float* act = (float*)malloc(sizeof(float) * (size_t)(n * I));

  for (int64_t r = 0; r < n; r++) orc_dequant_row(&m->t[T_EMBED], tokens[r], hid + r * H);

  for (int l = 0; l < c->layers; l++) {
    const orc_tensor* L = m->t + T_LAYER0 + l * L_COUNT;
    orc_rms_norm(hid, f32_weight(&L[L_ATTN_NORM]), n, H, c->eps, xn);
    orc_linear(&L[L_Q], xn, n, q, c->linear_mode);
    orc_linear(&L[L_K], xn, n, k, c->linear_mode);
    orc_linear(&L[L_V], xn, n, v, c->linear_mode);
    if (c->has_qk_norm) {
      /* QK-norm before RoPE: dense_decoder.rs:2431-2452 */
      orc_rms_norm(q, f32_weight(&L[L_Q_NORM]), n * nh, d, c->eps, q);
      orc_rms_norm(k, f32_weight(&L[L_K_NORM]), n * nkv, d, c->eps, k);
    }
    if (c->has_rope) {
      orc_rope(q, n, nh, d, start_pos, c->theta);
      orc_rope(k, n, nkv, d, start_pos, c->theta);
    }
    /* KV write, rows [start, start+n): dense_decoder.rs:1115-1197 */
    float* kc = m->kcache + (size_t)l * nkv * c->kv_cap * d;
    float* vc = m->vcache + (size_t)l * nkv * c->kv_cap * d;
    for (int64_t r = 0; r < n; r++)
      for (int64_t hh = 0; hh < nkv; hh++)
        for (int64_t t = 0; t < d; t++) {
          float kvv = k[(r * nkv + hh) * d + t], vvv = v[(r * nkv + hh) * d + t];
          if (c->kv_round == 1) {
            kvv = round_f16(kvv);
            vvv = round_f16(vvv);
          } else if (c->kv_round == 2) {
            kvv = round_bf16(kvv);
            vvv = round_bf16(vvv);
          }
          kc[(hh * c->kv_cap + start_pos + r) * d + t] = kvv;
          vc[(hh * c->kv_cap + start_pos + r) * d + t] = vvv;
        }
    orc_attention(q, kc, vc, n, nh, nkv, d, c->kv_cap, start_pos, n, c->page, ctx);
    orc_linear(&L[L_O], ctx, n, o, c->linear_mode);
    for (int64_t i = 0; i < n * H; i++) hid[i] = hid[i] + o[i];
    orc_rms_norm(hid, f32_weight(&L[L_FFN_NORM]), n, H, c->eps, xn);
    orc_linear(&L[L_GATE], xn, n, gate, c->linear_mode);
    orc_linear(&L[L_UP], xn, n, up, c->linear_mode);
    orc_silu_mul(gate, up, n * I, act);
    orc_linear(&L[L_DOWN], act, n, o, c->linear_mode);
    for (int64_t i = 0; i < n * H; i++) hid[i] = hid[i] + o[i];
  }
  if (hidden_out) memcpy(hidden_out, hid, sizeof(float) * (size_t)(n * H));
  /* final norm of row `last` only, lm_head with rows=1: dense_decoder.rs:1573-1615 */
  orc_rms_norm(hid + last * H, f32_weight(&m->t[T_OUT_NORM]), 1, H, c->eps, xn);
  orc_linear(&m->t[T_LM_HEAD], xn, 1, logits, c->linear_mode);
  int64_t tok = orc_argmax(logits, c->vocab);
  free(hid);
  free(xn);
  free(q);
  free(k);
  free(v);
  free(ctx);
  free(o);
  free(gate);
  free(up);
  free(act);
  return tok;
}

/* Sets the number of OpenMP threads of later calls (a launcher may have exported OMP_NUM_THREADS=1
 * for its workers; the timed CPU baseline states and uses the cores it was given). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
