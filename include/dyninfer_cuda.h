/*
 * libdyninfer_cuda — C ABI of the B200 (sm_100a) `cuda` target for dyninfer's
 * direct quantized decoder path.
 *
 * The session half of this header is modelled one to one on the reference's
 * native session boundary, third_party/iree_runtime_c_api/wrapper.h:14-122
 * (bound from Rust by crates/iree-runtime-sys/src/lib.rs:53-145). Each entry
 * point names the reference declaration it replaces. The per-operation half
 * (dequant / linear / norm / rope / attention / argmax) has no counterpart in
 * the reference ABI, where single operators are only reachable through a
 * compiled module; it exists so that each kernel can be checked alone.
 *
 * Conventions kept from the reference (wrapper.h:38, wrapper.c:82-109):
 *   - every call returns 0 on success and non-zero on failure;
 *   - after a failure dyninfer_cuda_last_error() returns a human-readable
 *     message; the message is thread-local, so independent sessions may be
 *     driven from different threads;
 *   - a session is thread-compatible, not thread-safe: the caller serialises
 *     calls on one session (the Rust side holds it in a Mutex,
 *     crates/iree-runtime/src/lib.rs:110-121);
 *   - there is no CPU fallback: if no CUDA device is usable the call fails.
 *
 * All `*_dev` pointers are device pointers on the current CUDA device.
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 * stream).
 */
#ifndef DYNINFER_CUDA_H_
#define DYNINFER_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DYNINFER_CUDA_ABI_VERSION 1

/* ---- physical encodings (crates/dyninfer-core/src/types.rs:108-149) ------ */
enum {
  DYNINFER_ENC_F32 = 0,    /* plain.f32  */
  DYNINFER_ENC_F16 = 1,    /* plain.f16  */
  DYNINFER_ENC_BF16 = 2,   /* plain.bf16 */
  DYNINFER_ENC_Q4_0 = 3,   /* gguf.q4_0:  32 el / 18 B */
  DYNINFER_ENC_Q4_1 = 4,   /* gguf.q4_1:  32 el / 20 B */
  DYNINFER_ENC_Q8_0 = 5,   /* gguf.q8_0:  32 el / 34 B */
  DYNINFER_ENC_Q6_K = 6,   /* gguf.q6_k: 256 el / 210 B */
  DYNINFER_ENC_MLX_U4 = 7, /* mlx.affine.u4: u32 words + scales + biases */
  DYNINFER_ENC_Q4_K = 8,   /* gguf.q4_k: 256 el / 144 B */
  DYNINFER_ENC_Q5_K = 9,   /* gguf.q5_k: 256 el / 176 B */
  DYNINFER_ENC_IQ4_XS = 10 /* gguf.iq4_xs: 256 el / 136 B */
};

/* One [rows, cols] parameter as the verbatim checkpoint bytes, resident in
 * device memory. rows = output features N, cols = input features K; storage is
 * row-major [N, K] (crates/dyninfer-quantization/src/quantizations/
 * gguf_codegen.rs:144-149). For MLX `data` is ui32[N, K/8], `scales`/`biases`
 * are [N, K/group] of `aux_type` (F32, F16 or BF16). */
typedef struct dyninfer_cuda_weight_t {
  int32_t encoding;
  int32_t aux_type;
  int32_t group;
  int32_t reserved;
  int64_t rows;
  int64_t cols;
  const void* data;
  const void* scales;
  const void* biases;
} dyninfer_cuda_weight_t;

/* ---- library -------------------------------------------------------------- */

int dyninfer_cuda_abi_version(void);
/* replaces dyninfer_iree_last_error (wrapper.h:63) */
const char* dyninfer_cuda_last_error(void);
/* Number of usable CUDA devices; fails when the driver reports none. */
int dyninfer_cuda_device_count(int* out_count);
/* Bytes per row of an encoded [*, cols] tensor; 0 if cols is not a whole number of blocks. */
uint64_t dyninfer_cuda_row_bytes(int encoding, int64_t cols);

/* The operator entry points below are asynchronous on the caller's stream, so a kernel whose
 * bounded wait (weight ring, GEMM pipeline) gives up cannot fail the call that launched it: it
 * leaves a code in a per-device error word instead. Call this after synchronising the stream:
 * non-zero (message via last_error, word cleared) means results since the last check are
 * invalid. Session calls check it themselves before they return. Error convention as
 * wrapper.h:38; the reference has no asynchronous operator surface, hence no counterpart. */
int dyninfer_cuda_check_device_error(void);

/* ---- single operators (device pointers) ----------------------------------- */

/* Bit-exact dequantisation to f32 [rows, cols]
 * (gguf_codegen.rs:350-526, mlx_affine.rs:590-600). */
int dyninfer_cuda_dequant(const dyninfer_cuda_weight_t* w, float* out_dev, void* stream);

/* out[i, :] = dequant(row tokens[i]) — the embedding lookup
 * (gguf_codegen.rs:316-348, mlx_affine.rs:628-675). */
int dyninfer_cuda_embedding_gather(const dyninfer_cuda_weight_t* w, const int64_t* tokens_dev,
                                   int64_t count, float* out_dev, void* stream);

/* y[m, n] = sum_k x[m, k] * w[n, k], f32 accumulation, fused dequantisation
 * (gguf_codegen.rs:268-314, mlx_affine.rs:557-626). x_type is DYNINFER_ENC_F32
 * or DYNINFER_ENC_BF16; y is f32 [m, rows]. Any m >= 1. */
int dyninfer_cuda_linear(const dyninfer_cuda_weight_t* w, const void* x_dev, int x_type,
                         int64_t m, float* y_dev, void* stream);

/* y = (x * rsqrt(mean(x^2) + eps)) * w over the last dim
 * (crates/dyninfer-compiler/src/lowering/kernels.rs:774-903). w_type gives the
 * element type of the weight vector (F32 / F16 / BF16). In place allowed. */
int dyninfer_cuda_rms_norm(const float* x_dev, const void* w_dev, int w_type, int64_t rows,
                           int64_t width, float eps, float* y_dev, void* stream);

/* Rotate-half RoPE on x [s, heads, d] in place, positions start_pos + row
 * (kernels.rs:1007-1070). */
int dyninfer_cuda_rope(float* x_dev, int64_t s, int64_t heads, int64_t d, int64_t start_pos,
                       float theta, void* stream);

/* y = silu(gate) * up (crates/dyninfer-compiler/src/lowering/dense_decoder.rs:1379-1385). */
int dyninfer_cuda_silu_mul(const float* gate_dev, const float* up_dev, int64_t n, float* y_dev,
                           void* stream);

/* GQA causal attention of q [s, heads, d] against caches [kv_heads, kv_cap, d]
 * holding keys/values for positions < start_pos + s; ctx is f32 [s, heads*d]
 * (kernels.rs:310-506, dense_decoder.rs:1317-1328,2454-2456). kv_type is F32, F16 or BF16. */
int dyninfer_cuda_attention(const float* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                            int kv_type, int64_t s, int64_t heads, int64_t kv_heads, int64_t d,
                            int64_t kv_cap, int64_t start_pos, float* ctx_dev, void* stream);

/* First strict maximum of v[0..n) (dense_decoder.rs:885-893). scratch_dev must hold
 * dyninfer_cuda_argmax_scratch_bytes(n) bytes. */
size_t dyninfer_cuda_argmax_scratch_bytes(int64_t n);
int dyninfer_cuda_argmax(const float* v_dev, int64_t n, int64_t* out_index_dev, void* scratch_dev,
                         void* stream);

/* Argmax that allocates nothing. No counterpart in the reference: it exists for hosts that must
 * not touch the device allocator on this call -- a serving loop that reserved all device memory
 * up front (so an allocation could fail or stall behind other work), or a caller between
 * operations that cannot tolerate the implicit synchronisation an allocation may bring. Same
 * result as dyninfer_cuda_argmax, without a scratch argument: the per-block partial results go
 * to a fixed 16 KiB array inside the library. n must not exceed
 * dyninfer_cuda_argmax_static_max_n() (4,194,304 elements); larger n fails with a message.
 * The first call on each device looks up the array's address (set-up work: make it before
 * starting a stream capture). All calls on a device share the array; each call rewrites the
 * slots it reads, so no clearing is needed between calls, but calls in flight at the same time
 * race on it. */
int64_t dyninfer_cuda_argmax_static_max_n(void);
int dyninfer_cuda_argmax_static(const float* v_dev, int64_t n, int64_t* out_index_dev, void* stream);

/* ---- session (paged-KV ABI) ----------------------------------------------- */

typedef struct dyninfer_cuda_session_t dyninfer_cuda_session_t;

/* replaces dyninfer_iree_parameter_file_t (wrapper.h:18-20) */
typedef struct dyninfer_cuda_parameter_file_t {
  const char* path;
} dyninfer_cuda_parameter_file_t;

/* replaces dyninfer_iree_file_param_t (wrapper.h:24-29): one stable external
 * key "weights::<canonical>::<component>" backed by one contiguous byte range
 * of an original checkpoint file. */
typedef struct dyninfer_cuda_file_param_t {
  const char* key;
  size_t source_file_index;
  uint64_t offset;
  uint64_t length;
} dyninfer_cuda_file_param_t;

/* replaces dyninfer_iree_session_create_with_file_params (wrapper.h:46-50).
 * `device_uri` is "cuda", "cuda:<ordinal>" or NULL (= "cuda:0"). `model_desc_json`
 * stands where the reference passes a compiled module path: it carries the
 * model geometry and, per parameter, encoding and logical shape. Every byte
 * range is read from its file and uploaded unchanged. */
int dyninfer_cuda_session_create_with_file_params(
    const char* device_uri, const char* model_desc_json,
    const dyninfer_cuda_parameter_file_t* files, size_t file_count,
    const dyninfer_cuda_file_param_t* params, size_t param_count,
    dyninfer_cuda_session_t** out_session);

/* replaces dyninfer_iree_session_destroy (wrapper.h:60) */
void dyninfer_cuda_session_destroy(dyninfer_cuda_session_t* session);

/* replaces dyninfer_iree_free (wrapper.h:67): logits are session scratch, so this is a no-op. */
void dyninfer_cuda_free(void* p);

/* replaces dyninfer_iree_session_configure_paged_kv (wrapper.h:90-94).
 * kv_element_byte_count 4 selects an f32 cache, 2 selects the 2-byte type the
 * descriptor names ("kv_dtype": "bf16" default, or "f16"). Fails once pages exist. */
int dyninfer_cuda_session_configure_paged_kv(dyninfer_cuda_session_t* session, size_t layer_count,
                                             size_t page_size, size_t kv_head_count,
                                             size_t head_dim, size_t kv_element_byte_count,
                                             size_t chunk_size, size_t vocab_size);
/* replaces dyninfer_iree_session_ensure_kv_pages (wrapper.h:95-96) */
int dyninfer_cuda_session_ensure_kv_pages(dyninfer_cuda_session_t* session, size_t page_count);

/* replaces dyninfer_iree_session_invoke_paged_chunk (wrapper.h:97-100).
 * token_count must be 1 or chunk_size; 0 <= last < token_count; start_pos >= 0.
 * *out_logits is session-owned scratch valid until the next invoke. With
 * want_logits = 0 the logits pointers may be NULL and only *out_token is produced. */
int dyninfer_cuda_session_invoke_paged_chunk(dyninfer_cuda_session_t* session,
                                             const int64_t* tokens, size_t token_count,
                                             int64_t last, int64_t start_pos, float** out_logits,
                                             size_t* out_count, int64_t* out_token,
                                             int want_logits);
/* replaces dyninfer_iree_session_reset_paged_kv (wrapper.h:101) */
int dyninfer_cuda_session_reset_paged_kv(dyninfer_cuda_session_t* session);
/* replace dyninfer_iree_session_kv_page_count / _kv_allocated_bytes (wrapper.h:102-105) */
size_t dyninfer_cuda_session_kv_page_count(const dyninfer_cuda_session_t* session);
size_t dyninfer_cuda_session_kv_allocated_bytes(const dyninfer_cuda_session_t* session);

/* replaces dyninfer_iree_allocator_statistics_t (wrapper.h:109-116) */
typedef struct dyninfer_cuda_allocator_statistics_t {
  uint64_t host_bytes_peak;
  uint64_t host_bytes_allocated;
  uint64_t host_bytes_freed;
  uint64_t device_bytes_peak;
  uint64_t device_bytes_allocated;
  uint64_t device_bytes_freed;
} dyninfer_cuda_allocator_statistics_t;
/* replaces dyninfer_iree_session_allocator_statistics (wrapper.h:120-122) */
int dyninfer_cuda_session_allocator_statistics(const dyninfer_cuda_session_t* session,
                                               dyninfer_cuda_allocator_statistics_t* out_stats);

/* ---- batching (extension: the reference session is batch 1) ----------------- */

/* invoke_paged_chunk for KV slot `slot` of a session whose descriptor sets "batch" > 1: the same
 * rules as dyninfer_cuda_session_invoke_paged_chunk (which is slot 0). Sequences in different
 * slots are independent; each has its own positions. */
int dyninfer_cuda_session_invoke_paged_chunk_slot(dyninfer_cuda_session_t* session,
                                                  const int64_t* tokens, size_t token_count,
                                                  int64_t last, int64_t start_pos, int64_t slot,
                                                  float** out_logits, size_t* out_count,
                                                  int64_t* out_token, int want_logits);

/* One decode step for `count` sequences at once (count <= "batch"): row i feeds tokens[i] at
 * positions[i] into slot slots[i] (all slots distinct) and out_tokens[i] receives the first strict
 * maximum of its logits. With want_logits != 0, *out_logits points at [count, vocab] floats of
 * session-owned pinned memory, borrowed until the next call. The linears run once for all rows
 * (one pass over the weights), attention runs per sequence. */
int dyninfer_cuda_session_decode_batch(dyninfer_cuda_session_t* session, const int64_t* tokens,
                                       const int64_t* positions, const int64_t* slots, size_t count,
                                       int64_t* out_tokens, float** out_logits, int want_logits);

/* ---- tensor parallelism (extension: one process per GPU, one session per rank) ------------- */

/* A session whose descriptor sets "tp_world" W > 1 and "tp_rank" r is one rank of a tensor-parallel
 * group. Its descriptor carries this rank's share of the geometry ("heads", "kv_heads",
 * "intermediate" divided by W; "lm_head_rows" = vocab / W) and its byte ranges are this rank's
 * slices, uploaded unchanged: consecutive rows of attn_q/k/v, ffn_gate/up and `output.weight`
 * (rows [r * vocab / W, ...) of the lm_head), and, for attn_output / ffn_down, one span of the
 * blocks of every row. Such a span is a strided range: the parameter's descriptor entry names it
 * under "strided": {"<component>": [rows, segment_bytes, row_stride_bytes]}, the file param's
 * `offset` is the first segment and `length` = rows * segment_bytes. Norm vectors and the embedding
 * table are replicated. Each step sums the ranks' partial o_proj and down products (all-reduce,
 * 2 per layer) and gathers the ranks' logits slices; KV cache and attention stay local to the
 * rank's heads. Every rank must make the same calls in the same order.
 *
 * One rank obtains an id (dyninfer_cuda_tp_unique_id), the host program hands the same bytes to
 * all ranks (any channel), and every rank calls dyninfer_cuda_session_tp_init before its first
 * invoke. NCCL is looked up at run time; without it these calls fail with a message. */
size_t dyninfer_cuda_tp_unique_id_bytes(void);
int dyninfer_cuda_tp_unique_id(uint8_t* out_id, size_t byte_count);
int dyninfer_cuda_session_tp_init(dyninfer_cuda_session_t* session, const uint8_t* id, size_t byte_count);

/* Optional: sum the partial products over peer memory (NVLink / NVSwitch loads) instead of the
 * all-reduce. After configure_paged_kv every rank calls _tp_peer_handle (allocates its exchange
 * region and returns an inter-process handle to it), the host program collects the handles of all
 * ranks in rank order and gives the concatenation to _tp_peer_attach on every rank. From then on
 * each o_proj / down product writes this rank's partial rows into its region and ONE kernel per
 * product signals the peers, waits for them (bounded; a rank that does not arrive makes the call
 * fail with a message), adds all ranks' rows in rank order to the residual and applies the RMSNorm
 * that feeds the next product. The logits slices are still gathered through the communicator. */
size_t dyninfer_cuda_tp_peer_handle_bytes(void);
int dyninfer_cuda_session_tp_peer_handle(dyninfer_cuda_session_t* session, uint8_t* out_handle,
                                         size_t byte_count);
int dyninfer_cuda_session_tp_peer_attach(dyninfer_cuda_session_t* session, const uint8_t* handles,
                                         size_t byte_count);
/* Diagnostic for the bounded wait of that kernel, on ONE device and without a peer: runs a
 * two-rank exchange ([rows, hidden], rows <= 64) whose second region is a local allocation
 * whose arrival flag is never raised, with the wait limited to `spin_limit` polls (~0.25 us each,
 * <= 10,000,000). The expected outcome is a non-zero return with the session's "did not
 * arrive" message and a device that still answers; 0 means the wait did not expire. No
 * counterpart in the reference (it has no multi-device path). */
int dyninfer_cuda_tp_exchange_wait_probe(int hidden, int64_t rows, int64_t spin_limit);

/* ---- session extensions (no reference precedent) --------------------------- */

/* Total bytes of uploaded parameters (the reference's schema total_bytes used by
 * eff_weight_bw_gbs, crates/dyninfer-runtime/src/perf.rs:298-305). */
uint64_t dyninfer_cuda_session_weight_bytes(const dyninfer_cuda_session_t* session);
/* Bytes of parameters one decode step reads (embedding counted as one row unless tied). */
uint64_t dyninfer_cuda_session_decode_weight_bytes(const dyninfer_cuda_session_t* session);

/* Device-resident greedy loop: feeds each argmax back as the next token without a
 * host round trip; `steps` decode steps starting from `first_token` at `start_pos`.
 * out_tokens (host, `steps` entries) may be NULL. *out_device_ms receives the
 * CUDA-event time of the loop on the session stream. */
int dyninfer_cuda_session_decode_loop(dyninfer_cuda_session_t* session, int64_t first_token,
                                      int64_t start_pos, size_t steps, int64_t* out_tokens,
                                      float* out_device_ms);

/* 1 when single-row steps of this session run as the persistent decode kernel (one launch per
 * token), 0 when they run as a captured graph of per-operator kernels. Decided by
 * configure_paged_kv (encodings, head dim and whether the per-CTA program fits shared memory). */
int dyninfer_cuda_session_uses_persistent_kernel(const dyninfer_cuda_session_t* session);

/* Time CTA 0 of the persistent decode kernel spent per phase kind during its most recent
 * launch, microseconds (device global timer): [0] embedding, [1] norm+QKV, [2] attention,
 * [3] o_proj, [4] gate/up, [5] down, [6] lm_head, [7] argmax, [8] whole kernel. Each phase
 * includes the grid barrier that ends it. Fails when the session uses the graph path. */
int dyninfer_cuda_session_decode_phase_profile(dyninfer_cuda_session_t* session, double* out_us,
                                               size_t count);

/* Event trace of the most recent persistent-kernel launch, recorded when the session was
 * configured with DYNINFER_CUDA_TRACE=1 in the environment: [CTAs][layers + 1][16] device
 * global-timer stamps (ns) taken by thread 0 of every CTA. Per layer: 0 QKV input staged, 1 its
 * tile steps done, 2 its outputs stored; 3 attention has q/k/v, 4 attention stored; 5-7 o_proj,
 * 8-10 gate/up, 11-13 down likewise; row `layers`: 0-2 = lm_head. *out_needed receives the number
 * of entries (0 when tracing is off); nothing is copied unless `count` covers it. */
int dyninfer_cuda_session_decode_trace(dyninfer_cuda_session_t* session, uint64_t* out, size_t count,
                                       size_t* out_needed);

/* Device-side stopwatch on the session's stream (CUDA events): stop = 0 records the start after
 * the work queued so far; stop = 1 records the end, waits for it and writes the milliseconds the
 * stream spent between the two to *out_ms. What the bench and the tensor-parallel runner time
 * multi-call regions with (no reference counterpart: the reference times on the host). */
int dyninfer_cuda_session_timer(dyninfer_cuda_session_t* session, int stop, float* out_ms);

/* Number of kernels this library has launched on behalf of `session` since creation. */
uint64_t dyninfer_cuda_session_launch_count(const dyninfer_cuda_session_t* session);

#ifdef __cplusplus
}
#endif

#endif /* DYNINFER_CUDA_H_ */
