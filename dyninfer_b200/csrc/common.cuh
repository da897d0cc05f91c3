// Shared declarations for libdyninfer_cuda (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dyninfer_cuda.h"

namespace dyn {

// ---- error channel: int rc + thread-local message ---------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define DYN_CUDA(expr)                                                      \
  do {                                                                      \
    cudaError_t _e = (expr);                                                \
    if (_e != cudaSuccess) return dyn::cuda_fail(_e, #expr, __FILE__, __LINE__); \
  } while (0)

#define DYN_CHECK(cond, ...)       \
  do {                             \
    if (!(cond)) {                 \
      dyn::set_error(__VA_ARGS__); \
      return 1;                    \
    }                              \
  } while (0)

int keep_scratch_pool_cached();  // raise the default memory pool's release threshold (idempotent)
// A caller-owned scratch region for the products launched by this thread (a session sets its own
// for the duration of a call): products whose scratch fits use it instead of the stream-ordered
// allocator, so consecutive kernels of a captured graph are not separated by allocation nodes.
void set_thread_scratch(void* ptr, size_t bytes);
void* thread_scratch(size_t bytes);  // the region when it holds `bytes`, else nullptr
// Keep the first `bytes` of the region out of the next products' reach (a product's K-slice sums wait
// there for the kernel that adds them); release_all gives the whole region back.
void thread_scratch_hold(size_t bytes);
void thread_scratch_release_all();

// The K-slice sums of a single-row product whose final addition is left to the caller's next kernel
// (QKV prepare, SwiGLU), which saves the reduction launch: y[i] = scale[0] * sum_j partial[j][i],
// j in ascending order, exactly what the product's own reduction kernel computes. S == 0: the product
// wrote y itself (another kernel took it, or K was not split).
struct Deferred {
  const float* partial = nullptr;  // [S][N]
  const float* scale = nullptr;    // device word
  int S = 0;
  int64_t N = 0;
  size_t ws_bytes = 0;             // scratch the product occupies (hold it until the sums are consumed)
};
// While a DeferScope lives, the first column-split product launched on this thread with K split fills
// `d` instead of launching its reduction.
void defer_request(Deferred* d);
Deferred* defer_take();
struct DeferScope {
  explicit DeferScope(Deferred* d) { *d = Deferred(); defer_request(d); }
  ~DeferScope() { defer_request(nullptr); }
};
// A column range of deferred sums (or nothing: S == 0)
struct DeferredCols {
  const float* partial = nullptr;
  const float* scale = nullptr;  // nullptr: the sums are already scaled (the dequant GEMM's)
  int S = 0;
  int64_t N = 0, col = 0;
  int64_t rows = 1;  // rows per slice: slice j of row r starts at partial + (j * rows + r) * N
};
inline DeferredCols deferred_cols(const Deferred& d, int64_t col) {
  DeferredCols c;
  c.partial = d.partial, c.scale = d.scale, c.S = d.S, c.N = d.N, c.col = col;
  return c;
}

// Programmatic dependent launch (sm_90+). A kernel launched with launch_pdl may start while the
// kernel before it in the stream is still running; it must not touch anything that kernel (or an
// earlier one) produces, nor write global memory, before pdl_wait(). pdl_trigger() lets the next
// kernel of the stream start early; kernels that never call it release it when they exit.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled();  // DYNINFER_CUDA_PDL=0 turns the attribute off (plain launches)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Facts about the current device, cached per device ordinal (a process may hold sessions on
// several devices).
int sm_count();  // multiprocessors of the current device; 0 when the query fails
// Opts `kernel` into `bytes` of dynamic shared memory on the current device (once per device
// and kernel; the attribute belongs to the device's context).
int ensure_dynamic_smem(const void* kernel, int bytes);
// The current device's sticky error word: pinned host memory mapped into the device. A kernel
// whose bounded wait gives up stores a non-zero code there and never clears it; the host reads
// and clears it with check_device_error() after the stream has drained. nullptr on failure
// (message set). The first call on a device allocates; sessions and the operator entry points
// make it before any launch or stream capture.
int* device_error_word();
int check_device_error(const char* what);  // 1 (message set, word cleared) when a wait expired
enum { DEV_ERR_GEMV_RING = 1, DEV_ERR_GEMM_PIPE = 2 };
__device__ __forceinline__ void report_wait_expired(int* word, int code) {
  if (word) {
    *reinterpret_cast<volatile int*>(word) = code;
    __threadfence_system();
  }
}

// Counts kernels launched by this library (per thread-attached counter).
void count_launch(int n = 1);
uint64_t* launch_counter_slot();  // where count_launch accumulates (thread-local pointer)

// ---- encodings ----------------------------------------------------------------
enum : int {
  E_F32 = DYNINFER_ENC_F32,
  E_F16 = DYNINFER_ENC_F16,
  E_BF16 = DYNINFER_ENC_BF16,
  E_Q4_0 = DYNINFER_ENC_Q4_0,
  E_Q4_1 = DYNINFER_ENC_Q4_1,
  E_Q8_0 = DYNINFER_ENC_Q8_0,
  E_Q6_K = DYNINFER_ENC_Q6_K,
  E_MLX_U4 = DYNINFER_ENC_MLX_U4,
  E_Q4_K = DYNINFER_ENC_Q4_K,
  E_Q5_K = DYNINFER_ENC_Q5_K,
  E_IQ4_XS = DYNINFER_ENC_IQ4_XS,
  E_LAST = DYNINFER_ENC_IQ4_XS,
};

__host__ __device__ inline int enc_block_elems(int enc) {
  switch (enc) {
    case E_Q4_0:
    case E_Q4_1:
    case E_Q8_0:
      return 32;
    case E_Q6_K:
    case E_Q4_K:
    case E_Q5_K:
    case E_IQ4_XS:
      return 256;
    case E_MLX_U4:
      return 8;
    default:
      return 1;
  }
}
__host__ __device__ inline int enc_block_bytes(int enc) {
  switch (enc) {
    case E_F32:
      return 4;
    case E_F16:
    case E_BF16:
      return 2;
    case E_Q4_0:
      return 18;
    case E_Q4_1:
      return 20;
    case E_Q8_0:
      return 34;
    case E_Q6_K:
      return 210;
    case E_Q4_K:
      return 144;
    case E_Q5_K:
      return 176;
    case E_IQ4_XS:
      return 136;
    case E_MLX_U4:
      return 4;
    default:
      return 0;
  }
}
__host__ __device__ inline int64_t enc_row_bytes(int enc, int64_t cols) {
  int be = enc_block_elems(enc);
  return (cols % be) ? 0 : cols / be * enc_block_bytes(enc);
}
inline int aux_elem_bytes(int t) { return t == E_F32 ? 4 : 2; }

// A weight as the kernels see it.
struct WRef {
  const uint8_t* data = nullptr;
  const uint8_t* scales = nullptr;
  const uint8_t* biases = nullptr;
  int enc = 0, aux = E_BF16, group = 64;
  int64_t rows = 0, cols = 0;
  __host__ __device__ int64_t row_bytes() const { return enc_row_bytes(enc, cols); }
  uint64_t total_bytes() const {
    uint64_t b = (uint64_t)rows * (uint64_t)enc_row_bytes(enc, cols);
    if (enc == E_MLX_U4) b += 2ull * rows * (cols / group) * aux_elem_bytes(aux);
    return b;
  }
};

int wref_from_api(const dyninfer_cuda_weight_t* w, WRef* out);

// ---- small device helpers -------------------------------------------------------
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
  return *reinterpret_cast<const uint16_t*>(p);
}
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {  // 2-byte aligned 32-bit load
  return ld_u16(p) | (ld_u16(p + 2) << 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t b) {
  return __half2float(__ushort_as_half((unsigned short)b));
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ float aux_load(const uint8_t* base, int type, int64_t idx) {
  if (type == E_F32) return reinterpret_cast<const float*>(base)[idx];
  uint32_t b = reinterpret_cast<const uint16_t*>(base)[idx];
  return type == E_F16 ? f16_bits_to_f32(b) : bf16_bits_to_f32(b);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct FreqTable {  // inverse RoPE frequencies, one per rotated pair (head_dim <= 256)
  float f[128];
};
void fill_freq_table(FreqTable* t, int64_t d, float theta);

// ---- launchers (one per kernel family) -------------------------------------------
int launch_dequant(const WRef& w, float* out, cudaStream_t s);
int launch_gather(const WRef& w, const int64_t* tokens, int64_t count, float* out, cudaStream_t s);

// y[m, N] = x[m, K] * W^T ; optional residual (added to result) ; x f32 or bf16.
int launch_linear(const WRef& w, const void* x, int x_type, int64_t m, float* y,
                  const float* residual, cudaStream_t s);
// Tensor-core GEMV for few activation rows (gemv_mma.cu); *handled tells whether it ran.
// Optional hand-overs around the dequant GEMM, for callers that fuse its neighbours (a session's prefill
// chunks): activations already in the GEMM's own form (f16 rows scaled by a power of two per row, the
// inverse scales beside them; rows_alloc >= dqgemm_tc_padded_rows), and a place where a K-split product
// leaves its sums [splits][M][N] instead of running its own reduction (the caller's next kernel adds them
// in ascending split order, then the residual: what tg_split_reduce_kernel computes).
struct TgIo {
  const __half* xh = nullptr;
  const float* inv_s = nullptr;
  int64_t rows_alloc = 0;
  float* partial = nullptr;
  size_t partial_bytes = 0;
  int splits = 0;  // out: > 1 when the sums were left in `partial` (y untouched)
};
int launch_dqgemm_tc(const WRef& w, const void* x, int x_type, int64_t M, float* y, const float* residual,
                     cudaStream_t s, bool* handled, TgIo* io = nullptr);
// Whether launch_dqgemm_tc takes the product, and the activation rows its tiling pads M to.
bool dqgemm_tc_takes(const WRef& w, int64_t M);
int64_t dqgemm_tc_padded_rows(const WRef& w, int64_t M);
bool gemv_cs_q8_0_shape_ok(const WRef& w, int M);
size_t gemv_cs_q8_0_workspace_bytes(const WRef& w, int M);
int launch_gemv_cs_q8_0(const WRef& w, const void* x, int x_type, float* y, const float* residual, uint8_t* ws,
                        cudaStream_t s);
bool gemv_cs_q6k_shape_ok(const WRef& w, int M);
size_t gemv_cs_q6k_workspace_bytes(const WRef& w, int M);
int launch_gemv_cs_q6k(const WRef& w, const void* x, int x_type, float* y, const float* residual, uint8_t* ws,
                       cudaStream_t s);
size_t gemv_cs_workspace_bytes(const WRef& w, int M);
int launch_gemv_cs(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                   uint8_t* ws, cudaStream_t s, bool* handled);
int launch_gemv_plain(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                      cudaStream_t s, bool* handled);
size_t gemv_mma_workspace_bytes(const WRef& w, int x_type, int M);
int launch_gemv_mma(const WRef& w, const void* x, int x_type, int M, float* y, const float* residual,
                    void* workspace, cudaStream_t s, bool* handled);
// y = silu(x Wg^T) * (x Wu^T)
int launch_linear_swiglu(const WRef& wg, const WRef& wu, const float* x, int64_t m, float* y,
                         cudaStream_t s);

int launch_rms_norm(const float* x, const void* w, int w_type, int64_t rows, int64_t width,
                    float eps, float* y, cudaStream_t s);
// Rows of a prefill chunk / batched step feeding the dequant GEMM, one launch instead of three or four:
//   v = (splits ? sum over the K-split sums partial[z][row][:] : x[row][:]) + residual[row][:]  -> hidden (if given)
//   y = RMSNorm(v) * w, written as the GEMM's activation operand: xh[row][:] = f16(y * 2^k), inv_s[row] = 2^-k.
// Bit for bit what tg_split_reduce_kernel, rms_norm_kernel and the GEMM's activation pass produce in turn.
int launch_norm_prepare(const float* x, const float* partial, int splits, const float* residual, float* hidden,
                        const void* w, int w_type, int64_t rows, int64_t width, float eps, __half* xh, float* inv_s,
                        cudaStream_t s);
// The same for the SwiGLU: rows of [gate | up] -> silu(gate) * up as the GEMM's activation operand.
int launch_silu_prepare(const float* gate_up, int64_t rows, int64_t inter, __half* xh, float* inv_s, cudaStream_t s);
// One row of [gate | up] (2 * inter values, deferred or in `gate_up`): y = silu(gate) * up
int launch_silu_mul_deferred(const Deferred& d, const float* gate_up, int64_t inter, float* y, cudaStream_t s);
int launch_rope(float* x, int64_t s_rows, int64_t heads, int64_t d, int64_t start_pos,
                const FreqTable& ft, cudaStream_t s);
int launch_silu_mul(const float* gate, const float* up, int64_t n, float* y, cudaStream_t s);
int launch_silu_mul_rows(const float* gate_up, int64_t rows, int64_t inter, float* y, cudaStream_t s);

struct QkvPrepArgs {
  float* q;        // [rows, nh, d]   normalised + rotated in place
  const float* k;  // [rows, nkv, d]
  const float* v;  // [rows, nkv, d]
  void* kcache;    // layer base: [seq][nkv][cap][d]
  void* vcache;
  const void* q_norm_w;  // nullable
  const void* k_norm_w;
  int norm_w_type;
  const int64_t* row_pos;  // [rows] absolute position of each row; NULL: base_pos + row
  const int64_t* row_seq;  // [rows] cache slot of each row; NULL: slot 0
  int64_t base_pos;
  int64_t rows, nh, nkv, d, cap;
  int kv_type, has_norm, has_rope;
  float eps;
  // floats between consecutive rows of q / k / v (0: dense, nh*d / nkv*d): the three may be column
  // ranges of one [rows, nh*d + 2*nkv*d] matrix, the output of the fused [q; k; v] product
  int64_t ldq = 0, ldk = 0, ldv = 0;
  // q / k / v still lie as K-slice sums of their product (the reduced q is written to `q`): a single row's
  // streaming GEMV, or all rows of a K-split dequant GEMM
  DeferredCols dq, dk, dv;
};
int launch_qkv_prepare(const QkvPrepArgs& a, const FreqTable& ft, cudaStream_t s);

struct AttnArgs {
  const float* q;  // [rows, nh, d]
  const void* kcache;
  const void* vcache;
  const int64_t* row_pos;  // NULL: base_pos + row
  const int64_t* row_seq;  // NULL: slot 0
  int64_t base_pos;
  float* ctx;  // [rows, nh*d]
  int64_t rows, nh, nkv, d, cap;
  int kv_type;
  // >= 0: the rows are consecutive positions uniform_base + row of sequence uniform_seq even though
  // row_pos / row_seq are given (prefill chunks); lets the tensor-core prefill kernel take them
  int64_t uniform_base = -1, uniform_seq = 0;
  int64_t ldq = 0;  // floats between consecutive rows of q (0: dense, nh*d)
};
int launch_attention(const AttnArgs& a, cudaStream_t s);
size_t attention_split_scratch_bytes(int64_t rows, int64_t nh, int64_t d, int nsplit);
int launch_attention_split(const AttnArgs& a, float* part, int nsplit, cudaStream_t s, bool* handled);
int launch_attention_prefill(const AttnArgs& a, int64_t base_pos, int64_t seq, cudaStream_t s, bool* handled);

size_t argmax_scratch_bytes(int64_t n);
int launch_argmax(const float* v, int64_t n, int64_t* out, void* scratch, cudaStream_t s);
int launch_argmax_rows(const float* v, int64_t rows, int64_t n, int64_t* out, cudaStream_t s);
// The same over logits held as `shards` slices [shards][rows][n_local]: index w * n_local + j.
int launch_argmax_rows_sharded(const float* v, int64_t rows, int64_t n_local, int shards, int64_t* out,
                               cudaStream_t s);

// ---- tensor-parallel exchange over peer memory (tp_peer.cu) ----
constexpr int TP_MAX_WORLD = 8;
constexpr int TP_PEER_BLOCKS = 128;
struct TpPeer {
  int rank = 0, world = 1;
  int64_t max_rows = 0;
  uint8_t* base[TP_MAX_WORLD] = {};  // every rank's region as mapped in this process (own: the allocation)
  size_t region_bytes = 0, flags_off = 0;
  unsigned* epochs = nullptr;        // [TP_PEER_BLOCKS] exchanges entered per block, own
  int* error_host = nullptr;         // pinned, mapped: which wait ran out (0 = none)
  int* error_dev = nullptr;
  bool attached = false;
  long long spin_limit = 0;          // polls before a wait gives up (0: the default, about ten seconds)
};
size_t tp_peer_region_bytes(int64_t max_rows, int hidden);
size_t tp_peer_flags_offset(int64_t max_rows, int hidden);
// hidden[rows, H] += sum over ranks of slot `slot` of their regions; xn = RMSNorm(hidden) * norm_w
// when xn is given. Every rank launches it with the same arguments in the same order.
int launch_tp_exchange(const TpPeer& p, int slot, int64_t rows, int H, float* hidden, float* xn,
                       const void* norm_w, int norm_type, float eps, cudaStream_t st);

// ---- tensor-parallel exchange (tp_comm.cu; NCCL looked up at run time) ----
size_t tp_unique_id_bytes();
int tp_unique_id(uint8_t* out);
int tp_comm_init(void** comm, const uint8_t* id_bytes, int rank, int world);
void tp_comm_destroy(void* comm);
int tp_all_reduce_sum(void* comm, const float* send, float* recv, size_t count, cudaStream_t st);
int tp_all_gather(void* comm, const float* send, float* recv, size_t count_per_rank, cudaStream_t st);

}  // namespace dyn
