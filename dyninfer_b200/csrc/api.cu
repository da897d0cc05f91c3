// extern "C" surface: error channel, library queries and the single-operator
// entry points. Argument validation happens here, on the host, before any
// launch (the reference validates at the same boundary,
// third_party/iree_runtime_c_api/wrapper.c:1230-1239).
#include <stdarg.h>
#include <stdio.h>

#include <map>
#include <mutex>
#include <string>

#include <stdlib.h>

#include "common.cuh"

namespace dyn {

static thread_local std::string g_last_error;
static thread_local uint64_t g_default_counter = 0;
static thread_local uint64_t* g_counter = &g_default_counter;

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
  return 1;
}

// Scratch taken from the stream-ordered allocator is returned right after use; without a release
// threshold the default pool trims to zero at every synchronisation and the next call pays a full
// device allocation. Once per thread and device.
int keep_scratch_pool_cached() {
  static thread_local int tuned_device = -1;
  int dev = 0;
  DYN_CUDA(cudaGetDevice(&dev));
  if (tuned_device == dev) return 0;
  cudaMemPool_t pool;
  DYN_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
  uint64_t keep = ~0ull;
  DYN_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
  tuned_device = dev;
  return 0;
}

static thread_local void* g_scratch = nullptr;
static thread_local size_t g_scratch_bytes = 0;
static thread_local size_t g_scratch_held = 0;
void set_thread_scratch(void* ptr, size_t bytes) { g_scratch = ptr, g_scratch_bytes = ptr ? bytes : 0, g_scratch_held = 0; }
void* thread_scratch(size_t bytes) {
  return g_scratch_held + bytes <= g_scratch_bytes ? static_cast<uint8_t*>(g_scratch) + g_scratch_held : nullptr;
}
void thread_scratch_hold(size_t bytes) { g_scratch_held += (bytes + 255) / 256 * 256; }
void thread_scratch_release_all() { g_scratch_held = 0; }

static thread_local Deferred* g_defer = nullptr;
void defer_request(Deferred* d) { g_defer = d; }
Deferred* defer_take() {
  Deferred* d = g_defer;
  g_defer = nullptr;
  return d;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("DYNINFER_CUDA_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// ---- per-device facts: SM count, opted-in shared memory per kernel, sticky error word ----------
namespace {
constexpr int MAX_DEVICES = 64;
struct DeviceSlot {
  int sms = 0;
  int* err_host = nullptr;  // pinned, mapped: written by kernels whose bounded wait gave up
  int* err_dev = nullptr;
  std::map<const void*, int> smem_attr;  // kernel -> largest dynamic shared memory opted into
};
std::mutex g_dev_mu;
DeviceSlot g_dev[MAX_DEVICES];
DeviceSlot* current_slot() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  return g_dev + dev;
}
}  // namespace

int sm_count() {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceSlot* d = current_slot();
  if (!d) return 0;
  if (!d->sms) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    d->sms = n;
  }
  return d->sms;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceSlot* d = current_slot();
  DYN_CHECK(d != nullptr, "no current CUDA device");
  auto it = d->smem_attr.find(kernel);
  if (it != d->smem_attr.end() && it->second >= bytes) return 0;
  DYN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  d->smem_attr[kernel] = bytes;
  return 0;
}

int* device_error_word() {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceSlot* d = current_slot();
  if (!d) {
    set_error("no current CUDA device");
    return nullptr;
  }
  if (!d->err_dev) {
    int* h = nullptr;
    int* p = nullptr;
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&p), h, 0);
    if (e != cudaSuccess) {
      cuda_fail(e, "allocating the device error word", __FILE__, __LINE__);
      return nullptr;
    }
    *h = 0;
    d->err_host = h, d->err_dev = p;
  }
  return d->err_dev;
}

int check_device_error(const char* what) {
  int code = 0;
  {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    DeviceSlot* d = current_slot();
    if (!d || !d->err_host) return 0;
    code = *reinterpret_cast<volatile int*>(d->err_host);
    if (code) *reinterpret_cast<volatile int*>(d->err_host) = 0;
  }
  if (!code) return 0;
  set_error("%s: a bounded wait inside a kernel expired (code %d: 1 single-row product weight ring, "
            "2 tensor-core GEMM pipeline); the results of the call are invalid", what, code);
  return 1;
}

void count_launch(int n) { *g_counter += (uint64_t)n; }
uint64_t* launch_counter_slot() { return g_counter; }
void set_launch_counter(uint64_t* p) { g_counter = p ? p : &g_default_counter; }

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int wref_from_api(const dyninfer_cuda_weight_t* w, WRef* out) {
  DYN_CHECK(w != nullptr, "weight descriptor is NULL");
  DYN_CHECK(w->encoding >= E_F32 && w->encoding <= E_LAST, "unknown encoding %d", w->encoding);
  DYN_CHECK(w->rows >= 0 && w->cols > 0, "weight shape [%lld, %lld] is invalid",
            (long long)w->rows, (long long)w->cols);
  int unit = enc_block_elems(w->encoding);
  if (unit < 4) unit = 4;
  DYN_CHECK(w->cols % unit == 0, "cols %lld is not a multiple of %d for encoding %d",
            (long long)w->cols, unit, w->encoding);
  DYN_CHECK(w->data != nullptr && aligned(w->data, 16), "weight data must be a 16-byte aligned device pointer");
  out->data = reinterpret_cast<const uint8_t*>(w->data);
  out->enc = w->encoding;
  out->rows = w->rows;
  out->cols = w->cols;
  out->scales = out->biases = nullptr;
  out->aux = E_BF16;
  out->group = 64;
  if (w->encoding == E_MLX_U4) {
    DYN_CHECK(w->group >= 8 && w->group % 8 == 0 && w->cols % w->group == 0,
              "MLX group %d does not divide cols %lld", w->group, (long long)w->cols);
    DYN_CHECK(w->aux_type == E_F32 || w->aux_type == E_F16 || w->aux_type == E_BF16,
              "MLX scales/biases type %d unsupported", w->aux_type);
    DYN_CHECK(w->scales && w->biases, "MLX weight needs scales and biases");
    out->scales = reinterpret_cast<const uint8_t*>(w->scales);
    out->biases = reinterpret_cast<const uint8_t*>(w->biases);
    out->aux = w->aux_type;
    out->group = w->group;
  }
  return 0;
}

static int require_device() {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    set_error("no usable CUDA device (%s); this target has no CPU fallback",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace dyn

using namespace dyn;

extern "C" {

int dyninfer_cuda_abi_version(void) { return DYNINFER_CUDA_ABI_VERSION; }

const char* dyninfer_cuda_last_error(void) { return g_last_error.c_str(); }

int dyninfer_cuda_device_count(int* out_count) {
  DYN_CHECK(out_count != nullptr, "out_count is NULL");
  *out_count = 0;
  if (require_device()) return 1;
  int n = 0;
  DYN_CUDA(cudaGetDeviceCount(&n));
  *out_count = n;
  return 0;
}

uint64_t dyninfer_cuda_row_bytes(int encoding, int64_t cols) {
  if (encoding < E_F32 || encoding > E_LAST || cols <= 0) return 0;
  return (uint64_t)enc_row_bytes(encoding, cols);
}

int dyninfer_cuda_dequant(const dyninfer_cuda_weight_t* w, float* out_dev, void* stream) {
  WRef r;
  if (wref_from_api(w, &r)) return 1;
  DYN_CHECK(out_dev && aligned(out_dev, 16), "out must be a 16-byte aligned device pointer");
  if (require_device()) return 1;
  return launch_dequant(r, out_dev, (cudaStream_t)stream);
}

int dyninfer_cuda_embedding_gather(const dyninfer_cuda_weight_t* w, const int64_t* tokens_dev,
                                   int64_t count, float* out_dev, void* stream) {
  WRef r;
  if (wref_from_api(w, &r)) return 1;
  DYN_CHECK(count >= 0, "count must be >= 0");
  DYN_CHECK(count == 0 || tokens_dev, "tokens is NULL");
  if (count == 0) return 0;
  DYN_CHECK(out_dev && aligned(out_dev, 16), "out must be a 16-byte aligned device pointer");
  if (require_device()) return 1;
  return launch_gather(r, tokens_dev, count, out_dev, (cudaStream_t)stream);
}

int dyninfer_cuda_linear(const dyninfer_cuda_weight_t* w, const void* x_dev, int x_type, int64_t m,
                         float* y_dev, void* stream) {
  WRef r;
  if (wref_from_api(w, &r)) return 1;
  DYN_CHECK(x_dev && aligned(x_dev, 16), "x must be a 16-byte aligned device pointer");
  DYN_CHECK(y_dev != nullptr, "y is NULL");
  if (require_device()) return 1;
  return launch_linear(r, x_dev, x_type, m, y_dev, nullptr, (cudaStream_t)stream);
}

int dyninfer_cuda_rms_norm(const float* x_dev, const void* w_dev, int w_type, int64_t rows,
                           int64_t width, float eps, float* y_dev, void* stream) {
  DYN_CHECK(x_dev && w_dev && y_dev, "rms_norm: NULL pointer");
  DYN_CHECK(rows >= 0 && width > 0, "rms_norm: bad shape");
  DYN_CHECK(w_type == E_F32 || w_type == E_F16 || w_type == E_BF16, "rms_norm: weight type %d",
            w_type);
  if (require_device()) return 1;
  return launch_rms_norm(x_dev, w_dev, w_type, rows, width, eps, y_dev, (cudaStream_t)stream);
}

int dyninfer_cuda_rope(float* x_dev, int64_t s, int64_t heads, int64_t d, int64_t start_pos,
                       float theta, void* stream) {
  DYN_CHECK(x_dev != nullptr, "rope: x is NULL");
  DYN_CHECK(s >= 0 && heads > 0 && d > 0 && d % 2 == 0 && d <= 256, "rope: bad shape");
  DYN_CHECK(start_pos >= 0, "rope: start_pos must be >= 0");
  if (require_device()) return 1;
  FreqTable ft;
  fill_freq_table(&ft, d, theta);
  return launch_rope(x_dev, s, heads, d, start_pos, ft, (cudaStream_t)stream);
}

int dyninfer_cuda_silu_mul(const float* gate_dev, const float* up_dev, int64_t n, float* y_dev,
                           void* stream) {
  DYN_CHECK(gate_dev && up_dev && y_dev, "silu_mul: NULL pointer");
  DYN_CHECK(n >= 0, "silu_mul: n must be >= 0");
  if (require_device()) return 1;
  return launch_silu_mul(gate_dev, up_dev, n, y_dev, (cudaStream_t)stream);
}

int dyninfer_cuda_attention(const float* q_dev, const void* k_cache_dev, const void* v_cache_dev,
                            int kv_type, int64_t s, int64_t heads, int64_t kv_heads, int64_t d,
                            int64_t kv_cap, int64_t start_pos, float* ctx_dev, void* stream) {
  DYN_CHECK(q_dev && k_cache_dev && v_cache_dev && ctx_dev, "attention: NULL pointer");
  DYN_CHECK(s >= 0 && heads > 0 && kv_heads > 0 && d > 0, "attention: bad shape");
  DYN_CHECK(start_pos >= 0 && start_pos + s <= kv_cap,
            "attention: rows [%lld, %lld) exceed cache capacity %lld", (long long)start_pos,
            (long long)(start_pos + s), (long long)kv_cap);
  if (require_device()) return 1;
  AttnArgs a{};
  a.q = q_dev;
  a.kcache = k_cache_dev;
  a.vcache = v_cache_dev;
  a.row_pos = nullptr;
  a.row_seq = nullptr;
  a.base_pos = start_pos;
  a.ctx = ctx_dev;
  a.rows = s, a.nh = heads, a.nkv = kv_heads, a.d = d, a.cap = kv_cap;
  a.kv_type = kv_type;
  return launch_attention(a, (cudaStream_t)stream);
}

size_t dyninfer_cuda_argmax_scratch_bytes(int64_t n) { return argmax_scratch_bytes(n); }

int dyninfer_cuda_argmax(const float* v_dev, int64_t n, int64_t* out_index_dev, void* scratch_dev,
                         void* stream) {
  DYN_CHECK(v_dev && out_index_dev && scratch_dev, "argmax: NULL pointer");
  DYN_CHECK(aligned(scratch_dev, 16), "argmax: scratch must be 16-byte aligned");
  if (require_device()) return 1;
  return launch_argmax(v_dev, n, out_index_dev, scratch_dev, (cudaStream_t)stream);
}

int dyninfer_cuda_check_device_error(void) {
  if (require_device()) return 1;
  return check_device_error("device error word");
}

void dyninfer_cuda_free(void*) {}

}  // extern "C"
