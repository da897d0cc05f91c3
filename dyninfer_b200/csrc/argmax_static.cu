// Argmax (first strict maximum, dense_decoder.rs:885-893) for callers that must not allocate.
//
// Same result as dyninfer_cuda_argmax, but the per-block partial results live in a fixed array
// that is part of the loaded module instead of a caller-provided buffer, so the call performs no
// device allocation and needs no scratch pointer. The array holds one (value, index) pair per
// block for at most ARGMAX_STATIC_MAX_BLOCKS blocks of ARGMAX_STATIC_SPAN elements, i.e. inputs
// up to ARGMAX_STATIC_MAX_N elements (16 KiB of device memory); longer inputs are rejected.
//
// The array's device address is looked up once per device, by the first call made while that
// device is current. That first call therefore does set-up work and should be made before any
// stream capture begins. All calls on a device share the one array: every call overwrites the
// slots it is going to read, so nothing has to be cleared between calls, but two calls that are
// in flight at the same time (different streams or threads) race on it and give undefined results.
#include <mutex>

#include "common.cuh"

namespace dyn {
namespace {

constexpr int ARGMAX_STATIC_MAX_BLOCKS = 1024;
constexpr int ARGMAX_STATIC_SPAN = 4096;  // elements one block scans
constexpr int64_t ARGMAX_STATIC_MAX_N = (int64_t)ARGMAX_STATIC_MAX_BLOCKS * ARGMAX_STATIC_SPAN;
constexpr int ARGMAX_STATIC_MAX_DEVICES = 64;
constexpr long long NO_INDEX = 0x7fffffffffffffffLL;

struct StaticPair {
  float v;
  int pad;
  long long i;
};

static __device__ __align__(256) StaticPair g_argmax_scratch[ARGMAX_STATIC_MAX_BLOCKS];

__device__ __forceinline__ bool better(float v, long long i, float bv, long long bi) {
  return v > bv || (v == bv && i < bi);
}

__device__ __forceinline__ void warp_best(float& bv, long long& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
  }
}

// block-wide best pair; the result is valid in thread 0
template <int WARPS>
__device__ __forceinline__ void block_best(float& bv, long long& bi) {
  __shared__ float sv[WARPS];
  __shared__ long long si[WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  warp_best(bv, bi);
  if (lane == 0) sv[warp] = bv, si[warp] = bi;
  __syncthreads();
  if (warp == 0) {
    bv = lane < WARPS ? sv[lane] : -INFINITY;
    bi = lane < WARPS ? si[lane] : NO_INDEX;
    warp_best(bv, bi);
  }
}

__global__ void __launch_bounds__(256)
argmax_static_partial_kernel(const float* __restrict__ v, int64_t n, StaticPair* part) {
  const int64_t lo = (int64_t)blockIdx.x * ARGMAX_STATIC_SPAN;
  const int64_t hi = lo + ARGMAX_STATIC_SPAN < n ? lo + ARGMAX_STATIC_SPAN : n;
  float bv = -INFINITY;
  long long bi = NO_INDEX;
  for (int64_t i = lo + threadIdx.x; i < hi; i += 256) {
    const float x = v[i];
    if (x > -INFINITY && better(x, i, bv, bi)) bv = x, bi = i;
  }
  block_best<8>(bv, bi);
  if (threadIdx.x == 0) {
    part[blockIdx.x].v = bv;
    part[blockIdx.x].i = bi;
  }
}

__global__ void __launch_bounds__(1024)
argmax_static_final_kernel(const StaticPair* part, int count, int64_t* out) {
  float bv = -INFINITY;
  long long bi = NO_INDEX;
  if ((int)threadIdx.x < count) bv = part[threadIdx.x].v, bi = part[threadIdx.x].i;
  block_best<32>(bv, bi);
  // all values NaN or -inf: the scan never moves off index 0 (generate.rs:16-26)
  if (threadIdx.x == 0) out[0] = bi == NO_INDEX ? 0 : bi;
}

std::mutex g_setup_mutex;
StaticPair* g_scratch_ptr[ARGMAX_STATIC_MAX_DEVICES] = {};

// Device address of the array for the current device; looked up on first use.
int scratch_for_current_device(StaticPair** out) {
  int dev = -1;
  DYN_CUDA(cudaGetDevice(&dev));
  DYN_CHECK(dev >= 0 && dev < ARGMAX_STATIC_MAX_DEVICES, "argmax_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    StaticPair* ptr = nullptr;
    DYN_CUDA(cudaGetSymbolAddress((void**)&ptr, g_argmax_scratch));
    DYN_CHECK(ptr != nullptr, "argmax_static: the scratch array has no device address");
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace dyn

extern "C" {

int64_t dyninfer_cuda_argmax_static_max_n(void) { return dyn::ARGMAX_STATIC_MAX_N; }

int dyninfer_cuda_argmax_static(const float* v_dev, int64_t n, int64_t* out_index_dev, void* stream) {
  using namespace dyn;
  DYN_CHECK(v_dev && out_index_dev, "argmax_static: NULL pointer");
  DYN_CHECK(n >= 1, "argmax_static: n must be >= 1");
  DYN_CHECK(n <= ARGMAX_STATIC_MAX_N,
            "argmax_static: n = %lld exceeds the fixed scratch array (at most %lld elements); use "
            "dyninfer_cuda_argmax with a caller-provided scratch buffer",
            (long long)n, (long long)ARGMAX_STATIC_MAX_N);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  DYN_CHECK(e == cudaSuccess && count > 0, "no usable CUDA device; this target has no CPU fallback");
  StaticPair* part = nullptr;
  if (scratch_for_current_device(&part)) return 1;
  const int blocks = (int)((n + ARGMAX_STATIC_SPAN - 1) / ARGMAX_STATIC_SPAN);
  cudaStream_t s = (cudaStream_t)stream;
  argmax_static_partial_kernel<<<blocks, 256, 0, s>>>(v_dev, n, part);
  argmax_static_final_kernel<<<1, 1024, 0, s>>>(part, blocks, out_index_dev);
  count_launch(2);
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
