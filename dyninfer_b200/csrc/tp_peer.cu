// Tensor-parallel exchange over peer memory (NVLink / NVSwitch), fused with what follows it:
// one kernel per row-parallel product that (1) tells every peer this rank's partial product is in
// place, (2) waits for theirs, (3) reads all partial rows straight from the peers' memory, adds
// them in rank order together with the residual and (4) applies the RMSNorm that feeds the next
// product. Every rank computes the same sum in the same order, so the hidden state stays
// bit-identical across ranks without a broadcast.
//
// Memory: every rank owns one region [2 slots][max_rows][hidden] f32 + flags, mapped into the
// peers through CUDA IPC. The o_proj partials use slot 0, the down partials slot 1: a slot is
// rewritten only after this rank has passed the next exchange's arrival step, by which time every
// peer has finished the kernel that read it (kernels of one stream run in order).
// Flags: flags[block][rank] holds the number of exchanges block `block` of rank `rank` has
// entered; a block handles rows block, block + grid, ... and counts its own exchanges in
// epochs[block]. All ranks launch the same sequence of exchanges with the same grids.
// Every wait is bounded; on expiry the kernel records it in a host-visible error word and goes on
// (the step's numbers are then wrong, the caller reports the error after the stream has drained).
#include "codec.cuh"
#include "common.cuh"

namespace dyn {
namespace {

constexpr int TP_THREADS = 1024;
constexpr long long TP_SPINS = 40LL * 1000 * 1000;  // x ~250 ns per poll: about ten seconds

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerArgs {
  const float* part[TP_MAX_WORLD];  // every rank's partial rows for this exchange (own included)
  unsigned* flags[TP_MAX_WORLD];    // every rank's flag array (own included)
  unsigned* epochs;                 // own, per block
  int* error;                       // host-visible
  float* hidden;                    // residual in, sum out [rows, H]
  float* xn;                        // normalised rows out (or nullptr)
  const void* norm_w;
  int norm_type;
  float eps;
  int rank, world, rows, H;
  long long spins;                  // polls before a wait gives up
};

__global__ void __launch_bounds__(TP_THREADS, 1) tp_exchange_kernel(const PeerArgs a) {
  __shared__ float red[32];
  __shared__ float s_inv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();  // a product launched next may begin fetching its weights
  // launched as a programmatic dependent: everything above and the launch itself overlap the tail
  // of the product before; its partial rows (and this kernel's own epoch word) are there after the wait
  pdl_wait();
  const unsigned e = a.epochs[blockIdx.x] + 1;
  // arrival: this rank's partial rows were written by the kernel before this one
  if (tid < a.world) {
    __threadfence_system();
    st_release_sys(a.flags[tid] + (size_t)blockIdx.x * TP_MAX_WORLD + a.rank, e);
    const unsigned* mine = a.flags[a.rank] + (size_t)blockIdx.x * TP_MAX_WORLD + tid;
    long long it = 0;
    unsigned seen = 0;
    for (; it < a.spins; it++) {
      seen = ld_acquire_sys(mine);
      if ((int)(seen - e) >= 0) break;
      __nanosleep(32);
    }
    if ((int)(seen - e) < 0) *a.error = 1 + tid;  // peer `tid` did not arrive
  }
  __syncthreads();
  const int H4 = a.H >> 2;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    float ss = 0.f;
    for (int i = tid; i < H4; i += TP_THREADS) {
      const size_t off = (size_t)row * H4 + i;
      float4 acc = reinterpret_cast<const float4*>(a.hidden)[off];
      for (int r = 0; r < a.world; r++) {
        const float4 p = __ldcg(reinterpret_cast<const float4*>(a.part[r]) + off);
        acc.x += p.x, acc.y += p.y, acc.z += p.z, acc.w += p.w;
      }
      reinterpret_cast<float4*>(a.hidden)[off] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
    if (a.xn == nullptr) continue;
    // RMSNorm of the finished row: inv = 1/sqrt(mean(x^2) + eps), y = (x * inv) * w
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      float t = red[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) s_inv = 1.0f / sqrtf(t / (float)a.H + a.eps);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int i = tid; i < H4; i += TP_THREADS) {
      const size_t off = (size_t)row * H4 + i;
      const float4 v = reinterpret_cast<const float4*>(a.hidden)[off];  // this thread wrote it above
      const uint8_t* w = reinterpret_cast<const uint8_t*>(a.norm_w);
      float4 y;
      y.x = __fmul_rn(__fmul_rn(v.x, inv), aux_load(w, a.norm_type, 4 * i + 0));
      y.y = __fmul_rn(__fmul_rn(v.y, inv), aux_load(w, a.norm_type, 4 * i + 1));
      y.z = __fmul_rn(__fmul_rn(v.z, inv), aux_load(w, a.norm_type, 4 * i + 2));
      y.w = __fmul_rn(__fmul_rn(v.w, inv), aux_load(w, a.norm_type, 4 * i + 3));
      reinterpret_cast<float4*>(a.xn)[off] = y;
    }
    __syncthreads();  // red / s_inv are reused by the next row
  }
  if (tid == 0) a.epochs[blockIdx.x] = e;
}

}  // namespace

size_t tp_peer_region_bytes(int64_t max_rows, int hidden) {
  const size_t data = 2 * (size_t)max_rows * hidden * 4;
  return (data + 255) / 256 * 256 + (size_t)TP_PEER_BLOCKS * TP_MAX_WORLD * 4;
}
size_t tp_peer_flags_offset(int64_t max_rows, int hidden) {
  return (2 * (size_t)max_rows * hidden * 4 + 255) / 256 * 256;
}

int launch_tp_exchange(const TpPeer& p, int slot, int64_t rows, int H, float* hidden, float* xn,
                       const void* norm_w, int norm_type, float eps, cudaStream_t st) {
  DYN_CHECK(H % 4 == 0 && rows >= 1 && rows <= p.max_rows, "tp exchange: rows %lld or hidden %d unsupported",
            (long long)rows, H);
  PeerArgs a{};
  for (int r = 0; r < p.world; r++) {
    a.part[r] = reinterpret_cast<const float*>(p.base[r]) + (size_t)slot * p.max_rows * H;
    a.flags[r] = reinterpret_cast<unsigned*>(p.base[r] + p.flags_off);
  }
  a.epochs = p.epochs, a.error = p.error_dev;
  a.hidden = hidden, a.xn = xn, a.norm_w = norm_w, a.norm_type = norm_type, a.eps = eps;
  a.rank = p.rank, a.world = p.world, a.rows = (int)rows, a.H = H;
  a.spins = p.spin_limit > 0 ? p.spin_limit : TP_SPINS;
  const int grid = (int)std::min<int64_t>(rows, TP_PEER_BLOCKS);
  DYN_CUDA(launch_pdl(tp_exchange_kernel, dim3(grid), dim3(TP_THREADS), 0, st, a));
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace dyn

// Exercises the bounded wait of the exchange on ONE device, with no peer involved: a two-rank
// exchange whose "peer" region is a second local allocation whose arrival flag nobody raises.
// The kernel must give up after `spin_limit` polls, record which rank was missing and finish;
// the call then fails with the same message a session reports. The device stays usable.
extern "C" int dyninfer_cuda_tp_exchange_wait_probe(int hidden, int64_t rows, int64_t spin_limit) {
  using namespace dyn;
  DYN_CHECK(hidden >= 4 && hidden % 4 == 0 && rows >= 1 && rows <= 64 && spin_limit >= 1 && spin_limit <= 10000000,
            "wait probe: hidden %d, rows %lld or spin_limit %lld out of range", hidden, (long long)rows,
            (long long)spin_limit);
  TpPeer p;
  p.rank = 0, p.world = 2, p.max_rows = rows, p.spin_limit = spin_limit;
  p.region_bytes = tp_peer_region_bytes(rows, hidden);
  p.flags_off = tp_peer_flags_offset(rows, hidden);
  float *hid = nullptr, *xn = nullptr, *ones = nullptr;
  cudaStream_t st = nullptr;
  int rc = 1;
  auto cleanup = [&]() {
    for (int r = 0; r < 2; r++)
      if (p.base[r]) cudaFree(p.base[r]);
    if (p.epochs) cudaFree(p.epochs);
    if (p.error_host) cudaFreeHost(p.error_host);
    if (hid) cudaFree(hid);
    if (xn) cudaFree(xn);
    if (ones) cudaFree(ones);
    if (st) cudaStreamDestroy(st);
  };
  do {
    bool ok = true;
    for (int r = 0; r < 2 && ok; r++)
      ok = cudaMalloc(reinterpret_cast<void**>(&p.base[r]), p.region_bytes) == cudaSuccess &&
           cudaMemset(p.base[r], 0, p.region_bytes) == cudaSuccess;
    const size_t vb = (size_t)rows * hidden * 4;
    ok = ok && cudaMalloc(reinterpret_cast<void**>(&p.epochs), TP_PEER_BLOCKS * 4) == cudaSuccess &&
         cudaMemset(p.epochs, 0, TP_PEER_BLOCKS * 4) == cudaSuccess &&
         cudaHostAlloc(reinterpret_cast<void**>(&p.error_host), 64, cudaHostAllocMapped) == cudaSuccess &&
         cudaHostGetDevicePointer(reinterpret_cast<void**>(&p.error_dev), p.error_host, 0) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&hid), vb) == cudaSuccess && cudaMemset(hid, 0, vb) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&xn), vb) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&ones), (size_t)hidden * 4) == cudaSuccess &&
         cudaMemset(ones, 0, (size_t)hidden * 4) == cudaSuccess &&
         cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
      cuda_fail(cudaGetLastError(), "wait probe set-up", __FILE__, __LINE__);
      break;
    }
    *p.error_host = 0;
    if (launch_tp_exchange(p, 0, rows, hidden, hid, xn, ones, E_F32, 1e-6f, st)) break;
    const cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
      cuda_fail(e, "wait probe kernel", __FILE__, __LINE__);
      break;
    }
    if (*p.error_host) {
      set_error("tensor-parallel exchange: rank %d did not arrive within the wait limit (rank %d gave up); "
                "the step's results are invalid", *p.error_host - 1, p.rank);
      break;
    }
    rc = 0;  // the wait did not expire: nothing to report
  } while (false);
  cleanup();
  return rc;
}
