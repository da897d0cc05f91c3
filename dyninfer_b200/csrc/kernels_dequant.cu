// Bit-exact dequantisation of whole tensors and of gathered rows (embedding).
#include "codec.cuh"

namespace dyn {

// One thread per part; consecutive threads take consecutive parts of a row so
// that a warp reads a contiguous byte span of the raw tensor.
template <int ENC>
__global__ void __launch_bounds__(256)
dequant_rows_kernel(WRef w, const int64_t* __restrict__ row_index, int64_t row_count,
                    float* __restrict__ out) {
  using C = Codec<ENC>;
  const int64_t parts_per_row = (w.cols / C::BLOCK) * C::PARTS;
  const int64_t total = parts_per_row * row_count;
  for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < total;
       it += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = it / parts_per_row;
    const int64_t pr = it - r * parts_per_row;
    const int64_t blk = pr / C::PARTS;
    const int part = (int)(pr - blk * C::PARTS);
    int64_t src = row_index ? row_index[r] : r;
    if (src < 0 || src >= w.rows) src = 0;  // ids are validated on the host; stay in bounds regardless
    const RowPtr rp = row_ptr(w, src);
    float v[4 * C::G];
    C::decode(rp, blk, part, v);
    float* o = out + r * w.cols + blk * C::BLOCK;
#pragma unroll
    for (int g = 0; g < C::G; g++)
      *reinterpret_cast<float4*>(o + C::xoff(part, g)) =
          make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
  }
}

template <int ENC>
static int run_dequant(const WRef& w, const int64_t* idx, int64_t count, float* out,
                       cudaStream_t s) {
  using C = Codec<ENC>;
  const int64_t total = (w.cols / C::BLOCK) * C::PARTS * count;
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  dequant_rows_kernel<ENC><<<(unsigned)blocks, 256, 0, s>>>(w, idx, count, out);
  count_launch();
  DYN_CUDA(cudaGetLastError());
  return 0;
}

int launch_dequant(const WRef& w, float* out, cudaStream_t s) {
  DYN_ENC_SWITCH(w.enc, return run_dequant<ENC>(w, nullptr, w.rows, out, s));
  return 0;
}

int launch_gather(const WRef& w, const int64_t* tokens, int64_t count, float* out,
                  cudaStream_t s) {
  DYN_ENC_SWITCH(w.enc, return run_dequant<ENC>(w, tokens, count, out, s));
  return 0;
}

}  // namespace dyn
