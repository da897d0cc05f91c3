// Session: owns the uploaded parameters (verbatim byte ranges), the paged KV pool,
// the activation scratch and the captured decode graph. Shape and conventions follow
// the reference's native session, third_party/iree_runtime_c_api/wrapper.c:914-1303.
#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "common.cuh"
#include "decode_mega.cuh"
#include "json_min.h"

namespace dyn {
void set_launch_counter(uint64_t* p);

struct NormW {
  const void* ptr = nullptr;
  int type = E_F32;
  uint64_t bytes = 0;
};

struct LayerW {
  NormW attn_norm, ffn_norm, q_norm, k_norm;
  WRef q, k, v, o, gate, up, down;
  // rows of consecutive matrices seen as one (data == nullptr: not laid back to back)
  WRef qkv;     // [q; k] or [q; k; v]
  int qkv_parts = 0;
  WRef gate_up; // [gate; up]
};

struct ModelCfg {
  int layers = 0, hidden = 0, inter = 0, heads = 0, kv_heads = 0, head_dim = 0, vocab = 0;
  float eps = 1e-6f, theta = 10000.f;
  bool qk_norm = true, rope = true;
  int batch = 1;
  int kv2_type = E_BF16;  // element type used when the KV cache is configured with 2 bytes
  bool persistent = true;  // single-token steps run as the persistent decode kernel
  // tensor parallelism: heads / kv_heads / inter above are this rank's share; the lm_head holds
  // lm_rows = vocab / tp_world consecutive rows starting at tp_rank * lm_rows
  int tp_rank = 0, tp_world = 1, lm_rows = 0;
};

}  // namespace dyn

using namespace dyn;

struct dyninfer_cuda_session_t {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t tm0 = nullptr, tm1 = nullptr;  // dyninfer_cuda_session_timer
  ModelCfg cfg;
  FreqTable freq;
  // parameters
  uint8_t* arena = nullptr;
  uint64_t arena_bytes = 0;
  uint64_t weight_bytes = 0;         // sum of uploaded range lengths
  uint64_t decode_weight_bytes = 0;  // linears + lm_head + norm vectors
  WRef embed, lm_head;
  NormW out_norm;
  std::vector<LayerW> layers;
  // KV pool
  bool kv_configured = false;
  size_t page_size = 0, chunk_size = 0, kv_elem = 0, pages = 0;
  int kv_type = E_F32;
  uint8_t* kcache = nullptr;  // [layer][seq][nkv][cap][d]
  uint8_t* vcache = nullptr;
  size_t kv_bytes_each = 0;
  // scratch
  int64_t max_rows = 0;
  float *hidden = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *ctx = nullptr,
        *act = nullptr, *up = nullptr, *logits = nullptr;
  // many-row steps: the dequant GEMM's activation operand written by the norm / SwiGLU kernels, and the
  // K-split sums of o / down waiting for the residual + norm kernel
  __half* xh = nullptr;
  float *xinv = nullptr, *gpart = nullptr;
  int64_t xh_rows = 0, xh_cols = 0;
  size_t gpart_bytes = 0;
  float *qkv1 = nullptr, *gu1 = nullptr;  // rows of [q | k | v] and of [gate | up] for the fused products
  int64_t *tokens_dev = nullptr, *row_pos_dev = nullptr, *row_seq_dev = nullptr,
          *out_token_dev = nullptr, *hist_dev = nullptr, *hist_count_dev = nullptr;
  size_t hist_cap = 0;
  void* argmax_scratch = nullptr;
  float* batch_logits = nullptr;      // [batch, vocab], allocated by the first batched step
  int64_t* batch_tokens_dev = nullptr; // [batch]
  float* batch_logits_host = nullptr;  // pinned, allocated when logits are first requested
  // pinned host staging
  float* logits_host = nullptr;
  int64_t* stage_host = nullptr;  // [0]=token [1]=pos [2]=seq [3]=out token, then chunk arrays
  // persistent decode kernel
  bool mega = false;
  int mega_grid = 0, mega_nslot = 0, mega_xs = 0, mega_max_split = 1;
  size_t mega_smem = 0;
  MegaLayer* mega_layers = nullptr;
  int64_t* io_dev = nullptr;  // [0] token [1] position [2] slot [3] produced token [4] error word
  unsigned long long* prof_dev = nullptr;
  unsigned long long* trace_dev = nullptr;  // [grid][layers + 1][16] event stamps (DYNINFER_CUDA_TRACE=1)
  uint8_t* prog_dev = nullptr;  // [grid] program blobs
  MegaProgLayout mega_lay;
  float* ll_dev = nullptr;  // hand-off vectors of (value, epoch) pairs, one allocation
  size_t ll_off[7] = {};    // float offsets: hidden0, hidden1, qkv, ctx, part, act, amax
  unsigned mega_epoch = 0;  // epochs used so far (each launch takes layers + 2)
  // graphs
  cudaGraphExec_t decode_graph = nullptr;  // H2D token/pos + forward + D2H token
  cudaGraphExec_t loop_graph = nullptr;    // forward + device-side advance
  std::map<int64_t, std::pair<cudaGraphExec_t, uint64_t>> batch_graphs;  // rows -> batched step (graph, nodes)
  uint64_t graph_nodes = 0, loop_nodes = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // tensor parallelism (tp_world > 1): communicator, partial-sum scratch, per-rank logits
  void* tp_comm = nullptr;
  float* tp_part = nullptr;    // [max_rows, hidden] partial o_proj / down products of ranks > 0
  float* tp_logits = nullptr;  // [max(1, batch), lm_rows] this rank's slice of the logits
  float* tp_gather = nullptr;  // [tp_world, batch, lm_rows] gathered slices of a batched step
  bool tp_warm = false;        // the collectives have run once outside a capture
  TpPeer peer;                 // peer-memory exchange (used instead of the all-reduce once attached)
  // scratch of the single-row products (K-slice partial sums), owned here so that a captured step
  // has no allocation nodes between its kernels
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // statistics
  dyninfer_cuda_allocator_statistics_t stats{};
  uint64_t launches = 0;
};

namespace {

typedef dyninfer_cuda_session_t Session;

int dev_alloc(Session* s, void** out, size_t bytes) {
  DYN_CUDA(cudaMalloc(out, bytes ? bytes : 16));
  s->stats.device_bytes_allocated += bytes;
  uint64_t live = s->stats.device_bytes_allocated - s->stats.device_bytes_freed;
  s->stats.device_bytes_peak = std::max(s->stats.device_bytes_peak, live);
  return 0;
}
void dev_free(Session* s, void* p, size_t bytes) {
  if (!p) return;
  cudaFree(p);
  s->stats.device_bytes_freed += bytes;
}
int host_alloc(Session* s, void** out, size_t bytes) {
  DYN_CUDA(cudaMallocHost(out, bytes ? bytes : 16));
  s->stats.host_bytes_allocated += bytes;
  uint64_t live = s->stats.host_bytes_allocated - s->stats.host_bytes_freed;
  s->stats.host_bytes_peak = std::max(s->stats.host_bytes_peak, live);
  return 0;
}

int enc_from_name(const std::string& n) {
  if (n == "plain.f32") return E_F32;
  if (n == "plain.f16") return E_F16;
  if (n == "plain.bf16") return E_BF16;
  if (n == "gguf.q4_0") return E_Q4_0;
  if (n == "gguf.q4_1") return E_Q4_1;
  if (n == "gguf.q8_0") return E_Q8_0;
  if (n == "gguf.q6_k") return E_Q6_K;
  if (n == "gguf.q4_k") return E_Q4_K;
  if (n == "gguf.q5_k") return E_Q5_K;
  if (n == "gguf.iq4_xs") return E_IQ4_XS;
  if (n == "mlx.affine.u4") return E_MLX_U4;
  return -1;
}

struct Upload {  // one byte range placed in the arena
  uint64_t arena_off = 0, length = 0;
  size_t file = 0;
  uint64_t file_off = 0;
  // strided source (a tensor-parallel slice of every row): `rows` segments of `seg` bytes,
  // `stride` bytes apart in the file, packed back to back in the arena; rows == 0: contiguous
  uint64_t rows = 0, seg = 0, stride = 0;
};

struct ParamDesc {
  int enc = -1, aux = E_BF16, group = 0;
  std::vector<int64_t> shape;
  std::map<std::string, Upload> comps;  // component name -> upload
  std::map<std::string, std::array<uint64_t, 3>> strided;  // component -> rows, seg bytes, row stride
};

int read_range(int fd, uint64_t off, uint64_t len, uint8_t* dst_dev, uint8_t* staging,
               size_t staging_bytes, const char* path) {
  uint64_t done = 0;
  while (done < len) {
    size_t n = (size_t)std::min<uint64_t>(staging_bytes, len - done);
    size_t got = 0;
    while (got < n) {
      ssize_t r = pread(fd, staging + got, n - got, (off_t)(off + done + got));
      if (r < 0 && errno == EINTR) continue;
      DYN_CHECK(r > 0, "short read of %s at offset %llu (%s)", path,
                (unsigned long long)(off + done + got), r == 0 ? "end of file" : strerror(errno));
      got += (size_t)r;
    }
    DYN_CUDA(cudaMemcpy(dst_dev + done, staging, n, cudaMemcpyHostToDevice));
    done += n;
  }
  return 0;
}

// A strided range (one span of every row): whole groups of rows are read in one piece and a
// 2-D copy packs their spans into the arena; the bytes themselves are uploaded unchanged.
int read_strided(int fd, const Upload& u, uint8_t* dst_dev, uint8_t* staging, size_t staging_bytes,
                 const char* path) {
  DYN_CHECK(u.stride <= staging_bytes, "row stride %llu of a strided range exceeds the staging buffer",
            (unsigned long long)u.stride);
  const uint64_t per = std::max<uint64_t>(1, staging_bytes / u.stride);
  for (uint64_t r0 = 0; r0 < u.rows; r0 += per) {
    const uint64_t n = std::min<uint64_t>(per, u.rows - r0);
    const uint64_t bytes = (n - 1) * u.stride + u.seg, off = u.file_off + r0 * u.stride;
    size_t got = 0;
    while (got < bytes) {
      ssize_t r = pread(fd, staging + got, bytes - got, (off_t)(off + got));
      if (r < 0 && errno == EINTR) continue;
      DYN_CHECK(r > 0, "short read of %s at offset %llu (%s)", path, (unsigned long long)(off + got),
                r == 0 ? "end of file" : strerror(errno));
      got += (size_t)r;
    }
    DYN_CUDA(cudaMemcpy2D(dst_dev + r0 * u.seg, u.seg, staging, u.stride, u.seg, n, cudaMemcpyHostToDevice));
  }
  return 0;
}

int bind_linear(const std::map<std::string, ParamDesc>& params, const uint8_t* arena,
                const std::string& name, int64_t rows, int64_t cols, WRef* out) {
  auto it = params.find(name);
  DYN_CHECK(it != params.end(), "model descriptor lacks parameter `%s`", name.c_str());
  const ParamDesc& p = it->second;
  DYN_CHECK(p.shape.size() == 2 && p.shape[0] == rows && p.shape[1] == cols,
            "parameter `%s` has the wrong logical shape (expected [%lld, %lld])", name.c_str(),
            (long long)rows, (long long)cols);
  out->enc = p.enc;
  out->rows = rows;
  out->cols = cols;
  int unit = std::max(4, enc_block_elems(p.enc));
  DYN_CHECK(cols % unit == 0, "parameter `%s`: cols %lld not a multiple of %d", name.c_str(),
            (long long)cols, unit);
  const char* main_comp = p.enc == E_MLX_U4 ? "packed" : "data";
  auto c = p.comps.find(main_comp);
  DYN_CHECK(c != p.comps.end(), "no byte range given for `weights::%s::%s`", name.c_str(), main_comp);
  const uint64_t expect = (uint64_t)rows * (uint64_t)enc_row_bytes(p.enc, cols);
  DYN_CHECK(c->second.length == expect,
            "byte range of `%s` is %llu bytes, encoding and shape need %llu", name.c_str(),
            (unsigned long long)c->second.length, (unsigned long long)expect);
  out->data = arena + c->second.arena_off;
  if (p.enc == E_MLX_U4) {
    DYN_CHECK(p.group >= 8 && p.group % 8 == 0 && cols % p.group == 0,
              "parameter `%s`: MLX group %d does not divide cols", name.c_str(), p.group);
    auto sc = p.comps.find("scales"), bi = p.comps.find("biases");
    DYN_CHECK(sc != p.comps.end() && bi != p.comps.end(),
              "parameter `%s` lacks scales/biases ranges", name.c_str());
    const uint64_t aux_expect = (uint64_t)rows * (cols / p.group) * aux_elem_bytes(p.aux);
    DYN_CHECK(sc->second.length == aux_expect && bi->second.length == aux_expect,
              "parameter `%s`: scales/biases byte length mismatch", name.c_str());
    out->scales = arena + sc->second.arena_off;
    out->biases = arena + bi->second.arena_off;
    out->aux = p.aux;
    out->group = p.group;
  }
  return 0;
}

int bind_norm(const std::map<std::string, ParamDesc>& params, const uint8_t* arena,
              const std::string& name, int64_t width, bool required, NormW* out) {
  auto it = params.find(name);
  if (it == params.end()) {
    DYN_CHECK(!required, "model descriptor lacks parameter `%s`", name.c_str());
    return 0;
  }
  const ParamDesc& p = it->second;
  DYN_CHECK(p.enc == E_F32 || p.enc == E_F16 || p.enc == E_BF16,
            "norm weight `%s` must be a plain float type", name.c_str());
  DYN_CHECK(p.shape.size() == 1 && p.shape[0] == width, "norm weight `%s` has the wrong shape",
            name.c_str());
  auto c = p.comps.find("data");
  DYN_CHECK(c != p.comps.end(), "no byte range given for `weights::%s::data`", name.c_str());
  DYN_CHECK(c->second.length == (uint64_t)width * aux_elem_bytes(p.enc),
            "norm weight `%s` byte length mismatch", name.c_str());
  out->ptr = arena + c->second.arena_off;
  out->type = p.enc;
  out->bytes = c->second.length;
  return 0;
}

void destroy_graphs(Session* s) {
  if (s->decode_graph) cudaGraphExecDestroy(s->decode_graph);
  if (s->loop_graph) cudaGraphExecDestroy(s->loop_graph);
  s->decode_graph = s->loop_graph = nullptr;
  for (auto& kv : s->batch_graphs)
    if (kv.second.first) cudaGraphExecDestroy(kv.second.first);
  s->batch_graphs.clear();
}

// Device-side greedy feedback: the produced token becomes the next input, the
// position advances, and the token is appended to the history buffer.
__global__ void advance_kernel(int64_t* tokens, int64_t* row_pos, const int64_t* out_token,
                               int64_t* hist, int64_t* hist_count, int64_t hist_cap) {
  const int64_t t = out_token[0];
  tokens[0] = t;
  row_pos[0] += 1;
  const int64_t c = hist_count[0];
  if (c < hist_cap) hist[c] = t;
  hist_count[0] = c + 1;
}

// A row-parallel product (o_proj, down) under tensor parallelism: every rank multiplies its span
// of the reduction dimension and the sum over ranks plus the residual lands in `hidden` on every
// rank (the same bits everywhere, so the ranks stay in step). With peer memory attached the
// partial rows go to this rank's exchange slot and one kernel sums all ranks' slots and applies
// the following RMSNorm (`norm` -> xn; *fused tells the caller). Otherwise rank 0 adds the
// residual and an all-reduce sums.
int tp_row_parallel(Session* s, const WRef& w, const float* x, int64_t rows, int slot, const NormW* norm,
                    bool* fused, cudaStream_t st) {
  *fused = false;
  const ModelCfg& c = s->cfg;
  if (s->peer.attached) {
    float* part = reinterpret_cast<float*>(s->peer.base[c.tp_rank]) + (size_t)slot * s->peer.max_rows * c.hidden;
    if (launch_linear(w, x, E_F32, rows, part, nullptr, st)) return 1;
    *fused = norm != nullptr;
    return launch_tp_exchange(s->peer, slot, rows, c.hidden, s->hidden, norm ? s->xn : nullptr,
                              norm ? norm->ptr : nullptr, norm ? norm->type : E_F32, c.eps, st);
  }
  DYN_CHECK(s->tp_comm != nullptr,
            "tensor-parallel session: dyninfer_cuda_session_tp_init has not been called");
  const size_t n = (size_t)rows * c.hidden;
  if (c.tp_rank == 0) {
    if (launch_linear(w, x, E_F32, rows, s->hidden, s->hidden, st)) return 1;
    return tp_all_reduce_sum(s->tp_comm, s->hidden, s->hidden, n, st);
  }
  if (launch_linear(w, x, E_F32, rows, s->tp_part, nullptr, st)) return 1;
  return tp_all_reduce_sum(s->tp_comm, s->tp_part, s->hidden, n, st);
}

// Enqueue the whole decoder for `rows` rows whose tokens / positions / slots are
// already in device memory; logits and argmax come from row `logits_row`.
int enqueue_forward(Session* s, int64_t rows, int64_t logits_row, bool all_rows = false,
                    int64_t chunk_start = -1, int64_t chunk_slot = 0) {
  const ModelCfg& c = s->cfg;
  cudaStream_t st = s->stream;
  const bool tp = c.tp_world > 1;
  const int64_t H = c.hidden, qd = (int64_t)c.heads * c.head_dim,
                kvd = (int64_t)c.kv_heads * c.head_dim;
  const int64_t cap = (int64_t)(s->pages * s->page_size);
  const size_t layer_stride = (size_t)c.batch * c.kv_heads * cap * c.head_dim * s->kv_elem;
  if (launch_gather(s->embed, s->tokens_dev, rows, s->hidden, st)) return 1;
  bool normed = false;  // xn already holds this layer's attn_norm rows (fused into the last exchange)
  // One row: the q / k / v and [gate; up] products (local also under tensor parallelism), when their K is
  // split over CTAs, leave the
  // addition of the K-slice sums to the kernel that consumes the result (QKV prepare, SwiGLU): three
  // launches fewer per layer (8B mixed: 3.24 -> 2.90 ms per step). The sums wait in the session's scratch,
  // held until that kernel is enqueued. The same for o / down with residual + RMSNorm in one single-block
  // kernel was slower (3.39 ms): their reductions stay separate, multi-block launches.
  const bool fuse1 = rows == 1;
  auto linear_deferred = [&](const WRef& w, const float* x, float* y, Deferred* d) -> int {
    DeferScope scope(d);
    if (launch_linear(w, x, E_F32, 1, y, nullptr, st)) return 1;
    if (d->S) thread_scratch_hold(d->ws_bytes);
    return 0;
  };
  // Many rows on one GPU (prefill chunks), every product on the dequant GEMM: RMSNorm
  // and SwiGLU write the GEMM's activation operand themselves (f16 rows + inverse scales) and the K-split
  // sums of o / down are added inside the following residual + RMSNorm kernel, those of a single [q; k; v]
  // product inside QKV prepare -- 10 instead of 16 launches
  // per layer and five passes over the activations fewer, with the same bits as the separate kernels.
  // (one block per row: with few rows -- batched decode steps -- the separate multi-block kernels are faster:
  // 32 rows of the 32B shape 13.5 against 14.4 ms per step)
  bool fuse_n = rows >= 64 && !tp && s->xh && H <= 8192;
  for (int l = 0; l < c.layers && fuse_n; l++) {
    const LayerW& L = s->layers[l];
    const WRef* ws[8] = {L.qkv_parts >= 2 ? &L.qkv : &L.q, L.qkv_parts >= 2 ? nullptr : &L.k, L.qkv_parts == 3 ? nullptr : &L.v,
                         &L.o, L.gate_up.data ? &L.gate_up : &L.gate, L.gate_up.data ? nullptr : &L.up, &L.down, nullptr};
    for (const WRef* w : ws)
      if (w && !(dqgemm_tc_takes(*w, rows) && dqgemm_tc_padded_rows(*w, rows) <= s->xh_rows)) fuse_n = false;
    if (H > s->xh_cols || c.inter > s->xh_cols) fuse_n = false;
  }
  bool xh_ready = false;  // xh already holds this layer's normalised rows (written by the layer before)
  auto gemm = [&](const WRef& w, const float* x, bool prepared, float* y, const float* residual, TgIo* io) -> int {
    TgIo local;
    if (!io) io = &local;
    if (prepared) io->xh = s->xh, io->inv_s = s->xinv, io->rows_alloc = s->xh_rows;
    bool handled = false;
    if (launch_dqgemm_tc(w, x, E_F32, rows, y, residual, st, &handled, io)) return 1;
    DYN_CHECK(handled, "dequant GEMM refused a product it had accepted");
    return 0;
  };
  for (int l = 0; l < c.layers; l++) {
    const LayerW& L = s->layers[l];
    if (fuse_n) {
      if (!xh_ready && launch_norm_prepare(s->hidden, nullptr, 0, nullptr, nullptr, L.attn_norm.ptr, L.attn_norm.type, rows, H,
                                           c.eps, s->xh, s->xinv, st))
        return 1;
      xh_ready = false;
      float *qp = s->q, *kp = s->k, *vp = s->v;
      int64_t ldq = 0, ldk = 0, ldv = 0;
      TgIo io_q;  // one [q; k; v] product: its K-split sums are added inside QKV prepare
      if (L.qkv_parts >= 2) {
        qp = s->qkv1, kp = qp + qd;
        ldq = ldk = L.qkv_parts == 3 ? qd + 2 * kvd : qd + kvd;
        if (L.qkv_parts == 3) io_q.partial = s->gpart, io_q.partial_bytes = s->gpart_bytes;
        if (gemm(L.qkv, nullptr, true, qp, nullptr, &io_q)) return 1;
        if (L.qkv_parts == 3) vp = kp + kvd, ldv = ldq;
        else if (gemm(L.v, nullptr, true, vp, nullptr, nullptr)) return 1;
      } else if (gemm(L.q, nullptr, true, qp, nullptr, nullptr) || gemm(L.k, nullptr, true, kp, nullptr, nullptr) ||
                 gemm(L.v, nullptr, true, vp, nullptr, nullptr)) {
        return 1;
      }
      QkvPrepArgs pa{};
      pa.q = qp, pa.k = kp, pa.v = vp;
      pa.kcache = s->kcache + (size_t)l * layer_stride;
      pa.vcache = s->vcache + (size_t)l * layer_stride;
      pa.q_norm_w = L.q_norm.ptr, pa.k_norm_w = L.k_norm.ptr, pa.norm_w_type = L.q_norm.type;
      pa.row_pos = s->row_pos_dev, pa.row_seq = s->row_seq_dev, pa.base_pos = 0;
      pa.rows = rows, pa.nh = c.heads, pa.nkv = c.kv_heads, pa.d = c.head_dim, pa.cap = cap;
      pa.kv_type = s->kv_type, pa.has_norm = c.qk_norm ? 1 : 0, pa.has_rope = c.rope ? 1 : 0;
      pa.eps = c.eps;
      pa.ldq = ldq, pa.ldk = ldk, pa.ldv = ldv;
      if (io_q.splits > 1) {
        DeferredCols dc;
        dc.partial = s->gpart, dc.S = io_q.splits, dc.N = qd + 2 * kvd, dc.rows = rows;
        pa.dq = dc, pa.dk = dc, pa.dv = dc;
        pa.dk.col = qd, pa.dv.col = qd + kvd;
      }
      if (launch_qkv_prepare(pa, s->freq, st)) return 1;
      AttnArgs aa{};
      aa.q = qp, aa.kcache = pa.kcache, aa.vcache = pa.vcache;
      aa.row_pos = s->row_pos_dev, aa.row_seq = s->row_seq_dev, aa.base_pos = 0;
      aa.ctx = s->ctx;
      aa.rows = rows, aa.nh = c.heads, aa.nkv = c.kv_heads, aa.d = c.head_dim, aa.cap = cap;
      aa.kv_type = s->kv_type;
      aa.ldq = ldq;
      aa.uniform_base = chunk_start, aa.uniform_seq = chunk_slot;
      if (launch_attention(aa, st)) return 1;
      // o: hidden += W ctx, then the FFN norm straight into the GEMM's operand
      TgIo io_o;
      io_o.partial = s->gpart, io_o.partial_bytes = s->gpart_bytes;
      if (gemm(L.o, s->ctx, false, s->hidden, s->hidden, &io_o)) return 1;
      if (io_o.splits > 1 ? launch_norm_prepare(nullptr, s->gpart, io_o.splits, s->hidden, s->hidden, L.ffn_norm.ptr,
                                                L.ffn_norm.type, rows, H, c.eps, s->xh, s->xinv, st)
                          : launch_norm_prepare(s->hidden, nullptr, 0, nullptr, nullptr, L.ffn_norm.ptr, L.ffn_norm.type, rows,
                                                H, c.eps, s->xh, s->xinv, st))
        return 1;
      bool act_prepared = false;
      if (L.gate_up.data) {
        if (gemm(L.gate_up, nullptr, true, s->gu1, nullptr, nullptr) ||
            launch_silu_prepare(s->gu1, rows, c.inter, s->xh, s->xinv, st))
          return 1;
        act_prepared = true;
      } else {
        if (gemm(L.gate, nullptr, true, s->act, nullptr, nullptr) || gemm(L.up, nullptr, true, s->up, nullptr, nullptr) ||
            launch_silu_mul(s->act, s->up, rows * c.inter, s->act, st))
          return 1;
      }
      // down: hidden += W act; with another layer to come, its attention norm rides on the addition
      TgIo io_d;
      if (l + 1 < c.layers) io_d.partial = s->gpart, io_d.partial_bytes = s->gpart_bytes;
      if (gemm(L.down, act_prepared ? nullptr : s->act, act_prepared, s->hidden, s->hidden, &io_d)) return 1;
      if (io_d.splits > 1) {
        const NormW& nw = s->layers[l + 1].attn_norm;
        if (launch_norm_prepare(nullptr, s->gpart, io_d.splits, s->hidden, s->hidden, nw.ptr, nw.type, rows, H, c.eps, s->xh,
                                s->xinv, st))
          return 1;
        xh_ready = true;
      }
      continue;
    }
    if (!normed &&
        launch_rms_norm(s->hidden, L.attn_norm.ptr, L.attn_norm.type, rows, H, c.eps, s->xn, st))
      return 1;
    // matrices laid back to back in the arena are one product into rows of [q | k | v] (or of
    // [q | k], v apart): one activation pass and one launch instead of three
    float *qp = s->q, *kp = s->k, *vp = s->v;
    int64_t ldq = 0, ldk = 0, ldv = 0;
    Deferred dq, dk, dv;
    int64_t colk = 0, colv = 0;  // where k and v start among dq's / dk's rows
    if (fuse1 && L.qkv_parts >= 2) {
      qp = s->qkv1, kp = qp + qd;
      if (linear_deferred(L.qkv, s->xn, qp, &dq)) return 1;
      dk = dq, colk = qd;
      if (L.qkv_parts == 3) {
        vp = kp + kvd, dv = dq, colv = qd + kvd;
      } else if (linear_deferred(L.v, s->xn, vp, &dv)) {
        return 1;
      }
    } else if (fuse1) {
      if (linear_deferred(L.q, s->xn, qp, &dq) || linear_deferred(L.k, s->xn, kp, &dk) ||
          linear_deferred(L.v, s->xn, vp, &dv))
        return 1;
    } else if (L.qkv_parts >= 2) {
      qp = s->qkv1, kp = qp + qd;
      ldq = ldk = L.qkv_parts == 3 ? qd + 2 * kvd : qd + kvd;
      if (launch_linear(L.qkv, s->xn, E_F32, rows, qp, nullptr, st)) return 1;
      if (L.qkv_parts == 3) vp = kp + kvd, ldv = ldq;
      else if (launch_linear(L.v, s->xn, E_F32, rows, vp, nullptr, st)) return 1;
    } else {
      if (launch_linear(L.q, s->xn, E_F32, rows, qp, nullptr, st)) return 1;
      if (launch_linear(L.k, s->xn, E_F32, rows, kp, nullptr, st)) return 1;
      if (launch_linear(L.v, s->xn, E_F32, rows, vp, nullptr, st)) return 1;
    }
    QkvPrepArgs pa{};
    pa.q = qp, pa.k = kp, pa.v = vp;
    pa.kcache = s->kcache + (size_t)l * layer_stride;
    pa.vcache = s->vcache + (size_t)l * layer_stride;
    pa.q_norm_w = L.q_norm.ptr, pa.k_norm_w = L.k_norm.ptr, pa.norm_w_type = L.q_norm.type;
    pa.row_pos = s->row_pos_dev, pa.row_seq = s->row_seq_dev, pa.base_pos = 0;
    pa.rows = rows, pa.nh = c.heads, pa.nkv = c.kv_heads, pa.d = c.head_dim, pa.cap = cap;
    pa.kv_type = s->kv_type, pa.has_norm = c.qk_norm ? 1 : 0, pa.has_rope = c.rope ? 1 : 0;
    pa.eps = c.eps;
    pa.ldq = ldq, pa.ldk = ldk, pa.ldv = ldv;
    pa.dq = deferred_cols(dq, 0), pa.dk = deferred_cols(dk, colk), pa.dv = deferred_cols(dv, colv);
    if (launch_qkv_prepare(pa, s->freq, st)) return 1;
    thread_scratch_release_all();
    AttnArgs aa{};
    aa.q = qp, aa.kcache = pa.kcache, aa.vcache = pa.vcache;
    aa.row_pos = s->row_pos_dev, aa.row_seq = s->row_seq_dev, aa.base_pos = 0;
    aa.ctx = s->ctx;
    aa.rows = rows, aa.nh = c.heads, aa.nkv = c.kv_heads, aa.d = c.head_dim, aa.cap = cap;
    aa.kv_type = s->kv_type;
    aa.ldq = ldq;
    aa.uniform_base = chunk_start, aa.uniform_seq = chunk_slot;  // a prefill chunk: consecutive positions
    if (launch_attention(aa, st)) return 1;
    bool ffn_normed = false;
    if (tp ? tp_row_parallel(s, L.o, s->ctx, rows, 0, &L.ffn_norm, &ffn_normed, st)
           : launch_linear(L.o, s->ctx, E_F32, rows, s->hidden, s->hidden, st))
      return 1;
    if (!ffn_normed &&
        launch_rms_norm(s->hidden, L.ffn_norm.ptr, L.ffn_norm.type, rows, H, c.eps, s->xn, st))
      return 1;
    // one row: the column-split GEMVs run at ~3x the fused scalar kernel's bandwidth, which more than
    // pays for the separate activation launch
    const bool fast_gemv = (rows == 1 && gemv_cs_workspace_bytes(L.gate, 1) && gemv_cs_workspace_bytes(L.up, 1)) ||
                           (rows <= 4 && gemv_mma_workspace_bytes(L.gate, E_F32, (int)rows) &&
                            gemv_mma_workspace_bytes(L.up, E_F32, (int)rows));
    if (fuse1 && L.gate_up.data && gemv_cs_workspace_bytes(L.gate_up, 1) != 0) {
      Deferred d_gu;
      if (linear_deferred(L.gate_up, s->xn, s->gu1, &d_gu) ||
          launch_silu_mul_deferred(d_gu, s->gu1, c.inter, s->act, st))
        return 1;
      thread_scratch_release_all();
    } else if (L.gate_up.data && (rows == 1 ? gemv_cs_workspace_bytes(L.gate_up, 1) != 0 : rows > 4 || fast_gemv)) {
      // [gate; up] as one product into rows of [gate | up], then the activation
      if (launch_linear(L.gate_up, s->xn, E_F32, rows, s->gu1, nullptr, st)) return 1;
      if (launch_silu_mul_rows(s->gu1, rows, c.inter, s->act, st)) return 1;
    } else if (L.gate.enc == L.up.enc && rows <= 4 && !fast_gemv) {
      if (launch_linear_swiglu(L.gate, L.up, s->xn, rows, s->act, st)) return 1;
    } else {
      // many rows (tensor-core GEMM) or mixed encodings: two products, then the activation
      if (launch_linear(L.gate, s->xn, E_F32, rows, s->act, nullptr, st)) return 1;
      if (launch_linear(L.up, s->xn, E_F32, rows, s->up, nullptr, st)) return 1;
      if (launch_silu_mul(s->act, s->up, rows * c.inter, s->act, st)) return 1;
    }
    normed = false;
    if (tp ? tp_row_parallel(s, L.down, s->act, rows, 1,
                             l + 1 < c.layers ? &s->layers[l + 1].attn_norm : nullptr, &normed, st)
           : launch_linear(L.down, s->act, E_F32, rows, s->hidden, s->hidden, st))
      return 1;
  }
  if (all_rows) {
    // batched decode: every row is the last token of its own sequence
    if (launch_rms_norm(s->hidden, s->out_norm.ptr, s->out_norm.type, rows, H, c.eps, s->xn, st)) return 1;
    if (tp) {
      // every rank scores its rows of the vocabulary; the slices are gathered as
      // [rank][row][lm_rows] and the first strict maximum is taken over all of them
      if (launch_linear(s->lm_head, s->xn, E_F32, rows, s->tp_logits, nullptr, st)) return 1;
      if (tp_all_gather(s->tp_comm, s->tp_logits, s->tp_gather, (size_t)rows * c.lm_rows, st)) return 1;
      return launch_argmax_rows_sharded(s->tp_gather, rows, c.lm_rows, c.tp_world, s->batch_tokens_dev, st);
    }
    if (launch_linear(s->lm_head, s->xn, E_F32, rows, s->batch_logits, nullptr, st)) return 1;
    if (launch_argmax_rows(s->batch_logits, rows, c.vocab, s->batch_tokens_dev, st)) return 1;
    return 0;
  }
  // final norm of the one row that feeds the lm_head (dense_decoder.rs:1573-1615)
  if (launch_rms_norm(s->hidden + logits_row * H, s->out_norm.ptr, s->out_norm.type, 1, H, c.eps,
                      s->xn, st))
    return 1;
  if (tp) {
    // one row: the gathered slices are the logits in vocabulary order
    if (launch_linear(s->lm_head, s->xn, E_F32, 1, s->tp_logits, nullptr, st)) return 1;
    if (tp_all_gather(s->tp_comm, s->tp_logits, s->logits, (size_t)c.lm_rows, st)) return 1;
  } else if (launch_linear(s->lm_head, s->xn, E_F32, 1, s->logits, nullptr, st)) {
    return 1;
  }
  if (launch_argmax(s->logits, c.vocab, s->out_token_dev, s->argmax_scratch, st)) return 1;
  (void)kvd;
  return 0;
}

// The exchange steps of a `rows`-row forward, run once on scratch data outside any capture, so
// that the communicator sets up whatever these sizes need before they are recorded into a graph.
int tp_warm_collectives(Session* s, int64_t rows, bool all_rows) {
  const ModelCfg& c = s->cfg;
  if (c.tp_world <= 1) return 0;
  DYN_CHECK(s->tp_comm != nullptr,
            "tensor-parallel session: dyninfer_cuda_session_tp_init has not been called");
  const size_t n = (size_t)rows * c.hidden;
  DYN_CUDA(cudaMemsetAsync(s->tp_part, 0, n * 4, s->stream));
  if (tp_all_reduce_sum(s->tp_comm, s->tp_part, s->tp_part, n, s->stream)) return 1;
  if (all_rows ? tp_all_gather(s->tp_comm, s->tp_logits, s->tp_gather, (size_t)rows * c.lm_rows, s->stream)
               : tp_all_gather(s->tp_comm, s->tp_logits, s->logits, (size_t)c.lm_rows, s->stream))
    return 1;
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  return 0;
}

int capture(Session* s, bool loop, cudaGraphExec_t* out, uint64_t* nodes) {
  cudaGraph_t g = nullptr;
  uint64_t before = s->launches;
  if (tp_warm_collectives(s, 1, false)) return 1;
  DYN_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
  int rc = 0;
  if (!loop) {
    if (cudaMemcpyAsync(s->tokens_dev, s->stage_host, 8, cudaMemcpyHostToDevice, s->stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(s->row_pos_dev, s->stage_host + 1, 8, cudaMemcpyHostToDevice, s->stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(s->row_seq_dev, s->stage_host + 2, 8, cudaMemcpyHostToDevice, s->stream) !=
            cudaSuccess)
      rc = 1;
  }
  if (!rc) rc = enqueue_forward(s, 1, 0);
  if (!rc) {
    if (loop) {
      advance_kernel<<<1, 1, 0, s->stream>>>(s->tokens_dev, s->row_pos_dev, s->out_token_dev,
                                             s->hist_dev, s->hist_count_dev, (int64_t)s->hist_cap);
      count_launch();
    } else if (cudaMemcpyAsync(s->stage_host + 3, s->out_token_dev, 8, cudaMemcpyDeviceToHost,
                               s->stream) != cudaSuccess) {
      rc = 1;
    }
  }
  cudaError_t e = cudaStreamEndCapture(s->stream, &g);
  if (rc) {
    if (g) cudaGraphDestroy(g);
    std::string keep = dyninfer_cuda_last_error();
    set_error("graph capture failed: %s", keep.c_str());
    return 1;
  }
  DYN_CUDA(e);
  *nodes = s->launches - before;
  s->launches = before;  // capture enqueues nothing; replays are counted per launch
  cudaError_t ie = cudaGraphInstantiate(out, g, 0);
  cudaGraphDestroy(g);
  DYN_CUDA(ie);
  return 0;
}

// Batched step for `rows` sequences as a graph: tokens / positions / slots are read from the device
// buffers the caller fills before every replay.
int capture_batch(Session* s, int64_t rows, cudaGraphExec_t* out, uint64_t* nodes) {
  cudaGraph_t g = nullptr;
  const uint64_t before = s->launches;
  if (tp_warm_collectives(s, rows, true)) return 1;
  DYN_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
  const int rc = enqueue_forward(s, rows, 0, true);
  cudaError_t e = cudaStreamEndCapture(s->stream, &g);
  if (rc) {
    if (g) cudaGraphDestroy(g);
    std::string keep = dyninfer_cuda_last_error();
    set_error("graph capture of the batched step failed: %s", keep.c_str());
    return 1;
  }
  DYN_CUDA(e);
  *nodes = s->launches - before;
  s->launches = before;
  cudaError_t ie = cudaGraphInstantiate(out, g, 0);
  cudaGraphDestroy(g);
  DYN_CUDA(ie);
  return 0;
}

int ensure_hist(Session* s, size_t steps) {
  if (steps <= s->hist_cap) return 0;
  if (s->hist_dev) dev_free(s, s->hist_dev, s->hist_cap * 8);
  s->hist_dev = nullptr;
  size_t cap = std::max<size_t>(steps, 4096);
  if (dev_alloc(s, (void**)&s->hist_dev, cap * 8)) return 1;
  s->hist_cap = cap;
  if (s->loop_graph) {
    cudaGraphExecDestroy(s->loop_graph);
    s->loop_graph = nullptr;
  }
  return 0;
}

int xl_for_encoding_host(int enc) {
  return (enc == E_Q4_0 || enc == E_Q4_1) ? 0 : (enc == E_MLX_U4 ? 1 : 2);
}

void fill_mega_args(Session* s, MegaArgs* a, int advance, int steps = 1) {
  const ModelCfg& c = s->cfg;
  a->layers = c.layers, a->H = c.hidden, a->I = c.inter, a->V = c.vocab;
  a->nh = c.heads, a->nkv = c.kv_heads, a->d = c.head_dim;
  a->eps = c.eps;
  a->has_norm = c.qk_norm ? 1 : 0, a->has_rope = c.rope ? 1 : 0;
  a->L = s->mega_layers;
  a->embed = s->embed, a->lm_head = s->lm_head;
  a->out_norm = s->out_norm.ptr, a->out_norm_type = s->out_norm.type;
  a->logits = s->logits;
  a->ll_hidden[0] = s->ll_dev + s->ll_off[0], a->ll_hidden[1] = s->ll_dev + s->ll_off[1];
  a->ll_qkv = s->ll_dev + s->ll_off[2], a->ll_ctx = s->ll_dev + s->ll_off[3];
  a->ll_part = s->ll_dev + s->ll_off[4], a->ll_act = s->ll_dev + s->ll_off[5];
  a->ll_amax = s->ll_dev + s->ll_off[6];
  // every launch gets epochs of its own; the buffers start zeroed, so epoch 0 is never used
  const unsigned span = (unsigned)steps * ((unsigned)c.layers + 2u);
  if (s->mega_epoch > 0xffffffffu - 2u * span) s->mega_epoch = 0;
  a->epoch_base = s->mega_epoch;
  s->mega_epoch += span;
  a->steps = steps;
  {
    const char* oe = getenv("DYNINFER_CUDA_MEGA_OPTS");
    a->opts = oe ? atoi(oe) : 0;
  }
  a->kcache = s->kcache, a->vcache = s->vcache;
  a->cap = (int64_t)(s->pages * s->page_size);
  a->layer_stride = (uint64_t)c.batch * c.kv_heads * (uint64_t)a->cap * c.head_dim * s->kv_elem;
  a->kv_type = s->kv_type;
  a->io = s->io_dev;
  a->inline_io = 0, a->in_token = a->in_pos = a->in_seq = 0, a->out_host = nullptr;
  a->hist = s->hist_dev, a->hist_count = s->hist_count_dev, a->hist_cap = (int64_t)s->hist_cap;
  a->advance = advance;
  a->error = reinterpret_cast<int*>(s->io_dev + 4);
  a->max_split = s->mega_max_split;
  // phase timing reads the global timer thousands of times per launch on CTA 0 and slows the
  // whole grid down; it is off unless DYNINFER_CUDA_PROFILE=1
  {
    const char* pe = getenv("DYNINFER_CUDA_PROFILE");
    a->prof = (pe && pe[0] == '1') ? s->prof_dev : nullptr;
    a->trace = s->trace_dev;
  }
  a->prog = s->prog_dev, a->lay = s->mega_lay;
  a->nslot = s->mega_nslot, a->xs_floats = s->mega_xs;
  a->ft = s->freq;
}

// A bounded wait inside the kernel gave up: report it and clear the word.
int mega_check_error(Session* s, int64_t word) {
  if ((int)word == 0) return 0;
  cudaMemsetAsync(s->io_dev + 4, 0, 8, s->stream);
  cudaStreamSynchronize(s->stream);
  set_error("persistent decode kernel: a bounded wait expired (code %d: 3 weight ring full-wait, "
            "4 ring empty-wait, 7 program copy, 8 hand-off vector never arrived); the step's results "
            "are invalid", (int)word);
  return 1;
}

// After the stream has drained: did a wait of the peer exchange run out during this call?
int tp_check_error(Session* s) {
  if (!s->peer.attached || !*s->peer.error_host) return 0;
  const int which = *s->peer.error_host - 1;
  *s->peer.error_host = 0;
  set_error("tensor-parallel exchange: rank %d did not arrive within the wait limit (rank %d gave up); "
            "the step's results are invalid", which, s->cfg.tp_rank);
  return 1;
}

struct CounterScope {  // routes count_launch() and product scratch to this session for one call
  explicit CounterScope(Session* s) {
    set_launch_counter(&s->launches);
    set_thread_scratch(s->scratch, s->scratch_bytes);
  }
  ~CounterScope() {
    set_launch_counter(nullptr);
    set_thread_scratch(nullptr, 0);
  }
};

}  // namespace

extern "C" {

int dyninfer_cuda_session_create_with_file_params(
    const char* device_uri, const char* model_desc_json,
    const dyninfer_cuda_parameter_file_t* files, size_t file_count,
    const dyninfer_cuda_file_param_t* params, size_t param_count,
    dyninfer_cuda_session_t** out_session) {
  DYN_CHECK(out_session != nullptr, "out_session is NULL");
  *out_session = nullptr;
  DYN_CHECK(model_desc_json != nullptr, "model_desc_json is NULL");
  DYN_CHECK(file_count == 0 || files != nullptr, "files is NULL");
  DYN_CHECK(param_count == 0 || params != nullptr, "params is NULL");

  int device = 0;
  {
    std::string uri = device_uri ? device_uri : "cuda";
    if (uri.empty()) uri = "cuda";
    DYN_CHECK(uri.compare(0, 4, "cuda") == 0,
              "device `%s` is not a cuda device; this library has no other backend and no CPU fallback",
              uri.c_str());
    if (uri.size() > 4) {
      DYN_CHECK(uri[4] == ':' && uri.size() > 5, "malformed device uri `%s`", uri.c_str());
      char* end = nullptr;
      long v = strtol(uri.c_str() + 5, &end, 10);
      DYN_CHECK(end && *end == 0 && v >= 0, "malformed device ordinal in `%s`", uri.c_str());
      device = (int)v;
    }
  }

  Json desc;
  {
    std::string err;
    JsonParser jp(model_desc_json);
    DYN_CHECK(jp.parse(&desc, &err) && desc.kind == Json::Obj, "model descriptor: %s", err.c_str());
  }
  ModelCfg cfg;
  cfg.layers = (int)desc.number("layers", 0);
  cfg.hidden = (int)desc.number("hidden", 0);
  cfg.inter = (int)desc.number("intermediate", 0);
  cfg.heads = (int)desc.number("heads", 0);
  cfg.kv_heads = (int)desc.number("kv_heads", cfg.heads);
  cfg.head_dim = (int)desc.number("head_dim", cfg.heads ? cfg.hidden / cfg.heads : 0);
  cfg.vocab = (int)desc.number("vocab", 0);
  cfg.eps = (float)desc.number("eps", 1e-6);
  cfg.theta = (float)desc.number("theta", 10000.0);
  cfg.qk_norm = desc.number("qk_norm", 1) != 0;
  cfg.rope = desc.number("rope", 1) != 0;
  cfg.batch = (int)desc.number("batch", 1);
  {
    std::string kvd = desc.string("kv_dtype", "bf16");
    DYN_CHECK(kvd == "bf16" || kvd == "f16" || kvd == "f32", "kv_dtype `%s` unsupported",
              kvd.c_str());
    cfg.kv2_type = kvd == "f16" ? E_F16 : E_BF16;
    std::string dk = desc.string("decode_kernel", "persistent");
    DYN_CHECK(dk == "persistent" || dk == "graph", "decode_kernel `%s` unknown (persistent | graph)",
              dk.c_str());
    cfg.persistent = dk == "persistent";
  }
  cfg.tp_world = (int)desc.number("tp_world", 1);
  cfg.tp_rank = (int)desc.number("tp_rank", 0);
  DYN_CHECK(cfg.tp_world >= 1 && cfg.tp_rank >= 0 && cfg.tp_rank < cfg.tp_world,
            "tensor-parallel rank %d outside [0, %d)", cfg.tp_rank, cfg.tp_world);
  if (cfg.tp_world > 1) cfg.persistent = false;  // the single-GPU persistent kernel has no exchange step
  DYN_CHECK(cfg.layers > 0 && cfg.hidden > 0 && cfg.inter > 0 && cfg.heads > 0 &&
                cfg.kv_heads > 0 && cfg.head_dim > 0 && cfg.vocab > 0 && cfg.batch > 0,
            "model descriptor lacks geometry (layers/hidden/intermediate/heads/kv_heads/head_dim/vocab)");
  DYN_CHECK(cfg.heads % cfg.kv_heads == 0, "heads %d is not a multiple of kv_heads %d", cfg.heads,
            cfg.kv_heads);
  cfg.lm_rows = (int)desc.number("lm_head_rows", cfg.vocab);
  DYN_CHECK(cfg.lm_rows > 0 && (int64_t)cfg.lm_rows * cfg.tp_world == cfg.vocab,
            "lm_head_rows %d x tp_world %d does not equal the vocabulary %d", cfg.lm_rows, cfg.tp_world,
            cfg.vocab);
  DYN_CHECK(cfg.head_dim % 2 == 0 && cfg.head_dim <= 256, "head_dim %d unsupported", cfg.head_dim);
  DYN_CHECK(cfg.hidden % 4 == 0 && cfg.inter % 4 == 0, "hidden and intermediate must be multiples of 4");

  // parameters: descriptor entries joined with their byte ranges
  std::map<std::string, ParamDesc> pd;
  const Json* jparams = desc.get("params");
  DYN_CHECK(jparams && jparams->kind == Json::Obj, "model descriptor lacks `params`");
  for (auto& kv : jparams->obj) {
    ParamDesc p;
    std::string en = kv.second.string("encoding", "");
    p.enc = enc_from_name(en);
    // strict rejection: an encoding without a registered cuda kernel is an error, never a fallback
    DYN_CHECK(p.enc >= 0, "E_KERNEL_COVERAGE: no cuda kernel for encoding `%s` (parameter `%s`)",
              en.c_str(), kv.first.c_str());
    p.group = (int)kv.second.number("group", 0);
    std::string aux = kv.second.string("aux", "");
    p.aux = aux == "plain.f32" ? E_F32 : (aux == "plain.f16" ? E_F16 : E_BF16);
    const Json* sh = kv.second.get("shape");
    DYN_CHECK(sh && sh->kind == Json::Arr, "parameter `%s` lacks a shape", kv.first.c_str());
    for (auto& d : sh->arr) p.shape.push_back((int64_t)d.num);
    if (const Json* st = kv.second.get("strided")) {
      DYN_CHECK(st->kind == Json::Obj, "parameter `%s`: `strided` must be an object", kv.first.c_str());
      for (auto& sc : st->obj) {
        DYN_CHECK(sc.second.kind == Json::Arr && sc.second.arr.size() == 3,
                  "parameter `%s`: strided component `%s` needs [rows, segment bytes, row stride]",
                  kv.first.c_str(), sc.first.c_str());
        p.strided[sc.first] = {(uint64_t)sc.second.arr[0].num, (uint64_t)sc.second.arr[1].num,
                               (uint64_t)sc.second.arr[2].num};
      }
    }
    pd.emplace(kv.first, std::move(p));
  }

  // open files, validate ranges (crates/iree-runtime/src/lib.rs:139-206)
  std::vector<int> fds(file_count, -1);
  std::vector<uint64_t> fsize(file_count, 0);
  auto close_all = [&]() {
    for (int fd : fds)
      if (fd >= 0) close(fd);
  };
  for (size_t i = 0; i < file_count; i++) {
    if (!files[i].path || (fds[i] = open(files[i].path, O_RDONLY)) < 0) {
      set_error("cannot open parameter file `%s`: %s", files[i].path ? files[i].path : "(null)",
                strerror(errno));
      close_all();
      return 1;
    }
    struct stat stt;
    fstat(fds[i], &stt);
    fsize[i] = (uint64_t)stt.st_size;
  }
  uint64_t arena_bytes = 0, weight_bytes = 0;
  int rc = 0;
  for (size_t i = 0; i < param_count && !rc; i++) {
    const dyninfer_cuda_file_param_t& fp = params[i];
    std::string key = fp.key ? fp.key : "";
    size_t a = key.find("::"), b = key.rfind("::");
    if (a == std::string::npos || b == a) {
      set_error("parameter key `%s` is not `<scope>::<name>::<component>`", key.c_str());
      rc = 1;
      break;
    }
    std::string name = key.substr(a + 2, b - a - 2), comp = key.substr(b + 2);
    auto it = pd.find(name);
    if (it == pd.end()) {
      set_error("byte range `%s` has no entry in the model descriptor", key.c_str());
      rc = 1;
    } else if (fp.source_file_index >= file_count) {
      set_error("parameter `%s`: source_file_index %zu out of range", key.c_str(),
                fp.source_file_index);
      rc = 1;
    } else if (it->second.strided.count(comp)) {
      // length = bytes uploaded = rows * segment; the file span runs to the last row's segment
      const auto& sd = it->second.strided[comp];
      // products checked for wrap-around before they are compared with the file size
      uint64_t span = 0, bytes = 0;
      const bool wraps = sd[0] == 0 || __builtin_mul_overflow(sd[0] - 1, sd[2], &span) ||
                         __builtin_add_overflow(span, sd[1], &span) ||
                         __builtin_mul_overflow(sd[0], sd[1], &bytes);
      if (wraps || sd[1] == 0 || sd[2] < sd[1] || bytes != fp.length ||
          fp.offset + span < fp.offset || fp.offset + span > fsize[fp.source_file_index]) {
        set_error("parameter `%s`: strided range (%llu rows of %llu bytes every %llu, %llu bytes in all) "
                  "is inconsistent or exceeds file size %llu", key.c_str(), (unsigned long long)sd[0],
                  (unsigned long long)sd[1], (unsigned long long)sd[2], (unsigned long long)fp.length,
                  (unsigned long long)fsize[fp.source_file_index]);
        rc = 1;
      } else if (it->second.comps.count(comp)) {
        set_error("duplicate parameter key `%s`", key.c_str());
        rc = 1;
      } else {
        Upload u;
        u.arena_off = arena_bytes;
        u.length = fp.length;
        u.file = fp.source_file_index;
        u.file_off = fp.offset;
        u.rows = sd[0], u.seg = sd[1], u.stride = sd[2];
        it->second.comps.emplace(comp, u);
        arena_bytes += (fp.length + 64 + 255) / 256 * 256;
        weight_bytes += fp.length;
      }
    } else if (fp.length == 0 || fp.offset + fp.length < fp.offset ||
               fp.offset + fp.length > fsize[fp.source_file_index]) {
      set_error("parameter `%s`: byte range [%llu, +%llu) exceeds file size %llu", key.c_str(),
                (unsigned long long)fp.offset, (unsigned long long)fp.length,
                (unsigned long long)fsize[fp.source_file_index]);
      rc = 1;
    } else if (it->second.comps.count(comp)) {
      set_error("duplicate parameter key `%s`", key.c_str());
      rc = 1;
    } else {
      Upload u;
      u.arena_off = arena_bytes;
      u.length = fp.length;
      u.file = fp.source_file_index;
      u.file_off = fp.offset;
      it->second.comps.emplace(comp, u);
      arena_bytes += (fp.length + 64 + 255) / 256 * 256;  // 64 B of readable slack per range
      weight_bytes += fp.length;
    }
  }
  if (rc) {
    close_all();
    return 1;
  }
  // Placement in the arena. The q, k, v matrices of a layer (and gate, up) that share encoding and
  // width are laid back to back: their rows then form ONE matrix [q; k; v] whose single-row
  // product is one launch instead of three (every range is still uploaded unchanged).
  {
    uint64_t cursor = 0;
    std::set<const Upload*> placed;
    auto plain_data = [&](const std::string& name) -> Upload* {
      auto it = pd.find(name);
      if (it == pd.end() || it->second.enc == E_MLX_U4 || it->second.shape.size() != 2) return nullptr;
      if (it->second.comps.size() != 1 || !it->second.comps.count("data")) return nullptr;
      return &it->second.comps["data"];
    };
    auto same_kind = [&](const std::string& a, const std::string& b) {
      const ParamDesc &pa = pd[a], &pb = pd[b];
      return pa.enc == pb.enc && pa.shape[1] == pb.shape[1];
    };
    auto place_run = [&](const std::vector<std::string>& names) {
      // the longest prefix of `names` that can be fused, at least two matrices
      std::vector<Upload*> run;
      for (const std::string& n : names) {
        Upload* u = plain_data(n);
        if (!u || u->length % 16 || (!run.empty() && !same_kind(names[0], n))) break;
        run.push_back(u);
      }
      if (run.size() < 2) return;
      for (size_t i = 0; i < run.size(); i++) {
        run[i]->arena_off = cursor;
        cursor += i + 1 < run.size() ? run[i]->length : (run[i]->length + 64 + 255) / 256 * 256;
        placed.insert(run[i]);
      }
    };
    for (int l = 0; l < cfg.layers; l++) {
      const std::string b = "blk." + std::to_string(l) + ".";
      place_run({b + "attn_q.weight", b + "attn_k.weight", b + "attn_v.weight"});
      place_run({b + "ffn_gate.weight", b + "ffn_up.weight"});
    }
    for (auto& p : pd)
      for (auto& c : p.second.comps) {
        if (placed.count(&c.second)) continue;
        c.second.arena_off = cursor;
        cursor += (c.second.length + 64 + 255) / 256 * 256;  // 64 B of readable slack per range
      }
    arena_bytes = cursor;
  }

  {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0 || device >= n) {
      set_error("cuda device %d is not available (%s); there is no CPU fallback", device,
                e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range");
      close_all();
      return 1;
    }
  }
  Session* s = new Session();
  s->device = device;
  s->cfg = cfg;
  CounterScope scope(s);
  auto fail = [&]() {
    close_all();
    std::string keep = dyninfer_cuda_last_error();
    dyninfer_cuda_session_destroy(s);
    set_error("%s", keep.c_str());
    return 1;
  };
  if (cudaSetDevice(device) != cudaSuccess ||
      cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess) {
    set_error("cannot initialise cuda device %d: %s", device, cudaGetErrorString(cudaGetLastError()));
    return fail();
  }
  cudaEventCreate(&s->ev0);
  cudaEventCreate(&s->ev1);
  if (!device_error_word()) return fail();  // allocated before any launch or stream capture
  fill_freq_table(&s->freq, cfg.head_dim, cfg.theta);
  if (dev_alloc(s, (void**)&s->arena, arena_bytes)) return fail();
  s->arena_bytes = arena_bytes;
  if (cudaMemset(s->arena, 0, arena_bytes) != cudaSuccess) {
    set_error("cudaMemset of the parameter arena failed");
    return fail();
  }
  {
    const size_t staging_bytes = 32u << 20;
    uint8_t* staging = nullptr;
    if (host_alloc(s, (void**)&staging, staging_bytes)) return fail();
    for (auto& p : pd)
      for (auto& c : p.second.comps) {
        const Upload& u = c.second;
        if (u.rows ? read_strided(fds[u.file], u, s->arena + u.arena_off, staging, staging_bytes,
                                  files[u.file].path)
                   : read_range(fds[u.file], u.file_off, u.length, s->arena + u.arena_off, staging,
                                staging_bytes, files[u.file].path)) {
          cudaFreeHost(staging);
          return fail();
        }
      }
    cudaFreeHost(staging);
    s->stats.host_bytes_freed += staging_bytes;
  }
  close_all();
  for (int& fd : fds) fd = -1;
  s->weight_bytes = weight_bytes;

  // bind tensors to roles
  const int64_t H = cfg.hidden, qd = (int64_t)cfg.heads * cfg.head_dim,
                kvd = (int64_t)cfg.kv_heads * cfg.head_dim, I = cfg.inter;
  if (bind_linear(pd, s->arena, "token_embd.weight", cfg.vocab, H, &s->embed)) return fail();
  if (pd.count("output.weight")) {
    if (bind_linear(pd, s->arena, "output.weight", cfg.lm_rows, H, &s->lm_head)) return fail();
  } else if (cfg.tp_world > 1) {
    set_error("a tensor-parallel session needs `output.weight` (this rank's rows of the lm_head)");
    return fail();
  } else {
    s->lm_head = s->embed;  // tied: same bytes (crates/dyninfer-architecture/src/naming.rs:70-96)
  }
  if (bind_norm(pd, s->arena, "output_norm.weight", H, true, &s->out_norm)) return fail();
  s->layers.resize(cfg.layers);
  uint64_t dwb = s->lm_head.total_bytes() + s->out_norm.bytes;
  for (int l = 0; l < cfg.layers; l++) {
    LayerW& L = s->layers[l];
    std::string p = "blk." + std::to_string(l) + ".";
    if (bind_norm(pd, s->arena, p + "attn_norm.weight", H, true, &L.attn_norm) ||
        bind_norm(pd, s->arena, p + "ffn_norm.weight", H, true, &L.ffn_norm) ||
        bind_norm(pd, s->arena, p + "attn_q_norm.weight", cfg.head_dim, cfg.qk_norm, &L.q_norm) ||
        bind_norm(pd, s->arena, p + "attn_k_norm.weight", cfg.head_dim, cfg.qk_norm, &L.k_norm) ||
        bind_linear(pd, s->arena, p + "attn_q.weight", qd, H, &L.q) ||
        bind_linear(pd, s->arena, p + "attn_k.weight", kvd, H, &L.k) ||
        bind_linear(pd, s->arena, p + "attn_v.weight", kvd, H, &L.v) ||
        bind_linear(pd, s->arena, p + "attn_output.weight", H, qd, &L.o) ||
        bind_linear(pd, s->arena, p + "ffn_gate.weight", I, H, &L.gate) ||
        bind_linear(pd, s->arena, p + "ffn_up.weight", I, H, &L.up) ||
        bind_linear(pd, s->arena, p + "ffn_down.weight", H, I, &L.down))
      return fail();
    {
      auto follows = [](const WRef& a, const WRef& b) {
        return a.enc == b.enc && a.enc != E_MLX_U4 && a.cols == b.cols &&
               reinterpret_cast<const uint8_t*>(b.data) == reinterpret_cast<const uint8_t*>(a.data) + a.total_bytes();
      };
      if (follows(L.q, L.k)) {
        L.qkv = L.q;
        L.qkv.rows = L.q.rows + L.k.rows;
        L.qkv_parts = 2;
        if (follows(L.k, L.v)) L.qkv.rows += L.v.rows, L.qkv_parts = 3;
      }
      if (follows(L.gate, L.up)) {
        L.gate_up = L.gate;
        L.gate_up.rows = L.gate.rows + L.up.rows;
      }
    }
    if (cfg.qk_norm && L.q_norm.type != L.k_norm.type) {
      set_error("q_norm and k_norm weights of layer %d differ in type", l);
      return fail();
    }
    dwb += L.q.total_bytes() + L.k.total_bytes() + L.v.total_bytes() + L.o.total_bytes() +
           L.gate.total_bytes() + L.up.total_bytes() + L.down.total_bytes() + L.attn_norm.bytes +
           L.ffn_norm.bytes + L.q_norm.bytes + L.k_norm.bytes;
  }
  s->decode_weight_bytes = dwb;
  {
    size_t need = 0;
    auto grow = [&](const WRef& w) {
      for (int m = 1; m <= 8; m++) need = std::max(need, gemv_mma_workspace_bytes(w, E_F32, m));
    };
    grow(s->lm_head);
    for (const LayerW& L : s->layers) {
      const WRef* ws[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
      for (const WRef* wp : ws) grow(*wp);
      if (L.qkv_parts >= 2) grow(L.qkv);
      if (L.gate_up.data) grow(L.gate_up);
    }
    if (need) {
      need = need * 3 + 1024;  // up to three products' K-slice sums wait for the kernel that adds them
      for (int64_t r : {(int64_t)1, (int64_t)std::max(1, cfg.batch)}) {  // decode attention's slice results
        const int64_t per = std::max<int64_t>(1, std::min<int64_t>(32, 592 / (r * cfg.heads)));
        need = std::max(need, attention_split_scratch_bytes(r, cfg.heads, cfg.head_dim, (int)per));
      }
      if (dev_alloc(s, &s->scratch, need)) return fail();
      s->scratch_bytes = need;
      set_thread_scratch(s->scratch, s->scratch_bytes);  // `scope` was entered before the region existed
    }
  }

  if (cfg.persistent) {
    // candidates: every linear readable by the tile steps, q/k/v sharing one activation layout,
    // gate/up sharing an encoding, head dim 64 or 128; the shared-memory plan (ring + program) is
    // made when the KV geometry is configured. Other models use the operator path.
    int nslot = 0, xs = 0;
    size_t smem = 0;
    bool ok = mega_plan(cfg.hidden, cfg.inter, (int)qd, cfg.head_dim, 0, &nslot, &xs, &smem) != 0;
    std::vector<MegaLayer> ml(cfg.layers);
    for (int l = 0; l < cfg.layers; l++) {
      const LayerW& L = s->layers[l];
      ml[l].q = L.q, ml[l].k = L.k, ml[l].v = L.v, ml[l].o = L.o;
      ml[l].gate = L.gate, ml[l].up = L.up, ml[l].down = L.down;
      ml[l].attn_norm = L.attn_norm.ptr, ml[l].ffn_norm = L.ffn_norm.ptr;
      ml[l].q_norm = L.q_norm.ptr, ml[l].k_norm = L.k_norm.ptr;
      ml[l].norm_type = L.attn_norm.type, ml[l].qk_norm_type = L.q_norm.type;
      const WRef* ws[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
      for (const WRef* wp : ws)
        if (!mega_supports_weight(*wp)) ok = false;
      if (L.attn_norm.type != L.ffn_norm.type || L.gate.enc != L.up.enc) ok = false;
      if (xl_for_encoding_host(L.q.enc) != xl_for_encoding_host(L.k.enc) ||
          xl_for_encoding_host(L.q.enc) != xl_for_encoding_host(L.v.enc))
        ok = false;
    }
    if (!mega_supports_weight(s->lm_head) || cfg.heads % cfg.kv_heads != 0) ok = false;
    if (ok) {
      if (mega_grid_size(device, smem, &s->mega_grid)) return fail();
      s->mega_max_split = std::max(1, std::min(16, s->mega_grid / std::max(1, cfg.heads)));
      if (dev_alloc(s, (void**)&s->mega_layers, ml.size() * sizeof(MegaLayer)) ||
          dev_alloc(s, (void**)&s->io_dev, 64) || dev_alloc(s, (void**)&s->prof_dev, 192))
        return fail();
      if (cudaMemcpy(s->mega_layers, ml.data(), ml.size() * sizeof(MegaLayer),
                     cudaMemcpyHostToDevice) != cudaSuccess ||
          cudaMemset(s->io_dev, 0, 64) != cudaSuccess) {
        set_error("initialising the persistent decode kernel state failed");
        return fail();
      }
      s->mega = true;
    }
  }
  if (cfg.tp_world > 1) {
    const size_t n = (size_t)std::max(1, cfg.batch) * cfg.lm_rows * 4;
    if (dev_alloc(s, (void**)&s->tp_logits, n)) return fail();
    if (cudaMemset(s->tp_logits, 0, n) != cudaSuccess) {
      set_error("cudaMemset of the logits slice failed");
      return fail();
    }
  }
  if (host_alloc(s, (void**)&s->logits_host, (size_t)cfg.vocab * 4)) return fail();
  if (dev_alloc(s, (void**)&s->logits, (size_t)cfg.vocab * 4) ||
      dev_alloc(s, (void**)&s->out_token_dev, 64) ||
      dev_alloc(s, (void**)&s->hist_count_dev, 64) ||
      dev_alloc(s, &s->argmax_scratch, argmax_scratch_bytes(cfg.vocab)))
    return fail();
  *out_session = s;
  return 0;
}

void dyninfer_cuda_session_destroy(dyninfer_cuda_session_t* s) {
  if (!s) return;
  cudaSetDevice(s->device);
  if (s->stream) cudaStreamSynchronize(s->stream);
  destroy_graphs(s);
  void* dev[] = {s->arena, s->kcache, s->vcache, s->hidden, s->xn, s->ctx, s->act,
                 s->logits, s->tokens_dev, s->row_pos_dev, s->row_seq_dev, s->out_token_dev,
                 s->hist_dev, s->hist_count_dev, s->argmax_scratch, s->mega_layers, s->io_dev,
                 s->prof_dev, s->trace_dev, s->prog_dev, s->ll_dev, s->batch_logits, s->batch_tokens_dev, s->tp_part, s->tp_logits,
                 s->tp_gather, s->scratch, s->qkv1, s->gu1, s->xh, s->xinv, s->gpart};
  for (void* p : dev)
    if (p) cudaFree(p);
  if (s->logits_host) cudaFreeHost(s->logits_host);
  if (s->batch_logits_host) cudaFreeHost(s->batch_logits_host);
  if (s->stage_host) cudaFreeHost(s->stage_host);
  if (s->tm0) cudaEventDestroy(s->tm0);
  if (s->tm1) cudaEventDestroy(s->tm1);
  if (s->ev0) cudaEventDestroy(s->ev0);
  if (s->ev1) cudaEventDestroy(s->ev1);
  for (int r = 0; r < s->peer.world; r++)
    if (r != s->peer.rank && s->peer.base[r]) cudaIpcCloseMemHandle(s->peer.base[r]);
  if (s->peer.base[s->peer.rank]) cudaFree(s->peer.base[s->peer.rank]);
  if (s->peer.epochs) cudaFree(s->peer.epochs);
  if (s->peer.error_host) cudaFreeHost(s->peer.error_host);
  if (s->tp_comm) tp_comm_destroy(s->tp_comm);
  if (s->stream) cudaStreamDestroy(s->stream);
  delete s;
}

int dyninfer_cuda_session_configure_paged_kv(dyninfer_cuda_session_t* s, size_t layer_count,
                                             size_t page_size, size_t kv_head_count,
                                             size_t head_dim, size_t kv_element_byte_count,
                                             size_t chunk_size, size_t vocab_size) {
  DYN_CHECK(s != nullptr, "session is NULL");
  // reconfiguring after allocation is an error (wrapper.c:927-930)
  DYN_CHECK(s->pages == 0, "paged KV is already allocated; it cannot be reconfigured");
  DYN_CHECK(layer_count == (size_t)s->cfg.layers && kv_head_count == (size_t)s->cfg.kv_heads &&
                head_dim == (size_t)s->cfg.head_dim && vocab_size == (size_t)s->cfg.vocab,
            "paged KV geometry (layers %zu, kv heads %zu, head_dim %zu, vocab %zu) does not match the model",
            layer_count, kv_head_count, head_dim, vocab_size);
  DYN_CHECK(page_size > 0 && chunk_size > 0, "page_size and chunk_size must be positive");
  // wrapper.c:921: one of the two must divide the other
  DYN_CHECK(page_size % chunk_size == 0 || chunk_size % page_size == 0,
            "invalid paged KV configuration: page_size %zu and chunk_size %zu do not divide one another",
            page_size, chunk_size);
  DYN_CHECK(kv_element_byte_count == 4 || kv_element_byte_count == 2,
            "kv_element_byte_count %zu unsupported (4 = f32, 2 = bf16/f16)", kv_element_byte_count);
  CounterScope scope(s);
  DYN_CUDA(cudaSetDevice(s->device));
  s->page_size = page_size;
  s->chunk_size = chunk_size;
  s->kv_elem = kv_element_byte_count;
  s->kv_type = kv_element_byte_count == 4 ? E_F32 : s->cfg.kv2_type;
  // activation scratch for the widest call: one prefill chunk or one batched step
  const ModelCfg& c = s->cfg;
  const int64_t rows = std::max<int64_t>((int64_t)chunk_size, c.batch);
  const int64_t qd = (int64_t)c.heads * c.head_dim, kvd = (int64_t)c.kv_heads * c.head_dim;
  if (!s->kv_configured) {
    if (dev_alloc(s, (void**)&s->hidden, (size_t)rows * c.hidden * 4) ||
        dev_alloc(s, (void**)&s->xn, (size_t)rows * c.hidden * 4) ||
        dev_alloc(s, (void**)&s->ctx, (size_t)rows * qd * 4) ||
        dev_alloc(s, (void**)&s->act, (size_t)rows * c.inter * 4) ||
        (c.tp_world == 1 && rows >= 64 &&
         (dev_alloc(s, (void**)&s->xh, (size_t)(rows + rows / 2 + 64) * std::max(c.hidden, c.inter) * 2) ||
          dev_alloc(s, (void**)&s->xinv, (size_t)(rows + rows / 2 + 64) * 4) ||
          dev_alloc(s, (void**)&s->gpart, (size_t)8 * rows * std::max<int64_t>(c.hidden, qd + 2 * kvd) * 4))) ||
        dev_alloc(s, (void**)&s->qkv1, (size_t)rows * (qd + 2 * kvd) * 4) ||
        dev_alloc(s, (void**)&s->gu1, (size_t)rows * 2 * c.inter * 4) ||
        (c.tp_world > 1 && dev_alloc(s, (void**)&s->tp_part, (size_t)rows * c.hidden * 4)) ||
        dev_alloc(s, (void**)&s->tokens_dev, (size_t)rows * 8) ||
        dev_alloc(s, (void**)&s->row_pos_dev, (size_t)rows * 8) ||
        dev_alloc(s, (void**)&s->row_seq_dev, (size_t)rows * 8) ||
        host_alloc(s, (void**)&s->stage_host, (size_t)(8 + 3 * rows) * 8))
      return 1;
    if (s->xh) s->xh_rows = rows + rows / 2 + 64, s->xh_cols = std::max(c.hidden, c.inter), s->gpart_bytes = (size_t)8 * rows * std::max<int64_t>(c.hidden, qd + 2 * kvd) * 4;
    // the separate-product path writes dense q, k, v and `up` into the same buffers
    s->q = s->qkv1, s->k = s->q + rows * qd, s->v = s->k + rows * kvd;
    s->up = s->gu1;
    s->max_rows = rows;
  } else {
    DYN_CHECK(rows <= s->max_rows, "chunk_size %zu exceeds the scratch sized at first configuration",
              chunk_size);
  }
  s->kv_configured = true;
  destroy_graphs(s);
  if (s->mega && !s->prog_dev) {
    std::vector<MegaBuildLayer> bl(c.layers);
    std::vector<MegaLayer> ml(c.layers);
    for (int l = 0; l < c.layers; l++) {
      const LayerW& L = s->layers[l];
      bl[l].q = L.q, bl[l].k = L.k, bl[l].v = L.v, bl[l].o = L.o;
      bl[l].gate = L.gate, bl[l].up = L.up, bl[l].down = L.down;
      ml[l].q = L.q, ml[l].k = L.k, ml[l].v = L.v, ml[l].o = L.o;
      ml[l].gate = L.gate, ml[l].up = L.up, ml[l].down = L.down;
      ml[l].attn_norm = L.attn_norm.ptr, ml[l].ffn_norm = L.ffn_norm.ptr;
      ml[l].q_norm = L.q_norm.ptr, ml[l].k_norm = L.k_norm.ptr;
      ml[l].norm_type = L.attn_norm.type, ml[l].qk_norm_type = L.q_norm.type;
    }
    std::vector<uint8_t> blob;
    if (mega_build_program(bl.data(), ml.data(), c.layers, s->lm_head, c.heads, c.kv_heads, c.head_dim, c.hidden,
                           c.inter, c.vocab, s->mega_grid, &blob, &s->mega_lay))
      return 1;
    // the program lives in shared memory beside the ring; a model whose program does not fit
    // decodes on the operator path
    if (!mega_plan(c.hidden, c.inter, c.heads * c.head_dim, c.head_dim, s->mega_lay.bytes, &s->mega_nslot,
                   &s->mega_xs, &s->mega_smem)) {
      s->mega = false;
    } else {
      if (mega_grid_size(s->device, s->mega_smem, &s->mega_grid)) return 1;
      if (dev_alloc(s, (void**)&s->prog_dev, blob.size())) return 1;
      DYN_CUDA(cudaMemcpy(s->prog_dev, blob.data(), blob.size(), cudaMemcpyHostToDevice));
      // hand-off vectors: (value, epoch) pairs = 2 floats per element, each vector 256-byte aligned
      const size_t qd = (size_t)c.heads * c.head_dim, kvd = (size_t)c.kv_heads * c.head_dim;
      const size_t elems[7] = {(size_t)c.hidden, (size_t)c.hidden, qd + 2 * kvd, qd,
                               (size_t)c.heads * s->mega_max_split * (c.head_dim + 4), (size_t)c.inter,
                               4 * (size_t)s->mega_grid};
      size_t off = 0;
      for (int i = 0; i < 7; i++) {
        s->ll_off[i] = off;
        off += (2 * elems[i] + 63) / 64 * 64;
      }
      if (dev_alloc(s, (void**)&s->ll_dev, off * 4)) return 1;
      DYN_CUDA(cudaMemset(s->ll_dev, 0, off * 4));
      s->mega_epoch = 0;
      const char* te = getenv("DYNINFER_CUDA_TRACE");
      if (te && te[0] == '1') {
        const size_t tb = (size_t)s->mega_grid * (c.layers + 1) * 16 * 8;
        if (dev_alloc(s, (void**)&s->trace_dev, tb)) return 1;
        DYN_CUDA(cudaMemset(s->trace_dev, 0, tb));
      }
    }
  }
  return 0;
}

int dyninfer_cuda_session_ensure_kv_pages(dyninfer_cuda_session_t* s, size_t page_count) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->kv_configured, "paged KV is not configured");
  if (page_count <= s->pages) return 0;
  CounterScope scope(s);
  DYN_CUDA(cudaSetDevice(s->device));
  const ModelCfg& c = s->cfg;
  const size_t planes = (size_t)c.layers * c.batch * c.kv_heads;
  const size_t new_row = page_count * s->page_size * c.head_dim * s->kv_elem;  // bytes per plane
  const size_t old_row = s->pages * s->page_size * c.head_dim * s->kv_elem;
  const size_t bytes = planes * new_row;
  uint8_t *nk = nullptr, *nv = nullptr;
  if (dev_alloc(s, (void**)&nk, bytes)) return 1;
  if (dev_alloc(s, (void**)&nv, bytes)) {
    dev_free(s, nk, bytes);
    return 1;
  }
  DYN_CUDA(cudaMemsetAsync(nk, 0, bytes, s->stream));
  DYN_CUDA(cudaMemsetAsync(nv, 0, bytes, s->stream));
  if (s->pages) {  // grow: keep what is already cached, plane by plane
    DYN_CUDA(cudaMemcpy2DAsync(nk, new_row, s->kcache, old_row, old_row, planes,
                               cudaMemcpyDeviceToDevice, s->stream));
    DYN_CUDA(cudaMemcpy2DAsync(nv, new_row, s->vcache, old_row, old_row, planes,
                               cudaMemcpyDeviceToDevice, s->stream));
  }
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  dev_free(s, s->kcache, s->kv_bytes_each);
  dev_free(s, s->vcache, s->kv_bytes_each);
  s->kcache = nk;
  s->vcache = nv;
  s->kv_bytes_each = bytes;
  s->pages = page_count;
  destroy_graphs(s);
  return 0;
}

int dyninfer_cuda_session_reset_paged_kv(dyninfer_cuda_session_t* s) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->kv_configured, "paged KV is not configured");
  if (!s->pages) return 0;
  DYN_CUDA(cudaSetDevice(s->device));
  // zero-fill in place, the pool is kept (wrapper.c:1273-1303)
  DYN_CUDA(cudaMemsetAsync(s->kcache, 0, s->kv_bytes_each, s->stream));
  DYN_CUDA(cudaMemsetAsync(s->vcache, 0, s->kv_bytes_each, s->stream));
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  return 0;
}

size_t dyninfer_cuda_session_kv_page_count(const dyninfer_cuda_session_t* s) {
  return s ? s->pages : 0;
}
size_t dyninfer_cuda_session_kv_allocated_bytes(const dyninfer_cuda_session_t* s) {
  return s ? 2 * s->kv_bytes_each : 0;
}

int dyninfer_cuda_session_allocator_statistics(const dyninfer_cuda_session_t* s,
                                               dyninfer_cuda_allocator_statistics_t* out) {
  DYN_CHECK(s != nullptr && out != nullptr, "session or out_stats is NULL");
  *out = s->stats;
  return 0;
}

uint64_t dyninfer_cuda_session_weight_bytes(const dyninfer_cuda_session_t* s) {
  return s ? s->weight_bytes : 0;
}
uint64_t dyninfer_cuda_session_decode_weight_bytes(const dyninfer_cuda_session_t* s) {
  return s ? s->decode_weight_bytes : 0;
}
int dyninfer_cuda_session_decode_phase_profile(dyninfer_cuda_session_t* s, double* out_us,
                                               size_t count) {
  DYN_CHECK(s != nullptr && out_us != nullptr, "session or out_us is NULL");
  DYN_CHECK(s->mega && s->prof_dev, "the persistent decode kernel is not in use");
  unsigned long long ns[24] = {0};
  DYN_CUDA(cudaSetDevice(s->device));
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  DYN_CUDA(cudaMemcpy(ns, s->prof_dev, sizeof ns, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < count && i < 24; i++) out_us[i] = (double)ns[i] * 1e-3;
  return 0;
}

int dyninfer_cuda_session_uses_persistent_kernel(const dyninfer_cuda_session_t* s) {
  return s && s->mega && s->prog_dev ? 1 : 0;
}

int dyninfer_cuda_session_decode_trace(dyninfer_cuda_session_t* s, uint64_t* out, size_t count, size_t* out_needed) {
  DYN_CHECK(s != nullptr && out_needed != nullptr, "session or out_needed is NULL");
  const size_t need = s->trace_dev ? (size_t)s->mega_grid * (s->cfg.layers + 1) * 16 : 0;
  *out_needed = need;
  if (!out || count < need || need == 0) return 0;
  DYN_CUDA(cudaSetDevice(s->device));
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  DYN_CUDA(cudaMemcpy(out, s->trace_dev, need * 8, cudaMemcpyDeviceToHost));
  return 0;
}

int dyninfer_cuda_session_timer(dyninfer_cuda_session_t* s, int stop, float* out_ms) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CUDA(cudaSetDevice(s->device));
  if (!s->tm0) {
    DYN_CUDA(cudaEventCreate(&s->tm0));
    DYN_CUDA(cudaEventCreate(&s->tm1));
  }
  if (!stop) {
    DYN_CUDA(cudaEventRecord(s->tm0, s->stream));
    return 0;
  }
  DYN_CHECK(out_ms != nullptr, "out_ms is NULL");
  DYN_CUDA(cudaEventRecord(s->tm1, s->stream));
  DYN_CUDA(cudaEventSynchronize(s->tm1));
  DYN_CUDA(cudaEventElapsedTime(out_ms, s->tm0, s->tm1));
  return check_device_error("session timer");
}

uint64_t dyninfer_cuda_session_launch_count(const dyninfer_cuda_session_t* s) {
  return s ? s->launches : 0;
}

int dyninfer_cuda_session_invoke_paged_chunk(dyninfer_cuda_session_t* s, const int64_t* tokens,
                                             size_t token_count, int64_t last, int64_t start_pos,
                                             float** out_logits, size_t* out_count,
                                             int64_t* out_token, int want_logits) {
  return dyninfer_cuda_session_invoke_paged_chunk_slot(s, tokens, token_count, last, start_pos, 0, out_logits,
                                                      out_count, out_token, want_logits);
}

int dyninfer_cuda_session_invoke_paged_chunk_slot(dyninfer_cuda_session_t* s, const int64_t* tokens,
                                                  size_t token_count, int64_t last, int64_t start_pos,
                                                  int64_t slot, float** out_logits, size_t* out_count,
                                                  int64_t* out_token, int want_logits) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(slot >= 0 && slot < s->cfg.batch, "slot %lld outside [0, %d) (the descriptor's \"batch\")",
            (long long)slot, s->cfg.batch);
  DYN_CHECK(s->kv_configured && s->pages > 0, "paged KV is not configured or has no pages");
  DYN_CHECK(tokens != nullptr, "tokens is NULL");
  // wrapper.c:1230-1235
  DYN_CHECK(token_count == 1 || token_count == s->chunk_size,
            "token_count %zu must be 1 or the chunk size %zu", token_count, s->chunk_size);
  DYN_CHECK(last >= 0 && (size_t)last < token_count, "last %lld out of range [0, %zu)",
            (long long)last, token_count);
  DYN_CHECK(start_pos >= 0, "start_pos must be >= 0");
  DYN_CHECK(!want_logits || (out_logits && out_count), "want_logits needs out_logits and out_count");
  const int64_t rows = last + 1;
  const int64_t cap = (int64_t)(s->pages * s->page_size);
  DYN_CHECK(start_pos + rows <= cap, "positions [%lld, %lld) exceed the KV capacity %lld",
            (long long)start_pos, (long long)(start_pos + rows), (long long)cap);
  for (int64_t i = 0; i < rows; i++)
    DYN_CHECK(tokens[i] >= 0 && tokens[i] < s->cfg.vocab, "token id %lld at %lld outside [0, %d)",
              (long long)tokens[i], (long long)i, s->cfg.vocab);
  CounterScope scope(s);
  DYN_CUDA(cudaSetDevice(s->device));
  if (rows == 1 && s->mega) {
    s->stage_host[0] = tokens[0];
    s->stage_host[1] = start_pos;
    s->stage_host[2] = slot;
    // token, position and slot travel as launch parameters; the kernel writes the produced token
    // (and the code of an expired wait) into the pinned staging words itself
    MegaArgs ma;
    fill_mega_args(s, &ma, 0);
    ma.inline_io = 1, ma.in_token = tokens[0], ma.in_pos = start_pos, ma.in_seq = slot;
    DYN_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&ma.out_host), s->stage_host + 3, 0));
    s->stage_host[4] = 0;
    if (launch_decode_mega(ma, s->mega_grid, s->mega_smem, s->stream)) return 1;
  } else if (rows == 1) {
    if (!s->decode_graph && capture(s, false, &s->decode_graph, &s->graph_nodes)) return 1;
    s->stage_host[0] = tokens[0];
    s->stage_host[1] = start_pos;
    s->stage_host[2] = slot;
    DYN_CUDA(cudaGraphLaunch(s->decode_graph, s->stream));
    s->launches += s->graph_nodes;
  } else {
    int64_t* st = s->stage_host + 8;
    for (int64_t i = 0; i < rows; i++) {
      st[i] = tokens[i];
      st[rows + i] = start_pos + i;
      st[2 * rows + i] = slot;
    }
    DYN_CUDA(cudaMemcpyAsync(s->tokens_dev, st, rows * 8, cudaMemcpyHostToDevice, s->stream));
    DYN_CUDA(cudaMemcpyAsync(s->row_pos_dev, st + rows, rows * 8, cudaMemcpyHostToDevice, s->stream));
    DYN_CUDA(cudaMemcpyAsync(s->row_seq_dev, st + 2 * rows, rows * 8, cudaMemcpyHostToDevice,
                             s->stream));
    if (enqueue_forward(s, rows, last, false, start_pos, slot)) return 1;
    DYN_CUDA(cudaMemcpyAsync(s->stage_host + 3, s->out_token_dev, 8, cudaMemcpyDeviceToHost,
                             s->stream));
  }
  if (want_logits)
    DYN_CUDA(cudaMemcpyAsync(s->logits_host, s->logits, (size_t)s->cfg.vocab * 4,
                             cudaMemcpyDeviceToHost, s->stream));
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  if (tp_check_error(s)) return 1;
  if (check_device_error("session step")) return 1;
  if (rows == 1 && s->mega && mega_check_error(s, s->stage_host[4])) return 1;
  if (out_token) *out_token = s->stage_host[3];
  if (want_logits) {
    *out_logits = s->logits_host;  // session scratch, borrowed until the next invoke
    *out_count = (size_t)s->cfg.vocab;
  } else {
    if (out_logits) *out_logits = nullptr;
    if (out_count) *out_count = 0;
  }
  return 0;
}

// One decode step for `count` independent sequences: row i feeds tokens[i] at positions[i] into the
// KV slot slots[i]; out_tokens[i] is the greedy next token of that sequence.
int dyninfer_cuda_session_decode_batch(dyninfer_cuda_session_t* s, const int64_t* tokens,
                                       const int64_t* positions, const int64_t* slots, size_t count,
                                       int64_t* out_tokens, float** out_logits, int want_logits) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->kv_configured && s->pages > 0, "paged KV is not configured or has no pages");
  DYN_CHECK(tokens && positions && slots && out_tokens, "tokens, positions, slots or out_tokens is NULL");
  DYN_CHECK(count >= 1 && (int64_t)count <= s->max_rows && (int)count <= s->cfg.batch,
            "count %zu must be in [1, %d] (the descriptor's \"batch\")", count, s->cfg.batch);
  DYN_CHECK(!want_logits || out_logits, "want_logits needs out_logits");
  const int64_t rows = (int64_t)count;
  const int64_t cap = (int64_t)(s->pages * s->page_size);
  std::vector<char> used((size_t)s->cfg.batch, 0);
  for (int64_t i = 0; i < rows; i++) {
    DYN_CHECK(tokens[i] >= 0 && tokens[i] < s->cfg.vocab, "token id %lld at %lld outside [0, %d)",
              (long long)tokens[i], (long long)i, s->cfg.vocab);
    DYN_CHECK(positions[i] >= 0 && positions[i] < cap, "position %lld at %lld exceeds the KV capacity %lld",
              (long long)positions[i], (long long)i, (long long)cap);
    DYN_CHECK(slots[i] >= 0 && slots[i] < s->cfg.batch && !used[(size_t)slots[i]],
              "slot %lld at %lld is out of range or used twice in one step", (long long)slots[i], (long long)i);
    used[(size_t)slots[i]] = 1;
  }
  if (rows == 1 && !want_logits) {  // a single sequence: the single-token fast path serves any slot
    if (out_logits) *out_logits = nullptr;
    return dyninfer_cuda_session_invoke_paged_chunk_slot(s, tokens, 1, 0, positions[0], slots[0], nullptr, nullptr,
                                                         out_tokens, 0);
  }
  CounterScope scope(s);
  DYN_CUDA(cudaSetDevice(s->device));
  if (!s->batch_logits) {
    if (dev_alloc(s, (void**)&s->batch_logits, (size_t)s->cfg.batch * s->cfg.vocab * 4) ||
        dev_alloc(s, (void**)&s->batch_tokens_dev, (size_t)s->cfg.batch * 8) ||
        (s->cfg.tp_world > 1 &&
         dev_alloc(s, (void**)&s->tp_gather, (size_t)s->cfg.batch * s->cfg.vocab * 4)))
      return 1;
  }
  int64_t* st = s->stage_host + 8;
  for (int64_t i = 0; i < rows; i++) {
    st[i] = tokens[i];
    st[rows + i] = positions[i];
    st[2 * rows + i] = slots[i];
  }
  DYN_CUDA(cudaMemcpyAsync(s->tokens_dev, st, rows * 8, cudaMemcpyHostToDevice, s->stream));
  DYN_CUDA(cudaMemcpyAsync(s->row_pos_dev, st + rows, rows * 8, cudaMemcpyHostToDevice, s->stream));
  DYN_CUDA(cudaMemcpyAsync(s->row_seq_dev, st + 2 * rows, rows * 8, cudaMemcpyHostToDevice, s->stream));
  auto it = s->batch_graphs.find(rows);
  if (it == s->batch_graphs.end()) {
    cudaGraphExec_t exec = nullptr;
    uint64_t nodes = 0;
    if (capture_batch(s, rows, &exec, &nodes)) return 1;
    it = s->batch_graphs.emplace(rows, std::make_pair(exec, nodes)).first;
  }
  DYN_CUDA(cudaGraphLaunch(it->second.first, s->stream));
  s->launches += it->second.second;
  DYN_CUDA(cudaMemcpyAsync(st, s->batch_tokens_dev, rows * 8, cudaMemcpyDeviceToHost, s->stream));
  if (want_logits) {
    if (!s->batch_logits_host &&
        host_alloc(s, (void**)&s->batch_logits_host, (size_t)s->cfg.batch * s->cfg.vocab * 4))
      return 1;
    // gathered slices [rank][row][lm_rows] -> rows of the whole vocabulary
    for (int w = 0; s->cfg.tp_world > 1 && w < s->cfg.tp_world; w++)
      DYN_CUDA(cudaMemcpy2DAsync(s->batch_logits + (size_t)w * s->cfg.lm_rows, (size_t)s->cfg.vocab * 4,
                                 s->tp_gather + (size_t)w * rows * s->cfg.lm_rows,
                                 (size_t)s->cfg.lm_rows * 4, (size_t)s->cfg.lm_rows * 4, (size_t)rows,
                                 cudaMemcpyDeviceToDevice, s->stream));
    DYN_CUDA(cudaMemcpyAsync(s->batch_logits_host, s->batch_logits, (size_t)rows * s->cfg.vocab * 4,
                             cudaMemcpyDeviceToHost, s->stream));
  }
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  if (tp_check_error(s)) return 1;
  if (check_device_error("session step")) return 1;
  for (int64_t i = 0; i < rows; i++) out_tokens[i] = st[i];
  if (out_logits) *out_logits = want_logits ? s->batch_logits_host : nullptr;  // borrowed until the next call
  return 0;
}

size_t dyninfer_cuda_tp_unique_id_bytes(void) { return tp_unique_id_bytes(); }

int dyninfer_cuda_tp_unique_id(uint8_t* out_id, size_t byte_count) {
  DYN_CHECK(out_id != nullptr && byte_count == tp_unique_id_bytes(),
            "out_id is NULL or byte_count is not dyninfer_cuda_tp_unique_id_bytes()");
  return tp_unique_id(out_id);
}

int dyninfer_cuda_session_tp_init(dyninfer_cuda_session_t* s, const uint8_t* id, size_t byte_count) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->cfg.tp_world > 1, "the session's descriptor does not set tp_world > 1");
  DYN_CHECK(id != nullptr && byte_count == tp_unique_id_bytes(),
            "id is NULL or byte_count is not dyninfer_cuda_tp_unique_id_bytes()");
  DYN_CHECK(s->tp_comm == nullptr, "the session already has a communicator");
  DYN_CUDA(cudaSetDevice(s->device));
  return tp_comm_init(&s->tp_comm, id, s->cfg.tp_rank, s->cfg.tp_world);
}

size_t dyninfer_cuda_tp_peer_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int dyninfer_cuda_session_tp_peer_handle(dyninfer_cuda_session_t* s, uint8_t* out_handle, size_t byte_count) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->cfg.tp_world > 1 && s->cfg.tp_world <= TP_MAX_WORLD,
            "peer exchange needs 2..%d tensor-parallel ranks", TP_MAX_WORLD);
  DYN_CHECK(s->kv_configured, "configure the paged KV first: the exchange region is sized by its chunk");
  DYN_CHECK(out_handle != nullptr && byte_count == sizeof(cudaIpcMemHandle_t),
            "out_handle is NULL or byte_count is not dyninfer_cuda_tp_peer_handle_bytes()");
  DYN_CHECK(s->cfg.hidden % 4 == 0, "peer exchange needs hidden to be a multiple of 4");
  DYN_CUDA(cudaSetDevice(s->device));
  TpPeer& p = s->peer;
  if (!p.base[s->cfg.tp_rank]) {
    p.rank = s->cfg.tp_rank, p.world = s->cfg.tp_world, p.max_rows = s->max_rows;
    p.region_bytes = tp_peer_region_bytes(s->max_rows, s->cfg.hidden);
    p.flags_off = tp_peer_flags_offset(s->max_rows, s->cfg.hidden);
    void* region = nullptr;
    if (dev_alloc(s, &region, p.region_bytes) || dev_alloc(s, (void**)&p.epochs, TP_PEER_BLOCKS * 4)) return 1;
    p.base[p.rank] = reinterpret_cast<uint8_t*>(region);
    DYN_CUDA(cudaMemset(region, 0, p.region_bytes));
    DYN_CUDA(cudaMemset(p.epochs, 0, TP_PEER_BLOCKS * 4));
    DYN_CUDA(cudaHostAlloc((void**)&p.error_host, 64, cudaHostAllocMapped));
    *p.error_host = 0;
    DYN_CUDA(cudaHostGetDevicePointer((void**)&p.error_dev, p.error_host, 0));
    DYN_CUDA(cudaDeviceSynchronize());
  }
  cudaIpcMemHandle_t h;
  DYN_CUDA(cudaIpcGetMemHandle(&h, p.base[p.rank]));
  memcpy(out_handle, &h, sizeof h);
  return 0;
}

int dyninfer_cuda_session_tp_peer_attach(dyninfer_cuda_session_t* s, const uint8_t* handles, size_t byte_count) {
  DYN_CHECK(s != nullptr, "session is NULL");
  TpPeer& p = s->peer;
  DYN_CHECK(p.base[s->cfg.tp_rank] != nullptr && !p.attached,
            "call dyninfer_cuda_session_tp_peer_handle first (and attach once)");
  DYN_CHECK(handles != nullptr && byte_count == (size_t)p.world * sizeof(cudaIpcMemHandle_t),
            "handles must hold one handle per rank, in rank order");
  DYN_CUDA(cudaSetDevice(s->device));
  for (int r = 0; r < p.world; r++) {
    if (r == p.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * sizeof h, sizeof h);
    void* ptr = nullptr;
    DYN_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    p.base[r] = reinterpret_cast<uint8_t*>(ptr);
  }
  p.attached = true;
  destroy_graphs(s);
  return 0;
}

int dyninfer_cuda_session_decode_loop(dyninfer_cuda_session_t* s, int64_t first_token,
                                      int64_t start_pos, size_t steps, int64_t* out_tokens,
                                      float* out_device_ms) {
  DYN_CHECK(s != nullptr, "session is NULL");
  DYN_CHECK(s->kv_configured && s->pages > 0, "paged KV is not configured or has no pages");
  DYN_CHECK(first_token >= 0 && first_token < s->cfg.vocab, "token id %lld outside [0, %d)",
            (long long)first_token, s->cfg.vocab);
  const int64_t cap = (int64_t)(s->pages * s->page_size);
  DYN_CHECK(start_pos >= 0 && start_pos + (int64_t)steps <= cap,
            "positions [%lld, %lld) exceed the KV capacity %lld", (long long)start_pos,
            (long long)(start_pos + (int64_t)steps), (long long)cap);
  if (out_device_ms) *out_device_ms = 0.f;
  if (steps == 0) return 0;
  CounterScope scope(s);
  DYN_CUDA(cudaSetDevice(s->device));
  if (ensure_hist(s, steps)) return 1;
  if (s->mega) {
    s->stage_host[0] = first_token;
    s->stage_host[1] = start_pos;
    s->stage_host[2] = 0;
    DYN_CUDA(cudaMemcpyAsync(s->io_dev, s->stage_host, 24, cudaMemcpyHostToDevice, s->stream));
    DYN_CUDA(cudaMemsetAsync(s->hist_count_dev, 0, 8, s->stream));
    DYN_CUDA(cudaEventRecord(s->ev0, s->stream));
    // several tokens per launch: the launch gap and the kernel's prologue are paid once per group
    size_t per = 16;
    if (const char* e = getenv("DYNINFER_CUDA_TOKENS_PER_LAUNCH")) per = (size_t)std::max(1, std::min(256, atoi(e)));
    for (size_t i = 0; i < steps; i += per) {
      MegaArgs ma;
      fill_mega_args(s, &ma, 1, (int)std::min(per, steps - i));
      if (launch_decode_mega(ma, s->mega_grid, s->mega_smem, s->stream)) return 1;
    }
    DYN_CUDA(cudaEventRecord(s->ev1, s->stream));
    DYN_CUDA(cudaMemcpyAsync(s->stage_host + 3, s->io_dev + 3, 16, cudaMemcpyDeviceToHost, s->stream));
    DYN_CUDA(cudaStreamSynchronize(s->stream));
    if (mega_check_error(s, s->stage_host[4])) return 1;
    if (out_device_ms) DYN_CUDA(cudaEventElapsedTime(out_device_ms, s->ev0, s->ev1));
    if (out_tokens)
      DYN_CUDA(cudaMemcpy(out_tokens, s->hist_dev, steps * 8, cudaMemcpyDeviceToHost));
    return 0;
  }
  if (!s->loop_graph && capture(s, true, &s->loop_graph, &s->loop_nodes)) return 1;
  s->stage_host[0] = first_token;
  s->stage_host[1] = start_pos;
  s->stage_host[2] = 0;
  DYN_CUDA(cudaMemcpyAsync(s->tokens_dev, s->stage_host, 8, cudaMemcpyHostToDevice, s->stream));
  DYN_CUDA(cudaMemcpyAsync(s->row_pos_dev, s->stage_host + 1, 8, cudaMemcpyHostToDevice, s->stream));
  DYN_CUDA(cudaMemcpyAsync(s->row_seq_dev, s->stage_host + 2, 8, cudaMemcpyHostToDevice, s->stream));
  DYN_CUDA(cudaMemsetAsync(s->hist_count_dev, 0, 8, s->stream));
  DYN_CUDA(cudaEventRecord(s->ev0, s->stream));
  for (size_t i = 0; i < steps; i++) DYN_CUDA(cudaGraphLaunch(s->loop_graph, s->stream));
  DYN_CUDA(cudaEventRecord(s->ev1, s->stream));
  s->launches += s->loop_nodes * steps;
  DYN_CUDA(cudaStreamSynchronize(s->stream));
  if (tp_check_error(s)) return 1;
  if (check_device_error("session step")) return 1;
  if (out_device_ms) DYN_CUDA(cudaEventElapsedTime(out_device_ms, s->ev0, s->ev1));
  if (out_tokens)
    DYN_CUDA(cudaMemcpy(out_tokens, s->hist_dev, steps * 8, cudaMemcpyDeviceToHost));
  return 0;
}

}  // extern "C"
