/* A host written in C against include/dyninfer_cuda.h and nothing else: what the Rust
 * `dyninfer-cuda-sys` binding does, without any Python in the process.
 *
 *   abi_driver <descriptor.json> <params.txt> <chunk_size> <prompt ids, comma separated> <steps>
 *
 * params.txt: first line = number of files F, then F lines with a path, then one line per
 * byte range: "<key> <source_file_index> <offset> <length>" (the provider plan of
 * crates/dyninfer-checkpoint/src/provider.rs:9-125).
 *
 * Drives the session the way `IreeSession` does (crates/dyninfer-runtime/src/session.rs:89-330):
 * create_with_file_params -> configure_paged_kv -> ensure_kv_pages -> one invoke_paged_chunk per
 * prompt chunk (right padded, last = n - 1) -> one invoke per decoded token -> statistics ->
 * reset -> destroy. Prints one line: "tokens: t0 t1 ...", then "logits0: <first 4 logits of the
 * prompt's last row>", then "pages: <count> bytes: <kv bytes> device_peak: <bytes>". Any failing
 * call prints the library's last error and exits 1.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "dyninfer_cuda.h"

#define CHECK(call)                                                                   \
  do {                                                                                \
    if ((call) != 0) {                                                                \
      fprintf(stderr, "%s failed: %s\n", #call, dyninfer_cuda_last_error());          \
      return 1;                                                                       \
    }                                                                                 \
  } while (0)

static char* read_file(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) return NULL;
  fseek(f, 0, SEEK_END);
  long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  char* buf = (char*)malloc((size_t)n + 1);
  if (buf && fread(buf, 1, (size_t)n, f) != (size_t)n) {
    free(buf);
    buf = NULL;
  }
  if (buf) buf[n] = 0;
  fclose(f);
  return buf;
}

/* Minimal lookup of an integer field of the flat descriptor ("layers": 2, ...). */
static long json_int(const char* json, const char* key) {
  char pat[64];
  snprintf(pat, sizeof pat, "\"%s\":", key);
  const char* p = strstr(json, pat);
  if (!p) return -1;
  return strtol(p + strlen(pat), NULL, 10);
}

int main(int argc, char** argv) {
  if (argc != 6) {
    fprintf(stderr, "usage: %s descriptor.json params.txt chunk_size prompt_ids steps\n", argv[0]);
    return 2;
  }
  char* desc = read_file(argv[1]);
  if (!desc) {
    fprintf(stderr, "cannot read %s\n", argv[1]);
    return 1;
  }
  FILE* pf = fopen(argv[2], "r");
  if (!pf) {
    fprintf(stderr, "cannot read %s\n", argv[2]);
    return 1;
  }
  const size_t chunk = (size_t)strtoul(argv[3], NULL, 10);
  const int steps = atoi(argv[5]);

  int nfiles = 0;
  if (fscanf(pf, "%d\n", &nfiles) != 1 || nfiles < 1 || nfiles > 64) return 1;
  dyninfer_cuda_parameter_file_t files[64];
  static char paths[64][4096];
  for (int i = 0; i < nfiles; i++) {
    if (!fgets(paths[i], sizeof paths[i], pf)) return 1;
    paths[i][strcspn(paths[i], "\n")] = 0;
    files[i].path = paths[i];
  }
  size_t cap = 1024, nparams = 0;
  dyninfer_cuda_file_param_t* params = (dyninfer_cuda_file_param_t*)malloc(cap * sizeof *params);
  char key[1024];
  unsigned long long idx, off, len;
  while (fscanf(pf, "%1023s %llu %llu %llu", key, &idx, &off, &len) == 4) {
    if (nparams == cap) {
      cap *= 2;
      params = (dyninfer_cuda_file_param_t*)realloc(params, cap * sizeof *params);
    }
    params[nparams].key = strdup(key);
    params[nparams].source_file_index = (size_t)idx;
    params[nparams].offset = off;
    params[nparams].length = len;
    nparams++;
  }
  fclose(pf);

  int64_t prompt[4096];
  size_t nprompt = 0;
  for (char* tok = strtok(argv[4], ","); tok && nprompt < 4096; tok = strtok(NULL, ",")) prompt[nprompt++] = atoll(tok);
  if (nprompt == 0) return 2;

  const long layers = json_int(desc, "layers"), kv_heads = json_int(desc, "kv_heads");
  const long head_dim = json_int(desc, "head_dim"), vocab = json_int(desc, "vocab");
  if (layers < 1 || kv_heads < 1 || head_dim < 1 || vocab < 1) {
    fprintf(stderr, "descriptor lacks layers / kv_heads / head_dim / vocab\n");
    return 1;
  }

  int ndev = 0;
  CHECK(dyninfer_cuda_device_count(&ndev));
  dyninfer_cuda_session_t* s = NULL;
  CHECK(dyninfer_cuda_session_create_with_file_params("cuda:0", desc, files, (size_t)nfiles, params, nparams, &s));
  const size_t page = 256;
  CHECK(dyninfer_cuda_session_configure_paged_kv(s, (size_t)layers, page, (size_t)kv_heads, (size_t)head_dim, 4, chunk,
                                                 (size_t)vocab));
  /* the reference rejects geometries where neither size divides the other (wrapper.c:921),
   * and a second configuration once pages exist (wrapper.c:927-930) */
  const size_t need = nprompt + (size_t)steps + 1;
  CHECK(dyninfer_cuda_session_ensure_kv_pages(s, (need + page - 1) / page));
  if (dyninfer_cuda_session_configure_paged_kv(s, (size_t)layers, page, (size_t)kv_heads, (size_t)head_dim, 4, chunk,
                                               (size_t)vocab) == 0) {
    fprintf(stderr, "reconfiguring after allocation must fail\n");
    return 1;
  }

  int64_t* window = (int64_t*)calloc(chunk, sizeof(int64_t));
  float* logits = NULL;
  size_t count = 0;
  int64_t token = -1;
  float first4[4] = {0, 0, 0, 0};
  size_t pos = 0;
  while (pos < nprompt) {
    const size_t n = nprompt - pos < chunk ? nprompt - pos : chunk;
    memset(window, 0, chunk * sizeof(int64_t)); /* right padding with the pad id 0 */
    memcpy(window, prompt + pos, n * sizeof(int64_t));
    const int last_chunk = pos + n == nprompt;
    CHECK(dyninfer_cuda_session_invoke_paged_chunk(s, window, chunk, (int64_t)n - 1, (int64_t)pos, &logits, &count,
                                                   &token, last_chunk));
    if (last_chunk) {
      if (count != (size_t)vocab || !logits) {
        fprintf(stderr, "logits view: count %zu\n", count);
        return 1;
      }
      memcpy(first4, logits, sizeof first4); /* borrowed until the next invoke: copy now */
      dyninfer_cuda_free(logits);            /* a no-op, as dyninfer_iree_free is for session scratch */
    }
    pos += n;
  }
  printf("tokens: %lld", (long long)token);
  for (int i = 0; i < steps; i++) {
    int64_t in = token;
    CHECK(dyninfer_cuda_session_invoke_paged_chunk(s, &in, 1, 0, (int64_t)pos, NULL, NULL, &token, 0));
    printf(" %lld", (long long)token);
    pos++;
  }
  printf("\nlogits0: %.9g %.9g %.9g %.9g\n", first4[0], first4[1], first4[2], first4[3]);
  dyninfer_cuda_allocator_statistics_t st;
  CHECK(dyninfer_cuda_session_allocator_statistics(s, &st));
  printf("pages: %zu bytes: %zu device_peak: %llu persistent: %d launches: %llu\n", dyninfer_cuda_session_kv_page_count(s),
         dyninfer_cuda_session_kv_allocated_bytes(s), (unsigned long long)st.device_bytes_peak,
         dyninfer_cuda_session_uses_persistent_kernel(s), (unsigned long long)dyninfer_cuda_session_launch_count(s));
  CHECK(dyninfer_cuda_session_reset_paged_kv(s));
  if (dyninfer_cuda_session_kv_page_count(s) == 0) {
    fprintf(stderr, "reset must keep the pool\n");
    return 1;
  }
  /* misuse is reported, not executed (wrapper.c:1230-1235) */
  if (dyninfer_cuda_session_invoke_paged_chunk(s, window, 3, 0, 0, NULL, NULL, &token, 0) == 0 && chunk != 3) {
    fprintf(stderr, "token_count 3 must be rejected\n");
    return 1;
  }
  dyninfer_cuda_session_destroy(s);
  free(window);
  free(desc);
  return 0;
}
