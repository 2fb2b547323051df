// A step program: the kernels of one model step, launched from native code in one call.
//
// The parts of a model describe what they launch once, when the model is built, as a list of
// operations over symbolic buffers (``ayaka_py_b200/engine/program.py``); here the list is run for
// a step: buffer addresses are laid out in a workspace from the step's row counts, every
// operation picks its kernel by the same rules as the Python dispatchers (``ops.linear``,
// ``ops.attention``) and launches it on the given stream.  A step of a 48-layer model is one call
// into this file instead of four hundred calls from Python, which is what bounds prompt and mixed
// steps of small models (about 20 us of interpreter time per launch against 2 us here).
//
// The reference runs every step from Python (runner/paged_runner.py:1067-1114) and hides the
// cost of decode steps in CUDA graphs (runner/paged_runner.py:595-683), as this engine does too;
// prompt and mixed steps have no graph in either.
#include <stdint.h>
#include <string.h>

#include "common.cuh"
#include "step_program.h"

extern "C" {
int ayk_embed(float* out, const int* tok, const int* pos, const void* wte, const void* wpe, int T, int d, int dtype,
              cudaStream_t stream);
int ayk_layernorm(void* out, const float* x, const float* gamma, const float* beta, const int* rows, int n_rows, int d,
                  float eps, int out_dtype, cudaStream_t stream);
int ayk_gemm_simt(void* C, const void* A, const void* W, const float* bias, const float* residual, int M, int N, int K,
                  int act, int in_dtype, int out_dtype, cudaStream_t stream);
int ayk_gemm_tc(void* C, const void* X, const void* W, const float* bias, const float* residual, int M, int N, int K,
                int act, int out_dtype, int splits, float* partials, unsigned int* counters, int weight_is_static,
                int cluster, cudaStream_t stream);
int ayk_gemm_tc_prefill(void* C, const void* X, const void* W, const float* bias, const float* residual, int M, int N,
                        int K, int act, int out_dtype, int tile_n, int sms, int pair, cudaStream_t stream);
int ayk_gemm_tc_prefill_kv(void* C, const void* X, const void* W, const float* bias, int M, int N, int K, int tile_n,
                           int sms, int pair, void* kcache, void* vcache, const int* row_req, const int* pos,
                           const int* table, int table_stride, int page_size, int col0, int width, cudaStream_t stream);
int ayk_kv_append(void* kcache, void* vcache, const void* k, const void* v, int row_stride, const int* row_req,
                  const int* pos, const int* table, int table_stride, int page_size, int T, int width, int dtype,
                  cudaStream_t stream);
int ayk_attention_simt(void* out, const void* q, int q_stride, const void* kcache, const void* vcache, const int* table,
                       int table_stride, const int* req_q_start, const int* req_pos0, int num_req, int total_rows, int H,
                       int Hkv, int Dh, int page_size, float scale, int window, int dtype, cudaStream_t stream);
int ayk_attention_decode(void* out, const void* q, int q_stride, void* kcache, void* vcache, const int* table,
                         int table_stride, const int* req_pos0, int R, int H, int Hkv, int Dh, int page_size, float scale,
                         int window, int parts, float* scratch, const void* knew, const void* vnew, int new_stride,
                         const int* row_req, long long cache_pages, int settled, int dtype, cudaStream_t stream);
int ayk_attention_tc(void* out, const void* q, int q_stride, int q_rows, int total_rows, const void* kcache,
                     const void* vcache, int pages, const int* table, int table_stride, const int* req_q_start,
                     const int* req_pos0, int num_req, int H, int Hkv, int Dh, int page_size, float scale, int window,
                     cudaStream_t stream);
}

namespace {

constexpr int PREFILL_ROWS = 16;     // more rows than this: the kernel with 128-row tiles and no split along K
constexpr int CLUSTER_ROWS = 64;     // up to this many rows the splits of a tile exchange their sums inside a cluster
constexpr int DECODE_PART = 128;     // keys per partition of the decode kernels

inline int elem_bytes(int dtype) { return dtype == AYK_DTYPE_BF16 ? 2 : 4; }

}  // namespace

// Split-K factor of the few-row tensor-core product: skinny products (few output tiles) are cut
// along K so that about one CTA per multiprocessor streams the weight.  1, 2, 4, 8 or 16: those
// splits form a cluster.  16 (beyond the portable cluster size) only where each split still has
// four K blocks.
AYK_EXPORT int ayk_tc_splits(int M, int N, int K) {
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  const int tiles = ((N + 127) / 128) * ((M + bt - 1) / bt);
  const int blocks = (K + 63) / 64;
  const int sms = ayk_sm_count();
  if (tiles >= sms || blocks < 4 || M > CLUSTER_ROWS) return 1;
  if (tiles * 16 <= sms * 3 / 2 && blocks >= 64) return 16;
  const int candidates[3] = {8, 4, 2};
  for (int p : candidates)
    if (tiles * p <= sms * 14 / 10 && blocks >= p) return p;
  return 1;
}

// act(a[M, K] @ w[N, K]^T + bias) (+ residual): float32 operands on the FP32 pipes (true 32-bit);
// bfloat16 operands on the tensor cores when K is a multiple of 8, else on the FP32 pipes with
// 32-bit sums.  kv (or null): the product is a q | k | v projection whose key and value columns
// belong in the paged cache; *filed tells whether this call stored them.
AYK_EXPORT int ayk_linear(void* out, const void* a, const void* w, const float* bias, const float* residual, int M, int N,
                          int K, int act, int in_dtype, int out_dtype, const AykKvTarget* kv, int* filed,
                          cudaStream_t stream) {
  if (filed) *filed = 0;
  if (M == 0 || N == 0) return 0;
  if (in_dtype == AYK_DTYPE_BF16 && K % 8 == 0) {
    // Up to 64 rows with few output tiles: weights as the MMA's M side, K split over a cluster.  More
    // rows: tiles of 128 rows by a width from the kernel's time model.  (An out width that is no multiple
    // of 8 makes rows of C that are no whole 16-byte pieces: the many-row kernel turns such tiles in
    // shared memory and stores them a row at a time, which beats the first kernel from 17 rows on, 30
    // against 38 us for 64 rows of an LM head of 50,257 x 768; with a residual to add, up to 128 rows
    // stay with the first kernel, whose loads and stores run along the features.)
    int splits = 1;
    if (M <= CLUSTER_ROWS) splits = ayk_tc_splits(M, N, K);
    if (M <= PREFILL_ROWS || (M <= CLUSTER_ROWS && splits > 1)) {
      const int cluster = splits > 1 ? 1 : 0;
      return ayk_gemm_tc(out, a, w, bias, residual, M, N, K, act, out_dtype, splits, nullptr, nullptr, 1, cluster, stream);
    }
    if (N % 8 == 0 || M > 128 || residual == nullptr) {
      if (kv != nullptr && N % 8 == 0 && act == AYK_ACT_NONE && residual == nullptr && out_dtype == AYK_DTYPE_BF16 &&
          kv->dtype == AYK_DTYPE_BF16 && kv->col0 % 8 == 0 && kv->width % 8 == 0 && N == kv->col0 + 2 * kv->width &&
          (bias == nullptr || (uintptr_t)bias % 16 == 0)) {
        const int rc = ayk_gemm_tc_prefill_kv(out, a, w, bias, M, N, K, 0, ayk_sm_count(), -1, kv->kcache, kv->vcache,
                                              kv->row_req, kv->positions, kv->table, kv->table_stride, kv->page_size,
                                              kv->col0, kv->width, stream);
        if (rc == 0 && filed) *filed = 1;
        return rc;
      }
      return ayk_gemm_tc_prefill(out, a, w, bias, residual, M, N, K, act, out_dtype, 0, ayk_sm_count(), -1, stream);
    }
    return ayk_gemm_tc(out, a, w, bias, residual, M, N, K, act, out_dtype, 1, nullptr, nullptr, 1, 0, stream);
  }
  return ayk_gemm_simt(out, a, w, bias, residual, M, N, K, act, in_dtype, out_dtype, stream);
}

// Attention of a step's rows over the paged cache; see AykAttention.  Returns the number of kernels
// launched through *launched.
AYK_EXPORT int ayk_attention(void* out, const void* q, const void* k, const void* v, int qkv_stride, const AykAttention* at,
                             const AykStepRows* rows, int append, float* decode_scratch, long long scratch_floats,
                             int* launched, cudaStream_t stream) {
  int count = 0;
  const int T = rows->T, R = rows->R, D = rows->num_single;
  const int parts = (rows->max_context + DECODE_PART - 1) / DECODE_PART;
  auto decode = [&](int n_req, const void* knew, const void* vnew) -> int {
    if ((long long)n_req * at->H * parts * (at->Dh + 2) > scratch_floats)
      return ayk_fail("ayk_attention: the scratch of the decode kernels holds %lld floats, %d requests x %d heads x %d "
                      "partitions need more", scratch_floats, n_req, at->H, parts);
    count += 2;
    return ayk_attention_decode(out, q, qkv_stride, at->kcache, at->vcache, rows->table, rows->table_stride, rows->req_pos0,
                                n_req, at->H, at->Hkv, at->Dh, at->page_size, at->scale, at->window, parts, decode_scratch,
                                knew, vnew, qkv_stride, rows->row_req, at->pages, rows->settled, at->dtype, stream);
  };
  if (rows->max_q_len == 1 && at->Dh % 16 == 0) {
    const int rc = decode(R, append ? k : nullptr, append ? v : nullptr);
    if (launched) *launched = count;
    return rc;
  }
  if (append) {
    ++count;
    if (ayk_kv_append(at->kcache, at->vcache, k, v, qkv_stride, rows->row_req, rows->positions, rows->table,
                      rows->table_stride, at->page_size, T, at->Hkv * at->Dh, at->dtype, stream) != 0)
      return -1;
  }
  const bool tc = at->dtype == AYK_DTYPE_BF16 && at->Dh == 64 && at->page_size >= 8 && at->page_size <= 128 &&
                  (at->page_size & (at->page_size - 1)) == 0 && qkv_stride % 8 == 0 && (uintptr_t)q % 16 == 0;
  int rc;
  if (tc) {
    // A mixed step: its single-token requests are its first rows.  They go through the split-context
    // decode kernels, the prompt portions through the tiled kernel: two launches on disjoint row
    // ranges over one block table.
    if (D >= 1 && D < R) {
      if (decode(D, nullptr, nullptr) != 0) return -1;
      ++count;
      rc = ayk_attention_tc(out, q, qkv_stride, T, T - D, at->kcache, at->vcache, (int)at->pages,
                            rows->table + (size_t)D * rows->table_stride, rows->table_stride, rows->req_q_start + D,
                            rows->req_pos0 + D, R - D, at->H, at->Hkv, at->Dh, at->page_size, at->scale, at->window, stream);
    } else {
      ++count;
      rc = ayk_attention_tc(out, q, qkv_stride, T, T, at->kcache, at->vcache, (int)at->pages, rows->table,
                            rows->table_stride, rows->req_q_start, rows->req_pos0, R, at->H, at->Hkv, at->Dh, at->page_size,
                            at->scale, at->window, stream);
    }
  } else {
    ++count;
    rc = ayk_attention_simt(out, q, qkv_stride, at->kcache, at->vcache, rows->table, rows->table_stride, rows->req_q_start,
                            rows->req_pos0, R, T, at->H, at->Hkv, at->Dh, at->page_size, at->scale, at->window, at->dtype,
                            stream);
  }
  if (launched) *launched = count;
  return rc;
}

// Bytes of workspace that a step of T rows and S wanted rows needs.
AYK_EXPORT long long ayk_program_workspace_bytes(const AykBuffer* buffers, int n_buffers, int T, int S) {
  long long total = 0;
  for (int i = 0; i < n_buffers; ++i) {
    const long long rows = buffers[i].rows_kind == AYK_ROWS_WANTED ? S : T;
    total += (rows * buffers[i].row_bytes + 255) / 256 * 256;
  }
  return total;
}

// Runs the operations in order.  Returns 0, or -1 with a text in ayk_last_error(); *launched counts
// the kernels that were launched.
AYK_EXPORT int ayk_program_run(const AykOp* ops, int n_ops, const AykBuffer* buffers, int n_buffers, const AykStep* step,
                               int* launched, cudaStream_t stream) {
  int count = 0;
  int filed_flags[1024];        // whether a q | k | v product filed its keys and values, for the attention that follows it
  if (launched) *launched = 0;
  AYK_REQUIRE(n_buffers <= AYK_MAX_BUFFERS, "ayk_program_run: %d buffers, at most %d", n_buffers, AYK_MAX_BUFFERS);
  uint8_t* address[AYK_MAX_BUFFERS];
  long long offset = 0;
  for (int i = 0; i < n_buffers; ++i) {
    const long long rows = buffers[i].rows_kind == AYK_ROWS_WANTED ? step->S : step->T;
    address[i] = (uint8_t*)step->workspace + offset;
    offset += (rows * buffers[i].row_bytes + 255) / 256 * 256;
  }
  AYK_REQUIRE(offset <= step->workspace_bytes, "ayk_program_run: the step needs %lld bytes of workspace, %lld are there",
              offset, step->workspace_bytes);
  auto at = [&](int id) -> uint8_t* {
    if (id == AYK_BUFFER_LOGITS) return (uint8_t*)step->logits;
    if (id < 0 || id >= n_buffers) return nullptr;
    return address[id];
  };
  for (int i = 0; i < n_ops; ++i) {
    const AykOp& op = ops[i];
    int rc = 0;
    switch (op.kind) {
      case AYK_OP_EMBED:
        ++count;
        rc = ayk_embed((float*)at(op.out), step->tokens, step->positions, op.p[0], op.p[1], step->T, op.i[0], op.i[1], stream);
        break;
      case AYK_OP_LAYERNORM: {
        const bool gather = op.i[2] != 0;
        ++count;
        rc = ayk_layernorm(at(op.out), (const float*)at(op.in), (const float*)op.p[0], (const float*)op.p[1],
                           gather ? step->want_rows : nullptr, gather ? step->S : step->T, op.i[0], op.f[0], op.i[1], stream);
        break;
      }
      case AYK_OP_LINEAR: {
        // i: N, K, act, in dtype, out dtype, rows kind, kv flag, group, col0, width, page size, cache dtype
        const int M = op.i[5] == AYK_ROWS_WANTED ? step->S : step->T;
        AykKvTarget kv;
        const AykKvTarget* kvp = nullptr;
        int filed = 0;
        if (op.i[6] && step->max_q_len > 1) {        // a decode step's rows are filed by its attention kernel
          const int g = op.i[7];
          kv.kcache = (void*)op.p[2]; kv.vcache = (void*)op.p[3];
          kv.row_req = step->row_req; kv.positions = step->positions;
          kv.table = step->tables[g]; kv.table_stride = step->table_stride[g];
          kv.page_size = op.i[10]; kv.col0 = op.i[8]; kv.width = op.i[9]; kv.dtype = op.i[11];
          kvp = &kv;
        }
        ++count;
        rc = ayk_linear(at(op.out), at(op.in), op.p[0], (const float*)op.p[1], op.in2 >= 0 ? (const float*)at(op.in2) : nullptr,
                        M, op.i[0], op.i[1], op.i[2], op.i[3], op.i[4], kvp, &filed, stream);
        if (op.i[6]) filed_flags[op.i[12] & 1023] = filed;
        break;
      }
      case AYK_OP_ATTENTION: {
        // i: H, Hkv, Dh, page size, window, dtype, group, q width, kv width, writes, filed slot; f: scale; p: kcache, vcache, pages
        AykAttention a;
        a.kcache = (void*)op.p[0]; a.vcache = (void*)op.p[1]; a.pages = (long long)(intptr_t)op.p[2];
        a.H = op.i[0]; a.Hkv = op.i[1]; a.Dh = op.i[2]; a.page_size = op.i[3]; a.window = op.i[4]; a.dtype = op.i[5];
        a.scale = op.f[0];
        const int g = op.i[6];
        AykStepRows rows;
        rows.T = step->T; rows.R = step->R; rows.num_single = step->num_single; rows.max_q_len = step->max_q_len;
        rows.max_context = step->max_context; rows.settled = step->settled;
        rows.table = step->tables[g]; rows.table_stride = step->table_stride[g];
        rows.req_q_start = step->req_q_start; rows.req_pos0 = step->req_pos0; rows.row_req = step->row_req;
        rows.positions = step->positions;
        const int eb = elem_bytes(a.dtype);
        const int stride = op.i[7] + 2 * op.i[8];
        const uint8_t* qkv = at(op.in);
        const int append = op.i[9] && !(op.i[10] >= 0 && filed_flags[op.i[10] & 1023]);
        int n = 0;
        rc = ayk_attention(at(op.out), qkv, qkv + (size_t)op.i[7] * eb, qkv + (size_t)(op.i[7] + op.i[8]) * eb, stride, &a,
                           &rows, append, step->decode_scratch, step->decode_scratch_floats, &n, stream);
        count += n;
        break;
      }
      default:
        return ayk_fail("ayk_program_run: operation %d has the unknown kind %d", i, op.kind);
    }
    if (rc != 0) {
      if (launched) *launched = count;
      return -1;
    }
  }
  if (launched) *launched = count;
  return 0;
}
