// Data that a step program is made of (see step_program.cu).  The same layouts are declared as
// ctypes structures in ayaka_py_b200/engine/program.py.
#pragma once

#include <stdint.h>

#define AYK_OP_EMBED 0
#define AYK_OP_LAYERNORM 1
#define AYK_OP_LINEAR 2
#define AYK_OP_ATTENTION 3

#define AYK_ROWS_ALL 0        // a buffer (or an operation) over the step's T rows
#define AYK_ROWS_WANTED 1     // ... over the S rows whose logits are wanted

#define AYK_BUFFER_LOGITS (-2)    // the step's output, given by the caller
#define AYK_MAX_BUFFERS 64
#define AYK_MAX_GROUPS 8

// A symbolic buffer: rows (all or wanted) times row_bytes, laid out in the workspace in order.
struct AykBuffer {
  int32_t rows_kind;
  int32_t row_bytes;
};

// One operation.  in / in2 / out name buffers (-1: none); the meaning of i, f and p is per kind.
struct AykOp {
  int32_t kind, in, in2, out;
  int32_t i[16];
  float f[2];
  const void* p[4];
};

// What a step brings: its row counts and the places of its metadata on the device.
struct AykStep {
  int32_t T, R, S, num_single, max_q_len, max_context, settled, pad_;
  const int *tokens, *positions, *row_req, *want_rows, *req_q_start, *req_pos0;
  const int* tables[AYK_MAX_GROUPS];
  int32_t table_stride[AYK_MAX_GROUPS];
  void* workspace;
  long long workspace_bytes;
  void* logits;
  float* decode_scratch;
  long long decode_scratch_floats;
};

// Where the key and value columns of a fused q | k | v projection belong in the paged cache.
struct AykKvTarget {
  void *kcache, *vcache;
  const int *row_req, *positions, *table;
  int32_t table_stride, page_size, col0, width, dtype;
};

// Geometry of one attention layer and its pages.
struct AykAttention {
  void *kcache, *vcache;
  long long pages;
  int32_t H, Hkv, Dh, page_size, window, dtype;
  float scale;
};

// The rows of a step as the attention kernels see them.
struct AykStepRows {
  int32_t T, R, num_single, max_q_len, max_context, settled;
  const int *table, *req_q_start, *req_pos0, *row_req, *positions;
  int32_t table_stride;
};
