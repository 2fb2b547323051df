// Embedding + learned positions, LayerNorm, paged KV append; and the host-side
// error channel of the library.
//
// Reference counterparts: embedding lookup kernel/triton/embedding.py:162-175
// plus the wpe add of models/gpt2.py:516-517 (fused here); LayerNorm
// kernel/triton/norm.py:311-374 (two-pass mean / biased variance in 32-bit);
// KV scatter kernel/triton/cache/paged_kv.py:141-214.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

// ------------------------------------------------------------ error channel --
static thread_local char g_error[512] = "";

int ayk_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return -1;
}

int ayk_check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return ayk_fail("%s: %s", what, cudaGetErrorString(err));
  return 0;
}

AYK_EXPORT const char* ayk_last_error() { return g_error; }

static int g_pdl = 0;
int ayk_pdl_enabled() { return g_pdl; }
// Launch kernels with programmatic stream serialization (1) or plainly (0).
AYK_EXPORT void ayk_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// Streaming multiprocessors of the current device (read once per device; 148 on a B200).
static int g_sm_count[64] = {0};
int ayk_sm_count() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (g_sm_count[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) return 148;
    g_sm_count[device] = n;
  }
  return g_sm_count[device];
}
AYK_EXPORT int ayk_device_sm_count() { return ayk_sm_count(); }

AYK_EXPORT int ayk_init(int device) {
  cudaError_t err = cudaSetDevice(device);
  if (err != cudaSuccess) return ayk_fail("cudaSetDevice(%d): %s", device, cudaGetErrorString(err));
  cudaDeviceProp prop;
  err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess) return ayk_fail("cudaGetDeviceProperties: %s", cudaGetErrorString(err));
  if (prop.major != 10) return ayk_fail("this library is built for sm_100a, device %d is sm_%d%d", device, prop.major, prop.minor);
  if (device >= 0 && device < 64) g_sm_count[device] = prop.multiProcessorCount;
  return 0;
}

// ------------------------------------------------------------------- embed --
template <typename W>
__global__ void embed_kernel(float* __restrict__ out, const int* __restrict__ tok,
                             const int* __restrict__ pos, const W* __restrict__ wte,
                             const W* __restrict__ wpe, int d) {
  pdl_trigger();
  pdl_wait();
  int t = blockIdx.x;
  const W* e = wte + (size_t)tok[t] * d;
  const W* p = wpe ? wpe + (size_t)pos[t] * d : nullptr;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = to_float<W>(e[i]);
    if (p) v += to_float<W>(p[i]);
    o[i] = v;
  }
}

// out[t, :] = wte[tok[t], :] (+ wpe[pos[t], :]) as float32.  The host has
// checked the ids against the table sizes.
AYK_EXPORT int ayk_embed(float* out, const int* tok, const int* pos, const void* wte,
                         const void* wpe, int T, int d, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  int threads = d >= 256 ? 256 : 128;
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, out, tok, pos, (const float*)wte, (const float*)wpe, d);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, tok, pos,
               (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, d);
  else
    return ayk_fail("ayk_embed: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_embed");
}

// --------------------------------------------------------------- layernorm --
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += red[w];   // same order in every thread
  return total;
}

template <typename O>
__global__ void layernorm_kernel(O* __restrict__ out, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 const int* __restrict__ rows, int d, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * d;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = src[i];
    row[i] = v;
    s += v;
  }
  float mean = block_sum(s, red) / (float)d;
  float q = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float c = row[i] - mean;
    q += c * c;
  }
  float var = block_sum(q, red) / (float)d;
  float rstd = rsqrtf(var + eps);
  O* dst = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = (row[i] - mean) * rstd * gamma[i] + (beta ? beta[i] : 0.f);
    dst[i] = from_float<O>(v);
  }
}

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 w;
  w.x = *reinterpret_cast<uint32_t*>(&lo);
  w.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;
}

// One block of 128 threads per row, the row in registers (width a multiple of 4, at most 2048): one
// pass over memory.  In a decode step the kernel sits on the critical path between two products, so
// what does not depend on the kernel before it (weight and bias of the norm, the row index) is
// fetched before the programmatic-launch wait, and the row is read with every load in flight at
// once.  It also serves prompts: 2,048 rows of 1,600 take 5.2 us (3.8 TB/s); a one-warp-per-row
// variant took 10.2 us and was removed.
template <typename O>
__global__ void __launch_bounds__(128)
layernorm_row_kernel(O* __restrict__ out, const float* __restrict__ x, const float* __restrict__ gamma,
                     const float* __restrict__ beta, const int* __restrict__ rows, int d, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  constexpr int HELD = 4;                        // float4 per thread: widths up to 2048
  const int r = blockIdx.x, nv = d >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  const float4* b4 = reinterpret_cast<const float4*>(beta);
  float4 g[HELD], b[HELD], v[HELD];
#pragma unroll
  for (int i = 0; i < HELD; ++i) {
    const int idx = threadIdx.x + 128 * i;
    g[i] = idx < nv ? __ldg(g4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
    b[i] = (idx < nv && beta) ? __ldg(b4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src_row = rows ? rows[r] : r;
  pdl_wait();
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)src_row * d);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < HELD; ++i) {
    const int idx = threadIdx.x + 128 * i;
    v[i] = idx < nv ? src[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = block_sum(s, red) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < HELD; ++i) {
    if (threadIdx.x + 128 * i < nv) {
      const float a = v[i].x - mean, bb = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      q += (a * a + bb * bb) + (c * c + e * e);
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / (float)d + eps);
  O* dst = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < HELD; ++i) {
    const int idx = threadIdx.x + 128 * i;
    if (idx < nv)
      store4(dst + 4 * idx, (v[i].x - mean) * rstd * g[i].x + b[i].x, (v[i].y - mean) * rstd * g[i].y + b[i].y,
             (v[i].z - mean) * rstd * g[i].z + b[i].z, (v[i].w - mean) * rstd * g[i].w + b[i].w);
  }
}

// out[r, :] = LayerNorm(x[rows ? rows[r] : r, :]); x float32, statistics and
// affine in 32-bit, result stored as out_dtype.
AYK_EXPORT int ayk_layernorm(void* out, const float* x, const float* gamma, const float* beta,
                             const int* rows, int n_rows, int d, float eps, int out_dtype,
                             cudaStream_t stream) {
  if (n_rows == 0) return 0;
  AYK_REQUIRE(d >= 1 && (size_t)d * 4 <= 48 * 1024, "ayk_layernorm: width %d is not in [1, 12288]", d);
  const bool aligned = (d % 4 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)gamma % 16 == 0) &&
                       (beta == nullptr || (uintptr_t)beta % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (aligned && d <= 2048 && (out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16)) {
    if (out_dtype == AYK_DTYPE_F32)
      ayk_launch(layernorm_row_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (float*)out, x, gamma, beta, rows, d, eps);
    else
      ayk_launch(layernorm_row_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, stream, (__nv_bfloat16*)out, x, gamma, beta, rows, d, eps);
    return ayk_check_launch("ayk_layernorm");
  }
  int threads = d >= 1024 ? 256 : 128;
  size_t smem = (size_t)d * sizeof(float);
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, (float*)out, x, gamma, beta, rows, d, eps);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, (__nv_bfloat16*)out, x, gamma, beta, rows, d, eps);
  else
    return ayk_fail("ayk_layernorm: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_layernorm");
}

// --------------------------------------------------------------- kv append --
template <typename T>
__global__ void kv_append_kernel(T* __restrict__ kcache, T* __restrict__ vcache,
                                 const T* __restrict__ k, const T* __restrict__ v, int row_stride,
                                 const int* __restrict__ row_req, const int* __restrict__ pos,
                                 const int* __restrict__ table, int table_stride, int page_size,
                                 int width, int vec_ok) {
  pdl_trigger();
  // positions and block table are the step's inputs, not the work of the kernel before this one
  int t = blockIdx.x;
  int p = pos[t];
  int page = table[(size_t)row_req[t] * table_stride + p / page_size];
  pdl_wait();
  if (page <= 0) return;   // the padding page holds nothing; a live row never maps to it
  size_t dst = ((size_t)page * page_size + (p % page_size)) * width;
  const T* ks = k + (size_t)t * row_stride;
  const T* vs = v + (size_t)t * row_stride;
  if (vec_ok) {            // rows of whole 16-byte pieces, 16-byte aligned on both sides
    constexpr int PER = 16 / sizeof(T);
    const uint4* k4 = reinterpret_cast<const uint4*>(ks);
    const uint4* v4 = reinterpret_cast<const uint4*>(vs);
    uint4* kd = reinterpret_cast<uint4*>(kcache + dst);
    uint4* vd = reinterpret_cast<uint4*>(vcache + dst);
    const int n = width / PER;
    for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
      if (i < n) kd[i] = k4[i];
      else vd[i - n] = v4[i - n];
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    kcache[dst + i] = ks[i];
    vcache[dst + i] = vs[i];
  }
}

// Writes the keys and values of the step's rows into their pages:
// cache[page(row), pos % P, :, :] = k[row, :]; page(row) = table[row_req[row], pos / P].
// width = kv_heads * head_dim; k and v are rows of a wider matrix (row_stride elements).
AYK_EXPORT int ayk_kv_append(void* kcache, void* vcache, const void* k, const void* v,
                             int row_stride, const int* row_req, const int* pos, const int* table,
                             int table_stride, int page_size, int T, int width, int dtype,
                             cudaStream_t stream) {
  if (T == 0) return 0;
  int threads = width >= 512 ? 256 : 128;
  const size_t elem = dtype == AYK_DTYPE_F32 ? 4 : 2;
  const int vec_ok = (width * elem) % 16 == 0 && ((size_t)row_stride * elem) % 16 == 0 && (uintptr_t)k % 16 == 0 &&
                     (uintptr_t)v % 16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0;
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(kv_append_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)kcache, (float*)vcache,
               (const float*)k, (const float*)v, row_stride, row_req, pos, table, table_stride, page_size, width, vec_ok);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(kv_append_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)kcache,
               (__nv_bfloat16*)vcache, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, row_stride, row_req, pos,
               table, table_stride, page_size, width, vec_ok);
  else
    return ayk_fail("ayk_kv_append: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_kv_append");
}
