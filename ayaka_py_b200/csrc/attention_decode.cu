// Decode attention: one query row per request over its paged keys and values,
// split along the context so that a batch of 1 still fills the GPU, then merged.
//
// The reference's decode path is a split-KV kernel over partitions of 512 keys
// with partial outputs and log-sum-exps in 32-bit scratch and a reduce kernel
// (kernel/triton/paged_attention.py:474-736).  Here a partition is 128 keys
// (PART), the grid is (request, head, partition) with a fixed number of
// partitions (those beyond a request's context return at once, so the launch
// does not depend on the context lengths and can be replayed from a CUDA graph),
// and nothing but the block table is needed to find the keys.
//
// Scores, softmax and the weighted sum are 32-bit.  Per partition: scores with
// one key per lane (16-byte loads along the head dimension), then the weighted
// sum with one pair of head-dim columns per lane (coalesced rows of V).
// Partials (unnormalised sum, running max, sum of exponentials) go to scratch
// [request, head, partition, Dh + 2]; the merge kernel combines them in
// partition order.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int PART = 128;      // keys per partition
constexpr int WARPS = 4;
constexpr int MAX_DH = 256;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
  float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 x = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ float2 load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(float* __restrict__ scratch, const T* __restrict__ q, int q_stride,
                    const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ table, int table_stride, const int* __restrict__ req_pos0,
                    int H, int Hkv, int Dh, int page_size, float scale, int window, int parts) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, part = blockIdx.z;
  const int pos = req_pos0[r];                 // the query's position; keys 0..pos are visible
  int k_lo = part * PART, k_hi = min(pos + 1, k_lo + PART);
  if (window > 0) k_lo = max(k_lo, pos - window + 1);
  float* out = scratch + ((size_t)(r * H + h) * parts + part) * (Dh + 2);
  if (k_lo >= k_hi) {                          // nothing of this request in this partition
    if (threadIdx.x == 0) { out[Dh] = -INFINITY; out[Dh + 1] = 0.f; }
    return;
  }
  const int kvh = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int VN = Vec<T>::N;

  __shared__ float qs[MAX_DH];
  __shared__ float ps[PART];
  __shared__ float red[WARPS];
  __shared__ float accs[WARPS][MAX_DH];
  const T* qrow = q + (size_t)r * q_stride + h * Dh;
  for (int d = threadIdx.x; d < Dh; d += blockDim.x) qs[d] = to_float<T>(qrow[d]) * scale;
  __syncthreads();

  const int* my_table = table + (size_t)r * table_stride;
  const size_t row_elems = (size_t)Hkv * Dh;

  // scores: thread t takes key k_lo + t
  const int kp = k_lo + threadIdx.x;
  float s = -INFINITY;
  if (kp < k_hi) {
    const int page = my_table[kp / page_size];
    if (page > 0) {
      const T* krow = kcache + ((size_t)page * page_size + (kp % page_size)) * row_elems + (size_t)kvh * Dh;
      float acc = 0.f;
      // Loads first, arithmetic after: several 16-byte loads in flight per thread.
      for (int d0 = 0; d0 < Dh; d0 += 4 * VN) {
        float kv[4][VN];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (d0 + u * VN < Dh) load_vec(krow + d0 + u * VN, kv[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (d0 + u * VN < Dh) {
#pragma unroll
            for (int i = 0; i < VN; ++i) acc = fmaf(qs[d0 + u * VN + i], kv[u][i], acc);
          }
      }
      s = acc;
    }
  }
  float m = warp_max(s);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float p = (s > -INFINITY) ? expf(s - m) : 0.f;
  ps[threadIdx.x] = p;
  float l = warp_sum(p);
  __syncthreads();
  if (lane == 0) red[warp] = l;
  __syncthreads();
  l = (red[0] + red[1]) + (red[2] + red[3]);

  // weighted sum: warp w takes keys w, w + 4, ...; lane takes head-dim pairs lane, lane + 32, ...
  float2 acc[MAX_DH / 64];
#pragma unroll
  for (int c = 0; c < MAX_DH / 64; ++c) acc[c] = make_float2(0.f, 0.f);
  const int pairs = Dh / 2;
  const int n_keys = k_hi - k_lo;
  constexpr int UNROLL = 8;            // keys whose rows are in flight at once per warp
  for (int j0 = warp; j0 < n_keys; j0 += WARPS * UNROLL) {
    float pj[UNROLL];
    const T* vrow[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int j = j0 + u * WARPS;
      pj[u] = j < n_keys ? ps[j] : 0.f;
      const int key = k_lo + (j < n_keys ? j : 0);
      const int page = pj[u] != 0.f ? my_table[key / page_size] : 0;
      vrow[u] = vcache + ((size_t)page * page_size + (key % page_size)) * row_elems + (size_t)kvh * Dh;
    }
#pragma unroll
    for (int c = 0; c < MAX_DH / 64; ++c) {
      const int pp = lane + 32 * c;
      if (pp < pairs) {
        float2 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) v[u] = pj[u] != 0.f ? load_pair(vrow[u] + 2 * pp) : make_float2(0.f, 0.f);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          acc[c].x = fmaf(pj[u], v[u].x, acc[c].x);
          acc[c].y = fmaf(pj[u], v[u].y, acc[c].y);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < MAX_DH / 64; ++c) {
    const int pp = lane + 32 * c;
    if (pp < pairs) { accs[warp][2 * pp] = acc[c].x; accs[warp][2 * pp + 1] = acc[c].y; }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < Dh; d += blockDim.x)
    out[d] = (accs[0][d] + accs[1][d]) + (accs[2][d] + accs[3][d]);
  if (threadIdx.x == 0) { out[Dh] = m; out[Dh + 1] = l; }
}

template <typename T>
__global__ void decode_merge_kernel(T* __restrict__ out, const float* __restrict__ scratch, int H, int Dh, int parts) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const float* base = scratch + (size_t)(r * H + h) * parts * (Dh + 2);
  float m = -INFINITY;
  for (int s = 0; s < parts; ++s) m = fmaxf(m, base[(size_t)s * (Dh + 2) + Dh]);
  float l = 0.f;
  for (int s = 0; s < parts; ++s) {
    const float ms = base[(size_t)s * (Dh + 2) + Dh];
    if (ms > -INFINITY) l += base[(size_t)s * (Dh + 2) + Dh + 1] * expf(ms - m);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* o = out + ((size_t)r * H + h) * Dh;
  for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < parts; ++s) {
      const float ms = base[(size_t)s * (Dh + 2) + Dh];
      if (ms > -INFINITY) acc += base[(size_t)s * (Dh + 2) + d] * expf(ms - m);
    }
    o[d] = from_float<T>(acc * inv);
  }
}

}  // namespace

AYK_EXPORT int ayk_attention_decode_part() { return PART; }

// One query row per request: out[R, H*Dh]; q rows of q_stride elements; caches
// [pages, page_size, Hkv, Dh]; table[R, table_stride]; req_pos0[R] = the row's
// position.  parts = ceil(longest possible context / 128) (fixed per engine);
// scratch holds R * H * parts * (Dh + 2) floats.
AYK_EXPORT int ayk_attention_decode(void* out, const void* q, int q_stride, const void* kcache, const void* vcache,
                                    const int* table, int table_stride, const int* req_pos0, int R, int H, int Hkv,
                                    int Dh, int page_size, float scale, int window, int parts, float* scratch,
                                    int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  AYK_REQUIRE(Dh >= 16 && Dh % 16 == 0 && Dh <= MAX_DH, "ayk_attention_decode: head size %d is not a multiple of 16 in [16, %d]", Dh, MAX_DH);
  AYK_REQUIRE(Hkv >= 1 && H % Hkv == 0, "ayk_attention_decode: %d heads cannot share %d key/value heads", H, Hkv);
  AYK_REQUIRE(parts >= 1 && parts <= 65535 && H <= 65535, "ayk_attention_decode: grid too large (heads %d, parts %d)", H, parts);
  dim3 grid(R, H, parts), mgrid(R, H);
  int mthreads = Dh <= 32 ? 32 : (Dh <= 64 ? 64 : 128);
  if (dtype == AYK_DTYPE_F32) {
    ayk_launch(decode_split_kernel<float>, grid, dim3(WARPS * 32), 0, stream, scratch, (const float*)q, q_stride,
               (const float*)kcache, (const float*)vcache, table, table_stride, req_pos0, H, Hkv, Dh, page_size, scale,
               window, parts);
    ayk_launch(decode_merge_kernel<float>, mgrid, dim3(mthreads), 0, stream, (float*)out, (const float*)scratch, H, Dh, parts);
  } else if (dtype == AYK_DTYPE_BF16) {
    ayk_launch(decode_split_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), 0, stream, scratch, (const __nv_bfloat16*)q,
               q_stride, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, table, table_stride, req_pos0, H, Hkv,
               Dh, page_size, scale, window, parts);
    ayk_launch(decode_merge_kernel<__nv_bfloat16>, mgrid, dim3(mthreads), 0, stream, (__nv_bfloat16*)out,
               (const float*)scratch, H, Dh, parts);
  } else {
    return ayk_fail("ayk_attention_decode: unknown dtype %d", dtype);
  }
  return ayk_check_launch("ayk_attention_decode");
}
