// Causal attention of a step's rows over the paged cache, any mix of prompt
// portions and single decoded tokens, on the FP32 pipes.  It is the attention
// of the true 32-bit path and the general fallback for head sizes and options
// that the faster kernels refuse.
//
// Formula (kernel/triton/paged_attention.py:295-355): for the query at absolute
// position p of a request, s_j = (q . k_j) * scale over the cached positions
// j <= p of that request (and j > p - window when a window is given), online
// softmax with running maximum and sum in 32-bit, o = sum_j a_j v_j; a query
// with no visible key gives 0.  The keys and values of the step's own rows are
// already in the cache (ayk_kv_append runs first, as attention/base.py:67-69
// stores before it attends).
//
// One block works on up to 32 consecutive rows of one request and one head: 4
// warps x 8 rows.  Keys are taken 32 at a time (one per lane for the scores, one
// head-dim column per lane for the weighted sum).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int BQ = 32;       // rows per block
constexpr int BKEYS = 32;    // keys per iteration
constexpr int WARPS = 4;
constexpr int RQ = BQ / WARPS;
constexpr int MAX_DH = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(T* __restrict__ out, const T* __restrict__ q, int q_stride,
                      const T* __restrict__ kcache, const T* __restrict__ vcache,
                      const int* __restrict__ table, int table_stride,
                      const int* __restrict__ req_q_start, const int* __restrict__ req_pos0,
                      int num_req, int H, int Hkv, int Dh, int page_size, float scale, int window) {
  pdl_trigger();
  pdl_wait();
  // Which request and which of its row tiles is this block?
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  for (int r = 0; r < num_req; ++r) {
    int len = req_q_start[r + 1] - req_q_start[r];
    int tiles = (len + BQ - 1) / BQ;
    if (tile < tiles) { req = r; q0 = tile * BQ; q_len = len; break; }
    tile -= tiles;
  }
  if (req < 0) return;
  const int h = blockIdx.y, kvh = h / (H / Hkv);
  const int rows = min(BQ, q_len - q0);
  const int row0 = req_q_start[req] + q0;       // first global row of the tile
  const int pos0 = req_pos0[req] + q0;          // its absolute position
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ldk = Dh + 1;
  const int ldq = (Dh + 3) & ~3;       // query rows start on 16-byte boundaries whatever the head size

  extern __shared__ float smem[];
  float* Qs = smem;                    // [BQ][ldq]
  float* Ks = Qs + BQ * ldq;           // [BKEYS][Dh + 1]
  float* Vs = Ks + BKEYS * ldk;        // [BKEYS][Dh]
  float* Ps = Vs + BKEYS * Dh;         // [BQ][BKEYS]

  for (int i = threadIdx.x; i < BQ * Dh; i += blockDim.x) {
    int r = i / Dh, d = i - r * Dh;
    Qs[r * ldq + d] = r < rows ? to_float<T>(q[(size_t)(row0 + r) * q_stride + h * Dh + d]) : 0.f;
  }

  const int NC = (Dh + 31) / 32;       // head-dim columns per lane
  float acc[RQ][MAX_DH / 32];
  float m_run[RQ], l_run[RQ];
#pragma unroll
  for (int r = 0; r < RQ; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_DH / 32; ++c) acc[r][c] = 0.f;
  }

  const int last_pos = pos0 + rows - 1;
  int k_begin = 0;
  if (window > 0) k_begin = max(0, pos0 - window + 1) / BKEYS * BKEYS;
  const int* my_table = table + (size_t)req * table_stride;

  for (int k0 = k_begin; k0 <= last_pos; k0 += BKEYS) {
    __syncthreads();   // previous tile's reads are done (and Qs is written)
    for (int i = threadIdx.x; i < BKEYS * Dh; i += blockDim.x) {
      int j = i / Dh, d = i - j * Dh;
      int kp = k0 + j;
      float kv = 0.f, vv = 0.f;
      if (kp <= last_pos) {
        int page = my_table[kp / page_size];
        if (page > 0) {
          size_t src = (((size_t)page * page_size + (kp % page_size)) * Hkv + kvh) * Dh + d;
          kv = to_float<T>(kcache[src]);
          vv = to_float<T>(vcache[src]);
        }
      }
      Ks[j * ldk + d] = kv;
      Vs[j * Dh + d] = vv;
    }
    __syncthreads();

    const int kp = k0 + lane;
    const bool page_ok = kp <= last_pos && my_table[kp / page_size] > 0;
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;      // warp-uniform
      if (row >= rows) break;
      const int qpos = pos0 + row;
      const float* qr = Qs + row * ldq;
      const float* kr = Ks + lane * ldk;
      float s = 0.f;
      int d = 0;
      for (; d + 4 <= Dh; d += 4) {
        float4 qv = *reinterpret_cast<const float4*>(qr + d);
        s = fmaf(qv.x, kr[d], s);
        s = fmaf(qv.y, kr[d + 1], s);
        s = fmaf(qv.z, kr[d + 2], s);
        s = fmaf(qv.w, kr[d + 3], s);
      }
      for (; d < Dh; ++d) s = fmaf(qr[d], kr[d], s);      // head sizes that are no multiple of 4
      bool valid = page_ok && kp <= qpos && (window <= 0 || kp > qpos - window);
      s = valid ? s * scale : -INFINITY;
      float m_new = fmaxf(m_run[r], warp_max(s));
      float p = 0.f, alpha = 1.f;
      if (m_new > -INFINITY) {
        p = valid ? expf(s - m_new) : 0.f;
        alpha = expf(m_run[r] - m_new);    // exp(-inf) = 0 on the first visible tile
      }
      l_run[r] = l_run[r] * alpha + warp_sum(p);
      m_run[r] = m_new;
      Ps[row * BKEYS + lane] = p;
#pragma unroll
      for (int c = 0; c < MAX_DH / 32; ++c) acc[r][c] *= alpha;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;
      if (row >= rows) break;
      const float* pr = Ps + row * BKEYS;
      for (int j = 0; j < BKEYS; ++j) {
        float p = pr[j];
        const float* vr = Vs + j * Dh;
#pragma unroll
        for (int c = 0; c < MAX_DH / 32; ++c) {
          int d = lane + 32 * c;
          if (c < NC && d < Dh) acc[r][c] = fmaf(p, vr[d], acc[r][c]);
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RQ; ++r) {
    const int row = warp * RQ + r;
    if (row >= rows) break;
    float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    T* o = out + (size_t)(row0 + row) * ((size_t)H * Dh) + h * Dh;
#pragma unroll
    for (int c = 0; c < MAX_DH / 32; ++c) {
      int d = lane + 32 * c;
      if (c < NC && d < Dh) o[d] = from_float<T>(acc[r][c] * inv);
    }
  }
}

}  // namespace

AYK_EXPORT int ayk_attention_tile_rows() { return BQ; }

// out[T, H*Dh]; q rows of q_stride elements (head h at offset h*Dh); caches
// [pages, page_size, Hkv, Dh]; table[num_req, table_stride]; req_q_start[num_req+1]
// row offsets of each request's rows; req_pos0[num_req] absolute position of a
// request's first row.  total_rows = req_q_start[num_req] (known to the host).
AYK_EXPORT int ayk_attention_simt(void* out, const void* q, int q_stride, const void* kcache,
                                  const void* vcache, const int* table, int table_stride,
                                  const int* req_q_start, const int* req_pos0, int num_req,
                                  int total_rows, int H, int Hkv, int Dh, int page_size, float scale,
                                  int window, int dtype, cudaStream_t stream) {
  if (num_req == 0 || total_rows == 0) return 0;
  AYK_REQUIRE(Dh >= 1 && Dh <= MAX_DH, "ayk_attention_simt: head size %d is not in [1, %d]", Dh, MAX_DH);
  AYK_REQUIRE(Hkv >= 1 && H % Hkv == 0, "ayk_attention_simt: %d heads cannot share %d key/value heads", H, Hkv);
  AYK_REQUIRE(H <= 65535, "ayk_attention_simt: too many heads (%d)", H);
  int max_tiles = total_rows / BQ + num_req;   // sum of ceil(len / BQ) never exceeds this
  size_t smem = ((size_t)BQ * ((Dh + 3) & ~3) + (size_t)BKEYS * (Dh + 1) + (size_t)BKEYS * Dh + (size_t)BQ * BKEYS) * sizeof(float);
  dim3 grid(max_tiles, H);
  cudaError_t err;
  static size_t configured[2] = {0, 0};      // largest shared-memory size asked for so far, per dtype
  if (dtype == AYK_DTYPE_F32) {
    if (smem > configured[0]) {
      err = cudaFuncSetAttribute(attention_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_attention_simt: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[0] = smem;
    }
    ayk_launch(attention_simt_kernel<float>, grid, dim3(WARPS * 32), smem, stream,
        (float*)out, (const float*)q, q_stride, (const float*)kcache, (const float*)vcache, table, table_stride,
        req_q_start, req_pos0, num_req, H, Hkv, Dh, page_size, scale, window);
  } else if (dtype == AYK_DTYPE_BF16) {
    if (smem > configured[1]) {
      err = cudaFuncSetAttribute(attention_simt_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_attention_simt: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[1] = smem;
    }
    ayk_launch(attention_simt_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, stream,
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kcache,
        (const __nv_bfloat16*)vcache, table, table_stride, req_q_start, req_pos0, num_req, H, Hkv, Dh,
        page_size, scale, window);
  } else {
    return ayk_fail("ayk_attention_simt: unknown dtype %d", dtype);
  }
  return ayk_check_launch("ayk_attention_simt");
}
