// Decode attention: one query row per request over its paged keys and values,
// split along the context so that a batch of 1 still fills the GPU, then merged.
//
// The reference's decode path is a split-KV kernel over partitions of 512 keys
// with partial outputs and log-sum-exps in 32-bit scratch and a reduce kernel
// (kernel/triton/paged_attention.py:474-736).  Here a partition is 128 keys
// (PART) and the number of partitions is fixed per engine (those beyond a
// request's context return at once), so the launch does not depend on the
// context lengths and can be replayed from a CUDA graph; nothing but the block
// table is needed to find the keys.  Partials (unnormalised sum, running
// maximum, sum of exponentials) go to scratch [request, head, partition, Dh + 2]
// and a second kernel combines them in partition order.  (Letting the CTA that
// finishes last do the merge was measured slower: 70 against 59 us at 64
// requests, since every CTA then waits for its stores to become visible.)
//
// Two kernels.  bfloat16 with head sizes 32, 64, 128 runs on the tensor cores
// (decode_mma_kernel, below); measured on B200 at 64 requests x 25 heads x 570
// keys it moves 4.0 TB/s against 2.1 TB/s of the kernel that does the products
// on the FP32 pipe, which is bound by instruction issue (about 10,000 warp
// instructions per partition against under 1,000).  Everything else (32-bit,
// other head sizes) takes decode_split_kernel: scores with one key per lane,
// the weighted sum with one pair of head-dim columns per lane, then
// decode_merge_kernel.  Softmax, maxima and sums are 32-bit in both.
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

// bfloat16 on the tensor cores (mma.sync m16n8k16; one query row per head leaves
// no work for a 128-row tcgen05 tile).  One CTA per (request, key/value head, up to 8
// query heads that share it, partition); each of its 4 warps owns 32 keys.  A warp
// copies its keys and values into shared memory with cp.async (16-byte pieces,
// swizzled so that ldmatrix meets no bank conflict; rows outside the context are
// zero-filled), computes the scores of its keys as soon as the keys have landed
// (the query heads are rows 0..7 of the A operand, rows 8..15 stay zero), the
// softmax of its 32 keys in 32-bit, and the weighted sum with the values read
// through ldmatrix.trans.  The four warps' results are joined through shared
// memory into one partial per partition.  Probabilities are rounded to bfloat16
// for the second product, as in prefill.
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// cp.async of 16 bytes, or 16 bytes of zeros when !valid (src must still be a mapped address)
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
// 16-byte piece `piece` of row `row` (PPR pieces per row) sits at this piece index of the row:
// eight consecutive rows at one logical piece fall into eight different 16-byte bank groups.
template <int PPR> __device__ __forceinline__ int swizzled_piece(int row, int piece) {
  if constexpr (PPR >= 8) return piece ^ (row & 7);
  else return piece ^ ((row >> 1) & 3);          // PPR == 4: two rows per 128 bytes
}

//
// knew / vnew (or null): the key and value rows of the step's own tokens, [request, new_stride]; the
// key at the query's position is then taken from there, and the CTA of the first group of query heads
// also stores it into its page, so that no separate append kernel runs before this one.
// (Letting the partitions of a head form a cluster that merges through distributed shared memory
// was measured too: +1 % at one request, -7 % at 8 and -18 % at 64 requests, because the CTAs of
// empty partitions then hold their place until the cluster's barrier.  The merge stays a kernel.
// A persistent form, CTAs walking the live partitions with two buffers so that the next unit's
// copies fly while this one is worked on, was measured as well: 22 against 28 us at 64 requests of
// 100 keys, but 79 against 54 us at 570 keys, because with 64 KB per CTA only 12 warps fit on an SM
// and the kernel is bound by issue slots and latency, not by bandwidth.)
template <int DH>
__global__ void __launch_bounds__(WARPS * 32)
decode_mma_kernel(float* __restrict__ scratch, const __nv_bfloat16* __restrict__ q, int q_stride,
                  __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                  const int* __restrict__ table, int table_stride, const int* __restrict__ req_pos0,
                  int H, int Hkv, int group, int page_shift, float scale_log2, int window, int parts, int chunks, int rows,
                  const __nv_bfloat16* __restrict__ knew, const __nv_bfloat16* __restrict__ vnew, int new_stride, int settled) {
  pdl_trigger();
  static_assert(WARPS * 32 == PART, "each warp owns 32 keys of the partition");
  constexpr int KS = DH / 16;                    // k steps of the first product
  constexpr int PPR = DH / 8;                    // 16-byte pieces per row
  constexpr int NT = DH / 8;                     // output tiles of the second product
  constexpr int ROW_BYTES = DH * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // Grid (key/value head x group of query heads, request, partition): no division to find one's work,
  // and the partition is the slowest index, so the CTAs of the first partitions, which every request
  // has, get their places first; those of partitions beyond a request's context come last and
  // leave at once (measured inside a decode step at 8 requests: empty CTAs had held a place for
  // 3.6 us each while they waited to write a marker).
  const int part = blockIdx.z, r = blockIdx.y;
  const int kvh = chunks == 1 ? (int)blockIdx.x : (int)blockIdx.x / chunks;
  const int chunk = chunks == 1 ? 0 : (int)blockIdx.x % chunks;
  const int head0 = kvh * group + chunk * 8;               // the query head of A row 0
  const int rows_here = min(rows, group - chunk * 8);
  // Positions and block table are the step's inputs: they are read while the kernels before this one
  // (the product that makes q, k, v and the append to the cache) may still be running.
  const int pos = req_pos0[r];
  const int page_size = 1 << page_shift;
  const int wk0 = part * PART + warp * 32;       // this warp's first key
  // pages of this warp's keys: lane l holds the page of keys [wk0 + l * page_size, ...)
  const int first_logical = wk0 >> page_shift;
  int my_page = 0;
  if (lane < ((32 + page_size - 1) >> page_shift) && first_logical + lane < table_stride)
    my_page = table[(size_t)r * table_stride + first_logical + lane];
  int k_lo = part * PART;
  const int k_hi = min(pos + 1, k_lo + PART);
  if (window > 0) k_lo = max(k_lo, pos - window + 1);
  const bool empty = k_lo >= k_hi;               // the same for the whole CTA
  if (empty) return;                             // the merge knows from the position which partitions exist
  extern __shared__ __align__(128) unsigned char smem_dyn[];
  const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(smem_dyn);
  const uint32_t vs_base = ks_base + PART * ROW_BYTES;
  float* comb = reinterpret_cast<float*>(smem_dyn + 2 * PART * ROW_BYTES);      // [WARPS][rows][DH + 2]

  const int w_lo = max(k_lo, wk0), w_hi = min(k_hi, wk0 + 32);
  const bool warp_has_keys = !empty && w_lo < w_hi;
  float m_w = -INFINITY, l_w = 0.f;
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }

  // copies: lane covers piece (lane % PPR) of rows (lane / PPR) + i * (32 / PPR)   [PPR <= 32].
  // Keys and values lie at the same offsets of their caches: the offsets are worked out once
  // (32-bit, in elements; the host has checked that a cache has fewer than 2^32).
  constexpr int RPI = 32 / PPR;                  // rows per instruction
  constexpr int COPIES = 32 / RPI;
  const int my_piece = lane % PPR, my_row0 = lane / PPR;
  const uint32_t lane_off = (uint32_t)(kvh * DH) + (uint32_t)my_piece * 8u;
  int fresh_i = -1;                              // the copy that brings the key at the query's position, if it is this lane's
  uint32_t fresh_off = 0u;
  // `settled`: the caller vouches that whatever wrote the keys before the query's position is
  // complete (the engine: between two steps lies the upload of the step's inputs or a graph
  // launch, both full dependencies).  Their copies then start now, while the kernels before this
  // one (the product that makes q, k and v) may still be running.  Without that word the
  // kernel waits first: the call before this one may be the one that wrote them.
  if (!settled) pdl_wait();
  if (warp_has_keys) {
    const uint32_t row_elems = (uint32_t)(Hkv * DH);
    uint32_t off[COPIES];
    uint32_t ok_bits = 0u;
#pragma unroll
    for (int i = 0; i < COPIES; ++i) {
      const int row = my_row0 + i * RPI;         // within the warp's 32 keys
      const int key = wk0 + row;
      const int page = __shfl_sync(0xffffffffu, my_page, (key >> page_shift) - first_logical);
      const bool ok = key >= w_lo && key < w_hi && page > 0;
      off[i] = ok ? (((uint32_t)page << page_shift) + (uint32_t)(key & (page_size - 1))) * row_elems + lane_off : 0u;
      if (key == pos && ok) { fresh_i = i; fresh_off = off[i]; }
      else ok_bits |= (ok ? 1u : 0u) << i;       // the fresh row's place stays empty until after the wait
    }
#pragma unroll
    for (int mat = 0; mat < 2; ++mat) {
      const __nv_bfloat16* cache = mat == 0 ? kcache : vcache;
      const uint32_t base = (mat == 0 ? ks_base : vs_base) + (uint32_t)(warp * 32 + my_row0) * ROW_BYTES;
#pragma unroll
      for (int i = 0; i < COPIES; ++i) {
        const int row = my_row0 + i * RPI;
        if (i != fresh_i)
          cp_async16_zfill(base + (uint32_t)(i * RPI) * ROW_BYTES + swizzled_piece<PPR>(row, my_piece) * 16, cache + off[i],
                           (ok_bits >> i) & 1u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  pdl_wait();
  if (warp_has_keys) {
    if (fresh_i >= 0) {
      // the key and value at the query's position: made by the kernels just before this one
      const int row = my_row0 + fresh_i * RPI;
      const uint32_t place = (uint32_t)(warp * 32 + row) * ROW_BYTES + swizzled_piece<PPR>(row, my_piece) * 16;
#pragma unroll
      for (int mat = 0; mat < 2; ++mat) {
        __nv_bfloat16* cache = mat == 0 ? kcache : vcache;
        const __nv_bfloat16* src = cache + fresh_off;
        if (knew != nullptr) {                   // not in the cache yet
          src = (mat == 0 ? knew : vnew) + (size_t)r * new_stride + lane_off;
          if (chunk == 0)                        // one CTA per key/value head files it
            *reinterpret_cast<uint4*>(cache + fresh_off) = *reinterpret_cast<const uint4*>(src);
        }
        cp_async16_zfill((mat == 0 ? ks_base : vs_base) + place, src, true);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the query rows as A operands (rows beyond the group stay zero)
    uint32_t qa[KS][2];
    {
      const bool row_ok = g < rows_here;
      const __nv_bfloat16* qrow = q + (size_t)r * q_stride + (size_t)(head0 + g) * DH;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        qa[ks][0] = row_ok ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
        qa[ks][1] = row_ok ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    // scores: 4 tiles of 8 keys
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sc[j][0] = 0.f; sc[j][1] = 0.f; sc[j][2] = 0.f; sc[j][3] = 0.f;
      const int row = j * 8 + (lane & 7);        // the row whose address this lane supplies
#pragma unroll
      for (int h = 0; h < PPR / 4; ++h) {
        uint32_t kb[4];
        ldmatrix_x4(kb, ks_base + (warp * 32 + row) * ROW_BYTES + swizzled_piece<PPR>(row, 4 * h + (lane >> 3)) * 16);
        mma_bf16(sc[j], qa[2 * h][0], qa[2 * h][1], kb[0], kb[1]);
        mma_bf16(sc[j], qa[2 * h + 1][0], qa[2 * h + 1][1], kb[2], kb[3]);
      }
    }
    float mb = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = wk0 + j * 8 + 2 * t + e;
        sc[j][e] = (key >= w_lo && key < w_hi) ? sc[j][e] * scale_log2 : -INFINITY;
        mb = fmaxf(mb, sc[j][e]);
      }
    }
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
    m_w = mb;                                    // finite: the warp has a visible key
    uint32_t pa[2][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = exp2f(sc[j][0] - m_w), p1 = exp2f(sc[j][1] - m_w);
      l_w += p0 + p1;
      pa[j >> 1][j & 1] = pack_bf16(p0, p1);
    }
    l_w += __shfl_xor_sync(0xffffffffu, l_w, 1);
    l_w += __shfl_xor_sync(0xffffffffu, l_w, 2);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int row = s * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vs_base + (warp * 32 + row) * ROW_BYTES + swizzled_piece<PPR>(row, 2 * np + (lane >> 4)) * 16);
        mma_bf16(o[2 * np], pa[s][0], pa[s][1], vb[0], vb[1]);
        mma_bf16(o[2 * np + 1], pa[s][0], pa[s][1], vb[2], vb[3]);
      }
    }
  }
  // join the warps
  if (!empty) {
    if (g < rows_here) {
      float* mine = comb + ((size_t)warp * rows + g) * (DH + 2);
#pragma unroll
      for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(mine + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
      if (t == 0) { mine[DH] = m_w; mine[DH + 1] = l_w; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_here * DH; idx += WARPS * 32) {
      const int row = idx / DH, d = idx % DH;
      float mw[WARPS], m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) { mw[w] = comb[((size_t)w * rows + row) * (DH + 2) + DH]; m = fmaxf(m, mw[w]); }
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        if (mw[w] > -INFINITY) {
          const float f = exp2f(mw[w] - m);
          acc = fmaf(comb[((size_t)w * rows + row) * (DH + 2) + d], f, acc);
          l = fmaf(comb[((size_t)w * rows + row) * (DH + 2) + DH + 1], f, l);
        }
      }
      float* dst = scratch + ((size_t)(r * H + head0 + row) * parts + part) * (DH + 2);
      dst[d] = acc;
      if (d == 0) { dst[DH] = m * 0.6931471805599453f; dst[DH + 1] = l; }    // the merge works with natural exponentials
    }
  }
}

// Combines the partitions of one (request, head) in partition order.  Eight partitions at a time:
// every load of the eight (maximum, sum, value) first, so that the kernel, which sits between the
// attention and the next product of a decode step, makes one trip to L2 instead of three.
// Which partitions hold keys follows from the request's position and the window, as in the
// kernels that fill them; the others' scratch is never read (nobody wrote it).
// exp() of the merge: the bfloat16 path takes ex2.approx (2 instructions; the kernel runs its code
// once, so every instruction counts), the 32-bit path the full-precision function.
template <typename T> __device__ __forceinline__ float merge_exp(float x) {
  if constexpr (sizeof(T) == 2) return fast_exp2(x * 1.4426950408889634f);
  else return expf(x);
}

template <typename T>
__global__ void decode_merge_kernel(T* __restrict__ out, const float* __restrict__ scratch, int H, int Dh, int parts,
                                    const int* __restrict__ req_pos0, int window) {
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y;
  const int pos = req_pos0[r];                   // the step's own input: read before the wait
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  pdl_wait();
  const float* base = scratch + (size_t)(r * H + h) * parts * (Dh + 2);
  T* o = out + ((size_t)r * H + h) * Dh;
  for (int d = threadIdx.x; d < Dh; d += blockDim.x) {
    float m = -INFINITY, l = 0.f, acc = 0.f;
    for (int s0 = 0; s0 < parts; s0 += 8) {
      float ms[8], ls[8], vs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int part = s0 + i;
        const bool in = part < parts && max(part * PART, first_key) < min(pos + 1, (part + 1) * PART);
        const float* p = base + (size_t)(in ? part : 0) * (Dh + 2);
        ms[i] = in ? p[Dh] : -INFINITY;
        ls[i] = in ? p[Dh + 1] : 0.f;
        vs[i] = in ? p[d] : 0.f;
      }
      float m_new = m;
#pragma unroll
      for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, ms[i]);
      if (m_new > -INFINITY) {
        const float f = merge_exp<T>(m - m_new);   // exp(-inf) = 0 before the first live partition
        acc *= f; l *= f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (ms[i] > -INFINITY) {
            const float w = merge_exp<T>(ms[i] - m_new);
            acc = fmaf(vs[i], w, acc);
            l = fmaf(ls[i], w, l);
          }
        }
        m = m_new;
      }
    }
    o[d] = from_float<T>(l > 0.f ? acc / l : 0.f);
  }
}

}  // namespace

AYK_EXPORT int ayk_attention_decode_part() { return PART; }

extern "C" int ayk_kv_append(void* kcache, void* vcache, const void* k, const void* v, int row_stride, const int* row_req,
                             const int* pos, const int* table, int table_stride, int page_size, int T, int width, int dtype,
                             cudaStream_t stream);

// One query row per request: out[R, H*Dh]; q rows of q_stride elements; caches
// [pages, page_size, Hkv, Dh]; table[R, table_stride]; req_pos0[R] = the row's
// position.  parts = ceil(longest possible context / 128) (fixed per engine);
// scratch holds R * H * parts * (Dh + 2) floats.  knew, vnew (or null): this step's key and
// value rows [R, new_stride], not yet in the cache: they are stored at (request r, position
// req_pos0[r]) on the way (row_req[r] must be r: one row per request, in order).  cache_pages: pages of
// a cache tensor (the tensor-core kernel addresses a cache with 32-bit element offsets).  settled != 0:
// every earlier write of the cache rows before the requests' positions is complete (no kernel that
// wrote them can still be running): the tensor-core kernel then copies them before it waits for the
// kernels launched before it.
AYK_EXPORT int ayk_attention_decode(void* out, const void* q, int q_stride, void* kcache, void* vcache,
                                    const int* table, int table_stride, const int* req_pos0, int R, int H, int Hkv,
                                    int Dh, int page_size, float scale, int window, int parts, float* scratch,
                                    const void* knew, const void* vnew, int new_stride, const int* row_req,
                                    long long cache_pages, int settled, int dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  AYK_REQUIRE(Dh >= 16 && Dh % 16 == 0 && Dh <= MAX_DH, "ayk_attention_decode: head size %d is not a multiple of 16 in [16, %d]", Dh, MAX_DH);
  AYK_REQUIRE(Hkv >= 1 && H % Hkv == 0, "ayk_attention_decode: %d heads cannot share %d key/value heads", H, Hkv);
  AYK_REQUIRE(parts >= 1 && parts <= 65535 && H <= 65535 && R <= 65535, "ayk_attention_decode: grid too large (requests %d, heads %d, parts %d)", R, H, parts);
  AYK_REQUIRE(dtype == AYK_DTYPE_F32 || dtype == AYK_DTYPE_BF16, "ayk_attention_decode: unknown dtype %d", dtype);
  AYK_REQUIRE((knew == nullptr) == (vnew == nullptr) && (knew == nullptr || row_req != nullptr),
              "ayk_attention_decode: new keys come with new values and the rows' requests");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const unsigned long long cache_elems = (unsigned long long)cache_pages * page_size * Hkv * Dh;    // of one cache tensor
  const bool mma_ok = dtype == AYK_DTYPE_BF16 && (Dh == 32 || Dh == 64 || Dh == 128) && (1 << page_shift) == page_size &&
                      page_size >= 4 && q_stride % 2 == 0 && (uintptr_t)q % 4 == 0 && (uintptr_t)kcache % 16 == 0 &&
                      (uintptr_t)vcache % 16 == 0 && cache_elems < (1ull << 32) &&
                      (knew == nullptr || (new_stride % 8 == 0 && (uintptr_t)knew % 16 == 0 && (uintptr_t)vnew % 16 == 0));
  if (mma_ok) {
    const int group = H / Hkv, chunks = (group + 7) / 8, rows = group < 8 ? group : 8;
    const long items = (long)R * Hkv * chunks * parts;
    AYK_REQUIRE(items <= 0x7fffffffL, "ayk_attention_decode: too many partitions (%ld)", items);
    const float scale_log2 = scale * 1.4426950408889634f;
    const size_t smem = 2 * (size_t)PART * Dh * 2 + (size_t)WARPS * rows * (Dh + 2) * sizeof(float);
    static AykPerDevice configured_on;
    bool& configured = configured_on.here();
    if (!configured) {
      const int most = 2 * PART * 128 * 2 + WARPS * 8 * (128 + 2) * 4;
      if (cudaFuncSetAttribute(decode_mma_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
          cudaFuncSetAttribute(decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
          cudaFuncSetAttribute(decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess)
        return ayk_fail("ayk_attention_decode: cannot reserve %d bytes of shared memory", most);
      configured = true;
    }
#define AYK_DECODE_MMA(D)                                                                                              \
  ayk_launch(decode_mma_kernel<D>, dim3(Hkv * chunks, R, parts), dim3(WARPS * 32), smem, stream, scratch,                      \
             (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, table, table_stride,    \
             req_pos0, H, Hkv, group, page_shift, scale_log2, window, parts, chunks, rows, (const __nv_bfloat16*)knew,  \
             (const __nv_bfloat16*)vnew, new_stride, settled)
    if (Dh == 32) AYK_DECODE_MMA(32); else if (Dh == 64) AYK_DECODE_MMA(64); else AYK_DECODE_MMA(128);
#undef AYK_DECODE_MMA
    ayk_launch(decode_merge_kernel<__nv_bfloat16>, dim3(R, H), dim3(Dh <= 32 ? 32 : (Dh <= 64 ? 64 : 128)), 0, stream,
               (__nv_bfloat16*)out, (const float*)scratch, H, Dh, parts, req_pos0, window);
    return ayk_check_launch("ayk_attention_decode");
  }
  if (knew != nullptr &&
      ayk_kv_append(kcache, vcache, knew, vnew, new_stride, row_req, req_pos0, table, table_stride, page_size, R, Hkv * Dh,
                    dtype, stream) != 0)
    return -1;
  dim3 grid(R, H, parts), mgrid(R, H);
  const int mthreads = Dh <= 32 ? 32 : (Dh <= 64 ? 64 : 128);
  if (dtype == AYK_DTYPE_F32) {
    ayk_launch(decode_split_kernel<float>, grid, dim3(WARPS * 32), 0, stream, scratch, (const float*)q, q_stride,
               (const float*)kcache, (const float*)vcache, table, table_stride, req_pos0, H, Hkv, Dh, page_size, scale,
               window, parts);
    ayk_launch(decode_merge_kernel<float>, mgrid, dim3(mthreads), 0, stream, (float*)out, (const float*)scratch, H, Dh, parts, req_pos0, window);
  } else {
    ayk_launch(decode_split_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), 0, stream, scratch, (const __nv_bfloat16*)q,
               q_stride, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, table, table_stride, req_pos0, H, Hkv,
               Dh, page_size, scale, window, parts);
    ayk_launch(decode_merge_kernel<__nv_bfloat16>, mgrid, dim3(mthreads), 0, stream, (__nv_bfloat16*)out,
               (const float*)scratch, H, Dh, parts, req_pos0, window);
  }
  return ayk_check_launch("ayk_attention_decode");
}
