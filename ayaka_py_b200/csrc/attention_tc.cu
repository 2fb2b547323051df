// Causal attention of prompt portions over the paged cache on the 5th-generation
// tensor cores (tcgen05), bfloat16, head size 64.
//
// One CTA takes up to 128 consecutive rows of one request and one head.  The
// keys and values of the request are walked 128 at a time: TMA brings each page
// (page_size keys x 64 x bf16, 128-byte swizzle) straight from the cache into a
// K tile and a V tile; S = Q K^T (128 x 128, float32) is made in tensor memory;
// four warps hold one row each per thread, read their row of S, apply scale and
// mask, keep the running maximum and sum in 32-bit (online softmax; scores are
// kept times log2(e) so that an exponential is one ex2), write P as bfloat16
// into shared memory in the MMA's swizzled layout;
// O_tile = P V (128 x 64) is made in tensor memory and added, per thread, to the
// row's running output in registers.  Formula and masking as in the general
// kernel (kernel/triton/paged_attention.py:295-355 in the reference, which walks
// the keys per query token without tensor cores).
//
// Warps 0..3: softmax and output (warp w owns TMEM lanes 32w..32w+31); warp 4:
// TMA producer (lane p brings page p of a tile); warp 5: MMA issue and TMEM
// allocation.  K/V tiles are double buffered; two CTAs share an SM.  The grid is
// (heads, row tiles) with the tiles that see the most keys first.  Every
// mbarrier wait is bounded; a wait that runs out records a code in the error
// word and the CTA winds down.
#include <cuda.h>
#include <math.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BQ = 128;          // rows per CTA
constexpr int BKV = 128;         // keys per iteration
constexpr int DH = 64;           // head size
constexpr int THREADS = 192;
constexpr int TILE_BYTES = 128 * 128;            // 128 rows x 64 bf16
constexpr int TMEM_COLS = 256;                   // S: columns 0..127, O: columns 128..191

struct AttnArgs {
  __nv_bfloat16* out;            // [T, H * 64]
  const int* table;              // [R, table_stride]
  const int* req_q_start;        // [R + 1]
  const int* req_pos0;           // [R]
  int* error;
  int table_stride, num_req, H, Hkv, page_size, window;
  float scale;
};

__global__ void __launch_bounds__(THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnArgs args) {
  // Row ranges, positions and block tables are the step's inputs: the set-up below (barriers, tensor
  // memory) runs while the kernel before this one finishes; pdl_wait() comes before the first access
  // to q, the cache or the output.
  // Which request and which of its 128-row tiles?  blockIdx.y counts tiles in the order "the last
  // tile of every request, then the one before it of every request that has one, ...": late tiles see
  // the most keys, and with the heads in blockIdx.x the whole grid starts its long CTAs first (measured:
  // 47 -> 30 us for two prompts of 1,024 tokens, where CTAs last from 8 to 31 us).  Every warp finds
  // its tile for itself, 32 requests at a time, from one load per lane and ballots.
  int tile = blockIdx.y, req = -1, q0 = 0, q_len = 0;
  {
    const int lane_id = threadIdx.x & 31;
    for (int r0 = 0; r0 < args.num_req && req < 0; r0 += 32) {
      const int r = r0 + lane_id;
      const int len = r < args.num_req ? args.req_q_start[r + 1] - args.req_q_start[r] : 0;
      const int tiles = (len + BQ - 1) / BQ;
      const int group_tiles = __reduce_add_sync(0xffffffffu, tiles);
      if (tile >= group_tiles) { tile -= group_tiles; continue; }
      for (int level = 0; req < 0; ++level) {            // ends: tile < group_tiles
        const unsigned have = __ballot_sync(0xffffffffu, tiles > level);
        const int n = __popc(have);
        if (tile < n) {
          const int src = __fns(have, 0, tile + 1);      // the lane of the (tile + 1)-th such request
          req = r0 + src;
          q_len = __shfl_sync(0xffffffffu, len, src);
          q0 = (__shfl_sync(0xffffffffu, tiles, src) - 1 - level) * BQ;
        } else {
          tile -= n;
        }
      }
    }
  }
  if (req < 0) { pdl_trigger(); return; }
  const int h = blockIdx.x, kvh = h / (args.H / args.Hkv);
  const int rows = min(BQ, q_len - q0);
  const int row0 = args.req_q_start[req] + q0;
  const int pos0 = args.req_pos0[req] + q0;
  const int last_pos = pos0 + rows - 1;
  int k_begin = 0;
  if (args.window > 0) k_begin = max(0, pos0 - args.window + 1) / BKV * BKV;
  const int num_tiles = (last_pos - k_begin) / BKV + 1;
  const int* my_table = args.table + (size_t)req * args.table_stride;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  if (raw & 1023u) {                 // the swizzled tiles need 1024-byte alignment; no slack is reserved for it
    if (threadIdx.x == 0) atomicExch(args.error, 18);
    pdl_trigger();
    return;
  }
  const uint32_t base = raw;
  const uint32_t q_tile = base;                                  // 16 KB
  const uint32_t kv_tile = base + TILE_BYTES;                    // 2 x (K 16 KB + V 16 KB)
  const uint32_t p_tile = kv_tile + 4 * TILE_BYTES;              // 2 x 16 KB (keys 0..63, 64..127)
  const uint32_t bars = p_tile + 2 * TILE_BYTES;
  const uint32_t q_full = bars, kv_full0 = bars + 8, kv_empty0 = bars + 24, s_full = bars + 40,
                 p_full = bars + 48, o_full = bars + 56, tmem_slot = bars + 64;
  uint8_t* generic_base = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(generic_base + (tmem_slot - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(kv_full0, 1); mbar_init(kv_full0 + 8, 1);
    mbar_init(kv_empty0, 1); mbar_init(kv_empty0 + 8, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;
  // Only now may the next kernel be scheduled: a dependent CTA that landed on this SM before the
  // allocation above could take tensor-memory columns that this CTA then waits for without bound,
  // while the dependent waits for this kernel.  (Kernels that can share an SM must ask for 512
  // columns or fewer between them.)
  pdl_trigger();

  pdl_wait();
  if (warp == 4) {
    // Lane 0 keeps the barriers; lane p brings page p of a tile (its own look-up in the block table
    // and its own two copies), so a tile costs one trip to the table instead of one per page.
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(q_tile, &map_q, h * DH, row0, q_full);
    }
    const int pages_per_tile = BKV / args.page_size;
    const uint32_t page_bytes = (uint32_t)args.page_size * 128u;
    bool ok = true;
    int issued = 0;
    for (int i = 0; i < num_tiles && ok; ++i) {
      const int b = i & 1;
      const int key0 = k_begin + i * BKV;
      int page = 0;
      if (lane < pages_per_tile) {
        const int logical = key0 / args.page_size + lane;
        page = logical < args.table_stride ? my_table[logical] : 0;               // beyond the table: the padding page
      }
      if (lane == 0) {
        if (i >= 2) ok = mbar_wait(kv_empty0 + 8 * b, (uint32_t)((i >> 1) & 1) ^ 1u, args.error, 11);
        if (ok) mbar_expect_tx(kv_full0 + 8 * b, 2 * TILE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < pages_per_tile) {
        const uint32_t k_dst = kv_tile + b * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
        tma_load_3d(k_dst + lane * page_bytes, &map_k, 0, kvh, page * args.page_size, kv_full0 + 8 * b);
        tma_load_3d(v_dst + lane * page_bytes, &map_v, 0, kvh, page * args.page_size, kv_full0 + 8 * b);
      }
      issued = i + 1;
    }
    if (!ok && lane == 0) {
      for (int i = max(0, issued - 2); i < issued; ++i)
        mbar_wait(kv_full0 + 8 * (i & 1), (uint32_t)(i >> 1) & 1u, args.error, 12);
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 0);
      constexpr uint32_t IDESC_O = make_idesc(BQ, DH, 1);
      bool ok = mbar_wait(q_full, 0u, args.error, 13);
      for (int i = 0; i < num_tiles && ok; ++i) {
        const int b = i & 1;
        ok = mbar_wait(kv_full0 + 8 * b, (uint32_t)(i >> 1) & 1u, args.error, 14);
        if (!ok) break;
        tc_fence_after();
        const uint32_t k_src = kv_tile + b * 2 * TILE_BYTES, v_src = k_src + TILE_BYTES;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)           // S = Q K^T over the head dimension
          umma(tmem_s, make_desc(q_tile + k * 32), make_desc(k_src + k * 32), IDESC_S, k > 0 ? 1u : 0u);
        umma_commit(s_full);
        ok = mbar_wait(p_full, (uint32_t)i & 1u, args.error, 15);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)          // O_tile = P V over the keys
          umma(tmem_o, make_desc(p_tile + (k >> 2) * TILE_BYTES + (k & 3) * 32), make_desc(v_src + k * 2048), IDESC_O,
               k > 0 ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(kv_empty0 + 8 * b);
      }
    }
    __syncwarp();
  } else {
    // Softmax: thread = row of the tile = TMEM lane.
    const int row = threadIdx.x;
    const int qpos = pos0 + row;
    const bool live = row < rows;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float o_acc[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) o_acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;          // the maximum is kept in units of log2(e)
    const float scale_log2 = args.scale * 1.4426950408889634f;
    uint8_t* p_row = generic_base + (p_tile - base) + row * 128;
    bool ok = true;
    for (int i = 0; i < num_tiles && ok; ++i) {
      // one lane per warp watches a barrier: 128 polling threads take issue slots from the other CTA of the SM
      if (lane == 0) ok = mbar_wait(s_full, (uint32_t)i & 1u, args.error, 16);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int key0 = k_begin + i * BKV;
      // The keys this row may see in this tile: key0 + j with lo <= j < hi.
      int hi = live ? min(BKV, qpos - key0 + 1) : 0;
      int lo = (args.window > 0) ? max(0, qpos - args.window + 1 - key0) : 0;
      if (hi < 0) hi = 0;
      const bool unmasked = lo <= 0 && hi >= BKV;  // every key of the tile is visible to this row
      // Scores are kept times log2(e), so that exp(s - m) is one ex2 each
      // (32-bit; the result is rounded to bfloat16 for the second product anyway).
      // The exponentials are what this kernel is made of (the special-function unit does 16 a clock
      // per SM): chunks of 32 keys that no row of the warp sees (above the diagonal, below the
      // window) are not read at all, and a row skips the arithmetic of chunks it does not see.
      const int warp_hi = __reduce_max_sync(0xffffffffu, hi), warp_lo = __reduce_min_sync(0xffffffffu, live ? lo : BKV);
      // Pass 1 over the row of S in tensor memory: its maximum.
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < BKV; c += 32) {
        if (c >= warp_hi || c + 32 <= warp_lo) continue;       // the same for the whole warp
        uint32_t r[32];
        tmem_ld32(tmem_s + lane_addr + c, r);
        tmem_ld_wait();
        if (unmasked) {
#pragma unroll
          for (int j = 0; j < 32; ++j) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        } else if (c < hi && c + 32 > lo) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c + j >= lo && c + j < hi) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        }
      }
      m_tile *= scale_log2;                        // the scale is positive: the maximum commutes with it
      const float m_new = fmaxf(m_run, m_tile);
      float alpha = 1.f, l_tile = 0.f;
      if (m_new > -INFINITY) alpha = fast_exp2(m_run - m_new);
      // Pass 2: exponentials, rounded to bfloat16, into the swizzled rows of P.
#pragma unroll
      for (int c = 0; c < BKV; c += 32) {
        const bool warp_sees = !(c >= warp_hi || c + 32 <= warp_lo);
        const bool row_sees = c < hi && c + 32 > lo;
        uint32_t r[32];
        if (warp_sees) { tmem_ld32(tmem_s + lane_addr + c, r); tmem_ld_wait(); }
#pragma unroll
        for (int g = 0; g < 32; g += 8) {           // 8 keys = one 16-byte chunk of the row of P
          uint32_t packed[4] = {0u, 0u, 0u, 0u};
          if (warp_sees && row_sees) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const int k0i = c + g + j;
              float p0 = fast_exp2(fmaf(__uint_as_float(r[g + j]), scale_log2, -m_new));
              float p1 = fast_exp2(fmaf(__uint_as_float(r[g + j + 1]), scale_log2, -m_new));
              if (!unmasked) {
                if (!(k0i >= lo && k0i < hi)) p0 = 0.f;
                if (!(k0i + 1 >= lo && k0i + 1 < hi)) p1 = 0.f;
              }
              l_tile += p0 + p1;                    // 32-bit sum of the unrounded values
              __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
              packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
            }
          }
          const int chunk = (c + g) >> 3;           // 0..15: tile = chunk / 8, 16-byte column = chunk % 8
          uint8_t* dst = p_row + (chunk >> 3) * TILE_BYTES + (((chunk & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
#pragma unroll
      for (int d = 0; d < DH; ++d) o_acc[d] *= alpha;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
      tc_fence_before();
      mbar_arrive(p_full);
      if (lane == 0) ok = mbar_wait(o_full, (uint32_t)i & 1u, args.error, 17);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_addr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o_acc[c + j] += __uint_as_float(r[j]);
      }
    }
    if (live && ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* o = args.out + (size_t)(row0 + row) * ((size_t)args.H * DH) + h * DH;
#pragma unroll
      for (int d = 0; d < DH; d += 8) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[d + j] * inv, o_acc[d + j + 1] * inv);
          w[j >> 1] = *reinterpret_cast<uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(o + d) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------- host --

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int* g_error_host = nullptr;
int* g_error_dev = nullptr;
std::mutex g_mutex;
bool g_configured = false;

struct CacheKey {
  const void* ptr; int tokens, heads, page;
  bool operator==(const CacheKey& o) const { return ptr == o.ptr && tokens == o.tokens && heads == o.heads && page == o.page; }
};
struct CacheHash {
  size_t operator()(const CacheKey& k) const { return std::hash<const void*>()(k.ptr) ^ ((size_t)k.tokens * 31u) ^ ((size_t)k.heads << 20) ^ (size_t)k.page; }
};
std::unordered_map<CacheKey, CUtensorMap, CacheHash> g_cache_maps;

constexpr size_t SMEM_BYTES = 7 * TILE_BYTES + 128;      // two CTAs fit one SM

int setup() {
  if (g_encode && g_error_host && g_configured) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (err != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
    return ayk_fail("ayk_attention_tc: cuTensorMapEncodeTiled is not available from this driver");
  g_encode = (EncodeTiledFn)fn;
  if (!g_error_host) {
    err = cudaHostAlloc((void**)&g_error_host, sizeof(int), cudaHostAllocMapped);
    if (err != cudaSuccess) return ayk_fail("ayk_attention_tc: cudaHostAlloc: %s", cudaGetErrorString(err));
    *g_error_host = 0;
    err = cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0);
    if (err != cudaSuccess) return ayk_fail("ayk_attention_tc: cudaHostGetDevicePointer: %s", cudaGetErrorString(err));
  }
  err = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (err != cudaSuccess) return ayk_fail("ayk_attention_tc: shared memory %zu: %s", SMEM_BYTES, cudaGetErrorString(err));
  g_configured = true;
  return 0;
}

// The cache of one layer as a 3-D tensor [tokens = pages * page_size][kv heads][64]; box = one page of one head.
int encode_cache(CUtensorMap* map, const void* ptr, int tokens, int heads, int page_size) {
  cuuint64_t dims[3] = {(cuuint64_t)DH, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)DH * 2, (cuuint64_t)heads * DH * 2};
  cuuint32_t box[3] = {(cuuint32_t)DH, 1, (cuuint32_t)page_size};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ayk_fail("ayk_attention_tc: cuTensorMapEncodeTiled(cache) failed with %d", (int)r);
  return 0;
}

int cache_map(CUtensorMap* map, const void* ptr, int tokens, int heads, int page_size) {
  std::lock_guard<std::mutex> lock(g_mutex);
  CacheKey key{ptr, tokens, heads, page_size};
  auto it = g_cache_maps.find(key);
  if (it != g_cache_maps.end()) { *map = it->second; return 0; }
  if (encode_cache(map, ptr, tokens, heads, page_size) != 0) return -1;
  g_cache_maps.emplace(key, *map);
  return 0;
}

}  // namespace

// 0 when the tensor-core kernel takes this geometry, else a text in ayk_last_error().
AYK_EXPORT int ayk_attention_tc_supported(int Dh, int page_size, int q_stride) {
  if (Dh != DH) return ayk_fail("ayk_attention_tc: head size %d (only 64)", Dh);
  if (page_size < 8 || page_size > BKV || (page_size & (page_size - 1)))
    return ayk_fail("ayk_attention_tc: page size %d is not a power of two in [8, 128]", page_size);
  if (q_stride % 8 != 0) return ayk_fail("ayk_attention_tc: query rows of %d elements are not 16-byte aligned", q_stride);
  return 0;
}

AYK_EXPORT int ayk_attention_tc_error() { return g_error_host ? *g_error_host : 0; }

// out [T, H*64] bf16; q: q_rows rows of q_stride elements (head h at column h*64);
// caches [pages, page_size, Hkv, 64] bf16.  The requests named by req_q_start / req_pos0 /
// table cover total_rows of q's rows (their row numbers are absolute); a step whose first rows
// are handled by another kernel passes the tail of the request arrays and the rows they cover.
AYK_EXPORT int ayk_attention_tc(void* out, const void* q, int q_stride, int q_rows, int total_rows, const void* kcache,
                                const void* vcache, int pages, const int* table, int table_stride,
                                const int* req_q_start, const int* req_pos0, int num_req, int H, int Hkv, int Dh,
                                int page_size, float scale, int window, cudaStream_t stream) {
  if (num_req == 0 || total_rows == 0) return 0;
  if (ayk_attention_tc_supported(Dh, page_size, q_stride) != 0) return -1;
  AYK_REQUIRE(q_rows >= total_rows, "ayk_attention_tc: %d rows named, q has %d", total_rows, q_rows);
  AYK_REQUIRE(Hkv >= 1 && H % Hkv == 0 && H <= 65535, "ayk_attention_tc: %d heads cannot share %d key/value heads", H, Hkv);
  AYK_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0 && (uintptr_t)out % 16 == 0,
              "ayk_attention_tc: operands must be 16-byte aligned");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (setup() != 0) return -1;
  }
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[2] = {(cuuint64_t)H * DH, (cuuint64_t)q_rows};
    cuuint64_t strides[1] = {(cuuint64_t)q_stride * 2};
    cuuint32_t box[2] = {(cuuint32_t)DH, (cuuint32_t)BQ};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ayk_fail("ayk_attention_tc: cuTensorMapEncodeTiled(q) failed with %d", (int)r);
  }
  if (cache_map(&mk, kcache, pages * page_size, Hkv, page_size) != 0) return -1;
  if (cache_map(&mv, vcache, pages * page_size, Hkv, page_size) != 0) return -1;
  AttnArgs args{(__nv_bfloat16*)out, table, req_q_start, req_pos0, g_error_dev, table_stride, num_req, H, Hkv, page_size,
                window, scale};
  AYK_REQUIRE(total_rows / BQ + num_req <= 65535 && H >= 1, "ayk_attention_tc: too many row tiles (%d rows, %d requests)", total_rows, num_req);
  dim3 grid(H, total_rows / BQ + num_req);      // heads fastest: see the tile order in the kernel
  ayk_launch(attention_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mq, mk, mv, args);
  return ayk_check_launch("ayk_attention_tc");
}
