// Causal attention of prompt portions over the paged cache on the 5th-generation
// tensor cores (tcgen05), bfloat16, head size 64.
//
// One CTA takes up to 128 consecutive rows of one request and one head.  The
// keys and values of the request are walked 128 at a time: TMA brings each page
// (page_size keys x 64 x bf16, 128-byte swizzle) straight from the cache into a
// K tile and a V tile; S = Q K^T (128 x 128, float32) is made in tensor memory;
// eight warps hold half a row each per thread (warps w and w + 4 share the rows
// 32 (w % 4) ... + 31, the first takes keys 0..63 of the tile, the second keys
// 64..127), read their half row of S, apply scale and mask, keep the running
// maximum and sum in 32-bit (online softmax; scores are kept times log2(e) so
// that an exponential is one ex2), write P as bfloat16 into shared memory in the
// MMA's swizzled layout; O_tile = P V (128 x 64) is made in tensor memory and
// added, per thread, to the row's running output in registers (32 columns per
// thread).  Formula and masking as in the general kernel
// (kernel/triton/paged_attention.py:295-355 in the reference, which walks the
// keys per query token without tensor cores).
//
// The key tiles of a CTA overlap: S lives in two buffers of tensor memory, and
// the MMA warp issues Q K^T of tile j + 1 before it waits for P of tile j, so the
// softmax of a tile never waits for its scores; O_tile of tile j is written into
// the columns that S of tile j has left (its scores are read by then) and is
// picked up by the threads one tile later, between the two passes over S of
// tile j + 1.  A CTA's time per key tile is then the softmax alone (the chain
// S -> softmax -> P -> P V -> O took 4.1 us per tile, and the CTA of a prompt's
// last rows walks 8 tiles one after the other).
//
// Warps 0..7: softmax and output; warp 8: TMA producer (lane p brings page p of
// a tile); warp 9: MMA issue and TMEM allocation.  K/V tiles are double
// buffered; two CTAs share an SM.  The grid is (heads, row tiles) with the tiles
// that see the most keys first.  Every mbarrier wait is bounded; a wait that
// runs out records a code in the error word and the CTA winds down.
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
constexpr int SOFTMAX_WARPS = 8;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr int TILE_BYTES = 128 * 128;            // 128 rows x 64 bf16
constexpr int TMEM_COLS = 256;                   // two buffers of 128 columns: S, then O_tile in the first 64 of them

struct AttnArgs {
  __nv_bfloat16* out;            // [T, H * 64]
  const int* table;              // [R, table_stride]
  const int* req_q_start;        // [R + 1]
  const int* req_pos0;           // [R]
  int* error;
  int table_stride, num_req, H, Hkv, page_size, window;
  float scale;
  long long* trace;              // cycle marks of CTA (0, 0) when built with -DAYK_TRACE, else unused
};

#ifdef AYK_TRACE
__device__ __forceinline__ void mark(const AttnArgs& a, int slot) {
  if (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && slot < 512) a.trace[slot] = clock64();
}
// every CTA's span: [512 + 4 * cta] = start ns, end ns, key tiles, SM
__device__ __forceinline__ void span(const AttnArgs& a, int which, long long value) {
  if (a.trace) a.trace[512 + 4 * (blockIdx.y * gridDim.x + blockIdx.x) + which] = value;
}
__device__ __forceinline__ long long now_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int sm_id() {
  int v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
#else
__device__ __forceinline__ void mark(const AttnArgs&, int) {}
__device__ __forceinline__ void span(const AttnArgs&, int, long long) {}
__device__ __forceinline__ long long now_ns() { return 0; }
__device__ __forceinline__ int sm_id() { return 0; }
#endif
long long* g_trace = nullptr;

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
  const uint32_t q_full = bars, k_full0 = bars + 8, k_empty0 = bars + 24, v_full0 = bars + 40, v_empty0 = bars + 56,
                 s_full0 = bars + 72, s_free0 = bars + 88, p_full = bars + 104, o_full = bars + 112, tmem_slot = bars + 120;
  const uint32_t pair_at = bars + 128;                           // one float per row: what its two halves tell each other
  uint8_t* generic_base = smem_raw + (base - raw);
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(generic_base + (tmem_slot - base));
  volatile float* pair_slot = (volatile float*)(generic_base + (pair_at - base));    // [128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full0, 1); mbar_init(k_full0 + 8, 1);
    mbar_init(k_empty0, 1); mbar_init(k_empty0 + 8, 1);
    mbar_init(v_full0, 1); mbar_init(v_full0 + 8, 1);
    mbar_init(v_empty0, 1); mbar_init(v_empty0 + 8, 1);
    mbar_init(s_full0, 1); mbar_init(s_full0 + 8, 1);
    mbar_init(s_free0, SOFTMAX_WARPS); mbar_init(s_free0 + 8, SOFTMAX_WARPS);
    mbar_init(p_full, SOFTMAX_WARPS);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == SOFTMAX_WARPS + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Only now may the next kernel be scheduled: a dependent CTA that landed on this SM before the
  // allocation above could take tensor-memory columns that this CTA then waits for without bound,
  // while the dependent waits for this kernel.  (Kernels that can share an SM must ask for 512
  // columns or fewer between them.)
  pdl_trigger();

  pdl_wait();
  if (threadIdx.x == 0) { mark(args, 0); span(args, 0, now_ns()); span(args, 2, num_tiles); span(args, 3, sm_id()); }
  if (warp == SOFTMAX_WARPS) {
    // Lane 0 keeps the barriers; lane p brings page p of a tile (its own look-up in the block table
    // and its own two copies), so a tile costs one trip to the table instead of one per page.
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(q_tile, &map_q, h * DH, row0, q_full);
    }
    // Keys run one tile ahead of values: K of tile t is wanted when its scores are issued, a whole
    // softmax before the values of tile t - 1 are; a K buffer is free as soon as its scores are
    // made, a V buffer only after its P V.  So the order of the copies is K(0), K(1), V(0), K(2),
    // V(1), ...: with K and V of a tile copied together, after the P V two tiles back, a CTA spent
    // most of a tile's time waiting for keys.
    const int pages_per_tile = BKV / args.page_size;
    const uint32_t page_bytes = (uint32_t)args.page_size * 128u;
    auto pages_of = [&](int t) -> int {               // lane p: the page of keys [p, p + 1) * page_size of tile t
      int page = 0;
      if (lane < pages_per_tile) {
        const int logical = (k_begin + t * BKV) / args.page_size + lane;
        page = logical < args.table_stride ? my_table[logical] : 0;               // beyond the table: the padding page
      }
      return page;
    };
    // one matrix (keys or values) of tile t into its buffer: lane 0 waits for the buffer and arms the barrier
    auto bring = [&](int t, int page, bool values) -> bool {
      const int b = t & 1;
      const uint32_t full = (values ? v_full0 : k_full0) + 8 * b, empty = (values ? v_empty0 : k_empty0) + 8 * b;
      bool fine = true;
      if (lane == 0) {
        if (t >= 2) fine = mbar_wait(empty, (uint32_t)((t >> 1) & 1) ^ 1u, args.error, 11);
        if (fine) mbar_expect_tx(full, TILE_BYTES);
      }
      fine = __shfl_sync(0xffffffffu, fine ? 1 : 0, 0) != 0;
      if (lane == 0) mark(args, (values ? 64 : 32) + t);
      if (fine && lane < pages_per_tile)
        tma_load_3d(kv_tile + b * 2 * TILE_BYTES + (values ? TILE_BYTES : 0) + lane * page_bytes, values ? &map_v : &map_k, 0,
                    kvh, page * args.page_size, full);
      return fine;
    };
    int page_now = pages_of(0);
    bool ok = bring(0, page_now, false);
    int k_issued = ok ? 1 : 0, v_issued = 0;
    for (int i = 0; i < num_tiles && ok; ++i) {
      int page_next = 0;
      if (i + 1 < num_tiles) {
        page_next = pages_of(i + 1);
        ok = bring(i + 1, page_next, false);
        if (!ok) break;
        k_issued = i + 2;
      }
      ok = bring(i, page_now, true);
      if (!ok) break;
      v_issued = i + 1;
      page_now = page_next;
    }
    if (!ok && lane == 0) {                          // nobody may be consuming any more: wait for the copies in flight
      for (int t = max(0, k_issued - 2); t < k_issued; ++t)
        mbar_wait(k_full0 + 8 * (t & 1), (uint32_t)(t >> 1) & 1u, args.error, 12);
      for (int t = max(0, v_issued - 2); t < v_issued; ++t)
        mbar_wait(v_full0 + 8 * (t & 1), (uint32_t)(t >> 1) & 1u, args.error, 12);
    }
    __syncwarp();
  } else if (warp == SOFTMAX_WARPS + 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 0);
      constexpr uint32_t IDESC_O = make_idesc(BQ, DH, 1);
      // S of tile t into buffer t % 2: needs its keys, and the buffer given back by the threads that
      // read O_tile of tile t - 2 out of it.
      auto scores = [&](int t) -> bool {
        const int b = t & 1;
        if (!mbar_wait(k_full0 + 8 * b, (uint32_t)(t >> 1) & 1u, args.error, 14)) return false;
        if (t >= 2 && !mbar_wait(s_free0 + 8 * b, ((uint32_t)(t >> 1) & 1u) ^ 1u, args.error, 19)) return false;
        tc_fence_after();
        mark(args, 96 + t);
        const uint32_t k_src = kv_tile + b * 2 * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)           // S = Q K^T over the head dimension
          umma(tmem_base + 128u * b, make_desc(q_tile + k * 32), make_desc(k_src + k * 32), IDESC_S, k > 0 ? 1u : 0u);
        umma_commit(s_full0 + 8 * b);
        umma_commit(k_empty0 + 8 * b);              // the keys' buffer is free once the scores are made
        return true;
      };
      bool ok = mbar_wait(q_full, 0u, args.error, 13);
      if (ok) ok = scores(0);
      for (int i = 0; i < num_tiles && ok; ++i) {
        const int b = i & 1;
        if (i + 1 < num_tiles) {                    // the next tile's scores are made while this tile's softmax runs
          ok = scores(i + 1);
          if (!ok) break;
        }
        ok = mbar_wait(v_full0 + 8 * b, (uint32_t)(i >> 1) & 1u, args.error, 14) &&
             mbar_wait(p_full, (uint32_t)i & 1u, args.error, 15);
        if (!ok) break;
        tc_fence_after();
        mark(args, 128 + i);
        const uint32_t v_src = kv_tile + b * 2 * TILE_BYTES + TILE_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)          // O_tile = P V over the keys, into the columns that S of this tile has left
          umma(tmem_base + 128u * b, make_desc(p_tile + (k >> 2) * TILE_BYTES + (k & 3) * 32), make_desc(v_src + k * 2048),
               IDESC_O, k > 0 ? 1u : 0u);
        umma_commit(o_full);
        umma_commit(v_empty0 + 8 * b);
      }
    }
    __syncwarp();
  } else {
    // Softmax: TMEM lane = row of the tile; warps w and w + 4 share the rows 32 (w % 4) ... + 31.
    const int half = warp >> 2;                    // 0: keys 0..63 and output columns 0..31; 1: keys 64..127, columns 32..63
    const int row = (warp & 3) * 32 + lane;
    const int qpos = pos0 + row;
    const bool live = row < rows;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int pair_barrier = 1 + (warp & 3);       // named barrier of the two warps that share these rows
    constexpr int OC = DH / 2;                     // output columns per thread
    float o_acc[OC];
#pragma unroll
    for (int d = 0; d < OC; ++d) o_acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;          // the maximum is kept in units of log2(e); l_run covers this thread's keys only
    float alpha_prev = 1.f;                        // the factor that belongs to the O_tile still to be picked up
    const float scale_log2 = args.scale * 1.4426950408889634f;
    uint8_t* p_row = generic_base + (p_tile - base) + half * TILE_BYTES + row * 128;
    const int c0 = half * 64;                      // this thread's first key of a tile
    const uint32_t row_xor = (uint32_t)(row & 7) << 4;      // the 128-byte swizzle: 16-byte column ^ (row % 8)
    bool ok = true;
    // The two threads of a row agree on one number (the larger of their maxima, or the sum of their
    // sums): the first half leaves its value, the second combines it with its own and leaves the
    // result, the first picks that up.  Two barriers of the two warps; shared memory has room for one
    // float per row and no more, if two CTAs are to share an SM.
    auto agree = [&](float mine, bool take_max) -> float {
      float both;
      if (half == 0) {
        pair_slot[row] = mine;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        both = pair_slot[row];
      } else {
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        const float other = pair_slot[row];
        both = take_max ? fmaxf(mine, other) : mine + other;
        pair_slot[row] = both;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
      }
      return both;
    };
    // O_tile of tile t: out of buffer t % 2, scaled into the running output, and the buffer given back.
    auto pick_up = [&](int t, float alpha) {
      const uint32_t o_at = tmem_base + 128u * (t & 1) + lane_addr + (uint32_t)(half * OC);
#pragma unroll
      for (int c = 0; c < OC; c += 16) {
        uint32_t r[16];
        tmem_ld16(o_at + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) o_acc[c + j] = fmaf(o_acc[c + j], alpha, __uint_as_float(r[j]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free0 + 8 * (t & 1));
    };
    for (int i = 0; i < num_tiles && ok; ++i) {
      const uint32_t s_at = tmem_base + 128u * (i & 1) + lane_addr + (uint32_t)c0;
      // one lane per warp watches a barrier: 256 polling threads take issue slots from the other CTA of the SM
      if (lane == 0) ok = mbar_wait(s_full0 + 8 * (i & 1), (uint32_t)(i >> 1) & 1u, args.error, 16);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      if (threadIdx.x == 0) mark(args, 160 + i);
      const int key0 = k_begin + i * BKV + c0;     // the first key of this thread's half
      // The keys this thread may see in its half of the tile: key0 + j with lo <= j < hi.
      int hi = live ? min(64, qpos - key0 + 1) : 0;
      int lo = (args.window > 0) ? max(0, qpos - args.window + 1 - key0) : 0;
      if (hi < 0) hi = 0;
      // Most tiles lie wholly below the diagonal (and inside the window): every key is visible to every
      // row of the warp, and the passes below run without a single comparison.  The kernel is bound by
      // the instructions it issues (exponentials are a quarter of the special-function unit's rate), so
      // the tiles on the diagonal get a copy of the passes of their own.
      const bool plain = __all_sync(0xffffffffu, lo <= 0 && hi >= 64);
      const int warp_hi = __reduce_max_sync(0xffffffffu, hi), warp_lo = __reduce_min_sync(0xffffffffu, live ? lo : 64);
      // Pass 1 over the half row of S in tensor memory: its maximum.  (16 columns at a time: with the
      // running output in registers there is no room for 32.)
      float m_tile = -INFINITY;
      if (plain) {
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
          uint32_t r[16];
          tmem_ld16(s_at + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
          if (c >= warp_hi || c + 16 <= warp_lo) continue;       // the same for the whole warp: not read at all
          uint32_t r[16];
          tmem_ld16(s_at + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c + j >= lo && c + j < hi) m_tile = fmaxf(m_tile, __uint_as_float(r[j]));
        }
      }
      if (threadIdx.x == 0) mark(args, 192 + i);
      m_tile = agree(m_tile, true);                // the row's maximum over the whole tile
      if (threadIdx.x == 0) mark(args, 224 + i);
      m_tile *= scale_log2;                        // the scale is positive: the maximum commutes with it
      const float m_new = fmaxf(m_run, m_tile);
      float alpha = 1.f, l_tile = 0.f;
      if (m_new > -INFINITY) alpha = fast_exp2(m_run - m_new);
      // Between the passes: O_tile of the tile before is in tensor memory by now (its P was handed
      // over a whole pass ago), and P's place in shared memory is free once it is.
      if (i > 0) {
        if (lane == 0) ok = mbar_wait(o_full, (uint32_t)(i - 1) & 1u, args.error, 17);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tc_fence_after();
        pick_up(i - 1, alpha_prev);
      }
      if (threadIdx.x == 0) mark(args, 256 + i);
      // Pass 2: exponentials (scores are kept times log2(e), so one ex2 each), rounded to bfloat16,
      // into the swizzled rows of P; their 32-bit sum, unrounded, into l_tile.
      if (plain) {
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
          uint32_t r[16];
          tmem_ld16(s_at + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 16; g += 8) {         // 8 keys = one 16-byte chunk of the row of P
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(r[g + j]), scale_log2, -m_new));
              const float p1 = fast_exp2(fmaf(__uint_as_float(r[g + j + 1]), scale_log2, -m_new));
              l_tile += p0 + p1;
              __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
              packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
            }
            *reinterpret_cast<uint4*>(p_row + ((uint32_t)(((c + g) >> 3) << 4) ^ row_xor)) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; c += 16) {
          const bool warp_sees = !(c >= warp_hi || c + 16 <= warp_lo);
          const bool row_sees = c < hi && c + 16 > lo;
          uint32_t r[16];
          if (warp_sees) { tmem_ld16(s_at + c, r); tmem_ld_wait(); }
#pragma unroll
          for (int g = 0; g < 16; g += 8) {
            uint32_t packed[4] = {0u, 0u, 0u, 0u};
            if (warp_sees && row_sees) {
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const int k0i = c + g + j;
                float p0 = fast_exp2(fmaf(__uint_as_float(r[g + j]), scale_log2, -m_new));
                float p1 = fast_exp2(fmaf(__uint_as_float(r[g + j + 1]), scale_log2, -m_new));
                if (!(k0i >= lo && k0i < hi)) p0 = 0.f;
                if (!(k0i + 1 >= lo && k0i + 1 < hi)) p1 = 0.f;
                l_tile += p0 + p1;                  // 32-bit sum of the unrounded values
                __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
              }
            }
            *reinterpret_cast<uint4*>(p_row + ((uint32_t)(((c + g) >> 3) << 4) ^ row_xor)) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      alpha_prev = alpha;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core's proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (threadIdx.x == 0) mark(args, 288 + i);
    }
    if (ok) {                                      // the last tile's O_tile
      if (lane == 0) ok = mbar_wait(o_full, (uint32_t)(num_tiles - 1) & 1u, args.error, 17);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok) {
        tc_fence_after();
        pick_up(num_tiles - 1, alpha_prev);
      }
    }
    // the row's sum of exponentials: both halves' parts (each relative to the same running maximum)
    l_run = agree(l_run, false);
    if (live && ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* o = args.out + (size_t)(row0 + row) * ((size_t)args.H * DH) + h * DH + half * OC;
#pragma unroll
      for (int d = 0; d < OC; d += 8) {
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
  if (threadIdx.x == 0) span(args, 1, now_ns());
  if (warp == SOFTMAX_WARPS + 1) {
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

constexpr size_t SMEM_BYTES = 7 * TILE_BYTES + 128 + 128 * sizeof(float);      // tiles, barriers, the halves' exchange: 115,328 bytes, two CTAs fit one SM (115,712 each at most)

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
// Where the cycle marks of the next launches go (device memory, 512 int64); only written by builds with -DAYK_TRACE.
AYK_EXPORT void ayk_attention_tc_set_trace(long long* p) { g_trace = p; }

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
                window, scale, g_trace};
  AYK_REQUIRE(total_rows / BQ + num_req <= 65535 && H >= 1, "ayk_attention_tc: too many row tiles (%d rows, %d requests)", total_rows, num_req);
  dim3 grid(H, total_rows / BQ + num_req);      // heads fastest: see the tile order in the kernel
  ayk_launch(attention_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mq, mk, mv, args);
  return ayk_check_launch("ayk_attention_tc");
}
