// bfloat16 matrix product for many rows (prompt portions) on tcgen05: persistent
// CTAs, two accumulators in tensor memory so that the epilogue of one tile runs
// under the main loop of the next.
//
//   C[M, N] = act(X[M, K] * W[N, K]^T + bias[N]) (+ residual[M, N])
//
// A tile is 128 rows of X (the MMA's M side, one row per TMEM lane) by BN out
// features (its N side, BN = 32 ... 256 in steps of 32, chosen by the host from
// a fitted model of the kernel's time, see whole_tiles_us).  Operands come by TMA in
// 64-element K blocks with the 128-byte swizzle through a ring of stages.
// Warp 0: TMA producer; warp 1: MMA issue and TMEM allocation; warps 2..9:
// epilogue, two warps per TMEM lane quarter, each taking half of the tile's
// columns.  An epilogue thread owns one row: it reads 32 accumulator columns
// with tcgen05.ld, adds the bias, applies the activation in 32-bit, adds the
// 32-bit residual (all loads of a chunk issued before its stores: the residual
// may alias C) and stores 128 contiguous bytes.  Where the output and the residual
// are 32-bit rows, both go through shared memory by TMA instead (PrefillArgs::staged).
//
// Where the tiles alone would leave most SMs idle (few out features, a long K)
// 2, 4 or 8 CTAs share a tile, each with an equal part of its K blocks: see
// PrefillArgs::splits.  (The reference leaves such choices to the library behind
// F.linear, layers/linear/methods.py:76.)
//
// Every wait is bounded; a wait that runs out records a code (21..26, 31..35 in
// the two-SM form) in the error word of the tensor-core kernels and the CTA
// winds down.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;
constexpr int BLOCK_K = 64;
constexpr int A_BYTES = BM * BLOCK_K * 2;
constexpr int THREADS = 320;
constexpr int EPI_WARPS = 8;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_TILES = 196608;             // bytes available to the stage ring
constexpr int TURNED_ROW_BYTES = 144;           // a row of the turned epilogue's 32 x 32 floats: 128 bytes + 16, which keeps 8 rows off each other's banks
constexpr int TURNED_BYTES = EPI_WARPS * 32 * TURNED_ROW_BYTES;
constexpr int STAGED_CHUNK = 16384;            // a buffer of the staged residual epilogue: 128 rows x 32 floats; it takes 2 halves x 1 or 2 of them

struct PrefillArgs {
  void* C;
  const float* bias;
  const float* residual;
  int* error;
  int M, N, K;
  int act, out_bf16;
  int BN, stages, m_tiles, n_tiles;
  int box_m;                 // rows of X that one TMA copy brings (128, fewer when M is small)
  int mode;                  // which compiled form of the epilogue (see epilogue_chunk)
  int vec_ok;                // N % 8 == 0 and bias, residual, C 16-byte aligned: whole chunks move in 16-byte pieces
  // mode 4: the columns from kv_col0 on are keys (kv_width of them) and then values of the rows' tokens; they
  // are also stored into the paged cache, at the place that (request, position) has in the block table
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  const int* kv_row_req;     // [M] the row's request within the step
  const int* kv_pos;         // [M] the row's position
  const int* kv_table;       // [requests, kv_table_stride] pages
  int kv_table_stride, kv_page_size, kv_col0, kv_width;
  // Split along K (one-SM form, when the tiles alone would leave most SMs idle): the `splits` CTAs of a
  // thread-block cluster share a tile, each running an equal part of its K blocks.  When every CTA of the
  // cluster is through with its main loop, each sends the others the columns of its sums that are theirs,
  // into their shared memory (the ring, idle by then); then each adds up, in the CTAs' order, the BN / splits
  // columns that are its share and finishes them (bias, activation, residual, store).  No global scratch.
  int splits;
  // Staged residual epilogue (one-SM form, float32 out over a float32 residual): the residual rows come by
  // TMA into shared memory, 128 rows x 32 columns at a time and a chunk ahead, the sums go back to the same
  // place and leave by a TMA store: whole 128-byte lines both ways, where a thread that owns a row would
  // otherwise read and write 16 bytes of 32 different lines per instruction.  staged = buffers per half of
  // the tile's columns (1 or 2; 0: the form is not taken): two where the ring keeps four stages beside them.
  int staged;
  // Turned epilogue (one-SM form, rows of C that are no whole 16-byte pieces, as the 50,257 columns of an LM
  // head give them): a warp leaves its 32 rows x 32 columns in shared memory and stores them row by row, a
  // lane per column, so that an instruction writes one run of up to 128 contiguous bytes whatever the rows'
  // alignment, where a thread that owns a row would store 32 separate elements.  No residual in this form.
  int turned;
};

// Where the keys of row `row` go: element offset of the row's place in a cache tensor, or -1 (a row
// beyond the matrix, or one that maps to the padding page).
__device__ __forceinline__ long long cache_place(const PrefillArgs& a, int row) {
  if (a.mode != 4 || row >= a.M) return -1;
  const int p = a.kv_pos[row];
  const int page = a.kv_table[(size_t)a.kv_row_req[row] * a.kv_table_stride + p / a.kv_page_size];
  return page > 0 ? ((long long)page * a.kv_page_size + p % a.kv_page_size) * a.kv_width : -1;
}

// One row, W consecutive columns (W = 16 or 32) starting at column n.  The epilogue competes
// with nothing for memory but it does for issue slots and registers, and with 25 K blocks per
// tile it is as long as the main loop.  So whole chunks inside the matrix take 16-byte loads of
// bias and residual and no test per element, and the three combinations that a transformer block
// uses are compiled on their own (MODE): 0 = bfloat16 out, no activation, no residual; 1 = float32
// out with residual; 2 = bfloat16 out with tanh-GELU; 3 = anything, decided at run time; 4 = as 0, and
// the key and value columns go into the paged cache as well (`place`: where this row's do, or -1).
template <int W, int MODE>
__device__ __forceinline__ void epilogue_chunk(const PrefillArgs& a, uint32_t taddr, int row, int n, bool row_ok,
                                               long long place) {
  constexpr int ACT = MODE == 2 ? AYK_ACT_GELU_TANH : (MODE == 3 ? -1 : AYK_ACT_NONE);
  uint32_t r[W];
  if (W == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
  const size_t idx = (size_t)row * a.N + n;
  const bool out_bf16 = MODE == 3 ? a.out_bf16 != 0 : MODE != 1;       // modes 0, 2 and 4 store bfloat16
  if (a.vec_ok) {            // N is a multiple of 8: every group of 8 columns lies inside the matrix or outside
    const bool with_res = (MODE == 1 || MODE == 3) && a.residual != nullptr && row_ok;
    float4 res[(MODE == 1 || MODE == 3) ? W / 4 : 1];
    if (MODE == 1 || MODE == 3) {
      if (with_res) {     // every load of the chunk before its first store: the residual may be C itself
#pragma unroll
        for (int j = 0; j < W / 4; ++j)
          if (n + 4 * j < a.N) res[j] = *reinterpret_cast<const float4*>(a.residual + idx + 4 * j);
      }
    }
    tmem_ld_wait();
    if (!row_ok) return;
#pragma unroll
    for (int j = 0; j < W; j += 8) {
      if (n + j >= a.N) break;
      float y[8];
#pragma unroll
      for (int u = 0; u < 8; u += 4) {
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.bias) bv = __ldg(reinterpret_cast<const float4*>(a.bias + n + j + u));
        y[u] = apply_activation_tc<ACT>(__uint_as_float(r[j + u]) + bv.x, a.act);
        y[u + 1] = apply_activation_tc<ACT>(__uint_as_float(r[j + u + 1]) + bv.y, a.act);
        y[u + 2] = apply_activation_tc<ACT>(__uint_as_float(r[j + u + 2]) + bv.z, a.act);
        y[u + 3] = apply_activation_tc<ACT>(__uint_as_float(r[j + u + 3]) + bv.w, a.act);
        if (MODE == 1 || MODE == 3) {
          if (with_res) {
            const float4 rv = res[(j + u) / 4];
            y[u] += rv.x; y[u + 1] += rv.y; y[u + 2] += rv.z; y[u + 3] += rv.w;
          }
        }
      }
      if (out_bf16) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 8; u += 2) {
          __nv_bfloat162 p = __floats2bfloat162_rn(y[u], y[u + 1]);
          w[u >> 1] = *reinterpret_cast<uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>((__nv_bfloat16*)a.C + idx + j) = make_uint4(w[0], w[1], w[2], w[3]);
        if (MODE == 4) {
          const int off = n + j - a.kv_col0;         // kv_col0 and kv_width are multiples of 8: a piece is all key or all value
          if (place >= 0 && off >= 0) {
            __nv_bfloat16* dst = off < a.kv_width ? a.kcache + place + off : a.vcache + place + (off - a.kv_width);
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else {
        float* dst = (float*)a.C + idx + j;
        *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(y[4], y[5], y[6], y[7]);
      }
    }
    return;
  }
  // the ragged edge of the matrix, or rows whose 16-byte pieces are not aligned: element by element
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < W; ++j) {
    if (row_ok && n + j < a.N) {
      const float b = a.bias ? __ldg(a.bias + n + j) : 0.f;
      const float res = a.residual ? a.residual[idx + j] : 0.f;
      const float y = apply_activation_tc<ACT>(__uint_as_float(r[j]) + b, a.act) + res;
      if (a.out_bf16) ((__nv_bfloat16*)a.C)[idx + j] = __float2bfloat16_rn(y);
      else ((float*)a.C)[idx + j] = y;
      if (MODE == 4) {
        const int off = n + j - a.kv_col0;
        if (place >= 0 && off >= 0)
          (off < a.kv_width ? a.kcache + place + off : a.vcache + place + (off - a.kv_width))[0] = __float2bfloat16_rn(y);
      }
    }
  }
}

// `cols` columns of one row, from column n on (cols a multiple of 16)
template <int MODE>
__device__ __forceinline__ void epilogue_row(const PrefillArgs& a, uint32_t taddr, int row, int n, int cols, bool row_ok,
                                             long long place) {
  int c = 0;
  for (; c + 32 <= cols; c += 32) epilogue_chunk<32, MODE>(a, taddr + c, row, n + c, row_ok, place);
  if (c < cols) epilogue_chunk<16, MODE>(a, taddr + c, row, n + c, row_ok, place);
}
__device__ __forceinline__ void epilogue_row_any(const PrefillArgs& a, uint32_t taddr, int row, int n, int cols, bool row_ok,
                                                 long long place) {
  if (a.mode == 0) epilogue_row<0>(a, taddr, row, n, cols, row_ok, place);
  else if (a.mode == 1) epilogue_row<1>(a, taddr, row, n, cols, row_ok, place);
  else if (a.mode == 2) epilogue_row<2>(a, taddr, row, n, cols, row_ok, place);
  else if (a.mode == 4) epilogue_row<4>(a, taddr, row, n, cols, row_ok, place);
  else epilogue_row<3>(a, taddr, row, n, cols, row_ok, place);
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Split along K: where the sums of the cluster's CTAs meet.  In every CTA the ring holds `splits` slots, one per
// sending CTA, of `share` columns (share = BN / splits) by 128 rows of floats, a column's rows side by side: the
// 32 threads of a warp own 32 consecutive rows, so their stores of one column are 128 contiguous bytes on their
// way to the owner's shared memory, and the owner's loads of one column fall into 32 different banks.  (With a
// row's columns side by side, 16 bytes per thread and row, the same exchange took 1 to 5 us longer: scattered
// pieces are what the network between the SMs of a cluster is slow at.)
constexpr uint32_t SPLIT_COL_BYTES = BM * 4u;

// This thread's `cols` accumulator columns (a multiple of 16, from tile column c0 on) of row `row_in_tile`, each
// into the shared memory of the CTA that owns it (share is a multiple of 16: sixteen columns have one owner).
__device__ __forceinline__ void send_partial_row(uint32_t taddr, uint32_t recv, int my_rank, int share, int row_in_tile, int c0,
                                                 int cols) {
  const uint32_t mine = recv + (uint32_t)my_rank * (uint32_t)share * SPLIT_COL_BYTES + (uint32_t)row_in_tile * 4u;   // offset within any CTA
  for (int c = 0; c < cols; c += 16) {
    uint32_t r[16];
    tmem_ld16(taddr + c, r);
    tmem_ld_wait();
    const int col = c0 + c, owner = col / share;
    const uint32_t at = map_to_cta(mine + (uint32_t)(col - owner * share) * SPLIT_COL_BYTES, (uint32_t)owner);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(at + (uint32_t)j * SPLIT_COL_BYTES), "f"(__uint_as_float(r[j])) : "memory");
  }
}

// This CTA's share of the tile: `cols` columns (a multiple of 8) from column `c0` of the share on, for the row
// `row_in_tile`, summed over the slots (in the CTAs' order, so every run adds alike) and finished eight columns
// at a time.  n0: the first column of the share in the matrix.
__device__ __forceinline__ void finish_split_cols(const PrefillArgs& a, uint32_t recv, int splits, int share, int m0, int n0,
                                                  int row_in_tile, int c0, int cols) {
  const int row = m0 + row_in_tile;
  if (row >= a.M) return;
  const uint32_t slot_bytes = (uint32_t)share * SPLIT_COL_BYTES;
  const long long place = cache_place(a, row);
  for (int c = c0; c < c0 + cols; c += 8) {
    const int col = n0 + c;
    if (col >= a.N) break;                         // N is a multiple of 8: a group lies inside the matrix or outside
    const uint32_t at = recv + (uint32_t)c * SPLIT_COL_BYTES + (uint32_t)row_in_tile * 4u;
    float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < splits; ++p) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(at + p * slot_bytes + (uint32_t)j * SPLIT_COL_BYTES));
        y[j] += v;
      }
    }
    if (a.bias) {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(a.bias + col)), b1 = __ldg(reinterpret_cast<const float4*>(a.bias + col + 4));
      y[0] += b0.x; y[1] += b0.y; y[2] += b0.z; y[3] += b0.w; y[4] += b1.x; y[5] += b1.y; y[6] += b1.z; y[7] += b1.w;
    }
    if (a.act == AYK_ACT_GELU_TANH) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = apply_activation_tc<AYK_ACT_GELU_TANH>(y[j], a.act);
    } else if (a.act != AYK_ACT_NONE) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = apply_activation(y[j], a.act);
    }
    const size_t idx = (size_t)row * a.N + col;
    if (a.residual) {
      const float4 r0 = *reinterpret_cast<const float4*>(a.residual + idx), r1 = *reinterpret_cast<const float4*>(a.residual + idx + 4);
      y[0] += r0.x; y[1] += r0.y; y[2] += r0.z; y[3] += r0.w; y[4] += r1.x; y[5] += r1.y; y[6] += r1.z; y[7] += r1.w;
    }
    if (a.out_bf16) {
      uint32_t w[4];
#pragma unroll
      for (int u = 0; u < 8; u += 2) {
        __nv_bfloat162 pr = __floats2bfloat162_rn(y[u], y[u + 1]);
        w[u >> 1] = *reinterpret_cast<uint32_t*>(&pr);
      }
      *reinterpret_cast<uint4*>((__nv_bfloat16*)a.C + idx) = make_uint4(w[0], w[1], w[2], w[3]);
      if (a.mode == 4) {
        const int off = col - a.kv_col0;             // kv_col0 and kv_width are multiples of 8: a group is all key or all value
        if (place >= 0 && off >= 0) {
          __nv_bfloat16* dst = off < a.kv_width ? a.kcache + place + off : a.vcache + place + (off - a.kv_width);
          *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else {
      float* dst = (float*)a.C + idx;
      *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(y[4], y[5], y[6], y[7]);
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_c,
                       const PrefillArgs args) {
  const int BN = args.BN, STAGES = args.stages;
  const uint32_t B_BYTES = (uint32_t)BN * BLOCK_K * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  // With fewer than 128 rows in all, only those rows are copied; the rest of the A tile keeps
  // whatever it held: its products land in accumulator rows that the epilogue never stores.
  const uint32_t TX_BYTES = (uint32_t)args.box_m * BLOCK_K * 2 + B_BYTES;
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + SMEM_TILES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto tmem_full = [&](int b) { return bars + 8u * (2 * MAX_STAGES + b); };
  auto tmem_empty = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * MAX_STAGES + 4);
  auto res_full = [&](int half, int buf) { return bars + 8u * (2 * MAX_STAGES + 5 + 2 * half + buf); };
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = args.m_tiles * args.n_tiles;
  const int num_kb = (args.K + BLOCK_K - 1) / BLOCK_K;
  // Whole tiles go round the CTAs; with a split along K a CTA has one tile and one part of its K blocks.
  const int splits = args.splits;
  const int first_tile = splits > 1 ? (int)blockIdx.x / splits : (int)blockIdx.x;
  const int tile_step = splits > 1 ? total_tiles : (int)gridDim.x;          // one tile per CTA when K is split
  const int part_kb = splits > 1 ? (num_kb + splits - 1) / splits : num_kb;
  const int kb_first = splits > 1 ? ((int)blockIdx.x % splits) * part_kb : 0;      // the cluster runs along x: rank = blockIdx.x % splits
  const int kb_last = min(num_kb, kb_first + part_kb);                       // this CTA's K blocks of each of its tiles
  const int my_kb = kb_last - kb_first;
  const int my_tiles = (first_tile < total_tiles) ? (total_tiles - 1 - first_tile) / tile_step + 1 : 0;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tmem_full(b), 1); mbar_init(tmem_empty(b), EPI_WARPS); }
    for (int h = 0; h < 2; ++h) { mbar_init(res_full(h, 0), 1); mbar_init(res_full(h, 1), 1); }
    if (args.staged) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_r) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      // A cursor walks this CTA's tiles and their K blocks; no division or modulo per K block
      // (one thread issues every copy, and its arithmetic set the pace of the whole pipeline).
      const int total_it = my_tiles * my_kb;
      struct Cursor { int tile, kx, m0, n0, kb; };
      auto start = [&]() {
        Cursor c; c.tile = first_tile; c.kb = kb_first; c.kx = kb_first * BLOCK_K;
        c.m0 = (c.tile / args.n_tiles) * BM; c.n0 = (c.tile % args.n_tiles) * BN;
        return c;
      };
      auto advance = [&](Cursor& c) {
        c.kx += BLOCK_K;
        if (++c.kb == kb_last) {
          c.kb = kb_first; c.kx = kb_first * BLOCK_K; c.tile += tile_step;
          c.m0 = (c.tile / args.n_tiles) * BM; c.n0 = (c.tile % args.n_tiles) * BN;
        }
      };
      // The weight does not depend on the kernels before this one: its first
      // stages start streaming at once; the rows X wait for the predecessor.
      const int pre = min(STAGES, total_it);
      Cursor cw = start();
      for (int s = 0; s < pre; ++s) {
        mbar_expect_tx(full_bar(s), TX_BYTES);
        tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &map_w, cw.kx, cw.n0, full_bar(s));
        advance(cw);
      }
      pdl_wait();
      Cursor cx = start();
      for (int s = 0; s < pre; ++s) {
        tma_load_2d(tiles + s * STAGE_BYTES, &map_x, cx.kx, cx.m0, full_bar(s));
        advance(cx);
      }
      bool ok = true;
      int issued = pre;
      int s = pre == STAGES ? 0 : pre;              // the stage of iteration `pre`
      uint32_t wait_parity = 0;                     // the first refill of a stage waits for its first release
      for (int it = pre; it < total_it; ++it) {
        ok = mbar_wait(empty_bar(s), wait_parity, args.error, 21);
        if (!ok) break;
        mbar_expect_tx(full_bar(s), TX_BYTES);
        const uint32_t dst = tiles + s * STAGE_BYTES;
        tma_load_2d(dst + A_BYTES, &map_w, cx.kx, cx.n0, full_bar(s));
        tma_load_2d(dst, &map_x, cx.kx, cx.m0, full_bar(s));
        advance(cx);
        issued = it + 1;
        if (++s == STAGES) { s = 0; wait_parity ^= 1u; }
      }
      if (!ok) {
        for (int j = max(0, issued - STAGES); j < issued; ++j)
          mbar_wait(full_bar(j % STAGES), (uint32_t)(j / STAGES) & 1u, args.error, 22);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      int s = 0;
      uint32_t full_parity = 0;
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int b = t & 1;
        if (t >= 2) {
          ok = mbar_wait(tmem_empty(b), (uint32_t)((t >> 1) & 1) ^ 1u, args.error, 23);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc = tmem_base + (uint32_t)b * 256u;
        for (int kb = 0; kb < my_kb && ok; ++kb) {
          ok = mbar_wait(full_bar(s), full_parity, args.error, 24);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_src = tiles + s * STAGE_BYTES;
          const uint64_t da0 = make_desc(a_src), db0 = make_desc(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 16; ++k)     // 32 bytes further along K: two 16-byte units of the address field
            umma(acc, da0 + (uint64_t)(2 * k), db0 + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));
          if (++s == STAGES) { s = 0; full_parity ^= 1u; }
        }
        umma_commit(tmem_full(b));
      }
    }
    __syncwarp();
  } else if (splits > 1) {
    pdl_wait();            // the residual and C belong to earlier kernels until here; the work follows below, with the whole CTA
  } else if (args.turned) {
    // ---- rows of C that are no whole 16-byte pieces: through shared memory, stored a row at a time (see PrefillArgs)
    pdl_wait();
    const int e = warp - 2;
    const int quarter = warp & 3, half = e >> 2;
    const int half_cols = BN >> 1;
    const uint32_t mine = tiles + (uint32_t)(SMEM_TILES - TURNED_BYTES) + (uint32_t)e * 32u * TURNED_ROW_BYTES;
    const int act = args.act;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int b = t & 1;
      const int tile = blockIdx.x + t * gridDim.x;
      const int m0 = (tile / args.n_tiles) * BM + quarter * 32, nh = (tile % args.n_tiles) * BN + half * half_cols;
      if (lane == 0) ok = mbar_wait(tmem_full(b), (uint32_t)(t >> 1) & 1u, args.error, 25);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t)b * 256u + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
      for (int c = 0; c < half_cols; c += 32) {
        const int w = min(32, half_cols - c);          // 32, or 16 at the end of a half of 48, 80 or 112 columns
        uint32_t r[32];
        if (w == 32) tmem_ld32(taddr + c, r); else tmem_ld16(taddr + c, r);
        tmem_ld_wait();
        // this thread's row of the chunk into shared memory ...
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (j < w)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine + (uint32_t)lane * TURNED_ROW_BYTES + (uint32_t)j * 4u),
                         "f"(__uint_as_float(r[j])), "f"(__uint_as_float(r[j + 1])), "f"(__uint_as_float(r[j + 2])),
                         "f"(__uint_as_float(r[j + 3])) : "memory");
        }
        __syncwarp();
        // ... and the warp's 32 rows out, a row an instruction, this lane's column of each
        const int col = nh + c + lane;
        const bool col_ok = lane < w && col < args.N;
        const float bias = (col_ok && args.bias) ? __ldg(args.bias + col) : 0.f;
        for (int i = 0; i < 32; ++i) {
          const int row = m0 + i;
          if (row >= args.M) break;
          float v;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(mine + (uint32_t)i * TURNED_ROW_BYTES + (uint32_t)lane * 4u));
          if (col_ok) {
            v += bias;
            if (act == AYK_ACT_GELU_TANH) v = apply_activation_tc<AYK_ACT_GELU_TANH>(v, act);
            else if (act != AYK_ACT_NONE) v = apply_activation(v, act);
            const size_t idx = (size_t)row * args.N + col;
            if (args.out_bf16) ((__nv_bfloat16*)args.C)[idx] = __float2bfloat16_rn(v);
            else ((float*)args.C)[idx] = v;
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty(b));
    }
  } else if (args.staged) {
    // ---- float32 out over a float32 residual, both through shared memory by TMA (see PrefillArgs)
    pdl_wait();
    const int e = warp - 2;
    const int quarter = warp & 3, half = e >> 2;
    const int half_cols = BN >> 1, chunks = half_cols >> 5;                  // 32 columns a chunk
    const bool chief = (e & 3) == 0 && lane == 0;                            // issues the copies of this half of the columns
    const int nbuf = args.staged;
    const uint32_t stage0 = tiles + (uint32_t)(SMEM_TILES - 2 * nbuf * STAGED_CHUNK) + (uint32_t)(half * nbuf) * STAGED_CHUNK;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t fills[2] = {0u, 0u};                // how often each buffer has been filled: the phase of its barrier
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int b = t & 1;
      const int tile = blockIdx.x + t * gridDim.x;
      const int m0 = (tile / args.n_tiles) * BM, nh = (tile % args.n_tiles) * BN + half * half_cols;
      // The tile's first chunks of the residual are asked for now and land under the main loop.  The
      // stores of the tile before must have read their buffers first.
      if (chief) {
        bulk_wait_read();
        for (int c = 0; c < nbuf && c < chunks; ++c) {
          mbar_expect_tx(res_full(half, c), STAGED_CHUNK);
          tma_load_2d(stage0 + c * STAGED_CHUNK, &map_r, nh + 32 * c, m0, res_full(half, c));
        }
      }
      if (lane == 0) ok = mbar_wait(tmem_full(b), (uint32_t)(t >> 1) & 1u, args.error, 25);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t)b * 256u + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
      for (int c = 0; c < chunks && ok; ++c) {
        const int buf = nbuf == 2 ? (c & 1) : 0;
        uint32_t r[32];
        tmem_ld32(taddr + 32 * c, r);
        if (lane == 0) ok = mbar_wait(res_full(half, buf), fills[buf] & 1u, args.error, 27);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        ++fills[buf];
        tmem_ld_wait();
        if (!ok) break;
        if (c == chunks - 1) {                   // the accumulator is in registers: the MMA warp may have it back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty(b));
        }
        const uint32_t mine = stage0 + buf * STAGED_CHUNK + (uint32_t)row_in_tile * 128u;
        const int col0 = nh + 32 * c;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t at = mine + (uint32_t)((j ^ (row_in_tile & 7)) << 4);     // the 128-byte swizzle of the copy
          float4 v;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(at));
          float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
          if (args.bias && col0 + 4 * j < args.N) bv = __ldg(reinterpret_cast<const float4*>(args.bias + col0 + 4 * j));
          v.x += __uint_as_float(r[4 * j]) + bv.x;
          v.y += __uint_as_float(r[4 * j + 1]) + bv.y;
          v.z += __uint_as_float(r[4 * j + 2]) + bv.z;
          v.w += __uint_as_float(r[4 * j + 3]) + bv.w;
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");           // the sums are there before the copy engine reads them
        if (half == 0) asm volatile("bar.sync 2, 128;" ::: "memory"); else asm volatile("bar.sync 3, 128;" ::: "memory");
        if (chief) {
          tma_store_2d(&map_c, col0, m0, stage0 + buf * STAGED_CHUNK);
          bulk_commit();
          if (c + nbuf < chunks) {               // this buffer's next chunk, once the store has read it
            bulk_wait_read();
            mbar_expect_tx(res_full(half, buf), STAGED_CHUNK);
            tma_load_2d(stage0 + buf * STAGED_CHUNK, &map_r, col0 + 32 * nbuf, m0, res_full(half, buf));
          }
        }
      }
    }
    if (chief) bulk_wait_all();                  // the last stores are out before the shared memory is given back
  } else {
    pdl_wait();            // residual and C belong to earlier kernels until here
    const int e = warp - 2;
    const int quarter = warp & 3, half = e >> 2;
    const int half_cols = BN >> 1;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int b = t & 1;
      const int tile = blockIdx.x + t * gridDim.x;
      const int m0 = (tile / args.n_tiles) * BM, n0 = (tile % args.n_tiles) * BN;
      const long long place = cache_place(args, m0 + quarter * 32 + lane);   // three dependent loads: under the main loop
      // One lane per warp watches the barrier; 256 threads polling it slow the producer and MMA warps down.
      if (lane == 0) ok = mbar_wait(tmem_full(b), (uint32_t)(t >> 1) & 1u, args.error, 25);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t taddr = tmem_base + (uint32_t)b * 256u + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
      epilogue_row_any(args, taddr, row, n0 + half * half_cols, half_cols, row_ok, place);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty(b));
    }
  }

  if (splits > 1) {
    // ---- K split over the CTAs of a cluster: one tile, one part of its K blocks each (see PrefillArgs).  Every
    // thread of the cluster meets at the two barriers, whatever happened to its waits.
    const int e = warp - 2;
    const int quarter = warp & 3, half = e >> 2;
    const int half_cols = BN >> 1, share = BN / splits;
    const int part = (int)cluster_rank();
    const int row_in_tile = quarter * 32 + lane;
    bool ok = my_tiles == 1;
    if (warp >= 2 && ok) {
      if (lane == 0) ok = mbar_wait(tmem_full(0), 0u, args.error, 25);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      tc_fence_after();
    }
    cluster_sync_all();                          // every CTA's MMAs have read its ring for the last time
    if (warp >= 2 && ok) {
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
      send_partial_row(taddr, tiles, part, share, row_in_tile, half * half_cols, half_cols);
      tc_fence_before();
    }
    cluster_sync_all();                          // the sums of all CTAs have arrived (release / acquire at cluster scope)
    if (warp >= 2 && ok) {
      const int tile = first_tile;
      const int m0 = (tile / args.n_tiles) * BM, n0 = (tile % args.n_tiles) * BN + part * share;
      const int mine = share >> 1;               // half of the share for each of the two warps that own a row
      finish_split_cols(args, tiles, splits, share, m0, n0, row_in_tile, half * mine, mine);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------- two SMs on one tile --
//
// From 129 rows on, two CTAs of a cluster share a tile of 256 rows by BN out features
// (tcgen05.mma.cta_group::2): each holds its own 128 rows of X and HALF of the tile's rows of
// W, so per 64-wide K block an SM takes in 16 KB + BN * 64 bytes instead of 16 KB + BN * 128.
// The product is bound by that traffic, not by the tensor pipe.  CTA 0 of the pair issues every
// MMA; both CTAs' copies signal CTA 0's "full" barrier (one arrival, the bytes of both);
// tcgen05.commit with a cluster multicast frees the stage in both CTAs and announces a finished
// accumulator to both epilogues; both epilogues release an accumulator at CTA 0's barrier.
// Each CTA's tensor memory holds its own 128 rows of the two accumulators.

// destination in this CTA, completion counted at `cluster_bar` (this CTA's or its partner's barrier)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives at the barrier of this offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}

constexpr int PAIR_ROWS = 2 * BM;

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const PrefillArgs args) {
  const int BN = args.BN, STAGES = args.stages;
  const int HALF_N = BN >> 1;                                   // rows of W per CTA
  const uint32_t B_BYTES = (uint32_t)HALF_N * BLOCK_K * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  const uint32_t TX_BYTES = 2u * STAGE_BYTES;                   // both CTAs' copies of a stage
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(PAIR_ROWS >> 4) << 24);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + SMEM_TILES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto tmem_full = [&](int b) { return bars + 8u * (2 * MAX_STAGES + b); };
  auto tmem_empty = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * MAX_STAGES + 4);
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                          // 0 issues the MMAs
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int total_tiles = args.m_tiles * args.n_tiles;           // m_tiles counts 256-row tiles here
  const int num_kb = (args.K + BLOCK_K - 1) / BLOCK_K;
  const int my_tiles = (pair < total_tiles) ? (total_tiles - 1 - pair) / pairs + 1 : 0;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tmem_full(b), 1); mbar_init(tmem_empty(b), 2 * EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {      // the same warp in both CTAs: the pair allocates together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      const int total_it = my_tiles * num_kb;
      struct Cursor { int tile, kx, m0, n0, kb; };
      auto place = [&](Cursor& c) {
        c.m0 = (c.tile / args.n_tiles) * PAIR_ROWS + (int)rank * BM;
        c.n0 = (c.tile % args.n_tiles) * BN + (int)rank * HALF_N;
      };
      auto start = [&]() { Cursor c; c.tile = pair; c.kb = 0; c.kx = 0; place(c); return c; };
      auto advance = [&](Cursor& c) {
        c.kx += BLOCK_K;
        if (++c.kb == num_kb) { c.kb = 0; c.kx = 0; c.tile += pairs; place(c); }
      };
      uint32_t full_at_leader[MAX_STAGES];
#pragma unroll
      for (int s = 0; s < MAX_STAGES; ++s) full_at_leader[s] = map_to_cta(full_bar(s), 0);
      const int pre = min(STAGES, total_it);
      Cursor cw = start();
      for (int s = 0; s < pre; ++s) {           // weights first: they do not depend on the kernel before
        if (rank == 0) mbar_expect_tx(full_bar(s), TX_BYTES);
        tma_load_2d_pair(tiles + s * STAGE_BYTES + A_BYTES, &map_w, cw.kx, cw.n0, full_at_leader[s]);
        advance(cw);
      }
      pdl_wait();
      Cursor cx = start();
      for (int s = 0; s < pre; ++s) {
        tma_load_2d_pair(tiles + s * STAGE_BYTES, &map_x, cx.kx, cx.m0, full_at_leader[s]);
        advance(cx);
      }
      bool ok = true;
      int s = pre == STAGES ? 0 : pre;
      uint32_t wait_parity = 0;
      for (int it = pre; it < total_it; ++it) {
        ok = mbar_wait(empty_bar(s), wait_parity, args.error, 31);
        if (!ok) break;
        if (rank == 0) mbar_expect_tx(full_bar(s), TX_BYTES);
        const uint32_t dst = tiles + s * STAGE_BYTES;
        tma_load_2d_pair(dst + A_BYTES, &map_w, cx.kx, cx.n0, full_at_leader[s]);
        tma_load_2d_pair(dst, &map_x, cx.kx, cx.m0, full_at_leader[s]);
        advance(cx);
        if (++s == STAGES) { s = 0; wait_parity ^= 1u; }
      }
      // Copies still in flight are waited for by the MMA thread of CTA 0 (it consumes every stage);
      // if that thread gave up, the epilogues time out, and the cluster barrier at the end holds
      // both CTAs until every thread has arrived.
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      bool ok = true;
      int s = 0;
      uint32_t full_parity = 0;
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int b = t & 1;
        if (t >= 2) {
          ok = mbar_wait(tmem_empty(b), (uint32_t)((t >> 1) & 1) ^ 1u, args.error, 33);
          if (!ok) break;
          tc_fence_after();
        }
        const uint32_t acc = tmem_base + (uint32_t)b * 256u;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait(full_bar(s), full_parity, args.error, 34);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_src = tiles + s * STAGE_BYTES;
          const uint64_t da0 = make_desc(a_src), db0 = make_desc(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 16; ++k)
            umma_pair(acc, da0 + (uint64_t)(2 * k), db0 + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(s));
          if (++s == STAGES) { s = 0; full_parity ^= 1u; }
        }
        umma_commit_pair(tmem_full(b));
      }
    }
    __syncwarp();
  } else {
    pdl_wait();
    const int e = warp - 2;
    const int quarter = warp & 3, half = e >> 2;
    const int half_cols = BN >> 1;
    uint32_t empty_at_leader[2] = {map_to_cta(tmem_empty(0), 0), map_to_cta(tmem_empty(1), 0)};
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int b = t & 1;
      const int tile = pair + t * pairs;
      const int m0 = (tile / args.n_tiles) * PAIR_ROWS + (int)rank * BM, n0 = (tile % args.n_tiles) * BN;
      const long long place = cache_place(args, m0 + quarter * 32 + lane);
      if (lane == 0) ok = mbar_wait(tmem_full(b), (uint32_t)(t >> 1) & 1u, args.error, 35);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      const uint32_t taddr = tmem_base + (uint32_t)b * 256u + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
      epilogue_row_any(args, taddr, row, n0 + half * half_cols, half_cols, row_ok, place);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty_at_leader[b]);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA frees tensor memory, or leaves, while its partner may still use it
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------------------------- host --

void prefill_kernel_symbol(const void** fn) { *fn = (const void*)gemm_tc_prefill_kernel; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int* g_error_host = nullptr;
int* g_error_dev = nullptr;
bool g_configured = false;
std::mutex g_mutex;
constexpr size_t SMEM_BYTES = 1024 + SMEM_TILES + 8 * (2 * MAX_STAGES + 9);

struct MapKey {
  const void* ptr; int rows, k, box;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box == o.box; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1000003u ^ (size_t)k.k * 10007u ^ (size_t)k.box; }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_weight_maps;

int setup() {
  if (g_configured) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (err != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
    return ayk_fail("ayk_gemm_tc_prefill: cuTensorMapEncodeTiled is not available from this driver");
  g_encode = (EncodeTiledFn)fn;
  err = cudaHostAlloc((void**)&g_error_host, sizeof(int), cudaHostAllocMapped);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc_prefill: cudaHostAlloc: %s", cudaGetErrorString(err));
  *g_error_host = 0;
  err = cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc_prefill: cudaHostGetDevicePointer: %s", cudaGetErrorString(err));
  err = cudaFuncSetAttribute(gemm_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc_prefill: shared memory %zu: %s", SMEM_BYTES, cudaGetErrorString(err));
  err = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc_prefill: shared memory %zu: %s", SMEM_BYTES, cudaGetErrorString(err));
  g_configured = true;
  return 0;
}

int encode(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ayk_fail("ayk_gemm_tc_prefill: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

// Split along K in the one-SM form: -1 the library decides per product, 0 or 1 never, 2 / 4 / 8 that many
// CTAs per tile wherever the tiles allow it.
int g_split = -1;
int g_last_splits = 1;          // parts per tile of the last one-SM launch (1: whole tiles), for tests and tuning

// How many clusters of `size` CTAs of the one-SM kernel the device runs at once.  A cluster lives inside one
// GPC, so fewer CTAs run at once the larger the cluster (on a B200 of 148 SMs the driver says 74 pairs, 33
// clusters of 4, 15 of 8).  Asked of the driver once per device where there is one; estimated from GPCs of 18 SMs otherwise
// (the plan can be asked for without a GPU).
void prefill_kernel_symbol(const void** fn);
int cluster_capacity(int sms, int size) {
  static int cached[64][9] = {};
  int device = -1;
  if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64 && size <= 8) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (cached[device][size] == 0 && g_configured) {         // once the kernel's shared memory has been granted
      const void* fn = nullptr;
      prefill_kernel_symbol(&fn);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(size * 64);
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = SMEM_BYTES;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) == cudaSuccess && n > 0) cached[device][size] = n;
      else { cudaGetLastError(); cached[device][size] = -1; }
    }
    if (cached[device][size] > 0) return cached[device][size];
  } else {
    cudaGetLastError();
  }
  const int gpcs = sms / 18 > 0 ? sms / 18 : 1;
  return gpcs * (18 / size);
}

// May a tile's K blocks be split over a cluster of `splits` CTAs?  Every tile's cluster runs at once, every
// part holds a K block, every CTA's share of the columns is whole 16-column pieces.
bool split_fits(int tiles, int num_kb, int splits, int sms, int bn) {
  if (splits < 2 || splits > 8 || bn % (16 * splits) != 0 || tiles > cluster_capacity(sms, splits)) return false;
  if (BM * bn * 4 > SMEM_TILES) return false;                       // the sums meet in the ring
  const int part = (num_kb + splits - 1) / splits;
  return part >= 2 && (splits - 1) * part < num_kb;
}

double kblock_us(int a_rows, int bn, int active);              // the model of the product's time, below
double whole_tiles_us(int M, int N, int K, int bn, int sms, bool wide_rows);

// Does splitting K beat whole tiles going round the CTAs, and with which tile width and how many parts?
// Times from the model above; the two cluster barriers, the exchange of the sums through shared memory and
// their addition cost the split form about 16 ns per column of the tile + 0.35 us per CTA of the cluster on
// top of its K blocks (fitted to 261 measured split products of GPT-2 small and XL layer shapes at 128 to 1,024
// rows, residual 0.7 us rms; with a split taken where it is modelled 10 % ahead, the choice is within 1.4 % of the
// best measured form in 46 of 48 cases and 4.3 % behind at worst).
constexpr double SPLIT_FIX_US = 0.0, SPLIT_FIX_PER_COL = 0.016, SPLIT_FIX_PER_CTA = 0.35, SPLIT_MARGIN = 0.90;
bool split_pays(int M, int N, int K, int sms, int tile_n, bool wide_rows, int* bn_out, int* splits_out) {
  const int m_tiles = (M + BM - 1) / BM, num_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (N % 8 != 0) return false;
  double best_whole = -1.0;
  for (int bn = 32; bn <= 256; bn += 32) {
    if (tile_n > 0 && bn != tile_n) continue;
    const double us = whole_tiles_us(M, N, K, bn, sms, wide_rows);
    if (best_whole < 0 || us < best_whole) best_whole = us;
  }
  double best_split = -1.0;
  for (int bn = 32; bn <= 256; bn += 32) {
    if (tile_n > 0 && bn != tile_n) continue;
    const long tiles = (long)m_tiles * ((N + bn - 1) / bn);
    for (int sp = 2; sp <= 8; sp *= 2) {
      if (!split_fits((int)tiles, num_kb, sp, sms, bn)) continue;
      const double us = 3.4 + (double)((num_kb + sp - 1) / sp) * kblock_us(M >= BM ? BM : (M + 7) / 8 * 8, bn, (int)tiles * sp) +
                        SPLIT_FIX_US + SPLIT_FIX_PER_COL * bn + SPLIT_FIX_PER_CTA * sp;
      if (best_split < 0 || us < best_split) { best_split = us; *bn_out = bn; *splits_out = sp; }
    }
  }
  return best_split > 0 && best_split < SPLIT_MARGIN * best_whole;
}

// rows x n float32, row-major; box of 128 rows x 32 columns (128 bytes), 128-byte swizzle: a chunk of the
// staged residual epilogue.
int encode_f32(CUtensorMap* map, const void* ptr, int rows, int n) {
  cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)n * 4};
  cuuint32_t box[2] = {32u, (cuuint32_t)BM};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ayk_fail("ayk_gemm_tc_prefill: cuTensorMapEncodeTiled (float32 rows) failed with %d", (int)r);
  return 0;
}
int g_staged = 1;             // the staged residual epilogue where it applies (0: the row-per-thread epilogue everywhere)
int g_last_staged = 0;        // buffers per half that the last one-SM launch staged its residual through (0: it did not)

int epilogue_mode(int act, bool with_residual, bool out_bf16) {
  if (act == AYK_ACT_NONE && !with_residual && out_bf16) return 0;
  if (act == AYK_ACT_NONE && !out_bf16) return 1;
  if (act == AYK_ACT_GELU_TANH && !with_residual && out_bf16) return 2;
  return 3;
}

}  // namespace

AYK_EXPORT int ayk_gemm_tc_prefill_error() { return g_error_host ? *g_error_host : 0; }
// Split along K in the one-SM product for many rows: -1 the library decides (default), 0 never, 2 / 4 / 8
// that many CTAs per tile wherever the tiles allow it.
AYK_EXPORT void ayk_gemm_tc_prefill_split(int mode) { g_split = mode; }
// The staged residual epilogue (float32 out over a float32 residual through shared memory by TMA): 1 where it
// applies (default), 0 never.
AYK_EXPORT void ayk_gemm_tc_prefill_staged(int on) { g_staged = on ? 1 : 0; }
AYK_EXPORT int ayk_gemm_tc_prefill_last_staged() { return g_last_staged; }
// How many clusters of `size` CTAs of the one-SM kernel run at once (asked of the driver once a product has run on
// the device, else estimated).
AYK_EXPORT int ayk_gemm_tc_prefill_cluster_capacity(int sms, int size) { return cluster_capacity(sms, size); }
// Into how many parts the last one-SM product split the K blocks of its tiles (1: it did not).
AYK_EXPORT int ayk_gemm_tc_prefill_last_split() { return g_last_splits; }

// A model of the one-SM product's time in microseconds, fitted to measurements on a B200 (graphs of 24
// products, GPT-2 XL and GPT-2 small shapes, 96 to 2,048 rows, tile widths 64 to 256; mean error 8 %):
// a fixed 3.4 us; per K block of a tile the larger of a latency floor (0.256 us + 0.285 ns per column) and
// the tile's operand bytes times the CTAs that run at once over 18 TB/s (what the SMs together draw
// from L2); the last tile's epilogue, which no main loop hides: 15.8 ns per column, and 26 ns more where it
// reads and writes 32-bit rows (a residual sum).  On the 80 measured cases the width it picks is within
// 0.1 % of the best measured one.
namespace {
double kblock_us(int a_rows, int bn, int active) {
  const double floor_us = 0.256 + 0.000285 * bn;
  const double stream_us = (double)(a_rows + bn) * 128.0 * active / 18.0e6;
  return floor_us > stream_us ? floor_us : stream_us;
}
double whole_tiles_us(int M, int N, int K, int bn, int sms, bool wide_rows) {
  const int m_tiles = (M + BM - 1) / BM, num_kb = (K + BLOCK_K - 1) / BLOCK_K;
  const int a_rows = M >= BM ? BM : (M + 7) / 8 * 8;
  const long tiles = (long)m_tiles * ((N + bn - 1) / bn);
  const long full = tiles / sms, rest = tiles % sms;
  // 32-bit rows cost the epilogue 26 ns more per column unless they go through the staged form (widths 64, 128, 192)
  const bool staged = wide_rows && bn % 64 == 0 && bn <= 192 && M >= BM;
  double t = 3.4 + (double)full * num_kb * kblock_us(a_rows, bn, sms) + (wide_rows && !staged ? 0.0418 : 0.0158) * bn;
  if (rest) t += (double)num_kb * kblock_us(a_rows, bn, (int)rest);
  return t;
}
}  // namespace

// The tile width (out features per tile) with the shortest modelled time on `sms` SMs.
// wide_rows: the epilogue reads or writes 32-bit rows (a residual sum, float32 out).
AYK_EXPORT int ayk_gemm_tc_prefill_tile_k(int M, int N, int K, int sms, int wide_rows);
AYK_EXPORT int ayk_gemm_tc_prefill_tile(int M, int N, int sms) { return ayk_gemm_tc_prefill_tile_k(M, N, 1600, sms, 0); }
AYK_EXPORT int ayk_gemm_tc_prefill_tile_k(int M, int N, int K, int sms, int wide_rows) {
  int best = 256;
  double best_us = -1.0;
  for (int bn = 32; bn <= 256; bn += 32) {
    const double us = whole_tiles_us(M, N, K, bn, sms, wide_rows != 0);
    if (best_us < 0 || us < best_us) { best_us = us; best = bn; }
  }
  return best;
}

// What the one-SM product would do for this shape on `sms` SMs: its tile width, and into how many parts it
// would split the K blocks of a tile (1: whole tiles).  Host arithmetic only; needs no device.
AYK_EXPORT void ayk_gemm_tc_prefill_plan(int M, int N, int K, int sms, int wide_rows, int* tile, int* parts) {
  int bn = ayk_gemm_tc_prefill_tile_k(M, N, K, sms, wide_rows), sp = 1, sbn = 0, ssp = 0;
  if (split_pays(M, N, K, sms, 0, wide_rows != 0, &sbn, &ssp)) { bn = sbn; sp = ssp; }
  if (tile) *tile = bn;
  if (parts) *parts = sp;
}

// The same for pairs of SMs on tiles of 256 rows (sms / 2 pairs).
AYK_EXPORT int ayk_gemm_tc_pair_tile(int M, int N, int sms) {
  int best = 256;
  long best_cost = -1;
  const int m_tiles = (M + PAIR_ROWS - 1) / PAIR_ROWS, pairs = sms / 2 > 0 ? sms / 2 : 1;
  for (int bn = 64; bn <= 256; bn += 32) {
    const long tiles = (long)m_tiles * ((N + bn - 1) / bn);
    const long waves = (tiles + pairs - 1) / pairs;
    // per K block an SM takes in 128 rows of X and bn / 2 rows of W (the bound), plus a fixed cost per tile
    const long cost = waves * (bn / 2 + 128 + 16);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// X [M, K], W [N, K] bfloat16, contiguous, 16-byte aligned, K a multiple of 8; C [M, N]
// float32 or bfloat16 with N a multiple of 8 (16-byte row segments); bias, residual
// float32 or null (residual may alias a float32 C).  tile_n: 0 lets the library choose.
// pair: 1 = two SMs per 256-row tile, 0 = one SM per 128-row tile, -1 = one SM unless the environment
// variable AYAKA_B200_GEMM_PAIR=1 asks for pairs from 129 rows on (measured equal on the XL shapes:
// both forms are bound by the tensor pipe's rate per instruction, not by operand traffic).
namespace {
struct CacheTarget {        // where the key and value columns of the product also go (see PrefillArgs, mode 4)
  void* kcache; void* vcache;
  const int* row_req; const int* pos; const int* table;
  int table_stride, page_size, col0, width;
};
// 0 when the epilogue that files keys and values applies to this call; its fields then go into `args`.
int take_cache_target(PrefillArgs& args, const CacheTarget* kv) {
  if (kv == nullptr) return 0;
  AYK_REQUIRE(args.mode == 0 && args.vec_ok && args.N == kv->col0 + 2 * kv->width && kv->col0 % 8 == 0 && kv->width % 8 == 0 &&
              kv->page_size >= 1 && (uintptr_t)kv->kcache % 16 == 0 && (uintptr_t)kv->vcache % 16 == 0,
              "ayk_gemm_tc_prefill_kv: needs bfloat16 out without activation or residual, and key and value columns in whole "
              "16-byte pieces after column %d (N %d, width %d)", kv->col0, args.N, kv->width);
  args.mode = 4;
  args.kcache = (__nv_bfloat16*)kv->kcache; args.vcache = (__nv_bfloat16*)kv->vcache;
  args.kv_row_req = kv->row_req; args.kv_pos = kv->pos; args.kv_table = kv->table;
  args.kv_table_stride = kv->table_stride; args.kv_page_size = kv->page_size; args.kv_col0 = kv->col0; args.kv_width = kv->width;
  return 0;
}
int prefill_product(void* C, const void* X, const void* W, const float* bias, const float* residual,
                    int M, int N, int K, int act, int out_dtype, int tile_n, int sms, int pair,
                    const CacheTarget* kv, cudaStream_t stream);
}  // namespace

AYK_EXPORT int ayk_gemm_tc_prefill(void* C, const void* X, const void* W, const float* bias, const float* residual,
                                   int M, int N, int K, int act, int out_dtype, int tile_n, int sms, int pair,
                                   cudaStream_t stream) {
  return prefill_product(C, X, W, bias, residual, M, N, K, act, out_dtype, tile_n, sms, pair, nullptr, stream);
}

// The same product for a fused q | k | v projection of prompt rows: the columns from col0 on, `width` keys and then
// `width` values per row, are stored into the paged caches [pages, page_size, width] as well, row t at the place
// that table[row_req[t], pos[t] / page_size] and pos[t] % page_size name (the padding page 0 takes nothing): no
// separate append kernel has to read them back.  bfloat16 out, no activation, no residual.
AYK_EXPORT int ayk_gemm_tc_prefill_kv(void* C, const void* X, const void* W, const float* bias, int M, int N, int K,
                                      int tile_n, int sms, int pair, void* kcache, void* vcache, const int* row_req,
                                      const int* pos, const int* table, int table_stride, int page_size, int col0,
                                      int width, cudaStream_t stream) {
  CacheTarget kv{kcache, vcache, row_req, pos, table, table_stride, page_size, col0, width};
  return prefill_product(C, X, W, bias, nullptr, M, N, K, AYK_ACT_NONE, AYK_DTYPE_BF16, tile_n, sms, pair, &kv, stream);
}

namespace {
int prefill_product(void* C, const void* X, const void* W, const float* bias, const float* residual,
                    int M, int N, int K, int act, int out_dtype, int tile_n, int sms, int pair,
                    const CacheTarget* kv, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  AYK_REQUIRE(K >= 8 && K % 8 == 0, "ayk_gemm_tc_prefill: K = %d must be a positive multiple of 8", K);
  AYK_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)C % 16 == 0) &&
              (residual == nullptr || (uintptr_t)residual % 16 == 0), "ayk_gemm_tc_prefill: operands must be 16-byte aligned");
  AYK_REQUIRE(out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16, "ayk_gemm_tc_prefill: unknown output dtype %d", out_dtype);
  AYK_REQUIRE(sms >= 1, "ayk_gemm_tc_prefill: sms must be positive");
  static const int pair_default = getenv("AYAKA_B200_GEMM_PAIR") ? atoi(getenv("AYAKA_B200_GEMM_PAIR")) : 0;
  const bool use_pair = pair > 0 || (pair < 0 && pair_default && M > BM && sms >= 2);
  if (use_pair) {
    AYK_REQUIRE(M > 8 && sms >= 2, "ayk_gemm_tc_prefill: pairs of SMs need more than 8 rows and 2 SMs (got %d, %d)", M, sms);
    const int BN = tile_n > 0 ? tile_n : ayk_gemm_tc_pair_tile(M, N, sms);
    AYK_REQUIRE(BN >= 64 && BN <= 256 && BN % 32 == 0, "ayk_gemm_tc_prefill: pair tile width %d is not a multiple of 32 in [64, 256]", BN);
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      if (setup() != 0) return -1;
    }
    CUtensorMap mx, mw;
    const int box_m = M >= BM ? BM : (M + 7) / 8 * 8;
    AYK_REQUIRE(box_m == BM, "ayk_gemm_tc_prefill: pairs of SMs need at least %d rows", BM);
    if (encode(&mx, X, M, K, BM) != 0) return -1;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      MapKey key{W, N, K, BN / 2};
      auto it = g_weight_maps.find(key);
      if (it == g_weight_maps.end()) {
        if (encode(&mw, W, N, K, BN / 2) != 0) return -1;
        g_weight_maps.emplace(key, mw);
      } else {
        mw = it->second;
      }
    }
    PrefillArgs args{};
    args.C = C; args.bias = bias; args.residual = residual; args.error = g_error_dev;
    args.M = M; args.N = N; args.K = K; args.act = act; args.out_bf16 = out_dtype == AYK_DTYPE_BF16;
    args.BN = BN;
    args.vec_ok = (N % 8 == 0) && (bias == nullptr || (uintptr_t)bias % 16 == 0);
    args.mode = epilogue_mode(act, residual != nullptr, args.out_bf16);
    if (take_cache_target(args, kv) != 0) return -1;
    args.box_m = BM;
    args.m_tiles = (M + PAIR_ROWS - 1) / PAIR_ROWS;
    args.n_tiles = (N + BN - 1) / BN;
    const int stages = SMEM_TILES / (A_BYTES + (BN / 2) * BLOCK_K * 2);
    args.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
    const int total = args.m_tiles * args.n_tiles, pairs = sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (total < pairs ? total : pairs));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ayk_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, mx, mw, args);
    return ayk_check_launch("ayk_gemm_tc_prefill (pairs)");
  }
  const bool wide_rows = residual != nullptr || out_dtype == AYK_DTYPE_F32;
  int BN = tile_n > 0 ? tile_n : ayk_gemm_tc_prefill_tile_k(M, N, K, sms, wide_rows ? 1 : 0);
  int splits = 1;
  if (g_split < 0) {
    int sbn = 0, ssp = 0;
    if (split_pays(M, N, K, sms, tile_n, wide_rows, &sbn, &ssp)) { BN = sbn; splits = ssp; }
  } else if (g_split >= 2) {
    splits = g_split;
  }
  AYK_REQUIRE(BN >= 32 && BN <= 256 && BN % 32 == 0, "ayk_gemm_tc_prefill: tile width %d is not a multiple of 32 in [32, 256]", BN);
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (setup() != 0) return -1;
  }
  CUtensorMap mx, mw;
  const int box_m = M >= BM ? BM : (M + 7) / 8 * 8;
  if (encode(&mx, X, M, K, box_m) != 0) return -1;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    MapKey key{W, N, K, BN};
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
      if (encode(&mw, W, N, K, BN) != 0) return -1;
      g_weight_maps.emplace(key, mw);
    } else {
      mw = it->second;
    }
  }
  PrefillArgs args{};
  args.C = C; args.bias = bias; args.residual = residual; args.error = g_error_dev;
  args.M = M; args.N = N; args.K = K; args.act = act; args.out_bf16 = out_dtype == AYK_DTYPE_BF16;
  args.BN = BN;
  args.vec_ok = (N % 8 == 0) && (bias == nullptr || (uintptr_t)bias % 16 == 0);
  args.mode = epilogue_mode(act, residual != nullptr, args.out_bf16);
  if (take_cache_target(args, kv) != 0) return -1;
  args.box_m = box_m;
  args.m_tiles = (M + BM - 1) / BM;
  args.n_tiles = (N + BN - 1) / BN;
  int stages = SMEM_TILES / (A_BYTES + BN * BLOCK_K * 2);
  args.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
  // Rows whose 16-byte segments are not aligned take the scalar path of the epilogue; N % 8 keeps them aligned.
  const int total = args.m_tiles * args.n_tiles;
  int grid_x = total < sms ? total : sms;
  args.splits = 1;
  if (splits > 1 && N % 8 == 0 && args.vec_ok && split_fits(total, (K + BLOCK_K - 1) / BLOCK_K, splits, sms, BN)) {
    args.splits = splits;
    grid_x = total * splits;
  }
  g_last_splits = args.splits;
  // float32 out over a float32 residual: both through shared memory by TMA when the tile's halves are whole
  // 32-column chunks; two buffers per half where the ring keeps four stages beside them (three for a short K),
  // else one (a long K wants its stages more than the epilogue wants its second buffer: proj2 at 2,048 rows
  // 44.0 us with two buffers and three stages, 40.7 with one and four), none below three stages
  CUtensorMap mr = mx, mc = mx;              // placeholders when the form is not taken
  args.staged = 0;
  if (g_staged && args.splits == 1 && args.mode == 1 && residual != nullptr && args.vec_ok && BN % 64 == 0 && box_m == BM &&
      (uintptr_t)C % 16 == 0 && (uintptr_t)residual % 16 == 0) {
    const int stage_bytes = A_BYTES + BN * BLOCK_K * 2;
    const int with_two = (SMEM_TILES - 4 * STAGED_CHUNK) / stage_bytes;
    const int nbuf = (with_two >= 4 || (with_two >= 3 && K <= 32 * BLOCK_K)) ? 2 : 1;     // a short K gets by with three stages
    const int left = (SMEM_TILES - 2 * nbuf * STAGED_CHUNK) / stage_bytes;
    if (left >= 3) {
      if (encode_f32(&mr, residual, M, N) != 0 || encode_f32(&mc, C, M, N) != 0) return -1;
      args.staged = nbuf;
      args.stages = left > MAX_STAGES ? MAX_STAGES : left;
    }
  }
  g_last_staged = args.staged;
  // rows of C that are no whole 16-byte pieces (N no multiple of 8), no residual: the turned epilogue
  args.turned = 0;
  if (g_staged && args.splits == 1 && !args.vec_ok && residual == nullptr && args.mode != 4) {
    const int left = (SMEM_TILES - TURNED_BYTES) / (A_BYTES + BN * BLOCK_K * 2);
    if (left >= 3) {
      args.turned = 1;
      args.stages = left > MAX_STAGES ? MAX_STAGES : left;
    }
  }
  if (args.splits > 1) {                          // the CTAs of a tile as one cluster along x
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_x);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = args.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ayk_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_prefill_kernel, mx, mw, mr, mc, args);
    return ayk_check_launch("ayk_gemm_tc_prefill (K split over a cluster)");
  }
  dim3 grid(grid_x);
  ayk_launch(gemm_tc_prefill_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mx, mw, mr, mc, args);
  return ayk_check_launch("ayk_gemm_tc_prefill");
}
}  // namespace
