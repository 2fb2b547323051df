// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), with
// operands staged by TMA and the accumulator in tensor memory:
//
//   C[M, N] = act(X[M, K] * W[N, K]^T + bias[N]) (+ residual[M, N])
//
// X are the step's rows (tokens), W a weight in [out, in] layout.  The product is
// issued "swapped": a CTA takes 128 rows of W as the MMA's M side and BT tokens
// as its N side (BT = 16 ... 256), so that a decode step with a handful of tokens
// still fills the 128 lanes of the tensor core and streams each weight byte once.
// The accumulator D[out feature, token] lies in TMEM with one out feature per
// lane; the epilogue warps read it with tcgen05.ld and write C[token, feature],
// 32 consecutive features per warp and token.
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = TMEM allocation and MMA
// issue (one lane), warps 2..5 = epilogue (bias, activation in 32-bit, residual
// sum in 32-bit).  K is cut into blocks of 64 elements (128 bytes, the 128-byte
// swizzle); a ring of stages connects producer and MMA through mbarriers.
//
// Split-K: for skinny products (decode) gridDim.z CTAs share one output tile.
// Up to 64 rows with 2, 4, 8 or 16 splits they form a thread-block cluster and
// exchange their 32-bit partial sums through distributed shared memory (see
// CLUSTER below); otherwise each writes its partial tile to scratch and the last
// to arrive sums the partials.  Either way the sum runs in split order, so the
// result does not depend on arrival order.
//
// Every wait on an mbarrier is bounded; on a time-out the kernel records an
// error word, waits (bounded) for its own copies, frees its TMEM and returns.
//
// The reference computes these products with F.linear / cuBLAS
// (layers/linear/methods.py:73-76) and the activation in a separate kernel
// (kernel/triton/activation.py:133-154).
#include <cuda.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BLOCK_N = 128;          // rows of W per CTA (UMMA M)
constexpr int BLOCK_K = 64;           // bf16 elements per stage and row: 128 bytes
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2;
constexpr int THREADS = 192;

// Up to 32 rows: 5 stages of 18-20 KB, about 100 KB per CTA, leave room for two CTAs per SM, so that
// the next kernel's CTAs (launched early, see pdl_wait) stream their weights beside the CTAs of the
// kernel before them.  Measured in a decode step at 8 requests: 3, 4, 5 stages give 3350, 3480, 3530
// tokens/s; 6 or 7 stages (one CTA per SM, no overlap with the kernel before) 2970.  64 rows are not
// split along K, so few CTAs stream a lot each: a deep ring of 8 stages.
constexpr int stages_for(int bt) { return bt >= 256 ? 4 : (bt >= 128 ? 6 : (bt >= 64 ? 8 : 5)); }
constexpr int tmem_cols_for(int bt) { return bt < 32 ? 32 : bt; }
// The cluster form adds 128 * BT floats for the exchange of partial sums and still wants two CTAs per SM.
constexpr int cluster_stages_for(int bt) { return bt >= 64 ? 3 : (bt >= 32 ? 4 : 5); }

struct EpilogueArgs {
  void* C;
  const float* bias;
  const float* residual;
  float* partials;           // [splits, M, N] float32 scratch (split-K only)
  unsigned int* counters;    // one per output tile, zero between launches (split-K only)
  int* error;
  int M, N, K;
  int act, out_bf16;
  int kb_per_split;
  int kb_base, kb_rem;        // cluster form: split z takes kb_base K blocks, one more if z < kb_rem
  long long* trace;          // cycle marks of CTA (0,0,0) when built with -DAYK_TRACE, else unused
};

#ifdef AYK_TRACE
__device__ __forceinline__ void mark(const EpilogueArgs& a, int slot) {
  if (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) a.trace[slot] = clock64();
}
#else
__device__ __forceinline__ void mark(const EpilogueArgs&, int) {}
#endif
long long* g_trace = nullptr;

// Epilogue of CNT consecutive tokens of one out feature.  All loads come first,
// arithmetic and stores after: the residual may alias C, so the compiler cannot
// move the loads ahead of the stores itself, and one load at a time would leave
// the epilogue waiting on memory latency CNT times over.
template <int CNT>
__device__ __forceinline__ void store_chunk(const EpilogueArgs& a, int tok0, int n, const float (&v)[CNT]) {
  const float b = a.bias ? a.bias[n] : 0.f;
  float res[CNT];
#pragma unroll
  for (int j = 0; j < CNT; ++j) {
    const int tok = tok0 + j;
    res[j] = (a.residual && tok < a.M) ? a.residual[(size_t)tok * a.N + n] : 0.f;
  }
#pragma unroll
  for (int j = 0; j < CNT; ++j) {
    const int tok = tok0 + j;
    if (tok < a.M) {
      const float y = apply_activation(v[j] + b, a.act) + res[j];
      const size_t idx = (size_t)tok * a.N + n;
      if (a.out_bf16) ((__nv_bfloat16*)a.C)[idx] = __float2bfloat16_rn(y);
      else ((float*)a.C)[idx] = y;
    }
  }
}

// The same with bias and residual already in registers (fetched while the main loop ran).
template <int CNT>
__device__ __forceinline__ void store_chunk_pre(const EpilogueArgs& a, int tok0, int n, const float (&v)[CNT], float b,
                                                const float* res) {
#pragma unroll
  for (int j = 0; j < CNT; ++j) {
    const int tok = tok0 + j;
    if (tok < a.M) {
      const float y = apply_activation(v[j] + b, a.act) + res[j];
      const size_t idx = (size_t)tok * a.N + n;
      if (a.out_bf16) ((__nv_bfloat16*)a.C)[idx] = __float2bfloat16_rn(y);
      else ((float*)a.C)[idx] = y;
    }
  }
}

// Split-K inside a thread-block cluster (up to 64 rows, 2, 4, 8 or 16 splits): the CTAs that share an
// output tile are one cluster along z.  Each owns 128 / splits of the tile's out features: every
// epilogue thread sends its partial sums straight into the owner's shared memory
// (st.shared::cluster); an owner that knows they are in adds the `splits` partials in split order
// and finishes its rows.  It knows either by one cluster barrier, or (DELIVERIES) by counting
// arrivals at an mbarrier of its own.  In the second form a CTA leaves only after every partner has
// delivered to it and after it has delivered to every partner, so nobody writes into a CTA that is
// gone; a cluster barrier at the head of the kernel (arrive in the set-up, wait just before the
// first delivery) makes sure the partners' mbarriers exist.  No scratch in global memory, no fence, no counter, no second pass
// through L2; measured against the scratch form inside the decode graph this takes the product
// from about 10 to 7.5 us.
template <int BT, bool CLUSTER = false>
__global__ void __launch_bounds__(THREADS, (BT <= 16 && !CLUSTER) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const EpilogueArgs args) {
  constexpr int STAGES = CLUSTER ? cluster_stages_for(BT) : stages_for(BT);
  // How an owner learns that the partial sums are in: 16 rows, one cluster barrier of all threads
  // (measured 2 % faster at one request); more rows, deliveries counted by the owner's mbarrier, so
  // that nobody waits for the slowest CTA of the cluster but the owner it delivers to (+4 % at 64).
  constexpr bool DELIVERIES = CLUSTER && BT > 16;
  constexpr int B_BYTES = BT * BLOCK_K * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TCOLS = tmem_cols_for(BT);
  constexpr uint32_t IDESC = make_idesc(BLOCK_N, BT);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;           // swizzled tiles need 1024-byte alignment
  const uint32_t bars = tiles + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t tmem_full_bar = bars + 8u * (2 * STAGES);
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 1);
  volatile uint32_t* tmem_slot_ptr = (volatile uint32_t*)(smem_raw + (tmem_slot - raw));
  volatile int* flag_ptr = (volatile int*)(smem_raw + (tmem_slot + 4 - raw));
  // cluster form: [split][row of this CTA's share][BT tokens] partial sums, 128 * BT floats
  const uint32_t share_bar = tmem_slot + 8u;                 // cluster form: deliveries of partial sums
  const uint32_t red = (tmem_slot + 16u + 15u) & ~15u;
  const float* red_ptr = (const float*)(smem_raw + (red - raw));

  if (threadIdx.x == 0) mark(args, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BLOCK_N, t0 = blockIdx.y * BT;
  const int total_kb = (args.K + BLOCK_K - 1) / BLOCK_K;
  const int kb_begin = CLUSTER ? (int)blockIdx.z * args.kb_base + min((int)blockIdx.z, args.kb_rem)
                               : (int)blockIdx.z * args.kb_per_split;
  const int num_kb = CLUSTER ? args.kb_base + ((int)blockIdx.z < args.kb_rem ? 1 : 0)
                             : min(total_kb, kb_begin + args.kb_per_split) - kb_begin;   // >= 1 by the host's choice

  if (threadIdx.x == 0) {
    // the descriptors are fetched now, not when the first copy needs them (the rows' copy comes after
    // the wait for the kernel before this one, on the critical path of a decode step)
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    if (DELIVERIES) mbar_init(share_bar, BLOCK_N / min(BLOCK_N / (int)gridDim.z, 32));   // one arrival per group of lanes
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TCOLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (DELIVERIES) cluster_arrive();       // matched by cluster_wait() in every role below
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) mark(args, 1);
  pdl_trigger();     // the next kernel may be scheduled; it waits for this one before it touches its data

  // cluster form: what the epilogue threads carry across the cluster barrier
  [[maybe_unused]] bool share_ok = false;
  constexpr int SHARE = BT / 2;                 // outputs per epilogue thread in the cluster form, at most (2 splits)
  [[maybe_unused]] float share_bias = 0.f, share_res[SHARE];
  [[maybe_unused]] int share_row = 0, share_group0 = 0, share_nn = 0;    // worked out before the main loop ends: divisions off the critical path

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      // The weight does not depend on the kernels before this one: its first
      // stages start streaming at once; the rows X wait for the predecessor.
      const int pre = min(num_kb, STAGES);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full_bar(i), STAGE_BYTES);
        tma_load_2d(tiles + i * STAGE_BYTES, &map_w, (kb_begin + i) * BLOCK_K, n0, full_bar(i));
      }
      mark(args, 2);
      pdl_wait();
      mark(args, 3);
      for (int i = 0; i < pre; ++i)
        tma_load_2d(tiles + i * STAGE_BYTES + A_BYTES, &map_x, (kb_begin + i) * BLOCK_K, t0, full_bar(i));
      int issued = pre;
      for (int i = pre; i < num_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(empty_bar(s), phase ^ 1u, args.error, 1);
        if (!ok) break;
        if (i < 12) mark(args, 32 + 4 * i);
        mbar_expect_tx(full_bar(s), STAGE_BYTES);
        const uint32_t a_dst = tiles + s * STAGE_BYTES;
        const int kx = (kb_begin + i) * BLOCK_K;
        if (i < 12) mark(args, 33 + 4 * i);
        tma_load_2d(a_dst, &map_w, kx, n0, full_bar(s));
        if (i < 12) mark(args, 34 + 4 * i);
        tma_load_2d(a_dst + A_BYTES, &map_x, kx, t0, full_bar(s));
        if (i < 12) mark(args, 35 + 4 * i);
        issued = i + 1;
      }
      if (!ok) {
        // Nobody may be consuming any more: wait for the copies already issued.
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(full_bar(i % STAGES), (uint32_t)(i / STAGES) & 1u, args.error, 2);
      }
    }
    __syncwarp();
    if (DELIVERIES) cluster_wait();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        ok = mbar_wait(full_bar(s), phase, args.error, 3);
        if (!ok) break;
        if (i == 0) mark(args, 4);
        if (i < 12) mark(args, 96 + 4 * i);
        tc_fence_after();
        const uint32_t a_src = tiles + s * STAGE_BYTES;
        const uint64_t da0 = make_desc(a_src), db0 = make_desc(a_src + A_BYTES);
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
          // 32 bytes further along K inside the swizzle atom: the address field counts 16-byte units
          const uint64_t da = da0 + (uint64_t)(k * UMMA_K * 2 / 16), db = db0 + (uint64_t)(k * UMMA_K * 2 / 16);
          umma(tmem_base, da, db, IDESC, (i > 0 || k > 0) ? 1u : 0u);
        }
        if (i < 12) mark(args, 97 + 4 * i);
        umma_commit(empty_bar(s));          // the stage is free once these MMAs have read it
        if (i < 12) mark(args, 98 + 4 * i);
      }
      umma_commit(tmem_full_bar);           // arrives when every MMA issued so far is done
      mark(args, 5);
    }
    __syncwarp();
    if (DELIVERIES) cluster_wait();
  } else {
    // Epilogue: warp w may read TMEM lanes 32 * (w % 4) ... + 31.
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    if constexpr (CLUSTER) {
      // This CTA finishes rows_per of the tile's out features.  Thread e of the epilogue takes feature
      // e % rows_per and the groups of four tokens e / rows_per + splits * i: neighbouring threads
      // write neighbouring features of one token, and a thread reads whole 16-byte pieces.
      const int splits = gridDim.z, rows_per = BLOCK_N / splits, e = threadIdx.x - 64;
      const int my_row = e % rows_per, group_first = e / rows_per;
      const int nn = n0 + (int)blockIdx.z * rows_per + my_row;
      share_row = my_row; share_group0 = group_first; share_nn = nn;
      share_bias = (nn < args.N && args.bias) ? __ldg(args.bias + nn) : 0.f;     // a weight: no need to wait for it
      pdl_wait();      // residual and C belong to kernels before this one until here
#pragma unroll
      for (int i = 0; i < SHARE / 4; ++i) {
        const int g = group_first + splits * i;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int tok = t0 + 4 * g + u;
          share_res[4 * i + u] = (g < BT / 4 && nn < args.N && args.residual && tok < args.M)
                                     ? args.residual[(size_t)tok * args.N + nn] : 0.f;
        }
      }
      // where this thread's partial sums go (worked out while the main loop runs)
      const int local = quarter * 32 + lane, rrow = local % rows_per, owner = local / rows_per;
      const uint32_t dst = map_to_cta(red + (uint32_t)((((int)blockIdx.z * rows_per + rrow) * BT) * 4), (uint32_t)owner);
      const uint32_t owner_bar = DELIVERIES ? map_to_cta(share_bar, (uint32_t)owner) : 0u;
      // The same for lanes 0, 8, 16 and 24 of this warp, plus this lane's 16 bytes: the staged form
      // below sends whole rows, 128 / BT of them per instruction, none of which straddles a group of 8
      // (a share of the tile is at least 8 features).
      [[maybe_unused]] uint32_t dst_group[4] = {0u, 0u, 0u, 0u};
      if constexpr (BT > 16) {
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const int first = quarter * 32 + 8 * h;
          dst_group[h] = map_to_cta(red + (uint32_t)((((int)blockIdx.z * rows_per + first % rows_per) * BT) * 4),
                                    (uint32_t)(first / rows_per)) + 16u * (uint32_t)lane;
        }
      }
      if (DELIVERIES) cluster_wait();      // every partner has set up its barriers (long ago; the main loop still runs)
      share_ok = mbar_wait(tmem_full_bar, 0u, args.error, 4);
      tc_fence_after();
      if (share_ok) {
        // Feature `local` of the tile belongs to CTA local / rows_per of the cluster; its BT sums go to
        // [this split][local % rows_per][0 .. BT) of that CTA's buffer, the 16-byte pieces of a row
        // rotated by the row number so that the readers (one feature per lane) spread over the banks.
        if constexpr (BT == 16) {
          uint32_t r[16];
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16), r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int piece = q ^ (rrow & (BT / 4 - 1));
            st_cluster_v4(dst + 16u * piece, __uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                          __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          }
        } else {
          // One lane holds one row: sent as it is, an instruction would touch 32 rows, 16 bytes of each,
          // and the 64-row product spent 1.8 us sending.  So the warp first lays its 32 rows down in
          // this CTA's shared memory as they shall lie in the owner's (the main loop's stages are
          // free: every MMA is done), then copies them 512 contiguous bytes per instruction.
          const uint32_t stage = tiles + (uint32_t)(quarter * 32 * BT * 4);
          const uint32_t my_stage = stage + (uint32_t)(lane * BT * 4);
#pragma unroll
          for (int c = 0; c < BT; c += 16) {
            uint32_t r[16];
            tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, r);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int piece = ((c >> 2) + q) ^ (rrow & (BT / 4 - 1));     // as the owner's readers expect it
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_stage + 16u * piece), "r"(r[4 * q]),
                           "r"(r[4 * q + 1]), "r"(r[4 * q + 2]), "r"(r[4 * q + 3]) : "memory");
            }
          }
          __syncwarp();
          constexpr int ROWS_PER_COPY = 128 / BT;
#pragma unroll
          for (int j = 0; j < BT / 4; ++j) {
            float a, b, c, d;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
                         : "r"(stage + (uint32_t)(j * 512 + lane * 16)) : "memory");
            const int row = j * ROWS_PER_COPY;
            st_cluster_v4(dst_group[row / 8] + (uint32_t)((row % 8) * BT * 4), a, b, c, d);
          }
        }
      }
      // delivered (or given up: the error word says so): one lane arrives for the lanes that share its owner
      if (DELIVERIES) {
        __syncwarp();
        if ((lane & (min(rows_per, 32) - 1)) == 0) mbar_arrive_cluster(owner_bar);
      }
    } else {
    pdl_wait();        // residual, partials and C belong to kernels before this one until here
    // Bias and the residual of the first 16 tokens are fetched while the main loop runs.
    const float bias_pre = (args.bias && n < args.N) ? args.bias[n] : 0.f;
    float res_pre[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int tok = t0 + j;
      res_pre[j] = (args.residual && n < args.N && tok < args.M) ? args.residual[(size_t)tok * args.N + n] : 0.f;
    }
    const bool ok = mbar_wait(tmem_full_bar, 0u, args.error, 4);
    if (threadIdx.x == 64) mark(args, 6);
    tc_fence_after();
    const int splits = gridDim.z;
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < BT; c += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, r);
        tmem_ld_wait();
        if (n < args.N && t0 + c < args.M) {
          if (splits == 1) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            if (c == 0) store_chunk_pre<16>(args, t0, n, v, bias_pre, res_pre);
            else store_chunk<16>(args, t0 + c, n, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = t0 + c + j;
              if (tok < args.M) args.partials[((size_t)blockIdx.z * args.M + tok) * args.N + n] = __uint_as_float(r[j]);
            }
          }
        }
      }
    }
    if (threadIdx.x == 64) mark(args, 9);
    if (splits > 1) {
      // The last CTA of this tile to arrive sums the partials in split order.
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const unsigned tile = blockIdx.y * gridDim.x + blockIdx.x;
      if (threadIdx.x == 64) {
        unsigned old = atomicAdd(&args.counters[tile], 1u);
        *flag_ptr = (old == (unsigned)splits - 1u) ? 1 : 0;
        if (old == (unsigned)splits - 1u) args.counters[tile] = 0u;    // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*flag_ptr && ok) {
        __threadfence();
        if (n < args.N) {
          // 4 tokens x 8 splits = 32 loads in flight per thread; summed in split
          // order, so the result does not depend on which CTA arrived last.
          constexpr int TK = 4;
          auto reduce = [&](int c, float (&v)[TK]) {
#pragma unroll
            for (int u = 0; u < TK; ++u) v[u] = 0.f;
            for (int z0 = 0; z0 < splits; z0 += 8) {
              float p[8][TK];
#pragma unroll
              for (int zz = 0; zz < 8; ++zz) {
#pragma unroll
                for (int u = 0; u < TK; ++u) {
                  const int z = z0 + zz, tok = t0 + c + u;
                  p[zz][u] = (z < splits && tok < args.M)
                                 ? __ldcg(&args.partials[((size_t)z * args.M + tok) * args.N + n]) : 0.f;
                }
              }
#pragma unroll
              for (int zz = 0; zz < 8; ++zz) {
#pragma unroll
                for (int u = 0; u < TK; ++u) v[u] += p[zz][u];
              }
            }
          };
          // The first 16 tokens use the bias and residual fetched before the main loop ended.
#pragma unroll
          for (int c = 0; c < 16; c += TK) {
            if (t0 + c < args.M) {
              float v[TK];
              reduce(c, v);
              float res[TK];
#pragma unroll
              for (int u = 0; u < TK; ++u) res[u] = res_pre[c + u];
              store_chunk_pre<TK>(args, t0 + c, n, v, bias_pre, res);
            }
          }
          for (int c = 16; c < BT && t0 + c < args.M; c += TK) {
            float v[TK];
            reduce(c, v);
            store_chunk<TK>(args, t0 + c, n, v);
          }
        }
      }
    }
    }   // !CLUSTER
  }

  if constexpr (CLUSTER) {
    if (!DELIVERIES) {                     // every thread of every CTA of the cluster
      cluster_arrive();
      cluster_wait();
    }
    if (warp >= 2) {
      bool got = true;
      if (DELIVERIES) {                    // one lane per warp watches for the deliveries to this CTA
        if (lane == 0) got = mbar_wait_cluster(share_bar, 0u, args.error, 6);
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
      }
      if (got && share_ok && share_nn < args.N) {
        // The loop below runs once per launch: what it costs is the fetching of its instructions, so
        // it is kept short (16-byte reads, the number of splits a constant of each copy).  Unrolled
        // over single outputs it took 0.9 us at 16 rows and 4.8 us at 64, mostly waiting for code.
        const int my_row = share_row, group_first = share_group0, nn = share_nn;
        auto finish = [&](auto split_count) {
          constexpr int S = decltype(split_count)::value, ROWS_PER = BLOCK_N / S;
          const float* mine = red_ptr + my_row * BT;
#pragma unroll
          for (int i = 0; i < SHARE / 4; ++i) {
            const int g = group_first + S * i;
            if (S * i < BT / 4 && g < BT / 4 && t0 + 4 * g < args.M) {
              const float* at = mine + ((g ^ (my_row & (BT / 4 - 1))) << 2);
              float4 part[S];
#pragma unroll
              for (int z = 0; z < S; ++z) part[z] = *(const float4*)(at + z * ROWS_PER * BT);
              float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int z = 0; z < S; ++z) {                     // split order
                v[0] += part[z].x; v[1] += part[z].y; v[2] += part[z].z; v[3] += part[z].w;
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int tok = t0 + 4 * g + u;
                if (tok < args.M) {
                  const float y = apply_activation(v[u] + share_bias, args.act) + share_res[4 * i + u];
                  const size_t idx = (size_t)tok * args.N + nn;
                  if (args.out_bf16) ((__nv_bfloat16*)args.C)[idx] = __float2bfloat16_rn(y);
                  else ((float*)args.C)[idx] = y;
                }
              }
            }
          }
        };
        const int splits = gridDim.z;
        if (splits == 16) finish(std::integral_constant<int, 16>());
        else if (splits == 8) finish(std::integral_constant<int, 8>());
        else if (splits == 4) finish(std::integral_constant<int, 4>());
        else finish(std::integral_constant<int, 2>());
      }
    }
  }
  if (threadIdx.x == 64) mark(args, 7);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) mark(args, 8);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TCOLS) : "memory");
  }
}

// ------------------------------------------------------------------- host --

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
int* g_error_host = nullptr;     // mapped pinned memory: the kernels write, the host reads without a copy
int* g_error_dev = nullptr;
std::mutex g_mutex;

struct MapKey {
  const void* ptr; int rows, k, box;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box == o.box; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1000003u ^ (size_t)k.k * 10007u ^ (size_t)k.box;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_weight_maps;

int setup() {
  if (g_encode && g_error_host) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (err != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
    return ayk_fail("ayk_gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  g_encode = (EncodeTiledFn)fn;
  err = cudaHostAlloc((void**)&g_error_host, sizeof(int), cudaHostAllocMapped);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc: cudaHostAlloc: %s", cudaGetErrorString(err));
  *g_error_host = 0;
  err = cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0);
  if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc: cudaHostGetDevicePointer: %s", cudaGetErrorString(err));
  return 0;
}

// rows x k bfloat16, row-major; box of `box_rows` rows x 64 elements, 128-byte swizzle.
int encode(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ayk_fail("ayk_gemm_tc: cuTensorMapEncodeTiled failed with %d (rows %d, k %d, box %d)", (int)r, rows, k, box_rows);
  return 0;
}

template <int BT>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const EpilogueArgs& args, int splits, cudaStream_t stream) {
  constexpr int STAGES = stages_for(BT);
  constexpr size_t SMEM = 1024 + (size_t)STAGES * (A_BYTES + BT * BLOCK_K * 2) + 8 * (2 * STAGES + 2);
  static AykPerDevice configured;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    bool& done = configured.here();
    if (!done) {
      cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc: shared memory %zu: %s", SMEM, cudaGetErrorString(err));
      done = true;
    }
  }
  dim3 grid((args.N + BLOCK_N - 1) / BLOCK_N, (args.M + BT - 1) / BT, splits);
  ayk_launch(gemm_tc_kernel<BT>, grid, dim3(THREADS), SMEM, stream, mw, mx, args);
  return ayk_check_launch("ayk_gemm_tc");
}

// Up to 64 rows, the CTAs of an output tile as one cluster along z.
template <int BT>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const EpilogueArgs& args, int splits, cudaStream_t stream) {
  constexpr int STAGES = cluster_stages_for(BT);
  constexpr size_t SMEM = 1024 + (size_t)STAGES * (A_BYTES + BT * BLOCK_K * 2) + 8 * (2 * STAGES + 3) + 16 + BLOCK_N * BT * sizeof(float);
  static AykPerDevice configured;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    bool& done = configured.here();
    if (!done) {
      cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc: shared memory %zu: %s", SMEM, cudaGetErrorString(err));
      // clusters of 16 are beyond the portable size of 8
      err = cudaFuncSetAttribute(gemm_tc_kernel<BT, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (err != cudaSuccess) return ayk_fail("ayk_gemm_tc: clusters of 16: %s", cudaGetErrorString(err));
      done = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((args.N + BLOCK_N - 1) / BLOCK_N, 1, splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ayk_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BT, true>, mw, mx, args);
  return ayk_check_launch("ayk_gemm_tc (cluster)");
}

}  // namespace

// 0 when the kernel takes this shape; otherwise a text in ayk_last_error().
AYK_EXPORT int ayk_gemm_tc_supported(int M, int N, int K) {
  if (M < 1 || N < 1 || K < 8 || K % 8 != 0)
    return ayk_fail("ayk_gemm_tc: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  return 0;
}

// The error word of the tensor-core kernels: 0, or the code of the wait that ran out.
// Where the cycle marks of the next launches go (device memory, 16 int64); only read by builds with -DAYK_TRACE.
AYK_EXPORT void ayk_gemm_tc_set_trace(long long* p) { g_trace = p; }
AYK_EXPORT int ayk_gemm_tc_error() { return g_error_host ? *g_error_host : 0; }
AYK_EXPORT void ayk_gemm_tc_clear_error() { if (g_error_host) *g_error_host = 0; }

// How many float32 scratch elements and tile counters a call needs.
AYK_EXPORT long long ayk_gemm_tc_scratch_floats(int M, int N, int splits) {
  return splits > 1 ? (long long)splits * M * N : 0;
}

// X [M, K] and W [N, K] bfloat16 (contiguous, 16-byte aligned); C [M, N] float32
// or bfloat16; bias, residual float32 or null (residual may alias a float32 C).
// splits > 1 needs `partials` (ayk_gemm_tc_scratch_floats) and `counters` (one
// zeroed unsigned per output tile; the kernel leaves them zero), unless cluster != 0: then the
// splits of a tile are one thread-block cluster and exchange their sums through shared memory
// (up to 64 rows; 2, 4, 8 or 16 splits; at least one K block each), and no scratch is touched.
AYK_EXPORT int ayk_gemm_tc(void* C, const void* X, const void* W, const float* bias, const float* residual,
                           int M, int N, int K, int act, int out_dtype, int splits, float* partials,
                           unsigned int* counters, int weight_is_static, int cluster, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (ayk_gemm_tc_supported(M, N, K) != 0) return -1;
  AYK_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "ayk_gemm_tc: operands must be 16-byte aligned");
  AYK_REQUIRE(out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16, "ayk_gemm_tc: unknown output dtype %d", out_dtype);
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (splits < 1) splits = 1;
  if (splits > total_kb) splits = total_kb;
  if (cluster) {
    AYK_REQUIRE(M <= 64 && (splits == 2 || splits == 4 || splits == 8 || splits == 16) && total_kb >= splits,
                "ayk_gemm_tc: the cluster form takes up to 64 rows and 2, 4, 8 or 16 splits of at least one K block (rows %d, splits %d, K blocks %d)",
                M, splits, total_kb);
  }
  int kb_per_split = (total_kb + splits - 1) / splits;
  if (!cluster) splits = (total_kb + kb_per_split - 1) / kb_per_split;       // no empty split
  AYK_REQUIRE(splits == 1 || cluster || (partials && counters), "ayk_gemm_tc: split-K needs scratch");
  AYK_REQUIRE(splits <= 65535, "ayk_gemm_tc: too many splits");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (setup() != 0) return -1;
  }
  const int BT = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  AYK_REQUIRE((M + BT - 1) / BT <= 65535, "ayk_gemm_tc: too many rows (%d)", M);
  CUtensorMap mw, mx;
  if (weight_is_static) {
    std::lock_guard<std::mutex> lock(g_mutex);
    MapKey key{W, N, K, BLOCK_N};
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
      if (encode(&mw, W, N, K, BLOCK_N) != 0) return -1;
      g_weight_maps.emplace(key, mw);
    } else {
      mw = it->second;
    }
  } else if (encode(&mw, W, N, K, BLOCK_N) != 0) {
    return -1;
  }
  if (encode(&mx, X, M, K, BT) != 0) return -1;
  EpilogueArgs args{C, bias, residual, partials, counters, g_error_dev, M, N, K, act, out_dtype == AYK_DTYPE_BF16, kb_per_split,
                    total_kb / splits, total_kb % splits, g_trace};
  if (cluster) return BT == 16 ? launch_cluster<16>(mw, mx, args, splits, stream)
                      : (BT == 32 ? launch_cluster<32>(mw, mx, args, splits, stream) : launch_cluster<64>(mw, mx, args, splits, stream));
  switch (BT) {
    case 16: return launch<16>(mw, mx, args, splits, stream);
    case 32: return launch<32>(mw, mx, args, splits, stream);
    case 64: return launch<64>(mw, mx, args, splits, stream);
    case 128: return launch<128>(mw, mx, args, splits, stream);
    default: return launch<256>(mw, mx, args, splits, stream);
  }
}

// ------------------------------------------------------ no-allocation entry --
// See no_alloc.h.  The scratch of the split-K product lives in the library image.
#include "no_alloc.h"

namespace {

static __device__ __align__(256) float g_na_partials[AYK_NO_ALLOC_MAX_PARTIALS];
static __device__ __align__(256) unsigned int g_na_counters[AYK_NO_ALLOC_MAX_TILES];
static __device__ __align__(256) int g_na_error[64];

constexpr int NA_MAX_DEVICES = 64;
struct NoAllocDevice {
  bool ready;
  float* partials;
  unsigned int* counters;
  int* error;
};
NoAllocDevice g_na_devices[NA_MAX_DEVICES];   // zero-initialised; one entry per device ordinal
EncodeTiledFn g_na_encode = nullptr;

// Once per device, with that device current: the names of the __device__ arrays
// are host-side stand-ins, so their device addresses are asked for here.
int no_alloc_setup(int device) {
  // Under the library's mutex: two threads that make their first call on a device together
  // would otherwise both write the table.
  std::lock_guard<std::mutex> lock(g_mutex);
  NoAllocDevice& d = g_na_devices[device];
  if (d.ready) return 0;
  if (g_na_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
      return ayk_fail("ayk_gemm_tc_no_alloc: cuTensorMapEncodeTiled is not available from this driver");
    g_na_encode = (EncodeTiledFn)fn;
  }
  cudaError_t e = cudaGetSymbolAddress((void**)&d.partials, g_na_partials);
  if (e != cudaSuccess) return ayk_fail("ayk_gemm_tc_no_alloc: cudaGetSymbolAddress(partials): %s", cudaGetErrorString(e));
  e = cudaGetSymbolAddress((void**)&d.counters, g_na_counters);
  if (e != cudaSuccess) return ayk_fail("ayk_gemm_tc_no_alloc: cudaGetSymbolAddress(counters): %s", cudaGetErrorString(e));
  e = cudaGetSymbolAddress((void**)&d.error, g_na_error);
  if (e != cudaSuccess) return ayk_fail("ayk_gemm_tc_no_alloc: cudaGetSymbolAddress(error): %s", cudaGetErrorString(e));
  d.ready = true;
  return 0;
}

int no_alloc_encode(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = g_na_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ayk_fail("ayk_gemm_tc_no_alloc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

}  // namespace

AYK_EXPORT int ayk_gemm_tc_no_alloc(void* C, const void* X, const void* W, const float* bias, const float* residual,
                                    int M, int N, int K, int act, int out_dtype, int splits, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (ayk_gemm_tc_supported(M, N, K) != 0) return -1;
  AYK_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "ayk_gemm_tc_no_alloc: operands must be 16-byte aligned");
  AYK_REQUIRE(out_dtype == AYK_DTYPE_F32 || out_dtype == AYK_DTYPE_BF16, "ayk_gemm_tc_no_alloc: unknown output dtype %d", out_dtype);
  const int BT = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  const int tiles = ((N + BLOCK_N - 1) / BLOCK_N) * ((M + BT - 1) / BT);
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (splits <= 0) {
    // The library chooses: about one CTA per multiprocessor, but never more partial sums than the
    // built-in scratch holds, and no split at all where the tile counters would not suffice.
    const int sms = ayk_sm_count();
    splits = tiles >= sms / 2 ? 1 : sms / tiles;
    const long long room = (long long)AYK_NO_ALLOC_MAX_PARTIALS / ((long long)M * N);
    if (splits > room) splits = room < 1 ? 1 : (int)room;
    if (tiles > AYK_NO_ALLOC_MAX_TILES) splits = 1;
  }
  if (splits > total_kb) splits = total_kb;
  const int kb_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + kb_per_split - 1) / kb_per_split;
  AYK_REQUIRE((M + BT - 1) / BT <= 65535 && splits <= 65535, "ayk_gemm_tc_no_alloc: the grid would be too large");
  if (splits > 1) {
    AYK_REQUIRE((long long)splits * M * N <= (long long)AYK_NO_ALLOC_MAX_PARTIALS,
                "ayk_gemm_tc_no_alloc: splits * M * N = %lld floats of scratch exceed the built-in %d; "
                "use fewer splits or the allocating entry point", (long long)splits * M * N, AYK_NO_ALLOC_MAX_PARTIALS);
    AYK_REQUIRE(tiles <= AYK_NO_ALLOC_MAX_TILES, "ayk_gemm_tc_no_alloc: %d output tiles exceed the built-in %d counters",
                tiles, AYK_NO_ALLOC_MAX_TILES);
  }
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return ayk_fail("ayk_gemm_tc_no_alloc: cudaGetDevice: %s", cudaGetErrorString(e));
  AYK_REQUIRE(device >= 0 && device < NA_MAX_DEVICES, "ayk_gemm_tc_no_alloc: device ordinal %d is out of range", device);
  if (no_alloc_setup(device) != 0) return -1;
  const NoAllocDevice& d = g_na_devices[device];
  if (splits > 1) {
    // The counters must start at zero; an earlier call that was cut short may have left them otherwise.
    e = cudaMemsetAsync(d.counters, 0, sizeof(unsigned int) * (size_t)tiles, stream);
    if (e != cudaSuccess) return ayk_fail("ayk_gemm_tc_no_alloc: cudaMemsetAsync: %s", cudaGetErrorString(e));
  }
  CUtensorMap mw, mx;
  if (no_alloc_encode(&mw, W, N, K, BLOCK_N) != 0) return -1;
  if (no_alloc_encode(&mx, X, M, K, BT) != 0) return -1;
  EpilogueArgs args{C, bias, residual, d.partials, d.counters, d.error, M, N, K, act, out_dtype == AYK_DTYPE_BF16, kb_per_split, 0, 0, g_trace};
  switch (BT) {
    case 16: return launch<16>(mw, mx, args, splits, stream);
    case 32: return launch<32>(mw, mx, args, splits, stream);
    case 64: return launch<64>(mw, mx, args, splits, stream);
    case 128: return launch<128>(mw, mx, args, splits, stream);
    default: return launch<256>(mw, mx, args, splits, stream);
  }
}

AYK_EXPORT int ayk_gemm_tc_no_alloc_error(void) {
  int value = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&value, g_na_error, sizeof(int));
  if (e != cudaSuccess) return -1;
  return value;
}
