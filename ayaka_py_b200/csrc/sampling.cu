// Greedy and temperature sampling over float32 logits, one block per row.
//
// Greedy: the lowest index among the maxima (argmax, sampling/plan.py:353-355).
// Temperature: scaled = logits / max(T, 1e-6) (sampling/plan.py:348-349),
// p = softmax(scaled) in 32-bit, one uniform u = Philox4x32-10(key = seed,
// counter = offset >> 1, words picked by offset & 1; 53 bits,
// sampling/rng.py:126-173), and the first token, in token-id order, at which the
// running sum of p reaches u * total.  (The reference walks the running sum in
// descending-probability order, sampling/ops/sampling.py:587-589: the same
// distribution.)  The draw depends only on the row's logits, seed and offset,
// never on which other rows share the batch.
//
// Filters, in the reference's order (sampling/ops/sampling.py:473-540): top_k
// (keep the k most probable), renormalise, top_p (keep a token while the
// probability mass of the more probable ones is <= top_p; the first always
// stays), min_p (keep p >= min_p * p_max).  Each becomes a threshold on
// exp(z - zmax): the k-th largest value is found by a radix select over the
// float's bits, the nucleus edge by the same walk over sums kept as 64-bit
// fixed point (integer atomics: the same result whatever the order).  Tokens
// of exactly equal probability at a threshold are kept together.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 512;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ double philox_uniform(unsigned long long seed, unsigned long long offset) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  unsigned long long ctr = offset >> 1;
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    if (r > 0) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
    philox_round(c, k0, k1);
  }
  uint32_t hi = (offset & 1ull) ? c[2] : c[0], lo = (offset & 1ull) ? c[3] : c[1];
  unsigned long long v = ((unsigned long long)hi << 32) | lo;
  return (double)(v >> 11) * (1.0 / 9007199254740992.0);
}

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ MaxIdx block_argmax(const float* row, int V, MaxIdx* red) {
  MaxIdx best = {-INFINITY, 0x7fffffff};
  // Sixteen independent loads in flight per thread (a row of 50,257 is six trips to L2 instead of
  // twelve); compared in ascending index order, so that the first maximum stays.
  constexpr int FLY = 16;
  for (int base = threadIdx.x; base < V; base += blockDim.x * FLY) {
    float v[FLY];
#pragma unroll
    for (int u = 0; u < FLY; ++u) {
      const int i = base + u * blockDim.x;
      v[u] = i < V ? row[i] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < FLY; ++u) {
      if (v[u] > best.v) { best.v = v[u]; best.i = base + u * blockDim.x; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = best;
  __syncthreads();
  MaxIdx total = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) total = better(total, red[w]);
  if (total.i == 0x7fffffff) total.i = 0;   // a row of NaN or -inf
  return total;
}


constexpr double FIXED_ONE = 1099511627776.0;   // 2^40: exp(z - zmax) <= 1 as fixed point

// exp(z - zmax) of one logit, z = logit / T rounded to 32-bit before the subtraction, as zmax is: the
// row's maximum then has the weight 1 exactly and no weight is above it.  (Left to the compiler, the
// product and the subtraction fuse, the maximum's own weight comes out as 1 - 4e-6 or 1 + 4e-6, and a
// filter that keeps "the maximum only" - min_p = 1, top_k = 1 - kept nothing or the wrong token.)
__device__ __forceinline__ float row_weight(float logit, float inv_t, float zmax) {
  return expf(__fsub_rn(__fmul_rn(logit, inv_t), zmax));
}

__device__ __forceinline__ unsigned long long to_fixed(float e) {
  return (unsigned long long)((double)e * FIXED_ONE);
}

// Bits of the k-th largest exp(z - zmax) of the row (0 when k >= V).
__device__ uint32_t select_kth(const float* row, int V, float inv_t, float zmax, long long k,
                               unsigned long long* hist, uint32_t* shared_u32) {
  if (k <= 0 || k >= V) return 0u;
  uint32_t prefix = 0u, mask = 0u;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      uint32_t bits = __float_as_uint(row_weight(row[i], inv_t, zmax));
      if ((bits & mask) == prefix) atomicAdd(&hist[(bits >> shift) & 255u], 1ull);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int chosen = 0;
      for (int b = 255; b >= 0; --b) {
        if ((long long)hist[b] >= k) { chosen = b; break; }
        k -= (long long)hist[b];
      }
      shared_u32[0] = (uint32_t)chosen;
      shared_u32[1] = (uint32_t)k;
    }
    __syncthreads();
    prefix |= shared_u32[0] << shift;
    mask |= 255u << shift;
    k = (long long)shared_u32[1];
    __syncthreads();
  }
  return prefix;
}

// Bits of the least probable token that top_p keeps among those with bits >= floor_bits.
__device__ uint32_t select_nucleus(const float* row, int V, float inv_t, float zmax, uint32_t floor_bits,
                                   float top_p, unsigned long long* hist, unsigned long long* shared_u64,
                                   uint32_t* shared_u32) {
  if (threadIdx.x == 0) shared_u64[0] = 0ull;
  __syncthreads();
  unsigned long long mine = 0ull;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float e = row_weight(row[i], inv_t, zmax);
    if (__float_as_uint(e) >= floor_bits) mine += to_fixed(e);
  }
  atomicAdd(&shared_u64[0], mine);
  __syncthreads();
  const unsigned long long limit = (unsigned long long)((double)top_p * (double)shared_u64[0]);
  __syncthreads();
  uint32_t prefix = 0u, mask = 0u;
  unsigned long long above = 0ull;     // mass of the tokens more probable than the current prefix range
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float e = row_weight(row[i], inv_t, zmax);
      uint32_t bits = __float_as_uint(e);
      if (bits >= floor_bits && (bits & mask) == prefix) atomicAdd(&hist[(bits >> shift) & 255u], to_fixed(e));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int chosen = -1;
      unsigned long long run = above;
      for (int b = 255; b >= 0; --b) {
        if (hist[b] == 0ull) continue;
        if (run + hist[b] > limit) { chosen = b; break; }
        run += hist[b];
      }
      shared_u32[0] = (uint32_t)(chosen < 0 ? 256 : chosen);
      shared_u64[1] = run;
    }
    __syncthreads();
    if (shared_u32[0] == 256u) return floor_bits;   // the whole mass fits: top_p drops nothing
    prefix |= shared_u32[0] << shift;
    mask |= 255u << shift;
    above = shared_u64[1];
    __syncthreads();
  }
  return prefix > floor_bits ? prefix : floor_bits;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int V,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const long long* __restrict__ offset, const long long* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p) {
  __shared__ MaxIdx red[THREADS / 32];
  __shared__ double partial[THREADS];
  __shared__ int chosen_thread;
  __shared__ double chosen_base, target_s;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  MaxIdx top = block_argmax(row, V, red);
  float temp = temperature ? temperature[r] : 0.f;
  if (temp <= 0.f) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float inv_t = 1.0f / fmaxf(temp, 1e-6f);
  const float zmax = __fmul_rn(top.v, inv_t);
  if (!(top.v > -INFINITY)) {                    // a row without a finite logit: as greedy
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long shared_u64[2];
  __shared__ uint32_t shared_u32[2];
  uint32_t keep_bits = 0u;       // a token stays when the bits of exp(z - zmax) reach this
  if (top_k && top_k[r] > 0) keep_bits = select_kth(row, V, inv_t, zmax, top_k[r], hist, shared_u32);
  if (top_p && top_p[r] < 1.0f)
    keep_bits = select_nucleus(row, V, inv_t, zmax, keep_bits, top_p[r], hist, shared_u64, shared_u32);
  if (min_p && min_p[r] > 0.f) keep_bits = max(keep_bits, __float_as_uint(fminf(min_p[r], 1.0f)));
  // Each thread owns one contiguous segment, so that the running sum goes
  // through the tokens in id order.
  const int seg = (V + THREADS - 1) / THREADS;
  const int lo = min(V, (int)threadIdx.x * seg), hi = min(V, lo + seg);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) {
    float e = row_weight(row[i], inv_t, zmax);
    if (__float_as_uint(e) >= keep_bits) s += e;
  }
  partial[threadIdx.x] = (double)s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int t = 0; t < THREADS; ++t) total += partial[t];
    double u = philox_uniform((unsigned long long)seed[r], (unsigned long long)offset[r]);
    double target = u * total;
    double run = 0.0;
    int pick = -1;
    for (int t = 0; t < THREADS; ++t) {
      if (partial[t] > 0.0 && run + partial[t] >= target) { pick = t; break; }
      run += partial[t];
    }
    if (pick < 0) {   // rounding left target above the last running sum
      run = 0.0;
      for (int t = 0; t < THREADS; ++t) {
        if (partial[t] > 0.0) pick = t;
      }
      for (int t = 0; t < pick; ++t) run += partial[t];
    }
    chosen_thread = pick;
    chosen_base = run;
    target_s = target;
  }
  __syncthreads();
  if ((int)threadIdx.x == chosen_thread) {
    double run = chosen_base;
    int token = -1, last_positive = lo;
    for (int i = lo; i < hi; ++i) {
      float p = row_weight(row[i], inv_t, zmax);
      if (__float_as_uint(p) < keep_bits) p = 0.f;
      if (p > 0.f) last_positive = i;
      run += (double)p;
      if (p > 0.f && run >= target_s) { token = i; break; }
    }
    out[r] = token >= 0 ? token : last_positive;
  }
}

// Tokens that a row must not produce yet (stop ids and EOS before the request's min_tokens,
// request/stream.py:130-136 in the reference): their logits become -inf before sampling.
__global__ void ban_tokens_kernel(float* logits, const int* rows, const int* tokens, int count, int S, int V) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int r = rows[i], t = tokens[i];
  if (r >= 0 && r < S && t >= 0 && t < V) logits[(size_t)r * V + t] = -INFINITY;
}

}  // namespace

// logits[rows[i], tokens[i]] = -inf for i < count (pairs outside [S, V] are ignored).
AYK_EXPORT int ayk_ban_tokens(float* logits, const int* rows, const int* tokens, int count, int S, int V,
                              cudaStream_t stream) {
  if (count == 0) return 0;
  ayk_launch(ban_tokens_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, logits, rows, tokens, count, S, V);
  return ayk_check_launch("ayk_ban_tokens");
}

// out[S] int32.  temperature null or 0 for a row: greedy.  seed/offset int64 [S].
// top_k (int64, <= 0 off), top_p and min_p (float32) are null or [S].
AYK_EXPORT int ayk_sample(int* out, const float* logits, int S, int V, const float* temperature,
                          const long long* seed, const long long* offset, const long long* top_k,
                          const float* top_p, const float* min_p, cudaStream_t stream) {
  if (S == 0) return 0;
  AYK_REQUIRE(V >= 1, "ayk_sample: empty vocabulary");
  AYK_REQUIRE(temperature == nullptr || (seed != nullptr && offset != nullptr),
              "ayk_sample: temperature sampling needs seeds and offsets");
  ayk_launch(sample_kernel, dim3(S), dim3(THREADS), 0, stream, out, logits, V, temperature, seed, offset, top_k, top_p, min_p);
  return ayk_check_launch("ayk_sample");
}
