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
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i];
    if (v > best.v) { best.v = v; best.i = i; }   // ascending i: the first maximum stays
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

__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int V,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const long long* __restrict__ offset) {
  __shared__ MaxIdx red[THREADS / 32];
  __shared__ double partial[THREADS];
  __shared__ int chosen_thread;
  __shared__ double chosen_base, target_s;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  MaxIdx top = block_argmax(row, V, red);
  float temp = temperature ? temperature[r] : 0.f;
  if (temp <= 0.f) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float inv_t = 1.0f / fmaxf(temp, 1e-6f);
  const float zmax = top.v * inv_t;
  // Each thread owns one contiguous segment, so that the running sum goes
  // through the tokens in id order.
  const int seg = (V + THREADS - 1) / THREADS;
  const int lo = min(V, (int)threadIdx.x * seg), hi = min(V, lo + seg);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) s += expf(row[i] * inv_t - zmax);
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
      float p = expf(row[i] * inv_t - zmax);
      if (p > 0.f) last_positive = i;
      run += (double)p;
      if (p > 0.f && run >= target_s) { token = i; break; }
    }
    out[r] = token >= 0 ? token : last_positive;
  }
}

}  // namespace

// out[S] int32.  temperature null or 0 for a row: greedy.  seed/offset int64 [S].
AYK_EXPORT int ayk_sample(int* out, const float* logits, int S, int V, const float* temperature,
                          const long long* seed, const long long* offset, cudaStream_t stream) {
  if (S == 0) return 0;
  AYK_REQUIRE(V >= 1, "ayk_sample: empty vocabulary");
  AYK_REQUIRE(temperature == nullptr || (seed != nullptr && offset != nullptr),
              "ayk_sample: temperature sampling needs seeds and offsets");
  sample_kernel<<<S, THREADS, 0, stream>>>(out, logits, V, temperature, seed, offset);
  return ayk_check_launch("ayk_sample");
}
