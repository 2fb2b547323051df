// C[M,N] = act(A[M,K] * W[N,K]^T + bias[N]) (+ residual[M,N]) on the FP32 FMA
// pipes: the matrix product of the true 32-bit path (no TF32, no tensor cores),
// also usable with bfloat16 operands.  The reference's linear layers are
// F.linear (layers/linear/methods.py:73-76); the activation formulas are those
// of kernel/triton/activation.py:145-154, applied in 32-bit in the epilogue.
//
// Tile 64x64x16, 256 threads, 4x4 outputs per thread; products are accumulated
// in ascending k in one float per output, so a row's result does not depend on
// which other rows are in the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 x = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&x.x);
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&x.y);
  v[0] = __bfloat162float(a.x); v[1] = __bfloat162float(a.y);
  v[2] = __bfloat162float(b.x); v[3] = __bfloat162float(b.y);
}

template <typename TA, typename TW, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TO* C, const TA* __restrict__ A, const TW* __restrict__ W,
                 const float* __restrict__ bias, const float* residual,      // C and residual may be one buffer (the residual stream in place)
                 int M, int N, int K, int act) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;       // loader: row of the tile, k offset
  const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;  // this thread's 4x4 outputs
  float acc[4][4] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
    if (VEC) {
      if (gm < M && gk < K) load4<TA>(A + (size_t)gm * K + gk, a);
      if (gn < N && gk < K) load4<TW>(W + (size_t)gn * K + gk, w);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (gm < M && gk + j < K) a[j] = to_float<TA>(A[(size_t)gm * K + gk + j]);
        if (gn < N && gk + j < K) w[j] = to_float<TW>(W[(size_t)gn * K + gk + j]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      As[lk + j][lr] = a[j];
      Ws[lk + j][lr] = w[j];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float4 av = *reinterpret_cast<const float4*>(&As[kk][tm]);
      float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tn]);
      float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j] + (bias ? bias[n] : 0.f);
      v = apply_activation(v, act);
      if (residual) v += residual[(size_t)m * N + n];
      C[(size_t)m * N + n] = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(void* C, const void* A, const void* W, const float* bias, const float* residual, int M,
           int N, int K, int act, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  bool vec = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
  if (vec)
    ayk_launch(gemm_simt_kernel<TA, TW, TO, true>, grid, dim3(256), 0, stream, (TO*)C, (const TA*)A, (const TW*)W, bias,
               residual, M, N, K, act);
  else
    ayk_launch(gemm_simt_kernel<TA, TW, TO, false>, grid, dim3(256), 0, stream, (TO*)C, (const TA*)A, (const TW*)W, bias,
               residual, M, N, K, act);
  return ayk_check_launch("ayk_gemm_simt");
}

}  // namespace

// in_dtype: dtype of A and W; out_dtype: dtype of C.  bias and residual are
// float32 or null; residual may alias C when out_dtype is float32.
AYK_EXPORT int ayk_gemm_simt(void* C, const void* A, const void* W, const float* bias,
                             const float* residual, int M, int N, int K, int act, int in_dtype,
                             int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  AYK_REQUIRE(K >= 1, "ayk_gemm_simt: K must be positive");
  AYK_REQUIRE((M + BM - 1) / BM <= 65535, "ayk_gemm_simt: M = %d exceeds %d rows", M, 65535 * BM);
  if (in_dtype == AYK_DTYPE_F32 && out_dtype == AYK_DTYPE_F32)
    return launch<float, float, float>(C, A, W, bias, residual, M, N, K, act, stream);
  if (in_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_F32)
    return launch<__nv_bfloat16, __nv_bfloat16, float>(C, A, W, bias, residual, M, N, K, act, stream);
  if (in_dtype == AYK_DTYPE_BF16 && out_dtype == AYK_DTYPE_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(C, A, W, bias, residual, M, N, K, act, stream);
  return ayk_fail("ayk_gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
