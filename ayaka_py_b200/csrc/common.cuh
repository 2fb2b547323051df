// Shared helpers of the sm_100a kernels: error reporting to the host, dtype
// tags, loads and stores that convert to and from float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define AYK_DTYPE_F32 0
#define AYK_DTYPE_BF16 1

#define AYK_ACT_NONE 0
#define AYK_ACT_GELU_ERF 1
#define AYK_ACT_GELU_TANH 2
#define AYK_ACT_QUICK_GELU 3

#define AYK_EXPORT extern "C" __attribute__((visibility("default")))

// Every entry point returns 0 or a negative code; the text is read back with
// ayk_last_error().
int ayk_fail(const char* fmt, ...);
int ayk_check_launch(const char* what);

#define AYK_REQUIRE(cond, ...)                 \
  do {                                         \
    if (!(cond)) return ayk_fail(__VA_ARGS__); \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float apply_activation(float x, int act) {
  // Formulas in 32-bit, as the reference's activation kernels compute them
  // (kernel/triton/activation.py:145-154).
  if (act == AYK_ACT_GELU_ERF) return x * 0.5f * (1.0f + erff(x * 0.7071067811865475f));
  if (act == AYK_ACT_GELU_TANH) {
    float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return x * 0.5f * (1.0f + tanhf(inner));
  }
  if (act == AYK_ACT_QUICK_GELU) return x / (1.0f + expf(-1.702f * x));
  return x;
}

// The same activations for the epilogues of the bfloat16 tensor-core products, where a
// row of the tile costs issue slots that the main loop cannot hide: tanh-GELU as
// x / (1 + 2^(-2 log2(e) u)), u = sqrt(2/pi) (x + 0.044715 x^3), with ex2.approx and a fast
// division (a few ulp in 32-bit, far inside a bfloat16 operand's rounding); the others as above.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int ACT>
__device__ __forceinline__ float apply_activation_tc(float x, int act) {
  if (ACT == AYK_ACT_NONE) return x;
  if (ACT == AYK_ACT_GELU_TANH) {
    const float x2 = x * x;
    const float t = x * fmaf(x2, -2.0f * 1.4426950408889634f * 0.7978845608028654f * 0.044715f,
                             -2.0f * 1.4426950408889634f * 0.7978845608028654f);
    return __fdividef(x, 1.0f + fast_exp2(t));
  }
  return apply_activation(x, act);
}

// Programmatic dependent launch: a kernel launched with the attribute may start
// while its predecessor in the stream still runs; it must not touch memory that
// the predecessor writes (or write memory that it reads) before pdl_wait().
// pdl_trigger() lets the successor be scheduled.  Without the attribute both
// are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

int ayk_pdl_enabled();
int ayk_sm_count();          // streaming multiprocessors of the current device

// "Has this kernel's launch attribute been set on the current device?"  Attributes of a kernel
// (dynamic shared memory, cluster size) belong to the device's copy of the kernel, so a flag per
// process would leave a second device unconfigured.  Returns a reference to the current device's flag.
struct AykPerDevice {
  bool done[64] = {};
  bool& here() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
    return done[device];
  }
};

template <typename... KArgs, typename... Args>
cudaError_t ayk_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ayk_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
