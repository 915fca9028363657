// Shared device/host helpers for the sm_100a kernel library.
//
// Every exported entry point is `extern "C"`, takes raw device pointers plus a
// `cudaStream_t`, launches asynchronously and returns a cudaError_t value (0 = ok).
// Nothing in the library allocates device memory: callers pass outputs and scratch.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define LLMB_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum { LLMB_F32 = 0, LLMB_BF16 = 1 };

// status codes written by kernels with bounded waits
enum { LLMB_OK = 0, LLMB_ERR_TIMEOUT = 1, LLMB_ERR_BAD_ARG = 2 };

// Checked build (-DLLMB_BOUNDS_CHECK, `python -m llm_mojo_b200.build --check` -> libllmb200_check.so): every index that comes
// out of DATA (token ids, target ids) is tested against its limit before it addresses memory; a bad index is recorded
// (first offender per translation unit: site, value, limit) and the access is skipped, so a corrupt batch shows up as a
// report instead of an illegal address.  In the normal build llmb_in_range() is `true` and compiles away.  The records
// are read with llmb_bounds_report_<file>(); the sites are listed there.
enum { LLMB_SITE_ENCODER_FWD_TOKEN = 1, LLMB_SITE_ENCODER_BWD_TOKEN = 2, LLMB_SITE_CLASSIFIER_TARGET = 3, LLMB_SITE_CE_TARGET = 4 };
#ifdef LLMB_BOUNDS_CHECK
static __device__ int llmb_bounds_rec[4];      // {seen, site, value, limit}
__device__ __forceinline__ bool llmb_in_range(long long v, long long limit, int site) {
  if (v >= 0 && v < limit) return true;
  if (atomicCAS(&llmb_bounds_rec[0], 0, 1) == 0) { llmb_bounds_rec[1] = site; llmb_bounds_rec[2] = (int)v; llmb_bounds_rec[3] = (int)limit; }
  return false;
}
#define LLMB_BOUNDS_REPORT_FN(name)                                                                      \
  LLMB_API int name(int* out4, int reset) {                                                              \
    int z[4] = {0, 0, 0, 0};                                                                             \
    cudaError_t e = cudaMemcpyFromSymbol(out4, llmb_bounds_rec, sizeof(z));                              \
    if (e == cudaSuccess && reset) e = cudaMemcpyToSymbol(llmb_bounds_rec, z, sizeof(z));                \
    return (int)e;                                                                                       \
  }
#else
__device__ __forceinline__ bool llmb_in_range(long long, long long, int) { return true; }
#define LLMB_BOUNDS_REPORT_FN(name)                                                                      \
  LLMB_API int name(int* out4, int reset) { (void)reset; out4[0] = out4[1] = out4[2] = out4[3] = 0; return 0; }
#endif

namespace llmb {

constexpr int WARP = 32;

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

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

// 16-byte vector of T
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// the value a float takes once it has been stored as T
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

// load/store 16 bytes worth of T as floats
template <typename T> struct Pack;
template <> struct Pack<float> {
  static constexpr int N = 4;
  float v[4];
  __device__ __forceinline__ void load(const float* p) { float4 t = *reinterpret_cast<const float4*>(p); v[0]=t.x; v[1]=t.y; v[2]=t.z; v[3]=t.w; }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  float v[8];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2*i] = f.x; v[2*i+1] = f.y; }
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint4 t; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2*i], v[2*i+1]);
    *reinterpret_cast<uint4*>(p) = t;
  }
};

// tanh-GELU (llmm/gelu.mojo:22-35) and its derivative
__device__ __forceinline__ float gelu_f(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  float u = k * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k = 0.7978845608028654f;
  float x2 = x * x;
  float u = k * (x + 0.044715f * x * x2);
  float t = tanhf(u);
  float sech2 = 1.0f - t * t;
  return 0.5f * (1.0f + t) + 0.5f * x * sech2 * k * (1.0f + 3.0f * 0.044715f * x2);
}

// single-instruction tanh (max abs error about 2^-11): enough for values that are rounded to bf16 next
__device__ __forceinline__ float tanh_fast(float x) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float gelu_fast_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.0f + tanh_fast(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_fast_f(float x) {
  const float k = 0.7978845608028654f;
  const float x2 = x * x;
  const float t = tanh_fast(k * (x + 0.044715f * x * x2));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * k * (1.0f + 3.0f * 0.044715f * x2);
}

// The same two functions on pairs, with packed fp32x2 arithmetic (half the FMA-pipe instructions per element; the two
// tanh stay scalar MUFU operations).  Used by the GEMM epilogues, whose eight warps, not the tensor core, bound the GELU layers.
__device__ __forceinline__ float2 gelu_fast2(float2 x) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const float2 x2 = __fmul2_rn(x, x);
  const float2 a = __fmul2_rn(x, __ffma2_rn(x2, make_float2(kc, kc), make_float2(k, k)));      // k (x + 0.044715 x^3)
  const float2 t = make_float2(tanh_fast(a.x), tanh_fast(a.y));
  const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
  return __ffma2_rn(h, t, h);                                                                   // 0.5 x (1 + t)
}
__device__ __forceinline__ float2 gelu_grad_fast2(float2 x) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const float2 half = make_float2(0.5f, 0.5f);
  const float2 x2 = __fmul2_rn(x, x);
  const float2 a = __fmul2_rn(x, __ffma2_rn(x2, make_float2(kc, kc), make_float2(k, k)));
  const float2 t = make_float2(tanh_fast(a.x), tanh_fast(a.y));
  const float2 s = __ffma2_rn(t, half, half);                                                   // 0.5 (1 + t)
  const float2 u = __ffma2_rn(__fmul2_rn(t, make_float2(-1.0f, -1.0f)), t, make_float2(1.0f, 1.0f));   // 1 - t^2
  const float2 d = __ffma2_rn(x2, make_float2(3.0f * kc, 3.0f * kc), make_float2(k, k));        // k (1 + 3 * 0.044715 x^2)
  return __ffma2_rn(__fmul2_rn(__fmul2_rn(x, half), d), u, s);
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); if (n <= 0) n = 148; }
  return n;
}

}  // namespace llmb
