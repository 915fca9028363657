// AdamW with fp32 master weights (optionally stochastic-rounded bf16 store) and the global
// gradient-norm reduction.
//
// Reference behaviour: llmm/adamw.mojo:93-211 (m, v update, bias correction, decoupled weight
// decay on every tensor, grad pre-multiplied by grad_scale, SR store), llmm/global_norm.mojo:156-282
// (two-stage sum of squares), llmm/rng_device.mojo:113-236 (Squares counter RNG, SR cast).
#include "common.cuh"
using namespace llmb;

namespace {
// Squares: a counter-based RNG (Widynski 2020), 4 rounds, 32-bit output.
__device__ __forceinline__ uint32_t squares32(uint64_t ctr, uint64_t key) {
  uint64_t x = ctr * key, y = x, z = y + key;
  x = x * x + y; x = (x >> 32) | (x << 32);
  x = x * x + z; x = (x >> 32) | (x << 32);
  x = x * x + y; x = (x >> 32) | (x << 32);
  return (uint32_t)((x * x + z) >> 32);
}
__device__ __forceinline__ __nv_bfloat16 sr_cast_bf16(float v, uint32_t rnd) {
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(v);  // inf/nan
  bits += rnd & 0xffffu;
  return __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

template <typename TP>
__global__ void adamw_kernel(TP* __restrict__ params, float* __restrict__ master, const float* __restrict__ grads,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float beta1,
                             float beta2, float bc1, float bc2, float eps, float wd, float grad_scale,
                             const float* __restrict__ dev_scale, unsigned long long seed, int use_sr) {
  if (dev_scale) grad_scale *= *dev_scale;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = grads[i] * grad_scale;
    float mi = beta1 * m[i] + (1.f - beta1) * g;
    float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi; v[i] = vi;
    float mh = mi / bc1, vh = vi / bc2;
    float p = master ? master[i] : to_f<TP>(params[i]);
    p -= lr * (mh / (sqrtf(vh) + eps) + wd * p);
    if (master) master[i] = p;
    if (sizeof(TP) == 2 && use_sr) {
      reinterpret_cast<__nv_bfloat16*>(params)[i] = sr_cast_bf16(p, squares32((uint64_t)i, seed));
    } else {
      params[i] = from_f<TP>(p);
    }
  }
}

__global__ void norm_sq_partial_kernel(float* __restrict__ partial, const float* __restrict__ x, long long n) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float t = x[i]; s += t * t;
  }
  s = warp_sum(s);
  int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  if (lane == 0) red[wid] = s;
  __syncthreads();
  if (wid == 0) { float t = lane < blockDim.x / 32 ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) partial[blockIdx.x] = t; }
}
__global__ void norm_sq_final_kernel(float* __restrict__ out, const float* __restrict__ partial, int nblocks, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  if (lane == 0) red[wid] = s;
  __syncthreads();
  if (wid == 0) { float t = lane < blockDim.x / 32 ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) out[0] = accumulate ? out[0] + t : t; }
}
}  // namespace

LLMB_API int llmb_adamw(void* params, float* master, const float* grads, float* m, float* v, long long n, float lr,
                        float beta1, float beta2, float eps, float wd, float grad_scale, const float* dev_scale, int t,
                        unsigned long long seed, int use_sr, int param_dtype, cudaStream_t st) {
  if (n <= 0) return 0;
  float bc1 = 1.f - powf(beta1, (float)t), bc2 = 1.f - powf(beta2, (float)t);
  long long blocks = ceil_div_ll(n, 256 * 4);
  int grid = (int)(blocks < (long long)sm_count() * 16 ? blocks : (long long)sm_count() * 16);
  if (param_dtype == LLMB_BF16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, use_sr);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>((float*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, 0);
  return (int)cudaGetLastError();
}

LLMB_API int llmb_norm_sq_blocks() { return sm_count() * 4; }
// out[0] (=|+=) sum(x^2); scratch holds llmb_norm_sq_blocks() floats.
LLMB_API int llmb_global_norm_sq(float* out, const float* x, long long n, float* scratch, int accumulate, cudaStream_t st) {
  int grid = llmb_norm_sq_blocks();
  norm_sq_partial_kernel<<<grid, 512, 0, st>>>(scratch, x, n);
  norm_sq_final_kernel<<<1, 256, 0, st>>>(out, scratch, grid, accumulate);
  return (int)cudaGetLastError();
}

// fp32 -> bf16 with stochastic rounding (test hook for the RNG statistics tests)
__global__ void sr_cast_kernel(__nv_bfloat16* out, const float* in, long long n, unsigned long long seed) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = sr_cast_bf16(in[i], squares32((uint64_t)i, seed));
}
LLMB_API int llmb_sr_cast_bf16(void* out, const float* in, long long n, unsigned long long seed, cudaStream_t st) {
  sr_cast_kernel<<<sm_count() * 8, 256, 0, st>>>((__nv_bfloat16*)out, in, n, seed);
  return (int)cudaGetLastError();
}
