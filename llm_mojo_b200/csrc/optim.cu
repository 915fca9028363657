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
__device__ __forceinline__ float adamw_one(TP* params, float* master, float g, float& mi, float& vi, float pin, float lr, float beta1,
                                           float beta2, float bc1, float bc2, float eps, float wd) {
  mi = beta1 * mi + (1.f - beta1) * g;
  vi = beta2 * vi + (1.f - beta2) * g * g;
  const float mh = mi / bc1, vh = vi / bc2;
  return pin - lr * (mh / (sqrtf(vh) + eps) + wd * pin);
}

// VEC: four elements per thread and iteration through 16-byte accesses (8-byte for bf16 parameters); the scalar form takes
// what is left over and buffers whose addresses do not allow it.  The arithmetic per element is the same in both.
template <typename TP, bool VEC>
__global__ void adamw_kernel(TP* __restrict__ params, float* __restrict__ master, const float* __restrict__ grads,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float beta1,
                             float beta2, float bc1, float bc2, float eps, float wd, float grad_scale,
                             const float* __restrict__ dev_scale, unsigned long long seed, int use_sr) {
  if (dev_scale) grad_scale *= *dev_scale;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if (VEC) {
    const long long nv = n / 4;
    for (long long iv = tid; iv < nv; iv += stride) {
      const float4 g4 = *reinterpret_cast<const float4*>(grads + 4 * iv);
      float4 m4 = *reinterpret_cast<const float4*>(m + 4 * iv), v4 = *reinterpret_cast<const float4*>(v + 4 * iv);
      float pin[4];
      if (master) {
        const float4 p4 = *reinterpret_cast<const float4*>(master + 4 * iv);
        pin[0] = p4.x; pin[1] = p4.y; pin[2] = p4.z; pin[3] = p4.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) pin[k] = to_f<TP>(params[4 * iv + k]);
      }
      const float g[4] = {g4.x * grad_scale, g4.y * grad_scale, g4.z * grad_scale, g4.w * grad_scale};
      float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, po[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) po[k] = adamw_one<TP>(params, master, g[k], mm[k], vv[k], pin[k], lr, beta1, beta2, bc1, bc2, eps, wd);
      *reinterpret_cast<float4*>(m + 4 * iv) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + 4 * iv) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (master) *reinterpret_cast<float4*>(master + 4 * iv) = make_float4(po[0], po[1], po[2], po[3]);
      if (sizeof(TP) == 2) {
        __nv_bfloat16 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = use_sr ? sr_cast_bf16(po[k], squares32((uint64_t)(4 * iv + k), seed)) : __float2bfloat16(po[k]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params) + 4 * iv) = *reinterpret_cast<const uint2*>(o);
      } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(params) + 4 * iv) = make_float4(po[0], po[1], po[2], po[3]);
      }
    }
    done = nv * 4;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float mi = m[i], vi = v[i];
    const float pin = master ? master[i] : to_f<TP>(params[i]);
    const float p = adamw_one<TP>(params, master, grads[i] * grad_scale, mi, vi, pin, lr, beta1, beta2, bc1, bc2, eps, wd);
    m[i] = mi; v[i] = vi;
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
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {          // 16-byte loads where the address allows them
    const long long nv = n / 4;
    for (long long iv = tid; iv < nv; iv += stride) {
      const float4 t = *reinterpret_cast<const float4*>(x + 4 * iv);
      s += t.x * t.x; s += t.y * t.y; s += t.z * t.z; s += t.w * t.w;
    }
    done = nv * 4;
  }
  for (long long i = done + tid; i < n; i += stride) {
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
  const uintptr_t bits = reinterpret_cast<uintptr_t>(grads) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(master) | (reinterpret_cast<uintptr_t>(params) << (param_dtype == LLMB_BF16 ? 1 : 0));
  const bool vec = (bits & 15) == 0 && n >= 4;
  if (param_dtype == LLMB_BF16) {
    if (vec) adamw_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>((__nv_bfloat16*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, use_sr);
    else adamw_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>((__nv_bfloat16*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, use_sr);
  } else {
    if (vec) adamw_kernel<float, true><<<grid, 256, 0, st>>>((float*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, 0);
    else adamw_kernel<float, false><<<grid, 256, 0, st>>>((float*)params, master, grads, m, v, n, lr, beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, seed, 0);
  }
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
