// Low-precision training support: amax, delayed scaling, FP8 quantisation, NVFP4 quantisation
// (e2m1 values + e4m3 block scales + fp32 tensor scale, RNE or stochastic rounding, optional
// 16-point randomised Hadamard transform), and the Squares counter RNG.
//
// Reference behaviour: llmm/amax.mojo:129-302 (NaN-infectious amax), :336-398 (scale from the
// pre-push history, own amax during warm-up), llmm/lowp.mojo:539-853 (quantise with a device
// scale), llmm/nvfp4_quant.mojo:202-282 (e2m1 encode), :528-571 (tensor scale amax/(448*6)),
// :604-724 (block quantise), :400-410 (128x4 scale swizzle), llmm/hadamard.mojo:73-264,
// llmm/rng_device.mojo:113-232.
//
// B200 design: FP8 operands feed tcgen05 kind::f8f6f4 GEMMs directly in whatever majorness the
// trainer stores them (no transposed copies: the UMMA descriptor handles MN-major e4m3/e5m2).
// The NVFP4 kernels emit the packed format (bytes + scales in the 128 x 4 atoms that the block-scaled
// tensor path reads, the operands of llmb_gemm_nvfp4) and, on request, the dequantised value x
// block-scale in bf16: every e2m1 x e4m3 product is exactly representable in bf16, so a bf16
// tensor-core GEMM over those values with the fp32 tensor scales folded into alpha reproduces
// the NVFP4 GEMM's arithmetic (the emulation the native kernel is tested against).  Rounding uses
// the hardware converts (cvt.rn / cvt.rs to e2m1).  llmb_fp8_block_quant does the same for FP8 with
// per-128 power-of-two scales (fp8 bytes + ue8m0 scale atoms, the operands of llmb_gemm_mxfp8).
#include "common.cuh"
#include <cuda_fp8.h>
#include <cuda_fp4.h>
using namespace llmb;

namespace {
// ------------------------------------------------------------------ Squares RNG
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ uint64_t rng_key(uint64_t seed, uint64_t stream) { return splitmix64(seed ^ splitmix64(stream)) | 1ull; }
__device__ __forceinline__ uint32_t squares32(uint64_t ctr, uint64_t key) {
  uint64_t x = ctr * key, y = x, z = y + key;
  x = x * x + y; x = (x >> 32) | (x << 32);
  x = x * x + z; x = (x >> 32) | (x << 32);
  x = x * x + y; x = (x >> 32) | (x << 32);
  return (uint32_t)((x * x + z) >> 32);
}
// The 64-bit output variant (one more round): eight values' worth of random bits for the stochastic-rounding converts.
__device__ __forceinline__ uint64_t squares64(uint64_t ctr, uint64_t key) {
  uint64_t x = ctr * key, y = x, z = y + key;
  x = x * x + y; x = (x >> 32) | (x << 32);
  x = x * x + z; x = (x >> 32) | (x << 32);
  x = x * x + y; x = (x >> 32) | (x << 32);
  x = x * x + z; const uint64_t t = x; x = (x >> 32) | (x << 32);
  return t ^ ((x * x + y) >> 32);
}
__device__ __forceinline__ float rng_uniform01(uint64_t seed, uint64_t ctr, uint64_t stream) {
  return (float)(squares32(ctr, rng_key(seed, stream)) >> 8) * (1.0f / 16777216.0f);
}
// ------------------------------------------------------------------ amax
template <typename T>
__global__ void amax_kernel(unsigned* __restrict__ out_bits, const T* __restrict__ x, long long n) {
  // |x| as raw bits orders like an unsigned integer and NaN patterns sort above +inf, so an
  // integer max is a NaN-infectious float max.
  constexpr int N = Pack<T>::N;
  unsigned m = 0;
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    Pack<T> p; p.load(x + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) m = max(m, __float_as_uint(p.v[k]) & 0x7fffffffu);
  }
  if (blockIdx.x == 0) for (long long i = nvec * N + threadIdx.x; i < n; i += blockDim.x) m = max(m, __float_as_uint(to_f<T>(x[i])) & 0x7fffffffu);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ unsigned red[32];
  const int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  if (lane == 0) red[wid] = m;
  __syncthreads();
  if (wid == 0) {
    m = lane < (int)(blockDim.x / 32) ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) atomicMax(out_bits, m);
  }
}

// state layout (floats): [0] scale  [1] scale_inv  [2] step counter (as float bits of int)  [3] pad  [4..4+H) history
constexpr int AMAX_HISTORY = 16;
__global__ void amax_update_kernel(float* state, const float* amax_cur, float fmt_max, float margin_mult) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int step = __float_as_int(state[2]);
  float* hist = state + 4;
  const float cur = *amax_cur;
  float a;
  if (step < AMAX_HISTORY) a = cur;
  else {
    float m = 0.f; bool bad = false;
    for (int i = 0; i < AMAX_HISTORY; ++i) { float h = hist[i]; if (isnan(h) || isinf(h)) bad = true; else m = fmaxf(m, h); }
    a = bad ? NAN : m;
  }
  float scale = (a <= 0.f || isnan(a) || isinf(a)) ? 1.0f : (fmt_max * margin_mult) / a;
  state[0] = scale; state[1] = 1.0f / scale;
  hist[step % AMAX_HISTORY] = cur;           // pushed after the scale was derived: a step never sees its own amax
  state[2] = __int_as_float(step + 1);
}

// ------------------------------------------------------------------ FP8 quantise (device scale)
template <typename T, int FMT>
__global__ void quantize_fp8_kernel(uint8_t* __restrict__ out, const T* __restrict__ x, const float* __restrict__ scale_ptr, long long n) {
  constexpr int N = Pack<T>::N;
  const float s = *scale_ptr;
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    Pack<T> p; p.load(x + i * N);
    uint8_t q[N];
#pragma unroll
    for (int k = 0; k < N; ++k)
      q[k] = (uint8_t)__nv_cvt_float_to_fp8(p.v[k] * s, __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
    if (N == 8) *reinterpret_cast<uint2*>(out + i * N) = *reinterpret_cast<uint2*>(q);
    else *reinterpret_cast<uint32_t*>(out + i * N) = *reinterpret_cast<uint32_t*>(q);
  }
}
__global__ void dequantize_fp8_kernel(float* __restrict__ out, const uint8_t* __restrict__ q, const float* __restrict__ scale_inv, long long n, int fmt) {
  const float s = *scale_inv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(q[i], fmt == 0 ? __NV_E4M3 : __NV_E5M2);
    out[i] = __half2float(*reinterpret_cast<__half*>(&h)) * s;
  }
}

// ------------------------------------------------------------------ NVFP4
// magnitude of a 3-bit e2m1 index {0, 0.5, 1, 1.5, 2, 3, 4, 6}, built from its exponent / mantissa bits (no table:
// a dynamically indexed local array would live in local memory and cost a load per element)
__device__ __forceinline__ float e2m1_value(int code) {
  const unsigned e = (code >> 1) & 3u, m = code & 1u;
  const unsigned bits = e ? (((126u + e) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
  return __uint_as_float(bits);
}
// Two values to e2m1 by the hardware convert (round to nearest, ties to even, saturating): lo in the low nibble.
__device__ __forceinline__ uint32_t e2m1x2_rn(float lo, float hi) {
  return (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}
// Four values to e2m1 with stochastic rounding by the hardware convert: it adds random bits below the kept mantissa
// bit and truncates, P(up) = distance to the lower neighbour / spacing; `rbits` are 32 uniform bits, a disjoint
// field per value.  v0 lands in the lowest nibble of the 16-bit result (the instruction packs its first operand highest).
__device__ __forceinline__ uint32_t e2m1x4_rs(float v0, float v1, float v2, float v3, uint32_t rbits) {
  uint16_t q;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(q) : "f"(v3), "f"(v2), "f"(v1), "f"(v0), "r"(rbits));
  return (uint32_t)q;
}
__device__ __forceinline__ uint8_t encode_e4m3(float v) { return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ float decode_e4m3(uint8_t c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// offset of block scale (row r, k-block kb) in the 128-row x 4-column tiled scale layout
__device__ __host__ inline long long nvfp4_scale_swizzle_offset(long long r, long long kb, long long n_col_tiles) {
  const long long tile_r = r / 128, tile_c = kb / 4;
  const long long in_r = r % 128, in_c = kb % 4;
  return (tile_r * n_col_tiles + tile_c) * 512 + (in_r % 32) * 16 + (in_r / 32) * 4 + in_c;
}
__device__ __forceinline__ float hadamard_sign(int i) {
  // fixed sign vector of the randomised Hadamard transform
  return ((0x9686 >> i) & 1) ? 1.0f : -1.0f;   // bit i set <=> +1: [-1,1,1,-1,-1,-1,-1,1,-1,1,1,-1,1,-1,-1,1]
}
__device__ __forceinline__ void fwht16(float (&b)[16]) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; i += 2 * h) {
#pragma unroll
      for (int j = i; j < i + h; ++j) { const float x = b[j], y = b[j + h]; b[j] = x + y; b[j + h] = x - y; }
    }
  }
}

// 16 consecutive bf16 values <-> 16 floats through two 16-byte accesses (the address must be 32-byte aligned)
__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
  const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(ha[i]), fb = __bfloat1622float2(hb[i]);
    v[2 * i] = fa.x; v[2 * i + 1] = fa.y; v[8 + 2 * i] = fb.x; v[8 + 2 * i + 1] = fb.y;
  }
}
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* p, const float (&v)[16]) {
  uint4 a, b;
  __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
  __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) { ha[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); hb[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]); }
  *reinterpret_cast<uint4*>(p) = a; *reinterpret_cast<uint4*>(p + 8) = b;
}

// One thread quantises one block: BLOCK_ROWS x 16 elements along the block axis.
//   axis 1: blocks run along the columns (K = last dim); axis 0: blocks run along the rows.
// Outputs (each optional): packed e2m1 (logical [outer, K/2] with K the block axis), e4m3 scales
// (swizzled 128x4 tiles, or row-major when n_col_tiles == 0), and dequantised bf16 = value x
// block scale (WITHOUT the fp32 tensor scale) in the source layout.
template <typename T, int BLOCK_ROWS>
__global__ void nvfp4_quantize_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ deq,
                                      const T* __restrict__ x, const float* __restrict__ tensor_scale_ptr, int rows, int cols,
                                      int axis, int rht, int sr, unsigned long long seed, unsigned long long stream,
                                      long long step, long long n_col_tiles) {
  const int outer = axis == 1 ? rows : cols;            // index across blocks' "rows"
  const int K = axis == 1 ? cols : rows;                // length along the block axis
  const int kblocks = K / 16;
  const int tile_rows = ceil_div(outer, BLOCK_ROWS);
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)tile_rows * kblocks) return;
  // consecutive threads walk the contiguous memory direction
  int br, kb;
  if (axis == 1) { br = (int)(idx / kblocks); kb = (int)(idx % kblocks); }
  else { kb = (int)(idx / tile_rows); br = (int)(idx % tile_rows); }
  const float ts = *tensor_scale_ptr;
  auto addr = [&](int o, int k) -> long long { return axis == 1 ? (long long)o * cols + k : (long long)k * cols + o; };

  float v[BLOCK_ROWS][16];
  float amax = 0.f;
  // Vector I/O whenever 16 consecutive elements of the block are contiguous in memory: along the block axis for
  // axis 1, across the 16 "outer" lines of a 16x16 block for axis 0 (bf16 storage, whole blocks, 32-byte aligned).
  constexpr bool kBf16 = sizeof(T) == 2;
  const bool vec_a = kBf16 && axis == 1 && (cols % 16) == 0 && (br + 1) * BLOCK_ROWS <= outer;
  const bool vec_b = false;                               // (16 x 16 blocks along axis 0 take the cooperative kernel)
  if (vec_b) {
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float t[16];
      load16_bf16(reinterpret_cast<const __nv_bfloat16*>(x) + (long long)(kb * 16 + kk) * cols + br * BLOCK_ROWS, t);
#pragma unroll
      for (int rr = 0; rr < BLOCK_ROWS; ++rr) v[rr][kk] = t[rr & 15];
    }
  }
#pragma unroll
  for (int rr = 0; rr < BLOCK_ROWS; ++rr) {
    const int o = br * BLOCK_ROWS + rr;
    if (vec_a) load16_bf16(reinterpret_cast<const __nv_bfloat16*>(x) + (long long)o * cols + kb * 16, v[rr]);
    else if (!vec_b) {
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) v[rr][kk] = o < outer ? to_f<T>(x[addr(o, kb * 16 + kk)]) : 0.f;
    }
    if (rht) {
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) v[rr][kk] *= hadamard_sign(kk);
      fwht16(v[rr]);
    }
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) amax = fmaxf(amax, fabsf(v[rr][kk]));
  }
  const float raw = (amax <= 0.f || ts <= 0.f) ? 1.0f : (amax / 6.0f) / ts;
  const uint8_t sc_code = encode_e4m3(raw);
  const float sc_dec = decode_e4m3(sc_code);
  float sc_val = sc_dec * ts;
  if (sc_val <= 0.f) sc_val = 1.0f;
  const float inv = 1.0f / sc_val;
  const uint64_t key = sr ? rng_key(seed, stream) : 0ull;
#pragma unroll
  for (int rr = 0; rr < BLOCK_ROWS; ++rr) {
    const int o = br * BLOCK_ROWS + rr;
    if (o >= outer) continue;
    if (scales) scales[n_col_tiles > 0 ? nvfp4_scale_swizzle_offset(o, kb, n_col_tiles) : (long long)o * kblocks + kb] = sc_code;
    uint8_t packed[8];
    uint64_t rbits = 0;
#pragma unroll
    for (int kk = 0; kk < 16; kk += 4) {
      const float s0 = v[rr][kk] * inv, s1 = v[rr][kk + 1] * inv, s2 = v[rr][kk + 2] * inv, s3 = v[rr][kk + 3] * inv;
      uint32_t code4;                                     // four codes, value kk in the lowest nibble
      if (sr) {                                           // one 64-bit draw per eight values, counted at the first of them
        if ((kk & 4) == 0) rbits = squares64(((unsigned long long)step << 32) | ((unsigned long long)o * K + kb * 16 + kk), key);
        code4 = e2m1x4_rs(s0, s1, s2, s3, (uint32_t)(rbits >> ((kk & 4) * 8)));
      } else code4 = e2m1x2_rn(s0, s1) | (e2m1x2_rn(s2, s3) << 8);
      packed[kk / 2] = (uint8_t)code4; packed[kk / 2 + 1] = (uint8_t)(code4 >> 8);
      if (deq) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int c = (code4 >> (4 * t)) & 15;
          const float dq = (c & 8 ? -1.f : 1.f) * e2m1_value(c) * sc_dec;
          if (vec_a || vec_b) v[rr][kk + t] = dq;           // written out as vectors below
          else deq[addr(o, kb * 16 + kk + t)] = __float2bfloat16_rn(dq);
        }
      }
    }
    if (q) *reinterpret_cast<uint2*>(q + ((long long)o * K + kb * 16) / 2) = *reinterpret_cast<uint2*>(packed);
    if (vec_a && deq) store16_bf16(deq + (long long)o * cols + kb * 16, v[rr]);
  }
  if (vec_b && deq) {
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float t[16];
#pragma unroll
      for (int rr = 0; rr < BLOCK_ROWS; ++rr) t[rr & 15] = v[rr][kk];
      store16_bf16(deq + (long long)(kb * 16 + kk) * cols + br * BLOCK_ROWS, t);
    }
  }
}

// 16 x 16 blocks of bf16 storage: sixteen lanes share one block, each taking the 16 values of the block that are
// contiguous in memory (a row of 16 k for axis 1, a k-row of 16 outer lines for axis 0).  The block amax is a
// half-warp shuffle reduction, all memory traffic is two 16-byte accesses per lane each way, and nobody holds 256
// values in registers.  Same rounding, scale encoding and RNG counters as the one-thread-per-block kernel.
__global__ void __launch_bounds__(256) nvfp4_quantize16_coop_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ scales,
                                                                   __nv_bfloat16* __restrict__ deq, const __nv_bfloat16* __restrict__ x,
                                                                   const float* __restrict__ tensor_scale_ptr, int rows, int cols, int axis,
                                                                   int sr, unsigned long long seed, unsigned long long stream, long long step,
                                                                   long long n_col_tiles) {
  const int outer = axis == 1 ? rows : cols, K = axis == 1 ? cols : rows;
  const int kblocks = K / 16, tile_rows = outer / 16;
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / 16;       // block index (half-warp uniform)
  const int l = threadIdx.x & 15;
  if (gid >= (long long)tile_rows * kblocks) return;
  int br, kb;
  if (axis == 1) { br = (int)(gid / kblocks); kb = (int)(gid % kblocks); }
  else { kb = (int)(gid / tile_rows); br = (int)(gid % tile_rows); }
  // the 16 contiguous values of this lane: axis 1 -> (o = br*16 + l, k = kb*16 + 0..15); axis 0 -> (o = br*16 + 0..15, k = kb*16 + l)
  const long long base = axis == 1 ? (long long)(br * 16 + l) * cols + kb * 16 : (long long)(kb * 16 + l) * cols + br * 16;
  float v[16];
  load16_bf16(x + base, v);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 16));
  const float ts = *tensor_scale_ptr;
  const float raw = (amax <= 0.f || ts <= 0.f) ? 1.0f : (amax / 6.0f) / ts;
  const uint8_t sc_code = encode_e4m3(raw);
  const float sc_dec = decode_e4m3(sc_code);
  float sc_val = sc_dec * ts;
  if (sc_val <= 0.f) sc_val = 1.0f;
  const float inv = 1.0f / sc_val;
  const uint64_t key = sr ? rng_key(seed, stream) : 0ull;
  if (scales) {                                            // one scale per (outer line, k-block): lane l writes line br*16 + l
    const int o = br * 16 + l;
    scales[n_col_tiles > 0 ? nvfp4_scale_swizzle_offset(o, kb, n_col_tiles) : (long long)o * kblocks + kb] = sc_code;
  }
  uint8_t packed[8];
  uint64_t rbits = 0;
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float s0 = v[i] * inv, s1 = v[i + 1] * inv, s2 = v[i + 2] * inv, s3 = v[i + 3] * inv;
    uint32_t code4;
    if (sr) {                                             // one 64-bit draw per eight values, counted at the first of them
      if ((i & 4) == 0) {
        const int o = axis == 1 ? br * 16 + l : br * 16 + i;
        const int k = axis == 1 ? kb * 16 + i : kb * 16 + l;
        rbits = squares64(((unsigned long long)step << 32) | ((unsigned long long)o * K + k), key);
      }
      code4 = e2m1x4_rs(s0, s1, s2, s3, (uint32_t)(rbits >> ((i & 4) * 8)));
    } else code4 = e2m1x2_rn(s0, s1) | (e2m1x2_rn(s2, s3) << 8);
    packed[i / 2] = (uint8_t)code4; packed[i / 2 + 1] = (uint8_t)(code4 >> 8);
    if (deq) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int c = (code4 >> (4 * t)) & 15;
        v[i + t] = (c & 8 ? -1.f : 1.f) * e2m1_value(c) * sc_dec;
      }
    }
  }
  if (q) {
    uint2 mine = *reinterpret_cast<uint2*>(packed);
    if (axis == 0) {
      // this lane holds one k of sixteen outer lines; the packed row of outer line br*16 + l wants the sixteen k of that
      // line: a 16 x 16 nibble transpose across the half-warp (nibble l of lane s becomes nibble s of lane l)
      uint2 t = make_uint2(0u, 0u);
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        const uint32_t wlo = __shfl_sync(0xffffffffu, mine.x, s, 16), whi = __shfl_sync(0xffffffffu, mine.y, s, 16);
        const uint32_t nib = ((l < 8 ? wlo : whi) >> ((l & 7) * 4)) & 15u;
        if (s < 8) t.x |= nib << (s * 4); else t.y |= nib << ((s - 8) * 4);
      }
      mine = t;
    }
    *reinterpret_cast<uint2*>(q + ((long long)(br * 16 + l) * K + kb * 16) / 2) = mine;
  }
  if (deq) store16_bf16(deq + base, v);
}

__global__ void nvfp4_tensor_scale_kernel(float* ts, const float* amax) {
  const float a = *amax;
  *ts = (a > 0.f && !isnan(a) && !isinf(a)) ? a / (448.0f * 6.0f) : 1.0f;
}
__global__ void nvfp4_dequant_kernel(float* __restrict__ out, const uint8_t* __restrict__ q, const uint8_t* __restrict__ scales,
                                     const float* __restrict__ ts, int rows, int K, long long n_col_tiles) {
  const long long n = (long long)rows * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / K), k = (int)(i % K);
    const uint8_t byte = q[i / 2];
    const int code = (i & 1) ? (byte >> 4) : (byte & 15);
    const uint8_t sc = scales[n_col_tiles > 0 ? nvfp4_scale_swizzle_offset(r, k / 16, n_col_tiles) : (long long)r * (K / 16) + k / 16];
    out[i] = (code & 8 ? -1.f : 1.f) * e2m1_value(code) * decode_e4m3(sc) * (*ts);
  }
}

template <typename T>
__global__ void hadamard16_kernel(T* __restrict__ out, const T* __restrict__ x, long long nblocks, int inverse) {
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = to_f<T>(x[b * 16 + i]) * (inverse ? 1.0f : hadamard_sign(i));
    fwht16(v);
#pragma unroll
    for (int i = 0; i < 16; ++i) out[b * 16 + i] = from_f<T>(inverse ? v[i] * hadamard_sign(i) * (1.0f / 16.0f) : v[i]);
  }
}

__global__ void rng_uniform_kernel(float* out, long long n, unsigned long long seed, unsigned long long stream, unsigned long long base) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = rng_uniform01(seed, base + i, stream);
}

// Delayed scaling after the warm-up: the scale of this step comes from the history BEFORE this step's amax is pushed, so the
// tensor needs to be read only once - quantise with the scale that `amax_scale_from_history_kernel` has just derived, take max|x|
// on the way (same NaN-infectious integer max as amax_kernel), and let `amax_push_kernel` append it to the history afterwards.
__global__ void amax_scale_from_history_kernel(float* state, unsigned* amax_bits, float fmt_max, float margin_mult) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const float* hist = state + 4;
  float m = 0.f; bool bad = false;
  for (int i = 0; i < AMAX_HISTORY; ++i) { float h = hist[i]; if (isnan(h) || isinf(h)) bad = true; else m = fmaxf(m, h); }
  const float a = bad ? NAN : m;
  const float scale = (a <= 0.f || isnan(a) || isinf(a)) ? 1.0f : (fmt_max * margin_mult) / a;
  state[0] = scale; state[1] = 1.0f / scale;
  *amax_bits = 0u;
}
__global__ void amax_push_kernel(float* state, const float* amax_cur) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int step = __float_as_int(state[2]);
  state[4 + step % AMAX_HISTORY] = *amax_cur;
  state[2] = __int_as_float(step + 1);
}
template <typename T, int FMT>
__global__ void __launch_bounds__(512) quantize_fp8_amax_kernel(uint8_t* __restrict__ out, unsigned* __restrict__ amax_bits, const T* __restrict__ x,
                                                               const float* __restrict__ scale_ptr, long long n) {
  constexpr int N = Pack<T>::N;
  const float s = *scale_ptr;
  unsigned m = 0;
  const long long nvec = n / N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    Pack<T> p; p.load(x + i * N);
    uint8_t q[N];
#pragma unroll
    for (int k = 0; k < N; ++k) {
      m = max(m, __float_as_uint(p.v[k]) & 0x7fffffffu);
      q[k] = (uint8_t)__nv_cvt_float_to_fp8(p.v[k] * s, __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
    }
    if (N == 8) *reinterpret_cast<uint2*>(out + i * N) = *reinterpret_cast<uint2*>(q);
    else *reinterpret_cast<uint32_t*>(out + i * N) = *reinterpret_cast<uint32_t*>(q);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ unsigned red[32];
  const int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  if (lane == 0) red[wid] = m;
  __syncthreads();
  if (wid == 0) {
    m = lane < (int)(blockDim.x / 32) ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) atomicMax(amax_bits, m);
  }
}
}  // namespace

// The same three steps for the operands of one linear layer with two tiny launches instead of two per operand plus the
// host-side products of the inverse scales: `llmb_fp8_prepare` derives the scales of up to two states from their histories,
// clears their amax words and writes up to two GEMM scale factors (products of inverse scales of states that are final by
// then); `llmb_quantize_fp8_amax` is the pass over a tensor; `llmb_fp8_push` appends the amax words to the histories.
namespace {
__device__ void derive_scale(float* state, unsigned* amax_bits, float fmt_max, float margin_mult) {
  const float* hist = state + 4;
  float m = 0.f; bool bad = false;
  for (int i = 0; i < AMAX_HISTORY; ++i) { float h = hist[i]; if (isnan(h) || isinf(h)) bad = true; else m = fmaxf(m, h); }
  const float a = bad ? NAN : m;
  const float scale = (a <= 0.f || isnan(a) || isinf(a)) ? 1.0f : (fmt_max * margin_mult) / a;
  state[0] = scale; state[1] = 1.0f / scale;
  *amax_bits = 0u;
}
__global__ void fp8_prepare_kernel(float* sa, unsigned* aa, float fa, float ma, float* sb, unsigned* ab, float fb, float mb,
                                   float* alpha1, const float* p1, const float* q1, float* alpha2, const float* p2, const float* q2) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (sa) derive_scale(sa, aa, fa, ma);
  if (sb) derive_scale(sb, ab, fb, mb);
  if (alpha1) *alpha1 = p1[1] * q1[1];
  if (alpha2) *alpha2 = p2[1] * q2[1];
}
__global__ void fp8_push_kernel(float* sa, const float* aa, float* sb, const float* ab) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (sa) { const int step = __float_as_int(sa[2]); sa[4 + step % AMAX_HISTORY] = *aa; sa[2] = __int_as_float(step + 1); }
  if (sb) { const int step = __float_as_int(sb[2]); sb[4 + step % AMAX_HISTORY] = *ab; sb[2] = __int_as_float(step + 1); }
}
}  // namespace
LLMB_API int llmb_fp8_prepare(float* sa, float* aa, float fa, float ma, float* sb, float* ab, float fb, float mb, float* alpha1,
                              const float* p1, const float* q1, float* alpha2, const float* p2, const float* q2, cudaStream_t st) {
  fp8_prepare_kernel<<<1, 32, 0, st>>>(sa, (unsigned*)aa, fa, ma, sb, (unsigned*)ab, fb, mb, alpha1, p1, q1, alpha2, p2, q2);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_fp8_push(float* sa, const float* aa, float* sb, const float* ab, cudaStream_t st) {
  fp8_push_kernel<<<1, 32, 0, st>>>(sa, aa, sb, ab);
  return (int)cudaGetLastError();
}
// out = fp8(x * state[0]) saturated and amax[0] = max(amax[0], max|x|) as raw bits (clear it first); n a multiple of the vector width
LLMB_API int llmb_quantize_fp8_amax(void* out, const void* x, const float* state, float* amax, long long n, int fmt, int dtype,
                                    cudaStream_t st) {
  if (n % (dtype == LLMB_BF16 ? 8 : 4)) return LLMB_ERR_BAD_ARG;
  long long blocks = ceil_div_ll(n, 512 * 8);
  int grid = (int)(blocks < (long long)sm_count() * 4 ? (blocks < 1 ? 1 : blocks) : (long long)sm_count() * 4);
  if (dtype == LLMB_BF16) {
    if (fmt == 0) quantize_fp8_amax_kernel<__nv_bfloat16, 0><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const __nv_bfloat16*)x, state, n);
    else quantize_fp8_amax_kernel<__nv_bfloat16, 1><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const __nv_bfloat16*)x, state, n);
  } else {
    if (fmt == 0) quantize_fp8_amax_kernel<float, 0><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const float*)x, state, n);
    else quantize_fp8_amax_kernel<float, 1><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const float*)x, state, n);
  }
  return (int)cudaGetLastError();
}

// One pass over x for a delayed-scaling operand whose history is full (the caller checks that: state[2] >= the history
// length): state[0..1] = scale / 1/scale from the history, out = fp8(x * scale) saturated, amax[0] = max|x| (NaN-infectious),
// then the amax is appended to the history.  n must be a multiple of the vector width (8 for bf16, 4 for fp32).
LLMB_API int llmb_quantize_fp8_delayed(void* out, const void* x, float* state, float* amax, long long n, int fmt, float fmt_max,
                                       float margin_mult, int dtype, cudaStream_t st) {
  if (n % (dtype == LLMB_BF16 ? 8 : 4)) return LLMB_ERR_BAD_ARG;
  amax_scale_from_history_kernel<<<1, 32, 0, st>>>(state, (unsigned*)amax, fmt_max, margin_mult);
  long long blocks = ceil_div_ll(n, 512 * 8);
  int grid = (int)(blocks < (long long)sm_count() * 4 ? (blocks < 1 ? 1 : blocks) : (long long)sm_count() * 4);
  if (dtype == LLMB_BF16) {
    if (fmt == 0) quantize_fp8_amax_kernel<__nv_bfloat16, 0><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const __nv_bfloat16*)x, state, n);
    else quantize_fp8_amax_kernel<__nv_bfloat16, 1><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const __nv_bfloat16*)x, state, n);
  } else {
    if (fmt == 0) quantize_fp8_amax_kernel<float, 0><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const float*)x, state, n);
    else quantize_fp8_amax_kernel<float, 1><<<grid, 512, 0, st>>>((uint8_t*)out, (unsigned*)amax, (const float*)x, state, n);
  }
  amax_push_kernel<<<1, 32, 0, st>>>(state, amax);
  return (int)cudaGetLastError();
}

// out (1 float, device) = max |x|, NaN if any element is NaN
LLMB_API int llmb_amax(float* out, const void* x, long long n, int dtype, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float), st);
  if (e != cudaSuccess) return (int)e;
  long long blocks = ceil_div_ll(n, 512 * 8);
  int grid = (int)(blocks < (long long)sm_count() * 4 ? (blocks < 1 ? 1 : blocks) : (long long)sm_count() * 4);
  if (dtype == LLMB_BF16) amax_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>((unsigned*)out, (const __nv_bfloat16*)x, n);
  else amax_kernel<float><<<grid, 512, 0, st>>>((unsigned*)out, (const float*)x, n);
  return (int)cudaGetLastError();
}
// amax of the 16-point randomised Hadamard transform of x taken along `axis` (blocks of 16 consecutive columns
// for axis 1, of 16 consecutive rows for axis 0), without materialising the transform: one thread per block.
namespace {
template <typename T>
__global__ void amax_rht_kernel(unsigned* __restrict__ out_bits, const T* __restrict__ x, int rows, int cols, int axis) {
  unsigned m = 0;
  const long long nblocks = (long long)rows * cols / 16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nblocks; i += (long long)gridDim.x * blockDim.x) {
    float v[16];
    if (axis == 1) {
      const T* p = x + i * 16;
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = to_f<T>(p[k]) * hadamard_sign(k);
    } else {                                   // adjacent threads take adjacent columns of the same 16 rows: coalesced
      const long long rb = i / cols; const int c = (int)(i % cols);
      const T* p = x + rb * 16 * cols + c;
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = to_f<T>(p[(long long)k * cols]) * hadamard_sign(k);
    }
    fwht16(v);
#pragma unroll
    for (int k = 0; k < 16; ++k) m = max(m, __float_as_uint(v[k]) & 0x7fffffffu);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ unsigned red[32];
  const int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  if (lane == 0) red[wid] = m;
  __syncthreads();
  if (wid == 0) {
    m = lane < (int)(blockDim.x / 32) ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) atomicMax(out_bits, m);
  }
}
}  // namespace
// rows (axis 0) or cols (axis 1) must be a multiple of 16
LLMB_API int llmb_amax_rht(float* out, const void* x, int rows, int cols, int axis, int dtype, cudaStream_t st) {
  if ((axis == 1 ? cols : rows) % 16) return LLMB_ERR_BAD_ARG;
  cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float), st);
  if (e != cudaSuccess) return (int)e;
  const long long nblocks = (long long)rows * cols / 16;
  long long want = (nblocks + 255) / 256;
  const int grid = (int)(want < 8LL * sm_count() ? (want < 1 ? 1 : want) : 8LL * sm_count());
  if (dtype == LLMB_BF16) amax_rht_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((unsigned*)out, (const __nv_bfloat16*)x, rows, cols, axis);
  else amax_rht_kernel<float><<<grid, 256, 0, st>>>((unsigned*)out, (const float*)x, rows, cols, axis);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_amax_state_floats() { return 4 + AMAX_HISTORY; }
// state: llmb_amax_state_floats() floats, initialised to {1, 1, 0, 0, 0...}; fmt_max 448 (e4m3) / 57344 (e5m2)
LLMB_API int llmb_amax_update(float* state, const float* amax_cur, float fmt_max, float margin_mult, cudaStream_t st) {
  amax_update_kernel<<<1, 32, 0, st>>>(state, amax_cur, fmt_max, margin_mult);
  return (int)cudaGetLastError();
}
// out[i] = fp8(x[i] * *scale); fmt 0 = e4m3, 1 = e5m2
LLMB_API int llmb_quantize_fp8(void* out, const void* x, const float* scale, long long n, int fmt, int dtype, cudaStream_t st) {
  int grid = sm_count() * 8;
  if (dtype == LLMB_BF16) {
    if (n % 8) return LLMB_ERR_BAD_ARG;
    if (fmt == 0) quantize_fp8_kernel<__nv_bfloat16, 0><<<grid, 256, 0, st>>>((uint8_t*)out, (const __nv_bfloat16*)x, scale, n);
    else quantize_fp8_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>((uint8_t*)out, (const __nv_bfloat16*)x, scale, n);
  } else {
    if (n % 4) return LLMB_ERR_BAD_ARG;
    if (fmt == 0) quantize_fp8_kernel<float, 0><<<grid, 256, 0, st>>>((uint8_t*)out, (const float*)x, scale, n);
    else quantize_fp8_kernel<float, 1><<<grid, 256, 0, st>>>((uint8_t*)out, (const float*)x, scale, n);
  }
  return (int)cudaGetLastError();
}
LLMB_API int llmb_dequantize_fp8(float* out, const void* q, const float* scale_inv, long long n, int fmt, cudaStream_t st) {
  dequantize_fp8_kernel<<<sm_count() * 8, 256, 0, st>>>(out, (const uint8_t*)q, scale_inv, n, fmt);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_nvfp4_tensor_scale(float* ts, const float* amax, cudaStream_t st) {
  nvfp4_tensor_scale_kernel<<<1, 1, 0, st>>>(ts, amax);
  return (int)cudaGetLastError();
}
// ------------------------------------------------------------------ FP8 with per-128 block scales (fake quantisation)
// x (bf16) -> bf16 holding fp8(x / s) * s with one power-of-two scale s = 2^ceil(log2(amax / fmt_max)) per block:
// 1 x 128 blocks along `axis` (activations, gradients) or 128 x 128 blocks (weights).  Power-of-two scales make
// value x scale exactly representable in bf16, so the block-scaled product can run on the bf16 tensor path with
// the numerics of a block-scaled FP8 GEMM.
namespace {
__device__ __forceinline__ float pow2_scale(float amax, float fmt_max) {
  if (!(amax > 0.f) || isinf(amax)) return 1.0f;
  int e; const float m = frexpf(amax / fmt_max, &e);     // amax / fmt_max = m * 2^e, m in [0.5, 1)
  return ldexpf(1.0f, m == 0.5f ? e - 1 : e);
}
template <int FMT>
__device__ __forceinline__ float fp8_round(float v) {     // value of the nearest fp8 number (saturating)
  const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// 1 x 128 blocks along the contiguous axis: sixteen lanes x 8 values per block
template <int FMT>
__global__ void __launch_bounds__(256) fp8_block_row_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, long long nblocks) {
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / 16;
  const int l = threadIdx.x & 15;
  if (gid >= nblocks) return;
  Pack<__nv_bfloat16> p; p.load(x + gid * 128 + l * 8);
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(p.v[k]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 16));
  const float s = pow2_scale(amax, FMT == 0 ? 448.0f : 57344.0f), inv = 1.0f / s;
#pragma unroll
  for (int k = 0; k < 8; ++k) p.v[k] = fp8_round<FMT>(p.v[k] * inv) * s;
  p.store(out + gid * 128 + l * 8);
}
// 128 x 1 blocks along the rows: one thread per (row block, 8 adjacent columns); two sweeps over the 128 rows
template <int FMT>
__global__ void __launch_bounds__(128) fp8_block_col_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, int rows, int cols) {
  const int cvecs = cols / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)(rows / 128) * cvecs) return;
  const int rb = (int)(idx / cvecs), cv = (int)(idx % cvecs);
  const __nv_bfloat16* src = x + (long long)rb * 128 * cols + cv * 8;
  float amax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int r = 0; r < 128; ++r) {
    Pack<__nv_bfloat16> p; p.load(src + (long long)r * cols);
#pragma unroll
    for (int k = 0; k < 8; ++k) amax[k] = fmaxf(amax[k], fabsf(p.v[k]));
  }
  float s[8], inv[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) { s[k] = pow2_scale(amax[k], FMT == 0 ? 448.0f : 57344.0f); inv[k] = 1.0f / s[k]; }
  __nv_bfloat16* dst = out + (long long)rb * 128 * cols + cv * 8;
  for (int r = 0; r < 128; ++r) {
    Pack<__nv_bfloat16> p; p.load(src + (long long)r * cols);
#pragma unroll
    for (int k = 0; k < 8; ++k) p.v[k] = fp8_round<FMT>(p.v[k] * inv[k]) * s[k];
    p.store(dst + (long long)r * cols);
  }
}
// 128 x 128 blocks: one CTA of 256 threads per block
template <int FMT>
__global__ void __launch_bounds__(256) fp8_block_tile_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, int rows, int cols) {
  const int tiles_c = cols / 128;
  const int tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const __nv_bfloat16* src = x + (long long)tr * 128 * cols + tc * 128;
  __nv_bfloat16* dst = out + (long long)tr * 128 * cols + tc * 128;
  Pack<__nv_bfloat16> p[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {                           // 2048 vectors of 8 in the tile: thread t takes t, t + 256, ...
    const int v = threadIdx.x + i * 256, r = v / 16, c = (v % 16) * 8;
    p[i].load(src + (long long)r * cols + c);
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(p[i].v[k]));
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = pow2_scale(amax, FMT == 0 ? 448.0f : 57344.0f), inv = 1.0f / s;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v = threadIdx.x + i * 256, r = v / 16, c = (v % 16) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) p[i].v[k] = fp8_round<FMT>(p[i].v[k] * inv) * s;
    p[i].store(dst + (long long)r * cols + c);
  }
}
// Block-scaled FP8 operands for the MXFP8 tensor path.  One CTA of 256 threads per 128 x 128 tile of x [rows, cols]:
// GRAN 0 = one scale per tile row (1 x 128 blocks), 1 = one per tile column (128 x 1), 2 = one per tile; TRANS writes the
// bytes transposed ([cols, rows]: the K-major operand of a product contracted over the rows).  The scales go out as the
// tensor core wants them: ue8m0 bytes, one per "outer" line (row of the written matrix) and 32 values of K, four equal
// bytes per 128-block, in 128-line x 4 atoms of 512 bytes, atoms of one line block contiguous along K.
template <int FMT, int GRAN, int TRANS>
__global__ void __launch_bounds__(256) fp8_block_quant_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                              const __nv_bfloat16* __restrict__ x, int rows, int cols) {
  __shared__ float red[16][128];                          // GRAN 1: partial column maxima; GRAN 2: warp maxima in red[0]
  __shared__ float line_scale[128];                       // scale of outer line o of the written tile
  __shared__ __align__(16) uint8_t tile[TRANS ? 128 * 128 : 16];   // transposed bytes, 8-byte chunks XOR-swizzled by line / 8
  const int tiles_c = cols / 128;
  const int tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const int t = threadIdx.x, g = t >> 4, l = t & 15;      // g: row group (rows 8 g + i), l: 8-column slot
  const __nv_bfloat16* src = x + (long long)tr * 128 * cols + tc * 128;
  const float fmax = FMT == 0 ? 448.0f : 57344.0f;
  Pack<__nv_bfloat16> p[8];
  float rmax[8];
  float cmax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    p[i].load(src + (long long)(8 * g + i) * cols + l * 8);
    rmax[i] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float a = fabsf(p[i].v[k]); rmax[i] = fmaxf(rmax[i], a); cmax[k] = fmaxf(cmax[k], a); }
  }
  float s_row[8], s_col[8];
  if (GRAN == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], o, 16));
      s_row[i] = pow2_scale(rmax[i], fmax);
      if (l == 0) line_scale[8 * g + i] = s_row[i];
    }
  } else if (GRAN == 1) {
#pragma unroll
    for (int k = 0; k < 8; ++k) red[g][l * 8 + k] = cmax[k];
    __syncthreads();
    if (t < 128) {
      float m = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) m = fmaxf(m, red[j][t]);
      line_scale[t] = pow2_scale(m, fmax);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) s_col[k] = line_scale[l * 8 + k];
  } else {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, rmax[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((t & 31) == 0) red[0][t >> 5] = m;
    __syncthreads();
    m = red[0][0];
#pragma unroll
    for (int j = 1; j < 8; ++j) m = fmaxf(m, red[0][j]);
    const float s = pow2_scale(m, fmax);
    if (t < 128) line_scale[t] = s;
#pragma unroll
    for (int i = 0; i < 8; ++i) s_row[i] = s;
  }
  uint8_t bt[8][8];                                      // [column slot k][row i]: the transposed 8 x 8 block of this thread
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint8_t b[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float inv = 1.0f / (GRAN == 1 ? s_col[k] : s_row[i]);      // a power of two: exact
      b[k] = (uint8_t)__nv_cvt_float_to_fp8(p[i].v[k] * inv, __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
      bt[k][i] = b[k];
    }
    if (!TRANS) *reinterpret_cast<uint2*>(q + (long long)(tr * 128 + 8 * g + i) * cols + tc * 128 + l * 8) = *reinterpret_cast<uint2*>(b);
  }
  if (TRANS) {
    // line c = 8 l + k of the transposed tile holds rows 8 g .. 8 g + 7 in its 8-byte chunk g, stored at chunk g ^ l:
    // the sixteen lanes that share g hit sixteen different chunks of their lines (no bank conflicts)
#pragma unroll
    for (int k = 0; k < 8; ++k)
      *reinterpret_cast<uint2*>(&tile[(l * 8 + k) * 128 + ((g ^ l) << 3)]) = *reinterpret_cast<uint2*>(bt[k]);
  }
  __syncthreads();
  if (TRANS) {                                            // 128 lines of 128 bytes = 1024 pieces of 16 bytes
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ch = t + j * 256, c = ch >> 3, part = ch & 7, ls = c >> 3;
      uint4 v = *reinterpret_cast<const uint4*>(&tile[c * 128 + ((part ^ (ls >> 1)) << 4)]);
      if (ls & 1) v = make_uint4(v.z, v.w, v.x, v.y);     // odd swizzle: the two chunks of the pair are exchanged
      *reinterpret_cast<uint4*>(q + (long long)(tc * 128 + c) * rows + tr * 128 + part * 16) = v;
    }
  }
  if (t < 128) {
    const uint32_t e = (__float_as_uint(line_scale[t]) >> 23) & 0xffu;   // ue8m0: the biased exponent of the power of two
    const long long atom = TRANS ? (long long)tc * (rows / 128) + tr : (long long)tr * tiles_c + tc;
    *reinterpret_cast<uint32_t*>(sf + atom * 512 + (t & 31) * 16 + (t >> 5) * 4) = e * 0x01010101u;
  }
}
// Both orientations of one operand from ONE read of the tile: q0 / sf0 as <FMT, 0, 0> writes them (1 x 128 blocks, bytes
// [rows, cols]: the operand of a product contracted over the columns) and q1 / sf1 as <FMT, 1, 1> does (128 x 1 blocks, bytes
// transposed [cols, rows]: the operand of a product contracted over the rows).  A layer input needs the first in the forward
// pass and the second for its weight gradient, an output gradient needs the first for dinp and the second for dW.
template <int FMT>
__global__ void __launch_bounds__(256) fp8_block_quant_dual_kernel(uint8_t* __restrict__ q0, uint8_t* __restrict__ sf0, uint8_t* __restrict__ q1,
                                                                   uint8_t* __restrict__ sf1, const __nv_bfloat16* __restrict__ x, int rows, int cols) {
  __shared__ float red[16][128];                          // partial column maxima
  __shared__ float row_scale[128], col_scale[128];
  __shared__ __align__(16) uint8_t tile[128 * 128];       // transposed bytes, 8-byte chunks XOR-swizzled by line / 8
  const int tiles_c = cols / 128;
  const int tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const int t = threadIdx.x, g = t >> 4, l = t & 15;      // g: row group (rows 8 g + i), l: 8-column slot
  const __nv_bfloat16* src = x + (long long)tr * 128 * cols + tc * 128;
  const float fmax = FMT == 0 ? 448.0f : 57344.0f;
  Pack<__nv_bfloat16> p[8];
  float rmax[8];
  float cmax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    p[i].load(src + (long long)(8 * g + i) * cols + l * 8);
    rmax[i] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { const float a = fabsf(p[i].v[k]); rmax[i] = fmaxf(rmax[i], a); cmax[k] = fmaxf(cmax[k], a); }
  }
  float s_row[8], s_col[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) rmax[i] = fmaxf(rmax[i], __shfl_xor_sync(0xffffffffu, rmax[i], o, 16));
    s_row[i] = pow2_scale(rmax[i], fmax);
    if (l == 0) row_scale[8 * g + i] = s_row[i];
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[g][l * 8 + k] = cmax[k];
  __syncthreads();
  if (t < 128) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) m = fmaxf(m, red[j][t]);
    col_scale[t] = pow2_scale(m, fmax);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 8; ++k) s_col[k] = col_scale[l * 8 + k];
  uint8_t bt[8][8];                                      // [column slot k][row i]: the transposed 8 x 8 block of this thread
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint8_t b[8];
    const float inv_r = 1.0f / s_row[i];                  // powers of two: exact
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      b[k] = (uint8_t)__nv_cvt_float_to_fp8(p[i].v[k] * inv_r, __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
      bt[k][i] = (uint8_t)__nv_cvt_float_to_fp8(p[i].v[k] * (1.0f / s_col[k]), __NV_SATFINITE, FMT == 0 ? __NV_E4M3 : __NV_E5M2);
    }
    *reinterpret_cast<uint2*>(q0 + (long long)(tr * 128 + 8 * g + i) * cols + tc * 128 + l * 8) = *reinterpret_cast<uint2*>(b);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k)
    *reinterpret_cast<uint2*>(&tile[(l * 8 + k) * 128 + ((g ^ l) << 3)]) = *reinterpret_cast<uint2*>(bt[k]);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {                           // 128 lines of 128 bytes = 1024 pieces of 16 bytes
    const int ch = t + j * 256, c = ch >> 3, part = ch & 7, ls = c >> 3;
    uint4 v = *reinterpret_cast<const uint4*>(&tile[c * 128 + ((part ^ (ls >> 1)) << 4)]);
    if (ls & 1) v = make_uint4(v.z, v.w, v.x, v.y);       // odd swizzle: the two chunks of the pair are exchanged
    *reinterpret_cast<uint4*>(q1 + (long long)(tc * 128 + c) * rows + tr * 128 + part * 16) = v;
  }
  if (t < 128) {
    const uint32_t er = (__float_as_uint(row_scale[t]) >> 23) & 0xffu, ec = (__float_as_uint(col_scale[t]) >> 23) & 0xffu;
    *reinterpret_cast<uint32_t*>(sf0 + ((long long)tr * tiles_c + tc) * 512 + (t & 31) * 16 + (t >> 5) * 4) = er * 0x01010101u;
    *reinterpret_cast<uint32_t*>(sf1 + ((long long)tc * (rows / 128) + tr) * 512 + (t & 31) * 16 + (t >> 5) * 4) = ec * 0x01010101u;
  }
}
}  // namespace
// mode 0: 1 x 128 blocks along axis 1 (cols % 128 == 0); mode 1: 128 x 1 blocks along axis 0 (rows % 128 == 0, cols % 8 == 0);
// mode 2: 128 x 128 blocks (both % 128 == 0).  fmt 0 = e4m3, 1 = e5m2.  x and out are contiguous [rows, cols] bf16.
LLMB_API int llmb_fp8_block_fake_quant(void* out, const void* x, int rows, int cols, int mode, int fmt, cudaStream_t st) {
  auto* o = (__nv_bfloat16*)out; auto* in = (const __nv_bfloat16*)x;
  if (mode == 0) {
    if (cols % 128) return LLMB_ERR_BAD_ARG;
    const long long nb = (long long)rows * cols / 128;
    const unsigned grid = (unsigned)ceil_div_ll(nb * 16, 256);
    if (fmt == 0) fp8_block_row_kernel<0><<<grid, 256, 0, st>>>(o, in, nb); else fp8_block_row_kernel<1><<<grid, 256, 0, st>>>(o, in, nb);
  } else if (mode == 1) {
    if (rows % 128 || cols % 8) return LLMB_ERR_BAD_ARG;
    const unsigned grid = (unsigned)ceil_div_ll((long long)(rows / 128) * (cols / 8), 128);
    if (fmt == 0) fp8_block_col_kernel<0><<<grid, 128, 0, st>>>(o, in, rows, cols); else fp8_block_col_kernel<1><<<grid, 128, 0, st>>>(o, in, rows, cols);
  } else if (mode == 2) {
    if (rows % 128 || cols % 128) return LLMB_ERR_BAD_ARG;
    const unsigned grid = (unsigned)((rows / 128) * (cols / 128));
    if (fmt == 0) fp8_block_tile_kernel<0><<<grid, 256, 0, st>>>(o, in, rows, cols); else fp8_block_tile_kernel<1><<<grid, 256, 0, st>>>(o, in, rows, cols);
  } else return LLMB_ERR_BAD_ARG;
  return (int)cudaGetLastError();
}

// x [rows, cols] bf16 (both multiples of 128) -> fp8 bytes q and ue8m0 scale atoms sf for llmb_gemm_mxfp8.
// gran 0: 1 x 128 blocks (q [rows, cols]); gran 1: 128 x 1 blocks, written transposed (q [cols, rows]); gran 2: 128 x 128
// blocks, q [rows, cols] or, with transpose, [cols, rows].  sf: (rows / 128) * (cols / 128) * 512 bytes.  fmt 0 e4m3, 1 e5m2.
LLMB_API int llmb_fp8_block_quant(void* q, void* sf, const void* x, int rows, int cols, int gran, int fmt, int transpose,
                                  cudaStream_t st) {
  if (rows % 128 || cols % 128 || fmt < 0 || fmt > 1) return LLMB_ERR_BAD_ARG;
  const unsigned grid = (unsigned)((rows / 128) * (cols / 128));
  auto* qo = (uint8_t*)q; auto* so = (uint8_t*)sf; auto* in = (const __nv_bfloat16*)x;
#define FP8Q(F, G, T) fp8_block_quant_kernel<F, G, T><<<grid, 256, 0, st>>>(qo, so, in, rows, cols)
  if (gran == 0 && !transpose) { if (fmt == 0) FP8Q(0, 0, 0); else FP8Q(1, 0, 0); }
  else if (gran == 1 && transpose) { if (fmt == 0) FP8Q(0, 1, 1); else FP8Q(1, 1, 1); }
  else if (gran == 2 && !transpose) { if (fmt == 0) FP8Q(0, 2, 0); else FP8Q(1, 2, 0); }
  else if (gran == 2 && transpose) { if (fmt == 0) FP8Q(0, 2, 1); else FP8Q(1, 2, 1); }
  else return LLMB_ERR_BAD_ARG;
#undef FP8Q
  return (int)cudaGetLastError();
}

// Both at once from one read of x: (q0, sf0) = llmb_fp8_block_quant(gran 0) and (q1, sf1) = llmb_fp8_block_quant(gran 1, transpose).
LLMB_API int llmb_fp8_block_quant_dual(void* q0, void* sf0, void* q1, void* sf1, const void* x, int rows, int cols, int fmt, cudaStream_t st) {
  if (rows % 128 || cols % 128 || fmt < 0 || fmt > 1) return LLMB_ERR_BAD_ARG;
  const unsigned grid = (unsigned)((rows / 128) * (cols / 128));
  if (fmt == 0) fp8_block_quant_dual_kernel<0><<<grid, 256, 0, st>>>((uint8_t*)q0, (uint8_t*)sf0, (uint8_t*)q1, (uint8_t*)sf1, (const __nv_bfloat16*)x, rows, cols);
  else fp8_block_quant_dual_kernel<1><<<grid, 256, 0, st>>>((uint8_t*)q0, (uint8_t*)sf0, (uint8_t*)q1, (uint8_t*)sf1, (const __nv_bfloat16*)x, rows, cols);
  return (int)cudaGetLastError();
}

LLMB_API long long llmb_nvfp4_scale_bytes(long long outer, long long K, int swizzled) {
  const long long kb = K / 16;
  if (!swizzled) return outer * kb;
  return ceil_div_ll(outer, 128) * ceil_div_ll(kb, 4) * 512;
}
// x [rows, cols]; blocks of (block_rows x 16) along `axis`; any of q / scales / deq may be null.
LLMB_API int llmb_nvfp4_quantize(void* q, void* scales, void* deq, const void* x, const float* tensor_scale, int rows, int cols,
                                 int axis, int block_rows, int rht, int sr, unsigned long long seed, unsigned long long stream,
                                 long long step, int swizzled, int dtype, cudaStream_t st) {
  const int outer = axis == 1 ? rows : cols, K = axis == 1 ? cols : rows;
  if (K % 16 || (block_rows != 1 && block_rows != 16)) return LLMB_ERR_BAD_ARG;
  const long long n_col_tiles = swizzled ? ceil_div_ll(K / 16, 4) : 0;
  const long long total = (long long)ceil_div(outer, block_rows) * (K / 16);
  const int threads = 128;
  const unsigned grid = (unsigned)ceil_div_ll(total, threads);
  if (dtype == LLMB_BF16 && block_rows == 16 && !rht && cols % 16 == 0 && outer % 16 == 0 && K % 16 == 0) {
    const long long lanes = total * 16;
    nvfp4_quantize16_coop_kernel<<<(unsigned)ceil_div_ll(lanes, 256), 256, 0, st>>>((uint8_t*)q, (uint8_t*)scales, (__nv_bfloat16*)deq,
        (const __nv_bfloat16*)x, tensor_scale, rows, cols, axis, sr, seed, stream, step, n_col_tiles);
    return (int)cudaGetLastError();
  }
#define NVFP4_LAUNCH(T, BR) nvfp4_quantize_kernel<T, BR><<<grid, threads, 0, st>>>((uint8_t*)q, (uint8_t*)scales, (__nv_bfloat16*)deq, (const T*)x, tensor_scale, rows, cols, axis, rht, sr, seed, stream, step, n_col_tiles)
  if (dtype == LLMB_BF16) { if (block_rows == 1) NVFP4_LAUNCH(__nv_bfloat16, 1); else NVFP4_LAUNCH(__nv_bfloat16, 16); }
  else { if (block_rows == 1) NVFP4_LAUNCH(float, 1); else NVFP4_LAUNCH(float, 16); }
#undef NVFP4_LAUNCH
  return (int)cudaGetLastError();
}
LLMB_API int llmb_nvfp4_dequantize(float* out, const void* q, const void* scales, const float* tensor_scale, int rows, int K,
                                   int swizzled, cudaStream_t st) {
  const long long n_col_tiles = swizzled ? ceil_div_ll(K / 16, 4) : 0;
  nvfp4_dequant_kernel<<<sm_count() * 8, 256, 0, st>>>(out, (const uint8_t*)q, (const uint8_t*)scales, tensor_scale, rows, K, n_col_tiles);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_hadamard16(void* out, const void* x, long long n, int inverse, int dtype, cudaStream_t st) {
  if (n % 16) return LLMB_ERR_BAD_ARG;
  if (dtype == LLMB_BF16) hadamard16_kernel<__nv_bfloat16><<<sm_count() * 4, 256, 0, st>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, n / 16, inverse);
  else hadamard16_kernel<float><<<sm_count() * 4, 256, 0, st>>>((float*)out, (const float*)x, n / 16, inverse);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_rng_uniform(float* out, long long n, unsigned long long seed, unsigned long long stream, unsigned long long base, cudaStream_t st) {
  rng_uniform_kernel<<<sm_count() * 4, 256, 0, st>>>(out, n, seed, stream, base);
  return (int)cudaGetLastError();
}
