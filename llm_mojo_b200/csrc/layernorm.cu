// LayerNorm forward (optionally fused with the residual add that precedes it) and backward
// with the residual-gradient accumulate and dgamma/dbeta reduction.
//
// Reference behaviour: llmm/layernorm.mojo:197-331 (fwd, mean/rstd saved fp32), :651-1096 (fused
// residual fwd), :1582-1895 (bwd with register-accumulated dgamma/dbeta partials + finalize),
// :2426-2614 (fused residual bwd).  B200 design: one warp per row, the row lives in registers
// (single HBM read), 16-byte accesses; backward is a persistent grid whose blocks write one
// dgamma/dbeta partial row each into scratch, summed in block order by a finalize kernel so
// the result does not depend on scheduling.
#include "common.cuh"
using namespace llmb;

namespace {
constexpr int LN_MAX_VEC = 16;  // 16-byte vectors per lane: C <= 32*16*8 = 4096 for bf16
constexpr float LN_EPS = 1e-5f;

template <typename T, bool RESID, int PER_LANE>
__global__ void __launch_bounds__(256) ln_fwd_kernel(T* __restrict__ out, float* __restrict__ mean_o, float* __restrict__ rstd_o,
                                                    T* __restrict__ resid_out, const T* __restrict__ inp1,
                                                    const T* __restrict__ inp2, const T* __restrict__ w,
                                                    const T* __restrict__ b, int rows, int C) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x % 32, wid = threadIdx.x / 32;
  const int nvec = C / N;                       // vectors per row
  constexpr int per_lane = PER_LANE;            // 16-byte vectors per lane: the row lives in registers
  int row = blockIdx.x * (blockDim.x / 32) + wid;
  if (row >= rows) return;
  float x[PER_LANE][N];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    if (i < per_lane) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
        Pack<T> p; p.load(inp1 + (size_t)row * C + vc * N);
        if (RESID) {
          Pack<T> q; q.load(inp2 + (size_t)row * C + vc * N);
#pragma unroll
          for (int k = 0; k < N; ++k) p.v[k] = to_f<T>(from_f<T>(p.v[k] + q.v[k]));  // round like the stored residual
          p.store(resid_out + (size_t)row * C + vc * N);
        }
#pragma unroll
        for (int k = 0; k < N; ++k) { x[i][k] = p.v[k]; sum += p.v[k]; }
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k) x[i][k] = 0.f;
      }
    }
  }
  float mean = warp_sum(sum) / C;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    if (i < per_lane) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
#pragma unroll
        for (int k = 0; k < N; ++k) { float d = x[i][k] - mean; var += d * d; }
      }
    }
  }
  float rstd = rsqrtf(warp_sum(var) / C + LN_EPS);
  if (lane == 0) { if (mean_o) mean_o[row] = mean; if (rstd_o) rstd_o[row] = rstd; }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    if (i < per_lane) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
        Pack<T> ww, bb, o; ww.load(w + vc * N); bb.load(b + vc * N);
#pragma unroll
        for (int k = 0; k < N; ++k) o.v[k] = (x[i][k] - mean) * rstd * ww.v[k] + bb.v[k];
        o.store(out + (size_t)row * C + vc * N);
      }
    }
  }
}

// Backward.  dres[row] (+)= LN'(dout[row]); partial dgamma/dbeta per block into scratch.
// Each warp walks rows grid-stride and keeps dgamma/dbeta partials for its lanes' channels in
// registers; warps of a block are then combined in fixed order through shared memory.
// SUMOUT: the column sums of the values written to dres are a third per-block partial (the bias gradient of the
// linear layer whose output gradient dres is), taken from the values as stored (after rounding to T).
template <typename T, int PER_LANE, bool ACCUM, bool SUMOUT = false>
__global__ void __launch_bounds__(256) ln_bwd_kernel(T* __restrict__ dres, float* __restrict__ partial,
                                                    const T* __restrict__ dout, const T* __restrict__ inp,
                                                    const T* __restrict__ w, const float* __restrict__ mean_i,
                                                    const float* __restrict__ rstd_i, int rows, int C) {
  constexpr int N = Pack<T>::N;
  constexpr int NS = SUMOUT ? 3 : 2;
  extern __shared__ float sm[];  // [warps][NS][C]
  const int lane = threadIdx.x % 32, wid = threadIdx.x / 32, nwarps = blockDim.x / 32;
  const int nvec = C / N;
  float dg[PER_LANE][N], db[PER_LANE][N], ds[SUMOUT ? PER_LANE : 1][N];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
#pragma unroll
    for (int k = 0; k < N; ++k) { dg[i][k] = 0.f; db[i][k] = 0.f; if (SUMOUT) ds[i][k] = 0.f; }
  }
  for (int row = blockIdx.x * nwarps + wid; row < rows; row += gridDim.x * nwarps) {
    float mean = mean_i[row], rstd = rstd_i[row];
    uint4 xr[PER_LANE], dr[PER_LANE], ar[PER_LANE];   // raw 16-byte vectors: the row stays in registers
    float s1 = 0.f, s2 = 0.f;
    // all global loads of the row (input, upstream gradient and the gradient accumulated so far) are issued
    // before the first use, so the row costs one memory round trip instead of two
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
        xr[i] = *reinterpret_cast<const uint4*>(inp + (size_t)row * C + vc * N);
        dr[i] = *reinterpret_cast<const uint4*>(dout + (size_t)row * C + vc * N);
        if (ACCUM) ar[i] = *reinterpret_cast<const uint4*>(dres + (size_t)row * C + vc * N);
      }
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
        Pack<T> x, d, ww; x.load(reinterpret_cast<const T*>(&xr[i])); d.load(reinterpret_cast<const T*>(&dr[i]));
        ww.load(w + vc * N);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          float n_ = (x.v[k] - mean) * rstd;
          float dn_ = d.v[k] * ww.v[k];
          s1 += dn_; s2 += dn_ * n_;
          dg[i][k] += d.v[k] * n_; db[i][k] += d.v[k];
        }
      }
    }
    s1 = warp_sum(s1) / C; s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      int vc = i * 32 + lane;
      if (vc < nvec) {
        Pack<T> x, d, ww, o; x.load(reinterpret_cast<const T*>(&xr[i])); d.load(reinterpret_cast<const T*>(&dr[i]));
        ww.load(w + vc * N);
        if (ACCUM) o.load(reinterpret_cast<const T*>(&ar[i]));
#pragma unroll
        for (int k = 0; k < N; ++k) {
          float n_ = (x.v[k] - mean) * rstd;
          float g = (d.v[k] * ww.v[k] - s1 - n_ * s2) * rstd;
          o.v[k] = ACCUM ? o.v[k] + g : g;
          if (SUMOUT) ds[i][k] += round_to<T>(o.v[k]);
        }
        o.store(dres + (size_t)row * C + vc * N);
      }
    }
  }
  // block combine (fixed warp order)
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    int vc = i * 32 + lane;
    if (vc < nvec) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        sm[(wid * NS + 0) * C + vc * N + k] = dg[i][k];
        sm[(wid * NS + 1) * C + vc * N + k] = db[i][k];
        if (SUMOUT) sm[(wid * NS + 2) * C + vc * N + k] = ds[i][k];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < NS * C; c += blockDim.x) {
    int which = c / C, cc = c % C;
    float s = 0.f;
    for (int wdx = 0; wdx < nwarps; ++wdx) s += sm[(wdx * NS + which) * C + cc];
    partial[(size_t)blockIdx.x * NS * C + c] = s;
  }
}

// dw[c] += sum_i partial[i][c], db[c] += sum_i partial[i][C + c] over the per-block partial rows.  A block of
// 32 x 8 threads owns 32 adjacent columns of the 2C-wide partial matrix: 8 row groups walk the rows in parallel
// (coalesced 128-byte reads) and are combined in fixed order through shared memory.
__global__ void __launch_bounds__(256) ln_bwd_final_kernel(float* __restrict__ dw, float* __restrict__ db, float* __restrict__ dsum,
                                                          const float* __restrict__ partial, int C, int nblocks) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  const int NS = dsum ? 3 : 2;                           // dsum: third partial = column sums of the stored dres
  float s = 0.f;
  if (c < NS * C)
    for (int i = ty; i < nblocks; i += 8) s += partial[(size_t)i * NS * C + c];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < NS * C) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][tx];
    if (c < C) dw[c] += t; else if (c < 2 * C) db[c - C] += t; else dsum[c - 2 * C] += t;
  }
}

template <typename T, int PER_LANE>
int ln_fwd_launch_n(void* out, float* mean, float* rstd, void* resid_out, const void* inp1, const void* inp2,
                    const void* w, const void* b, int rows, int C, cudaStream_t st) {
  int grid = ceil_div(rows, 8);
  if (inp2)
    ln_fwd_kernel<T, true, PER_LANE><<<grid, 256, 0, st>>>((T*)out, mean, rstd, (T*)resid_out, (const T*)inp1, (const T*)inp2, (const T*)w, (const T*)b, rows, C);
  else
    ln_fwd_kernel<T, false, PER_LANE><<<grid, 256, 0, st>>>((T*)out, mean, rstd, nullptr, (const T*)inp1, nullptr, (const T*)w, (const T*)b, rows, C);
  return (int)cudaGetLastError();
}

template <typename T>
int ln_fwd_launch(void* out, float* mean, float* rstd, void* resid_out, const void* inp1, const void* inp2,
                  const void* w, const void* b, int rows, int C, cudaStream_t st) {
  constexpr int N = Pack<T>::N;
  if (C % N || C / N > 32 * LN_MAX_VEC) return LLMB_ERR_BAD_ARG;
  const int per = ceil_div(C / N, 32);
#define LNF(P) return ln_fwd_launch_n<T, P>(out, mean, rstd, resid_out, inp1, inp2, w, b, rows, C, st)
  if (per <= 1) LNF(1); if (per <= 2) LNF(2); if (per <= 3) LNF(3); if (per <= 4) LNF(4); if (per <= 5) LNF(5);
  if (per <= 6) LNF(6); if (per <= 7) LNF(7); if (per <= 8) LNF(8); if (per <= 10) LNF(10); if (per <= 12) LNF(12);
  if (per <= 13) LNF(13); LNF(16);
#undef LNF
}

template <typename T, int PER_LANE>
int ln_bwd_launch_n(void* dres, float* partial, const void* dout, const void* inp, const void* w, const float* mean,
                    const float* rstd, int rows, int C, int accumulate, int grid, cudaStream_t st, bool sumout = false) {
  size_t smem = (size_t)8 * (sumout ? 3 : 2) * C * sizeof(float);
  if (smem > 220 * 1024) return LLMB_ERR_BAD_ARG;
  auto kern_a = ln_bwd_kernel<T, PER_LANE, true>;
  auto kern_n = ln_bwd_kernel<T, PER_LANE, false>;
  auto kern_as = ln_bwd_kernel<T, PER_LANE, true, true>;
  auto kern_ns = ln_bwd_kernel<T, PER_LANE, false, true>;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(kern_a, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(kern_n, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(kern_as, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(kern_ns, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  auto kern = sumout ? (accumulate ? kern_as : kern_ns) : (accumulate ? kern_a : kern_n);
  kern<<<grid, 256, smem, st>>>((T*)dres, partial, (const T*)dout, (const T*)inp, (const T*)w, mean, rstd, rows, C);
  return (int)cudaGetLastError();
}
}  // namespace

LLMB_API int llmb_layernorm_fwd(void* out, float* mean, float* rstd, void* resid_out, const void* inp1,
                                const void* inp2, const void* w, const void* b, int rows, int C, int dtype,
                                cudaStream_t st) {
  return dtype == LLMB_BF16 ? ln_fwd_launch<__nv_bfloat16>(out, mean, rstd, resid_out, inp1, inp2, w, b, rows, C, st)
                            : ln_fwd_launch<float>(out, mean, rstd, resid_out, inp1, inp2, w, b, rows, C, st);
}

LLMB_API int llmb_layernorm_bwd_blocks(int rows) { int g = sm_count() * 2; int need = ceil_div(rows, 8); return need < g ? need : g; }
LLMB_API long long llmb_layernorm_bwd_scratch_bytes(int rows, int C) {
  return (long long)llmb_layernorm_bwd_blocks(rows) * 3 * C * sizeof(float);      // room for the optional column-sum partial
}

// dres (+)= LN-backward(dout); dw += ..., db += ...  (dw/db fp32).  accumulate=1 adds into dres.
LLMB_API int llmb_layernorm_bwd_colsum(void* dres, float* dw, float* db, float* dsum, float* scratch, long long scratch_bytes,
                                       const void* dout, const void* inp, const void* w, const float* mean,
                                       const float* rstd, int rows, int C, int accumulate, int dtype, cudaStream_t st);
LLMB_API int llmb_layernorm_bwd(void* dres, float* dw, float* db, float* scratch, long long scratch_bytes,
                                const void* dout, const void* inp, const void* w, const float* mean,
                                const float* rstd, int rows, int C, int accumulate, int dtype, cudaStream_t st) {
  return llmb_layernorm_bwd_colsum(dres, dw, db, nullptr, scratch, scratch_bytes, dout, inp, w, mean, rstd, rows, C, accumulate, dtype, st);
}
// As llmb_layernorm_bwd; with dsum != nullptr additionally dsum[c] += sum over rows of the values written to dres[:, c]
// (fp32 [C]): the bias gradient of the linear layer whose output gradient dres is, without another pass over dres.
LLMB_API int llmb_layernorm_bwd_colsum(void* dres, float* dw, float* db, float* dsum, float* scratch, long long scratch_bytes,
                                       const void* dout, const void* inp, const void* w, const float* mean,
                                       const float* rstd, int rows, int C, int accumulate, int dtype, cudaStream_t st) {
  int grid = llmb_layernorm_bwd_blocks(rows);
  const bool sumout = dsum != nullptr;
  if (scratch_bytes < (long long)grid * (sumout ? 3 : 2) * C * (long long)sizeof(float)) return LLMB_ERR_BAD_ARG;
  int rc;
  if (dtype == LLMB_BF16) {
    int per = ceil_div(C / 8, 32);
    if (C % 8) return LLMB_ERR_BAD_ARG;
#define LN_CASE(P) rc = ln_bwd_launch_n<__nv_bfloat16, P>(dres, scratch, dout, inp, w, mean, rstd, rows, C, accumulate, grid, st, sumout)
    if (per <= 2) LN_CASE(2); else if (per <= 3) LN_CASE(3); else if (per <= 4) LN_CASE(4); else if (per <= 5) LN_CASE(5);
    else if (per <= 7) LN_CASE(7); else if (per <= 8) LN_CASE(8); else if (per <= 12) LN_CASE(12); else if (per <= 16) LN_CASE(16);
    else return LLMB_ERR_BAD_ARG;
#undef LN_CASE
  } else {
    int per = ceil_div(C / 4, 32);
    if (C % 4) return LLMB_ERR_BAD_ARG;
#define LN_CASE(P) rc = ln_bwd_launch_n<float, P>(dres, scratch, dout, inp, w, mean, rstd, rows, C, accumulate, grid, st, sumout)
    if (per <= 2) LN_CASE(2); else if (per <= 4) LN_CASE(4); else if (per <= 6) LN_CASE(6); else if (per <= 8) LN_CASE(8);
    else if (per <= 10) LN_CASE(10); else if (per <= 13) LN_CASE(13); else if (per <= 16) LN_CASE(16);
    else return LLMB_ERR_BAD_ARG;
#undef LN_CASE
  }
  if (rc) return rc;
  ln_bwd_final_kernel<<<ceil_div((sumout ? 3 : 2) * C, 32), 256, 0, st>>>(dw, db, dsum, scratch, C, grid);
  return (int)cudaGetLastError();
}
