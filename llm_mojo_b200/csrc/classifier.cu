// Fused softmax + cross-entropy + in-place dlogits over the padded vocabulary, plus the
// generic row softmax used by sampling.
//
// Reference behaviour: llmm/fused_classifier.mojo:186-279, :311-370 (per row: max, sum exp,
// loss, dlogits = (p - 1[y])·dloss written over the logits, padded tail [V, Vp) zeroed);
// llmm/softmax.mojo:172-304.  B200 design: the whole row (Vp·2 B ≈ 100 KB for GPT-2) is staged once
// in shared memory so HBM sees exactly one read and one write.  bf16 rows stream through a persistent
// CTA per SM: the bulk-copy engine loads row r+1 into one buffer and stores row r-1 out of it while the
// 1024 threads make their three passes (max, exponentials + sum, scale) over row r in the other.
#include "tc05.cuh"
using namespace llmb;
using namespace tc05;

namespace {
template <typename T>
__global__ void __launch_bounds__(1024) classifier_kernel(T* __restrict__ logits, float* __restrict__ losses,
                                                         const int* __restrict__ targets, float dloss, int V, int Vp,
                                                         int write_dlogits) {
  constexpr int N = Pack<T>::N;
  extern __shared__ __align__(16) unsigned char smraw[];
  T* row_s = reinterpret_cast<T*>(smraw);
  __shared__ float red[32];
  __shared__ float bcast[2];
  const int row = blockIdx.x;
  T* g = logits + (size_t)row * Vp;
  const int nvec = Vp / N;
  const int tid = threadIdx.x, lane = tid % 32, wid = tid / 32, nw = blockDim.x / 32;
  float mx = -INFINITY;
  for (int v = tid; v < nvec; v += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(g + v * N);
    *reinterpret_cast<uint4*>(row_s + v * N) = raw;
    Pack<T> p; p.load(row_s + v * N);
#pragma unroll
    for (int k = 0; k < N; ++k) if (v * N + k < V) mx = fmaxf(mx, p.v[k]);
  }
  mx = warp_max(mx);
  if (lane == 0) red[wid] = mx;
  __syncthreads();
  if (wid == 0) { float m = lane < nw ? red[lane] : -INFINITY; m = warp_max(m); if (lane == 0) bcast[0] = m; }
  __syncthreads();
  mx = bcast[0];
  const float L2E = 1.4426950408889634f;
  // second pass: e = 2^((x - max)·log2e) once per element; the row buffer is overwritten with e (in the
  // storage dtype) so that the third pass is a multiply, not another exponential
  const int tgt_raw = targets[row];
  const int tgt = llmb_in_range(tgt_raw, V, LLMB_SITE_CLASSIFIER_TARGET) ? tgt_raw : 0;   // checked build: a bad target is recorded and clamped
  const float x_tgt = to_f<T>(row_s[tgt]);            // read before the buffer is overwritten
  __syncthreads();
  float sum = 0.f;
  for (int v = tid; v < nvec; v += blockDim.x) {
    Pack<T> p; p.load(row_s + v * N);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const float e = (v * N + k < V) ? exp2f((p.v[k] - mx) * L2E) : 0.f;
      sum += e;
      p.v[k] = e;
    }
    if (write_dlogits) p.store(row_s + v * N);
  }
  sum = warp_sum(sum);
  if (lane == 0) red[wid] = sum;
  __syncthreads();
  if (wid == 0) { float s = lane < nw ? red[lane] : 0.f; s = warp_sum(s); if (lane == 0) bcast[1] = s; }
  __syncthreads();
  sum = bcast[1];
  if (tid == 0 && losses) losses[row] = -(x_tgt - mx - logf(sum));
  if (!write_dlogits) return;
  const float inv = dloss / sum;
  for (int v = tid; v < nvec; v += blockDim.x) {
    Pack<T> p; p.load(row_s + v * N);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      const int i = v * N + k;
      p.v[k] = p.v[k] * inv - (i == tgt ? dloss : 0.f);      // padded columns hold e = 0
    }
    p.store(g + v * N);
  }
}

// Persistent streaming variant for bf16 rows (two row buffers fit in shared memory).
__device__ __forceinline__ float ex2_fast(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(ssrc)), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(1024, 1) classifier_stream_kernel(__nv_bfloat16* __restrict__ logits, float* __restrict__ losses,
                                                                   const int* __restrict__ targets, float dloss, int rows, int V,
                                                                   int Vp, int write_dlogits, int buf_bytes, int* status) {
  using T = __nv_bfloat16;
  constexpr int N = 8;
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ uint64_t full[2];
  __shared__ float red[32];
  __shared__ float bcast[2];
  __shared__ int fail_s;
  const int tid = threadIdx.x, lane = tid % 32, wid = tid / 32, nw = blockDim.x / 32;
  const uint32_t row_bytes = (uint32_t)Vp * 2;
  const int nvec = Vp / N;
  if (tid == 0) { mbar_init(&full[0], 1); mbar_init(&full[1], 1); fail_s = 0; fence_barrier_init(); }
  __syncthreads();
  int r = blockIdx.x;
  if (tid == 0 && r < rows) {
    mbar_expect_tx(&full[0], row_bytes);
    bulk_load_1d(smraw, logits + (size_t)r * Vp, row_bytes, &full[0]);
  }
  const float L2E = 1.4426950408889634f;
  for (int it = 0; r < rows; r += gridDim.x, ++it) {
    const int b = it & 1;
    T* row_s = reinterpret_cast<T*>(smraw + (size_t)b * buf_bytes);
    const int rn = r + gridDim.x;
    if (tid == 0 && rn < rows) {
      bulk_wait_read<0>();                  // the store of the previous row has finished reading the other buffer
      mbar_expect_tx(&full[b ^ 1], row_bytes);
      bulk_load_1d(smraw + (size_t)(b ^ 1) * buf_bytes, logits + (size_t)rn * Vp, row_bytes, &full[b ^ 1]);
    }
    if (!mbar_wait(&full[b], (it >> 1) & 1)) { atomicExch(status, LLMB_ERR_TIMEOUT); fail_s = 1; }
    __syncthreads();
    if (fail_s) break;
    // Vectors that lie wholly inside the real vocabulary [0, V) need no per-element bound checks; the one
    // vector that straddles V and the padded ones after it are handled by a second, checked loop.
    const int nfull = V / N;                 // vectors entirely below V
    // pass 1: row maximum over the real vocabulary
    float mx = -INFINITY;
    for (int v = tid; v < nfull; v += blockDim.x) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) mx = fmaxf(mx, p.v[k]);
    }
    for (int v = nfull + tid; v < nvec; v += blockDim.x) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) if (v * N + k < V) mx = fmaxf(mx, p.v[k]);
    }
    mx = warp_max(mx);
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    if (wid == 0) { float m = lane < nw ? red[lane] : -INFINITY; m = warp_max(m); if (lane == 0) bcast[0] = m; }
    __syncthreads();
    mx = bcast[0];
    const int tgt_raw = targets[r];
  const int tgt = llmb_in_range(tgt_raw, V, LLMB_SITE_CLASSIFIER_TARGET) ? tgt_raw : 0;   // checked build: a bad target is recorded and clamped
    const float x_tgt = __bfloat162float(row_s[tgt]);     // read before the buffer is overwritten
    __syncthreads();
    // pass 2: e = 2^((x - max) log2 e), once per element, written back over the row
    float sum = 0.f;
    const float mb = mx * L2E;
    for (int v = tid; v < nfull; v += blockDim.x) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { p.v[k] = ex2_fast(fmaf(p.v[k], L2E, -mb)); sum += p.v[k]; }
      if (write_dlogits) p.store(row_s + v * N);
    }
    for (int v = nfull + tid; v < nvec; v += blockDim.x) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { p.v[k] = (v * N + k < V) ? ex2_fast(fmaf(p.v[k], L2E, -mb)) : 0.f; sum += p.v[k]; }
      if (write_dlogits) p.store(row_s + v * N);
    }
    sum = warp_sum(sum);
    if (lane == 0) red[wid] = sum;
    __syncthreads();
    if (wid == 0) { float s = lane < nw ? red[lane] : 0.f; s = warp_sum(s); if (lane == 0) bcast[1] = s; }
    __syncthreads();
    sum = bcast[1];
    if (tid == 0 && losses) losses[r] = -(x_tgt - mx - logf(sum));
    if (write_dlogits) {
      // pass 3: dlogits = (e / sum - 1[target]) dloss in place (padded columns hold e = 0); the target column is
      // corrected afterwards by the one thread that owns it; then one bulk store of the row
      const float inv = dloss / sum;
      for (int v = tid; v < nvec; v += blockDim.x) {
        Pack<T> p; p.load(row_s + v * N);
#pragma unroll
        for (int k = 0; k < N; ++k) p.v[k] *= inv;
        p.store(row_s + v * N);
      }
      __syncthreads();
      if (tid == 0) {
        const float e_t = ex2_fast(fmaf(x_tgt, L2E, -mb));
        row_s[tgt] = __float2bfloat16(__bfloat162float(__float2bfloat16(e_t)) * inv - dloss);
      }
      fence_proxy_async();
      __syncthreads();
      if (tid == 0) { bulk_store_1d(logits + (size_t)r * Vp, row_s, row_bytes); bulk_commit(); }
    } else {
      __syncthreads();                      // everyone is done with the buffer before it is reloaded
    }
  }
  if (tid == 0) bulk_wait<0>();             // shared memory must outlive the last store
}

// The same streaming kernel with the row traffic on its own warp.  In the kernel above thread 0 waits for the previous
// row's store to have read its buffer before it may prefetch the next row, and everybody waits for thread 0 at the next
// barrier: the store's read-out is serialised with the row's arithmetic.  Here warps 0..30 (992 threads, named barrier 1)
// only compute; warp 31 moves rows: it stores a buffer once the compute warps hand it over (`done`), waits for that
// store to have read the buffer and refills it with the row after next (`full`).  Per row the steady state is
// max(arithmetic, (arithmetic + store + load) / 2) instead of store + arithmetic.
__global__ void __launch_bounds__(1024, 1) classifier_stream2_kernel(__nv_bfloat16* __restrict__ logits, float* __restrict__ losses,
                                                                     const int* __restrict__ targets, float dloss, int rows, int V,
                                                                     int Vp, int write_dlogits, int buf_bytes, int* status) {
  using T = __nv_bfloat16;
  constexpr int N = 8;
  constexpr int NC = 992, NCW = 31;                       // compute threads / warps
  extern __shared__ __align__(128) unsigned char smraw[];
  __shared__ uint64_t full[2], done[2];
  __shared__ float red[32];
  __shared__ float bcast[2];
  __shared__ int fail_s;
  const int tid = threadIdx.x, lane = tid % 32, wid = tid / 32;
  const uint32_t row_bytes = (uint32_t)Vp * 2;
  const int nvec = Vp / N;
  if (tid == 0) {
    mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(&done[0], 1); mbar_init(&done[1], 1);
    fail_s = 0; fence_barrier_init();
  }
  __syncthreads();
  auto csync = [] { asm volatile("bar.sync 1, 992;" ::: "memory"); };

  if (wid == NCW) {
    // ------------------------------------------------------------ row mover (one lane)
    if (lane == 0) {
      for (int j = 0; j < 2; ++j) {
        const long long r = (long long)blockIdx.x + (long long)j * gridDim.x;
        if (r < rows) { mbar_expect_tx(&full[j], row_bytes); bulk_load_1d(smraw + (size_t)j * buf_bytes, logits + (size_t)r * Vp, row_bytes, &full[j]); }
      }
      int it = 0;
      for (int r = blockIdx.x; r < rows; r += gridDim.x, ++it) {
        const int b = it & 1;
        unsigned char* buf = smraw + (size_t)b * buf_bytes;
        if (!mbar_wait(&done[b], (it >> 1) & 1)) { atomicExch(status, LLMB_ERR_TIMEOUT); break; }
        if (write_dlogits) { bulk_store_1d(logits + (size_t)r * Vp, buf, row_bytes); bulk_commit(); }
        const long long rn = (long long)r + 2ll * gridDim.x;
        if (rn < rows) {
          if (write_dlogits) bulk_wait_read<0>();         // the store has read the buffer
          mbar_expect_tx(&full[b], row_bytes);
          bulk_load_1d(buf, logits + (size_t)rn * Vp, row_bytes, &full[b]);
        }
      }
      bulk_wait<0>();                                     // shared memory must outlive the last store
    }
    return;
  }

  // -------------------------------------------------------------- compute warps
  const float L2E = 1.4426950408889634f;
  const int nfull = V / N;                                // vectors entirely below V
  int it = 0;
  for (int r = blockIdx.x; r < rows; r += gridDim.x, ++it) {
    const int b = it & 1;
    T* row_s = reinterpret_cast<T*>(smraw + (size_t)b * buf_bytes);
    if (!mbar_wait(&full[b], (it >> 1) & 1)) { atomicExch(status, LLMB_ERR_TIMEOUT); fail_s = 1; }
    csync();
    if (fail_s) break;
    // pass 1: row maximum over the real vocabulary
    float mx = -INFINITY;
    for (int v = tid; v < nfull; v += NC) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) mx = fmaxf(mx, p.v[k]);
    }
    for (int v = nfull + tid; v < nvec; v += NC) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) if (v * N + k < V) mx = fmaxf(mx, p.v[k]);
    }
    mx = warp_max(mx);
    if (lane == 0) red[wid] = mx;
    csync();
    if (wid == 0) { float m = lane < NCW ? red[lane] : -INFINITY; m = warp_max(m); if (lane == 0) bcast[0] = m; }
    csync();
    mx = bcast[0];
    const int tgt_raw = targets[r];
  const int tgt = llmb_in_range(tgt_raw, V, LLMB_SITE_CLASSIFIER_TARGET) ? tgt_raw : 0;   // checked build: a bad target is recorded and clamped
    const float x_tgt = __bfloat162float(row_s[tgt]);     // read before the buffer is overwritten
    csync();
    // pass 2: e = 2^((x - max) log2 e), once per element, written back over the row
    float sum = 0.f;
    const float mb = mx * L2E;
    for (int v = tid; v < nfull; v += NC) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { p.v[k] = ex2_fast(fmaf(p.v[k], L2E, -mb)); sum += p.v[k]; }
      if (write_dlogits) p.store(row_s + v * N);
    }
    for (int v = nfull + tid; v < nvec; v += NC) {
      Pack<T> p; p.load(row_s + v * N);
#pragma unroll
      for (int k = 0; k < N; ++k) { p.v[k] = (v * N + k < V) ? ex2_fast(fmaf(p.v[k], L2E, -mb)) : 0.f; sum += p.v[k]; }
      if (write_dlogits) p.store(row_s + v * N);
    }
    sum = warp_sum(sum);
    if (lane == 0) red[wid] = sum;
    csync();
    if (wid == 0) { float s = lane < NCW ? red[lane] : 0.f; s = warp_sum(s); if (lane == 0) bcast[1] = s; }
    csync();
    sum = bcast[1];
    if (tid == 0 && losses) losses[r] = -(x_tgt - mx - logf(sum));
    if (write_dlogits) {
      // pass 3: dlogits = (e / sum - 1[target]) dloss in place (padded columns hold e = 0); the target column is
      // corrected afterwards by one thread; then the row is handed to the mover
      const float inv = dloss / sum;
      for (int v = tid; v < nvec; v += NC) {
        Pack<T> p; p.load(row_s + v * N);
#pragma unroll
        for (int k = 0; k < N; ++k) p.v[k] *= inv;
        p.store(row_s + v * N);
      }
      fence_proxy_async();                                // these writes, before the mover's bulk store reads them
      csync();
      if (tid == 0) {
        const float e_t = ex2_fast(fmaf(x_tgt, L2E, -mb));
        row_s[tgt] = __float2bfloat16(__bfloat162float(__float2bfloat16(e_t)) * inv - dloss);
        fence_proxy_async();
        mbar_arrive(&done[b]);
      }
    } else {
      csync();                                            // everyone is done with the buffer before it is reloaded
      if (tid == 0) mbar_arrive(&done[b]);
    }
  }
}

template <typename T>
__global__ void softmax_rows_kernel(float* __restrict__ out, const T* __restrict__ inp, int V, int ld, float inv_temp) {
  __shared__ float red[32];
  __shared__ float bc;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid % 32, wid = tid / 32, nw = blockDim.x / 32;
  const T* g = inp + (size_t)row * ld;
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, to_f<T>(g[i]) * inv_temp);
  mx = warp_max(mx); if (lane == 0) red[wid] = mx; __syncthreads();
  if (wid == 0) { float m = lane < nw ? red[lane] : -INFINITY; m = warp_max(m); if (lane == 0) bc = m; } __syncthreads();
  mx = bc; float s = 0.f;
  for (int i = tid; i < V; i += blockDim.x) s += expf(to_f<T>(g[i]) * inv_temp - mx);
  s = warp_sum(s); __syncthreads(); if (lane == 0) red[wid] = s; __syncthreads();
  if (wid == 0) { float t = lane < nw ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) bc = t; } __syncthreads();
  float inv = 1.f / bc;
  for (int i = tid; i < V; i += blockDim.x) out[(size_t)row * V + i] = expf(to_f<T>(g[i]) * inv_temp - mx) * inv;
}

// dlogits = probs * (dprobs - sum_k dprobs[k] * probs[k]) over the first V columns of a row (one block per row);
// columns V..ld-1 of dlogits are zeroed.  (llmm/softmax.mojo:632, softmax_bwd)
__global__ void softmax_bwd_kernel(float* __restrict__ dlogits, const float* __restrict__ dprobs, const float* __restrict__ probs,
                                   int V, int ld) {
  __shared__ float red[32];
  __shared__ float bc;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid % 32, wid = tid / 32, nw = blockDim.x / 32;
  const float* dp = dprobs + (size_t)row * ld;
  const float* pr = probs + (size_t)row * ld;
  float dot = 0.f;
  for (int i = tid; i < V; i += blockDim.x) dot = fmaf(dp[i], pr[i], dot);
  dot = warp_sum(dot); if (lane == 0) red[wid] = dot; __syncthreads();
  if (wid == 0) { float t = lane < nw ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) bc = t; } __syncthreads();
  dot = bc;
  float* out = dlogits + (size_t)row * ld;
  for (int i = tid; i < ld; i += blockDim.x) out[i] = i < V ? pr[i] * (dp[i] - dot) : 0.f;
}

// Unfused cross-entropy over stored probabilities (llmm/crossentropy.mojo:110, :284): loss = -log p[target];
// backward writes only the target slot, dprobs[target] = -dloss / p[target] (the caller zeroes dprobs first).
__global__ void crossentropy_fwd_kernel(float* __restrict__ losses, const float* __restrict__ probs, const int* __restrict__ targets,
                                        int rows, int ld) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) losses[i] = -logf(probs[(size_t)i * ld + targets[i]]);
}
__global__ void crossentropy_bwd_kernel(float* __restrict__ dprobs, const float* __restrict__ dlosses, const float* __restrict__ probs,
                                        const int* __restrict__ targets, int rows, int ld) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) { const size_t o = (size_t)i * ld + targets[i]; dprobs[o] = -dlosses[i] / probs[o]; }
}
}  // namespace

LLMB_API int llmb_softmax_bwd(float* dlogits, const float* dprobs, const float* probs, int rows, int V, int ld, cudaStream_t st) {
  if (rows <= 0 || V <= 0 || ld < V) return LLMB_ERR_BAD_ARG;
  softmax_bwd_kernel<<<rows, 256, 0, st>>>(dlogits, dprobs, probs, V, ld);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_crossentropy_fwd(float* losses, const float* probs, const int* targets, int rows, int ld, cudaStream_t st) {
  if (rows <= 0) return LLMB_ERR_BAD_ARG;
  crossentropy_fwd_kernel<<<ceil_div(rows, 256), 256, 0, st>>>(losses, probs, targets, rows, ld);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_crossentropy_bwd(float* dprobs, const float* dlosses, const float* probs, const int* targets, int rows, int ld,
                                   cudaStream_t st) {
  if (rows <= 0) return LLMB_ERR_BAD_ARG;
  crossentropy_bwd_kernel<<<ceil_div(rows, 256), 256, 0, st>>>(dprobs, dlosses, probs, targets, rows, ld);
  return (int)cudaGetLastError();
}

LLMB_BOUNDS_REPORT_FN(llmb_bounds_report_classifier)

// logits [rows, Vp] are overwritten with dlogits when write_dlogits != 0.
LLMB_API int llmb_fused_classifier(void* logits, float* losses, const int* targets, float dloss, int rows, int V,
                                   int Vp, int write_dlogits, int dtype, int* status, cudaStream_t st) {
  if (dtype == LLMB_BF16) {
    if (Vp % 8) return LLMB_ERR_BAD_ARG;
    static int stream_on = -1;
    if (stream_on < 0) { const char* e = getenv("LLMB_CLASSIFIER_STREAM"); stream_on = (e && e[0] == '0') ? 0 : (e && e[0] == '2') ? 2 : 1; }
    const int buf_bytes = (Vp * 2 + 127) & ~127;
    if (stream_on && status && 2 * buf_bytes <= 224 * 1024 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
      const int grid = rows < sm_count() ? rows : sm_count();
      if (stream_on == 2) {                               // LLMB_CLASSIFIER_STREAM=2: row traffic on thread 0 of the compute block
        cudaFuncSetAttribute(classifier_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * buf_bytes);
        classifier_stream_kernel<<<grid, 1024, 2 * buf_bytes, st>>>((__nv_bfloat16*)logits, losses, targets, dloss, rows, V, Vp,
                                                                   write_dlogits, buf_bytes, status);
      } else {
        cudaFuncSetAttribute(classifier_stream2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * buf_bytes);
        classifier_stream2_kernel<<<grid, 1024, 2 * buf_bytes, st>>>((__nv_bfloat16*)logits, losses, targets, dloss, rows, V, Vp,
                                                                    write_dlogits, buf_bytes, status);
      }
      return (int)cudaGetLastError();
    }
    size_t smem = (size_t)Vp * 2;
    if (smem > 200 * 1024) return LLMB_ERR_BAD_ARG;
    cudaFuncSetAttribute(classifier_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    classifier_kernel<__nv_bfloat16><<<rows, 1024, smem, st>>>((__nv_bfloat16*)logits, losses, targets, dloss, V, Vp, write_dlogits);
  } else {
    if (Vp % 4) return LLMB_ERR_BAD_ARG;
    size_t smem = (size_t)Vp * 4;
    if (smem > 220 * 1024) return LLMB_ERR_BAD_ARG;
    cudaFuncSetAttribute(classifier_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    classifier_kernel<float><<<rows, 1024, smem, st>>>((float*)logits, losses, targets, dloss, V, Vp, write_dlogits);
  }
  return (int)cudaGetLastError();
}

LLMB_API int llmb_softmax_rows(float* out, const void* inp, int rows, int V, int ld, float inv_temp, int dtype,
                               cudaStream_t st) {
  if (dtype == LLMB_BF16) softmax_rows_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(out, (const __nv_bfloat16*)inp, V, ld, inv_temp);
  else softmax_rows_kernel<float><<<rows, 256, 0, st>>>(out, (const float*)inp, V, ld, inv_temp);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- chunked cross-entropy
// Two-pass online-softmax CE over vocabulary tiles, so the full [rows, Vp] logits never exist
// (llmm/fused_classifier.mojo:503-841).  stats[row] = {running max, running sum-exp, target logit, -}.
namespace {
template <typename T>
__global__ void __launch_bounds__(256) ce_pass1_kernel(float4* __restrict__ stats, const T* __restrict__ tile, const int* __restrict__ targets,
                                                      int ld, int col0, int width, int V, int first) {
  __shared__ float red[32];
  __shared__ float bc;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid % 32, wid = tid / 32, nw = blockDim.x / 32;
  const T* g = tile + (size_t)row * ld;
  const int valid = min(width, V - col0);           // columns of this tile that are real vocabulary
  float mx = -INFINITY;
  for (int i = tid; i < valid; i += blockDim.x) mx = fmaxf(mx, to_f<T>(g[i]));
  mx = warp_max(mx); if (lane == 0) red[wid] = mx; __syncthreads();
  if (wid == 0) { float m = lane < nw ? red[lane] : -INFINITY; m = warp_max(m); if (lane == 0) bc = m; } __syncthreads();
  mx = bc;
  float s = 0.f;
  for (int i = tid; i < valid; i += blockDim.x) s += expf(to_f<T>(g[i]) - mx);
  s = warp_sum(s); __syncthreads(); if (lane == 0) red[wid] = s; __syncthreads();
  if (wid == 0) { float t = lane < nw ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) bc = t; } __syncthreads();
  if (tid == 0) {
    float4 st = first ? make_float4(-INFINITY, 0.f, 0.f, 0.f) : stats[row];
    if (valid > 0) {
      const float m_new = fmaxf(st.x, mx);
      st.y = st.y * expf(st.x - m_new) + bc * expf(mx - m_new);
      st.x = m_new;
    }
    const int tgt = targets[row];
    if (tgt >= col0 && tgt < col0 + valid) st.z = to_f<T>(g[tgt - col0]);
    stats[row] = st;
  }
}
__global__ void ce_loss_kernel(float* __restrict__ losses, const float4* __restrict__ stats, int rows) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) { float4 st = stats[r]; losses[r] = -(st.z - st.x - logf(st.y)); }
}
template <typename T>
__global__ void __launch_bounds__(256) ce_pass2_kernel(T* __restrict__ tile, const float4* __restrict__ stats, const int* __restrict__ targets,
                                                      int ld, int col0, int width, int V, float dloss) {
  const int row = blockIdx.x;
  T* g = tile + (size_t)row * ld;
  const float4 st = stats[row];
  const float lse = st.x + logf(st.y);
  const int tgt = targets[row] - col0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = 0.f;
    if (col0 + i < V) v = (expf(to_f<T>(g[i]) - lse) - (i == tgt ? 1.f : 0.f)) * dloss;
    g[i] = from_f<T>(v);
  }
}
}  // namespace

LLMB_API int llmb_ce_pass1(float* stats, const void* tile, const int* targets, int rows, int ld, int col0, int width, int V,
                           int first, int dtype, cudaStream_t st) {
  if (dtype == LLMB_BF16) ce_pass1_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((float4*)stats, (const __nv_bfloat16*)tile, targets, ld, col0, width, V, first);
  else ce_pass1_kernel<float><<<rows, 256, 0, st>>>((float4*)stats, (const float*)tile, targets, ld, col0, width, V, first);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_ce_loss(float* losses, const float* stats, int rows, cudaStream_t st) {
  ce_loss_kernel<<<ceil_div(rows, 256), 256, 0, st>>>(losses, (const float4*)stats, rows);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_ce_pass2(void* tile, const float* stats, const int* targets, int rows, int ld, int col0, int width, int V,
                           float dloss, int dtype, cudaStream_t st) {
  if (dtype == LLMB_BF16) ce_pass2_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((__nv_bfloat16*)tile, (const float4*)stats, targets, ld, col0, width, V, dloss);
  else ce_pass2_kernel<float><<<rows, 256, 0, st>>>((float*)tile, (const float4*)stats, targets, ld, col0, width, V, dloss);
  return (int)cudaGetLastError();
}
