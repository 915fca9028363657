// Encoder (wte + wpe) forward / deterministic backward, tanh-GELU forward/backward,
// bias-gradient column reduction, and small utility kernels.
//
// Reference behaviour: llmm/encoder.mojo:131-281 (fwd), :459-536 / :775-1029 (deterministic
// bucketed dwte and dwpe), llmm/gelu.mojo:82-430, llmm/matmul.mojo:2353-2539 (dbias).
// B200 design: all accesses are 16-byte vectors; dwte is made deterministic by a device-side
// radix sort of (token, position) keys followed by one block per token run, instead of the
// reference's host-side counting sort.
#include "common.cuh"
#include <cub/device/device_radix_sort.cuh>

using namespace llmb;

// ---------------------------------------------------------------- encoder forward
template <typename T>
__global__ void encoder_fwd_kernel(T* __restrict__ out, const int* __restrict__ tok, const T* __restrict__ wte,
                                   const T* __restrict__ wpe, int BT, int Tlen, int C, int V) {
  constexpr int N = Pack<T>::N;
  const int vec_per_row = C / N;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)BT * vec_per_row;
  if (idx >= total) return;
  int row = (int)(idx / vec_per_row), c = (int)(idx % vec_per_row) * N;
  int t = row % Tlen;
  int id = tok[row];
  if (!llmb_in_range(id, V, LLMB_SITE_ENCODER_FWD_TOKEN)) return;
  Pack<T> a, b;
  a.load(wte + (size_t)id * C + c);
  b.load(wpe + (size_t)t * C + c);
#pragma unroll
  for (int i = 0; i < N; ++i) a.v[i] += b.v[i];
  a.store(out + (size_t)row * C + c);
}

LLMB_BOUNDS_REPORT_FN(llmb_bounds_report_elementwise)

// V: rows of wte (token ids must be below it; tested in the checked build only)
LLMB_API int llmb_encoder_fwd(void* out, const int* tok, const void* wte, const void* wpe, int B, int T, int C, int V,
                              int dtype, cudaStream_t st) {
  int BT = B * T;
  if (dtype == LLMB_BF16) {
    if (C % 8) return LLMB_ERR_BAD_ARG;
    long long total = (long long)BT * (C / 8);
    encoder_fwd_kernel<__nv_bfloat16><<<(unsigned)ceil_div_ll(total, 256), 256, 0, st>>>(
        (__nv_bfloat16*)out, tok, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, BT, T, C, V);
  } else {
    if (C % 4) return LLMB_ERR_BAD_ARG;
    long long total = (long long)BT * (C / 4);
    encoder_fwd_kernel<float><<<(unsigned)ceil_div_ll(total, 256), 256, 0, st>>>(
        (float*)out, tok, (const float*)wte, (const float*)wpe, BT, T, C, V);
  }
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- encoder backward
__global__ void make_keys_kernel(unsigned long long* keys, const int* tok, int BT) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < BT) keys[i] = ((unsigned long long)(unsigned)tok[i] << 32) | (unsigned)i;
}

// dwte[token] += sum of the dout rows of that token's positions, deterministic and independent of how skewed the token
// distribution is (on real text a handful of tokens own several per cent of the positions; a loop over one token's run
// would take milliseconds).  The sorted keys are cut into segments of 16; one warp sums the runs inside its segment.  A run
// that lies inside one segment is added to dwte at once (nothing else touches that row); the piece of a run that crosses a
// segment border goes to a per-segment partial row (slot 0: the run began in an earlier segment, slot 1: it goes on in the
// next one), and wte_bwd_combine_kernel adds up the pieces of each such run in segment order.
constexpr int WTE_SEG = 16;
template <typename T>
__global__ void __launch_bounds__(256) wte_bwd_kernel(float* __restrict__ dwte, float* __restrict__ partial, const T* __restrict__ dout,
                                                      const unsigned long long* __restrict__ keys, int BT, int C, int V) {
  constexpr int N = Pack<T>::N;
  const int lane = threadIdx.x % 32, seg = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const int j0 = seg * WTE_SEG;
  if (j0 >= BT) return;
  const int cnt = min(WTE_SEG, BT - j0);
  unsigned long long mykey = lane < cnt ? keys[j0 + lane] : 0ull;
  const unsigned prev_tok = j0 > 0 ? (unsigned)(keys[j0 - 1] >> 32) : 0xffffffffu;
  const unsigned next_tok = j0 + cnt < BT ? (unsigned)(keys[j0 + cnt] >> 32) : 0xffffffffu;
  const int vec_per_row = C / N;
  for (int vc0 = 0; vc0 < vec_per_row; vc0 += 32) {       // this lane's channel vectors, one after the other; every lane walks the
    const int vc = vc0 + lane;                             // loop (the shuffles below need the whole warp), idle ones past the row end
    const bool live = vc < vec_per_row;
    float acc[N];
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] = 0.f;
    int a = 0;                                              // first position of the current run inside the segment
    for (int j = 0; j < cnt; ++j) {
      const unsigned long long key = __shfl_sync(0xffffffffu, mykey, j);
      const unsigned tokv = (unsigned)(key >> 32);
      const bool ok = llmb_in_range((long long)tokv, V, LLMB_SITE_ENCODER_BWD_TOKEN);
      if (ok && live) {
        Pack<T> p; p.load(dout + (size_t)(unsigned)(key & 0xffffffffu) * C + vc * N);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += p.v[k];
      }
      const unsigned nxt = j + 1 < cnt ? (unsigned)(__shfl_sync(0xffffffffu, mykey, j + 1) >> 32) : next_tok;
      if (j + 1 == cnt || nxt != tokv) {                    // the run (or its piece in this segment) ends here
        const bool from_before = a == 0 && prev_tok == tokv, goes_on = j + 1 == cnt && next_tok == tokv;
        if (ok && live) {
          float* dst = (from_before || goes_on) ? partial + ((size_t)seg * 2 + (from_before ? 0 : 1)) * C + vc * N
                                                : dwte + (size_t)tokv * C + vc * N;
          if (from_before || goes_on) {
#pragma unroll
            for (int k = 0; k < N; ++k) dst[k] = acc[k];
          } else {
#pragma unroll
            for (int k = 0; k < N; ++k) dst[k] += acc[k];
          }
        }
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] = 0.f;
        a = j + 1;
      }
    }
  }
}
// One block per segment: if a run leaves this segment through its end (and did not enter through its start, i.e. this
// is where the run's first piece lives), its pieces are summed in segment order and added to dwte.
__global__ void __launch_bounds__(256) wte_bwd_combine_kernel(float* __restrict__ dwte, const float* __restrict__ partial,
                                                              const unsigned long long* __restrict__ keys, int BT, int C, int V) {
  const int seg = blockIdx.x, j0 = seg * WTE_SEG, cnt = min(WTE_SEG, BT - j0);
  const unsigned tokv = (unsigned)(keys[j0 + cnt - 1] >> 32);
  if (j0 + cnt >= BT || (unsigned)(keys[j0 + cnt] >> 32) != tokv) return;            // nothing leaves through the end
  const bool whole = (unsigned)(keys[j0] >> 32) == tokv;                              // the segment holds this token only
  if (whole && j0 > 0 && (unsigned)(keys[j0 - 1] >> 32) == tokv) return;              // a middle piece: the run's first segment does the sum
  if (!llmb_in_range((long long)tokv, V, LLMB_SITE_ENCODER_BWD_TOKEN)) return;
  // the run's end by bisection over the sorted keys (the loop below then has no load in its condition)
  __shared__ int last_seg_s;
  if (threadIdx.x == 0) {
    int lo = j0 + cnt, hi = BT;                            // keys[lo] is this token; first index beyond the run in (lo, hi]
    while (lo + 1 < hi) {
      const int mid = lo + (hi - lo) / 2;
      if ((unsigned)(keys[mid] >> 32) == tokv) lo = mid; else hi = mid;
    }
    last_seg_s = lo / WTE_SEG;
  }
  __syncthreads();
  const int last_seg = last_seg_s;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float s = partial[((size_t)seg * 2 + 1) * C + c];
#pragma unroll 8
    for (int t = seg + 1; t <= last_seg; ++t) s += partial[((size_t)t * 2) * C + c];
    dwte[(size_t)tokv * C + c] += s;
  }
}

template <typename T>
__global__ void wpe_bwd_kernel(float* __restrict__ dwpe, const T* __restrict__ dout, int B, int Tlen, int C) {
  constexpr int N = Pack<T>::N;
  const int vec_per_row = C / N;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= Tlen * vec_per_row) return;
  int t = idx / vec_per_row, c = (idx % vec_per_row) * N;
  float acc[N];
#pragma unroll
  for (int k = 0; k < N; ++k) acc[k] = 0.f;
  for (int b = 0; b < B; ++b) {
    Pack<T> p; p.load(dout + ((size_t)b * Tlen + t) * C + c);
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] += p.v[k];
  }
#pragma unroll
  for (int k = 0; k < N; ++k) dwpe[(size_t)t * C + c + k] += acc[k];
}

// Scratch layout: keys_in[BT] u64 | keys_out[BT] u64 | cub temp | partial rows [segments][2][C] fp32.  Query the size first.
static size_t encoder_bwd_sort_bytes(int BT) {
  size_t temp = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, temp, (unsigned long long*)nullptr, (unsigned long long*)nullptr, BT);
  return 2 * (size_t)BT * sizeof(unsigned long long) + ((temp + 255) / 256) * 256 + 256;
}
LLMB_API long long llmb_encoder_bwd_scratch_bytes(int BT, int C) {
  return (long long)(encoder_bwd_sort_bytes(BT) + (size_t)ceil_div(BT, WTE_SEG) * 2 * C * sizeof(float));
}

LLMB_API int llmb_encoder_bwd(float* dwte, float* dwpe, const void* dout, const int* tok, void* scratch,
                              long long scratch_bytes, int B, int T, int C, int V, int vocab_bits, int dtype,
                              cudaStream_t st) {
  int BT = B * T;
  if (scratch_bytes < llmb_encoder_bwd_scratch_bytes(BT, C)) return LLMB_ERR_BAD_ARG;
  unsigned long long* kin = (unsigned long long*)scratch;
  unsigned long long* kout = kin + BT;
  void* temp = (void*)(kout + BT);
  const size_t sort_bytes = encoder_bwd_sort_bytes(BT);
  size_t temp_bytes = sort_bytes - 2 * (size_t)BT * sizeof(unsigned long long);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(scratch) + sort_bytes);
  make_keys_kernel<<<ceil_div(BT, 256), 256, 0, st>>>(kin, tok, BT);
  // position bits live in [0, 32); token bits in [32, 32 + vocab_bits). Sort only the used bits.
  cudaError_t e = cub::DeviceRadixSort::SortKeys(temp, temp_bytes, kin, kout, BT, 0, 32 + vocab_bits, st);
  if (e != cudaSuccess) return (int)e;
  const int nseg = ceil_div(BT, WTE_SEG);
  if (dtype == LLMB_BF16) {
    if (C % 8) return LLMB_ERR_BAD_ARG;
    wte_bwd_kernel<__nv_bfloat16><<<ceil_div(nseg, 8), 256, 0, st>>>(dwte, partial, (const __nv_bfloat16*)dout, kout, BT, C, V);
    wte_bwd_combine_kernel<<<nseg, 256, 0, st>>>(dwte, partial, kout, BT, C, V);
    wpe_bwd_kernel<__nv_bfloat16><<<ceil_div(T * (C / 8), 256), 256, 0, st>>>(dwpe, (const __nv_bfloat16*)dout, B, T, C);
  } else {
    if (C % 4) return LLMB_ERR_BAD_ARG;
    wte_bwd_kernel<float><<<ceil_div(nseg, 8), 256, 0, st>>>(dwte, partial, (const float*)dout, kout, BT, C, V);
    wte_bwd_combine_kernel<<<nseg, 256, 0, st>>>(dwte, partial, kout, BT, C, V);
    wpe_bwd_kernel<float><<<ceil_div(T * (C / 4), 256), 256, 0, st>>>(dwpe, (const float*)dout, B, T, C);
  }
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- GELU
template <typename T>
__global__ void gelu_fwd_kernel(T* __restrict__ out, const T* __restrict__ inp, long long nvec) {
  constexpr int N = Pack<T>::N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    Pack<T> p; p.load(inp + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) p.v[k] = gelu_f(p.v[k]);
    p.store(out + i * N);
  }
}
template <typename T>
__global__ void gelu_bwd_kernel(T* __restrict__ dinp, const T* __restrict__ inp, const T* __restrict__ dout, long long nvec) {
  constexpr int N = Pack<T>::N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    Pack<T> x, d; x.load(inp + i * N); d.load(dout + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) d.v[k] *= gelu_grad_f(x.v[k]);
    d.store(dinp + i * N);
  }
}
LLMB_API int llmb_gelu_fwd(void* out, const void* inp, long long n, int dtype, cudaStream_t st) {
  int grid = sm_count() * 8;
  if (dtype == LLMB_BF16) { if (n % 8) return LLMB_ERR_BAD_ARG; gelu_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)inp, n / 8); }
  else { if (n % 4) return LLMB_ERR_BAD_ARG; gelu_fwd_kernel<float><<<grid, 256, 0, st>>>((float*)out, (const float*)inp, n / 4); }
  return (int)cudaGetLastError();
}
LLMB_API int llmb_gelu_bwd(void* dinp, const void* inp, const void* dout, long long n, int dtype, cudaStream_t st) {
  int grid = sm_count() * 8;
  if (dtype == LLMB_BF16) { if (n % 8) return LLMB_ERR_BAD_ARG; gelu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)dinp, (const __nv_bfloat16*)inp, (const __nv_bfloat16*)dout, n / 8); }
  else { if (n % 4) return LLMB_ERR_BAD_ARG; gelu_bwd_kernel<float><<<grid, 256, 0, st>>>((float*)dinp, (const float*)inp, (const float*)dout, n / 4); }
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- dbias: dbias[c] += sum_rows dout[row, c]
// Stage 1: grid (col blocks, row slabs); each block owns 32*N columns... threads (8 row lanes x 32 col vecs).
// partial[slab][c] written to scratch; stage 2 sums slabs in order (deterministic) and accumulates.
template <typename T, int RL>
__global__ void __launch_bounds__(256) dbias_partial_kernel(float* __restrict__ partial, const T* __restrict__ dout, int rows, int OC, int rows_per_slab) {
  constexpr int N = Pack<T>::N;
  constexpr int CV = 256 / RL;                           // column vectors per block; RL row lanes
  __shared__ float sm[RL][CV * N + 1];
  int cv = threadIdx.x % CV, rl = threadIdx.x / CV;
  int c0 = (blockIdx.x * CV + cv) * N;
  int r0 = blockIdx.y * rows_per_slab, r1 = min(rows, r0 + rows_per_slab);
  float acc[N];
#pragma unroll
  for (int k = 0; k < N; ++k) acc[k] = 0.f;
  if (c0 < OC) {
    int r = r0 + rl;
    for (; r + 3 * RL < r1; r += 4 * RL) {              // four independent loads in flight per thread
      Pack<T> p0, p1, p2, p3;
      p0.load(dout + (size_t)r * OC + c0); p1.load(dout + (size_t)(r + RL) * OC + c0);
      p2.load(dout + (size_t)(r + 2 * RL) * OC + c0); p3.load(dout + (size_t)(r + 3 * RL) * OC + c0);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] += (p0.v[k] + p1.v[k]) + (p2.v[k] + p3.v[k]);
    }
    for (; r < r1; r += RL) {
      Pack<T> p; p.load(dout + (size_t)r * OC + c0);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] += p.v[k];
    }
  }
#pragma unroll
  for (int k = 0; k < N; ++k) sm[rl][cv * N + k] = acc[k];
  __syncthreads();
  for (int c = threadIdx.x; c < CV * N; c += blockDim.x) {
    int col = blockIdx.x * CV * N + c;
    if (col < OC) {
      float s = 0.f;
#pragma unroll
      for (int l = 0; l < RL; ++l) s += sm[l][c];
      partial[(size_t)blockIdx.y * OC + col] = s;
    }
  }
}
// narrow matrices get more row lanes per block (fewer columns per block) so that the grid still fills the machine
template <typename T>
void dbias_partial_launch(float* partial, const T* dout, int rows, int OC, int rows_per_slab, int slabs, cudaStream_t st) {
  constexpr int N = Pack<T>::N;
  const int want = 6 * sm_count();
  if (ceil_div(OC, 32 * N) * slabs >= want)
    dbias_partial_kernel<T, 8><<<dim3(ceil_div(OC, 32 * N), slabs), 256, 0, st>>>(partial, dout, rows, OC, rows_per_slab);
  else if (ceil_div(OC, 16 * N) * slabs >= want)
    dbias_partial_kernel<T, 16><<<dim3(ceil_div(OC, 16 * N), slabs), 256, 0, st>>>(partial, dout, rows, OC, rows_per_slab);
  else
    dbias_partial_kernel<T, 32><<<dim3(ceil_div(OC, 8 * N), slabs), 256, 0, st>>>(partial, dout, rows, OC, rows_per_slab);
}
// Stage 2: 32 columns per block, eight threads per column each summing every eighth slab (independent loads in flight
// instead of one thread walking all slabs), then a fixed-order sum of the eight: deterministic.
__global__ void __launch_bounds__(256) dbias_final_kernel(float* __restrict__ dbias, const float* __restrict__ partial, int OC, int slabs) {
  __shared__ float sm[8][33];
  const int cl = threadIdx.x % 32, sl = threadIdx.x / 32;
  const int c = blockIdx.x * 32 + cl;
  float s = 0.f;
  if (c < OC) {
#pragma unroll 4
    for (int i = sl; i < slabs; i += 8) s += partial[(size_t)i * OC + c];
  }
  sm[sl][cl] = s;
  __syncthreads();
  if (sl == 0 && c < OC) {
    float t = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) t += sm[l][cl];
    dbias[c] += t;
  }
}
LLMB_API int llmb_dbias_slabs(int rows) { int s = ceil_div(rows, 128); return s > 128 ? 128 : (s < 1 ? 1 : s); }
LLMB_API long long llmb_dbias_scratch_bytes(int rows, int OC) { return (long long)llmb_dbias_slabs(rows) * OC * sizeof(float); }
LLMB_API int llmb_dbias(float* dbias, const void* dout, float* scratch, long long scratch_bytes, int rows, int OC,
                        int dtype, cudaStream_t st) {
  int slabs = llmb_dbias_slabs(rows);
  if (scratch_bytes < (long long)slabs * OC * (long long)sizeof(float)) return LLMB_ERR_BAD_ARG;  // regression guard: never overrun
  int rows_per_slab = ceil_div(rows, slabs);
  if (dtype == LLMB_BF16) {
    if (OC % 8) return LLMB_ERR_BAD_ARG;
    dbias_partial_launch<__nv_bfloat16>(scratch, (const __nv_bfloat16*)dout, rows, OC, rows_per_slab, slabs, st);
  } else {
    if (OC % 4) return LLMB_ERR_BAD_ARG;
    dbias_partial_launch<float>(scratch, (const float*)dout, rows, OC, rows_per_slab, slabs, st);
  }
  dbias_final_kernel<<<ceil_div(OC, 32), 256, 0, st>>>(dbias, scratch, OC, slabs);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- casts
__global__ void cast_f32_to_bf16_kernel(__nv_bfloat16* out, const float* in, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}
// ----------------------------------------------------------------------------- non-finite census
// counts[0] += number of NaN, counts[1] += number of +-Inf in x[0..n) (debug scan of a named tensor;
// reference: _debug_grad_nanscan, train_gpt2.mojo:5385-5577)
template <typename T>
__global__ void nan_census_kernel(const T* __restrict__ x, long long n, int* __restrict__ counts) {
  int nan = 0, inf = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = (float)x[i];
    nan += isnan(v) ? 1 : 0;
    inf += isinf(v) ? 1 : 0;
  }
  for (int o = 16; o > 0; o >>= 1) { nan += __shfl_xor_sync(0xffffffffu, nan, o); inf += __shfl_xor_sync(0xffffffffu, inf, o); }
  if ((threadIdx.x & 31) == 0) {
    if (nan) atomicAdd(&counts[0], nan);
    if (inf) atomicAdd(&counts[1], inf);
  }
}
LLMB_API int llmb_nan_census(int* counts, const void* x, long long n, int dtype, cudaStream_t st) {
  if (n <= 0) return 0;
  const int block = 256;
  long long want = (n + block - 1) / block;
  const int grid = (int)(want < 4LL * sm_count() ? want : 4LL * sm_count());
  if (dtype == 1) nan_census_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)x, n, counts);
  else nan_census_kernel<float><<<grid, block, 0, st>>>((const float*)x, n, counts);
  return (int)cudaGetLastError();
}

LLMB_API int llmb_cast_f32_to_bf16(void* out, const float* in, long long n, cudaStream_t st) {
  cast_f32_to_bf16_kernel<<<sm_count() * 8, 256, 0, st>>>((__nv_bfloat16*)out, in, n);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- dbias without caller scratch
// Variant of llmb_dbias for callers that cannot allocate device memory (see llmb_noalloc.h).
// The partial sums live in a file-scope device array.  In host code `g_dbias_noalloc_scratch`
// only names the symbol; its device address is fetched with cudaGetSymbolAddress once per
// device and that pointer is what the kernels receive.
#include "llmb_noalloc.h"
static __device__ __align__(256) float g_dbias_noalloc_scratch[LLMB_DBIAS_NOALLOC_MAX_FLOATS];

#include <mutex>
namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;      // host threads may make their first call on a device at the same time
}

LLMB_API int llmb_dbias_noalloc(float* dbias, const void* dout, int rows, int OC, int dtype, cudaStream_t st) {
  if (rows <= 0 || OC <= 0 || !dbias || !dout) return LLMB_ERR_BAD_ARG;
  const int slabs = llmb_dbias_slabs(rows);
  if ((long long)slabs * OC > (long long)LLMB_DBIAS_NOALLOC_MAX_FLOATS) return LLMB_ERR_BAD_ARG;   // beyond the built-in scratch
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return LLMB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(dout) & 15) || (reinterpret_cast<uintptr_t>(dbias) & 3)) return LLMB_ERR_BAD_ARG;   // 16-byte row loads
  float* scratch;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {   // set-up, once per device, with that device current
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_dbias_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  const int rows_per_slab = ceil_div(rows, slabs);
  if (dtype == LLMB_BF16) {
    if (OC % 8) return LLMB_ERR_BAD_ARG;
    dbias_partial_launch<__nv_bfloat16>(scratch, (const __nv_bfloat16*)dout, rows, OC, rows_per_slab, slabs, st);
  } else if (dtype == LLMB_F32) {
    if (OC % 4) return LLMB_ERR_BAD_ARG;
    dbias_partial_launch<float>(scratch, (const float*)dout, rows, OC, rows_per_slab, slabs, st);
  } else {
    return LLMB_ERR_BAD_ARG;
  }
  dbias_final_kernel<<<ceil_div(OC, 32), 256, 0, st>>>(dbias, scratch, OC, slabs);
  return (int)cudaGetLastError();
}
