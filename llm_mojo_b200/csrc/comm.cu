// Peer-memory collectives over NVLink / NVSwitch, fused with the compute that surrounds them.
//
// The reference's collectives are host-driven staged copies plus one add kernel
// (llmm/zero.mojo:267-284, :579-1318): every collective drains the stream, meets the other rank
// threads at a CPU barrier and moves data with driver copies.  Here every rank maps every
// peer's communication arena (CUDA IPC) and the collectives are kernels that load / store peer
// memory directly, so that they run on a side stream under the backward pass:
//
//   pack      fp32 gradient ranges -> bf16 (x 1/W) into this rank's send buffer, then signal
//   reduce    wait for all peers' send buffers, pull the elements this rank owns from every
//             peer in rank order (bitwise identical on all ranks), sum in fp32, then either
//               RS: add into the fp32 gradient shard and emit sum-of-squares partials, or
//               AR: push the bf16 result into every peer's receive buffer and signal
//   unpack    (AR) wait for all owners, receive buffer -> fp32 gradients + sum-of-squares
//   adamw_push  sharded AdamW that stores each new bf16 parameter into every rank's copy
//             (optimizer step + parameter all-gather in one kernel)
//   gather    (ZeRO-3) pull parameter ranges from their owners' shards into a local window
//   scalar_allreduce  W floats exchanged through peer stores, summed in rank order
//
// Synchronisation is by monotonically increasing sequence numbers in per-rank flag words that
// the producer stores into every peer's arena (st.release.sys) and the consumer polls in its
// own memory (ld.acquire.sys).  Every wait is bounded; on expiry the kernel records
// LLMB_ERR_TIMEOUT in the status word and returns without touching peer memory.  Only plain
// peer loads / stores are used (no multimem, no TMA multicast).
#include "common.cuh"
using namespace llmb;

namespace {
constexpr int MAX_RANKS = 8;
constexpr int MAX_SEGS = 40;
enum { FLAG_READY = 0, FLAG_DONE = 1, FLAG_READY2 = 2, FLAG_PARAM = 3, FLAG_SCALAR = 4, FLAG_DONE2 = 5, FLAG_ROWS_READY = 6,
       FLAG_ROWS_DONE = 7, FLAG_STATS_READY = 8, FLAG_STATS_DONE = 9, NUM_FLAG_KINDS = 10 };

struct PeerPtrs { void* p[MAX_RANKS]; };
struct SegList {
  int n;
  int owner[MAX_SEGS];
  long long src_off[MAX_SEGS], dst_off[MAX_SEGS], len[MAX_SEGS];   // elements; all multiples of 8
  long long vec_prefix[MAX_SEGS + 1];                              // prefix sums of len/8
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// flags layout inside an arena: unsigned flags[NUM_FLAG_KINDS][MAX_RANKS]
__device__ __forceinline__ unsigned* flag_ptr(void* flags_base, int kind, int rank) {
  return reinterpret_cast<unsigned*>(flags_base) + kind * MAX_RANKS + rank;
}

__device__ unsigned g_wait_budget = 1u << 24;   // polls of ~400 ns each; tests shrink it to provoke a clean expiry

// Bounded wait until every rank's flag of `kind` in OUR arena reaches `seq` (budget: several seconds).
__device__ bool wait_all(void* my_flags, int kind, unsigned seq, int W, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < W && ok; ++r) {
      const unsigned* f = flag_ptr(my_flags, kind, r);
      unsigned it = 0;
      while ((int)(ld_acquire_sys(f) - seq) < 0) {
        if (++it > g_wait_budget) { ok = 0; break; }
        __nanosleep(400);
      }
    }
    if (!ok) atomicExch(status, LLMB_ERR_TIMEOUT);
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}

// The last block to finish stores `seq` into flag (kind, me) of every rank's arena.
__device__ void signal_all_last_block(unsigned* counter, PeerPtrs flags, int kind, int me, unsigned seq, int W) {
  __threadfence_system();                 // this block's peer stores are visible system-wide before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned done = atomicAdd(counter, 1u);
    if (done == gridDim.x - 1) {
      *counter = 0;                       // re-arm for the next launch (stream ordered)
      __threadfence_system();
      for (int r = 0; r < W; ++r) st_release_sys(flag_ptr(flags.p[r], kind, me), seq);
    }
  }
}

__device__ __forceinline__ int find_seg(const SegList& s, long long v) {
  int i = 0;
  while (i + 1 < s.n && v >= s.vec_prefix[i + 1]) ++i;
  return i;
}

__device__ __forceinline__ void load_bf16x8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 t = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  uint4 t; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return t;
}

// ------------------------------------------------------------------ pack
__global__ void __launch_bounds__(512) pack_kernel(__nv_bfloat16* __restrict__ send, const float* __restrict__ src, SegList segs,
                                                  float scale, void* my_flags, PeerPtrs flags, int me, int W,
                                                  unsigned seq, unsigned wait_done_seq, unsigned* counter, int* status) {
  // the previous user of this send buffer must have been consumed by every peer
  if (wait_done_seq && !wait_all(my_flags, FLAG_DONE, wait_done_seq, W, status)) return;
  const long long total = segs.vec_prefix[segs.n];
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const int s = find_seg(segs, v);
    const long long e = (v - segs.vec_prefix[s]) * 8;
    const float4 a = *reinterpret_cast<const float4*>(src + segs.src_off[s] + e);
    const float4 b = *reinterpret_cast<const float4*>(src + segs.src_off[s] + e + 4);
    float x[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale, b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    *reinterpret_cast<uint4*>(send + segs.dst_off[s] + e) = pack_bf16x8(x);
  }
  signal_all_last_block(counter, flags, FLAG_READY, me, seq, W);
}

// ------------------------------------------------------------------ reduce
// mode 0 (reduce-scatter): dst_f32[dst_off + e] (+)= sum_p send_p[src_off + e]; norm partials.
// mode 1 (all-reduce, two-shot): recv_p[src_off + e] = bf16(sum) for every rank p.
template <int WT>   // WT > 0: world size known at compile time (peer loads unrolled and all in flight together); 0: runtime W
__global__ void __launch_bounds__(512) reduce_kernel(PeerPtrs sends, SegList owned, int mode, float* __restrict__ dst_f32,
                                                    int accumulate, PeerPtrs recvs, float* __restrict__ norm_partials,
                                                    void* my_flags, PeerPtrs flags, int me, int W, unsigned seq,
                                                    unsigned wait_done2_seq, unsigned* counter, unsigned* counter2, int* status) {
  if (!wait_all(my_flags, FLAG_READY, seq, W, status)) return;
  if (mode == 1 && wait_done2_seq && !wait_all(my_flags, FLAG_DONE2, wait_done2_seq, W, status)) return;
  const long long total = owned.vec_prefix[owned.n];
  float nsq = 0.f;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const int s = find_seg(owned, v);
    const long long e = (v - owned.vec_prefix[s]) * 8;
    const long long so = owned.src_off[s] + e;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (WT > 0) {
      uint4 raw[WT > 0 ? WT : 1];
#pragma unroll
      for (int r = 0; r < WT; ++r) raw[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(sends.p[r]) + so);
#pragma unroll
      for (int r = 0; r < WT; ++r) {       // fixed rank order: identical bits on every rank
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
      }
    } else {
      for (int r = 0; r < W; ++r) {
        float x[8];
        load_bf16x8(reinterpret_cast<const __nv_bfloat16*>(sends.p[r]) + so, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += x[k];
      }
    }
    if (mode == 0) {
      float* d = dst_f32 + owned.dst_off[s] + e;
      float4 o0 = make_float4(acc[0], acc[1], acc[2], acc[3]), o1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (accumulate) {
        const float4 c0 = *reinterpret_cast<const float4*>(d), c1 = *reinterpret_cast<const float4*>(d + 4);
        o0.x += c0.x; o0.y += c0.y; o0.z += c0.z; o0.w += c0.w; o1.x += c1.x; o1.y += c1.y; o1.z += c1.z; o1.w += c1.w;
      }
      *reinterpret_cast<float4*>(d) = o0; *reinterpret_cast<float4*>(d + 4) = o1;
      nsq += o0.x * o0.x + o0.y * o0.y + o0.z * o0.z + o0.w * o0.w + o1.x * o1.x + o1.y * o1.y + o1.z * o1.z + o1.w * o1.w;
    } else {
      const uint4 packed = pack_bf16x8(acc);
      if (WT > 0) {
#pragma unroll
        for (int r = 0; r < WT; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recvs.p[r]) + so) = packed;
      } else {
        for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recvs.p[r]) + so) = packed;
      }
    }
  }
  if (mode == 0 && norm_partials) {        // sum of squares of the reduced gradients this rank owns
    __shared__ float red[16];
    nsq = warp_sum(nsq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = nsq;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) atomicAdd(norm_partials, t);
    }
  }
  // peers may now overwrite their send buffers; (AR) results are in everybody's receive buffer
  signal_all_last_block(counter, flags, FLAG_DONE, me, seq, W);
  if (mode == 1) signal_all_last_block(counter2, flags, FLAG_READY2, me, seq, W);
}

// ------------------------------------------------------------------ unpack (all-reduce tail)
__global__ void __launch_bounds__(512) unpack_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ recv, SegList segs,
                                                    void* my_flags, PeerPtrs flags, int me, int W, unsigned seq,
                                                    unsigned* counter, int* status) {
  if (!wait_all(my_flags, FLAG_READY2, seq, W, status)) return;
  const long long total = segs.vec_prefix[segs.n];
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const int s = find_seg(segs, v);
    const long long e = (v - segs.vec_prefix[s]) * 8;
    float x[8];
    load_bf16x8(recv + segs.src_off[s] + e, x);
    float* d = dst + segs.dst_off[s] + e;
    *reinterpret_cast<float4*>(d) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(d + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
  signal_all_last_block(counter, flags, FLAG_DONE2, me, seq, W);   // receive buffer may be reused
}

// ------------------------------------------------------------------ ZeRO-3 gather
__global__ void __launch_bounds__(512) gather_kernel(__nv_bfloat16* __restrict__ dst, PeerPtrs shards, SegList segs, void* my_flags,
                                                    int W, unsigned param_seq, int* status) {
  if (param_seq && !wait_all(my_flags, FLAG_PARAM, param_seq, W, status)) return;
  const long long total = segs.vec_prefix[segs.n];
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const int s = find_seg(segs, v);
    const long long e = (v - segs.vec_prefix[s]) * 8;
    const uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(shards.p[segs.owner[s]]) + segs.src_off[s] + e);
    *reinterpret_cast<uint4*>(dst + segs.dst_off[s] + e) = t;
  }
}

// ------------------------------------------------------------------ sharded AdamW + parameter push
__global__ void __launch_bounds__(256) adamw_push_kernel(PeerPtrs params, long long param_off, __nv_bfloat16* __restrict__ shard_copy,
                                                        float* __restrict__ master, const float* __restrict__ grads,
                                                        float* __restrict__ m, float* __restrict__ v, long long n, float lr,
                                                        float beta1, float beta2, float bc1, float bc2, float eps, float wd,
                                                        float grad_scale, const float* __restrict__ dev_scale, int push_w,
                                                        PeerPtrs flags, int me, int W, unsigned seq, unsigned* counter) {
  if (dev_scale) grad_scale *= *dev_scale;
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 8;
    float g[8], mm[8], vv[8], pp[8];
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(grads + e);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(grads + e + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + e);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + e + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + e);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + e + 4);
    *reinterpret_cast<float4*>(pp) = *reinterpret_cast<const float4*>(master + e);
    *reinterpret_cast<float4*>(pp + 4) = *reinterpret_cast<const float4*>(master + e + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gg = g[k] * grad_scale;
      mm[k] = beta1 * mm[k] + (1.f - beta1) * gg;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gg * gg;
      pp[k] -= lr * ((mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps) + wd * pp[k]);
    }
    *reinterpret_cast<float4*>(m + e) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(m + e + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(v + e) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + e + 4) = *reinterpret_cast<float4*>(vv + 4);
    *reinterpret_cast<float4*>(master + e) = *reinterpret_cast<float4*>(pp);
    *reinterpret_cast<float4*>(master + e + 4) = *reinterpret_cast<float4*>(pp + 4);
    const uint4 packed = pack_bf16x8(pp);
    if (shard_copy) *reinterpret_cast<uint4*>(shard_copy + e) = packed;
    for (int r = 0; r < push_w; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + param_off + e) = packed;
  }
  signal_all_last_block(counter, flags, FLAG_PARAM, me, seq, W);
}

// everything this stream wrote so far is visible system-wide before the flag: announces (kind, me) = seq to every rank
__global__ void signal_flags_kernel(PeerPtrs flags, int kind, int me, int W, unsigned seq) {
  __threadfence_system();
  for (int r = 0; r < W; ++r) st_release_sys(flag_ptr(flags.p[r], kind, me), seq);
}

__global__ void wait_flags_kernel(void* my_flags, int kind, unsigned seq, int W, int* status) {
  wait_all(my_flags, kind, seq, W, status);
}

// ------------------------------------------------------------------ scalar all-reduce (sum, rank order)
// scalars layout in an arena: float slots[2][MAX_RANKS] (double-buffered by seq parity)
__global__ void scalar_allreduce_kernel(float* __restrict__ out, const float* __restrict__ in, void* my_scalars, PeerPtrs scalars,
                                        void* my_flags, PeerPtrs flags, int me, int W, unsigned seq, int* status) {
  const int par = seq & 1;
  if (threadIdx.x == 0) {
    const float v = *in;
    for (int r = 0; r < W; ++r) reinterpret_cast<float*>(scalars.p[r])[par * MAX_RANKS + me] = v;
    __threadfence_system();
    for (int r = 0; r < W; ++r) st_release_sys(flag_ptr(flags.p[r], FLAG_SCALAR, me), seq);
  }
  if (!wait_all(my_flags, FLAG_SCALAR, seq, W, status)) return;
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int r = 0; r < W; ++r) s += reinterpret_cast<volatile float*>(my_scalars)[par * MAX_RANKS + r];
    *out = s;
  }
}

// ------------------------------------------------------------------ cross-rank merge of softmax statistics
// Vocabulary-parallel LM head: every rank holds {max, sum-exp, target logit, -} of ITS vocabulary slice for ALL rows in a
// symmetric buffer.  Each rank reads the W copies of a row with peer loads and writes the statistics of the whole
// vocabulary to a local buffer: max over ranks, sum-exps rescaled to it, target logits added (exactly one rank's is
// non-zero).  READY: "my slice's statistics are written"; DONE: "I have read everybody's" (the buffers may be rewritten).
__global__ void __launch_bounds__(256) ce_stats_merge_kernel(float4* __restrict__ out, PeerPtrs stats, long long rows, void* my_flags,
                                                            PeerPtrs flags, int me, int W, unsigned seq, unsigned* counter, int* status) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < W; ++r) st_release_sys(flag_ptr(flags.p[r], FLAG_STATS_READY, me), seq);
  }
  if (!wait_all(my_flags, FLAG_STATS_READY, seq, W, status)) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += (long long)gridDim.x * blockDim.x) {
    float4 v[MAX_RANKS];
    float m = -INFINITY;
    for (int r = 0; r < W; ++r) { v[r] = reinterpret_cast<const float4*>(stats.p[r])[i]; m = fmaxf(m, v[r].x); }
    float sum = 0.f, tgt = 0.f;
    for (int r = 0; r < W; ++r) {
      if (v[r].y > 0.f) sum += v[r].y * expf(v[r].x - m);       // an empty slice has max -inf and sum 0
      tgt += v[r].z;
    }
    out[i] = make_float4(m, sum, tgt, 0.f);
  }
  signal_all_last_block(counter, flags, FLAG_STATS_DONE, me, seq, W);
}

struct SegArgs { int n; const int* owner; const long long* src_off; const long long* dst_off; const long long* len; };
bool fill(SegList& s, int n, const int* owner, const long long* src, const long long* dst, const long long* len) {
  if (n < 0 || n > MAX_SEGS) return false;
  s.n = n; s.vec_prefix[0] = 0;
  for (int i = 0; i < n; ++i) {
    if ((src[i] | dst[i] | len[i]) & 7) return false;
    s.owner[i] = owner ? owner[i] : 0; s.src_off[i] = src[i]; s.dst_off[i] = dst[i]; s.len[i] = len[i];
    s.vec_prefix[i + 1] = s.vec_prefix[i] + len[i] / 8;
  }
  return true;
}
PeerPtrs to_peers(void* const* p, int W) { PeerPtrs o{}; for (int i = 0; i < W && i < MAX_RANKS; ++i) o.p[i] = p[i]; return o; }
int comm_grid(long long vecs, int blocks) { long long need = ceil_div_ll(vecs, 512); if (need < 1) need = 1; return (int)(need < blocks ? need : blocks); }
}  // namespace

// ------------------------------------------------------------------ arena + IPC plumbing
LLMB_API int llmb_comm_max_ranks() { return MAX_RANKS; }
LLMB_API int llmb_comm_flag_bytes() { return NUM_FLAG_KINDS * MAX_RANKS * (int)sizeof(unsigned); }
LLMB_API int llmb_comm_alloc(void** ptr, long long bytes) {
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, (size_t)bytes);
  return (int)e;
}
LLMB_API int llmb_comm_free(void* ptr) { return (int)cudaFree(ptr); }
LLMB_API int llmb_ipc_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h; cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e == cudaSuccess) memcpy(handle64, &h, sizeof(h));
  return (int)e;
}
LLMB_API int llmb_ipc_open(void** ptr, const void* handle64) {
  cudaIpcMemHandle_t h; memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
LLMB_API int llmb_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
LLMB_API int llmb_enable_peer(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
  return (int)e;
}

// ------------------------------------------------------------------ launchers
LLMB_API int llmb_comm_pack(void* send, const float* src, int nseg, const long long* src_off, const long long* dst_off,
                            const long long* len, float scale, void* my_flags, void* const* flag_ptrs, int me, int W,
                            unsigned seq, unsigned wait_done_seq, unsigned* counter, int* status, int blocks, cudaStream_t st) {
  SegList s; if (!fill(s, nseg, nullptr, src_off, dst_off, len)) return LLMB_ERR_BAD_ARG;
  pack_kernel<<<comm_grid(s.vec_prefix[s.n], blocks), 512, 0, st>>>((__nv_bfloat16*)send, src, s, scale, my_flags, to_peers(flag_ptrs, W),
                                                                   me, W, seq, wait_done_seq, counter, status);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_reduce(void* const* send_ptrs, int nseg, const long long* src_off, const long long* dst_off,
                              const long long* len, int mode, float* dst_f32, int accumulate, void* const* recv_ptrs,
                              float* norm_acc, void* my_flags, void* const* flag_ptrs, int me, int W, unsigned seq, unsigned wait_done2_seq,
                              unsigned* counter, unsigned* counter2, int* status, int blocks, cudaStream_t st) {
  SegList s; if (!fill(s, nseg, nullptr, src_off, dst_off, len)) return LLMB_ERR_BAD_ARG;
  const int grid = comm_grid(s.vec_prefix[s.n], blocks);
#define LLMB_REDUCE(WT) reduce_kernel<WT><<<grid, 512, 0, st>>>(to_peers(send_ptrs, W), s, mode, dst_f32, accumulate, \
                          recv_ptrs ? to_peers(recv_ptrs, W) : PeerPtrs{}, norm_acc, my_flags, to_peers(flag_ptrs, W), me, W, seq, \
                          wait_done2_seq, counter, counter2, status)
  switch (W) {
    case 2: LLMB_REDUCE(2); break;
    case 4: LLMB_REDUCE(4); break;
    case 8: LLMB_REDUCE(8); break;
    default: LLMB_REDUCE(0); break;
  }
#undef LLMB_REDUCE
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_unpack(float* dst, const void* recv, int nseg, const long long* src_off, const long long* dst_off,
                              const long long* len, void* my_flags, void* const* flag_ptrs, int me, int W, unsigned seq,
                              unsigned* counter, int* status, int blocks, cudaStream_t st) {
  SegList s; if (!fill(s, nseg, nullptr, src_off, dst_off, len)) return LLMB_ERR_BAD_ARG;
  unpack_kernel<<<comm_grid(s.vec_prefix[s.n], blocks), 512, 0, st>>>(dst, (const __nv_bfloat16*)recv, s, my_flags, to_peers(flag_ptrs, W),
                                                                     me, W, seq, counter, status);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_gather(void* dst, void* const* shard_ptrs, int nseg, const int* owner, const long long* src_off,
                              const long long* dst_off, const long long* len, void* my_flags, int W, unsigned param_seq,
                              int* status, int blocks, cudaStream_t st) {
  SegList s; if (!fill(s, nseg, owner, src_off, dst_off, len)) return LLMB_ERR_BAD_ARG;
  gather_kernel<<<comm_grid(s.vec_prefix[s.n], blocks), 512, 0, st>>>((__nv_bfloat16*)dst, to_peers(shard_ptrs, W), s, my_flags, W, param_seq, status);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_adamw_push(void* const* param_ptrs, long long param_off, void* shard_copy, float* master,
                                  const float* grads, float* m, float* v, long long n, float lr, float beta1, float beta2,
                                  float eps, float wd, float grad_scale, const float* dev_scale, int t, int push_w,
                                  void* const* flag_ptrs, int me, int W, unsigned seq, unsigned* counter, cudaStream_t st) {
  if (n % 8 || param_off % 8) return LLMB_ERR_BAD_ARG;
  const float bc1 = 1.f - powf(beta1, (float)t), bc2 = 1.f - powf(beta2, (float)t);
  long long blocks = ceil_div_ll(n / 8, 256);
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (grid < 1) grid = 1;
  adamw_push_kernel<<<grid, 256, 0, st>>>(to_peers(param_ptrs, push_w), param_off, (__nv_bfloat16*)shard_copy, master, grads, m, v, n, lr,
                                         beta1, beta2, bc1, bc2, eps, wd, grad_scale, dev_scale, push_w, to_peers(flag_ptrs, W), me, W, seq, counter);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_set_wait_budget(unsigned polls) {
  return (int)cudaMemcpyToSymbol(g_wait_budget, &polls, sizeof(polls));
}
LLMB_API int llmb_comm_signal(void* const* flag_ptrs, int kind, int me, int W, unsigned seq, cudaStream_t st) {
  signal_flags_kernel<<<1, 1, 0, st>>>(to_peers(flag_ptrs, W), kind, me, W, seq);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_wait(void* my_flags, int kind, unsigned seq, int W, int* status, cudaStream_t st) {
  wait_flags_kernel<<<1, 32, 0, st>>>(my_flags, kind, seq, W, status);
  return (int)cudaGetLastError();
}
// out [rows] float4 (local) = statistics merged over the W ranks' symmetric `stats` buffers; see ce_stats_merge_kernel
LLMB_API int llmb_comm_ce_stats_merge(void* out, void* const* stats_ptrs, long long rows, void* my_flags, void* const* flag_ptrs,
                                      int me, int W, unsigned seq, unsigned* counter, int* status, int blocks, cudaStream_t st) {
  if (rows <= 0 || W < 1 || W > MAX_RANKS) return LLMB_ERR_BAD_ARG;
  long long need = ceil_div_ll(rows, 256);
  const int grid = (int)(need < blocks ? need : blocks);
  ce_stats_merge_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<float4*>(out), to_peers(stats_ptrs, W), rows, my_flags,
                                              to_peers(flag_ptrs, W), me, W, seq, counter, status);
  return (int)cudaGetLastError();
}
LLMB_API int llmb_comm_scalar_allreduce(float* out, const float* in, void* my_scalars, void* const* scalar_ptrs, void* my_flags,
                                        void* const* flag_ptrs, int me, int W, unsigned seq, int* status, cudaStream_t st) {
  scalar_allreduce_kernel<<<1, 32, 0, st>>>(out, in, my_scalars, to_peers(scalar_ptrs, W), my_flags, to_peers(flag_ptrs, W), me, W, seq, status);
  return (int)cudaGetLastError();
}
