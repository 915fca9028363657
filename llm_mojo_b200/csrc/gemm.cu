// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  D[M,N] = epilogue(A[M,K] · B[N,K]^T).
//
// Covers every linear-layer GEMM of the trainer (reference call sites: llmm/matmul.mojo:463-696
// forward + bias / bias+GELU epilogues, :2789-2938 dinp with the dGELU epilogue, :3231-3509 dW
// with beta=1 accumulate, :3671-3908 LM head; all of them cuBLASLt calls in the reference).
//
// Design (one CTA per SM, 192 threads):
//   warp 0   TMA producer: streams 128x(128 B) A tiles and 256x(128 B) B tiles through a
//            4-stage shared-memory ring (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma 128x256xK_mma into one of two
//            256-column TMEM accumulators and commits stage / accumulator mbarriers
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (each warp its own 32-lane TMEM
//            quarter), apply bias / GELU / dGELU / fp32 accumulate, store 16-byte vectors
// so the epilogue of tile i overlaps the main loop of tile i+1.  Operands may be K-major or
// MN-major (the UMMA descriptor and the TMA box change, not the data), which is how dinp
// (B = W as stored) and dW (A = dout^T, B = inp^T as stored) run without any transposes.
// Split-K work units reduce through fp32 red.global.add into the (fp32) gradient buffer.
//
// Three kernels share these parts: gemm_kernel (the design above, kept as the single-CTA comparator),
// gemm_pair_kernel (the default: two CTAs per 256 x 256 tile with cta_group::2 MMAs, eight epilogue warps, TMA-store
// epilogue, optional all-gather of A from peer GPUs and optional column sums of the result) and gemm_nvfp4_kernel
// (block-scaled NVFP4 / MXFP8 operands with their scales in tensor memory, 128 x 256 tiles); each is described where
// it is defined.
#include <stdlib.h>
#include "tc05.cuh"
using namespace llmb;
using namespace tc05;

namespace {
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint4 ld_nc_v4(const uint4* p) {     // streaming 16-byte load (peer memory: read once)
  uint4 v; asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
constexpr int BM = 128, BN = 256;
constexpr int STAGES = 4;
constexpr int ROW_BYTES = 128;                       // one swizzled row
constexpr int A_STAGE = BM * ROW_BYTES;              // 16 KB
constexpr int B_STAGE = BN * ROW_BYTES;              // 32 KB
constexpr int STAGE_BYTES = A_STAGE + B_STAGE;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * 32 * 256 /*epilogue transpose*/ + 1024 /*align*/ + 256 /*barriers*/;
constexpr int BAND = 16;                             // m-tiles per rasterisation band

enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_DGELU = 3, EPI_ACC_F32 = 4, EPI_BIAS_RESID = 5, EPI_STORE_F32 = 6 };

// All-gather fused into the GEMM: the A matrix [W*n, K] is the concatenation of W row chunks, chunk r produced by
// rank r.  Every rank holds a full-size local buffer whose own chunk is already in place; two copier warps per
// CTA pull the other chunks out of the peers' buffers (plain 16-byte peer loads over NVLink, each byte crosses
// once) into the local buffer WHILE the tile loop runs, starting with the tiles of the local chunk and taking the
// remote chunks in ring order.  A chunk's tiles are fetched (TMA, local memory) once every CTA's copiers have
// counted it complete.
struct GatherArgs {
  const void* peer_src[8];     // [r]: start of chunk r inside rank r's buffer
  void* local;                 // start of this rank's [W*n, K] buffer
  const void* flags;           // this rank's flag words: peers announce "my chunk is written" (kind ROWS_READY)
  unsigned* counts;            // [16] local counters, zeroed before the launch: [r] = slices of chunk r copied, [8 + r] = slice tickets
  long long chunk_vecs;        // 16-byte vectors per chunk
  unsigned seq, target;        // announce sequence number to wait for; slices per chunk (counts[r] == target: chunk landed)
  int W, me, tiles_per_chunk;  // W = 0: no gather
};

// Parameter pull fused into a GEMM (ZeRO-3): the kernel's copier warps copy up to 8 segments of weights out of their
// owners' parameter shards (plain 16-byte loads over NVLink, or local memory for the rank's own part) into this
// rank's layer window while the tensor-core tile loop of the SAME kernel runs.  The segments may belong to the B
// operand of this GEMM (then its TMA producer waits for them) or to the operand of a later GEMM of the layer, which
// only checks the counters: every weight then arrives under the math of a tile loop.  Owners announce "my shard
// holds the parameters of optimizer step seq" at flag kind PARAM; all waits are bounded.
struct PullArgs {
  const void* src[8];          // segment source (peer or local shard memory), 16-byte aligned
  void* dst[8];                // segment destination inside the local window
  long long vecs[8];           // 16-byte vectors per segment
  const void* flags;           // this rank's flag words
  unsigned* counts;            // [16] zeroed before the launch: [s] = slices of segment s landed, [8 + s] = slice tickets
  const unsigned* wait_counts[8];   // counters this GEMM's B operand depends on ...
  unsigned wait_target[8];          // ... and the value each must reach
  unsigned seq;                // parameter sequence number the owners must have announced (0: none yet, no wait)
  int owner[8];
  int nseg, nwait, W;          // nseg = 0: nothing to pull; nwait = 0: nothing to wait for
};

struct GemmParams {
  GatherArgs g;
  PullArgs pull;
  void* D; const void* bias; void* aux; const float* alpha;
  int M, N, K;                 // K in elements
  long long ldd, ldaux;
  int a_mn, b_mn;              // operand majorness (0 = K-major)
  int a_3d, b_3d;              // MN-major operand fetched with ONE 3-D box (chunk, k, chunk index) per stage
  uint32_t a_lbo, a_sbo, a_kstep, b_lbo, b_sbo, b_kstep;   // bytes
  uint32_t a_layout, b_layout; // UMMA layout type: 2 = SWIZZLE_128B, 1 = SWIZZLE_128B with 32-byte base (fp32 MN-major)
  uint32_t idesc;
  int bke;                     // K elements per stage
  int m_tiles, n_tiles, splits, kb_per_split, kb_total;
  int io_f32;                  // 1: D, bias and aux are fp32 (tf32 kind); 0: bf16
  int tma_epi;                 // 1: bf16 outputs leave (and auxiliary inputs arrive) by TMA; 0: register/shared-memory epilogue
  int bias_vec;                // bias pointer is 16-byte aligned (vector loads)
  float* colsum;               // EPI_DGELU, TMA epilogue: colsum[n] += sum over rows of the (bf16) result, i.e. the bias gradient of the layer below
  int dbg;                     // measurement switches: 1 = drain accumulators without storing, 2 = always fetch tile (0,0), 8 = skip the GELU math
  int* status;
};

// ------------------------------------------------------------------------------------------------
// Coalesced epilogue.  tcgen05.ld hands each thread one accumulator ROW; stored directly, a warp
// would touch 32 different rows per instruction.  Instead every 64-column slab of the warp's
// 32 x 256 block goes through an 8 KB shared-memory transpose (XOR-swizzled 16-byte chunks, conflict
// free in both directions) so that 8 consecutive lanes cover 64 contiguous bytes of one output row
// and all global traffic of the epilogue (output, bias, GELU aux, residual) is sector-aligned.
constexpr int EPI_STAGE_BYTES = 32 * 256;             // per epilogue warp: 32 rows x 64 fp32

template <int EPI>
__device__ __forceinline__ void epi4(const GemmParams& p, float (&v)[4], int row, int col, float alpha) {
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] *= alpha;
  if (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU || EPI == EPI_BIAS_RESID) {
    if (p.bias && p.io_f32) {
      const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + col);
      v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    } else if (p.bias) {
      const uint2 braw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.bias) + col);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&braw);
      const float2 b0 = __bfloat1622float2(bh[0]), b1 = __bfloat1622float2(bh[1]);
      v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y;
    }
  }
  if (EPI == EPI_ACC_F32 || EPI == EPI_STORE_F32) {
    float* dp = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + col;
    if (EPI == EPI_ACC_F32)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
    else
      *reinterpret_cast<float4*>(dp) = make_float4(v[0], v[1], v[2], v[3]);
    return;
  }
  if (p.io_f32) {                                       // fp32 storage (tf32 tensor path)
    float* dp = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + col;
    float* ap = reinterpret_cast<float*>(p.aux) + (size_t)row * p.ldaux + col;
    if (EPI == EPI_BIAS_GELU) {
      *reinterpret_cast<float4*>(ap) = make_float4(v[0], v[1], v[2], v[3]);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = gelu_f(v[k]);
    } else if (EPI == EPI_DGELU) {
      const float4 x = *reinterpret_cast<const float4*>(ap);
      v[0] *= gelu_grad_f(x.x); v[1] *= gelu_grad_f(x.y); v[2] *= gelu_grad_f(x.z); v[3] *= gelu_grad_f(x.w);
    } else if (EPI == EPI_BIAS_RESID) {
      const float4 x = *reinterpret_cast<const float4*>(ap);
      v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
    }
    *reinterpret_cast<float4*>(dp) = make_float4(v[0], v[1], v[2], v[3]);
    return;
  }
  __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + (size_t)row * p.ldd + col;
  __nv_bfloat16* ap = reinterpret_cast<__nv_bfloat16*>(p.aux) + (size_t)row * p.ldaux + col;
  auto pack4 = [](const float (&x)[4]) {
    uint2 u; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
    h[0] = __floats2bfloat162_rn(x[0], x[1]); h[1] = __floats2bfloat162_rn(x[2], x[3]);
    return u;
  };
  auto unpack4 = [](uint2 u, float (&x)[4]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  };
  if (EPI == EPI_BIAS_GELU) {
    const uint2 pre = pack4(v);
    *reinterpret_cast<uint2*>(ap) = pre;               // pre-GELU activations (bf16)
    float x[4]; unpack4(pre, x);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = gelu_f(x[k]);
  } else if (EPI == EPI_DGELU) {
    float x[4]; unpack4(*reinterpret_cast<const uint2*>(ap), x);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] *= gelu_grad_f(x[k]);
  } else if (EPI == EPI_BIAS_RESID) {
    float x[4]; unpack4(*reinterpret_cast<const uint2*>(ap), x);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] += x[k];
  }
  const uint2 o = pack4(v);
  if (p.dbg & 4) asm volatile("st.global.cs.v2.b32 [%0], {%1, %2};" ::"l"(dp), "r"(o.x), "r"(o.y) : "memory");   // streaming store (measurement switch)
  else *reinterpret_cast<uint2*>(dp) = o;
}

// One epilogue warp drains its 32 rows x NCOLS columns of accumulator `tacc` (TMEM address incl. lane quarter).
template <int EPI, int NCOLS = BN>
__device__ __forceinline__ void epilogue_warp(const GemmParams& p, uint32_t tacc, unsigned char* stage, int row_base, int n0,
                                              float alpha, int lane) {
  const int rsub = lane >> 3, cl = lane & 7;
#pragma unroll 1
  for (int s = 0; s < NCOLS / 64; ++s) {
    if (n0 + s * 64 >= p.N) break;                      // warp-uniform
    uint32_t r0[32], r1[32];
    tmem_ld32(tacc + s * 64, r0);
    tmem_ld32(tacc + s * 64 + 32, r1);
    tmem_wait_ld();
    unsigned char* myrow = stage + lane * 256;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      *reinterpret_cast<uint4*>(myrow + ((c ^ (lane & 15)) << 4)) = make_uint4(r0[4 * c], r0[4 * c + 1], r0[4 * c + 2], r0[4 * c + 3]);
      *reinterpret_cast<uint4*>(myrow + (((c + 8) ^ (lane & 15)) << 4)) = make_uint4(r1[4 * c], r1[4 * c + 1], r1[4 * c + 2], r1[4 * c + 3]);
    }
    __syncwarp();
    if (!(p.dbg & 1)) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rr = it * 4 + rsub;
        const int row = row_base + rr;
        const unsigned char* src = stage + rr * 256;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int chunk = cl + half * 8;
          const float4 f = *reinterpret_cast<const float4*>(src + ((chunk ^ (rr & 15)) << 4));
          const int col = n0 + s * 64 + chunk * 4;
          if (row < p.M && col < p.N) {
            float v[4] = {f.x, f.y, f.z, f.w};
            epi4<EPI>(p, v, row, col, alpha);
          }
        }
      }
    }
    __syncwarp();
  }
}

template <int KIND, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_stage = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + 4 * 32 * 256);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;      // [2] accumulator ready
  uint64_t* tempty_bar = tfull_bar + 2;          // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_split = p.m_tiles * p.n_tiles;
  const int total_units = tiles_per_split * p.splits;

  auto unit_coords = [&](int unit, int& m_blk, int& n_blk, int& kb0, int& kb1) {
    int split = unit / tiles_per_split, t = unit % tiles_per_split;
    int band_sz = BAND * p.n_tiles;
    int b = t / band_sz, r = t % band_sz;
    int m_in_band = min(BAND, p.m_tiles - b * BAND);
    m_blk = b * BAND + r % m_in_band;
    n_blk = r / m_in_band;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x) {
        int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
          unsigned char* sa = smem + stage * STAGE_BYTES;
          unsigned char* sb = sa + A_STAGE;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = kb * p.bke;
          if (!p.a_mn) tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          else if (p.a_3d) tma_load_3d(sa, &tmA, &full_bar[stage], 0, k0, m0 / p.bke);
          else {
            const int chunk_elems = p.bke;   // elements per 128-byte row
            const int nchunk = BM / chunk_elems;
            for (int c = 0; c < nchunk; ++c) tma_load_2d(sa + c * p.bke * ROW_BYTES, &tmA, &full_bar[stage], m0 + c * chunk_elems, k0);
          }
          if (!p.b_mn) tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          else if (p.b_3d) tma_load_3d(sb, &tmB, &full_bar[stage], 0, k0, n0 / p.bke);
          else {
            const int chunk_elems = p.bke;
            const int nchunk = BN / chunk_elems;
            for (int c = 0; c < nchunk; ++c) tma_load_2d(sb + c * p.bke * ROW_BYTES, &tmB, &full_bar[stage], n0 + c * chunk_elems, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // warp-uniform loop, one elected lane issues; descriptors of stage 0 and the per-MMA increments are hoisted
    {
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      const uint64_t adesc0 = make_smem_desc(smem_u32(smem), p.a_lbo, p.a_sbo, p.a_layout);
      const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + A_STAGE, p.b_lbo, p.b_sbo, p.b_layout);
      const uint64_t a_inc = (uint64_t)(p.a_kstep >> 4), b_inc = (uint64_t)(p.b_kstep >> 4);
      const uint32_t idesc = p.idesc;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x, ++it) {
        int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          fence_after_sync();
          const uint64_t adesc = adesc0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
          if (elect_one()) {
            umma_ss<KIND>(d_tmem, adesc, bdesc, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < 4; ++k) umma_ss<KIND>(d_tmem, adesc + k * a_inc, bdesc + k * b_inc, idesc, 1u);
            umma_commit(&empty_bar[stage]);   // stage reusable once these MMAs have read it
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(&tfull_bar[acc]);
        __syncwarp();
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    int it = 0;
    for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x, ++it) {
      int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
      fence_after_sync();
      const int n0 = n_blk * BN;
      const float alpha = p.alpha ? *p.alpha : 1.0f;
      epilogue_warp<EPI>(p, tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN, epi_stage + (warp - 2) * EPI_STAGE_BYTES,
                         m_blk * BM + q * 32, n0, alpha, lane);
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc<512>(tmem_base); }
}


// ------------------------------------------------------------------------------------------------
// Epilogue through TMA (bf16 outputs of the CTA-pair kernel).  Each of the eight epilogue warps owns
// 32 rows x 128 columns of the accumulator and moves them as two slabs of 64 columns = one
// 128-byte-swizzled box of 32 rows x 128 B (4 KB) each:
//   * tcgen05.ld gives each lane one row of the slab; bias, GELU, dGELU and the residual add happen in
//     registers in that layout;
//   * the auxiliary INPUT (residual stream, pre-GELU activations) arrives by TMA loads that are issued a
//     whole tile ahead - while the tensor core is still busy with that tile - into the buffer the
//     result is then written to in place;
//   * results leave by TMA stores (bulk groups), so no lane ever waits on global memory and every
//     global access of the epilogue is a full 128-byte row segment; out-of-range rows and columns are
//     clipped by the tensor maps.
// Epilogues with an auxiliary input or a second output (BIAS_GELU stores the pre-activation too) get
// two 4 KB buffers per warp and a 5-deep operand ring, and so do the fp32 outputs (two 32-column boxes of a 64-column slab,
// added into or stored to global memory by TMA); the others one buffer and a 6-deep ring.
template <int EPI> struct EpiCfg {
  static constexpr bool AUX_IN = EPI == EPI_DGELU || EPI == EPI_BIAS_RESID;
  static constexpr bool TWO_OUT = EPI == EPI_BIAS_GELU;
  static constexpr bool F32_OUT = EPI == EPI_ACC_F32 || EPI == EPI_STORE_F32;
  static constexpr int STAGES = (F32_OUT || AUX_IN || TWO_OUT) ? 5 : 6;
  static constexpr int WARP_STAGE = STAGES == 5 ? 16384 : 8192;     // staging bytes per warp of the 4-warp register epilogue (half that per warp of the 8-warp TMA epilogue)
};
constexpr int SLAB_BYTES = 32 * 128;

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 u; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
  return u;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}

// One slab (this lane's row, 64 columns) from registers to the swizzled staging buffer.  With an
// auxiliary input the buffer holds it on entry and the result replaces it; BIAS_GELU writes the
// pre-activation to `buf` and the activation to `buf + SLAB_BYTES`.
template <int EPI>
__device__ __forceinline__ void epi_slab_bf16(const GemmParams& p, const uint32_t (&r0)[32], const uint32_t (&r1)[32],
                                              unsigned char* buf, int col0, float alpha, int lane) {
  unsigned char* myrow = buf + lane * 128;
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float v[8], b[8];
    const int col = col0 + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = 0.f;
    if (EPI == EPI_BIAS || EPI == EPI_BIAS_GELU || EPI == EPI_BIAS_RESID) {
      if (bias && col < p.N) {
        if (p.bias_vec) unpack8(__ldg(reinterpret_cast<const uint4*>(bias + col)), b);
        else {
#pragma unroll
          for (int j = 0; j < 8; ++j) b[j] = __bfloat162float(bias[col + j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const uint32_t (&r)[32] = c < 4 ? r0 : r1;
      const float2 y = __ffma2_rn(make_float2(__uint_as_float(r[(c & 3) * 8 + j]), __uint_as_float(r[(c & 3) * 8 + j + 1])),
                                  make_float2(alpha, alpha), make_float2(b[j], b[j + 1]));
      v[j] = y.x; v[j + 1] = y.y;
    }
    unsigned char* slot = myrow + ((c ^ (lane & 7)) << 4);
    if (EPI == EPI_BIAS_GELU) {
      const uint4 pre = pack8(v);
      *reinterpret_cast<uint4*>(slot) = pre;
      float x[8]; unpack8(pre, x);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float2 y = (p.dbg & 8) ? make_float2(x[j], x[j + 1]) : gelu_fast2(make_float2(x[j], x[j + 1]));
        v[j] = y.x; v[j + 1] = y.y;
      }
      *reinterpret_cast<uint4*>(slot + SLAB_BYTES) = pack8(v);
    } else {
      if (EPI == EPI_DGELU || EPI == EPI_BIAS_RESID) {
        float x[8]; unpack8(*reinterpret_cast<const uint4*>(slot), x);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float2 xx = make_float2(x[j], x[j + 1]), vv = make_float2(v[j], v[j + 1]);
          const float2 y = (EPI == EPI_DGELU) ? __fmul2_rn(vv, gelu_grad_fast2(xx)) : __fadd2_rn(vv, xx);
          v[j] = y.x; v[j + 1] = y.y;
        }
      }
      *reinterpret_cast<uint4*>(slot) = pack8(v);
    }
  }
}

// The two halves of the bias + GELU epilogue, so that the pre-activation box can start leaving by TMA while the GELU of the
// same slab is still being computed: first alpha, bias and the bf16 pre-activations (kept in registers as well) ...
__device__ __forceinline__ void epi_slab_pre(const GemmParams& p, const uint32_t (&r0)[32], const uint32_t (&r1)[32],
                                             unsigned char* buf, int col0, float alpha, int lane, uint4 (&pre)[8]) {
  unsigned char* myrow = buf + lane * 128;
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float v[8], b[8];
    const int col = col0 + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) b[j] = 0.f;
    if (bias && col < p.N) {
      if (p.bias_vec) unpack8(__ldg(reinterpret_cast<const uint4*>(bias + col)), b);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) b[j] = __bfloat162float(bias[col + j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const uint32_t (&r)[32] = c < 4 ? r0 : r1;
      const float2 y = __ffma2_rn(make_float2(__uint_as_float(r[(c & 3) * 8 + j]), __uint_as_float(r[(c & 3) * 8 + j + 1])),
                                  make_float2(alpha, alpha), make_float2(b[j], b[j + 1]));
      v[j] = y.x; v[j + 1] = y.y;
    }
    pre[c] = pack8(v);
    *reinterpret_cast<uint4*>(myrow + ((c ^ (lane & 7)) << 4)) = pre[c];
  }
}
// ... then GELU of those bf16 values into the second box.
__device__ __forceinline__ void epi_slab_gelu(const GemmParams& p, const uint4 (&pre)[8], unsigned char* buf, int lane) {
  unsigned char* myrow = buf + lane * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float x[8]; unpack8(pre[c], x);
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const float2 y = (p.dbg & 8) ? make_float2(x[j], x[j + 1]) : gelu_fast2(make_float2(x[j], x[j + 1]));
      x[j] = y.x; x[j + 1] = y.y;
    }
    *reinterpret_cast<uint4*>(myrow + ((c ^ (lane & 7)) << 4)) = pack8(x);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes a 256 x 256 tile with cta_group::2 MMAs.  Each
// CTA stages its own 128 rows of A and its own 128-row half of B (half the B traffic per SM, and
// a ring of 32 KB stages instead of 48 KB ones), the leader issues the MMAs, and both
// CTAs drain their 128 x 256 accumulator halves.  No load is multicast: every CTA fetches only
// the tiles it owns; the peer's TMA completions are reported to the leader's mbarrier.
constexpr int B2_STAGE = 128 * ROW_BYTES;             // 16 KB: this CTA's half of the B tile
constexpr int STAGE2_BYTES = A_STAGE + B2_STAGE;      // 32 KB
constexpr int PAIR_THREADS = 384;                      // TMA producer, MMA issuer, 8 epilogue warps, 2 gather copier warps
constexpr int FLAG_ROWS_READY = 6;                     // flag kind (layout of comm.cu: flags[kind][8 ranks])
constexpr int FLAG_PARAM = 3;                          // owners announce the optimizer step their parameter shard holds
constexpr int SMEM2_TAIL = 512;                        // barriers, TMEM slot, abort flag
template <int EPI> constexpr int smem2_bytes() { return EpiCfg<EPI>::STAGES * STAGE2_BYTES + 4 * EpiCfg<EPI>::WARP_STAGE + 1024 + SMEM2_TAIL; }

template <int KIND, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, const GemmParams p) {
  using Cfg = EpiCfg<EPI>;
  constexpr int NST = Cfg::STAGES;
  constexpr int WSB = Cfg::WARP_STAGE;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_stage = smem + NST * STAGE2_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + 4 * WSB);
  uint64_t* empty_bar = full_bar + NST;
  uint64_t* tfull_bar = empty_bar + NST;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* aux_bar = tempty_bar + 2;                   // [8 warps][2 slabs] auxiliary-input tiles landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t cta = cluster_ctarank();              // 0 = leader
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 16); }   // 8 warps x 2 CTAs
    for (int a = 0; a < 16; ++a) mbar_init(&aux_bar[a], 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (p.tma_epi) { prefetch_tmap(&tmD); prefetch_tmap(&tmAux); }
  }
  if (warp == 1) tmem_alloc_pair<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                   // both CTAs' barriers exist before any remote signal
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = ceil_div(p.M, 2 * BM);            // cluster tiles of 256 rows
  const int tiles_per_split = m_tiles * p.n_tiles;
  const int total_units = tiles_per_split * p.splits;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  constexpr int BAND2 = 8;

  auto unit_coords = [&](int unit, int& m_blk, int& n_blk, int& kb0, int& kb1) {
    int split = unit / tiles_per_split, t = unit % tiles_per_split;
    int band_sz = BAND2 * p.n_tiles;
    int b = t / band_sz, r = t % band_sz;
    int m_in_band = min(BAND2, m_tiles - b * BAND2);
    m_blk = b * BAND2 + r % m_in_band;
    n_blk = r / m_in_band;
    if (p.g.W > 1) m_blk = (m_blk + p.g.me * p.g.tiles_per_chunk) % m_tiles;   // the local chunk's tiles come first
    kb0 = split * p.kb_per_split;
    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    // warp-uniform loop, one elected lane issues (same reasoning as for the MMA issuer below)
    {
      int stage = 0; uint32_t phase = 0;
      const uint32_t lead_full0 = mapa_u32(smem_u32(&full_bar[0]), 0);
      bool ok = true;
      int landed = -1;
      // B operand pulled from peers (by this kernel's copier warps or by an earlier kernel's): all of it must have landed
      for (int w = 0; w < p.pull.nwait && ok; ++w) {
        unsigned spins = 0;
        while ((int)(ld_acquire_gpu(p.pull.wait_counts[w]) - p.pull.wait_target[w]) < 0) {
          if (++spins > (1u << 24)) { ok = false; break; }
          __nanosleep(100);
        }
      }
      if (p.pull.nwait) fence_proxy_async_all();          // the copiers' generic-proxy stores before this warp's TMA reads
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
      for (int unit = cluster_id; unit < total_units && ok && !*abort_flag; unit += num_clusters) {
        int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
        int m0 = m_blk * 2 * BM + (int)cta * BM, n0 = n_blk * BN + (int)cta * 128;
        if (p.dbg & 2) { m0 = (int)cta * BM; n0 = (int)cta * 128; }
        if (p.g.W > 1) {                                 // gathered A: this tile's chunk must have landed in local memory
          const int chunk = m_blk / p.g.tiles_per_chunk;
          if (chunk != p.g.me && chunk != landed) {
            unsigned spins = 0;
            while ((int)(ld_acquire_gpu(&p.g.counts[chunk]) - p.g.target) < 0) {
              if (++spins > (1u << 24)) { ok = false; break; }
              __nanosleep(100);
            }
            if (!ok) break;
            fence_proxy_async_all();                      // the copiers' generic-proxy stores before this warp's TMA reads
            landed = chunk;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
          unsigned char* sa = smem + stage * STAGE2_BYTES;
          unsigned char* sb = sa + A_STAGE;
          const uint32_t lead_full = lead_full0 + stage * 8;
          const int k0 = (p.dbg & 2) ? 0 : kb * p.bke;
          if (elect_one()) {
            if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE2_BYTES);     // bytes of both CTAs
            if (!p.a_mn) tma_load_2d_pair(sa, &tmA, lead_full, k0, m0);
            else if (p.a_3d) tma_load_3d_pair(sa, &tmA, lead_full, 0, k0, m0 / p.bke);
            else {
              const int chunk_elems = p.bke, nchunk = BM / chunk_elems;
              for (int c = 0; c < nchunk; ++c) tma_load_2d_pair(sa + c * p.bke * ROW_BYTES, &tmA, lead_full, m0 + c * chunk_elems, k0);
            }
            if (!p.b_mn) tma_load_2d_pair(sb, &tmB, lead_full, k0, n0);
            else if (p.b_3d) tma_load_3d_pair(sb, &tmB, lead_full, 0, k0, n0 / p.bke);
            else {
              const int chunk_elems = p.bke, nchunk = 128 / chunk_elems;
              for (int c = 0; c < nchunk; ++c) tma_load_2d_pair(sb + c * p.bke * ROW_BYTES, &tmB, lead_full, n0 + c * chunk_elems, k0);
            }
          }
          __syncwarp();
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    // The whole warp walks the loop (uniform control flow, so descriptors and barrier addresses stay in
    // uniform registers) and one elected lane issues.  Everything that does not change per k-block is
    // computed once: the descriptors of stage 0 (a later stage only adds its byte offset >> 4 to the
    // address field), the per-MMA descriptor increments and the cluster addresses of the barriers.
    if (leader) {
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      const uint64_t adesc0 = make_smem_desc(smem_u32(smem), p.a_lbo, p.a_sbo, p.a_layout);
      const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + A_STAGE, p.b_lbo, p.b_sbo, p.b_layout);
      const uint64_t a_inc = (uint64_t)(p.a_kstep >> 4), b_inc = (uint64_t)(p.b_kstep >> 4);
      const uint32_t idesc = p.idesc;
      const uint32_t eb0 = mapa_u32(smem_u32(&empty_bar[0]), 0), eb1 = mapa_u32(smem_u32(&empty_bar[0]), 1);
      const uint32_t tb0 = mapa_u32(smem_u32(&tfull_bar[0]), 0), tb1 = mapa_u32(smem_u32(&tfull_bar[0]), 1);
      bool ok = true;
      for (int unit = cluster_id; unit < total_units && !*abort_flag; unit += num_clusters, ++it) {
        int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          fence_after_sync();
          const uint64_t adesc = adesc0 + (uint64_t)(stage * (STAGE2_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(stage * (STAGE2_BYTES >> 4));
          if (elect_one()) {
            umma_ss_pair<KIND>(d_tmem, adesc, bdesc, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < 4; ++k) umma_ss_pair<KIND>(d_tmem, adesc + k * a_inc, bdesc + k * b_inc, idesc, 1u);
            umma_commit_pair(eb0 + stage * 8);            // stage free in both CTAs once these MMAs have read it
            umma_commit_pair(eb1 + stage * 8);
          }
          __syncwarp();
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) {
          umma_commit_pair(tb0 + acc * 8);
          umma_commit_pair(tb1 + acc * 8);
        }
        __syncwarp();
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------ gather copiers (warps 10, 11, both CTAs)
    if (p.g.W > 1) {
      // Slices of 32 KB are handed out by ticket, so the copy completes with whatever CTAs are resident.
      constexpr long long SLICE = 2048;                  // 16-byte vectors
      bool ok = true;
      for (int step = 1; step < p.g.W && ok; ++step) {
        const int r = (p.g.me + step) % p.g.W;
        // rank r has announced that its chunk is complete (bounded wait, one lane polls)
        if (lane == 0) {
          const unsigned* f = reinterpret_cast<const unsigned*>(p.g.flags) + FLAG_ROWS_READY * 8 + r;
          unsigned spins = 0;
          while ((int)(ld_acquire_sys(f) - p.g.seq) < 0) {
            if (++spins > (1u << 24)) { ok = false; break; }
            __nanosleep(200);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint4* src = reinterpret_cast<const uint4*>(p.g.peer_src[r]);
        uint4* dst = reinterpret_cast<uint4*>(p.g.local) + (long long)r * p.g.chunk_vecs;
        for (;;) {
          unsigned ticket = 0;
          if (lane == 0) ticket = atomicAdd(&p.g.counts[8 + r], 1u);
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket >= p.g.target) break;
          const long long v0 = (long long)ticket * SLICE;
          const long long v1 = v0 + SLICE < p.g.chunk_vecs ? v0 + SLICE : p.g.chunk_vecs;
          long long v = v0 + lane;
          for (; v + 7 * 32 < v1; v += 8 * 32) {         // eight peer loads in flight per thread
            uint4 t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = ld_nc_v4(src + v + k * 32);
#pragma unroll
            for (int k = 0; k < 8; ++k) dst[v + k * 32] = t[k];
          }
          for (; v < v1; v += 32) dst[v] = ld_nc_v4(src + v);
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(&p.g.counts[r], 1u);
        }
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
    } else if (p.pull.nseg > 0) {
      // ZeRO-3 parameter pull: same ticketed 32 KB slices, one list of segments instead of one chunk per rank
      constexpr long long SLICE = 2048;                  // 16-byte vectors
      bool ok = true;
      for (int sgm = 0; sgm < p.pull.nseg && ok; ++sgm) {
        if (p.pull.seq && lane == 0) {                    // the owner's shard holds this step's parameters
          const unsigned* f = reinterpret_cast<const unsigned*>(p.pull.flags) + FLAG_PARAM * 8 + p.pull.owner[sgm];
          unsigned spins = 0;
          while ((int)(ld_acquire_sys(f) - p.pull.seq) < 0) {
            if (++spins > (1u << 24)) { ok = false; break; }
            __nanosleep(200);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint4* src = reinterpret_cast<const uint4*>(p.pull.src[sgm]);
        uint4* dst = reinterpret_cast<uint4*>(p.pull.dst[sgm]);
        const long long nvec = p.pull.vecs[sgm];
        const unsigned target = (unsigned)((nvec + SLICE - 1) / SLICE);
        for (;;) {
          unsigned ticket = 0;
          if (lane == 0) ticket = atomicAdd(&p.pull.counts[8 + sgm], 1u);
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket >= target) break;
          const long long v0 = (long long)ticket * SLICE;
          const long long v1 = v0 + SLICE < nvec ? v0 + SLICE : nvec;
          long long v = v0 + lane;
          for (; v + 7 * 32 < v1; v += 8 * 32) {         // eight loads in flight per thread
            uint4 t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = ld_nc_v4(src + v + k * 32);
#pragma unroll
            for (int k = 0; k < 8; ++k) dst[v + k * 32] = t[k];
          }
          for (; v < v1; v += 32) dst[v] = ld_nc_v4(src + v);
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(&p.pull.counts[sgm], 1u);
        }
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    // Eight warps: warp % 4 selects the 32-row band (the TMEM lane quarter a warp may read), (warp - 2) / 4 the
    // 128-column half of the tile, i.e. two 64-column slabs per warp and tile.  The register epilogue (fp32
    // outputs, layouts without a tensor map) keeps four working warps with all four slabs of a band each.
    const int q = warp & 3, e = warp - 2, hcol = e >> 2;
    const bool tma_epi = p.tma_epi;                       // warp-uniform
    unsigned char* wstage = epi_stage + e * (tma_epi ? WSB / 2 : WSB);
    uint64_t* abar = aux_bar + e * 2;
    const int band_off = (int)cta * BM + q * 32;
    uint32_t aux_phase = 0, aux_pending = 0;              // per-slab-buffer phase bits / loads in flight (warp-uniform)
    // auxiliary-input tiles of a work unit: one box per 64-column slab that lies inside the matrix (ls = 0, 1)
    auto slab_valid = [&](int row0, int n0, int ls) { return row0 < p.M && n0 + (hcol * 2 + ls) * 64 < p.N; };
    auto aux_issue = [&](int row0, int n0, int ls) {      // all lanes keep the books, lane 0 issues
      if (!slab_valid(row0, n0, ls)) return;
      aux_pending |= 1u << ls;
      if (lane == 0) {
        mbar_expect_tx(&abar[ls], SLAB_BYTES);
        tma_load_2d(wstage + ls * SLAB_BYTES, &tmAux, &abar[ls], n0 + (hcol * 2 + ls) * 64, row0);
      }
    };
    if (Cfg::AUX_IN && tma_epi && cluster_id < total_units) {
      int m_blk, n_blk, kb0, kb1; unit_coords(cluster_id, m_blk, n_blk, kb0, kb1);
      for (int ls = 0; ls < 2; ++ls) aux_issue(m_blk * 2 * BM + band_off, n_blk * BN, ls);
    }
    int it = 0;
    for (int unit = cluster_id; unit < total_units && !*abort_flag; unit += num_clusters, ++it) {
      int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
      fence_after_sync();
      const int n0 = n_blk * BN;
      const int row0 = m_blk * 2 * BM + band_off;
      const float alpha = p.alpha ? *p.alpha : 1.0f;
      const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if (!tma_epi) {
        if (e < 4) epilogue_warp<EPI>(p, tacc, wstage, row0, n0, alpha, lane);
      } else {
        const int nunit = unit + num_clusters;
        const bool has_next = Cfg::AUX_IN && nunit < total_units;
        int nrow0 = 0, nn0 = 0;
        if (has_next) { int mb, nb, k0, k1; unit_coords(nunit, mb, nb, k0, k1); nrow0 = mb * 2 * BM + band_off; nn0 = nb * BN; }
        bool ok = true;
#pragma unroll 1
        for (int ls = 0; ls < 2; ++ls) {
          if (!slab_valid(row0, n0, ls)) break;            // warp-uniform
          const int col0 = n0 + (hcol * 2 + ls) * 64;
          uint32_t r0[32], r1[32];
          tmem_ld32(tacc + (hcol * 2 + ls) * 64, r0);
          tmem_ld32(tacc + (hcol * 2 + ls) * 64 + 32, r1);
          tmem_wait_ld();
          unsigned char* buf;
          if (Cfg::F32_OUT) {
            // fp32 accumulate / store: the slab leaves as two boxes of 32 rows x 32 fp32 columns (128-byte rows, swizzled), which
            // the TMA engine adds into (split-K partial sums, gradient accumulation) or writes to the output; the warp goes on
            // to its next slab at once instead of waiting on 64 vector reductions per lane.
            buf = wstage;
            if (lane == 0) bulk_wait_read<0>();           // the previous slab's boxes have been read
            __syncwarp();
            unsigned char* myrow = buf + lane * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const int sw = (c ^ (lane & 7)) << 4;
              *reinterpret_cast<float4*>(myrow + sw) = make_float4(__uint_as_float(r0[4 * c]) * alpha, __uint_as_float(r0[4 * c + 1]) * alpha,
                                                                   __uint_as_float(r0[4 * c + 2]) * alpha, __uint_as_float(r0[4 * c + 3]) * alpha);
              *reinterpret_cast<float4*>(myrow + SLAB_BYTES + sw) = make_float4(__uint_as_float(r1[4 * c]) * alpha, __uint_as_float(r1[4 * c + 1]) * alpha,
                                                                                __uint_as_float(r1[4 * c + 2]) * alpha, __uint_as_float(r1[4 * c + 3]) * alpha);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && !(p.dbg & 1)) {
              if (EPI == EPI_ACC_F32) {
                tma_reduce_add_2d(&tmD, buf, col0, row0);
                if (col0 + 32 < p.N) tma_reduce_add_2d(&tmD, buf + SLAB_BYTES, col0 + 32, row0);
              } else {
                tma_store_2d(&tmD, buf, col0, row0);
                if (col0 + 32 < p.N) tma_store_2d(&tmD, buf + SLAB_BYTES, col0 + 32, row0);
              }
              bulk_commit();
            }
            continue;
          }
          if (Cfg::AUX_IN) {
            buf = wstage + ls * SLAB_BYTES;
            if (!mbar_wait(&abar[ls], (aux_phase >> ls) & 1)) { ok = false; break; }
            aux_phase ^= 1u << ls; aux_pending &= ~(1u << ls);
          } else {
            buf = wstage;
            if (lane == 0) bulk_wait_read<0>();           // the previous slab's stores have read the buffer
            __syncwarp();
          }
          if (Cfg::TWO_OUT) {
            uint4 pre[8];
            epi_slab_pre(p, r0, r1, buf, col0, alpha, lane, pre);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && !(p.dbg & 1)) { tma_store_2d(&tmAux, buf, col0, row0); bulk_commit(); }
            epi_slab_gelu(p, pre, buf + SLAB_BYTES, lane);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && !(p.dbg & 1)) { tma_store_2d(&tmD, buf + SLAB_BYTES, col0, row0); bulk_commit(); }
            continue;
          }
          epi_slab_bf16<EPI>(p, r0, r1, buf, col0, alpha, lane);
          fence_proxy_async();
          __syncwarp();
          if (EPI == EPI_DGELU && p.colsum) {
            // column sums of the slab as stored (bf16): lane l adds up columns 2l and 2l + 1 of the warp's rows out of the
            // swizzled box (conflict-free: the 32 lanes read the 128 bytes of one row) and adds them to colsum
            float s0 = 0.f, s1 = 0.f;
            const int nrows = min(32, p.M - row0);
#pragma unroll 8
            for (int r = 0; r < nrows; ++r) {
              const uint32_t w = *reinterpret_cast<const uint32_t*>(buf + r * 128 + ((((lane >> 2) ^ (r & 7))) << 4) + (lane & 3) * 4);
              s0 += __uint_as_float(w << 16); s1 += __uint_as_float(w & 0xffff0000u);
            }
            const int col = col0 + 2 * lane;
            if (col < p.N) {
              asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p.colsum + col), "f"(s0) : "memory");
              asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p.colsum + col + 1), "f"(s1) : "memory");
            }
          }
          if (lane == 0 && !(p.dbg & 1)) {
            if (Cfg::TWO_OUT) {
              tma_store_2d(&tmAux, buf, col0, row0);
              tma_store_2d(&tmD, buf + SLAB_BYTES, col0, row0);
            } else {
              tma_store_2d(&tmD, buf, col0, row0);
            }
            bulk_commit();
          }
        }
        if (!ok) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
        if (Cfg::AUX_IN && has_next) {                    // refill each buffer once its store has been read
          if (lane == 0) bulk_wait_read<1>();
          __syncwarp();
          aux_issue(nrow0, nn0, 0);
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
          aux_issue(nrow0, nn0, 1);
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty_bar[acc]), 0));   // the leader owns the accumulator hand-back
    }
    if (tma_epi) {
      // nothing of this CTA's shared memory may still be a source or a destination of a copy at exit
      for (int ls = 0; ls < 2; ++ls)
        if (aux_pending & (1u << ls)) (void)mbar_wait(&abar[ls], (aux_phase >> ls) & 1);
      if (lane == 0) bulk_wait<0>();
      __syncwarp();
    }
  }

  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                   // the peer may still be signalling / reading this CTA's smem
  if (warp == 1) { fence_after_sync(); tmem_dealloc_pair<512>(tmem_base); }
}

template <int KIND> struct KindTraits;
template <> struct KindTraits<KIND_F16> { static constexpr int ESZ = 2; static constexpr CUtensorMapDataType DT = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; };
template <> struct KindTraits<KIND_TF32> { static constexpr int ESZ = 4; static constexpr CUtensorMapDataType DT = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; };
template <> struct KindTraits<KIND_F8F6F4> { static constexpr int ESZ = 1; static constexpr CUtensorMapDataType DT = CU_TENSOR_MAP_DATA_TYPE_UINT8; };

int g_dbg_mn_lbo = -1, g_dbg_mn_sbo = -1;   // test hooks: override the MN-major descriptor strides
thread_local float* g_pending_colsum = nullptr;   // armed by llmb_gemm_set_colsum, consumed by the calling thread's next llmb_gemm
thread_local GatherArgs g_pending_gather{};   // armed by llmb_gemm_set_gather, consumed (and cleared) by the calling thread's next llmb_gemm
thread_local PullArgs g_pending_pull{};       // armed by llmb_gemm_set_pull, consumed (and cleared) the same way
int g_pair_mode = -1;                         // -1: read LLMB_GEMM_PAIR once; 0: single-CTA tiles; 1: CTA-pair tiles

bool pair_mode() {
  if (g_pair_mode < 0) { const char* e = getenv("LLMB_GEMM_PAIR"); g_pair_mode = (e && e[0] == '0') ? 0 : 1; }
  return g_pair_mode == 1;
}

template <int KIND, int EPI>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& taux,
                const GemmParams& p, int grid, cudaStream_t st) {
  static bool attr_done = false;
  constexpr int SMEM = smem2_bytes<EPI>();
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<KIND, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_pair_kernel<KIND, EPI><<<grid, PAIR_THREADS, SMEM, st>>>(ta, tb, td, taux, p);
  return (int)cudaGetLastError();
}

template <int KIND, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<KIND, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_kernel<KIND, EPI><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

template <int KIND>
int gemm_dispatch(void* D, const void* A, const void* B, const void* bias, void* aux, const float* alpha, int M, int N,
                  int K, long long lda, long long ldb, long long ldd, long long ldaux, int a_mn, int b_mn, int a_fmt,
                  int b_fmt, int epi, int splits, int* status, cudaStream_t st) {
  constexpr int ESZ = KindTraits<KIND>::ESZ;
  constexpr int ROW_ELEMS = ROW_BYTES / ESZ;          // elements per swizzled row
  constexpr int BKE = ROW_ELEMS;                      // K elements per stage
  constexpr int MMA_K = 32 / ESZ;
  if (M <= 0 || N <= 0 || K <= 0) return LLMB_ERR_BAD_ARG;
  if ((lda * ESZ) % 16 || (ldb * ESZ) % 16 || N % 8) return LLMB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D)) & 15) return LLMB_ERR_BAD_ARG;

  const bool pair = pair_mode();
  CUtensorMap ta, tb;
  int rc;
  // K-major: global [MN rows, K cols], box [tile rows, ROW_ELEMS]; MN-major: global [K rows, MN cols], box [BKE, ROW_ELEMS]
  // (in pair mode each CTA fetches a 128-row half of the B tile)
  const bool base32 = (KIND == KIND_TF32);            // fp32 operands stored MN-major need the 32-byte-base swizzle
  const CUtensorMapSwizzle mn_swz = base32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  rc = a_mn ? make_tmap_2d(&ta, A, KindTraits<KIND>::DT, ESZ, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BKE, ROW_ELEMS, mn_swz)
            : make_tmap_2d(&ta, A, KindTraits<KIND>::DT, ESZ, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, ROW_ELEMS);
  if (rc) return 1000 + rc;
  int a_3d = 0, b_3d = 0;
  static int use3d = -1;
  if (use3d < 0) { const char* e = getenv("LLMB_GEMM_3D"); use3d = (e && e[0] == '0') ? 0 : 1; }
  // MN-major tiles as one 3-D box: (elements of one 128-byte row, k rows, row-chunks) - one TMA request per operand and stage
  if (a_mn && use3d && M % ROW_ELEMS == 0) {
    CUtensorMap t3;
    if (make_tmap_3d(&t3, A, KindTraits<KIND>::DT, ESZ, ROW_ELEMS, (uint64_t)K, (uint64_t)(M / ROW_ELEMS), (uint64_t)lda, ROW_ELEMS,
                     ROW_ELEMS, BKE, BM / ROW_ELEMS, mn_swz) == 0) { ta = t3; a_3d = 1; }
  }
  rc = b_mn ? make_tmap_2d(&tb, B, KindTraits<KIND>::DT, ESZ, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BKE, ROW_ELEMS, mn_swz)
            : make_tmap_2d(&tb, B, KindTraits<KIND>::DT, ESZ, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? 128 : BN, ROW_ELEMS);
  if (rc) return 1000 + rc;

  if (b_mn && use3d && N % ROW_ELEMS == 0) {
    CUtensorMap t3;
    if (make_tmap_3d(&t3, B, KindTraits<KIND>::DT, ESZ, ROW_ELEMS, (uint64_t)K, (uint64_t)(N / ROW_ELEMS), (uint64_t)ldb, ROW_ELEMS,
                     ROW_ELEMS, BKE, (pair ? 128 : BN) / ROW_ELEMS, mn_swz) == 0) { tb = t3; b_3d = 1; }
  }
  GemmParams p;
  p.g = g_pending_gather;
  g_pending_gather.W = 0;
  p.pull = g_pending_pull;
  g_pending_pull.nseg = 0; g_pending_pull.nwait = 0;
  if ((p.pull.nseg > 0 || p.pull.nwait > 0) && (!pair || p.g.W > 1)) return LLMB_ERR_BAD_ARG;   // copier warps exist in the pair kernel only
  p.colsum = g_pending_colsum;
  g_pending_colsum = nullptr;
  if (p.colsum && !(pair && epi == EPI_DGELU && (KIND == KIND_F16 || KIND == KIND_F8F6F4))) return LLMB_ERR_BAD_ARG;   // bf16 output, TMA epilogue
  if (p.g.W > 1) {
    // gathered A: K-major bf16 rows, CTA-pair kernel, whole 256-row tiles per chunk, no split-K
    if (!pair || a_mn || KIND != KIND_F16 || p.g.tiles_per_chunk <= 0 || M != p.g.W * p.g.tiles_per_chunk * 2 * BM || epi == EPI_ACC_F32)
      return LLMB_ERR_BAD_ARG;
  }
  p.a_3d = a_3d; p.b_3d = b_3d;
  p.D = D; p.bias = bias; p.aux = aux; p.alpha = alpha;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldaux = ldaux;
  p.a_mn = a_mn; p.b_mn = b_mn;
  const uint32_t mn_lbo = g_dbg_mn_lbo >= 0 ? (uint32_t)g_dbg_mn_lbo : (uint32_t)(BKE * ROW_BYTES);
  const uint32_t mn_sbo = g_dbg_mn_sbo >= 0 ? (uint32_t)g_dbg_mn_sbo : (base32 ? 512u : 1024u);
  p.a_layout = (a_mn && base32) ? 1u : 2u;
  p.b_layout = (b_mn && base32) ? 1u : 2u;
  p.a_lbo = a_mn ? mn_lbo : 16; p.a_sbo = a_mn ? mn_sbo : 1024; p.a_kstep = a_mn ? MMA_K * ROW_BYTES : 32;
  p.b_lbo = b_mn ? mn_lbo : 16; p.b_sbo = b_mn ? mn_sbo : 1024; p.b_kstep = b_mn ? MMA_K * ROW_BYTES : 32;
  p.idesc = make_idesc((uint32_t)a_fmt, (uint32_t)b_fmt, (uint32_t)a_mn, (uint32_t)b_mn, pair ? 2 * BM : BM, BN);
  p.bke = BKE;                                          // a 128-byte stage row holds BKE / MMA_K = 4 MMA k-steps for every kind
  p.m_tiles = ceil_div(M, BM); p.n_tiles = ceil_div(N, BN);
  p.kb_total = ceil_div(K, BKE);
  if (splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  if (epi != EPI_ACC_F32) splits = 1;
  p.kb_per_split = ceil_div(p.kb_total, splits);
  p.splits = ceil_div(p.kb_total, p.kb_per_split);
  p.status = status;
  p.io_f32 = (KIND == KIND_TF32) ? 1 : 0;
  p.bias_vec = (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
  p.tma_epi = 0;
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("LLMB_GEMM_DBG"); dbg = e ? atoi(e) : 0; } p.dbg = dbg; }
  if (pair) {
    const long long units2 = (long long)ceil_div(M, 2 * BM) * p.n_tiles * p.splits;
    const int max_clusters = sm_count() / 2;
    const int grid2 = 2 * (int)(units2 < max_clusters ? units2 : max_clusters);
    // bf16 outputs (and bf16 auxiliary tensors) travel by TMA when their layout allows a tensor map
    CUtensorMap td = ta, taux = ta;                       // placeholders when the register epilogue runs
    static int tma_epi_on = -1;
    if (tma_epi_on < 0) { const char* e = getenv("LLMB_GEMM_TMA_EPI"); tma_epi_on = (e && e[0] == '0') ? 0 : 1; }
    const bool needs_aux = epi == EPI_BIAS_GELU || epi == EPI_DGELU || epi == EPI_BIAS_RESID;
    if (tma_epi_on && !p.io_f32 && epi != EPI_ACC_F32 && epi != EPI_STORE_F32 && (ldd * 2) % 16 == 0 &&
        (!needs_aux || (aux && (reinterpret_cast<uintptr_t>(aux) & 15) == 0 && (ldaux * 2) % 16 == 0))) {
      int ok = make_tmap_2d(&td, D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 64) == 0;
      if (ok && needs_aux)
        ok = make_tmap_2d(&taux, aux, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldaux, 32, 64) == 0;
      p.tma_epi = ok;
    }
    if (tma_epi_on && !p.io_f32 && (epi == EPI_ACC_F32 || epi == EPI_STORE_F32) && (ldd * 4) % 16 == 0 &&
        (reinterpret_cast<uintptr_t>(D) & 15) == 0)
      p.tma_epi = make_tmap_2d(&td, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 32) == 0;
    if (p.colsum && !p.tma_epi) return LLMB_ERR_BAD_ARG;   // the column sums are taken in the TMA epilogue only
    switch (epi) {
      case EPI_NONE: return launch_pair<KIND, EPI_NONE>(ta, tb, td, taux, p, grid2, st);
      case EPI_BIAS: return launch_pair<KIND, EPI_BIAS>(ta, tb, td, taux, p, grid2, st);
      case EPI_BIAS_GELU: return launch_pair<KIND, EPI_BIAS_GELU>(ta, tb, td, taux, p, grid2, st);
      case EPI_DGELU: return launch_pair<KIND, EPI_DGELU>(ta, tb, td, taux, p, grid2, st);
      case EPI_ACC_F32: return launch_pair<KIND, EPI_ACC_F32>(ta, tb, td, taux, p, grid2, st);
      case EPI_BIAS_RESID: return launch_pair<KIND, EPI_BIAS_RESID>(ta, tb, td, taux, p, grid2, st);
      case EPI_STORE_F32: return launch_pair<KIND, EPI_STORE_F32>(ta, tb, td, taux, p, grid2, st);
    }
    return LLMB_ERR_BAD_ARG;
  }
  long long units = (long long)p.m_tiles * p.n_tiles * p.splits;
  int grid = (int)(units < sm_count() ? units : sm_count());

  switch (epi) {
    case EPI_NONE: return launch<KIND, EPI_NONE>(ta, tb, p, grid, st);
    case EPI_BIAS: return launch<KIND, EPI_BIAS>(ta, tb, p, grid, st);
    case EPI_BIAS_GELU: return launch<KIND, EPI_BIAS_GELU>(ta, tb, p, grid, st);
    case EPI_DGELU: return launch<KIND, EPI_DGELU>(ta, tb, p, grid, st);
    case EPI_ACC_F32: return launch<KIND, EPI_ACC_F32>(ta, tb, p, grid, st);
    case EPI_BIAS_RESID: return launch<KIND, EPI_BIAS_RESID>(ta, tb, p, grid, st);
    case EPI_STORE_F32: return launch<KIND, EPI_STORE_F32>(ta, tb, p, grid, st);
  }
  return LLMB_ERR_BAD_ARG;
}
// ------------------------------------------------------------------------------------------------
// Native block-scaled GEMMs:  D[M,N] = epi(alpha * sum_k (A[m,k] sfa[m,k/B]) (B[n,k] sfb[n,k/B])).
// NVFP4 (MX = 0): A and B are packed e2m1 (two values per byte, even index in the low nibble), one ue4m3
// scale per 16 values (`kind::mxf4nvf4.block_scale.scale_vec::4X`, K = 64 per MMA).  MXFP8 (MX = 1): e4m3 /
// e5m2 bytes, one ue8m0 scale per 32 values (`kind::mxf8f6f4.block_scale`, K = 32 per MMA).  Both operands
// K-major.  The scales come in 128-row x 4-block atoms of 512 bytes (byte (r % 32) * 16 + (r / 32) * 4 +
// block), atoms of one row block contiguous along K: the layout the tensor core's scale path wants, so an
// atom goes from global to shared memory as part of one bulk copy and from there to tensor memory as one
// tcgen05.cp (32 rows x 16 bytes -> 4 columns, replicated to the four lane quarters), issued by the MMA
// thread just ahead of the MMAs that use it.
//
// One CTA per SM owns 128 x 256 tiles.  A stage is 128 bytes of K per row (256 e2m1 / 128 fp8 values): A
// 16 KB, B 32 KB, scales 2 + 4 KB; four MMAs per stage.  Tensor memory: 48 columns of scales (A: 4 per
// k-step, B: 8 per k-step) do not leave room for two 256-column fp32 accumulators, so these OVERLAP in one
// 64-column slab: accumulator 0 = [0, 256), accumulator 1 = [192, 448), scales from 448.  The epilogue of a
// tile reads the shared slab first and says so (`tover`); the next tile's MMAs start when it is read and the
// tile before that has been drained completely (`tempty`), so the epilogue of one tile still overlaps the
// MMAs of the next.
// Eight epilogue warps: warp % 4 is the 32-row band (TMEM lane quarter), (warp - 2) / 4 the 128-column half,
// two 64-column slabs per warp; bf16 results leave (and auxiliary inputs arrive) as 128-byte-swizzled 32 x 64
// boxes by TMA; fp32 outputs and layouts without a tensor map use the register epilogue on four warps.
constexpr int NV_BN = 256;
constexpr int NV_STAGES = 3;
constexpr int NV_THREADS = 320;                        // TMA producer, MMA issuer, 8 epilogue warps
constexpr int NV_A_TILE = 128 * ROW_BYTES;             // 16 KB
constexpr int NV_B_TILE = 256 * ROW_BYTES;             // 32 KB
constexpr int NV_SF = 4 * 512;                         // scales of 128 rows x one stage (NVFP4: 4 atoms; MXFP8: 1)
constexpr int NV_STAGE_BYTES = NV_A_TILE + NV_B_TILE + 3 * NV_SF;     // 54 KB
constexpr int NV_EPI_BYTES = 8 * EPI_STAGE_BYTES;      // two 4 KB boxes per epilogue warp
constexpr int NV_BAR_BYTES = 256;
constexpr int NV_SMEM_BYTES = 232448;                  // the whole CTA budget: 3 stages + boxes + barriers + 768 B of alignment slack
static_assert(NV_STAGES * NV_STAGE_BYTES + NV_EPI_BYTES + NV_BAR_BYTES + 768 == NV_SMEM_BYTES, "shared-memory budget");
constexpr int NV_BKE = 256;                            // K values per stage (NVFP4)
constexpr int NV_BKE_MX = 128;                         // K values per stage (MXFP8)
constexpr uint32_t NV_ACC1_COL = 192, NV_SFA_COL = 448, NV_SFB_COL = 464;

struct Nvfp4Params {
  GemmParams g;                                         // epilogue fields, tile counts, split-K (operand fields unused)
  const unsigned char* sfa; const unsigned char* sfb;   // scale atoms of A ([ceil(M/128)][atoms_k][512]) and of B ([ceil(N/128)][atoms_k][512])
  int atoms_k;                                          // scale atoms along K: ceil(K / 64) for NVFP4, ceil(K / 128) for MXFP8
  int b_row_blocks;                                     // ceil(N / 128)
  uint32_t idesc;
};

template <int MX, int EPI>
__global__ void __launch_bounds__(NV_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmAux, const Nvfp4Params q) {
  using Cfg = EpiCfg<EPI>;
  const GemmParams& p = q.g;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem - smem_raw > 768) {                          // the alignment slack this launch was given does not cover the base it got
    if (threadIdx.x == 0) atomicExch(p.status, LLMB_ERR_BAD_ARG);
    return;
  }
  unsigned char* epi_stage = smem + NV_STAGES * NV_STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + NV_EPI_BYTES);
  uint64_t* empty_bar = full_bar + NV_STAGES;
  uint64_t* tfull_bar = empty_bar + NV_STAGES;     // [2] accumulator complete
  uint64_t* tempty_bar = tfull_bar + 2;            // [2] accumulator drained (8 warps)
  uint64_t* tover_bar = tempty_bar + 2;            // [2] the slab it shares with the other accumulator is read (4 warps)
  uint64_t* aux_bar = tover_bar + 2;               // [16] two per epilogue warp: auxiliary-input box landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NV_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 8); mbar_init(&tover_bar[a], 4); }
    for (int w = 0; w < 16; ++w) mbar_init(&aux_bar[w], 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmD); prefetch_tmap(&tmAux);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_split = p.m_tiles * p.n_tiles;
  const int total_units = tiles_per_split * p.splits;
  auto unit_coords = [&](int unit, int& m_blk, int& n_blk, int& kb0, int& kb1) {
    int split = unit / tiles_per_split, t = unit % tiles_per_split;
    int band_sz = BAND * p.n_tiles;
    int b = t / band_sz, r = t % band_sz;
    int m_in_band = min(BAND, p.m_tiles - b * BAND);
    m_blk = b * BAND + r % m_in_band;
    n_blk = r / m_in_band;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  };
  constexpr int APS = MX ? 1 : 4;                   // scale atoms per row block and stage

  if (warp == 0) {
    // ------------------------------------------------------------ producer: operand tiles by TMA, scale atoms by bulk copy
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x) {
        int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
        const int rb0 = 2 * n_blk;                      // the tile's two 128-row blocks of B scales; the second may not exist
        const bool second = rb0 + 1 < q.b_row_blocks;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
          unsigned char* sa = smem + stage * NV_STAGE_BYTES;
          unsigned char* sb = sa + NV_A_TILE;
          unsigned char* sf = sb + NV_B_TILE;           // [A][B rows 0..127][B rows 128..255], 2 KB each
          const int atoms = min(APS, q.atoms_k - kb * APS);
          const uint32_t sf_bytes = (uint32_t)atoms * 512u;
          mbar_expect_tx(&full_bar[stage], NV_A_TILE + NV_B_TILE + (second ? 3u : 2u) * sf_bytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * ROW_BYTES, m_blk * BM);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * ROW_BYTES, n_blk * NV_BN);
          const size_t koff = (size_t)kb * APS;
          bulk_load_1d(sf, q.sfa + ((size_t)m_blk * q.atoms_k + koff) * 512, sf_bytes, &full_bar[stage]);
          bulk_load_1d(sf + NV_SF, q.sfb + ((size_t)rb0 * q.atoms_k + koff) * 512, sf_bytes, &full_bar[stage]);
          if (second) bulk_load_1d(sf + 2 * NV_SF, q.sfb + ((size_t)(rb0 + 1) * q.atoms_k + koff) * 512, sf_bytes, &full_bar[stage]);
          if (++stage == NV_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: scales to TMEM, then four MMAs per stage
    int stage = 0; uint32_t phase = 0;
    int it = 0;
    const uint64_t adesc0 = make_smem_desc(smem_u32(smem), 16, 1024, 2);
    const uint64_t bdesc0 = make_smem_desc(smem_u32(smem) + NV_A_TILE, 16, 1024, 2);
    const uint64_t sfa0 = make_sf_desc(smem_u32(smem) + NV_A_TILE + NV_B_TILE);
    const uint64_t sfb0 = make_sf_desc(smem_u32(smem) + NV_A_TILE + NV_B_TILE + NV_SF);
    const uint32_t idesc = q.idesc;
    const uint32_t sfa_t = tmem_base + NV_SFA_COL, sfb_t = tmem_base + NV_SFB_COL;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x, ++it) {
      int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
      const int acc = it & 1;
      // this accumulator's previous tile is drained, and the previous tile (other accumulator) has read the shared columns
      if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1)) { ok = false; break; }
      if (it > 0 && !mbar_wait(&tover_bar[acc ^ 1], ((it - 1) >> 1) & 1)) { ok = false; break; }
      fence_after_sync();
      const uint32_t d_tmem = tmem_base + (acc ? NV_ACC1_COL : 0u);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
        fence_after_sync();
        const uint64_t soff = (uint64_t)(stage * (NV_STAGE_BYTES >> 4));
        if (MX) {
          const int nk = min(4, (p.K - kb * NV_BKE_MX + 31) / 32);
          if (elect_one()) {
            tmem_cp_sf(sfa_t, sfa0 + soff);
            tmem_cp_sf(sfb_t, sfb0 + soff);
            tmem_cp_sf(sfb_t + 4, sfb0 + soff + (uint64_t)(NV_SF >> 4));
            for (int k = 0; k < nk; ++k)
              umma_mxfp8(d_tmem, adesc0 + soff + (uint64_t)(k * 2), bdesc0 + soff + (uint64_t)(k * 2),
                         idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4), sfa_t | ((uint32_t)k << 30), sfb_t | ((uint32_t)k << 30),
                         (kb > kb0 || k > 0) ? 1u : 0u);
            umma_commit(&empty_bar[stage]);
          }
        } else {
          const int atoms = min(4, q.atoms_k - kb * 4);
          if (elect_one()) {
            for (int k = 0; k < atoms; ++k) {
              tmem_cp_sf(sfa_t + 4 * k, sfa0 + soff + (uint64_t)(k * 32));
              tmem_cp_sf(sfb_t + 8 * k, sfb0 + soff + (uint64_t)(k * 32));
              tmem_cp_sf(sfb_t + 8 * k + 4, sfb0 + soff + (uint64_t)((NV_SF >> 4) + k * 32));
            }
            for (int k = 0; k < atoms; ++k)
              umma_nvfp4(d_tmem, adesc0 + soff + (uint64_t)(k * 2), bdesc0 + soff + (uint64_t)(k * 2), idesc, sfa_t + 4 * k, sfb_t + 8 * k,
                         (kb > kb0 || k > 0) ? 1u : 0u);
            umma_commit(&empty_bar[stage]);             // operand tiles and scale atoms reusable once these have run
          }
        }
        __syncwarp();
        if (++stage == NV_STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (elect_one()) umma_commit(&tfull_bar[acc]);
      __syncwarp();
    }
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int qd = warp & 3, e = warp - 2, hc = e >> 2;   // TMEM lane quarter, warp slot, 128-column half
    const bool tma_epi = !Cfg::F32_OUT && p.tma_epi;      // warp-uniform
    unsigned char* buf = epi_stage + e * EPI_STAGE_BYTES; // two 4 KB boxes
    uint64_t* abar = &aux_bar[e * 2];
    uint32_t aux_phase = 0;                               // bit ls: phase of abar[ls]
    uint32_t nstores = 0;                                 // slabs stored so far (plain epilogues alternate the two boxes)
    int it = 0;
    for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x, ++it) {
      int m_blk, n_blk, kb0, kb1; unit_coords(unit, m_blk, n_blk, kb0, kb1);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int row0 = m_blk * BM + qd * 32, colh = n_blk * NV_BN + hc * 128;
      // the slab shared with the other accumulator goes first: the last 64 columns of accumulator 0, the first 64 of
      // accumulator 1; the four warps that own it report it read
      const bool reporter = tma_epi ? (hc == (acc ? 0 : 1)) : (e < 4);
      const int first = (acc == 0 && hc == 1) ? 1 : 0;
      if (tma_epi && Cfg::AUX_IN && row0 < p.M) {         // the auxiliary boxes travel while the tile's MMAs run
        if (lane == 0) {
          bulk_wait_read<0>();                            // the previous tile's stores have read the boxes
          for (int ls = 0; ls < 2; ++ls)
            if (colh + ls * 64 < p.N) {
              mbar_expect_tx(&abar[ls], SLAB_BYTES);
              tma_load_2d(buf + ls * SLAB_BYTES, &tmAux, &abar[ls], colh + ls * 64, row0);
            }
        }
        __syncwarp();
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
      fence_after_sync();
      const float alpha = p.alpha ? *p.alpha : 1.0f;
      const uint32_t tacc = tmem_base + ((uint32_t)(qd * 32) << 16) + (acc ? NV_ACC1_COL : 0u);
      if (!tma_epi) {
        if (e < 4) epilogue_warp<EPI, NV_BN>(p, tacc, buf, row0, n_blk * NV_BN, alpha, lane);
        if (reporter) {
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tover_bar[acc]);
        }
      } else {
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < 2; ++j) {
          const int ls = j ^ first;
          const int col0 = colh + ls * 64;
          const bool valid = row0 < p.M && col0 < p.N;    // warp-uniform
          uint32_t r0[32], r1[32];
          if (valid) {
            tmem_ld32(tacc + hc * 128 + ls * 64, r0);
            tmem_ld32(tacc + hc * 128 + ls * 64 + 32, r1);
            tmem_wait_ld();
          }
          if (j == 0 && reporter) {
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tover_bar[acc]);
          }
          if (!valid) continue;
          unsigned char* box;
          if (Cfg::AUX_IN) {
            box = buf + ls * SLAB_BYTES;
            if (!mbar_wait(&abar[ls], (aux_phase >> ls) & 1)) { ok = false; break; }
            aux_phase ^= 1u << ls;
          } else if (Cfg::TWO_OUT) {
            box = buf;                                    // pre-activation box, result box behind it
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
          } else {
            box = buf + (nstores++ & 1) * SLAB_BYTES;     // alternate boxes: only the store before last must have been read
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
          }
          epi_slab_bf16<EPI>(p, r0, r1, box, col0, alpha, lane);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (Cfg::TWO_OUT) {
              tma_store_2d(&tmAux, box, col0, row0);
              tma_store_2d(&tmD, box + SLAB_BYTES, col0, row0);
            } else {
              tma_store_2d(&tmD, box, col0, row0);
            }
            bulk_commit();
          }
        }
        if (!ok) { *abort_flag = 1; atomicExch(p.status, LLMB_ERR_TIMEOUT); break; }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    if (tma_epi) {                                        // no copy may still read this CTA's shared memory at exit
      if (lane == 0) bulk_wait<0>();
      __syncwarp();
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc<512>(tmem_base); }
}

template <int MX, int EPI>
int launch_nvfp4(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& taux, const Nvfp4Params& q,
                 int grid, cudaStream_t st) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<MX, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, NV_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  gemm_nvfp4_kernel<MX, EPI><<<grid, NV_THREADS, NV_SMEM_BYTES, st>>>(ta, tb, td, taux, q);
  return (int)cudaGetLastError();
}
}  // namespace

// D[M,N] = epi(alpha * A·B^T).  a_mn/b_mn = 1 when the operand is stored [K, M] / [K, N].
// kind: 0 bf16, 1 tf32 (fp32 storage), 2 fp8 (a_fmt/b_fmt: 0 e4m3, 1 e5m2).  D is bf16 except for the
// fp32 epilogues (4 = accumulate with red.add, split-K allowed; 6 = plain fp32 store).
// `status` is a device int the kernel sets to LLMB_ERR_TIMEOUT if a bounded wait expires.
LLMB_API int llmb_gemm(void* D, const void* A, const void* B, const void* bias, void* aux, const float* alpha, int M,
                       int N, int K, long long lda, long long ldb, long long ldd, long long ldaux, int a_mn, int b_mn,
                       int kind, int a_fmt, int b_fmt, int epi, int splits, int* status, cudaStream_t st) {
  switch (kind) {
    case 0: return gemm_dispatch<KIND_F16>(D, A, B, bias, aux, alpha, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, FMT_BF16, FMT_BF16, epi, splits, status, st);
    case 1: return gemm_dispatch<KIND_TF32>(D, A, B, bias, aux, alpha, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, FMT_TF32, FMT_TF32, epi, splits, status, st);
    case 2: return gemm_dispatch<KIND_F8F6F4>(D, A, B, bias, aux, alpha, M, N, K, lda, ldb, ldd, ldaux, a_mn, b_mn, a_fmt, b_fmt, epi, splits, status, st);
  }
  return LLMB_ERR_BAD_ARG;
}

// Arms the calling thread's NEXT llmb_gemm call to gather its A matrix from W ranks (see GatherArgs): A must be the
// local [W*n, K] buffer, n a multiple of 256; peer_src[r] = address of chunk r in rank r's buffer; flags = this
// rank's flag words; counts = 16 local counters that the caller zeroes (stream-ordered) before the GEMM.
LLMB_API void llmb_gemm_set_gather(void* const* peer_src, void* local, const void* flags, unsigned* counts, long long chunk_bytes,
                                   unsigned seq, int W, int me, int rows_per_rank) {
  GatherArgs g{};
  for (int r = 0; r < W && r < 8; ++r) g.peer_src[r] = peer_src[r];
  g.local = local; g.flags = flags; g.counts = counts; g.chunk_vecs = chunk_bytes / 16;
  g.seq = seq; g.target = (unsigned)((g.chunk_vecs + 2047) / 2048); g.W = W; g.me = me; g.tiles_per_chunk = rows_per_rank / (2 * BM);
  g_pending_gather = g;
}
// Arms the calling thread's NEXT llmb_gemm call (CTA-pair kernel) with a parameter pull and / or a wait (see PullArgs).
// Segment s copies nbytes[s] bytes (a multiple of 16, both addresses 16-byte aligned) from src[s] (memory of rank
// owner[s], mapped here) to dst[s]; counts = 16 counters zeroed (stream-ordered) before the launch.  wait_counts[i]
// must reach wait_bytes[i] / 32 KB (rounded up) before the GEMM's B operand is read.  seq: parameter sequence number
// every owner must have announced (0 = parameters as loaded, nothing to wait for).
LLMB_API int llmb_gemm_set_pull(const void* const* src, void* const* dst, const long long* nbytes, const int* owner, int nseg,
                                const void* flags, unsigned seq, unsigned* counts, const unsigned* const* wait_counts,
                                const long long* wait_bytes, int nwait, int W) {
  if (nseg < 0 || nseg > 8 || nwait < 0 || nwait > 8) return LLMB_ERR_BAD_ARG;
  PullArgs a{};
  for (int i = 0; i < nseg; ++i) {
    if ((reinterpret_cast<uintptr_t>(src[i]) | reinterpret_cast<uintptr_t>(dst[i]) | (uintptr_t)nbytes[i]) & 15) return LLMB_ERR_BAD_ARG;
    a.src[i] = src[i]; a.dst[i] = dst[i]; a.vecs[i] = nbytes[i] / 16; a.owner[i] = owner[i];
  }
  for (int i = 0; i < nwait; ++i) { a.wait_counts[i] = wait_counts[i]; a.wait_target[i] = (unsigned)((wait_bytes[i] / 16 + 2047) / 2048); }
  a.flags = flags; a.counts = counts; a.seq = seq; a.nseg = nseg; a.nwait = nwait; a.W = W;
  g_pending_pull = a;
  return 0;
}
// Arms the calling thread's NEXT llmb_gemm call (bf16, epilogue 3 = dGELU, CTA-pair kernel with the TMA epilogue) to add the column
// sums of its result to colsum[N] (fp32, red.add): the bias gradient of the layer that produced the pre-activations.
LLMB_API void llmb_gemm_set_colsum(float* colsum) { g_pending_colsum = colsum; }
LLMB_API void llmb_gemm_debug_mn_strides(int lbo_bytes, int sbo_bytes) { g_dbg_mn_lbo = lbo_bytes; g_dbg_mn_sbo = sbo_bytes; }
// 0: single-CTA 128x256 tiles, 1: CTA-pair 256x256 tiles (default; env LLMB_GEMM_PAIR=0 selects the former)
LLMB_API void llmb_gemm_set_pair_mode(int on) { g_pair_mode = on ? 1 : 0; }

// D[M,N] = epi(alpha * (A sfa)(B sfb)^T) on the NVFP4 tensor path (`kind::mxf4nvf4`, 16-value blocks, ue4m3 scales).
// A [M, K/2] and B [N, K/2]: packed e2m1 bytes as llmb_nvfp4_quantize writes them (K % 32 == 0); sfa / sfb: its
// swizzled scale buffers (llmb_nvfp4_scale_bytes(rows, K, 1) bytes, zero where no block exists).  D is bf16
// except for epi 4 / 6 (fp32 accumulate with split-K / fp32 store); bias and aux are bf16.
namespace {
template <int MX>
int gemm_block_scaled(void* D, const void* A, const void* B, const void* sfa, const void* sfb, const void* bias, void* aux,
                      const float* alpha, int M, int N, int K, int a_fmt, int b_fmt, long long ldd, long long ldaux, int epi,
                      int splits, int* status, cudaStream_t st) {
  constexpr int EPB = MX ? 1 : 2;                         // elements per byte
  constexpr int BKE = MX ? NV_BKE_MX : NV_BKE;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 || N % 8) return LLMB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(D) |
       reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb)) & 15) return LLMB_ERR_BAD_ARG;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)(K / EPB), (uint64_t)(K / EPB), BM, ROW_BYTES);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)(K / EPB), (uint64_t)(K / EPB), NV_BN, ROW_BYTES);
  if (rc) return 1000 + rc;
  Nvfp4Params q{};
  GemmParams& p = q.g;
  p.D = D; p.bias = bias; p.aux = aux; p.alpha = alpha;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldaux = ldaux;
  p.bke = BKE;
  p.m_tiles = ceil_div(M, BM); p.n_tiles = ceil_div(N, NV_BN);
  p.kb_total = ceil_div(K, BKE);
  if (splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  if (epi != EPI_ACC_F32) splits = 1;
  p.kb_per_split = ceil_div(p.kb_total, splits);
  p.splits = ceil_div(p.kb_total, p.kb_per_split);
  p.status = status;
  p.bias_vec = (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
  q.sfa = (const unsigned char*)sfa; q.sfb = (const unsigned char*)sfb;
  q.atoms_k = ceil_div(K, MX ? 128 : 64);
  q.b_row_blocks = ceil_div(N, 128);
  q.idesc = MX ? make_idesc_mxfp8((uint32_t)a_fmt, (uint32_t)b_fmt, BM, NV_BN) : make_idesc_nvfp4(BM, NV_BN);
  // bf16 outputs (and bf16 auxiliary tensors) travel by TMA when their layout allows a tensor map
  CUtensorMap td = ta, taux = ta;
  const bool needs_aux = epi == EPI_BIAS_GELU || epi == EPI_DGELU || epi == EPI_BIAS_RESID;
  if (epi != EPI_ACC_F32 && epi != EPI_STORE_F32 && (ldd * 2) % 16 == 0 &&
      (!needs_aux || (aux && (reinterpret_cast<uintptr_t>(aux) & 15) == 0 && (ldaux * 2) % 16 == 0))) {
    int ok = make_tmap_2d(&td, D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 64) == 0;
    if (ok && needs_aux)
      ok = make_tmap_2d(&taux, aux, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldaux, 32, 64) == 0;
    p.tma_epi = ok;
  }
  const long long units = (long long)p.m_tiles * p.n_tiles * p.splits;
  const int grid = (int)(units < sm_count() ? units : sm_count());
  switch (epi) {
    case EPI_NONE: return launch_nvfp4<MX, EPI_NONE>(ta, tb, td, taux, q, grid, st);
    case EPI_BIAS: return launch_nvfp4<MX, EPI_BIAS>(ta, tb, td, taux, q, grid, st);
    case EPI_BIAS_GELU: return launch_nvfp4<MX, EPI_BIAS_GELU>(ta, tb, td, taux, q, grid, st);
    case EPI_DGELU: return launch_nvfp4<MX, EPI_DGELU>(ta, tb, td, taux, q, grid, st);
    case EPI_ACC_F32: return launch_nvfp4<MX, EPI_ACC_F32>(ta, tb, td, taux, q, grid, st);
    case EPI_BIAS_RESID: return launch_nvfp4<MX, EPI_BIAS_RESID>(ta, tb, td, taux, q, grid, st);
    case EPI_STORE_F32: return launch_nvfp4<MX, EPI_STORE_F32>(ta, tb, td, taux, q, grid, st);
  }
  return LLMB_ERR_BAD_ARG;
}
}  // namespace

LLMB_API int llmb_gemm_nvfp4(void* D, const void* A, const void* B, const void* sfa, const void* sfb, const void* bias, void* aux,
                             const float* alpha, int M, int N, int K, long long ldd, long long ldaux, int epi, int splits,
                             int* status, cudaStream_t st) {
  return gemm_block_scaled<0>(D, A, B, sfa, sfb, bias, aux, alpha, M, N, K, 0, 0, ldd, ldaux, epi, splits, status, st);
}

// The same product on the MXFP8 tensor path (`kind::mxf8f6f4`): A [M, K] and B [N, K] are e4m3 (fmt 0) or e5m2 (fmt 1) bytes,
// sfa / sfb one ue8m0 scale (byte = biased exponent of a power of two) per row and 32 values of K in the same 128 x 4 atoms,
// ceil(K / 128) atoms per row block.
LLMB_API int llmb_gemm_mxfp8(void* D, const void* A, const void* B, const void* sfa, const void* sfb, const void* bias, void* aux,
                             const float* alpha, int M, int N, int K, int a_fmt, int b_fmt, long long ldd, long long ldaux,
                             int epi, int splits, int* status, cudaStream_t st) {
  return gemm_block_scaled<1>(D, A, B, sfa, sfb, bias, aux, alpha, M, N, K, a_fmt, b_fmt, ldd, ldaux, epi, splits, status, st);
}
