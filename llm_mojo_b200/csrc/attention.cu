// Causal flash attention forward / backward for head size 64 on tcgen05 + TMEM.
//
// Reference behaviour: llmm/attention.mojo:1557-1745 (forward: split -> QK^T -> causal softmax ->
// PV -> merge, storing [T,T] probabilities) and :4692-5030 (backward via dP, row-dot D, dS, and
// the dQ/dK/dV batched GEMMs).  Here nothing of size T x T ever reaches HBM: the kernels read
// the packed [B,T,3C] QKV activations directly through a 3-D TMA map (no split/merge
// permutes), keep S/P and the running output in TMEM / shared memory, and store only the
// output [B,T,C] plus one log-sum-exp per row.
//
// Default kernels (persistent, warp-specialised; described where they are defined below):
//   attn_fwd2_kernel      one CTA per SM, two independent tile streams, 64-key chunks
//   attn_bwd_dkv2_kernel  dK/dV per 128-key tile over 64-row query chunks   } two deterministic kernels,
//   attn_bwd_dq2_kernel   dQ per 128-row query tile over 64-key chunks      } no atomics
// The first-generation kernels are kept as comparators (LLMB_ATTN_FWD=1 / LLMB_ATTN_BWD=1): one CTA per 128-row
// tile, 256 threads, the phases MMA -> softmax -> MMA run one after another:
//   Forward  : two threads share a row, each owning one 64-column half of the 128-key score tile;
//              S = Q K^T (tcgen05, fp32 in TMEM) -> online softmax in registers -> P (bf16, swizzled smem)
//              -> O += P V (tcgen05, O in TMEM, rescaled in place).
//   dK/dV    : CTA = 128 key rows; loops over 64-row query chunks:  S^T = K Q^T, dP^T = V dO^T,
//              P^T and dS^T to smem, dV += P^T dO, dK += dS^T Q   (accumulators in TMEM).
//   dQ       : CTA = 128 query rows; loops over 64-row key chunks:   S = Q K^T, dP = dO V^T,
//              dS to smem, dQ += dS K.
// The MN-major UMMA descriptor lets the same TMA-written tile serve as a K-major operand of
// one product and as the transposed operand of the next.
// LSE is stored in the log2 domain of the scaled scores: lse2 = m + log2(sum 2^(s2 - m)).
#include "tc05.cuh"
using namespace llmb;
using namespace tc05;

namespace {
constexpr int HS = 64;
constexpr int TILE = 128;
constexpr int ROWB = 128;              // bytes per swizzled row (64 bf16)
constexpr int T64 = 64 * ROWB;         // 8 KB: 64-row tile
constexpr int T128 = 128 * ROWB;       // 16 KB: 128-row tile

struct AttnParams {
  void* out;            // fwd: O [B,T,C] bf16          bwd: dqkv [B,T,3C] bf16
  float* lse;           // [B,NH,T] log2-domain LSE
  const void* dout;     // bwd: dO [B,T,C]
  const float* dvec;    // bwd: D [B,NH,T]
  const float* packed;  // bwd: per 64-row chunk (lse[64], D[64]) [B,NH,ceil(T/64),128]
  int B, T, NH, C;
  float scale_log2;     // (1/sqrt(HS)) * log2(e)
  float scale;          // 1/sqrt(HS)
  int* status;
};

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a 128B-swizzled tile
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * ROWB + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// write 32 consecutive values (columns c0..c0+31 of `row`) as bf16 into a K-major swizzled tile
// whose row holds 64 columns
__device__ __forceinline__ void store_row32(unsigned char* tile, int row, int c0, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u;
    u.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]); u.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
    u.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]); u.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + sw128(row, c0 / 8 + j)) = u;
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y;
}

constexpr uint32_t IDESC_S_128x128 = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, 128);   // K-major x K-major
constexpr uint32_t IDESC_128x64_KK = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, 64);
constexpr uint32_t IDESC_128x64_KMN = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, 64);   // B stored [K rows, N]

// issue `nk` MMAs of K=16 over a K-major A tile and a K-major B tile (both advance 32 B per step)
__device__ __forceinline__ void mma_kk(uint32_t d, uint32_t a_addr, uint32_t b_addr, uint32_t idesc, int nk, bool acc_first) {
  const uint64_t ad = make_smem_desc(a_addr, 16, 1024), bd = make_smem_desc(b_addr, 16, 1024);
#pragma unroll
  for (int k = 0; k < nk; ++k) umma_ss<KIND_F16>(d, ad + 2 * k, bd + 2 * k, idesc, (acc_first || k > 0) ? 1u : 0u);
}
// A K-major (32 B per step), B MN-major single 64-wide chunk (16 k-rows = 2048 B per step)
__device__ __forceinline__ void mma_kmn(uint32_t d, uint32_t a_addr, uint32_t b_addr, uint32_t idesc, int nk, bool acc_first) {
  const uint64_t ad = make_smem_desc(a_addr, 16, 1024), bd = make_smem_desc(b_addr, 8192, 1024);
#pragma unroll
  for (int k = 0; k < nk; ++k) umma_ss<KIND_F16>(d, ad + 2 * k, bd + 128 * k, idesc, (acc_first || k > 0) ? 1u : 0u);
}

#define ATTN_FAIL() do { atomicExch(p.status, LLMB_ERR_TIMEOUT); fail = 1; } while (0)

// a 128-row tile is fetched as two 64-row boxes (same swizzled layout, one tensor map for every tile size)
__device__ __forceinline__ void load128(unsigned char* dst, const CUtensorMap* t, uint64_t* bar, int col, int row, int b) {
  tma_load_3d(dst, t, bar, col, row, b);
  tma_load_3d(dst + T64, t, bar, col, row + 64, b);
}

// =================================================================== forward
// No alignment slack here: 2 x (7 x 16 KB + 128 B + 1 KB reserved) must fit the SM's 228 KB, so the
// dynamic segment is declared 1024-byte aligned and the kernel verifies that before touching it.
constexpr int FWD_SMEM = T128 /*Q*/ + 2 * T128 /*K*/ + 2 * T128 /*V*/ + 2 * T128 /*P*/ + 128;

__global__ void __launch_bounds__(256, 2) attn_fwd_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  extern __shared__ __align__(1024) unsigned char smem_fwd[];
  unsigned char* sm = smem_fwd;
  if (smem_u32(sm) & 1023u) { if (threadIdx.x == 0) atomicExch(p.status, LLMB_ERR_BAD_ARG); return; }
  unsigned char* sQ = sm;
  unsigned char* sK = sQ + T128;           // 2 stages
  unsigned char* sV = sK + 2 * T128;       // 2 stages
  unsigned char* sP = sV + 2 * T128;       // two 64-column halves of P [128 x 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * T128);
  uint64_t* q_bar = bars; uint64_t* kv_bar = bars + 1; uint64_t* s_bar = bars + 3; uint64_t* o_bar = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int fail = 0, stopped = 0;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hb = warp >> 2;                // which 64-column half of S / 32-column half of O this thread owns
  const int row = (warp & 3) * 32 + lane;  // row of the tile == TMEM lane
  const int n_qt = ceil_div(p.T, TILE);
  const int qt = n_qt - 1 - blockIdx.x;    // heavy tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * TILE;

  if (tid == 0) {
    mbar_init(q_bar, 1); mbar_init(&kv_bar[0], 1); mbar_init(&kv_bar[1], 1); mbar_init(s_bar, 1); mbar_init(o_bar, 1);
    fence_barrier_init();
    prefetch_tmap(&tm);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

  const int n_kv = qt + 1;
  const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
  if (tid == 0) {
    mbar_expect_tx(q_bar, T128);
    load128(sQ, &tm, q_bar, colQ, q0, b);
    mbar_expect_tx(&kv_bar[0], 2 * T128);
    load128(sK, &tm, &kv_bar[0], colK, 0, b);
    load128(sV, &tm, &kv_bar[0], colV, 0, b);
  }

  const int qi = q0 + row;
  const float sc = p.scale_log2;
  float m_run = -INFINITY, l_run = 0.f;    // l_run: partial row sum over this thread's column half

  for (int j = 0; j < n_kv; ++j) {
    const int st = j & 1;
    if (tid == 0) {
      if (j + 1 < n_kv) {
        const int ns = (j + 1) & 1;
        mbar_expect_tx(&kv_bar[ns], 2 * T128);
        load128(sK + ns * T128, &tm, &kv_bar[ns], colK, (j + 1) * TILE, b);
        load128(sV + ns * T128, &tm, &kv_bar[ns], colV, (j + 1) * TILE, b);
      }
      bool ok = (j > 0) || mbar_wait(q_bar, 0);
      ok = ok && mbar_wait(&kv_bar[st], (j >> 1) & 1);
      if (!ok) ATTN_FAIL();
      fence_after_sync();
      mma_kk(tS, smem_u32(sQ), smem_u32(sK + st * T128), IDESC_S_128x128, HS / 16, false);
      umma_commit(s_bar);
    }
    if (!mbar_wait(s_bar, j & 1)) ATTN_FAIL();
    fence_after_sync();

    // ---- pass 1: full-row max (both threads of a row read all 128 columns; own half stays in registers)
    const bool diag = (j == n_kv - 1);
    uint32_t own[2][32];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const bool mine = (c >> 1) == hb;
      if (diag && c > (warp & 3)) {                       // chunk entirely above the diagonal for this warp
        if (mine) {
#pragma unroll
          for (int i = 0; i < 32; ++i) own[c & 1][i] = 0xff800000u;   // -inf
        }
        continue;
      }
      uint32_t r[32];
      tmem_ld32(tS + lane_addr + c * 32, r);
      tmem_wait_ld();
      if (diag && c == (warp & 3)) {
#pragma unroll
        for (int i = 0; i < 32; ++i) if (i > lane) r[i] = 0xff800000u;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      if (mine) {
#pragma unroll
        for (int i = 0; i < 32; ++i) own[c & 1][i] = r[i];
      }
    }
    const float m_new = fmaxf(m_run, mx * sc);
    const float alpha = ex2_approx(m_run - m_new);
    m_run = m_new;
    // ---- pass 2: p = 2^(s*sc - m) over the own half, row sum, P -> smem (half hb of the P tile)
    float rs = 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float e = ex2_approx(fmaf(__uint_as_float(own[c][i]), sc, -m_new));
        v[i] = e; rs += e;
      }
      store_row32(sP + hb * T128, row, c * 32, v);
    }
    l_run = l_run * alpha + rs;
    // ---- rescale the running output (this thread: 32 of the 64 columns); skipped when no row of the warp moved
    if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
      uint32_t r[32];
      tmem_ld32(tO + lane_addr + hb * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
      tmem_st32(tO + lane_addr + hb * 32, r);
      tmem_wait_st();
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      // O (+)= P V : two 64-column halves of P, V tile viewed MN-major
      mma_kmn(tO, smem_u32(sP), smem_u32(sV + st * T128), IDESC_128x64_KMN, 4, j > 0);
      mma_kmn(tO, smem_u32(sP + T128), smem_u32(sV + st * T128) + 64 * ROWB, IDESC_128x64_KMN, 4, true);
      umma_commit(o_bar);
    }
    if (!mbar_wait(o_bar, j & 1)) ATTN_FAIL();
    fence_after_sync();
    if (__syncthreads_or(fail)) { stopped = 1; break; }
  }

  // ---- epilogue: combine the two partial row sums, O / l -> bf16, LSE
  if (!stopped) {
    float* lsum = reinterpret_cast<float*>(sP);           // P is dead after the last PV product
    lsum[hb * 128 + row] = l_run;
    __syncthreads();
    const float l_tot = lsum[row] + lsum[128 + row];
    const float inv = 1.0f / l_tot;
    __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)b * p.T + qi) * p.C + h * HS + hb * 32;
    uint32_t r[32];
    tmem_ld32(tO + lane_addr + hb * 32, r);
    tmem_wait_ld();
    if (qi < p.T) {
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(r[j8 * 8 + 0]) * inv, __uint_as_float(r[j8 * 8 + 1]) * inv);
        u.y = pack_bf16x2(__uint_as_float(r[j8 * 8 + 2]) * inv, __uint_as_float(r[j8 * 8 + 3]) * inv);
        u.z = pack_bf16x2(__uint_as_float(r[j8 * 8 + 4]) * inv, __uint_as_float(r[j8 * 8 + 5]) * inv);
        u.w = pack_bf16x2(__uint_as_float(r[j8 * 8 + 6]) * inv, __uint_as_float(r[j8 * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(op + j8 * 8) = u;
      }
      if (hb == 0) p.lse[((size_t)b * p.NH + h) * p.T + qi] = m_run + log2f(l_tot);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc<256>(tmem); }
}

// =================================================================== backward: D = rowsum(dO * O)
__global__ void attn_bwd_prep_kernel(float* __restrict__ dvec, float* __restrict__ packed, const float* __restrict__ lse,
                                     const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                     int B, int T, int NH, int C) {
  // one thread per (b, h, t) with t running over whole 64-row chunks: D[b,h,t] = sum_d dO*O, plus a copy of
  // (lse, D) packed per chunk as 64 + 64 floats, which the dK/dV kernel fetches with one bulk copy per chunk
  const int n_qc = ceil_div(T, 64), Tp = n_qc * 64;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // ((b * NH + h) * Tp + t)
  long long total = (long long)B * NH * Tp;
  if (idx >= total) return;
  const int t = (int)(idx % Tp); const long long bh = idx / Tp;
  const int h = (int)(bh % NH), b = (int)(bh / NH);
  float s = 0.f, l = INFINITY;
  if (t < T) {
    const long long bt = (long long)b * T + t;
    const __nv_bfloat16* a = dout + bt * C + h * HS;
    const __nv_bfloat16* o = out + bt * C + h * HS;
#pragma unroll
    for (int j = 0; j < HS / 8; ++j) {
      Pack<__nv_bfloat16> x, y; x.load(a + j * 8); y.load(o + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) s += x.v[k] * y.v[k];
    }
    l = lse[bh * T + t];
    dvec[bh * T + t] = s;
  }
  float* pk = packed + (bh * n_qc + t / 64) * 128 + (t & 63);
  pk[0] = l; pk[64] = s;
}

// =================================================================== backward: dK, dV
constexpr int DKV_SMEM = 2 * T128 /*K,V*/ + 4 * T64 /*Q,dO x2 stages*/ + 2 * T128 /*PT,dST*/ + 4 * 64 * 4 + 1024 + 128;

__global__ void __launch_bounds__(256, 2) attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                             const __grid_constant__ CUtensorMap tmDO, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = sm;
  unsigned char* sV = sK + T128;
  unsigned char* sQ = sV + T128;          // 2 stages x 8 KB
  unsigned char* sDO = sQ + 2 * T64;      // 2 stages x 8 KB
  unsigned char* sPT = sDO + 2 * T64;     // [128 kv x 64 q]
  unsigned char* sDST = sPT + T128;
  float* sLse = reinterpret_cast<float*>(sDST + T128);   // [2][64]
  float* sD = sLse + 128;                                // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sD + 128);
  uint64_t* kv_bar = bars; uint64_t* q_bar = bars + 1; uint64_t* b1 = bars + 3; uint64_t* b2 = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int fail = 0, stopped = 0;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hb = warp >> 2;                // 32-column half of each 64-column tile this thread owns
  const int row = (warp & 3) * 32 + lane;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kv0 = kt * TILE;
  const int n_qc = ceil_div(p.T, 64);
  const int i0 = kt * 2;                  // first query chunk that can see these keys

  if (tid == 0) {
    mbar_init(kv_bar, 1); mbar_init(&q_bar[0], 1); mbar_init(&q_bar[1], 1); mbar_init(b1, 1); mbar_init(b2, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tDPT = tmem + 64, tDV = tmem + 128, tDK = tmem + 192;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

  const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
  if (tid == 0) {
    mbar_expect_tx(kv_bar, 2 * T128);
    load128(sK, &tmQKV, kv_bar, colK, kv0, b);
    load128(sV, &tmQKV, kv_bar, colV, kv0, b);
    if (i0 < n_qc) {
      mbar_expect_tx(&q_bar[0], 2 * T64);
      tma_load_3d(sQ, &tmQKV, &q_bar[0], colQ, i0 * 64, b);
      tma_load_3d(sDO, &tmDO, &q_bar[0], colQ, i0 * 64, b);
    }
  }
  const int kj = kv0 + row;
  const size_t stat_base = ((size_t)b * p.NH + h) * p.T;

  for (int i = i0, n = 0; i < n_qc; ++i, ++n) {
    const int st = n & 1;
    // per-column statistics of this chunk
    {
      const int qcol = i * 64 + (tid & 63);
      if (tid < 64) sLse[st * 64 + tid] = qcol < p.T ? p.lse[stat_base + qcol] : INFINITY;
      else if (tid < 128) sD[st * 64 + (tid & 63)] = qcol < p.T ? p.dvec[stat_base + qcol] : 0.f;
    }
    if (tid == 0) {
      if (i + 1 < n_qc) {
        const int ns = (n + 1) & 1;
        mbar_expect_tx(&q_bar[ns], 2 * T64);
        tma_load_3d(sQ + ns * T64, &tmQKV, &q_bar[ns], colQ, (i + 1) * 64, b);
        tma_load_3d(sDO + ns * T64, &tmDO, &q_bar[ns], colQ, (i + 1) * 64, b);
      }
      bool ok = (n > 0) || mbar_wait(kv_bar, 0);
      ok = ok && mbar_wait(&q_bar[st], (n >> 1) & 1);
      if (!ok) ATTN_FAIL();
      fence_after_sync();
      mma_kk(tST, smem_u32(sK), smem_u32(sQ + st * T64), IDESC_128x64_KK, HS / 16, false);     // S^T = K Q^T
      mma_kk(tDPT, smem_u32(sV), smem_u32(sDO + st * T64), IDESC_128x64_KK, HS / 16, false);   // dP^T = V dO^T
      umma_commit(b1);
    }
    __syncthreads();                       // sLse / sD visible
    if (!mbar_wait(b1, n & 1)) ATTN_FAIL();
    fence_after_sync();

    const bool need_mask = (i * 64 < kv0 + TILE);
    {
      const int c = hb;
      uint32_t rs[32], rp[32];
      tmem_ld32(tST + lane_addr + c * 32, rs);
      tmem_ld32(tDPT + lane_addr + c * 32, rp);
      tmem_wait_ld();
      float pv[32], dv[32];
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const int col = c * 32 + x;
        float pr = ex2_approx(fmaf(__uint_as_float(rs[x]), p.scale_log2, -sLse[st * 64 + col]));
        if (need_mask && (kj > i * 64 + col)) pr = 0.f;
        pv[x] = pr;
        dv[x] = pr * (__uint_as_float(rp[x]) - sD[st * 64 + col]) * p.scale;
      }
      store_row32(sPT, row, c * 32, pv);
      store_row32(sDST, row, c * 32, dv);
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      mma_kmn(tDV, smem_u32(sPT), smem_u32(sDO + st * T64), IDESC_128x64_KMN, 4, n > 0);   // dV += P^T dO
      mma_kmn(tDK, smem_u32(sDST), smem_u32(sQ + st * T64), IDESC_128x64_KMN, 4, n > 0);   // dK += dS^T Q
      umma_commit(b2);
    }
    if (!mbar_wait(b2, n & 1)) ATTN_FAIL();
    fence_after_sync();
    if (__syncthreads_or(fail)) { stopped = 1; break; }
  }

  if (!stopped) {
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)b * p.T + kj) * (3 * (size_t)p.C) + h * HS;
    const bool have = i0 < n_qc;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dp = base + (which == 0 ? 2 * p.C : p.C) + hb * 32;
      const uint32_t tsrc = which == 0 ? tDV : tDK;
      uint32_t r[32];
      tmem_ld32(tsrc + lane_addr + hb * 32, r);
      tmem_wait_ld();
      if (kj < p.T) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          uint4 u;
          if (have) {
            u.x = pack_bf16x2(__uint_as_float(r[j8 * 8 + 0]), __uint_as_float(r[j8 * 8 + 1]));
            u.y = pack_bf16x2(__uint_as_float(r[j8 * 8 + 2]), __uint_as_float(r[j8 * 8 + 3]));
            u.z = pack_bf16x2(__uint_as_float(r[j8 * 8 + 4]), __uint_as_float(r[j8 * 8 + 5]));
            u.w = pack_bf16x2(__uint_as_float(r[j8 * 8 + 6]), __uint_as_float(r[j8 * 8 + 7]));
          } else { u = make_uint4(0, 0, 0, 0); }
          *reinterpret_cast<uint4*>(dp + j8 * 8) = u;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc<256>(tmem); }
}

// =================================================================== backward: dQ
constexpr int DQ_SMEM = 2 * T128 /*Q,dO*/ + 4 * T64 /*K,V x2 stages*/ + T128 /*dS*/ + 1024 + 128;

__global__ void __launch_bounds__(256, 2) attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                            const __grid_constant__ CUtensorMap tmDO, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = sm;
  unsigned char* sDO = sQ + T128;
  unsigned char* sK = sDO + T128;         // 2 stages x 8 KB
  unsigned char* sV = sK + 2 * T64;       // 2 stages x 8 KB
  unsigned char* sDS = sV + 2 * T64;      // [128 q x 64 kv]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + T128);
  uint64_t* q_bar = bars; uint64_t* kv_bar = bars + 1; uint64_t* b1 = bars + 3; uint64_t* b2 = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int fail = 0, stopped = 0;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hb = warp >> 2;
  const int row = (warp & 3) * 32 + lane;
  const int n_qt = ceil_div(p.T, TILE);
  const int qt = n_qt - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * TILE;
  int n_kc = ceil_div(min(p.T, q0 + TILE), 64);

  if (tid == 0) {
    mbar_init(q_bar, 1); mbar_init(&kv_bar[0], 1); mbar_init(&kv_bar[1], 1); mbar_init(b1, 1); mbar_init(b2, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 64, tDQ = tmem + 128;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

  const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
  if (tid == 0) {
    mbar_expect_tx(q_bar, 2 * T128);
    load128(sQ, &tmQKV, q_bar, colQ, q0, b);
    load128(sDO, &tmDO, q_bar, colQ, q0, b);
    mbar_expect_tx(&kv_bar[0], 2 * T64);
    tma_load_3d(sK, &tmQKV, &kv_bar[0], colK, 0, b);
    tma_load_3d(sV, &tmQKV, &kv_bar[0], colV, 0, b);
  }
  const int qi = q0 + row;
  const size_t stat = ((size_t)b * p.NH + h) * p.T + qi;
  const float lse = qi < p.T ? p.lse[stat] : INFINITY;
  const float dsum = qi < p.T ? p.dvec[stat] : 0.f;

  for (int j = 0; j < n_kc; ++j) {
    const int st = j & 1;
    if (tid == 0) {
      if (j + 1 < n_kc) {
        const int ns = (j + 1) & 1;
        mbar_expect_tx(&kv_bar[ns], 2 * T64);
        tma_load_3d(sK + ns * T64, &tmQKV, &kv_bar[ns], colK, (j + 1) * 64, b);
        tma_load_3d(sV + ns * T64, &tmQKV, &kv_bar[ns], colV, (j + 1) * 64, b);
      }
      bool ok = (j > 0) || mbar_wait(q_bar, 0);
      ok = ok && mbar_wait(&kv_bar[st], (j >> 1) & 1);
      if (!ok) ATTN_FAIL();
      fence_after_sync();
      mma_kk(tS, smem_u32(sQ), smem_u32(sK + st * T64), IDESC_128x64_KK, HS / 16, false);     // S = Q K^T
      mma_kk(tDP, smem_u32(sDO), smem_u32(sV + st * T64), IDESC_128x64_KK, HS / 16, false);   // dP = dO V^T
      umma_commit(b1);
    }
    if (!mbar_wait(b1, j & 1)) ATTN_FAIL();
    fence_after_sync();
    const bool need_mask = ((j + 1) * 64 - 1 > q0);
    {
      const int c = hb;
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_addr + c * 32, rs);
      tmem_ld32(tDP + lane_addr + c * 32, rp);
      tmem_wait_ld();
      float dv[32];
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const int kcol = j * 64 + c * 32 + x;
        float pr = ex2_approx(fmaf(__uint_as_float(rs[x]), p.scale_log2, -lse));
        if (need_mask && kcol > qi) pr = 0.f;
        dv[x] = pr * (__uint_as_float(rp[x]) - dsum) * p.scale;
      }
      store_row32(sDS, row, c * 32, dv);
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      mma_kmn(tDQ, smem_u32(sDS), smem_u32(sK + st * T64), IDESC_128x64_KMN, 4, j > 0);   // dQ += dS K
      umma_commit(b2);
    }
    if (!mbar_wait(b2, j & 1)) ATTN_FAIL();
    fence_after_sync();
    if (__syncthreads_or(fail)) { stopped = 1; break; }
  }

  if (!stopped) {
    __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)b * p.T + qi) * (3 * (size_t)p.C) + h * HS + hb * 32;
    uint32_t r[32];
    tmem_ld32(tDQ + lane_addr + hb * 32, r);
    tmem_wait_ld();
    if (qi < p.T) {
#pragma unroll
      for (int j8 = 0; j8 < 4; ++j8) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(r[j8 * 8 + 0]), __uint_as_float(r[j8 * 8 + 1]));
        u.y = pack_bf16x2(__uint_as_float(r[j8 * 8 + 2]), __uint_as_float(r[j8 * 8 + 3]));
        u.z = pack_bf16x2(__uint_as_float(r[j8 * 8 + 4]), __uint_as_float(r[j8 * 8 + 5]));
        u.w = pack_bf16x2(__uint_as_float(r[j8 * 8 + 6]), __uint_as_float(r[j8 * 8 + 7]));
        *reinterpret_cast<uint4*>(dp + j8 * 8) = u;
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc<256>(tmem); }
}

// =================================================================== backward, persistent and warp-specialised
// The two kernels above run their phases one after another (MMA, wait, exponentials, barrier, MMA, wait)
// and pay the whole CTA prologue and epilogue (launch, TMEM allocation, first loads, output stores) once
// per 128-row tile, which at T = 1024 is as long as the tile's useful work.  The versions below are
// persistent - one CTA per SM walks a static list of tiles - and split the CTA into roles that only meet
// at mbarriers:
//   warp 0      TMA producer: the tile's resident operands (double-buffered, so the next tile's arrive
//               while this one computes), then 64-row chunks into a 4-deep ring that runs across tiles
//   warp 1      issues the score products (S, dP) up to two chunks ahead - also into the NEXT tile - so
//               they run while the compute warps are still in the exponentials of earlier chunks
//   warps 2..9  two groups of 128 compute threads on alternate chunks, one thread per tile row
//   warp 10     issues the accumulating products (dQ, or dV and dK); a second issuing warp because the
//               wait - fence - issue - commit chain of one warp alone takes longer than a chunk's math
// S / dP live in two TMEM buffers each, the bf16 operand tiles written by the compute warps in two
// shared-memory buffers each, and the output accumulators in two TMEM buffers, so the tensor core, the
// MUFU pipe, the loads and the output stores all work on different chunks or tiles at the same time.
// Tiles are handed out in pairs (heaviest with lightest) so that every work item costs the same and a
// static round-robin over the CTAs is balanced; the two tiles of an item and consecutive items belong to
// the same (batch, head), which keeps K/V (or Q/dO) in L2.  Results do not depend on the schedule: every
// output tile is produced by exactly one CTA in a fixed order.
constexpr int BW_THREADS = 352;                        // producer, score issuer, 8 compute warps, accumulate issuer
constexpr int BW_ACC_WARP = 10;

#define BW_FAIL() do { atomicExch(p.status, LLMB_ERR_TIMEOUT); failed = true; } while (0)

struct TileCursor {
  int w, sub;        // work item; 0 = heavy tile of the pair, 1 = light tile
  int t, g;          // tiles / chunks this role has consumed so far (select buffers and barrier phases)
  int bh, tile;      // current tile: (batch * NH + head), tile index along T
  bool done;
};
// n_t tiles along T, n_items = ceil(n_t / 2) * B * NH work items; `heavy_low`: tile 0 is the heaviest
__device__ __forceinline__ void cursor_seek(TileCursor& c, int n_t, int n_items, bool heavy_low, int stride = 0) {
  const int n_pairs = (n_t + 1) / 2;
  if (stride == 0) stride = gridDim.x;
  for (;;) {
    if (c.w >= n_items) { c.done = true; return; }
    const int x = c.w % n_pairs;
    c.bh = c.w / n_pairs;
    const int lo = x, hi = n_t - 1 - x;
    if (c.sub == 0) { c.tile = heavy_low ? lo : hi; return; }
    if (lo != hi) { c.tile = heavy_low ? hi : lo; return; }
    c.w += stride; c.sub = 0;
  }
}
__device__ __forceinline__ TileCursor cursor_begin(int n_t, int n_items, bool heavy_low) {
  TileCursor c{(int)blockIdx.x, 0, 0, 0, 0, 0, false};
  cursor_seek(c, n_t, n_items, heavy_low);
  return c;
}
__device__ __forceinline__ void cursor_next(TileCursor& c, int chunks, int n_t, int n_items, bool heavy_low, int stride = 0) {
  if (stride == 0) stride = gridDim.x;
  c.t += 1; c.g += chunks;
  if (c.sub == 0) c.sub = 1; else { c.sub = 0; c.w += stride; }
  cursor_seek(c, n_t, n_items, heavy_low, stride);
}
// a CTA may run several independent tile streams: stream `vid` of `vgrid`
__device__ __forceinline__ TileCursor cursor_begin_v(int vid, int vgrid, int n_t, int n_items, bool heavy_low) {
  TileCursor c{vid, 0, 0, 0, 0, 0, false};
  cursor_seek(c, n_t, n_items, heavy_low, vgrid);
  return c;
}

// ------------------------------------------------------------------- forward, persistent
// One CTA per SM runs TWO independent tile streams (groups): each group has its own TMA producer warp, its
// own issuing warp and four softmax warps (one thread per query row), its own Q / K,V ring / P buffers and
// its own TMEM columns, so the online-softmax chain of one group's tile never waits on the other's, and the
// tensor core, both groups' MUFU work and the loads overlap.  Keys are taken in chunks of 64:
//   S(j) = Q K_j^T (TMEM, double-buffered) -> softmax warps: row max, p = 2^(s - m), row sum, P(j) as bf16
//   into shared memory (the running output in TMEM is rescaled only when a row's maximum grew by more than
//   2^8) -> O += P(j) V_j.  The issuing warp keeps S two chunks ahead of the softmax warps.
// warps: 0 producer A, 1 issuer A, 2 issuer B, 3 producer B, 4..7 softmax A, 8..11 softmax B.
constexpr int FW_NS = 4;                                 // K/V chunk ring depth per group
constexpr int FW_THREADS = 384;
constexpr int FW_GROUP_SMEM = 2 * T128 /*Q x2*/ + FW_NS * 2 * T64 /*K,V ring*/ + T128 /*P*/;
constexpr int FWD2_SMEM = 2 * FW_GROUP_SMEM + 1024 + 512;

__global__ void __launch_bounds__(FW_THREADS, 1) attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int grp = (warp == 0 || warp == 1 || (warp >= 4 && warp < 8)) ? 0 : 1;
  unsigned char* gs = sm + grp * FW_GROUP_SMEM;
  unsigned char* sQ = gs;                        // two buffers
  unsigned char* sKV = sQ + 2 * T128;            // ring: stage s holds the K chunk at +0, the V chunk at +T64
  unsigned char* sP = sKV + FW_NS * 2 * T64;     // [128 q x 64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + 2 * FW_GROUP_SMEM) + grp * 24;
  uint64_t* q_full = bars;                       // [2]
  uint64_t* q_empty = q_full + 2;                // [2] the tile's last score product is complete
  uint64_t* kv_full = q_empty + 2;               // [NS]
  uint64_t* kv_empty = kv_full + FW_NS;          // [NS] O += P V of the chunk is complete (stage, P buffer and O are free)
  uint64_t* s_full = kv_empty + FW_NS;           // [2]
  uint64_t* p_full = s_full + 2;                 // P(j) written (and S(j) read)
  uint64_t* o_free = p_full + 1;                 // the tile's output has been read out of TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + 2 * FW_GROUP_SMEM + 2 * 24 * 8);

  const int n_t = ceil_div(p.T, TILE);
  const int n_items = ((n_t + 1) / 2) * p.B * p.NH;
  const int vid = 2 * blockIdx.x + grp, vgrid = 2 * gridDim.x;
  auto chunks_of = [&](int qt) { return ceil_div(min(p.T, (qt + 1) * TILE), 64); };

  if (tid == 0) {
    uint64_t* b0 = reinterpret_cast<uint64_t*>(sm + 2 * FW_GROUP_SMEM);
    for (int g = 0; g < 2; ++g) {
      uint64_t* b = b0 + g * 24;
      for (int i = 0; i < 2; ++i) { mbar_init(&b[i], 1); mbar_init(&b[2 + i], 1); mbar_init(&b[4 + 2 * FW_NS + i], 1); }
      for (int i = 0; i < FW_NS; ++i) { mbar_init(&b[4 + i], 1); mbar_init(&b[4 + FW_NS + i], 1); }
      mbar_init(&b[4 + 2 * FW_NS + 2], 4);       // p_full: four softmax warps
      mbar_init(&b[4 + 2 * FW_NS + 3], 4);       // o_free
    }
    fence_barrier_init();
    prefetch_tmap(&tm);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot + grp * 256;
  const uint32_t tS = tmem, tO = tmem + 128;             // S: two 64-column buffers; O: 64 columns
  bool failed = false;

  if (warp == 0 || warp == 3) {
    // ------------------------------------------------------------ TMA producer of this group
    for (TileCursor c = cursor_begin_v(vid, vgrid, n_t, n_items, false); !c.done && !failed;) {
      const int b = c.bh / p.NH, h = c.bh % p.NH, qb = c.t & 1, n_kc = chunks_of(c.tile);
      const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
      if (c.t >= 2 && !mbar_wait(&q_empty[qb], ((c.t >> 1) + 1) & 1)) { BW_FAIL(); break; }
      if (elect_one()) {
        mbar_expect_tx(&q_full[qb], T128);
        load128(sQ + qb * T128, &tm, &q_full[qb], colQ, c.tile * TILE, b);
      }
      __syncwarp();
      for (int j = 0; j < n_kc; ++j) {
        const int g = c.g + j, st = g % FW_NS;
        if (g >= FW_NS && !mbar_wait(&kv_empty[st], ((g / FW_NS) + 1) & 1)) { BW_FAIL(); break; }
        if (elect_one()) {
          mbar_expect_tx(&kv_full[st], 2 * T64);
          tma_load_3d(sKV + st * 2 * T64, &tm, &kv_full[st], colK, j * 64, b);
          tma_load_3d(sKV + st * 2 * T64 + T64, &tm, &kv_full[st], colV, j * 64, b);
        }
        __syncwarp();
      }
      cursor_next(c, n_kc, n_t, n_items, false, vgrid);
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------------------ MMA issuer of this group
    // fixed pipeline per tile: S(0), S(1); then for every chunk: wait P(j) -> O += P(j) V_j -> S(j + 2)
    for (TileCursor c = cursor_begin_v(vid, vgrid, n_t, n_items, false); !c.done && !failed;) {
      const int qb = c.t & 1, n_kc = chunks_of(c.tile);
      const uint32_t q_addr = smem_u32(sQ + qb * T128);
      if (!mbar_wait(&q_full[qb], (c.t >> 1) & 1)) { BW_FAIL(); break; }
      auto issue_s = [&](int j) {
        const int g = c.g + j, st = g % FW_NS;
        if (!mbar_wait(&kv_full[st], (g / FW_NS) & 1)) { BW_FAIL(); return; }
        fence_after_sync();
        if (elect_one()) {
          mma_kk(tS + (g & 1) * 64, q_addr, smem_u32(sKV + st * 2 * T64), IDESC_128x64_KK, HS / 16, false);   // S = Q K^T
          umma_commit(&s_full[g & 1]);
          if (j == n_kc - 1) umma_commit(&q_empty[qb]);
        }
        __syncwarp();
      };
      issue_s(0);
      if (n_kc > 1 && !failed) issue_s(1);
      // the previous tile's output must have left TMEM before this tile's first product overwrites it
      if (c.t >= 1 && !failed && !mbar_wait(o_free, (c.t + 1) & 1)) BW_FAIL();
      for (int j = 0; j < n_kc && !failed; ++j) {
        const int g = c.g + j, st = g % FW_NS;
        if (!mbar_wait(p_full, g & 1)) { BW_FAIL(); break; }
        fence_after_sync();
        if (elect_one()) {
          mma_kmn(tO, smem_u32(sP), smem_u32(sKV + st * 2 * T64 + T64), IDESC_128x64_KMN, 4, j > 0);   // O (+)= P V
          umma_commit(&kv_empty[st]);
        }
        __syncwarp();
        if (j + 2 < n_kc) issue_s(j + 2);
      }
      cursor_next(c, n_kc, n_t, n_items, false, vgrid);
    }
  } else {
    // ------------------------------------------------------------ softmax warps: one thread per query row
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale_log2;
    for (TileCursor c = cursor_begin_v(vid, vgrid, n_t, n_items, false); !c.done && !failed;) {
      const int b = c.bh / p.NH, h = c.bh % p.NH, q0 = c.tile * TILE, qi = q0 + row, n_kc = chunks_of(c.tile);
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_kc; ++j) {
        const int g = c.g + j;
        if (!mbar_wait(&s_full[g & 1], (g >> 1) & 1)) { BW_FAIL(); break; }
        fence_after_sync();
        uint32_t r0[32], r1[32];
        tmem_ld32(tS + (g & 1) * 64 + lane_addr, r0);
        tmem_ld32(tS + (g & 1) * 64 + lane_addr + 32, r1);
        tmem_wait_ld();
        fence_before_sync();
        if ((j + 1) * 64 - 1 > q0) {                    // chunk touches the diagonal: mask keys after the query
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            if (j * 64 + x > qi) r0[x] = 0xff800000u;
            if (j * 64 + 32 + x > qi) r1[x] = 0xff800000u;
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int x = 0; x < 32; ++x) mx = fmaxf(mx, fmaxf(__uint_as_float(r0[x]), __uint_as_float(r1[x])));
        // the running maximum only moves when it grew by more than 8 (a factor 256 in p): rescales of O become rare
        float m_new = fmaxf(m_run, mx * sc);
        if (m_new - m_run <= 8.0f) m_new = m_run;
        const float alpha = ex2_approx(m_run - m_new);   // m_run = -inf on the first chunk gives 0
        m_run = m_new;
        float rs = 0.f;
        uint32_t pk[32];                                 // 64 probabilities as bf16 pairs
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(r0[2 * x]), sc, -m_new));
          const float e1 = ex2_approx(fmaf(__uint_as_float(r0[2 * x + 1]), sc, -m_new));
          const float e2 = ex2_approx(fmaf(__uint_as_float(r1[2 * x]), sc, -m_new));
          const float e3 = ex2_approx(fmaf(__uint_as_float(r1[2 * x + 1]), sc, -m_new));
          rs += (e0 + e1) + (e2 + e3);
          pk[x] = pack_bf16x2(e0, e1);
          pk[16 + x] = pack_bf16x2(e2, e3);
        }
        l_run = l_run * alpha + rs;
        // O += P(j-1) V must be complete before O is rescaled and before P is overwritten
        if (g >= 1 && !mbar_wait(&kv_empty[(g - 1) % FW_NS], ((g - 1) / FW_NS) & 1)) { BW_FAIL(); break; }
        if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
          fence_after_sync();
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            uint32_t o[32];
            tmem_ld32(tO + lane_addr + half * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
            tmem_st32(tO + lane_addr + half * 32, o);
          }
          tmem_wait_st();
          fence_before_sync();
        }
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8)
          *reinterpret_cast<uint4*>(sP + sw128(row, c8)) = make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      if (failed) break;
      // tile epilogue: O / l -> bf16, log-sum-exp
      const int gl = c.g + n_kc - 1;
      if (!mbar_wait(&kv_empty[gl % FW_NS], (gl / FW_NS) & 1)) { BW_FAIL(); break; }
      fence_after_sync();
      uint32_t o0[32], o1[32];
      tmem_ld32(tO + lane_addr, o0);
      tmem_ld32(tO + lane_addr + 32, o1);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
      if (qi < p.T) {
        const float inv = 1.0f / l_run;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)b * p.T + qi) * p.C + h * HS;
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(o0[j8 * 8 + 0]) * inv, __uint_as_float(o0[j8 * 8 + 1]) * inv);
          u.y = pack_bf16x2(__uint_as_float(o0[j8 * 8 + 2]) * inv, __uint_as_float(o0[j8 * 8 + 3]) * inv);
          u.z = pack_bf16x2(__uint_as_float(o0[j8 * 8 + 4]) * inv, __uint_as_float(o0[j8 * 8 + 5]) * inv);
          u.w = pack_bf16x2(__uint_as_float(o0[j8 * 8 + 6]) * inv, __uint_as_float(o0[j8 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(op + j8 * 8) = u;
          u.x = pack_bf16x2(__uint_as_float(o1[j8 * 8 + 0]) * inv, __uint_as_float(o1[j8 * 8 + 1]) * inv);
          u.y = pack_bf16x2(__uint_as_float(o1[j8 * 8 + 2]) * inv, __uint_as_float(o1[j8 * 8 + 3]) * inv);
          u.z = pack_bf16x2(__uint_as_float(o1[j8 * 8 + 4]) * inv, __uint_as_float(o1[j8 * 8 + 5]) * inv);
          u.w = pack_bf16x2(__uint_as_float(o1[j8 * 8 + 6]) * inv, __uint_as_float(o1[j8 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(op + 32 + j8 * 8) = u;
        }
        p.lse[(size_t)c.bh * p.T + qi] = m_run + log2f(l_run);
      }
      cursor_next(c, n_kc, n_t, n_items, false, vgrid);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc<512>(*tmem_slot); }
}

// ------------------------------------------------------------------- dQ
constexpr int DQ_NS = 6;                                // chunk ring depth
constexpr int DQ2_SMEM = 4 * T128 /*Q,dO x2*/ + DQ_NS * 2 * T64 /*K,V ring*/ + 2 * T128 /*dS x2*/ + 1024 + 256;

__global__ void __launch_bounds__(BW_THREADS, 1) attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                    const __grid_constant__ CUtensorMap tmDO, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQO = sm;                 // resident buffer r: Q at r*2*T128, dO at +T128
  unsigned char* sKV = sQO + 4 * T128;     // ring: stage s holds the K chunk at +0, the V chunk at +T64
  unsigned char* sDS = sKV + DQ_NS * 2 * T64;   // two buffers [128 q x 64 kv]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * T128);
  uint64_t* r_full = bars;                       // [2] Q and dO landed
  uint64_t* r_empty = r_full + 2;                // [2] the last product reading them is complete
  uint64_t* kv_full = r_empty + 2;               // [NS]
  uint64_t* kv_empty = kv_full + DQ_NS;          // [NS] the dQ product that read the stage (and its dS tile) is complete
  uint64_t* sdp_full = kv_empty + DQ_NS;         // [2] S and dP of a chunk are in TMEM
  uint64_t* sdp_free = sdp_full + 2;             // [2] all compute warps hold S and dP in registers
  uint64_t* ds_full = sdp_free + 2;              // [2] dS tile written
  uint64_t* acc_full = ds_full + 2;              // [2] dQ of a tile complete
  uint64_t* acc_free = acc_full + 2;             // [2] all compute warps hold it in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_t = ceil_div(p.T, TILE);
  const int n_items = ((n_t + 1) / 2) * p.B * p.NH;
  auto chunks_of = [&](int qt) { return ceil_div(min(p.T, (qt + 1) * TILE), 64); };

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&r_full[s], 1); mbar_init(&r_empty[s], 1);
      mbar_init(&sdp_full[s], 1); mbar_init(&sdp_free[s], 4); mbar_init(&ds_full[s], 4);
      mbar_init(&acc_full[s], 1); mbar_init(&acc_free[s], 8);
    }
    for (int s = 0; s < DQ_NS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;     // two 64-column buffers each
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {
      for (TileCursor c = cursor_begin(n_t, n_items, false); !c.done && !failed;) {
        const int b = c.bh / p.NH, h = c.bh % p.NH, rb = c.t & 1, n_kc = chunks_of(c.tile);
        const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
        if (c.sub == 0 && c.w + (int)gridDim.x < n_items) {
          // the next work item belongs to another (batch, head): start pulling its K, V, Q and dO into L2 now
          const int nw = c.w + gridDim.x, n_pairs = (n_t + 1) / 2, nbh = nw / n_pairs, nqt = n_t - 1 - nw % n_pairs;
          const int nb = nbh / p.NH, nh = nbh % p.NH;
          for (int j = 0; j < chunks_of(nqt); ++j) {
            tma_prefetch_l2_3d(&tmQKV, p.C + nh * HS, j * 64, nb);
            tma_prefetch_l2_3d(&tmQKV, 2 * p.C + nh * HS, j * 64, nb);
            tma_prefetch_l2_3d(&tmQKV, nh * HS, j * 64, nb);
            tma_prefetch_l2_3d(&tmDO, nh * HS, j * 64, nb);
          }
        }
        if (c.t >= 2 && !mbar_wait(&r_empty[rb], ((c.t >> 1) + 1) & 1)) { BW_FAIL(); break; }
        mbar_expect_tx(&r_full[rb], 2 * T128);
        load128(sQO + rb * 2 * T128, &tmQKV, &r_full[rb], colQ, c.tile * TILE, b);
        load128(sQO + rb * 2 * T128 + T128, &tmDO, &r_full[rb], colQ, c.tile * TILE, b);
        for (int j = 0; j < n_kc; ++j) {
          const int g = c.g + j, st = g % DQ_NS;
          if (g >= DQ_NS && !mbar_wait(&kv_empty[st], ((g / DQ_NS) + 1) & 1)) { BW_FAIL(); break; }
          mbar_expect_tx(&kv_full[st], 2 * T64);
          tma_load_3d(sKV + st * 2 * T64, &tmQKV, &kv_full[st], colK, j * 64, b);
          tma_load_3d(sKV + st * 2 * T64 + T64, &tmQKV, &kv_full[st], colV, j * 64, b);
        }
        cursor_next(c, n_kc, n_t, n_items, false);
      }
    }
  } else if (warp == 1) {
    // score products S = Q K^T and dP = dO V^T, up to two chunks ahead of the compute warps.  The whole warp
    // walks the loop (uniform control flow); one elected lane issues.
    int js = 0;
    for (TileCursor cs = cursor_begin(n_t, n_items, false); !cs.done && !failed;) {
      const int g = cs.g + js, bf = g & 1, st = g % DQ_NS, rb = cs.t & 1;
      const int n_kc = chunks_of(cs.tile);
      const bool last = js + 1 == n_kc;
      if (js == 0 && !mbar_wait(&r_full[rb], (cs.t >> 1) & 1)) { BW_FAIL(); break; }
      if (!mbar_wait(&kv_full[st], (g / DQ_NS) & 1)) { BW_FAIL(); break; }
      if (g >= 2 && !mbar_wait(&sdp_free[bf], ((g >> 1) + 1) & 1)) { BW_FAIL(); break; }   // S(g-2) / dP(g-2) are in registers
      fence_after_sync();
      const uint32_t q_addr = smem_u32(sQO + rb * 2 * T128), k_addr = smem_u32(sKV + st * 2 * T64);
      if (elect_one()) {
        mma_kk(tS + bf * 64, q_addr, k_addr, IDESC_128x64_KK, HS / 16, false);                    // S = Q K^T
        mma_kk(tDP + bf * 64, q_addr + T128, k_addr + T64, IDESC_128x64_KK, HS / 16, false);      // dP = dO V^T
        umma_commit(&sdp_full[bf]);
        if (last) umma_commit(&r_empty[rb]);
      }
      __syncwarp();
      if (last) { js = 0; cursor_next(cs, n_kc, n_t, n_items, false); } else ++js;
    }
  } else if (warp == BW_ACC_WARP) {
    // accumulating product dQ += dS K, issued by its own warp so that neither issue loop waits for the other
    int ja = 0;
    for (TileCursor ca = cursor_begin(n_t, n_items, false); !ca.done && !failed;) {
      const int g = ca.g + ja, bf = g & 1, st = g % DQ_NS, ab = ca.t & 1;
      const int n_kc = chunks_of(ca.tile);
      const bool last = ja + 1 == n_kc;
      if (ja == 0 && ca.t >= 2 && !mbar_wait(&acc_free[ab], ((ca.t >> 1) + 1) & 1)) { BW_FAIL(); break; }
      if (!mbar_wait(&ds_full[bf], (g >> 1) & 1)) { BW_FAIL(); break; }
      fence_after_sync();
      if (elect_one()) {
        mma_kmn(tDQ + ab * 64, smem_u32(sDS + bf * T128), smem_u32(sKV + st * 2 * T64), IDESC_128x64_KMN, 4, ja > 0);   // dQ += dS K
        umma_commit(&kv_empty[st]);          // frees the K/V stage and the dS buffer
        if (last) umma_commit(&acc_full[ab]);
      }
      __syncwarp();
      if (last) { ja = 0; cursor_next(ca, n_kc, n_t, n_items, false); } else ++ja;
    }
  } else {
    // Two groups of four warps take alternate chunks (group = chunk parity = S/dP/dS buffer index), one thread
    // per tile row and all 64 columns of the chunk: while one group waits for its scores, loads them or
    // stores dS, the other has the MUFU pipe of every SM sub-partition to itself.
    const int grp = (warp - 2) >> 2;
    const int row = (warp & 3) * 32 + lane;  // tile row == TMEM lane (a warp may only touch lane quarter warp % 4)
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    TileCursor c = cursor_begin(n_t, n_items, false);
    float lse = INFINITY, dsum = 0.f;
    auto load_stats = [&](const TileCursor& cc, float& l, float& d) {
      const int qi = cc.tile * TILE + row;
      const size_t stat = (size_t)cc.bh * p.T + qi;
      l = (!cc.done && qi < p.T) ? p.lse[stat] : INFINITY;
      d = (!cc.done && qi < p.T) ? p.dvec[stat] : 0.f;
    };
    // The output of a tile is written after the first chunk of the NEXT tile, when its last dQ product has
    // long completed; each thread stores 32 of its row's 64 columns (half `grp`).
    bool pend = false; int pend_t = 0, pend_qi = 0, pend_b = 0, pend_h = 0;
    auto epilogue = [&]() {
      const int ab = pend_t & 1;
      pend = false;
      if (!mbar_wait(&acc_full[ab], (pend_t >> 1) & 1)) { BW_FAIL(); return; }
      fence_after_sync();
      uint32_t r[32];
      tmem_ld32(tDQ + ab * 64 + lane_addr + grp * 32, r);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[ab]);
      if (pend_qi < p.T) {
        __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)pend_b * p.T + pend_qi) * (3 * (size_t)p.C) + pend_h * HS + grp * 32;
        const float sc = p.scale;             // dS was stored without the 1/sqrt(HS) factor
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(r[j8 * 8 + 0]) * sc, __uint_as_float(r[j8 * 8 + 1]) * sc);
          u.y = pack_bf16x2(__uint_as_float(r[j8 * 8 + 2]) * sc, __uint_as_float(r[j8 * 8 + 3]) * sc);
          u.z = pack_bf16x2(__uint_as_float(r[j8 * 8 + 4]) * sc, __uint_as_float(r[j8 * 8 + 5]) * sc);
          u.w = pack_bf16x2(__uint_as_float(r[j8 * 8 + 6]) * sc, __uint_as_float(r[j8 * 8 + 7]) * sc);
          *reinterpret_cast<uint4*>(dp + j8 * 8) = u;
        }
      }
    };
    load_stats(c, lse, dsum);
    while (!c.done && !failed) {
      const int b = c.bh / p.NH, h = c.bh % p.NH, q0 = c.tile * TILE, qi = q0 + row, n_kc = chunks_of(c.tile);
      TileCursor cn = c;
      cursor_next(cn, n_kc, n_t, n_items, false);
      float lse_n, dsum_n;
      load_stats(cn, lse_n, dsum_n);          // the next tile's row statistics travel while this tile computes
      for (int j = 0; j < n_kc && !failed; ++j) {
        const int g = c.g + j, bf = grp;
        if ((g & 1) != grp) continue;         // the other group's chunk
        if (!mbar_wait(&sdp_full[bf], (g >> 1) & 1)) { BW_FAIL(); break; }
        fence_after_sync();
        const bool need_mask = ((j + 1) * 64 - 1 > q0);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t rs[32], rp[32];
          tmem_ld32(tS + bf * 64 + lane_addr + half * 32, rs);
          tmem_ld32(tDP + bf * 64 + lane_addr + half * 32, rp);
          tmem_wait_ld();
          if (half == 1) {                    // S and dP of this chunk are in registers: the buffer can take chunk g + 2
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sdp_free[bf]);
          }
          float dv[32];
          if (need_mask) {                    // chunk on the diagonal: keys after the query contribute nothing
            const int lim = qi - (j * 64 + half * 32);      // columns x > lim are masked
#pragma unroll
            for (int x = 0; x < 32; ++x) {
              const float pr = x > lim ? 0.f : ex2_approx(fmaf(__uint_as_float(rs[x]), p.scale_log2, -lse));
              dv[x] = pr * (__uint_as_float(rp[x]) - dsum);
            }
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              dv[x] = ex2_approx(fmaf(__uint_as_float(rs[x]), p.scale_log2, -lse)) * (__uint_as_float(rp[x]) - dsum);
          }
          // dQ product of chunk g-2 done: the dS buffer is free
          if (half == 0 && g >= 2 && !mbar_wait(&kv_empty[(g - 2) % DQ_NS], ((g - 2) / DQ_NS) & 1)) { BW_FAIL(); break; }
          store_row32(sDS + bf * T128, row, half * 32, dv);
        }
        if (failed) break;
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_full[bf]);
        if (pend) epilogue();
      }
      if (failed) break;
      if (pend) epilogue();                   // this group had no chunk in the tile
      pend = true; pend_t = c.t; pend_qi = qi; pend_b = b; pend_h = h;
      c = cn; lse = lse_n; dsum = dsum_n;
    }
    if (pend && !failed) epilogue();
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc<512>(tmem); }
}

// ------------------------------------------------------------------- dK, dV
constexpr int DKV_NS = 5;
constexpr int DKV2_SMEM = 4 * T128 /*K,V x2*/ + DKV_NS * 2 * T64 /*Q,dO ring*/ + 4 * T128 /*P^T x2, dS^T x2*/ +
                          DKV_NS * 128 * 4 /*lse, D per chunk*/ + 1024 + 256;

__global__ void __launch_bounds__(BW_THREADS, 1) attn_bwd_dkv2_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                     const __grid_constant__ CUtensorMap tmDO, const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sKVr = sm;                // resident buffer r: K at r*2*T128, V at +T128
  unsigned char* sQD = sKVr + 4 * T128;    // ring: stage s holds the Q chunk at +0, the dO chunk at +T64
  unsigned char* sPT = sQD + DKV_NS * 2 * T64;    // two buffers [128 kv x 64 q]
  unsigned char* sDST = sPT + 2 * T128;          // two buffers
  float* sStat = reinterpret_cast<float*>(sDST + 2 * T128);   // per stage: 64 x lse, 64 x D
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + DKV_NS * 128);
  uint64_t* r_full = bars;                       // [2] K and V landed
  uint64_t* r_empty = r_full + 2;                // [2]
  uint64_t* q_full = r_empty + 2;                // [NS] Q chunk, dO chunk and row statistics landed
  uint64_t* q_empty = q_full + DKV_NS;            // [NS]
  uint64_t* st_full = q_empty + DKV_NS;           // [2] S^T and dP^T of a chunk are in TMEM
  uint64_t* st_free = st_full + 2;               // [2] all compute warps hold S^T and dP^T in registers
  uint64_t* pd_full = st_free + 2;               // [2] P^T and dS^T tiles written
  uint64_t* acc_full = pd_full + 2;              // [2] dV and dK of a tile complete
  uint64_t* acc_free = acc_full + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_t = ceil_div(p.T, TILE);
  const int n_items = ((n_t + 1) / 2) * p.B * p.NH;
  const int n_qc = ceil_div(p.T, 64);
  auto chunks_of = [&](int kt) { return n_qc - 2 * kt; };   // query chunks that can see key tile kt

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&r_full[s], 1); mbar_init(&r_empty[s], 1);
      mbar_init(&st_full[s], 1); mbar_init(&st_free[s], 4); mbar_init(&pd_full[s], 4);
      mbar_init(&acc_full[s], 1); mbar_init(&acc_free[s], 8);
    }
    for (int s = 0; s < DKV_NS; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tDPT = tmem + 128, tACC = tmem + 256;   // accumulator buffer a: dV at a*128, dK at +64
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {
      for (TileCursor c = cursor_begin(n_t, n_items, true); !c.done && !failed;) {
        const int b = c.bh / p.NH, h = c.bh % p.NH, rb = c.t & 1, n_ch = chunks_of(c.tile), i0 = 2 * c.tile;
        const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
        if (c.sub == 0 && c.w + (int)gridDim.x < n_items) {
          // the next work item belongs to another (batch, head): start pulling its K, V, Q and dO into L2 now
          const int nw = c.w + gridDim.x, n_pairs = (n_t + 1) / 2, nbh = nw / n_pairs, nkt = nw % n_pairs;
          const int nb = nbh / p.NH, nh = nbh % p.NH;
          for (int i = 2 * nkt; i < n_qc; ++i) {
            tma_prefetch_l2_3d(&tmQKV, p.C + nh * HS, i * 64, nb);
            tma_prefetch_l2_3d(&tmQKV, 2 * p.C + nh * HS, i * 64, nb);
            tma_prefetch_l2_3d(&tmQKV, nh * HS, i * 64, nb);
            tma_prefetch_l2_3d(&tmDO, nh * HS, i * 64, nb);
          }
        }
        if (c.t >= 2 && !mbar_wait(&r_empty[rb], ((c.t >> 1) + 1) & 1)) { BW_FAIL(); break; }
        mbar_expect_tx(&r_full[rb], 2 * T128);
        load128(sKVr + rb * 2 * T128, &tmQKV, &r_full[rb], colK, c.tile * TILE, b);
        load128(sKVr + rb * 2 * T128 + T128, &tmQKV, &r_full[rb], colV, c.tile * TILE, b);
        const float* stats = p.packed + ((size_t)c.bh * n_qc + i0) * 128;
        for (int n = 0; n < n_ch; ++n) {
          const int g = c.g + n, st = g % DKV_NS, i = i0 + n;
          if (g >= DKV_NS && !mbar_wait(&q_empty[st], ((g / DKV_NS) + 1) & 1)) { BW_FAIL(); break; }
          mbar_expect_tx(&q_full[st], 2 * T64 + 512);
          tma_load_3d(sQD + st * 2 * T64, &tmQKV, &q_full[st], colQ, i * 64, b);
          tma_load_3d(sQD + st * 2 * T64 + T64, &tmDO, &q_full[st], colQ, i * 64, b);
          bulk_load_1d(sStat + st * 128, stats + (size_t)n * 128, 512, &q_full[st]);
        }
        cursor_next(c, n_ch, n_t, n_items, true);
      }
    }
  } else if (warp == 1) {
    // score products S^T = K Q^T and dP^T = V dO^T, up to two chunks ahead of the compute warps
    int js = 0;
    for (TileCursor cs = cursor_begin(n_t, n_items, true); !cs.done && !failed;) {
      const int g = cs.g + js, bf = g & 1, st = g % DKV_NS, rb = cs.t & 1;
      const int n_ch = chunks_of(cs.tile);
      const bool last = js + 1 == n_ch;
      if (js == 0 && !mbar_wait(&r_full[rb], (cs.t >> 1) & 1)) { BW_FAIL(); break; }
      if (!mbar_wait(&q_full[st], (g / DKV_NS) & 1)) { BW_FAIL(); break; }
      if (g >= 2 && !mbar_wait(&st_free[bf], ((g >> 1) + 1) & 1)) { BW_FAIL(); break; }   // S^T(g-2) / dP^T(g-2) are in registers
      fence_after_sync();
      const uint32_t k_addr = smem_u32(sKVr + rb * 2 * T128), q_addr = smem_u32(sQD + st * 2 * T64);
      if (elect_one()) {
        mma_kk(tST + bf * 64, k_addr, q_addr, IDESC_128x64_KK, HS / 16, false);                     // S^T = K Q^T
        mma_kk(tDPT + bf * 64, k_addr + T128, q_addr + T64, IDESC_128x64_KK, HS / 16, false);       // dP^T = V dO^T
        umma_commit(&st_full[bf]);
        if (last) umma_commit(&r_empty[rb]);
      }
      __syncwarp();
      if (last) { js = 0; cursor_next(cs, n_ch, n_t, n_items, true); } else ++js;
    }
  } else if (warp == BW_ACC_WARP) {
    // accumulating products dV += P^T dO and dK += dS^T Q, issued by their own warp
    int ja = 0;
    for (TileCursor ca = cursor_begin(n_t, n_items, true); !ca.done && !failed;) {
      const int g = ca.g + ja, bf = g & 1, st = g % DKV_NS, ab = ca.t & 1;
      const int n_ch = chunks_of(ca.tile);
      const bool last = ja + 1 == n_ch;
      if (ja == 0 && ca.t >= 2 && !mbar_wait(&acc_free[ab], ((ca.t >> 1) + 1) & 1)) { BW_FAIL(); break; }
      if (!mbar_wait(&pd_full[bf], (g >> 1) & 1)) { BW_FAIL(); break; }
      fence_after_sync();
      const uint32_t q_addr = smem_u32(sQD + st * 2 * T64);
      if (elect_one()) {
        mma_kmn(tACC + ab * 128, smem_u32(sPT + bf * T128), q_addr + T64, IDESC_128x64_KMN, 4, ja > 0);        // dV += P^T dO
        mma_kmn(tACC + ab * 128 + 64, smem_u32(sDST + bf * T128), q_addr, IDESC_128x64_KMN, 4, ja > 0);        // dK += dS^T Q
        umma_commit(&q_empty[st]);           // frees the Q/dO stage and the P^T / dS^T buffers
        if (last) umma_commit(&acc_full[ab]);
      }
      __syncwarp();
      if (last) { ja = 0; cursor_next(ca, n_ch, n_t, n_items, true); } else ++ja;
    }
  } else {
    // two groups of four warps on alternate chunks, one thread per key row and all 64 query columns of the chunk
    const int grp = (warp - 2) >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    // the outputs of a tile are written after the first chunk of the NEXT tile (32 of the 64 columns per thread)
    bool pend = false; int pend_t = 0, pend_kj = 0, pend_b = 0, pend_h = 0;
    auto epilogue = [&]() {
      const int ab = pend_t & 1;
      pend = false;
      if (!mbar_wait(&acc_full[ab], (pend_t >> 1) & 1)) { BW_FAIL(); return; }
      fence_after_sync();
      uint32_t rv[32], rk[32];
      tmem_ld32(tACC + ab * 128 + lane_addr + grp * 32, rv);
      tmem_ld32(tACC + ab * 128 + 64 + lane_addr + grp * 32, rk);
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[ab]);
      if (pend_kj < p.T) {
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)pend_b * p.T + pend_kj) * (3 * (size_t)p.C) + pend_h * HS + grp * 32;
        const float sc = p.scale;             // dS^T was stored without the 1/sqrt(HS) factor
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 0]), __uint_as_float(rv[j8 * 8 + 1]));
          u.y = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 2]), __uint_as_float(rv[j8 * 8 + 3]));
          u.z = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 4]), __uint_as_float(rv[j8 * 8 + 5]));
          u.w = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 6]), __uint_as_float(rv[j8 * 8 + 7]));
          *reinterpret_cast<uint4*>(base + 2 * p.C + j8 * 8) = u;
          u.x = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 0]) * sc, __uint_as_float(rk[j8 * 8 + 1]) * sc);
          u.y = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 2]) * sc, __uint_as_float(rk[j8 * 8 + 3]) * sc);
          u.z = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 4]) * sc, __uint_as_float(rk[j8 * 8 + 5]) * sc);
          u.w = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 6]) * sc, __uint_as_float(rk[j8 * 8 + 7]) * sc);
          *reinterpret_cast<uint4*>(base + p.C + j8 * 8) = u;
        }
      }
    };
    for (TileCursor c = cursor_begin(n_t, n_items, true); !c.done && !failed;) {
      const int b = c.bh / p.NH, h = c.bh % p.NH, kv0 = c.tile * TILE, kj = kv0 + row, n_ch = chunks_of(c.tile);
      const int i0 = 2 * c.tile;
      for (int n = 0; n < n_ch && !failed; ++n) {
        const int g = c.g + n, bf = grp, st = g % DKV_NS, i = i0 + n;
        if ((g & 1) != grp) continue;         // the other group's chunk
        if (!mbar_wait(&st_full[bf], (g >> 1) & 1)) { BW_FAIL(); break; }
        fence_after_sync();
        if (!mbar_wait(&q_full[st], (g / DKV_NS) & 1)) { BW_FAIL(); break; }      // acquire the chunk's row statistics
        const bool need_mask = (i * 64 < kv0 + TILE);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t rs[32], rp[32];
          tmem_ld32(tST + bf * 64 + lane_addr + half * 32, rs);
          tmem_ld32(tDPT + bf * 64 + lane_addr + half * 32, rp);
          tmem_wait_ld();
          if (half == 1) {                    // S^T and dP^T of this chunk are in registers
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&st_free[bf]);
          }
          const float4* l4 = reinterpret_cast<const float4*>(sStat + st * 128 + half * 32);
          const float4* d4 = reinterpret_cast<const float4*>(sStat + st * 128 + 64 + half * 32);
          const int qbase = i * 64 + half * 32;
          float pv[32], dv[32];
#pragma unroll
          for (int x4 = 0; x4 < 8; ++x4) {
            const float4 l = l4[x4], d = d4[x4];
            const float ls[4] = {l.x, l.y, l.z, l.w}, ds[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int x = x4 * 4 + k;
              float pr = ex2_approx(fmaf(__uint_as_float(rs[x]), p.scale_log2, -ls[k]));
              if (need_mask && kj > qbase + x) pr = 0.f;
              pv[x] = pr;
              dv[x] = pr * (__uint_as_float(rp[x]) - ds[k]);
            }
          }
          // products of chunk g-2 done: the P^T / dS^T buffers are free
          if (half == 0 && g >= 2 && !mbar_wait(&q_empty[(g - 2) % DKV_NS], ((g - 2) / DKV_NS) & 1)) { BW_FAIL(); break; }
          store_row32(sPT + bf * T128, row, half * 32, pv);
          store_row32(sDST + bf * T128, row, half * 32, dv);
        }
        if (failed) break;
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pd_full[bf]);
        if (pend) epilogue();
      }
      if (failed) break;
      if (pend) epilogue();
      pend = true; pend_t = c.t; pend_kj = kj; pend_b = b; pend_h = h;
      cursor_next(c, n_ch, n_t, n_items, true);
    }
    if (pend && !failed) epilogue();
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) { fence_after_sync(); tmem_dealloc<512>(tmem); }
}

// [B, T, width] bf16 viewed as a 3-D tensor; every load is a box of 64 rows x 64 columns
int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int T, int width) {
  return make_tmap_3d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)T, (uint64_t)B,
                      (uint64_t)width, (uint64_t)width * T, HS, 64);
}
}  // namespace

// out [B,T,C] bf16, lse [B,NH,T] fp32 (log2 domain), qkv [B,T,3C] bf16; C = NH*64.
LLMB_API int llmb_attention_fwd(void* out, float* lse, const void* qkv, int B, int T, int NH, int* status, cudaStream_t st) {
  const int C = NH * HS;
  CUtensorMap tm;
  int rc = make_qkv_map(&tm, qkv, B, T, 3 * C);
  if (rc) return 1000 + rc;
  AttnParams p{}; p.out = out; p.lse = lse; p.B = B; p.T = T; p.NH = NH; p.C = C;
  p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) { cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM); if (e) return (int)e; attr = true; }
  static int ver = -1;
  if (ver < 0) { const char* e = getenv("LLMB_ATTN_FWD"); ver = e ? atoi(e) : 2; }
  if (ver == 2) {
    static bool attr2 = false;
    if (!attr2) { cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD2_SMEM); if (e) return (int)e; attr2 = true; }
    const int n_t = ceil_div(T, TILE);
    const long long n_items = (long long)((n_t + 1) / 2) * B * NH;
    const long long want = (n_items + 1) / 2;            // two tile streams per CTA
    const int pgrid = (int)(want < sm_count() ? want : sm_count());
    attn_fwd2_kernel<<<pgrid, FW_THREADS, FWD2_SMEM, st>>>(tm, p);
    return (int)cudaGetLastError();
  }
  dim3 grid(ceil_div(T, TILE), NH, B);
  attn_fwd_kernel<<<grid, 256, FWD_SMEM, st>>>(tm, p);
  return (int)cudaGetLastError();
}

// dqkv [B,T,3C] bf16 (fully overwritten); dvec: 16-byte aligned fp32 scratch of B*NH*(T + 128*ceil(T/64)) + 4 elements.
LLMB_API int llmb_attention_bwd(void* dqkv, float* dvec, const void* dout, const void* qkv, const void* out,
                                const float* lse, int B, int T, int NH, int* status, cudaStream_t st) {
  const int C = NH * HS;
  CUtensorMap tq, td;
  int rc = make_qkv_map(&tq, qkv, B, T, 3 * C); if (rc) return 1000 + rc;
  rc = make_qkv_map(&td, dout, B, T, C); if (rc) return 1000 + rc;
  AttnParams p{}; p.out = dqkv; p.lse = const_cast<float*>(lse); p.dout = dout; p.dvec = dvec;
  p.B = B; p.T = T; p.NH = NH; p.C = C; p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV_SMEM); if (e) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM); if (e) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dkv2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV2_SMEM); if (e) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dq2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ2_SMEM); if (e) return (int)e;
    attr = true;
  }
  const int n_qc = ceil_div(T, 64);
  float* packed = dvec + (((size_t)B * NH * T + 3) & ~(size_t)3);   // scratch layout: D [B,NH,T], then (16-byte aligned) the packed chunks
  long long total = (long long)B * NH * n_qc * 64;
  attn_bwd_prep_kernel<<<(unsigned)ceil_div_ll(total, 256), 256, 0, st>>>(dvec, packed, lse, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, B, T, NH, C);
  p.packed = packed;
  dim3 grid(ceil_div(T, TILE), NH, B);
  static int ver = -1;
  if (ver < 0) { const char* e = getenv("LLMB_ATTN_BWD"); ver = e ? atoi(e) : 2; }
  if (ver == 2) {
    const int n_t = ceil_div(T, TILE);
    const long long n_items = (long long)((n_t + 1) / 2) * B * NH;
    const int pgrid = (int)(n_items < sm_count() ? n_items : sm_count());     // persistent: one CTA per SM
    attn_bwd_dkv2_kernel<<<pgrid, BW_THREADS, DKV2_SMEM, st>>>(tq, td, p);
    attn_bwd_dq2_kernel<<<pgrid, BW_THREADS, DQ2_SMEM, st>>>(tq, td, p);
  } else {
    attn_bwd_dkv_kernel<<<grid, 256, DKV_SMEM, st>>>(tq, td, p);
    attn_bwd_dq_kernel<<<grid, 256, DQ_SMEM, st>>>(tq, td, p);
  }
  return (int)cudaGetLastError();
}
