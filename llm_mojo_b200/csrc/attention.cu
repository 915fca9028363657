// Causal flash attention forward / backward for head size 64 on tcgen05 + TMEM.
//
// Reference behaviour: llmm/attention.mojo:1557-1745 (forward: split -> QK^T -> causal softmax ->
// PV -> merge, storing [T,T] probabilities) and :4692-5030 (backward via dP, row-dot D, dS, and
// the dQ/dK/dV batched GEMMs).  Here nothing of size T x T ever reaches HBM: the kernels read
// the packed [B,T,3C] QKV activations directly through a 3-D TMA map (no split/merge
// permutes), keep S/P and the running output in TMEM / shared memory, and store only the
// output [B,T,C] plus one log-sum-exp per row.
//
// Forward  : CTA = 128 query rows of one (batch, head), 256 threads: two threads share a row, each
//            owning one 64-column half of the score tile (warps w and w+4 read the same TMEM lanes).
//            S = Q K^T (tcgen05, 128x128 fp32 in TMEM) -> online softmax in registers ->
//            P (bf16, swizzled smem) -> O += P V (tcgen05, O in TMEM, rescaled in place).
// Backward : two deterministic kernels (no atomics).
//   dK/dV  : CTA = 128 key rows; loops over 64-row query chunks:  S^T = K Q^T, dP^T = V dO^T,
//            P^T and dS^T to smem, dV += P^T dO, dK += dS^T Q   (accumulators in TMEM).
//   dQ     : CTA = 128 query rows; loops over 64-row key chunks:   S = Q K^T, dP = dO V^T,
//            dS to smem, dQ += dS K.
// The MN-major UMMA descriptor lets the same TMA-written tile serve as a K-major operand of
// one product and as the transposed operand of the next.  Two CTAs fit per SM (<= 112 KB of
// shared memory, 256 TMEM columns each) so one CTA's MMAs overlap the other's softmax.
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
  for (int k = 0; k < nk; ++k) umma_ss<KIND_F16>(d, ad + 2 * k, bd + 2 * k, idesc, (acc_first || k > 0) ? 1u : 0u);
}
// A K-major (32 B per step), B MN-major single 64-wide chunk (16 k-rows = 2048 B per step)
__device__ __forceinline__ void mma_kmn(uint32_t d, uint32_t a_addr, uint32_t b_addr, uint32_t idesc, int nk, bool acc_first) {
  const uint64_t ad = make_smem_desc(a_addr, 16, 1024), bd = make_smem_desc(b_addr, 8192, 1024);
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
__global__ void attn_bwd_prep_kernel(float* __restrict__ dvec, const __nv_bfloat16* __restrict__ dout,
                                     const __nv_bfloat16* __restrict__ out, int B, int T, int NH, int C) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // (b, t, h)
  long long total = (long long)B * T * NH;
  if (idx >= total) return;
  int h = (int)(idx % NH); long long bt = idx / NH;
  int t = (int)(bt % T), b = (int)(bt / T);
  const __nv_bfloat16* a = dout + bt * C + h * HS;
  const __nv_bfloat16* o = out + bt * C + h * HS;
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < HS / 8; ++j) {
    Pack<__nv_bfloat16> x, y; x.load(a + j * 8); y.load(o + j * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += x.v[k] * y.v[k];
  }
  dvec[((size_t)b * NH + h) * T + t] = s;
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
  dim3 grid(ceil_div(T, TILE), NH, B);
  attn_fwd_kernel<<<grid, 256, FWD_SMEM, st>>>(tm, p);
  return (int)cudaGetLastError();
}

// dqkv [B,T,3C] bf16 (fully overwritten), dvec scratch [B,NH,T] fp32.
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
    attr = true;
  }
  long long total = (long long)B * T * NH;
  attn_bwd_prep_kernel<<<(unsigned)ceil_div_ll(total, 256), 256, 0, st>>>(dvec, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, B, T, NH, C);
  dim3 grid(ceil_div(T, TILE), NH, B);
  attn_bwd_dkv_kernel<<<grid, 256, DKV_SMEM, st>>>(tq, td, p);
  attn_bwd_dq_kernel<<<grid, 256, DQ_SMEM, st>>>(tq, td, p);
  return (int)cudaGetLastError();
}
