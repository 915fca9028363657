// Causal flash attention backward for head size 64 on tcgen05 + TMEM (the forward lives in attention_fwd.cu).
//
// Reference behaviour: llmm/attention.mojo:4692-5030 / :5033-5276 (backward via dP, row-dot D, dS, and the
// dQ/dK/dV batched GEMMs over stored [T,T] probabilities).  Here nothing of size T x T ever reaches HBM: the
// kernels read the packed [B,T,3C] QKV activations directly through a 3-D TMA map (no split/merge permutes),
// recompute S from Q, K and the forward's log-sum-exp, and keep S / dP / the accumulators in TMEM.
//
//   attn_bwd_prep_kernel  D = rowsum(dO * O), plus (lse, D) packed per 64-row chunk for bulk copies
//   attn_bwd_dkv2_kernel  dK/dV per 128-key tile over 64-row query chunks   } two deterministic persistent kernels,
//   attn_bwd_dq2_kernel   dQ per 128-row query tile over 64-key chunks      } no atomics
// The MN-major UMMA descriptor lets the same TMA-written tile serve as a K-major operand of one product and as
// the transposed operand of the next.  LSE is in the log2 domain of the scaled scores: lse2 = m + log2(sum 2^(s2 - m)).
#include "attention_common.cuh"

namespace {
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
      if (p.dbias) {                          // qkv bias gradient, dQ part: column sums of this warp's 32 rows
        float cv[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) cv[x] = pend_qi < p.T ? __uint_as_float(r[x]) * p.scale : 0.f;
        const float cs = warp_colsum32(cv, lane);
        atomicAdd(p.dbias + pend_h * HS + grp * 32 + lane, cs);
      }
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
      if (p.dbias) {                          // qkv bias gradient, dK and dV parts
        float cv[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) cv[x] = pend_kj < p.T ? __uint_as_float(rk[x]) * p.scale : 0.f;
        const float ck = warp_colsum32(cv, lane);
#pragma unroll
        for (int x = 0; x < 32; ++x) cv[x] = pend_kj < p.T ? __uint_as_float(rv[x]) : 0.f;
        const float cvv = warp_colsum32(cv, lane);
        atomicAdd(p.dbias + p.C + pend_h * HS + grp * 32 + lane, ck);
        atomicAdd(p.dbias + 2 * p.C + pend_h * HS + grp * 32 + lane, cvv);
      }
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

}  // namespace

extern "C" int llmb_attention_fwd_pair(void* out, float* lse, const void* qkv, int B, int T, int NH, int* status, cudaStream_t st);

// out [B,T,C] bf16, lse [B,NH,T] fp32 (log2 domain), qkv [B,T,3C] bf16; C = NH*64.
LLMB_API int llmb_attention_fwd(void* out, float* lse, const void* qkv, int B, int T, int NH, int* status, cudaStream_t st) {
  return llmb_attention_fwd_pair(out, lse, qkv, B, T, NH, status, st);
}

// dqkv [B,T,3C] bf16 (fully overwritten); dvec: 16-byte aligned fp32 scratch of B*NH*(T + 128*ceil(T/64)) + 4 elements.
LLMB_API int llmb_attention_bwd_dbias(void* dqkv, float* dbias, float* dvec, const void* dout, const void* qkv, const void* out,
                                      const float* lse, int B, int T, int NH, int* status, cudaStream_t st);
LLMB_API int llmb_attention_bwd(void* dqkv, float* dvec, const void* dout, const void* qkv, const void* out,
                                const float* lse, int B, int T, int NH, int* status, cudaStream_t st) {
  return llmb_attention_bwd_dbias(dqkv, nullptr, dvec, dout, qkv, out, lse, B, T, NH, status, st);
}
// As llmb_attention_bwd; with dbias != nullptr (fp32 [3C]) additionally dbias[c] += sum over all B*T rows of dqkv[:, c], i.e. the
// gradient of the qkv bias, taken from the fp32 accumulators in the kernels' epilogues (atomic adds: not bitwise reproducible).
LLMB_API int llmb_attention_bwd_dbias(void* dqkv, float* dbias, float* dvec, const void* dout, const void* qkv, const void* out,
                                      const float* lse, int B, int T, int NH, int* status, cudaStream_t st) {
  const int C = NH * HS;
  CUtensorMap tq, td;
  int rc = make_qkv_map(&tq, qkv, B, T, 3 * C); if (rc) return 1000 + rc;
  rc = make_qkv_map(&td, dout, B, T, C); if (rc) return 1000 + rc;
  AttnParams p{}; p.out = dqkv; p.lse = const_cast<float*>(lse); p.dout = dout; p.dvec = dvec; p.dbias = dbias;
  p.B = B; p.T = T; p.NH = NH; p.C = C; p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV2_SMEM); if (e) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dq2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ2_SMEM); if (e) return (int)e;
    attr = true;
  }
  const int n_qc = ceil_div(T, 64);
  float* packed = dvec + (((size_t)B * NH * T + 3) & ~(size_t)3);   // scratch layout: D [B,NH,T], then (16-byte aligned) the packed chunks
  long long total = (long long)B * NH * n_qc * 64;
  attn_bwd_prep_kernel<<<(unsigned)ceil_div_ll(total, 256), 256, 0, st>>>(dvec, packed, lse, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, B, T, NH, C);
  p.packed = packed;
  const int n_t = ceil_div(T, TILE);
  const long long n_items = (long long)((n_t + 1) / 2) * B * NH;
  const int pgrid = (int)(n_items < sm_count() ? n_items : sm_count());     // persistent: one CTA per SM
  attn_bwd_dkv2_kernel<<<pgrid, BW_THREADS, DKV2_SMEM, st>>>(tq, td, p);
  attn_bwd_dq2_kernel<<<pgrid, BW_THREADS, DQ2_SMEM, st>>>(tq, td, p);
  return (int)cudaGetLastError();
}
