// Causal flash attention backward for head size 64 on tcgen05 + TMEM: one fused persistent kernel.
//
// Reference behaviour: llmm/attention.mojo:4692-5030 / :5033-5276 (backward via dP, the row dot D = sum(dO * O), dS,
// and the dQ / dK / dV products over stored [T,T] probabilities).  Here nothing of size T x T reaches HBM and the
// scores are recomputed ONCE: a CTA owns a 128-key tile (K and V resident in shared memory, dK and dV accumulating
// in TMEM) and walks the 128-row query blocks i that can see it.  Per block, with lanes = keys, columns = queries:
//   S^T  = K Q_i^T          (tensor core, fp32 in TMEM)
//   dP^T = V dO_i^T         (tensor core, fp32 in TMEM)
//   P^T  = 2^(S^T * a - lse[q])          compute warps; packed bf16 into its own TMEM columns
//   dV  += P^T dO_i         (A operand read from TMEM, dO_i as an MN-major shared-memory operand)
//   dS^T = P^T * (dP^T - D[q])           compute warps; bf16 into a swizzled shared-memory tile [keys, queries]
//   dK  += dS^T Q_i         (A K-major from that tile)
//   dQ_i partial = dS K     (A MN-major from the SAME tile, B = the resident K tile as an MN-major operand)
// Because P^T does not live in the columns of S^T, the issuer can start S^T(n+1) as soon as the compute warps hold
// S^T(n) in registers (and dP^T(n+1) when they hold dP^T(n)): the scores of a block are in TMEM a whole block
// before they are used, and no compute warp waits for a tcgen05.commit round trip in steady state.
// The dQ partials of the key tiles are summed in an fp32 buffer by vector reductions (`red.global.add.v4.f32`, 16
// per thread and block, laid out so that a warp's 32 lanes hit 512 consecutive bytes); a small second kernel scales
// and rounds that buffer into the dQ part of dqkv and leaves it zeroed for the next call.  dK and dV are produced
// by exactly one CTA each in a fixed order and leave through a staging tile as TMA stores.
//
// Roles of the 512 threads:
//   warps 0..3 / 4..7   compute warpgroups: one thread per key row, query columns 0..63 / 64..127 of the block
//   warps 8..11         dQ warpgroup: TMEM -> reductions per block, and the dK / dV epilogue per tile
//   warp 12             TMA producer: K, V per tile (two buffers), Q_i, dO_i and the row statistics per block (ring),
//                       and L2 prefetches of the CTA's next tile
//   warp 13             MMA issuer (one warp: several issuing warps measured slower)
// TMEM columns (512): S^T 0..127 | dP^T 128..255 | dV 256..319 | dK 320..383 | dQ 384..447 | P^T 448..511.
// Every wait is bounded; a wait that runs out sets the status word and the role leaves its loop.
#include <type_traits>
#include "attention_common.cuh"

namespace {
constexpr int B3_NS = 3;                                   // ring depth in blocks: Q_i and dO_i, 16 KB each
constexpr int B3_THREADS = 512;
constexpr int B3_SMEM = 4 * T128 /*K,V x2*/ + B3_NS * 2 * T128 + 2 * T128 /*dS^T*/ + T128 /*epilogue staging*/ + B3_NS * 1024 /*-lse, -D*/ +
                        1024 /*alignment*/ + 512 /*barriers*/;
constexpr uint32_t IDESC_TS_MN = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, 64);     // A K-major (TMEM or smem), B stored [K rows, 64]
constexpr uint32_t IDESC_MN_MN = make_idesc(FMT_BF16, FMT_BF16, 1, 1, 128, 64);     // A stored [K rows, 128], B stored [K rows, 64]

#define B3_FAIL() do { atomicExch(p.status, LLMB_ERR_TIMEOUT); failed = true; } while (0)

struct B3Params {
  void* dqkv;            // [B,T,3C] bf16
  const float* stats;    // per (batch, head, 128-row tile): -lse[128] (log2 domain; -inf beyond T), -D[128]
  float* dq_acc;         // per (batch, head, tile): [16 column groups][128 rows][4] fp32, zero on entry
  float* dbias;          // optional fp32 [3C]
  int B, T, NH, C;
  float scale_log2, scale;
  int* status;
};

// D = rowsum(dO * O) and the packed row statistics of every 128-row tile.  Eight threads per row, 16 bytes of dO and O each,
// so that a warp reads four whole 128-byte rows per instruction.
__global__ void attn_bwd3_prep_kernel(float* __restrict__ stats, const float* __restrict__ lse, const __nv_bfloat16* __restrict__ dout,
                                      const __nv_bfloat16* __restrict__ out, int B, int T, int NH, int C) {
  const int n_t = ceil_div(T, TILE), Tp = n_t * TILE;
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;   // (b * NH + h) * Tp + t
  const int part = threadIdx.x & 7;
  if (idx >= (long long)B * NH * Tp) return;                                       // whole groups of eight leave together
  const int t = (int)(idx % Tp); const long long bh = idx / Tp;
  const int h = (int)(bh % NH), b = (int)(bh / NH);
  float s = 0.f;
  if (t < T) {
    const long long bt = (long long)b * T + t;
    Pack<__nv_bfloat16> x, y;
    x.load(dout + bt * C + h * HS + part * 8); y.load(out + bt * C + h * HS + part * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += x.v[k] * y.v[k];
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1); s += __shfl_xor_sync(0xffffffffu, s, 2); s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (part == 0) {
    float* pk = stats + (bh * n_t + t / TILE) * 256 + (t % TILE);
    pk[0] = t < T ? -lse[bh * T + t] : -INFINITY;
    pk[128] = -s;
  }
}

struct Tile3 { int w, t, g, bh, tile; bool sub, done; };    // work item, tiles / blocks consumed so far, current tile
// Work item w = (batch, head) w / n_pairs and the key tiles x = w % n_pairs (n_t - x blocks) and n_t - 1 - x (x + 1
// blocks): n_t + 1 blocks whatever x.  Neighbouring CTAs work on the same (batch, head), so its Q and dO are read
// from HBM once.
__device__ __forceinline__ void tile3_seek(Tile3& c, int n_t, int n_items) {
  const int n_pairs = (n_t + 1) / 2;
  for (;;) {
    if (c.w >= n_items) { c.done = true; return; }
    const int x = c.w % n_pairs;
    c.bh = c.w / n_pairs;
    if (!c.sub) { c.tile = x; return; }
    if (n_t - 1 - x != x) { c.tile = n_t - 1 - x; return; }
    c.w += gridDim.x; c.sub = false;
  }
}
struct Blk3 { Tile3 c; int ib, nbt, n; };                   // block within the tile, blocks of the tile, blocks so far
__device__ __forceinline__ Blk3 blk3_begin(int n_t, int n_items) {
  Blk3 it;
  it.c = Tile3{(int)blockIdx.x, 0, 0, 0, 0, false, false};
  tile3_seek(it.c, n_t, n_items);
  it.ib = 0; it.n = 0; it.nbt = it.c.done ? 0 : n_t - it.c.tile;
  return it;
}
__device__ __forceinline__ void tile3_next(Tile3& c, int nbt, int n_t, int n_items) {
  c.t += 1; c.g += nbt;
  if (!c.sub) c.sub = true; else { c.sub = false; c.w += gridDim.x; }
  tile3_seek(c, n_t, n_items);
}
__device__ __forceinline__ void blk3_next(Blk3& it, int n_t, int n_items) {
  ++it.n;
  if (++it.ib == it.nbt) {
    tile3_next(it.c, it.nbt, n_t, n_items);
    it.ib = 0; it.nbt = it.c.done ? 0 : n_t - it.c.tile;
  }
}

__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void __launch_bounds__(B3_THREADS, 1) attn_bwd3_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                  const __grid_constant__ CUtensorMap tmDO,
                                                                  const __grid_constant__ CUtensorMap tmOUT, const B3Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sKV = sm;                                  // buffer kb: K at kb*2*T128, V at +T128
  unsigned char* sST = sKV + 4 * T128;                      // ring: stage s holds Q_i at s*2*T128, dO_i at +T128
  unsigned char* sDS = sST + B3_NS * 2 * T128;              // dS^T: queries 0..63 at +0, 64..127 at +T128 ([128 keys][64] each)
  unsigned char* sEP = sDS + 2 * T128;                      // staging tile of the dK / dV epilogue ([128 keys][64] bf16, swizzled)
  float* sStat = reinterpret_cast<float*>(sEP + T128);      // per stage: -lse[128], -D[128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + B3_NS * 256);
  uint64_t* kv_full = bars;                                 // [2]
  uint64_t* kv_empty = kv_full + 2;                         // [2] the tile's last reads of K and V are complete 
  uint64_t* st_full = kv_empty + 2;                         // [NS]
  uint64_t* st_empty = st_full + B3_NS;                     // [NS] the block's reads of Q and dO are complete 
  uint64_t* s_full = st_empty + B3_NS;                      // S^T is in TMEM
  uint64_t* s_free = s_full + 1;                            // the compute warps hold S^T in registers (8 warps)
  uint64_t* dp_full = s_free + 1;                           // dP^T is in TMEM
  uint64_t* dp_free = dp_full + 1;                          // the compute warps hold dP^T in registers (8 warps)
  uint64_t* p_full = dp_free + 1;                           // P^T is in TMEM (8 warps)
  uint64_t* p_used = p_full + 1;                            // dV has read P^T
  uint64_t* ds_full = p_used + 1;                           // dS^T is in shared memory (8 warps)
  uint64_t* ds_free = ds_full + 1;                          // dK and dQ have read dS^T
  uint64_t* dq_full = ds_free + 1;                          // the block's dQ partial is in TMEM
  uint64_t* dq_free = dq_full + 1;                          // ... and has left it (4 warps)
  uint64_t* acc_full = dq_free + 1;                         // dK and dV of a tile are complete 
  uint64_t* acc_free = acc_full + 1;                        // ... and have left TMEM (4 warps)
  uint64_t* ep_ready = acc_free + 1;                        // the epilogue's staging tile is written (4 warps)
  uint64_t* ep_done = ep_ready + 1;                         // ... and its TMA stores have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ep_done + 1);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_t = ceil_div(p.T, TILE);
  const int n_items = ((n_t + 1) / 2) * p.B * p.NH;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < B3_NS; ++i) { mbar_init(&st_full[i], 1); mbar_init(&st_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(s_free, 8); mbar_init(dp_full, 1); mbar_init(dp_free, 8);
    mbar_init(p_full, 8); mbar_init(p_used, 1); mbar_init(ds_full, 8); mbar_init(ds_free, 1);
    mbar_init(dq_full, 1); mbar_init(dq_free, 4); mbar_init(acc_full, 1); mbar_init(acc_free, 4); mbar_init(ep_ready, 4); mbar_init(ep_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO); prefetch_tmap(&tmOUT);
  }
  if (warp == 13) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 320, tDQ = tmem + 384, tP = tmem + 448;
  bool failed = false;

  // Registers move from the dQ warpgroup and the producer / issuer warpgroup to the two compute warpgroups:
  // 2 x 128 x 176 + 2 x 128 x 80 = 65536 = the registers of the launch (512 x 128).
  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if (warp == 12) {
      // ------------------------------------------------------------ TMA producer
      Tile3 c{(int)blockIdx.x, 0, 0, 0, 0, false, false};
      for (tile3_seek(c, n_t, n_items); !c.done && !failed;) {
        const int b = c.bh / p.NH, h = c.bh % p.NH, kb = c.t & 1, nbt = n_t - c.tile;
        const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
        if (c.t >= 2 && !mbar_wait_sleep(&kv_empty[kb], ((c.t >> 1) + 1) & 1)) { B3_FAIL(); break; }
        if (elect_one()) {
          mbar_expect_tx(&kv_full[kb], 2 * T128);
          load128(sKV + kb * 2 * T128, &tmQKV, &kv_full[kb], colK, c.tile * TILE, b);
          load128(sKV + kb * 2 * T128 + T128, &tmQKV, &kv_full[kb], colV, c.tile * TILE, b);
        }
        __syncwarp();
        // While this tile's blocks are loaded, the operands of the CTA's NEXT tile are pulled into L2, a few boxes per
        // block, so that its loads find them there.
        Tile3 nx = c;
        tile3_next(nx, nbt, n_t, n_items);
        const int nxb = nx.bh / p.NH, nxh = nx.bh % p.NH, nx0 = nx.tile * TILE;
        const int pf_per = nx.done ? 0 : ceil_div(2 + 2 * (n_t - nx.tile), nbt);     // prefetch steps (64 rows) per block of this tile
        int pf = nx0 - 128;                                                          // next row to prefetch; the first two steps take K and V
        for (int ib = 0; ib < nbt; ++ib) {
          const int n = c.g + ib, st = n % B3_NS, i = c.tile + ib;
          if (n >= B3_NS && !mbar_wait_sleep(&st_empty[st], ((n / B3_NS) + 1) & 1)) { B3_FAIL(); break; }
          if (elect_one()) {
            unsigned char* stg = sST + st * 2 * T128;
            mbar_expect_tx(&st_full[st], 2 * T128 + 1024);
            load128(stg, &tmQKV, &st_full[st], colQ, i * TILE, b);
            load128(stg + T128, &tmDO, &st_full[st], colQ, i * TILE, b);
            bulk_load_1d(sStat + st * 256, p.stats + ((size_t)c.bh * n_t + i) * 256, 1024, &st_full[st]);
            for (int k = 0; k < pf_per; ++k) {
              const int r = pf + 64 * k;
              if (r < nx0) {
                tma_prefetch_l2_3d(&tmQKV, p.C + nxh * HS, r + 128, nxb);
                tma_prefetch_l2_3d(&tmQKV, 2 * p.C + nxh * HS, r + 128, nxb);
              } else if (r < n_t * TILE) {
                tma_prefetch_l2_3d(&tmQKV, nxh * HS, r, nxb);
                tma_prefetch_l2_3d(&tmDO, nxh * HS, r, nxb);
              }
            }
          }
          pf += 64 * pf_per;
          __syncwarp();
        }
        if (failed) break;
        tile3_next(c, nbt, n_t, n_items);
      }
    } else if (warp == 13) {
      // ------------------------------------------------------------ MMA issuer.  Per block n, in the order in which the compute warps'
      // signals arrive: S^T(n+1) when they hold S^T(n) in registers, dV(n) when P^T(n) is written, dP^T(n+1) when they hold
      // dP^T(n), dK(n) and dQ(n) when dS^T(n) is written - so the scores of a block are ready a whole block before their use.
      const uint64_t k_kk0 = make_smem_desc(smem_u32(sKV), 16, 1024);                 // K / V as K-major A operands
      const uint64_t k_mn0 = make_smem_desc(smem_u32(sKV), 8192, 1024);               // K as an MN-major B operand
      const uint64_t q_kk0 = make_smem_desc(smem_u32(sST), 16, 1024);                 // Q_i / dO_i as K-major B operands
      const uint64_t q_mn0 = make_smem_desc(smem_u32(sST), 8192, 1024);               // Q_i / dO_i as MN-major B operands
      const uint64_t ds_kk = make_smem_desc(smem_u32(sDS), 16, 1024);                 // dS^T as a K-major A operand (K = queries)
      const uint64_t ds_mn = make_smem_desc(smem_u32(sDS), T128, 1024);               // dS^T as an MN-major A operand (M = queries)
      Blk3 nx = blk3_begin(n_t, n_items), it = nx;                                    // block n+1 (scores), block n (accumulating products)
      auto scores_s = [&]() {                                                         // S^T of block nx
        const int n = nx.n, st = n % B3_NS, kb = nx.c.t & 1;
        if (nx.ib == 0 && !mbar_wait(&kv_full[kb], (nx.c.t >> 1) & 1)) { B3_FAIL(); return; }
        if (!mbar_wait(&st_full[st], (n / B3_NS) & 1)) { B3_FAIL(); return; }
        if (n >= 1 && !mbar_wait(s_free, (n - 1) & 1)) { B3_FAIL(); return; }
        fence_after_sync();
        const uint64_t kd = k_kk0 + (uint64_t)((kb * 2 * T128) >> 4), qd = q_kk0 + (uint64_t)((st * 2 * T128) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < HS / 16; ++ks) umma_ss<KIND_F16>(tS, kd + 2 * ks, qd + 2 * ks, IDESC_S_128x128, ks > 0 ? 1u : 0u);
          umma_commit(s_full);
        }
        __syncwarp();
      };
      auto scores_dp = [&]() {                                                        // dP^T of block nx, then nx moves on
        const int n = nx.n, st = n % B3_NS, kb = nx.c.t & 1;
        if (n >= 1 && !mbar_wait(dp_free, (n - 1) & 1)) { B3_FAIL(); return; }
        fence_after_sync();
        const uint64_t vd = k_kk0 + (uint64_t)((kb * 2 * T128 + T128) >> 4), dod = q_kk0 + (uint64_t)((st * 2 * T128 + T128) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < HS / 16; ++ks) umma_ss<KIND_F16>(tDP, vd + 2 * ks, dod + 2 * ks, IDESC_S_128x128, ks > 0 ? 1u : 0u);
          umma_commit(dp_full);
        }
        __syncwarp();
        blk3_next(nx, n_t, n_items);
      };
      if (!nx.c.done) { scores_s(); if (!failed) scores_dp(); }                       // block 0
      while (!it.c.done && !failed) {
        const int n = it.n, st = n % B3_NS, kb = it.c.t & 1;
        const bool first = it.ib == 0, last = it.ib + 1 == it.nbt;
        if (!nx.c.done) { scores_s(); if (failed) break; }                            // waits for s_free(n)
        if (!mbar_wait(p_full, n & 1)) { B3_FAIL(); break; }
        if (first && it.c.t >= 1 && !mbar_wait(acc_free, (it.c.t - 1) & 1)) { B3_FAIL(); break; }
        fence_after_sync();
        const uint64_t do_mn = q_mn0 + (uint64_t)((st * 2 * T128 + T128) >> 4), q_mn = q_mn0 + (uint64_t)((st * 2 * T128) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks) umma_ts(tDV, tP + ks * 8, do_mn + 128 * ks, IDESC_TS_MN, (ks > 0 || !first) ? 1u : 0u);   // dV += P^T dO
          umma_commit(p_used);                                                        // the compute warps may write P^T(n+1)
        }
        __syncwarp();
        if (!nx.c.done) { scores_dp(); if (failed) break; }                           // waits for dp_free(n)
        if (!mbar_wait(ds_full, n & 1)) { B3_FAIL(); break; }
        if (n >= 1 && !mbar_wait(dq_free, (n - 1) & 1)) { B3_FAIL(); break; }
        fence_after_sync();
        const uint64_t kmn = k_mn0 + (uint64_t)((kb * 2 * T128) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks)                                                                                          // dK += dS^T Q
            umma_ss<KIND_F16>(tDK, ds_kk + (ks < 4 ? 2 * ks : (T128 >> 4) + 2 * (ks - 4)), q_mn + 128 * ks, IDESC_TS_MN, (ks > 0 || !first) ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < TILE / 16; ++ks) umma_ss<KIND_F16>(tDQ, ds_mn + 128 * ks, kmn + 128 * ks, IDESC_MN_MN, ks > 0 ? 1u : 0u);  // dQ = dS K
          umma_commit(dq_full);
          umma_commit(ds_free);
          umma_commit(&st_empty[st]);
          if (last) { umma_commit(acc_full); umma_commit(&kv_empty[kb]); }
        }
        __syncwarp();
        blk3_next(it, n_t, n_items);
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- dQ warpgroup: one thread per query row (dQ) / key row (dK, dV)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    int ne = 0;                                             // epilogue rounds so far
    for (Blk3 it = blk3_begin(n_t, n_items); !it.c.done && !failed; blk3_next(it, n_t, n_items)) {
      const int n = it.n, i = it.c.tile + it.ib;
      if (!mbar_wait_sleep(dq_full, n & 1)) { B3_FAIL(); break; }
      fence_after_sync();
      float* dst = p.dq_acc + ((size_t)it.c.bh * n_t + i) * (TILE * HS) + row * 4;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld32(tDQ + lane_addr + half * 32, r);
        tmem_wait_ld();
        if (half == 1) {
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_free);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          red_add_v4(dst + (half * 8 + c) * (TILE * 4), __uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]),
                     __uint_as_float(r[4 * c + 3]));
      }
      if (it.ib + 1 < it.nbt) continue;
      // The tile's dV and dK: rounded rows go through a swizzled staging tile and leave as TMA stores (whole 128-byte
      // rows; rows beyond T are clipped by the tensor map).  Per-thread stores of 16 bytes at a row stride of 3C would
      // keep this warpgroup busy for longer than a whole block takes.
      if (!mbar_wait_sleep(acc_full, it.c.t & 1)) { B3_FAIL(); break; }
      fence_after_sync();
      const int b = it.c.bh / p.NH, h = it.c.bh % p.NH, k0 = it.c.tile * TILE, kj = k0 + row;
#pragma unroll 1
      for (int mat = 0; mat < 2; ++mat) {                   // 0: dV, 1: dK
        const float sc = mat ? p.scale : 1.0f;              // dS^T was stored without the 1/sqrt(HS) factor
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32((mat ? tDK : tDV) + lane_addr + half * 32, r);
          tmem_wait_ld();
          if (mat == 1 && half == 1) {
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free);
          }
          float v[32];
#pragma unroll
          for (int x = 0; x < 32; ++x) v[x] = kj < p.T ? __uint_as_float(r[x]) * sc : 0.f;
          store_row32(sEP, row, half * 32, v);
          if (p.dbias) {                                    // qkv bias gradient, dK and dV parts: column sums of this warp's 32 rows
            const float cs = warp_colsum32(v, lane);
            atomicAdd(p.dbias + (mat ? 1 : 2) * p.C + h * HS + half * 32 + lane, cs);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(ep_ready);
        if (warp == 8) {
          if (!mbar_wait_sleep(ep_ready, ne & 1)) { B3_FAIL(); break; }
          if (elect_one()) {
            const int col = (mat ? 1 : 2) * p.C + h * HS;
            tma_store_3d(&tmOUT, sEP, col, k0, b);
            tma_store_3d(&tmOUT, sEP + T64, col, k0 + 64, b);
            bulk_commit();
            bulk_wait_read<0>();
            mbar_arrive(ep_done);
          }
          __syncwarp();
        }
        if (!mbar_wait_sleep(ep_done, ne & 1)) { B3_FAIL(); break; }      // the staging tile may be rewritten
        ++ne;
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroup hq: one thread per key row, query columns hq*64 .. +63
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int hq = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tSh = tS + lane_addr + hq * 64, tDPh = tDP + lane_addr + hq * 64, tPh = tP + lane_addr + hq * 32;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    for (Blk3 it = blk3_begin(n_t, n_items); !it.c.done && !failed; blk3_next(it, n_t, n_items)) {
      const int n = it.n, st = n % B3_NS;
      const float* stat = sStat + st * 256 + hq * 64;
      if (!mbar_wait_sleep(&st_full[st], (n / B3_NS) & 1)) { B3_FAIL(); break; }      // acquire the block's row statistics
      if (!mbar_wait_sleep(s_full, n & 1)) { B3_FAIL(); break; }
      fence_after_sync();
      uint32_t s[64];
      {
        uint32_t (&q0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[0]);
        uint32_t (&q1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[32]);
        tmem_ld32(tSh, q0); tmem_ld32(tSh + 32, q1);
      }
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);                   // S^T(n+1) may be issued now
      {
        uint32_t pk[32];
        const float4* nl4 = reinterpret_cast<const float4*>(stat);
        auto p_phase = [&](auto diag) {
          const int lim = row - hq * 64;                    // diagonal block: local query columns x < lim see nothing of this key
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const float4 l = nl4[x];
            const float2 t01 = __ffma2_rn(make_float2(__uint_as_float(s[4 * x]), __uint_as_float(s[4 * x + 1])), sc2, make_float2(l.x, l.y));
            const float2 t23 = __ffma2_rn(make_float2(__uint_as_float(s[4 * x + 2]), __uint_as_float(s[4 * x + 3])), sc2, make_float2(l.z, l.w));
            float e0 = ex2_approx(t01.x), e1 = ex2_approx(t01.y), e2 = ex2_approx(t23.x), e3 = ex2_approx(t23.y);
            if (decltype(diag)::value) {
              e0 = 4 * x < lim ? 0.f : e0; e1 = 4 * x + 1 < lim ? 0.f : e1;
              e2 = 4 * x + 2 < lim ? 0.f : e2; e3 = 4 * x + 3 < lim ? 0.f : e3;
            }
            s[4 * x] = __float_as_uint(e0); s[4 * x + 1] = __float_as_uint(e1);
            s[4 * x + 2] = __float_as_uint(e2); s[4 * x + 3] = __float_as_uint(e3);
            pk[2 * x] = pack_bf16x2(e0, e1); pk[2 * x + 1] = pack_bf16x2(e2, e3);
          }
        };
        if (it.ib == 0) p_phase(std::true_type{}); else p_phase(std::false_type{});
        if (n >= 1 && !mbar_wait_sleep(p_used, (n - 1) & 1)) { B3_FAIL(); break; }   // dV has read P^T(n-1)
        fence_after_sync();
        tmem_st32(tPh, pk);
      }
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait_sleep(dp_full, n & 1)) { B3_FAIL(); break; }
      fence_after_sync();
      uint32_t d[64];
      {
        uint32_t (&q0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&d[0]);
        uint32_t (&q1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&d[32]);
        tmem_ld32(tDPh, q0); tmem_ld32(tDPh + 32, q1);
      }
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_free);                  // dP^T(n+1) may be issued now
      {
        const float4* nd4 = reinterpret_cast<const float4*>(stat + 128);
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float4 nd = nd4[x];
          const float2 a01 = __fadd2_rn(make_float2(__uint_as_float(d[4 * x]), __uint_as_float(d[4 * x + 1])), make_float2(nd.x, nd.y));
          const float2 a23 = __fadd2_rn(make_float2(__uint_as_float(d[4 * x + 2]), __uint_as_float(d[4 * x + 3])), make_float2(nd.z, nd.w));
          const float2 r01 = __fmul2_rn(make_float2(__uint_as_float(s[4 * x]), __uint_as_float(s[4 * x + 1])), a01);
          const float2 r23 = __fmul2_rn(make_float2(__uint_as_float(s[4 * x + 2]), __uint_as_float(s[4 * x + 3])), a23);
          s[4 * x] = __float_as_uint(r01.x); s[4 * x + 1] = __float_as_uint(r01.y);
          s[4 * x + 2] = __float_as_uint(r23.x); s[4 * x + 3] = __float_as_uint(r23.y);
        }
      }
      if (n >= 1 && !mbar_wait_sleep(ds_free, (n - 1) & 1)) { B3_FAIL(); break; }   // dK and dQ of block n-1 have read the tile
      {
        const float (&v0)[32] = *reinterpret_cast<const float (*)[32]>(&s[0]);
        const float (&v1)[32] = *reinterpret_cast<const float (*)[32]>(&s[32]);
        store_row32(sDS + hq * T128, row, 0, v0);
        store_row32(sDS + hq * T128, row, 32, v1);
      }
      fence_proxy_async();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 13) { fence_after_sync(); tmem_dealloc<512>(tmem); }
}

// dq_acc -> the dQ part of dqkv (scaled, rounded), the buffer zeroed again, and optionally the dQ part of the bias gradient.
// One block of 128 threads per (batch, head, tile): thread r reads row r (a warp reads 512 consecutive bytes per load), the
// rounded rows cross a swizzled shared-memory tile, and every warp then writes four whole 128-byte rows per instruction.
__global__ void __launch_bounds__(128) attn_bwd3_dq_kernel(__nv_bfloat16* __restrict__ dqkv, float* __restrict__ dbias, float* __restrict__ dq_acc,
                                                           int T, int NH, int C, float scale) {
  __shared__ float part[4][HS];
  __shared__ __align__(16) unsigned char tile_s[TILE * ROWB];
  const int n_t = ceil_div(T, TILE);
  const int tile = blockIdx.x % n_t, bh = blockIdx.x / n_t, h = bh % NH, b = bh / NH;
  const int r = threadIdx.x, lane = r % 32, warp = r / 32;
  float* src = dq_acc + (size_t)blockIdx.x * (TILE * HS) + r * 4;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    float v[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float4 x = *reinterpret_cast<const float4*>(src + (half * 8 + c) * (TILE * 4));
      v[4 * c] = x.x * scale; v[4 * c + 1] = x.y * scale; v[4 * c + 2] = x.z * scale; v[4 * c + 3] = x.w * scale;
    }
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      uint4 u;
      u.x = pack_bf16x2(v[j8 * 8 + 0], v[j8 * 8 + 1]); u.y = pack_bf16x2(v[j8 * 8 + 2], v[j8 * 8 + 3]);
      u.z = pack_bf16x2(v[j8 * 8 + 4], v[j8 * 8 + 5]); u.w = pack_bf16x2(v[j8 * 8 + 6], v[j8 * 8 + 7]);
      *reinterpret_cast<uint4*>(tile_s + sw128(r, half * 4 + j8)) = u;
    }
    if (dbias) {                                            // rows beyond T hold zeros: their dS was zero
      const float cs = warp_colsum32(v, lane);
      part[warp][half * 32 + lane] = cs;
    }
  }
  __syncthreads();
  const int chunk = r & 7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int row = k * 16 + (r >> 3), qi = tile * TILE + row;
    if (qi < T)
      *reinterpret_cast<uint4*>(dqkv + ((size_t)b * T + qi) * (3 * (size_t)C) + h * HS + chunk * 8) =
          *reinterpret_cast<const uint4*>(tile_s + sw128(row, chunk));
  }
  // Zeroed only now, when every load above has returned its data: a store to an address whose load is still in flight
  // waits for it, and the kernel then runs at a quarter of the memory bandwidth.
#pragma unroll
  for (int c = 0; c < 16; ++c) *reinterpret_cast<float4*>(src + c * (TILE * 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
  if (dbias && r < HS) atomicAdd(dbias + h * HS + r, part[0][r] + part[1][r] + part[2][r] + part[3][r]);
}
}  // namespace

// Sizes (in floats) of the two scratch buffers of llmb_attention_bwd_fused.
LLMB_API long long llmb_attention_bwd_fused_stats_floats(int B, int T, int NH) { return (long long)B * NH * ceil_div(T, TILE) * 256; }
LLMB_API long long llmb_attention_bwd_fused_acc_floats(int B, int T, int NH) { return (long long)B * NH * ceil_div(T, TILE) * (TILE * HS); }

// dqkv [B,T,3C] bf16 (fully overwritten) from dout [B,T,C], qkv [B,T,3C], out [B,T,C] (bf16) and the forward's lse [B,NH,T]
// (log2 domain); C = NH*64.  `stats`: fp32 scratch of ..._stats_floats elements.  `dq_acc`: fp32 scratch of ..._acc_floats
// elements, 16-byte aligned, which must be ZERO on entry and is zero again when the call has completed without an error in
// the status word.  dbias (optional, fp32 [3C]) += column sums of dqkv, by atomic adds.
LLMB_API int llmb_attention_bwd_fused(void* dqkv, float* dbias, float* stats, float* dq_acc, const void* dout, const void* qkv, const void* out,
                                      const float* lse, int B, int T, int NH, int* status, cudaStream_t st) {
  const int C = NH * HS;
  CUtensorMap tq, td;
  int rc = make_qkv_map(&tq, qkv, B, T, 3 * C); if (rc) return 1000 + rc;
  rc = make_qkv_map(&td, dout, B, T, C); if (rc) return 1000 + rc;
  CUtensorMap to;
  rc = make_qkv_map(&to, dqkv, B, T, 3 * C); if (rc) return 1000 + rc;
  B3Params p{}; p.dqkv = dqkv; p.stats = stats; p.dq_acc = dq_acc; p.dbias = dbias;
  p.B = B; p.T = T; p.NH = NH; p.C = C; p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, B3_SMEM); if (e) return (int)e;
    attr = true;
  }
  const int n_t = ceil_div(T, TILE);
  const long long rows = (long long)B * NH * n_t * TILE;
  attn_bwd3_prep_kernel<<<(unsigned)ceil_div_ll(rows * 8, 256), 256, 0, st>>>(stats, lse, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, B, T, NH, C);
  const long long n_items = (long long)((n_t + 1) / 2) * B * NH;
  const int grid = (int)(n_items < sm_count() ? n_items : sm_count());          // persistent: one CTA per SM
  attn_bwd3_kernel<<<grid, B3_THREADS, B3_SMEM, st>>>(tq, td, to, p);
  attn_bwd3_dq_kernel<<<(unsigned)(B * NH * n_t), 128, 0, st>>>((__nv_bfloat16*)dqkv, dbias, dq_acc, T, NH, C, p.scale);
  return (int)cudaGetLastError();
}
