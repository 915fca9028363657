// Causal flash attention backward for head size 64 on tcgen05 + TMEM: one fused persistent kernel.
//
// Reference behaviour: llmm/attention.mojo:4692-5030 / :5033-5276 (backward via dP, the row dot D = sum(dO * O), dS,
// and the dQ / dK / dV products over stored [T,T] probabilities).  Here nothing of size T x T reaches HBM and the
// scores are recomputed ONCE: a CTA owns a 128-key tile (K and V resident in shared memory, dK and dV accumulating
// in TMEM) and walks the 128-row query blocks that can see it, each as two chunks of 64 queries.  Per chunk c, with
// lanes = keys, columns = queries:
//   S^T  = K Q_c^T          (tensor core, fp32 in TMEM)
//   dP^T = V dO_c^T         (tensor core, fp32 in TMEM)
//   P^T  = 2^(S^T * a - lse[q])          compute warps; written back over S^T as packed bf16
//   dV  += P^T dO_c         (A operand read from TMEM, dO_c as an MN-major shared-memory operand)
//   dS^T = P^T * (dP^T - D[q])           compute warps; bf16 into a swizzled shared-memory tile [keys, 64 queries]
//   dK  += dS^T Q_c         (A K-major from that tile)
// and per block, once both chunks' dS^T tiles are written,
//   dQ partial = dS K       (A MN-major from the two tiles side by side, B = the resident K tile as an MN-major operand)
// The two compute warpgroups take alternate chunks and run half a period apart: while one is in its exponentials
// the other does the multiplies and stores of dS, and every product is issued at least one chunk before its
// result is needed, so no warp waits for the latency of a tcgen05.commit round trip in steady state.
// The dQ partials of the key tiles are summed in an fp32 buffer by vector reductions (`red.global.add.v4.f32`, 16
// per thread and block, laid out so that a warp's 32 lanes hit 512 consecutive bytes); a small second kernel scales
// and rounds that buffer into the dQ part of dqkv and leaves it zeroed for the next call.  dK and dV are produced
// by exactly one CTA each in a fixed order.
//
// Roles of the 512 threads:
//   warps 0..3 / 4..7   compute warpgroup 0 / 1: one thread per key row, the 64 query columns of chunks 2n / 2n+1
//   warps 8..11         dQ warpgroup: TMEM -> reductions per block, and the dK / dV epilogue per tile
//   warp 12             TMA producer: K, V per tile (two buffers), Q_c, dO_c and the row statistics per chunk (ring)
//   warp 13             MMA issuer
// TMEM columns (512): S^T / P^T of warpgroup 0, 1: 0..63, 64..127 | dP^T: 128..191, 192..255 | dV 256..319 |
// dK 320..383 | dQ 384..447, 448..511.  S^T(c+2) is issued behind dV(c) on the (in-order) tensor pipe, so it
// overwrites P^T(c) only after that product has read it.
#include <type_traits>
#include "attention_common.cuh"

namespace {
constexpr int B3_NS = 5;                                   // ring depth in chunks: Q_c and dO_c, 8 KB each
constexpr int B3_DSB = 2;                                  // dS^T buffers (each two chunk tiles of 16 KB)
constexpr int B3_THREADS = 512;
constexpr int B3_SMEM = 4 * T128 /*K,V x2*/ + B3_NS * 2 * T64 + B3_DSB * 2 * T128 /*dS^T: buffers x 2 chunks*/ + B3_NS * 512 /*-lse, -D*/ +
                        1024 /*alignment*/ + 512 /*barriers*/;
constexpr uint32_t IDESC_TS_MN = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, 64);     // A K-major (TMEM or smem), B stored [K rows, 64]
constexpr uint32_t IDESC_MN_MN = make_idesc(FMT_BF16, FMT_BF16, 1, 1, 128, 64);     // A stored [K rows, 128], B stored [K rows, 64]

__device__ long long g_b3_trace[8 * 128 * 4];
#define B3_TR(role, step, k) do { if ((p.dbg & 16384) && blockIdx.x == 0 && (step) < 128 && lane == 0) g_b3_trace[((role) * 128 + (step)) * 4 + (k)] = clock64(); } while (0)
#define B3_FAIL() do { atomicExch(p.status, LLMB_ERR_TIMEOUT); failed = true; } while (0)

struct B3Params {
  void* dqkv;            // [B,T,3C] bf16
  const float* stats;    // per (batch, head, 128-row tile): -lse[128] (log2 domain; -inf beyond T), -D[128]
  float* dq_acc;         // per (batch, head, tile): [16 column groups][128 rows][4] fp32, zero on entry
  float* dbias;          // optional fp32 [3C]
  int B, T, NH, C;
  float scale_log2, scale;
  int* status;
  int dbg;
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

// chunk cursor: block cursor plus which half of the block
struct Chk3 { Blk3 b; int g; };
__device__ __forceinline__ void chk3_next(Chk3& c, int n_t, int n_items) {
  c.g ^= 1;
  if (c.g == 0) blk3_next(c.b, n_t, n_items);
}

__global__ void __launch_bounds__(B3_THREADS, 1) attn_bwd3_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                                                  const __grid_constant__ CUtensorMap tmDO, const B3Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sKV = sm;                                  // buffer kb: K at kb*2*T128, V at +T128
  unsigned char* sST = sKV + 4 * T128;                      // ring: stage s holds Q_c at s*2*T64, dO_c at +T64
  unsigned char* sDS = sST + B3_NS * 2 * T64;               // dS^T: buffer b at b*2*T128: chunk 0 at +0, chunk 1 at +T128 ([128 keys][64] each)
  float* sStat = reinterpret_cast<float*>(sDS + B3_DSB * 2 * T128);  // per stage: -lse[64], -D[64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + B3_NS * 128);
  uint64_t* kv_full = bars;                                 // [2]
  uint64_t* kv_empty = kv_full + 2;                         // [2] the tile's last product is complete
  uint64_t* st_full = kv_empty + 2;                         // [NS]
  uint64_t* st_empty = st_full + B3_NS;                     // [NS] the chunk's dV and dK products are complete
  uint64_t* s_full = st_empty + B3_NS;                      // [2] per warpgroup: S^T is in TMEM
  uint64_t* dp_full = s_full + 2;                           // [2] dP^T is in TMEM
  uint64_t* p_full = dp_full + 2;                           // [2] P^T is in TMEM (4 warps)
  uint64_t* p_used = p_full + 2;                            // [2] dV has read P^T
  uint64_t* dp_free = p_used + 2;                           // [2] the warpgroup holds dP^T in registers (4 warps)
  uint64_t* ds_full = dp_free + 2;                          // [2] the chunk's dS^T is in shared memory (4 warps)
  uint64_t* ds_free = ds_full + 2;                          // [2] per dS^T buffer: the block's dK and dQ products are complete
  uint64_t* dq_full = ds_free + 2;                          // [2]
  uint64_t* dq_free = dq_full + 2;                          // [2] (4 warps)
  uint64_t* acc_full = dq_free + 2;                         // dK and dV of a tile are complete
  uint64_t* acc_free = acc_full + 1;                        // ... and have left TMEM (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_t = ceil_div(p.T, TILE);
  const int n_items = ((n_t + 1) / 2) * p.B * p.NH;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 2); mbar_init(&p_used[i], 1); mbar_init(&dp_free[i], 4); mbar_init(&dq_full[i], 1); mbar_init(&dq_free[i], 4);
      mbar_init(&s_full[i], 1); mbar_init(&dp_full[i], 1); mbar_init(&p_full[i], 4);
      mbar_init(&ds_full[i], 4); mbar_init(&ds_free[i], 1);
    }
    for (int i = 0; i < B3_NS; ++i) { mbar_init(&st_full[i], 1); mbar_init(&st_empty[i], 3); }
    mbar_init(acc_full, 2); mbar_init(acc_free, 4);
    fence_barrier_init();
    prefetch_tmap(&tmQKV); prefetch_tmap(&tmDO);
  }
  if (warp == 13) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 320, tDQ = tmem + 384;
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
        if (c.t >= 2 && !mbar_wait(&kv_empty[kb], ((c.t >> 1) + 1) & 1)) { B3_FAIL(); break; }
        if (elect_one()) {
          mbar_expect_tx(&kv_full[kb], 2 * T128);
          load128(sKV + kb * 2 * T128, &tmQKV, &kv_full[kb], colK, c.tile * TILE, b);
          load128(sKV + kb * 2 * T128 + T128, &tmQKV, &kv_full[kb], colV, c.tile * TILE, b);
        }
        __syncwarp();
        // While this tile's chunks are loaded, the operands of the CTA's NEXT tile are pulled into L2, two boxes per
        // chunk, so that its loads find them there.
        Tile3 nx = c;
        tile3_next(nx, nbt, n_t, n_items);
        const int nxb = nx.bh / p.NH, nxh = nx.bh % p.NH, nx0 = nx.tile * TILE;
        const bool pf_on = !nx.done && !(p.dbg & 8192);
        const int pf_per = pf_on ? ceil_div(2 + 2 * (n_t - nx.tile), 2 * nbt) : 0;   // prefetch steps per chunk of this tile
        int pf = nx0 - 128;                                                          // next row to prefetch; the first two steps take K and V
        for (int ic = 0; ic < 2 * nbt; ++ic) {
          const int cc = 2 * c.g + ic, st = cc % B3_NS, i = c.tile + (ic >> 1), g = ic & 1;
          if (cc >= B3_NS && !mbar_wait(&st_empty[st], ((cc / B3_NS) + 1) & 1)) { B3_FAIL(); break; }
          B3_TR(4, cc, 0);
          if (elect_one()) {
            unsigned char* stg = sST + st * 2 * T64;
            const float* src = p.stats + ((size_t)c.bh * n_t + i) * 256 + g * 64;
            mbar_expect_tx(&st_full[st], 2 * T64 + 512);
            tma_load_3d(stg, &tmQKV, &st_full[st], colQ, i * TILE + g * 64, b);
            tma_load_3d(stg + T64, &tmDO, &st_full[st], colQ, i * TILE + g * 64, b);
            bulk_load_1d(sStat + st * 128, src, 256, &st_full[st]);
            bulk_load_1d(sStat + st * 128 + 64, src + 128, 256, &st_full[st]);
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
      // ------------------------------------------------------------ MMA issuer: dV += P^T(c) dO_c
      const uint64_t q_mn0 = make_smem_desc(smem_u32(sST), 8192, 1024);               // dO_c as an MN-major B operand
      for (Chk3 iv{blk3_begin(n_t, n_items), 0}; !iv.b.c.done && !failed; chk3_next(iv, n_t, n_items)) {
        const int cc = 2 * iv.b.n + iv.g, st = cc % B3_NS, g = iv.g;
        const bool first = iv.b.ib == 0 && g == 0, last = iv.b.ib + 1 == iv.b.nbt && g == 1;
        if (!mbar_wait(&p_full[g], iv.b.n & 1)) { B3_FAIL(); break; }
        if (first && iv.b.c.t >= 1 && !mbar_wait(acc_free, (iv.b.c.t - 1) & 1)) { B3_FAIL(); break; }
        fence_after_sync();
        const uint64_t do_mn = q_mn0 + (uint64_t)((st * 2 * T64 + T64) >> 4);
        if (elect_one()) {
          if (!(p.dbg & 128))
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_ts(tDV, tS + g * 64 + ks * 8, do_mn + 128 * ks, IDESC_TS_MN, (ks > 0 || !first) ? 1u : 0u);
          umma_commit(&p_used[g]);                                                    // P^T(c) has been read: S^T(c+2) may overwrite it
          umma_commit(&st_empty[st]);
          if (last) umma_commit(acc_full);
        }
        __syncwarp();
      }
    } else if (warp == 14) {
      // ------------------------------------------------------------ MMA issuer: dK += dS^T(c) Q_c, and per block dQ = dS K
      const uint64_t k_mn0 = make_smem_desc(smem_u32(sKV), 8192, 1024);               // K as an MN-major B operand
      const uint64_t q_mn0 = make_smem_desc(smem_u32(sST), 8192, 1024);               // Q_c as an MN-major B operand
      const uint64_t ds_kk0 = make_smem_desc(smem_u32(sDS), 16, 1024);                // a dS^T chunk tile as a K-major A operand (K = queries)
      const uint64_t ds_mn0 = make_smem_desc(smem_u32(sDS), T128, 1024);              // a dS^T buffer as an MN-major A operand (M = 128 queries)
      for (Chk3 ik{blk3_begin(n_t, n_items), 0}; !ik.b.c.done && !failed; chk3_next(ik, n_t, n_items)) {
        const int cc = 2 * ik.b.n + ik.g, st = cc % B3_NS, g = ik.g, n = ik.b.n, bb = n & 1, db = n % B3_DSB, kb = ik.b.c.t & 1;
        const bool first = ik.b.ib == 0 && g == 0, last = ik.b.ib + 1 == ik.b.nbt && g == 1;
        if (!mbar_wait(&ds_full[g], n & 1)) { B3_FAIL(); break; }
        if (first && ik.b.c.t >= 1 && !mbar_wait(acc_free, (ik.b.c.t - 1) & 1)) { B3_FAIL(); break; }
        if (g == 1 && n >= 2 && !mbar_wait(&dq_free[bb], ((n >> 1) + 1) & 1)) { B3_FAIL(); break; }
        fence_after_sync();
        const uint64_t q_mn = q_mn0 + (uint64_t)((st * 2 * T64) >> 4);
        const uint64_t dsk = ds_kk0 + (uint64_t)((db * 2 * T128 + g * T128) >> 4), dsm = ds_mn0 + (uint64_t)((db * 2 * T128) >> 4);
        const uint64_t kmn = k_mn0 + (uint64_t)((kb * 2 * T128) >> 4);
        if (elect_one()) {
          if (!(p.dbg & 64))
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_ss<KIND_F16>(tDK, dsk + 2 * ks, q_mn + 128 * ks, IDESC_TS_MN, (ks > 0 || !first) ? 1u : 0u);
          umma_commit(&st_empty[st]);
          if (g == 1) {
            if (!(p.dbg & 1024))
#pragma unroll
            for (int ks = 0; ks < TILE / 16; ++ks) umma_ss<KIND_F16>(tDQ + bb * 64, dsm + 128 * ks, kmn + 128 * ks, IDESC_MN_MN, ks > 0 ? 1u : 0u);
            umma_commit(&dq_full[bb]);
            umma_commit(&ds_free[db]);
            if (last) { umma_commit(acc_full); umma_commit(&kv_empty[kb]); }
          }
        }
        __syncwarp();
      }
    } else {
      // ------------------------------------------------------------ MMA issuer: S^T(c+2) = K Q^T as soon as dV has read P^T(c), then dP^T(c+1) = V dO^T
      const uint64_t k_kk0 = make_smem_desc(smem_u32(sKV), 16, 1024);                 // K / V as K-major A operands
      const uint64_t q_kk0 = make_smem_desc(smem_u32(sST), 16, 1024);                 // Q_c / dO_c as K-major B operands
      Chk3 is{blk3_begin(n_t, n_items), 0}, ip = is;
      auto do_s = [&]() {
        const int cc = 2 * is.b.n + is.g, st = cc % B3_NS, g = is.g, n = is.b.n, kb = is.b.c.t & 1;
        if (is.b.ib == 0 && g == 0 && !mbar_wait(&kv_full[kb], (is.b.c.t >> 1) & 1)) { B3_FAIL(); return; }
        if (!mbar_wait(&st_full[st], (cc / B3_NS) & 1)) { B3_FAIL(); return; }
        if (n >= 1 && !mbar_wait(&p_used[g], (n - 1) & 1)) { B3_FAIL(); return; }     // dV has read the P^T this goes over
        fence_after_sync();
        const uint64_t kd = k_kk0 + (uint64_t)((kb * 2 * T128) >> 4), qd = q_kk0 + (uint64_t)((st * 2 * T64) >> 4);
        if (elect_one()) {
          if (!(p.dbg & 256))
#pragma unroll
          for (int ks = 0; ks < HS / 16; ++ks) umma_ss<KIND_F16>(tS + g * 64, kd + 2 * ks, qd + 2 * ks, IDESC_128x64_KK, ks > 0 ? 1u : 0u);
          umma_commit(&s_full[g]);
        }
        __syncwarp();
        chk3_next(is, n_t, n_items);
      };
      auto do_dp = [&]() {                                                            // st_full / kv_full of this chunk were acquired by do_s
        const int cc = 2 * ip.b.n + ip.g, st = cc % B3_NS, g = ip.g, n = ip.b.n, kb = ip.b.c.t & 1;
        const bool last = ip.b.ib + 1 == ip.b.nbt && g == 1;
        if (n >= 1 && !mbar_wait(&dp_free[g], (n - 1) & 1)) { B3_FAIL(); return; }    // the warpgroup holds dP^T(c-2) in registers
        fence_after_sync();
        const uint64_t vd = k_kk0 + (uint64_t)((kb * 2 * T128 + T128) >> 4), dod = q_kk0 + (uint64_t)((st * 2 * T64 + T64) >> 4);
        if (elect_one()) {
          if (!(p.dbg & 256))
#pragma unroll
          for (int ks = 0; ks < HS / 16; ++ks) umma_ss<KIND_F16>(tDP + g * 64, vd + 2 * ks, dod + 2 * ks, IDESC_128x64_KK, ks > 0 ? 1u : 0u);
          umma_commit(&dp_full[g]);
          umma_commit(&st_empty[st]);                                                 // this warp's reads of the stage (S^T, dP^T)
          if (last) umma_commit(&kv_empty[kb]);
        }
        __syncwarp();
        chk3_next(ip, n_t, n_items);
      };
      if (!is.b.c.done) {
        do_s(); if (!failed) do_s();                                                  // chunks 0 and 1
        if (!failed) do_dp();                                                         // chunk 0
        while (!ip.b.c.done && !failed) {                                             // step m: S^T(m+2), dP^T(m+1)
          if (!is.b.c.done) { do_s(); if (failed) break; }
          do_dp();
        }
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- dQ warpgroup: one thread per query row (dQ) / key row (dK, dV)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    for (Blk3 it = blk3_begin(n_t, n_items); !it.c.done && !failed; blk3_next(it, n_t, n_items)) {
      const int n = it.n, buf = n & 1, i = it.c.tile + it.ib;
      if (!mbar_wait(&dq_full[buf], (n >> 1) & 1)) { B3_FAIL(); break; }
      if (warp == 8) B3_TR(3, n, 0);
      fence_after_sync();
      float* dst = p.dq_acc + ((size_t)it.c.bh * n_t + i) * (TILE * HS) + row * 4;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld32(tDQ + buf * 64 + lane_addr + half * 32, r);
        tmem_wait_ld();
        if (half == 1) {
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&dq_free[buf]);
        }
        if (!(p.dbg & 1))
#pragma unroll
        for (int c = 0; c < 8; ++c)
          red_add_v4(dst + (half * 8 + c) * (TILE * 4), __uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]), __uint_as_float(r[4 * c + 2]),
                     __uint_as_float(r[4 * c + 3]));
      }
      if (it.ib + 1 < it.nbt) continue;
      // the tile's dV and dK
      if (!mbar_wait(acc_full, it.c.t & 1)) { B3_FAIL(); break; }
      fence_after_sync();
      const int b = it.c.bh / p.NH, h = it.c.bh % p.NH, kj = it.c.tile * TILE + row;
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.dqkv) + ((size_t)b * p.T + kj) * (3 * (size_t)p.C) + h * HS;
      const float sc = p.scale;                             // dS^T was stored without the 1/sqrt(HS) factor
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t rv[32], rk[32];
        tmem_ld32(tDV + lane_addr + half * 32, rv);
        tmem_ld32(tDK + lane_addr + half * 32, rk);
        tmem_wait_ld();
        if (half == 1) {
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_free);
        }
        if (kj < p.T) {
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 0]), __uint_as_float(rv[j8 * 8 + 1]));
            u.y = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 2]), __uint_as_float(rv[j8 * 8 + 3]));
            u.z = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 4]), __uint_as_float(rv[j8 * 8 + 5]));
            u.w = pack_bf16x2(__uint_as_float(rv[j8 * 8 + 6]), __uint_as_float(rv[j8 * 8 + 7]));
            *reinterpret_cast<uint4*>(base + 2 * p.C + half * 32 + j8 * 8) = u;
            u.x = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 0]) * sc, __uint_as_float(rk[j8 * 8 + 1]) * sc);
            u.y = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 2]) * sc, __uint_as_float(rk[j8 * 8 + 3]) * sc);
            u.z = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 4]) * sc, __uint_as_float(rk[j8 * 8 + 5]) * sc);
            u.w = pack_bf16x2(__uint_as_float(rk[j8 * 8 + 6]) * sc, __uint_as_float(rk[j8 * 8 + 7]) * sc);
            *reinterpret_cast<uint4*>(base + p.C + half * 32 + j8 * 8) = u;
          }
        }
        if (p.dbias) {                                      // qkv bias gradient, dK and dV parts: column sums of this warp's 32 rows
          float cv[32];
#pragma unroll
          for (int x = 0; x < 32; ++x) cv[x] = kj < p.T ? __uint_as_float(rk[x]) * sc : 0.f;
          const float ck = warp_colsum32(cv, lane);
#pragma unroll
          for (int x = 0; x < 32; ++x) cv[x] = kj < p.T ? __uint_as_float(rv[x]) : 0.f;
          const float cvv = warp_colsum32(cv, lane);
          atomicAdd(p.dbias + p.C + h * HS + half * 32 + lane, ck);
          atomicAdd(p.dbias + 2 * p.C + h * HS + half * 32 + lane, cvv);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroup g: one thread per key row, chunk 2n + g of every block
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tSg = tS + lane_addr + g * 64, tDPg = tDP + lane_addr + g * 64;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    for (Blk3 it = blk3_begin(n_t, n_items); !it.c.done && !failed; blk3_next(it, n_t, n_items)) {
      const int n = it.n, cc = 2 * n + g, st = cc % B3_NS, bb = n & 1;
      const float* stat = sStat + st * 128;
      if (!mbar_wait(&st_full[st], (cc / B3_NS) & 1)) { B3_FAIL(); break; }      // acquire the chunk's row statistics
      if (!mbar_wait(&s_full[g], n & 1)) { B3_FAIL(); break; }
      if ((warp & 3) == 0) B3_TR(1 + g, n, 0);
      fence_after_sync();
      uint32_t s[64];
      {
        uint32_t (&q0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[0]);
        uint32_t (&q1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[32]);
        tmem_ld32(tSg, q0); tmem_ld32(tSg + 32, q1);
      }
      tmem_wait_ld();
      {
        uint32_t pk[32];
        const float4* nl4 = reinterpret_cast<const float4*>(stat);
        auto p_phase = [&](auto diag) {
          const int lim = row - g * 64;                     // diagonal block: local query columns x < lim see nothing of this key
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
        if (p.dbg & 16) { for (int x = 0; x < 32; ++x) pk[x] = s[x]; }
        else if (it.ib == 0) p_phase(std::true_type{}); else p_phase(std::false_type{});
        tmem_st32(tSg, pk);                                 // P^T over the first half of the chunk's score columns
      }
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[g]);
      if ((warp & 3) == 0) B3_TR(1 + g, n, 1);
      if (!mbar_wait(&dp_full[g], n & 1)) { B3_FAIL(); break; }
      if ((warp & 3) == 0) B3_TR(1 + g, n, 2);
      fence_after_sync();
      uint32_t d[64];
      {
        uint32_t (&q0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&d[0]);
        uint32_t (&q1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&d[32]);
        tmem_ld32(tDPg, q0); tmem_ld32(tDPg + 32, q1);
      }
      tmem_wait_ld();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dp_free[g]);
      if (!(p.dbg & 32)) {
        const float4* nd4 = reinterpret_cast<const float4*>(stat + 64);
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
      if (n >= B3_DSB && !mbar_wait(&ds_free[n % B3_DSB], ((n / B3_DSB) + 1) & 1)) { B3_FAIL(); break; }   // the products of the buffer's previous block have read it
      if (!(p.dbg & 512)) {
        const float (&v0)[32] = *reinterpret_cast<const float (*)[32]>(&s[0]);
        const float (&v1)[32] = *reinterpret_cast<const float (*)[32]>(&s[32]);
        store_row32(sDS + (n % B3_DSB) * 2 * T128 + g * T128, row, 0, v0);
        store_row32(sDS + (n % B3_DSB) * 2 * T128 + g * T128, row, 32, v1);
      }
      fence_proxy_async();
      fence_before_sync();                                  // also orders this warp's read of dP^T before the product that overwrites it
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[g]);
      if ((warp & 3) == 0) B3_TR(1 + g, n, 3);
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
                                                           int T, int NH, int C, float scale, int dbg) {
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
    if (qi < T && !(dbg & 4096))
      *reinterpret_cast<uint4*>(dqkv + ((size_t)b * T + qi) * (3 * (size_t)C) + h * HS + chunk * 8) =
          *reinterpret_cast<const uint4*>(tile_s + sw128(row, chunk));
  }
  // Zeroed only now, when every load above has returned its data: a store to an address whose load is still in flight
  // waits for it, and the kernel then runs at a quarter of the memory bandwidth.
  if (!(dbg & 2048))
#pragma unroll
  for (int c = 0; c < 16; ++c) *reinterpret_cast<float4*>(src + c * (TILE * 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
  if (dbias && r < HS) atomicAdd(dbias + h * HS + r, part[0][r] + part[1][r] + part[2][r] + part[3][r]);
}
}  // namespace

LLMB_API int llmb_b3_trace_read(long long* host) { return (int)cudaMemcpyFromSymbol(host, g_b3_trace, sizeof(long long) * 8 * 128 * 4); }

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
  B3Params p{}; p.dqkv = dqkv; p.stats = stats; p.dq_acc = dq_acc; p.dbias = dbias;
  p.B = B; p.T = T; p.NH = NH; p.C = C; p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, B3_SMEM); if (e) return (int)e;
    attr = true;
  }
  const int n_t = ceil_div(T, TILE);
  const long long rows = (long long)B * NH * n_t * TILE;
  { const char* e = getenv("LLMB_B3_DBG"); p.dbg = e ? atoi(e) : 0; }
  if (!(p.dbg & 4))
  attn_bwd3_prep_kernel<<<(unsigned)ceil_div_ll(rows * 8, 256), 256, 0, st>>>(stats, lse, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, B, T, NH, C);
  const long long n_items = (long long)((n_t + 1) / 2) * B * NH;
  const int grid = (int)(n_items < sm_count() ? n_items : sm_count());          // persistent: one CTA per SM
  if (!(p.dbg & 8))
  attn_bwd3_kernel<<<grid, B3_THREADS, B3_SMEM, st>>>(tq, td, p);
  if (!(p.dbg & 2))
  attn_bwd3_dq_kernel<<<(unsigned)(B * NH * n_t), 128, 0, st>>>((__nv_bfloat16*)dqkv, dbias, dq_acc, T, NH, C, p.scale, p.dbg);
  return (int)cudaGetLastError();
}
