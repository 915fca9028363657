// Causal flash attention forward for head size 64 on tcgen05 + TMEM: two query tiles per CTA sharing one
// stream of 128-key blocks, probabilities handed to the second product through tensor memory.
//
// Reference behaviour: llmm/attention.mojo:1748-1945 (attention_fwd: scores, causal softmax, weighted values).
//
// One persistent CTA per SM.  A work item is one (batch, head) and a PAIR of 128-row query tiles (2i, 2i+1);
// the CTA walks the key/value blocks 0 .. 2i+1 once for both tiles (tile 2i stops one block earlier).  The CTA
// has two "lanes" r = 0, 1, each with its own softmax warpgroup, issuing warp and TMEM columns; in item k lane r
// takes tile 2i + (r xor k mod 2), so the longer and the shorter tile alternate between the lanes.  Roles:
//   warps 0..3 / 4..7   softmax of lane 0 / 1: one thread per query row holds the row's 128 scores in registers:
//                       row max, p = 2^(s - m), row sum, P as packed bf16 back into TMEM
//   warps 8..11         output warpgroup: once a tile's last product is complete it reads O from TMEM, divides
//                       by the row sums the softmax warps left in shared memory and stores O and the log-sum-exp,
//                       while the softmax warps are already in the next item
//   warp 12             TMA producer: the item's two Q tiles (double-buffered across items), K/V blocks into a ring
//   warp 13 / 14        MMA issuer of lane 0 / 1: S(j) = Q K_j^T (128 x 128, fp32 in TMEM), one block ahead of the
//                       softmax warps, then O += P(j) V_j with P read from TMEM (the A operand of tcgen05.mma may
//                       live in tensor memory), V_j as an MN-major shared-memory operand
// While one lane's warps are in their exponentials the tensor core runs the other lane's products, so the MUFU
// pipe, the tensor pipe and the loads overlap.  The running output stays in TMEM and is rescaled (by the softmax
// warps, in place) only when a row's maximum grew by more than 2^8 since the last rescale (the row sum is kept
// relative to the same reference maximum).
// TMEM columns (512): S0 0..127 | S1 128..255 | O0 256..319 | O1 320..383 | P0 384..447 | P1 448..511.
//
// Items are scheduled so that the tiles of one (batch, head) run on neighbouring CTAs at the same time (their
// K/V blocks are then read from HBM once and served from L2 to the others) while every CTA still sees each
// tile-pair class (cost 4i + 3 blocks) equally often: in round k, CTA c works on (batch, head)
// k * G + c / n_pairs and pair (c + k) mod n_pairs, with G = gridDim / n_pairs.
#include "attention_common.cuh"

namespace {
constexpr int F3_NS = 3;                                  // K/V ring depth (32 KB per stage)
constexpr int F3_THREADS = 512;                           // 2 softmax warpgroups | output warpgroup | producer, two issuers, one idle warp
constexpr int F3_SMEM = 4 * T128 /*Q: 2 buffers x 2 tiles*/ + F3_NS * 2 * T128 /*K,V ring*/ + 2 * T128 /*output staging, one tile per lane*/ +
                        1024 /*alignment*/ + 512 /*barriers*/ + 4096 /*row statistics*/;
constexpr int F3_POLY = 0;                                // of every 8 score pairs, how many take their exponential on the FMA pipe
constexpr uint32_t IDESC_PV = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, 64);   // A (P) K-major from TMEM, B (V) stored [keys, HS]

#define F3_FAIL() do { atomicExch(p.status, LLMB_ERR_TIMEOUT); failed = true; } while (0)

// D[tmem] (+)= A[tmem] * B[smem]; A: 128 lanes x 8 columns of packed bf16 pairs per K = 16 step.  One thread issues.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d;
}

struct F3Item { int bh, t0, nb0, nb1, nb; bool valid; };
__device__ __forceinline__ F3Item f3_item(int k, int n_t, int n_pairs, int gpw, int BH) {
  const int c = blockIdx.x, grp = c / n_pairs;
  F3Item it;
  it.bh = k * gpw + grp;
  it.valid = grp < gpw && it.bh < BH;
  const int pi = (c % n_pairs + k) % n_pairs;
  it.t0 = 2 * pi;
  it.nb0 = it.t0 + 1;                                     // key blocks tile 2i can see
  it.nb1 = (it.t0 + 1 < n_t) ? it.t0 + 2 : 0;             // tile 2i+1 (absent when the tile count is odd)
  it.nb = it.nb1 ? it.nb1 : it.nb0;
  return it;
}

__global__ void __launch_bounds__(F3_THREADS, 1) attn_fwd3_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tmO,
                                                                   const AttnParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = sm;                                 // buffer qb: tile 2i at qb*2*T128, tile 2i+1 at +T128
  unsigned char* sKV = sQ + 4 * T128;                     // stage s: K block at s*2*T128, V block at +T128
  unsigned char* sOut = sKV + F3_NS * 2 * T128;           // lane r: the tile's rounded output rows, swizzled, source of its TMA stores
  uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + 2 * T128);
  uint64_t* q_full = bars;                                // [2]
  uint64_t* q_empty = q_full + 2;                         // [lane][2] the lane's last score product of the item is complete
  uint64_t* kv_full = q_empty + 4;                        // [NS]
  uint64_t* kv_empty = kv_full + F3_NS;                   // [lane][NS] the lane is done with the stage
  uint64_t* s_full = kv_empty + 2 * F3_NS;                // [2] per lane: S is in TMEM
  uint64_t* s_free = s_full + 2;                          // [2] per lane: the softmax warps hold S in registers
  uint64_t* p_full = s_free + 2;                          // [2] per lane: P is in TMEM (and O rescaled if needed)
  uint64_t* pv_done = p_full + 2;                         // [2] per lane: O += P V complete (P may be overwritten)
  uint64_t* o_free = pv_done + 2;                         // [2] per lane: the item's output has left TMEM
  uint64_t* fin = o_free + 2;                             // [2] per lane: the item's row statistics are in shared memory
  uint64_t* out_ready = fin + 2;                          // [2] per lane: the staging tile is written (4 warps)
  uint64_t* out_done = out_ready + 2;                     // [2] per lane: its TMA stores have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(out_done + 2);
  float* stats = reinterpret_cast<float*>(bars + 64);     // [lane][item parity][m | l][128 rows]

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int n_t = ceil_div(p.T, TILE), n_pairs = (n_t + 1) / 2, BH = p.B * p.NH;
  const int gpw = max(1, min((int)gridDim.x / n_pairs, BH));

  if (tid == 0) {
    // Every "empty" barrier has ONE arriving thread (the lane's issuer, through tcgen05.commit), so arrivals can
    // never spill into a neighbouring phase; the producer waits for both lanes' barriers.
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); mbar_init(&q_empty[2 + i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1); mbar_init(&o_free[i], 4); mbar_init(&fin[i], 4);
      mbar_init(&out_ready[i], 4); mbar_init(&out_done[i], 1);
    }
    for (int i = 0; i < F3_NS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&kv_empty[F3_NS + i], 1); }
    fence_barrier_init();
    prefetch_tmap(&tm); prefetch_tmap(&tmO);
  }
  if (warp == 13) tmem_alloc<512>(tmem_slot);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;
  // Registers move from the output and producer / issuer warpgroups to the two softmax warpgroups:
  // 2 x 128 x 176 + 2 x 128 x 80 = 65536 = the 512 x 128 registers the CTA was launched with.  A warpgroup can only
  // grow into registers that warpgroups of the same CTA have released: asking for more than that would block
  // forever.  Each role sets its limit at the top of its own branch (the register allocator follows control flow).
  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if (warp == 12) {
      // ---------------------------------------------------------- TMA producer
      int g = 0;
      for (int k = 0; !failed; ++k) {
        const F3Item it = f3_item(k, n_t, n_pairs, gpw, BH);
        if (!it.valid) break;
        const int b = it.bh / p.NH, h = it.bh % p.NH, qb = k & 1;
        const int colQ = h * HS, colK = p.C + h * HS, colV = 2 * p.C + h * HS;
        if (k >= 2 && !(mbar_wait(&q_empty[qb], ((k >> 1) + 1) & 1) && mbar_wait(&q_empty[2 + qb], ((k >> 1) + 1) & 1))) { F3_FAIL(); break; }
        if (elect_one()) {
          mbar_expect_tx(&q_full[qb], 2 * T128);
          load128(sQ + qb * 2 * T128, &tm, &q_full[qb], colQ, it.t0 * TILE, b);
          load128(sQ + qb * 2 * T128 + T128, &tm, &q_full[qb], colQ, (it.t0 + 1) * TILE, b);
        }
        __syncwarp();
        for (int j = 0; j < it.nb; ++j, ++g) {
          const int st = g % F3_NS;
          if (g >= F3_NS && !(mbar_wait(&kv_empty[st], ((g / F3_NS) + 1) & 1) && mbar_wait(&kv_empty[F3_NS + st], ((g / F3_NS) + 1) & 1))) { F3_FAIL(); break; }
          if (elect_one()) {
            mbar_expect_tx(&kv_full[st], 2 * T128);
            load128(sKV + st * 2 * T128, &tm, &kv_full[st], colK, j * TILE, b);
            load128(sKV + st * 2 * T128 + T128, &tm, &kv_full[st], colV, j * TILE, b);
          }
          __syncwarp();
        }
      }
    } else if (warp == 13 || warp == 14) {
      // ---------------------------------------------------------- MMA issuer of lane r
      const int r = warp - 13;
      const uint32_t tS = tmem + r * 128, tO = tmem + 256 + r * 64, tP = tmem + 384 + r * 64;
      uint64_t* my_q_empty = q_empty + 2 * r;
      uint64_t* my_kv_empty = kv_empty + F3_NS * r;
      int g0 = 0, cs = 0, cp = 0, no = 0;                 // blocks before this item; S / PV / item counts of this lane
      // Descriptors are built by the whole warp outside the single-lane branches (warp-uniform values stay in uniform
      // registers; a descriptor assembled inside a one-lane branch costs the issuing thread far more than the MMA).
      const uint64_t q_desc0 = make_smem_desc(smem_u32(sQ), 16, 1024);
      const uint64_t k_desc0 = make_smem_desc(smem_u32(sKV), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc(smem_u32(sKV + T128), 8192, 1024);
      for (int k = 0; !failed; ++k) {
        const F3Item it = f3_item(k, n_t, n_pairs, gpw, BH);
        if (!it.valid) break;
        const int qb = k & 1, tt = r ^ (k & 1), nbt = tt ? it.nb1 : it.nb0;
        const uint64_t q_desc = q_desc0 + (uint64_t)(((qb * 2 + tt) * T128) >> 4);
        // the item's Q buffer and every K/V stage are acquired before they are released, also where this lane does
        // not read them: the producer has then finished its wait for the previous release of the same buffer
        if (!mbar_wait(&q_full[qb], (k >> 1) & 1)) { F3_FAIL(); break; }
        if (nbt > 0) {
          auto issue_s = [&](int j) {
            const int g = g0 + j, st = g % F3_NS;
            if (!mbar_wait(&kv_full[st], (g / F3_NS) & 1)) { F3_FAIL(); return; }
            if (cs >= 1 && !mbar_wait(&s_free[r], (cs - 1) & 1)) { F3_FAIL(); return; }
            fence_after_sync();
            const uint64_t k_desc = k_desc0 + (uint64_t)((st * 2 * T128) >> 4);
            if (elect_one()) {
#pragma unroll
              for (int ks = 0; ks < HS / 16; ++ks)                                              // S = Q K^T
                umma_ss<KIND_F16>(tS, q_desc + 2 * ks, k_desc + 2 * ks, IDESC_S_128x128, ks > 0 ? 1u : 0u);
              umma_commit(&s_full[r]);
              if (j == nbt - 1) umma_commit(&my_q_empty[qb]);
            }
            __syncwarp();
            ++cs;
          };
          issue_s(0);
          for (int j = 0; j < nbt && !failed; ++j) {
            if (j + 1 < nbt) issue_s(j + 1);
            if (failed) break;
            const int st = (g0 + j) % F3_NS;
            if (!mbar_wait(&p_full[r], cp & 1)) { F3_FAIL(); break; }
            if (j == 0 && no >= 1 && !mbar_wait(&o_free[r], (no - 1) & 1)) { F3_FAIL(); break; }
            fence_after_sync();
            const uint64_t vd = v_desc0 + (uint64_t)((st * 2 * T128) >> 4);
            const uint32_t acc0 = j > 0 ? 1u : 0u;
            if (elect_one()) {
#pragma unroll
              for (int ks = 0; ks < TILE / 16; ++ks)                                            // O (+)= P V
                umma_ts(tO, tP + ks * 8, vd + 128 * ks, IDESC_PV, ks > 0 ? 1u : acc0);
              umma_commit(&pv_done[r]);
              umma_commit(&my_kv_empty[st]);
            }
            __syncwarp();
            ++cp;
          }
          ++no;
        } else if (elect_one()) {
          umma_commit(&my_q_empty[qb]);                   // tile absent: nothing of it reads this Q buffer
        }
        if (failed) break;
        // blocks this lane does not look at: release them in order behind the lane's own products
        for (int j = nbt; j < it.nb && !failed; ++j) {
          const int g = g0 + j, st = g % F3_NS;
          if (!mbar_wait(&kv_full[st], (g / F3_NS) & 1)) { F3_FAIL(); break; }
          if (elect_one()) umma_commit(&my_kv_empty[st]);
          __syncwarp();
        }
        g0 += it.nb;
      }
    }
  } else if (warp >= 8) {
    // -------------------------------------------------------------- output warpgroup: one thread per query row
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    int cp[2] = {0, 0}, ni[2] = {0, 0}, no[2] = {0, 0};   // per lane: products / items / output tiles so far
    for (int k = 0; !failed; ++k) {
      const F3Item it = f3_item(k, n_t, n_pairs, gpw, BH);
      if (!it.valid) break;
      const int b = it.bh / p.NH, h = it.bh % p.NH;
      // the shorter tile (2i) finishes first; waits suspend the warp instead of spinning next to the softmax warps
      for (int tt = 0; tt < 2 && !failed; ++tt) {
        {
          const int r = tt ^ (k & 1);
          if ((tt ? it.nb1 : it.nb0) == 0) continue;
          if (!mbar_wait(&fin[r], ni[r] & 1)) { F3_FAIL(); break; }
          const int nbt = tt ? it.nb1 : it.nb0, qi = (it.t0 + tt) * TILE + row;
          cp[r] += nbt;
          const float* st = stats + r * 512 + (ni[r] & 1) * 256;
          const float m_run = st[row], l_run = st[128 + row];
          ++ni[r];
          if (!mbar_wait(&pv_done[r], (cp[r] - 1) & 1)) { F3_FAIL(); break; }      // the tile's last product
          fence_after_sync();
          const uint32_t tO = tmem + 256 + r * 64 + lane_addr;
          const float inv = 1.0f / l_run;
          // The rounded rows go through a swizzled staging tile and leave as two TMA stores (whole 128-byte rows, rows beyond
          // T clipped by the tensor map): 16-byte stores per thread at a row stride of C keep a warp on 32 sectors per
          // instruction and this warpgroup busy for longer than a short item takes.
          unsigned char* stg = sOut + r * T128;
          if (no[r] >= 1 && !mbar_wait(&out_done[r], (no[r] - 1) & 1)) { F3_FAIL(); break; }   // the previous tile's stores have read it
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            uint32_t o[32];
            tmem_ld32(tO + half * 32, o);
            tmem_wait_ld();
            if (half == 1) {                              // O has left TMEM: the lane's next item may overwrite it
              fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&o_free[r]);
            }
            float v[32];
#pragma unroll
            for (int x = 0; x < 32; ++x) v[x] = __uint_as_float(o[x]) * inv;
            store_row32(stg, row, half * 32, v);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&out_ready[r]);
          if (warp == 8) {
            if (!mbar_wait(&out_ready[r], no[r] & 1)) { F3_FAIL(); break; }
            if (elect_one()) {
              tma_store_3d(&tmO, stg, h * HS, (it.t0 + tt) * TILE, b);
              tma_store_3d(&tmO, stg + T64, h * HS, (it.t0 + tt) * TILE + 64, b);
              bulk_commit();
              bulk_wait_read<0>();
              mbar_arrive(&out_done[r]);
            }
            __syncwarp();
          }
          ++no[r];
          if (qi < p.T) p.lse[(size_t)it.bh * p.T + qi] = m_run + log2f(l_run);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- softmax warps of lane r: one thread per query row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int r = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + r * 128 + lane_addr, tO = tmem + 256 + r * 64 + lane_addr, tP = tmem + 384 + r * 64 + lane_addr;
    const float sc = p.scale_log2;
    const float2 sc2 = make_float2(sc, sc);
    int cs = 0, cp = 0, ni = 0;
    for (int k = 0; !failed; ++k) {
      const F3Item it = f3_item(k, n_t, n_pairs, gpw, BH);
      if (!it.valid) break;
      const int tt = r ^ (k & 1), nbt = tt ? it.nb1 : it.nb0;
      if (nbt == 0) continue;
      const int tile = it.t0 + tt;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < nbt; ++j) {
        if (!mbar_wait(&s_full[r], cs & 1)) { F3_FAIL(); break; }
        fence_after_sync();
        uint32_t s[128];
        {
          uint32_t (&q0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[0]);
          uint32_t (&q1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[32]);
          uint32_t (&q2)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[64]);
          uint32_t (&q3)[32] = *reinterpret_cast<uint32_t (*)[32]>(&s[96]);
          tmem_ld32(tS, q0); tmem_ld32(tS + 32, q1); tmem_ld32(tS + 64, q2); tmem_ld32(tS + 96, q3);
        }
        tmem_wait_ld();
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[r]);           // the next block's scores may overwrite S now
        ++cs;
        if (j == tile) {                                  // diagonal block: keys after the query are masked
#pragma unroll
          for (int x = 0; x < 128; ++x)
            if (x > row) s[x] = 0xff800000u;
        }
        float mx4[4];                                     // four independent chains: the row maximum is latency, not work
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mx4[c] = fmaxf(__uint_as_float(s[c * 32]), __uint_as_float(s[c * 32 + 1]));
#pragma unroll
          for (int x = 2; x < 32; x += 2) mx4[c] = max3(mx4[c], __uint_as_float(s[c * 32 + x]), __uint_as_float(s[c * 32 + x + 1]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
        // the reference maximum only moves when it grew by more than 8 (a factor 256 in p): rescales of O become rare
        float m_new = fmaxf(m_run, mx);
        if (m_new - m_run <= 8.0f) m_new = m_run;
        const float alpha = ex2_approx(m_run - m_new);    // m_run = -inf on the first block gives 0
        m_run = m_new;
        // O += P(j-1) V must be complete before O is rescaled and before P is overwritten
        if (cp >= 1 && !mbar_wait(&pv_done[r], (cp - 1) & 1)) { F3_FAIL(); break; }
        fence_after_sync();
        if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.0f)) {
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            uint32_t o[32];
            tmem_ld32(tO + half * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
            tmem_st32(tO + half * 32, o);
          }
        }
        const float2 nm2 = make_float2(-m_new, -m_new);
        float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        // F3_POLY of every 8 score pairs can take their exponential on the FMA pipe instead of the MUFU pipe:
        // 2^t = 2^n * q(f) with n = round(t), f = t - n in [-0.5, 0.5] and q a cubic (relative error 8e-5, far below
        // the bf16 rounding of P), n added to the exponent bits.  Measured: a polynomial pair costs 18 cycles of the FMA
        // and integer pipes against 16 of the MUFU pipe for two ex2, and the kernel is bound by the latencies of its
        // load / store / wait chain rather than by either pipe, so the default is 0.
#pragma unroll
        for (int x = 0; x < 64; ++x) {
          const float2 t2 = __ffma2_rn(make_float2(__uint_as_float(s[2 * x]), __uint_as_float(s[2 * x + 1])), sc2, nm2);
          float e0, e1;
          if ((x & 7) < F3_POLY) {
            const float2 magic = make_float2(12582912.f, 12582912.f);               // 1.5 * 2^23: adding it rounds to an integer
            const float2 tc = make_float2(fmaxf(t2.x, -126.f), fmaxf(t2.y, -126.f));
            const float2 fl = __fadd2_rn(tc, magic);
            const float2 f = __fadd2_rn(tc, __fadd2_rn(magic, make_float2(-fl.x, -fl.y)));   // t - round(t)
            float2 q = __ffma2_rn(make_float2(0.05520550534f, 0.05520550534f), f, make_float2(0.2426139712f, 0.2426139712f));
            q = __ffma2_rn(q, f, make_float2(0.6932547688f, 0.6932547688f));
            q = __ffma2_rn(q, f, make_float2(0.9999276996f, 0.9999276996f));
            e0 = __uint_as_float(__float_as_uint(q.x) + (__float_as_uint(fl.x) << 23));
            e1 = __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(fl.y) << 23));
          } else {
            e0 = ex2_approx(t2.x); e1 = ex2_approx(t2.y);
          }
          acc[x & 3] = __fadd2_rn(acc[x & 3], make_float2(e0, e1));
          s[x] = pack_bf16x2(e0, e1);                     // P(j) as bf16 pairs replaces the scores already consumed
        }
        {
          const uint32_t (&p0)[32] = *reinterpret_cast<const uint32_t (*)[32]>(&s[0]);
          const uint32_t (&p1)[32] = *reinterpret_cast<const uint32_t (*)[32]>(&s[32]);
          tmem_st32(tP, p0); tmem_st32(tP + 32, p1);
        }
        const float2 a01 = __fadd2_rn(acc[0], acc[1]), a23 = __fadd2_rn(acc[2], acc[3]);
        l_run = l_run * alpha + ((a01.x + a01.y) + (a23.x + a23.y));
        tmem_wait_st();
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[r]);
        ++cp;
      }
      if (failed) break;
      // Hand the row statistics to the output warpgroup and go on with the next item.  The previous item's output
      // must have been taken first, so that `fin` never runs two phases ahead of its reader.
      if (ni >= 1 && !mbar_wait(&o_free[r], (ni - 1) & 1)) { F3_FAIL(); break; }
      float* st = stats + r * 512 + (ni & 1) * 256;
      st[row] = m_run; st[128 + row] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&fin[r]);
      ++ni;
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 13) { fence_after_sync(); tmem_dealloc<512>(tmem); }
}
}  // namespace

// out [B,T,C] bf16, lse [B,NH,T] fp32 (log2 domain), qkv [B,T,3C] bf16; C = NH*64.
LLMB_API int llmb_attention_fwd_pair(void* out, float* lse, const void* qkv, int B, int T, int NH, int* status, cudaStream_t st) {
  const int C = NH * HS;
  CUtensorMap tm;
  int rc = make_qkv_map(&tm, qkv, B, T, 3 * C);
  if (rc) return 1000 + rc;
  CUtensorMap tmo;
  rc = make_qkv_map(&tmo, out, B, T, C);
  if (rc) return 1000 + rc;
  AttnParams p{}; p.out = out; p.lse = lse; p.B = B; p.T = T; p.NH = NH; p.C = C;
  p.scale = 0.125f; p.scale_log2 = 0.125f * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) { cudaError_t e = cudaFuncSetAttribute(attn_fwd3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F3_SMEM); if (e) return (int)e; attr = true; }
  const int n_t = ceil_div(T, TILE), n_pairs = (n_t + 1) / 2;
  const long long n_items = (long long)n_pairs * B * NH;
  int grid = sm_count();
  if (n_items < grid) grid = (int)n_items;
  if (grid < n_pairs) grid = n_pairs;                     // one (batch, head) needs n_pairs CTAs side by side
  attn_fwd3_kernel<<<grid, F3_THREADS, F3_SMEM, st>>>(tm, tmo, p);
  return (int)cudaGetLastError();
}
