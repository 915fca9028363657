// Shared pieces of the attention kernels (head size 64): tile constants, the parameter block, swizzled
// shared-memory addressing and the tcgen05 issue helpers.  Included by attention.cu (backward) and
// attention_fwd.cu (forward); everything lives in an anonymous namespace per translation unit.
#pragma once
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
  float* dbias;         // bwd, optional: fp32 [3C], += column sums of dqkv (the gradient of the qkv bias)
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

// Column sums across a warp: every lane holds 32 values (one row, 32 columns); afterwards lane c holds the sum of
// column c over the 32 lanes.  Butterfly reduce-scatter: 31 shuffles instead of 32 x 5.
template <int NLEFT>
__device__ __forceinline__ void colsum_step(float (&v)[32], int lane) {
  constexpr int H = NLEFT / 2;
  const bool upper = (lane & H) != 0;
#pragma unroll
  for (int i = 0; i < H; ++i) {
    const float send = upper ? v[i] : v[i + H];
    const float keep = upper ? v[i + H] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, H);
  }
}
__device__ __forceinline__ float warp_colsum32(float (&v)[32], int lane) {
  colsum_step<32>(v, lane); colsum_step<16>(v, lane); colsum_step<8>(v, lane); colsum_step<4>(v, lane); colsum_step<2>(v, lane);
  return v[0];
}

// a 128-row tile is fetched as two 64-row boxes (same swizzled layout, one tensor map for every tile size)
__device__ __forceinline__ void load128(unsigned char* dst, const CUtensorMap* t, uint64_t* bar, int col, int row, int b) {
  tma_load_3d(dst, t, bar, col, row, b);
  tma_load_3d(dst + T64, t, bar, col, row + 64, b);
}


// [B, T, width] bf16 viewed as a 3-D tensor; every load is a box of 64 rows x 64 columns
inline int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int T, int width) {
  return make_tmap_3d(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)T, (uint64_t)B,
                      (uint64_t)width, (uint64_t)width * T, HS, 64);
}
}  // namespace
