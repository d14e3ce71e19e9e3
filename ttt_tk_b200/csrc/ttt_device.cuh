// Device helpers shared by the forward and backward TTT-MLP kernels: the GELU family
// (reference: include/common/base_ops.cuh:465-548 and kernels/ttt_backward/matching.py:42-55),
// bf16 row access to 128-byte-swizzled tiles, and the two MMA forms every contraction of
// the operator reduces to.
#pragma once

#include "sm100_ptx.cuh"

namespace tttdev {

using namespace sm100;

constexpr uint32_t TILE = 8192;    // 64 x 64 bf16 tile
constexpr uint32_t BIG = 32768;    // 256 x 64 bf16 tile ("hidden-major": one row per hidden unit)

constexpr float kG0 = 0.79788456f, kG1 = 0.044715f, kG2 = 0.1070322243f;

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// gelu(x) and gelu'(x), tanh approximation
__device__ __forceinline__ void gelu_pair(float x, float& g, float& gp) {
  const float x2 = x * x;
  const float t = tanh_fast(kG0 * x * fmaf(kG1, x2, 1.f));
  const float h = 0.5f * (1.f + t);
  g = x * h;
  gp = fmaf(0.5f * x * (1.f - t * t), fmaf(kG2, x2, kG0), h);
}
__device__ __forceinline__ float gelu_only(float x) {
  const float t = tanh_fast(kG0 * x * fmaf(kG1, x * x, 1.f));
  return 0.5f * x * (1.f + t);
}
__device__ __forceinline__ float gelu_grad(float x) {
  const float x2 = x * x;
  const float t = tanh_fast(kG0 * x * fmaf(kG1, x2, 1.f));
  return fmaf(0.5f * x * (1.f - t * t), fmaf(kG2, x2, kG0), 0.5f * (1.f + t));
}
// gelu'(x) and gelu''(x)
__device__ __forceinline__ void gelu_grad_pair(float x, float& gp, float& gpp) {
  const float x2 = x * x;
  const float t = tanh_fast(kG0 * x * fmaf(kG1, x2, 1.f));
  const float s = 1.f - t * t;
  const float q = fmaf(kG2, x2, kG0);                 // kG0 + 3 kG0 kG1 x^2
  gp = fmaf(0.5f * x * s, q, 0.5f * (1.f + t));
  gpp = s * (fmaf(2.f * kG2, x2, kG0) - x * t * q * q);  // kG0 + 6 kG0 kG1 x^2 - x t q^2
}

__device__ __forceinline__ uint4 pack_chunk(const float* v) {
  uint4 w;
  w.x = pack_bf16(v[0], v[1]);
  w.y = pack_bf16(v[2], v[3]);
  w.z = pack_bf16(v[4], v[5]);
  w.w = pack_bf16(v[6], v[7]);
  return w;
}
__device__ __forceinline__ void unpack_chunk(const uint4 w, float* v) {
  v[0] = bf16_lo(w.x); v[1] = bf16_hi(w.x);
  v[2] = bf16_lo(w.y); v[3] = bf16_hi(w.y);
  v[4] = bf16_lo(w.z); v[5] = bf16_hi(w.z);
  v[6] = bf16_lo(w.w); v[7] = bf16_hi(w.w);
}
// 8 consecutive elements (16-byte chunk `chunk`) of row `row` of a swizzled tile
__device__ __forceinline__ void st_chunk(uint8_t* tile, uint32_t row, uint32_t chunk, const float* v) {
  *reinterpret_cast<uint4*>(tile + sw128_off(row, chunk)) = pack_chunk(v);
}
__device__ __forceinline__ void ld_chunk(const uint8_t* tile, uint32_t row, uint32_t chunk, float* v) {
  unpack_chunk(*reinterpret_cast<const uint4*>(tile + sw128_off(row, chunk)), v);
}
__device__ __forceinline__ float ld_elem(const uint8_t* tile, uint32_t row, uint32_t col) {
  return __bfloat162float(
      *reinterpret_cast<const __nv_bfloat16*>(tile + sw128_off(row, col >> 3) + (col & 7) * 2));
}

// ---- MMA issue.  One thread issues every MMA of the kernels, so the instruction stream
// around each tcgen05.mma is kept to two integer adds: the descriptors' high words are the
// same constant for every operand (stride byte offset 1024, version 1, 128-byte swizzle) and
// the low words (start address | leading byte offset) advance by a constant per K step.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_issue(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %4};\n\t"
      "mov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kDescHi), "n"(kAccumulate ? 1 : 0)
      : "memory");
}

// "Hidden-major" product: D[256 x 64] (two M=128 blocks, 64 fp32 columns each, at tmem_d and
// tmem_d + 64) (+)= A * B with A a [256][64] bf16 tile read K-major (row = hidden unit) and B a
// [64][64] tile read K-major (row = N index) or MN-major (row = K index).
template <bool kBMn, bool kAccumulate>
__device__ __forceinline__ void mma_hidden_major_t(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 64, false, kBMn, false);
  const uint32_t a0 = desc_lo(a_smem, 16);
  const uint32_t b0 = desc_lo(b_smem, kBMn ? 8192 : 16);
  constexpr uint32_t bstep = kBMn ? (2048u >> 4) : (32u >> 4);
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    if (kAccumulate) mma_issue<true>(tmem_d + blk * 64, a0 + blk * (16384u >> 4), b0, idesc);
    else             mma_issue<false>(tmem_d + blk * 64, a0 + blk * (16384u >> 4), b0, idesc);
#pragma unroll
    for (int j = 1; j < 4; ++j)
      mma_issue<true>(tmem_d + blk * 64, a0 + blk * (16384u >> 4) + j * 2, b0 + j * bstep, idesc);
  }
}
__device__ __forceinline__ void mma_hidden_major(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem, bool b_mn,
                                                 bool accumulate) {
  if (b_mn) {
    if (accumulate) mma_hidden_major_t<true, true>(tmem_d, a_smem, b_smem);
    else            mma_hidden_major_t<true, false>(tmem_d, a_smem, b_smem);
  } else {
    if (accumulate) mma_hidden_major_t<false, true>(tmem_d, a_smem, b_smem);
    else            mma_hidden_major_t<false, false>(tmem_d, a_smem, b_smem);
  }
}
// "Token-major" product: D[64 tok x 64] (M = 64: row r in TMEM lane (r % 16) + 32 * (r / 16))
// = X[64 x 256] * W[256 x 64], both operands [256][64] tiles read MN-major (row = hidden unit).
__device__ __forceinline__ void mma_token_major(uint32_t tmem_d, uint32_t x_smem, uint32_t w_smem) {
  constexpr uint32_t idesc = umma_idesc_bf16(64, 64, true, true, false);
  const uint32_t a0 = desc_lo(x_smem, BIG);
  const uint32_t b0 = desc_lo(w_smem, BIG);
  mma_issue<false>(tmem_d, a0, b0, idesc);
#pragma unroll
  for (int j = 1; j < 16; ++j) mma_issue<true>(tmem_d, a0 + j * (2048u >> 4), b0 + j * (2048u >> 4), idesc);
}

}  // namespace tttdev
