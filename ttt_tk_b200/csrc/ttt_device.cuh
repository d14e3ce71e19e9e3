// Device helpers shared by the forward and backward TTT-MLP kernels: the GELU family
// (reference: include/common/base_ops.cuh:465-548 and kernels/ttt_backward/matching.py:42-55),
// bf16 row access to 128-byte-swizzled tiles, and the two MMA forms every contraction of
// the operator reduces to.
#pragma once

#include "sm100_ptx.cuh"
#include <cuda_fp16.h>

namespace tttdev {

using namespace sm100;

constexpr uint32_t TILE = 8192;    // 64 x 64 bf16 tile
constexpr uint32_t BIG = 32768;    // 256 x 64 bf16 tile ("hidden-major": one row per hidden unit)

constexpr float kG0 = 0.79788456f, kG1 = 0.044715f, kG2 = 0.1070322243f;
constexpr float kG01 = kG0 * kG1;      // tanh argument: kG0 x (1 + kG1 x^2) = x (kG0 + kG01 x^2), one multiply less

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// gelu(x), gelu'(x), gelu''(x), tanh approximation.  With t = tanh(x (kG0 + kG01 x^2)), h = (1 + t) / 2
// and q = kG0 + kG2 x^2 (the argument's derivative):
//   gelu = x h,   gelu' = h + x (1 - t^2) q / 2 = h + (g - g t) q   (since (1 - t^2) / 2 = h (1 - t)),
//   gelu'' = (1 - t^2) (kG0 + 2 kG2 x^2 - x t q^2).
__device__ __forceinline__ void gelu_pair(float x, float& g, float& gp) {
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(kG01, x2, kG0));
  const float h = fmaf(0.5f, t, 0.5f);
  g = x * h;
  gp = fmaf(fmaf(-g, t, g), fmaf(kG2, x2, kG0), h);
}
__device__ __forceinline__ float gelu_only(float x) {
  const float t = tanh_fast(x * fmaf(kG01, x * x, kG0));
  return x * fmaf(0.5f, t, 0.5f);
}
// gelu'(x) and gelu''(x)
__device__ __forceinline__ void gelu_grad_pair(float x, float& gp, float& gpp) {
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(kG01, x2, kG0));
  const float h = fmaf(0.5f, t, 0.5f);
  const float g = x * h;
  const float q = fmaf(kG2, x2, kG0);                 // kG0 + 3 kG0 kG1 x^2
  gp = fmaf(fmaf(-g, t, g), q, h);
  gpp = fmaf(-t, t, 1.f) * fmaf(-(x * t * q), q, fmaf(2.f * kG2, x2, kG0));
}

// ---- The same family on two elements at a time in packed fp16 arithmetic.  The tanh-GELU and its
// derivatives are O(1) functions of O(1) arguments, so fp16 (11 significand bits) evaluates them to
// ~5e-4 (gelu'': ~2e-3), below the bf16 rounding (4e-3) every result meets when it is stored as an MMA
// operand; one instruction then serves two elements.  The argument is clamped to +-20, beyond which
// gelu' is 0 or 1 and gelu'' is 0 to fp16 precision (and x^3 would leave the fp16 range); gelu
// itself stays in fp32: on fp32 arguments the conversions cost what the packed arithmetic saves, so
// only the derivatives of arguments read from bf16 tiles use this path.
struct GeluH2 {
  __half2 x, x2, t, hh;   // clamped argument, its square, tanh(u), 0.5 (1 + tanh(u))
};
__device__ __forceinline__ __half2 h2c(float v) { return __float2half2_rn(v); }
__device__ __forceinline__ __half2 tanh_h2(__half2 u) {
  uint32_t r;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(r) : "r"(*reinterpret_cast<const uint32_t*>(&u)));
  return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ GeluH2 gelu_h2_core(float x0, float x1) {
  GeluH2 c;
  c.x = __hmax2(__hmin2(__floats2half2_rn(x0, x1), h2c(20.f)), h2c(-20.f));
  c.x2 = __hmul2(c.x, c.x);
  const __half2 u = __hmul2(c.x, __hfma2(h2c(kG01), c.x2, h2c(kG0)));
  c.t = tanh_h2(u);
  c.hh = __hfma2(h2c(0.5f), c.t, h2c(0.5f));
  return c;
}
// gelu'(x) from the core values: h + (g - g t) q
__device__ __forceinline__ __half2 gelu_h2_grad(const GeluH2& c, __half2& q) {
  const __half2 g = __hmul2(c.x, c.hh);
  q = __hfma2(h2c(kG2), c.x2, h2c(kG0));
  return __hfma2(__hfma2(__hneg2(g), c.t, g), q, c.hh);
}
__device__ __forceinline__ void gelu_grad_pair2(float x0, float x1, float& gp0, float& gp1, float& gpp0,
                                                float& gpp1) {
  const GeluH2 c = gelu_h2_core(x0, x1);
  __half2 q;
  const float2 gp = __half22float2(gelu_h2_grad(c, q));
  const __half2 s = __hfma2(__hneg2(c.t), c.t, h2c(1.f));
  const __half2 cc = __hfma2(h2c(2.f * kG2), c.x2, h2c(kG0));
  const __half2 xtq = __hmul2(__hmul2(c.x, c.t), q);
  const float2 gpp = __half22float2(__hmul2(s, __hfma2(__hneg2(xtq), q, cc)));
  gp0 = gp.x;
  gp1 = gp.y;
  gpp0 = gpp.x;
  gpp1 = gpp.y;
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
// the raw 16 bytes of a chunk: requested between a tensor-memory load and its wait, unpacked after
__device__ __forceinline__ uint4 ld_chunk_raw(const uint8_t* tile, uint32_t row, uint32_t chunk) {
  return *reinterpret_cast<const uint4*>(tile + sw128_off(row, chunk));
}
__device__ __forceinline__ float ld_elem(const uint8_t* tile, uint32_t row, uint32_t col) {
  return __bfloat162float(
      *reinterpret_cast<const __nv_bfloat16*>(tile + sw128_off(row, col >> 3) + (col & 7) * 2));
}

// A kernel whose instruction footprint exceeds the instruction cache defines TTT_MMA_ROLLED 1 before
// including this header (rolled issue loops); a small kernel keeps them unrolled (lower issue latency).
#ifndef TTT_MMA_ROLLED
#define TTT_MMA_ROLLED 0
#endif
#ifndef TTT_MMA_SHARED_LOOP
#define TTT_MMA_SHARED_LOOP (TTT_MMA_ROLLED == 1)
#endif
#if TTT_MMA_ROLLED == 1
#define TTT_MMA_LOOP _Pragma("unroll 1")
#define TTT_MMA_OUTER _Pragma("unroll 1")
#elif TTT_MMA_ROLLED == 2
#define TTT_MMA_LOOP _Pragma("unroll 4")
#define TTT_MMA_OUTER _Pragma("unroll 1")
#else
#define TTT_MMA_LOOP _Pragma("unroll")
#define TTT_MMA_OUTER _Pragma("unroll")
#endif

// ---- MMA issue.  Four threads (lane 0 of warps 0..3) issue the MMAs of a phase; the instruction
// stream around each tcgen05.mma is kept to two integer adds: the descriptors' high words are the
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

// Issue with the accumulate flag in a register, and the one shared copy of the issue loop that a
// kernel with rolled loops (TTT_MMA_ROLLED 1) calls for every product: n MMAs whose operand
// descriptors advance by a constant per K step; the first one overwrites D unless `acc` is set.
// A tcgen05.mma costs about ten instructions of set-up, so one out-of-line loop instead of one per
// product shrinks such a kernel by roughly a tenth; only the issuing threads ever run it.
__device__ __forceinline__ void mma_issue_rt(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %4};\n\t"
      "mov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kDescHi), "r"(accumulate)
      : "memory");
}
static __device__ __noinline__ void mma_run(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                            uint32_t n, uint32_t astep, uint32_t bstep, uint32_t acc) {
  // n is a multiple of 4 at every call
#pragma unroll 1
  for (uint32_t j = 0; j < n; j += 4) {
    mma_issue_rt(tmem_d, a_lo, b_lo, idesc, acc | j);
    mma_issue_rt(tmem_d, a_lo + astep, b_lo + bstep, idesc, 1u);
    mma_issue_rt(tmem_d, a_lo + 2 * astep, b_lo + 2 * bstep, idesc, 1u);
    mma_issue_rt(tmem_d, a_lo + 3 * astep, b_lo + 3 * bstep, idesc, 1u);
    a_lo += 4 * astep;
    b_lo += 4 * bstep;
  }
}

// "Hidden-major" product: D[256 x 64] (two M=128 blocks, 64 fp32 columns each, at tmem_d and
// tmem_d + 64) (+)= A * B with A a [256][64] bf16 tile read K-major (row = hidden unit) and B a
// [64][64] tile read K-major (row = N index) or MN-major (row = K index).
// One M = 128 block (`blk` = 0 or 1: hidden units 128 blk .. 128 blk + 127) of the product.  The two
// blocks are independent, so two threads may issue one each.
template <bool kBMn, bool kAccumulate>
__device__ __forceinline__ void mma_hidden_half_t(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem, int blk) {
  constexpr uint32_t idesc = umma_idesc_bf16(128, 64, false, kBMn, false);
  const uint32_t a0 = desc_lo(a_smem, 16) + blk * (16384u >> 4);
  const uint32_t b0 = desc_lo(b_smem, kBMn ? 8192 : 16);
  constexpr uint32_t bstep = kBMn ? (2048u >> 4) : (32u >> 4);
  const uint32_t d = tmem_d + blk * 64;
#if TTT_MMA_SHARED_LOOP
  mma_run(d, a0, b0, idesc, 4, 2, bstep, kAccumulate ? 1u : 0u);
#else
  if (kAccumulate) mma_issue<true>(d, a0, b0, idesc);
  else             mma_issue<false>(d, a0, b0, idesc);
TTT_MMA_LOOP
  for (int j = 1; j < 4; ++j) mma_issue<true>(d, a0 + j * 2, b0 + j * bstep, idesc);
#endif
}
template <bool kBMn, bool kAccumulate>
__device__ __forceinline__ void mma_hidden_major_t(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem) {
TTT_MMA_OUTER
  for (int blk = 0; blk < 2; ++blk) mma_hidden_half_t<kBMn, kAccumulate>(tmem_d, a_smem, b_smem, blk);
}
__device__ __forceinline__ void mma_hidden_half(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem, bool b_mn,
                                                bool accumulate, int blk) {
  if (b_mn) {
    if (accumulate) mma_hidden_half_t<true, true>(tmem_d, a_smem, b_smem, blk);
    else            mma_hidden_half_t<true, false>(tmem_d, a_smem, b_smem, blk);
  } else {
    if (accumulate) mma_hidden_half_t<false, true>(tmem_d, a_smem, b_smem, blk);
    else            mma_hidden_half_t<false, false>(tmem_d, a_smem, b_smem, blk);
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
#if TTT_MMA_SHARED_LOOP
  mma_run(tmem_d, a0, b0, idesc, 16, 2048u >> 4, 2048u >> 4, 0u);
#else
  mma_issue<false>(tmem_d, a0, b0, idesc);
TTT_MMA_LOOP
  for (int j = 1; j < 16; ++j) mma_issue<true>(tmem_d, a0 + j * (2048u >> 4), b0 + j * (2048u >> 4), idesc);
#endif
}

// ---- A warp's 32 rows x 32 fp32 columns (lane = row, v = the row's 32 values) -> a row-major global
// matrix with `ld` floats per row, as whole 128-byte lines: written straight from the registers the
// 16-byte stores of a warp would land in 32 different lines (measured: the fp32 W2 checkpoint written
// that way cost 4 % of the forward), so the block is turned through a warp-private staging area
// (32 rows x 144 bytes of shared memory; the 16-byte pad keeps both directions conflict-free).
// `dst` points at the block's first element (row of lane 0, first of the 32 columns).  The caller makes
// sure that no other warp writes the bytes of this warp's staging area while the call runs.
__device__ __forceinline__ void store_rows_coalesced(float* dst, int ld, const uint32_t (&v)[32], uint8_t* stage,
                                                     int lane) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(stage + lane * 144 + c * 16) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = 4 * i + (lane >> 3), ch = lane & 7;
    const uint4 w = *reinterpret_cast<const uint4*>(stage + r * 144 + ch * 16);
    *reinterpret_cast<uint4*>(dst + static_cast<long>(r) * ld + ch * 4) = w;
  }
  __syncwarp();
}
constexpr uint32_t kRowStageBytes = 32 * 144;     // per warp

// ---- Token-major 64 x 64 accumulators spread over 8 warps (256 threads).
// A token-major accumulator (M = 64) keeps row r in TMEM lane (r % 16) + 32 * (r / 16): quadrant q
// holds rows 16q .. 16q+15 in its first 16 lanes.  The two warps that may touch quadrant q (q and
// q + 4) each take 32 of the 64 columns with one 16x256b.x4 load, so every thread owns 16 values:
//   rows r0 = 16q + lane/4 and r1 = r0 + 8;  for j = 0..3 the column pair c = 32*colhalf + 8j + 2(lane%4):
//   v[4j], v[4j+1] = (r0, c), (r0, c+1);   v[4j+2], v[4j+3] = (r1, c), (r1, c+1).
// A row is shared by 8 threads: the 4 lanes of a quad in each of the two warps; row sums go through
// two shuffles and one exchange in shared memory between the warp pair (named barrier 1 + q).
struct TokMap {
  int quad, colhalf, l3;
  int r0, r1;
  uint32_t taddr;      // lane/column offset to add to the accumulator's TMEM address
  __device__ __forceinline__ TokMap(int warp, int lane)
      : quad(warp & 3), colhalf(warp >> 2), l3(lane & 3), r0((warp & 3) * 16 + (lane >> 2)),
        r1((warp & 3) * 16 + (lane >> 2) + 8),
        taddr((static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>((warp >> 2) * 32)) {}
  __device__ __forceinline__ int col(int j) const { return colhalf * 32 + j * 8 + l3 * 2; }
  // byte offset of the column pair j of row r inside a swizzled [64][64] bf16 tile
  __device__ __forceinline__ uint32_t off(int r, int j) const { return sw128_off(r, colhalf * 4 + j) + l3 * 4; }
};
// three accumulators with one wait (the loads overlap)
__device__ __forceinline__ void tok_ld3(const TokMap& m, uint32_t acc_a, float (&a)[16], uint32_t acc_b,
                                        float (&b)[16], uint32_t acc_c, float (&c)[16]) {
  uint32_t ua[16], ub[16], uc[16];
  tmem_ld_16x256b_x4(acc_a + m.taddr, ua);
  tmem_ld_16x256b_x4(acc_b + m.taddr, ub);
  tmem_ld_16x256b_x4(acc_c + m.taddr, uc);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    a[i] = __uint_as_float(ua[i]);
    b[i] = __uint_as_float(ub[i]);
    c[i] = __uint_as_float(uc[i]);
  }
}
__device__ __forceinline__ void tok_ld(const TokMap& m, uint32_t tmem_acc, float (&v)[16]) {
  uint32_t u[16];
  tmem_ld_16x256b_x4(tmem_acc + m.taddr, u);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(u[i]);
}
// the thread's 16 values of a swizzled bf16 tile, same order as the accumulator fragment
__device__ __forceinline__ void tok_ld_tile(const TokMap& m, const uint8_t* tile, float (&v)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(tile + m.off(m.r0, j));
    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(tile + m.off(m.r1, j));
    v[4 * j] = bf16_lo(w0); v[4 * j + 1] = bf16_hi(w0);
    v[4 * j + 2] = bf16_lo(w1); v[4 * j + 3] = bf16_hi(w1);
  }
}
__device__ __forceinline__ void tok_st_tile(const TokMap& m, uint8_t* tile, const float (&v)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    *reinterpret_cast<uint32_t*>(tile + m.off(m.r0, j)) = pack_bf16(v[4 * j], v[4 * j + 1]);
    *reinterpret_cast<uint32_t*>(tile + m.off(m.r1, j)) = pack_bf16(v[4 * j + 2], v[4 * j + 3]);
  }
}
// per-column vector (fp32[64] in shared memory) -> the thread's 8 columns: c[2j], c[2j+1]
__device__ __forceinline__ void tok_ld_cols(const TokMap& m, const float* vec, float (&c)[8]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = *reinterpret_cast<const float2*>(vec + m.col(j));
    c[2 * j] = f.x; c[2 * j + 1] = f.y;
  }
}
// All-reduce N per-row partial sums over the 8 threads that share each row.  a[] belongs to row
// r0, b[] to row r1.  xch: fp32[2][64][8] in shared memory; the call uses columns kSlot .. kSlot+N-1
// of it.  There is no barrier after the read-back: the all-reduces of one epilogue phase must use
// disjoint columns, and a CTA barrier must separate phases (every phase ends with one).
template <int N, int kSlot>
__device__ __forceinline__ void tok_row_allreduce(const TokMap& m, float (&a)[N], float (&b)[N], float* xch) {
  static_assert(kSlot >= 0 && kSlot + N <= 8, "the exchange buffer has 8 columns per row");
#pragma unroll
  for (int i = 0; i < N; ++i) {
    a[i] += __shfl_xor_sync(0xffffffffu, a[i], 1);
    b[i] += __shfl_xor_sync(0xffffffffu, b[i], 1);
    a[i] += __shfl_xor_sync(0xffffffffu, a[i], 2);
    b[i] += __shfl_xor_sync(0xffffffffu, b[i], 2);
  }
  if (m.l3 == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      xch[(m.colhalf * 64 + m.r0) * 8 + kSlot + i] = a[i];
      xch[(m.colhalf * 64 + m.r1) * 8 + kSlot + i] = b[i];
    }
  }
  named_bar_sync(1 + m.quad, 64);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    a[i] += xch[((m.colhalf ^ 1) * 64 + m.r0) * 8 + kSlot + i];
    b[i] += xch[((m.colhalf ^ 1) * 64 + m.r1) * 8 + kSlot + i];
  }
}
// LayerNorm statistics of the thread's two rows: centres z in place, returns 1/std per row.  Uses the
// exchange columns 0 and 1.
__device__ __forceinline__ void tok_layernorm(const TokMap& m, float (&z)[16], float eps, float* xch, float& rstd0,
                                              float& rstd1) {
  float s0[1] = {0.f}, s1[1] = {0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s0[0] += z[4 * j] + z[4 * j + 1];
    s1[0] += z[4 * j + 2] + z[4 * j + 3];
  }
  tok_row_allreduce<1, 0>(m, s0, s1, xch);
  const float mu0 = s0[0] * (1.f / 64.f), mu1 = s1[0] * (1.f / 64.f);
  s0[0] = 0.f; s1[0] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    z[4 * j] -= mu0; z[4 * j + 1] -= mu0;
    z[4 * j + 2] -= mu1; z[4 * j + 3] -= mu1;
    s0[0] = fmaf(z[4 * j], z[4 * j], fmaf(z[4 * j + 1], z[4 * j + 1], s0[0]));
    s1[0] = fmaf(z[4 * j + 2], z[4 * j + 2], fmaf(z[4 * j + 3], z[4 * j + 3], s1[0]));
  }
  tok_row_allreduce<1, 1>(m, s0, s1, xch);
  rstd0 = rsqrtf(s0[0] * (1.f / 64.f) + eps);
  rstd1 = rsqrtf(s1[0] * (1.f / 64.f) + eps);
}

}  // namespace tttdev
