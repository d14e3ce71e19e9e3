// TTT-Linear backward for sm_100a: gradients of the TTT-Linear forward (ttt_linear_fwd_sm100.cu) from its
// checkpoints, one persistent CTA of 256 threads per (batch, head) stream.
//
// The reference has no counterpart (it ships the TTT-MLP operator only, README.md:18); the structure is its
// backward's (kernels/ttt_backward/ttt.cu:453-1424, math kernels/ttt_backward/matching.py:173-342) with the
// hidden layer removed: per checkpoint group, last to first, recompute the group's mini-batches from the
// checkpoint, keeping what the reverse sweep needs in the caller's scratch buffer, then sweep the group in
// reverse.  Every tile is 64 x 64: token-major tiles and the 64 x 64 state alike are M = 64 accumulators read
// with the 16x256b fragments of TokMap by all eight warps.  The state W^T and the gradient state
// G^T = (dL/dW)^T live side by side in tensor memory as the accumulators of their own update MMAs (the MLP
// kernel has to park one of them: here both fit), b and dL/db in shared memory.
//
// Recompute of mini-batch j (3 MMA phases, the forward's):
//   Z = K W;  x_f = LN(Z + b), e = gamma x_f + beta - (V - K), gZ = LNbwd(e gamma), U = -eta gZ;
//   W^T += U^T K, b += colsum U;  Zb = Q W+;  x_ln = LN(Zb + b+)
//   slot j of the scratch buffer <- bf16 W^T before the update, x_f, gZ, x_ln (raw images of the swizzled
//   shared-memory tiles, stored and read back with bulk copies), 1/std of both LayerNorms.
// Reverse step of mini-batch j (3 MMA phases), with go = dL/dOut and the state after j's update W+ = the
// pre-update state of j + 1 (or the group's last state):
//   S4   gZb = LNbwd(go gamma; x_ln);  d_beta += colsum go;  d_gamma += colsum go x_ln;  G_b += colsum gZb
//   A    dQ = go + gZb W+^T;  G^T += gZb^T Q
//   B    A1 = -eta (K G + G_b);  T1 = gZ G^T;  d_eta = -rowsum(T1 K) - rowsum(G_b gZ)
//   E4   second order through the fused LayerNorm + L2 gradient: Bt, d_gamma, d_beta, dV = -gamma Bt,
//        gZin (the formulas of the MLP kernel's E4 with A1 in the place of A2 and gZ in the place of dl/dZ2)
//   C    dK = gamma Bt - eta T1 + gZin W^T;  G^T += gZin^T K;  G_b += colsum gZin
// All waits are bounded; on expiry the CTA reports through the status word, drains its own copies, frees its
// tensor memory and returns.
#include <cstdlib>
#include <mutex>

#include "ttt_cluster.cuh"
#include "ttt_internal.h"

using namespace tttcl;

namespace {

constexpr int kThreads = 256;
constexpr int kProd = 128;     // issues the bulk copies; not the MMA issuer (lane 0 of warp 0)

// scratch slot (one per mini-batch of a checkpoint group and stream)
constexpr uint32_t SL_W = 0;
constexpr uint32_t SL_XF = TILE;
constexpr uint32_t SL_GZ = 2 * TILE;
constexpr uint32_t SL_XL = 3 * TILE;
constexpr uint32_t SL_SIG = 4 * TILE;          // fp32[64] 1/std of the fused LayerNorm, fp32[64] of the output one
constexpr uint32_t SLOT_BYTES = 4 * TILE + 512;

// Shared memory.  kStages = 2: every per-mini-batch tile has two stages, the next mini-batch's loads are issued a
// whole step ahead, one CTA per SM (for launches with no more streams than SMs, where nothing else could hide
// the load latency).  kStages = 1: single tiles, loads issued when the step before has ended, half the shared
// memory and a 128-register budget: two CTAs per SM, which hide each other's latencies (for launches with more
// streams than SMs).  Tiles that are never live at the same time share their place: the bf16 copy of G^T with the
// state copy W^T (read as the post-update state by the first reverse step only, before G^T is first copied), gZin
// with gZb / U, the d_gamma addends with dL/dOut.
template <int kStages>
struct Lay {
  static constexpr uint32_t OFF_K = 0;
  static constexpr uint32_t OFF_Q = OFF_K + kStages * TILE;
  static constexpr uint32_t OFF_V = OFF_Q + kStages * TILE;
  static constexpr uint32_t OFF_GO = OFF_V + kStages * TILE;
  static constexpr uint32_t OFF_XL = OFF_GO + kStages * TILE;
  static constexpr uint32_t OFF_XF = OFF_XL + kStages * TILE;
  static constexpr uint32_t OFF_GZ = OFF_XF + kStages * TILE;
  static constexpr uint32_t OFF_WP = OFF_GZ + kStages * TILE;   // pre-update W^T of the sweep's mini-batch (always two)
  static constexpr uint32_t OFF_W = OFF_WP + 2 * TILE;          // bf16 operand copy of the current state W^T / of G^T
  static constexpr uint32_t OFF_A = OFF_W + TILE;               // U (recompute) / gZb, then gZin (sweep)
  static constexpr uint32_t OFF_ETA = OFF_A + TILE;             // bf16[kStages][64]
  static constexpr uint32_t OFF_SIG = OFF_ETA + 256;            // fp32[kStages][128]: both 1/std vectors of the sweep's mini-batch
  static constexpr uint32_t OFF_B = OFF_SIG + 1024;
  static constexpr uint32_t OFF_GB = OFF_B + 256;
  static constexpr uint32_t OFF_GAMMA = OFF_GB + 256;
  static constexpr uint32_t OFF_BETA = OFF_GAMMA + 256;
  static constexpr uint32_t OFF_DG = OFF_BETA + 256;
  static constexpr uint32_t OFF_DB = OFF_DG + 256;
  static constexpr uint32_t OFF_PART = OFF_DB + 256;            // fp32[3][4][64] column-sum partials
  static constexpr uint32_t OFF_BAR = OFF_PART + 3072;
  static constexpr uint32_t OFF_MISC = OFF_BAR + 64;
  static constexpr uint32_t OFF_XCH = OFF_MISC + 64;            // fp32[2][64][8] row-sum exchange between warp pairs
  static constexpr uint32_t OFF_ONES = (OFF_XCH + 4096 + 1023) & ~1023u;   // bf16[8][64] ones: B operand of the column sums
  static constexpr uint32_t SMEM_USED = OFF_ONES + 1024;
  static constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;
  static constexpr int kCtasPerSm = kStages == 1 ? 2 : 1;
  static_assert(kCtasPerSm * (SMEM_BYTES + 1024) <= 233472, "exceeds the shared memory of an SM of sm_100");
};

constexpr int BAR_IN = 0;      // +stage: K, Q, V, eta (and dL/dOut in the sweep)
constexpr int BAR_SC = 2;      // +stage: scratch tiles of the sweep
constexpr int BAR_MMA = 4;
constexpr int BAR_DRAIN = 5;
constexpr int NUM_BARS = 6;

constexpr uint32_t TM_W = 0;
constexpr uint32_t TM_G = 64;
constexpr uint32_t TM_A = 128;
constexpr uint32_t TM_B = 192;
constexpr uint32_t TM_COLS = 256;

struct LinBwdParams {
  const __nv_bfloat16* eta;
  const float* gamma;
  const float* beta;
  const float* Wc;
  const float* bc;
  const float* gW_last;
  const float* gb_last;
  uint8_t* scratch;
  float* d_gamma;
  float* d_beta;
  float* gW;
  float* gb;
  __nv_bfloat16* d_eta;
  __nv_bfloat16* dXQ;
  __nv_bfloat16* dXK;
  __nv_bfloat16* dXV;
  int H, NC, cgs, nck;
  int drop_load;            // test only: mini-batch whose recompute inputs stream 0 never loads (-1: none)
  uint32_t* status;
  uint64_t wait_limit_ns;
};

// D[64 x 64] += A^T B with both operands [64 k][64] tiles read MN-major (row = contraction index)
__device__ __forceinline__ void mma_mn_accumulate(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem) {
  constexpr uint32_t idesc = umma_idesc_bf16(64, 64, true, true, false);
  const uint32_t a0 = desc_lo(a_smem, TILE);
  const uint32_t b0 = desc_lo(b_smem, TILE);
#pragma unroll
  for (int j = 0; j < 4; ++j) mma_issue_rt(tmem_d, a0 + j * (2048u >> 4), b0 + j * (2048u >> 4), idesc, 1u);
}

template <int kStages>
__global__ void __launch_bounds__(kThreads, Lay<kStages>::kCtasPerSm)
ttt_linear_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmGo,
                      const LinBwdParams p) {
  using L = Lay<kStages>;
  constexpr uint32_t OFF_K = L::OFF_K, OFF_Q = L::OFF_Q, OFF_V = L::OFF_V, OFF_GO = L::OFF_GO, OFF_XL = L::OFF_XL,
                     OFF_XF = L::OFF_XF, OFF_GZ = L::OFF_GZ, OFF_WP = L::OFF_WP, OFF_W = L::OFF_W, OFF_A = L::OFF_A,
                     OFF_ETA = L::OFF_ETA, OFF_SIG = L::OFF_SIG, OFF_B = L::OFF_B, OFF_GB = L::OFF_GB,
                     OFF_GAMMA = L::OFF_GAMMA, OFF_BETA = L::OFF_BETA, OFF_DG = L::OFF_DG, OFF_DB = L::OFF_DB,
                     OFF_PART = L::OFF_PART, OFF_BAR = L::OFF_BAR, OFF_MISC = L::OFF_MISC, OFF_XCH = L::OFF_XCH;
  constexpr int kSt = kStages - 1;            // stage of mini-batch j: j & kSt
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const TokMap tm(warp, lane);
  const long sid = blockIdx.x;
  const int head = static_cast<int>(sid % p.H);
  const int NC = p.NC, cgs = p.cgs;
  const bool row_writer = tm.colhalf == 0 && tm.l3 == 0;   // of the 8 threads that share a row, the one that stores per-row values

  auto tK = [&](int s) { return smem + OFF_K + s * TILE; };
  auto tQ = [&](int s) { return smem + OFF_Q + s * TILE; };
  auto tV = [&](int s) { return smem + OFF_V + s * TILE; };
  auto tGo = [&](int s) { return smem + OFF_GO + s * TILE; };
  auto tXL = [&](int s) { return smem + OFF_XL + s * TILE; };
  auto tXF = [&](int s) { return smem + OFF_XF + s * TILE; };
  auto tGZ = [&](int s) { return smem + OFF_GZ + s * TILE; };
  auto tWP = [&](int s) { return smem + OFF_WP + s * TILE; };
  uint8_t* sW = smem + OFF_W;
  uint8_t* sA = smem + OFF_A;
  uint8_t* sG = sW;        // see Lay
  uint8_t* sZin = sA;
  __nv_bfloat16* sEta = reinterpret_cast<__nv_bfloat16*>(smem + OFF_ETA);
  float* sSig = reinterpret_cast<float*>(smem + OFF_SIG);
  float* sB = reinterpret_cast<float*>(smem + OFF_B);
  float* sGb = reinterpret_cast<float*>(smem + OFF_GB);
  float* sGamma = reinterpret_cast<float*>(smem + OFF_GAMMA);
  float* sBeta = reinterpret_cast<float*>(smem + OFF_BETA);
  float* sDG = reinterpret_cast<float*>(smem + OFF_DG);
  float* sDB = reinterpret_cast<float*>(smem + OFF_DB);
  float* part = reinterpret_cast<float*>(smem + OFF_PART);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  float* sXch = reinterpret_cast<float*>(smem + OFF_XCH);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 4);
  volatile uint32_t* never_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 8);   // stays 0
  const uint64_t limit = p.wait_limit_ns;

  if (tid == kProd) {
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
    *abort_flag = 0;
    *never_flag = 0;
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmGo);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  if (tid < 64) {
    sGamma[tid] = p.gamma[head * 64 + tid];
    sBeta[tid] = p.beta[head * 64 + tid];
    sGb[tid] = p.gb_last[sid * 64 + tid];
    sDG[tid] = 0.f;
    sDB[tid] = 0.f;
  }
  reinterpret_cast<uint32_t*>(smem + L::OFF_ONES)[tid] = 0x3F803F80u;     // 256 x two bf16 ones
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t sOnes = smem_u32(smem + L::OFF_ONES);
  // Column sums over the tokens of a bf16 tile are taken by the tensor pipe (mma_colsum: the MMA windows of
  // these 64 x 64 products are too short to hide a pass over the tile by the warps), into accumulator columns
  // that are free in that phase; warps 0..3 read them back after the phase (16 sums per warp).
  auto add_colsum = [&](float* vec, uint32_t tm_cols, float sign) {
    if (warp < 4) {
      const float cs = colsum_read(tmem + tm_cols, warp);
      if (lane < 16) vec[16 * warp + lane] += sign * cs;
    }
  };

  // ---- barrier bookkeeping: every thread waits on every barrier use, in program order
  uint32_t ph = 0;        // expected parity per barrier
  uint32_t pending = 0;   // kProd: loads issued and not yet waited for
  auto wait_bar = [&](int b) {
    if (mbar_wait_bounded(&bars[b], (ph >> b) & 1u, abort_flag, limit)) {
      ph ^= 1u << b;
      pending &= ~(1u << b);
    }
  };
  auto wait_mma = [&]() {
    wait_bar(BAR_MMA);
    __syncwarp();
    tc_fence_after_sync();
  };
  auto publish = [&]() {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
  };
  auto publish_vote = [&]() -> bool {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    return __syncthreads_or(*abort_flag != 0) != 0;
  };
#define TTT_ISSUE1(WORK)            \
  if (warp == 0) {                  \
    if (elect_one()) {              \
      tc_fence_after_sync();        \
      WORK;                         \
      umma_commit(&bars[BAR_MMA]);  \
    }                               \
    __syncwarp();                   \
  }

  const int cs_q = tid >> 6, cs_f = tid & 63;
  auto colsum16 = [&](const uint8_t* t) {
    float acc = 0.f;
#pragma unroll 8
    for (int r = cs_q * 16; r < cs_q * 16 + 16; ++r) acc += ld_elem(t, r, cs_f);
    return acc;
  };
  auto part_sum = [&](int k) {
    return (part[k * 256 + tid] + part[k * 256 + 64 + tid]) + (part[k * 256 + 128 + tid] + part[k * 256 + 192 + tid]);
  };

  // ---- state <-> global memory.  W-shaped matrices are [64 in][64 out] in global memory; the fragment of the
  // transposed matrix holds output features r0 / r1 (rows) and the input-feature pairs col(j), col(j) + 1.
  auto load_frag = [&](const float* Wg, float (&w)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      w[4 * j] = Wg[c * 64 + tm.r0];
      w[4 * j + 1] = Wg[(c + 1) * 64 + tm.r0];
      w[4 * j + 2] = Wg[c * 64 + tm.r1];
      w[4 * j + 3] = Wg[(c + 1) * 64 + tm.r1];
    }
  };
  {   // the gradient state starts as dL/d(final state)
    float w[16];
    load_frag(p.gW_last + sid * 4096, w);
    tok_st_tmem(tm, tmem + TM_G, w);
    tmem_wait_st();
  }

  const long tok_rows0 = sid * NC * 64;
  bool aborted = false;

  for (int ck = p.nck - 1; ck >= 0 && !aborted; --ck) {
    const int i0 = ck * cgs;
    const int gsz = min(cgs, NC - i0);
    uint8_t* slots = p.scratch + sid * cgs * static_cast<long>(SLOT_BYTES);

    auto issue_inputs = [&](int j, bool with_go) {   // kProd
      if (!with_go && i0 + j == p.drop_load && sid == 0) return;
      const int s = j & kSt;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      mbar_expect_tx(&bars[BAR_IN + s], (with_go ? 4 : 3) * TILE + 128);
      tma_load_2d(tK(s), &tmK, &bars[BAR_IN + s], 0, row0);
      tma_load_2d(tQ(s), &tmQ, &bars[BAR_IN + s], 0, row0);
      tma_load_2d(tV(s), &tmV, &bars[BAR_IN + s], 0, row0);
      if (with_go) tma_load_2d(tGo(s), &tmGo, &bars[BAR_IN + s], 0, row0);
      bulk_load_1d(sEta + s * 64, p.eta + (sid * NC + i0 + j) * 64, 128, &bars[BAR_IN + s]);
      pending |= 1u << (BAR_IN + s);
    };
    // The barrier is armed with all the bytes of the slot; the pre-update state copy follows separately
    // (issue_wp) when its tile, which holds the post-update state of the step before, is free.
    auto issue_wp = [&](int j) {                     // kProd
      bulk_load_1d(tWP(j & 1), slots + static_cast<long>(j) * SLOT_BYTES + SL_W, TILE, &bars[BAR_SC + (j & kSt)]);
    };
    auto issue_scratch = [&](int j) {                // kProd
      const int s = j & kSt;
      const uint8_t* sl = slots + static_cast<long>(j) * SLOT_BYTES;
      mbar_expect_tx(&bars[BAR_SC + s], 4 * TILE + 512);
      bulk_load_1d(tXF(s), sl + SL_XF, TILE, &bars[BAR_SC + s]);
      bulk_load_1d(tGZ(s), sl + SL_GZ, TILE, &bars[BAR_SC + s]);
      bulk_load_1d(tXL(s), sl + SL_XL, TILE, &bars[BAR_SC + s]);
      bulk_load_1d(sSig + s * 128, sl + SL_SIG, 512, &bars[BAR_SC + s]);
      pending |= 1u << (BAR_SC + s);
    };
    if (tid == kProd) {
      issue_inputs(0, false);
      if (kStages == 2 && gsz > 1) issue_inputs(1, false);
    }
    // ---- checkpoint -> tensor memory (fp32) + shared memory (bf16)
    {
      float w[16];
      load_frag(p.Wc + (sid * p.nck + ck) * 4096, w);
      tok_st_tmem(tm, tmem + TM_W, w);
      tok_st_tile(tm, sW, w);
      tmem_wait_st();
      if (tid < 64) sB[tid] = p.bc[(sid * p.nck + ck) * 64 + tid];
    }
    publish();

    // ================================================================== recompute the group
    for (int j = 0; j < gsz; ++j) {
      const int s = j & kSt;
      uint8_t* sl = slots + static_cast<long>(j) * SLOT_BYTES;
      float* sig = reinterpret_cast<float*>(sl + SL_SIG);
      const __nv_bfloat16* eta = sEta + s * 64;
      wait_bar(BAR_IN + s);

      // MMA1: Z = K W
      TTT_ISSUE1(mma_hid64<false>(tmem + TM_A, smem_u32(tK(s)), smem_u32(sW), 0u))
      wait_mma();
      {
        float xh[16], bc[8], gam[8], bet[8];
        tok_ld(tm, tmem + TM_A, xh);
        tok_ld_cols(tm, sB, bc);
        tok_ld_cols(tm, sGamma, gam);
        tok_ld_cols(tm, sBeta, bet);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          xh[4 * q] += bc[2 * q]; xh[4 * q + 1] += bc[2 * q + 1];
          xh[4 * q + 2] += bc[2 * q]; xh[4 * q + 3] += bc[2 * q + 1];
        }
        float rs0, rs1;
        float kk[16], vv[16], g[16];
        tok_ld_tile(tm, tK(s), kk);
        tok_ld_tile(tm, tV(s), vv);
        tok_layernorm(tm, xh, TTT_LN_EPS, sXch, rs0, rs1);
        float a[2] = {0.f, 0.f}, b[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h, c = 2 * q + h;
            xh[x0] *= rs0;
            xh[x1] *= rs1;
            g[x0] = (fmaf(gam[c], xh[x0], bet[c]) - (vv[x0] - kk[x0])) * gam[c];
            g[x1] = (fmaf(gam[c], xh[x1], bet[c]) - (vv[x1] - kk[x1])) * gam[c];
            a[0] += g[x0]; a[1] = fmaf(g[x0], xh[x0], a[1]);
            b[0] += g[x1]; b[1] = fmaf(g[x1], xh[x1], b[1]);
          }
        }
        tok_st_tile(tm, tXF(s), xh);
        tok_row_allreduce<2, 2>(tm, a, b, sXch);
        const float sc0 = rs0 * (1.f / 64.f), sc1 = rs1 * (1.f / 64.f);
        const float ne0 = -__bfloat162float(eta[tm.r0]), ne1 = -__bfloat162float(eta[tm.r1]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            // dl/dZ, rounded to bf16 once: the update below uses -eta times the rounded value
            g[x0] = __bfloat162float(__float2bfloat16((64.f * g[x0] - a[0] - xh[x0] * a[1]) * sc0));
            g[x1] = __bfloat162float(__float2bfloat16((64.f * g[x1] - b[0] - xh[x1] * b[1]) * sc1));
          }
        }
        tok_st_tile(tm, tGZ(s), g);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          g[4 * q] *= ne0; g[4 * q + 1] *= ne0;
          g[4 * q + 2] *= ne1; g[4 * q + 3] *= ne1;
        }
        tok_st_tile(tm, sA, g);
        if (row_writer) {
          sig[tm.r0] = rs0;
          sig[tm.r1] = rs1;
        }
      }
      publish();
      if (tid == kProd) {   // the pre-update state and the fused-LayerNorm tiles of this mini-batch leave for its slot
        bulk_store_1d(sl + SL_W, sW, TILE);
        bulk_store_1d(sl + SL_XF, tXF(s), TILE);
        bulk_store_1d(sl + SL_GZ, tGZ(s), TILE);
        tma_commit_group();
      }

      // MMA2: W^T += U^T K;  b += column sums of U
      TTT_ISSUE1(mma_mn_accumulate(tmem + TM_W, smem_u32(sA), smem_u32(tK(s)));
                 mma_colsum(tmem + TM_B, smem_u32(sA), sOnes))
      if (tid == kProd) tma_wait_group_read<0>();   // the state copy has left shared memory: the refresh below may overwrite it
      __syncthreads();
      wait_mma();
      add_colsum(sB, TM_B, 1.f);
      {
        float w[16];
        tok_ld(tm, tmem + TM_W, w);
        tok_st_tile(tm, sW, w);
      }
      publish();

      // MMA3: Zb = Q W+;  output LayerNorm statistics
      TTT_ISSUE1(mma_hid64<false>(tmem + TM_A, smem_u32(tQ(s)), smem_u32(sW), 0u))
      wait_mma();
      {
        float z[16], bc[8];
        tok_ld(tm, tmem + TM_A, z);
        tok_ld_cols(tm, sB, bc);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          z[4 * q] += bc[2 * q]; z[4 * q + 1] += bc[2 * q + 1];
          z[4 * q + 2] += bc[2 * q]; z[4 * q + 3] += bc[2 * q + 1];
        }
        float rs0, rs1;
        tok_layernorm(tm, z, TTT_LN_EPS, sXch, rs0, rs1);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          z[4 * q] *= rs0; z[4 * q + 1] *= rs0;
          z[4 * q + 2] *= rs1; z[4 * q + 3] *= rs1;
        }
        tok_st_tile(tm, tXL(s), z);
        if (row_writer) {
          sig[64 + tm.r0] = rs0;
          sig[64 + tm.r1] = rs1;
        }
      }
      aborted = publish_vote();
      if (tid == kProd && !aborted) {
        bulk_store_1d(sl + SL_XL, tXL(s), TILE);
        tma_commit_group();
        if (j + kStages < gsz) issue_inputs(j + kStages, false);   // this stage's K, Q, V have been read by everybody
      }
      if (aborted) break;
    }
    if (aborted) break;

    // ================================================================== reverse sweep
    // scratch was written partly with generic-proxy stores by all threads (the 1/std vectors), partly with bulk
    // stores by one thread: order both before the bulk copies that read it back
    asm volatile("fence.proxy.async;" ::: "memory");
    if (tid == kProd) tma_wait_group<0>();
    publish();
    if (tid == kProd) {
      issue_inputs(gsz - 1, true);
      issue_scratch(gsz - 1);
      issue_wp(gsz - 1);
    }
    for (int j = gsz - 1; j >= 0; --j) {
      const int s = j & kSt;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      uint8_t* sDga = tGo(s);      // see Lay
      // the state after this mini-batch's update: the next mini-batch's pre-update copy, loaded for the previous
      // step, or the group's last state
      const uint8_t* Wpost = (j == gsz - 1) ? sW : tWP((j & 1) ^ 1);
      // two stages: the other stage is free (the previous step has ended), the next step's tiles are requested now
      if (kStages == 2 && tid == kProd && j > 0) {
        issue_inputs(j - 1, true);
        issue_scratch(j - 1);
      }
      wait_bar(BAR_IN + s);
      wait_bar(BAR_SC + s);
      const float* sigf = sSig + s * 128;
      const float* sigl = sigf + 64;
      const __nv_bfloat16* eta = sEta + s * 64;

      // ---- S4: backward of the output LayerNorm
      {
        float go[16], xl[16], gam[8];
        tok_ld_tile(tm, tGo(s), go);
        tok_ld_tile(tm, tXL(s), xl);
        tok_ld_cols(tm, sGamma, gam);
        float a[2] = {0.f, 0.f}, b[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            go[x0] *= gam[2 * q + h];
            go[x1] *= gam[2 * q + h];
            a[0] += go[x0]; a[1] = fmaf(go[x0], xl[x0], a[1]);
            b[0] += go[x1]; b[1] = fmaf(go[x1], xl[x1], b[1]);
          }
        }
        tok_row_allreduce<2, 2>(tm, a, b, sXch);
        const float q0 = sigl[tm.r0] * (1.f / 64.f), q1 = sigl[tm.r1] * (1.f / 64.f);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            go[x0] = (64.f * go[x0] - a[0] - xl[x0] * a[1]) * q0;
            go[x1] = (64.f * go[x1] - b[0] - xl[x1] * b[1]) * q1;
          }
        }
        tok_st_tile(tm, sA, go);
      }
      publish();
      // ---- A: dQ part = gZb W+^T;  G^T += gZb^T Q
      TTT_ISSUE1(mma_hid64<true>(tmem + TM_A, smem_u32(sA), smem_u32(Wpost), 0u);
                 mma_mn_accumulate(tmem + TM_G, smem_u32(sA), smem_u32(tQ(s)));
                 mma_colsum(tmem + TM_B, smem_u32(sA), sOnes);
                 mma_colsum(tmem + TM_B + 8, smem_u32(tGo(s)), sOnes))
      {
        // column sums over the tokens: d_beta += sum go and G_b += sum gZb by the tensor pipe, d_gamma += sum
        // go * x_ln (a product of two tiles) by the warps
        float a = 0.f;
#pragma unroll 8
        for (int r = cs_q * 16; r < cs_q * 16 + 16; ++r) a = fmaf(ld_elem(tGo(s), r, cs_f), ld_elem(tXL(s), r, cs_f), a);
        part[tid] = a;
        __syncthreads();
        if (tid < 64) sDG[tid] += part_sum(0);
      }
      wait_mma();
      add_colsum(sGb, TM_B, 1.f);
      add_colsum(sDB, TM_B + 8, 1.f);
      if (kStages == 2 && tid == kProd && j > 0) issue_wp(j - 1);   // the post-update copy has been read: its tile takes the next step's
      {
        float dq[16], go[16], w[16];
        tok_ld(tm, tmem + TM_A, dq);
        tok_ld_tile(tm, tGo(s), go);
#pragma unroll
        for (int q = 0; q < 16; ++q) go[q] += dq[q];
        tok_st_global(tm, p.dXQ + static_cast<long>(row0) * 64, go);
        tok_ld(tm, tmem + TM_G, w);
        tok_st_tile(tm, sG, w);
      }
      publish();     // also orders the update of G_b before its use below
      // ---- B: A1raw = K G;  T1 = gZ G^T
      TTT_ISSUE1(mma_hid64<false>(tmem + TM_A, smem_u32(tK(s)), smem_u32(sG), 0u);
                 mma_hid64<true>(tmem + TM_B, smem_u32(tGZ(s)), smem_u32(sG), 0u))
      wait_mma();
      float kp[16];        // gamma Bt - eta T1, completed to dK after phase C
      {
        float A[16], t1[16], gz[16], xh[16], go[16], kk[16];
        float gam[8], bet[8], gb[8];
        tok_ld(tm, tmem + TM_A, A);
        tok_ld(tm, tmem + TM_B, t1);
        tok_ld_tile(tm, tGZ(s), gz);
        tok_ld_tile(tm, tXF(s), xh);
        tok_ld_tile(tm, tV(s), go);
        tok_ld_tile(tm, tK(s), kk);
        tok_ld_cols(tm, sGamma, gam);
        tok_ld_cols(tm, sBeta, bet);
        tok_ld_cols(tm, sGb, gb);
        const float eta0 = __bfloat162float(eta[tm.r0]), eta1 = __bfloat162float(eta[tm.r1]);
        const float rs0 = sigf[tm.r0], rs1 = sigf[tm.r1];      // 1 / std
        float ra[5] = {0.f, 0.f, 0.f, 0.f, 0.f}, rb[5] = {0.f, 0.f, 0.f, 0.f, 0.f};   // d_eta terms, (unused), sum A, sum A xh, sum g xh
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h, c = 2 * q + h;
            ra[0] = fmaf(t1[x0], kk[x0], fmaf(gb[c], gz[x0], ra[0]));
            rb[0] = fmaf(t1[x1], kk[x1], fmaf(gb[c], gz[x1], rb[0]));
            kp[x0] = -eta0 * t1[x0];
            kp[x1] = -eta1 * t1[x1];
            A[x0] = -eta0 * (A[x0] + gb[c]);
            A[x1] = -eta1 * (A[x1] + gb[c]);
            // go[] arrives holding V: grad_output_fused = gamma x_hat_fused + beta - (V - K)
            go[x0] = fmaf(gam[c], xh[x0], bet[c]) - (go[x0] - kk[x0]);
            go[x1] = fmaf(gam[c], xh[x1], bet[c]) - (go[x1] - kk[x1]);
            ra[2] += A[x0];
            rb[2] += A[x1];
            ra[3] = fmaf(A[x0], xh[x0], ra[3]);
            rb[3] = fmaf(A[x1], xh[x1], rb[3]);
            ra[4] = fmaf(go[x0] * gam[c], xh[x0], ra[4]);
            rb[4] = fmaf(go[x1] * gam[c], xh[x1], rb[4]);
          }
        }
        tok_row_allreduce<5, 0>(tm, ra, rb, sXch);
        float sa[2] = {0.f, 0.f}, sb[2] = {0.f, 0.f};      // sum g_std, sum g_xhat
        float dga[16], dv[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int c = 2 * q + h;
            const float gm = gam[c];
            {
              const int x = 4 * q + h;
              const float bt = (A[x] - (ra[2] + xh[x] * ra[3]) * (1.f / 64.f)) * rs0;
              const float gly = gm * bt;
              dga[x] = fmaf(go[x], bt, gly * xh[x]);
              dv[x] = -gly;
              kp[x] += gly;
              const float gxh = fmaf(gly, gm, -(go[x] * gm * ra[3] + A[x] * ra[4]) * rs0 * (1.f / 64.f));
              sa[0] += (-gxh * xh[x] - A[x] * gz[x]) * rs0;
              sa[1] += gxh;
              A[x] = gxh;
            }
            {
              const int x = 4 * q + 2 + h;
              const float bt = (A[x] - (rb[2] + xh[x] * rb[3]) * (1.f / 64.f)) * rs1;
              const float gly = gm * bt;
              dga[x] = fmaf(go[x], bt, gly * xh[x]);
              dv[x] = -gly;
              kp[x] += gly;
              const float gxh = fmaf(gly, gm, -(go[x] * gm * rb[3] + A[x] * rb[4]) * rs1 * (1.f / 64.f));
              sb[0] += (-gxh * xh[x] - A[x] * gz[x]) * rs1;
              sb[1] += gxh;
              A[x] = gxh;
            }
          }
        }
        tok_st_tile(tm, sDga, dga);                          // d_gamma addends
        tok_st_tile(tm, tV(s), dv);                          // dV over V: column-summed for d_beta
        tok_st_global(tm, p.dXV + static_cast<long>(row0) * 64, dv);
        tok_row_allreduce<2, 5>(tm, sa, sb, sXch);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            A[x0] = fmaf(A[x0], rs0, (sa[0] * xh[x0] - sa[1] * rs0) * (1.f / 64.f));   // gZin
            A[x1] = fmaf(A[x1], rs1, (sb[0] * xh[x1] - sb[1] * rs1) * (1.f / 64.f));
          }
        }
        tok_st_tile(tm, sZin, A);
        if (row_writer) {
          p.d_eta[(sid * NC + i0 + j) * 64 + tm.r0] = __float2bfloat16(-ra[0]);
          p.d_eta[(sid * NC + i0 + j) * 64 + tm.r1] = __float2bfloat16(-rb[0]);
        }
      }
      publish();
      // ---- C: dK part = gZin W^T;  G^T += gZin^T K
      // (T1 in the second accumulator has been read: its columns take the three column sums of this phase)
      TTT_ISSUE1(mma_hid64<true>(tmem + TM_A, smem_u32(sZin), smem_u32(tWP(j & 1)), 0u);
                 mma_mn_accumulate(tmem + TM_G, smem_u32(sZin), smem_u32(tK(s)));
                 mma_colsum(tmem + TM_B, smem_u32(sZin), sOnes);
                 mma_colsum(tmem + TM_B + 8, smem_u32(sDga), sOnes);
                 mma_colsum(tmem + TM_B + 16, smem_u32(tV(s)), sOnes))
      wait_mma();
      add_colsum(sGb, TM_B, 1.f);
      add_colsum(sDG, TM_B + 8, 1.f);
      add_colsum(sDB, TM_B + 16, -1.f);
      {
        float acc[16];
        tok_ld(tm, tmem + TM_A, acc);
#pragma unroll
        for (int q = 0; q < 16; ++q) kp[q] += acc[q];
        tok_st_global(tm, p.dXK + static_cast<long>(row0) * 64, kp);
      }
      aborted = publish_vote();
      if (aborted) break;
      // one stage: everything of this step has been read, the next step's tiles are requested now
      if (kStages == 1 && tid == kProd && j > 0) {
        issue_inputs(j - 1, true);
        issue_scratch(j - 1);
        issue_wp(j - 1);
      }
    }
  }
#undef TTT_ISSUE1

  // ---- final outputs: dL/d(initial state), norm gradients of this stream
  if (!aborted) {
    float w[16];
    tok_ld(tm, tmem + TM_G, w);
    float* Wo = p.gW + sid * 4096;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      Wo[c * 64 + tm.r0] = w[4 * j];
      Wo[(c + 1) * 64 + tm.r0] = w[4 * j + 1];
      Wo[c * 64 + tm.r1] = w[4 * j + 2];
      Wo[(c + 1) * 64 + tm.r1] = w[4 * j + 3];
    }
    if (tid < 64) {
      p.gb[sid * 64 + tid] = sGb[tid];
      p.d_gamma[sid * 64 + tid] = sDG[tid];
      p.d_beta[sid * 64 + tid] = sDB[tid];
    }
  }
  if (tid == kProd) tma_wait_group<0>();
  if (aborted) {
    // everything this CTA still has in flight is waited for (bounded, not cut short by the abort flag)
    // before its shared and tensor memory go away: the issuer's tensor-core work ...
    if (warp == 0) {
      if (elect_one()) umma_commit(&bars[BAR_DRAIN]);
      __syncwarp();
    }
    if (tid == kProd) {
      mbar_wait_bounded(&bars[BAR_DRAIN], 0, never_flag, limit);
      // ... and its own loads
      for (int b = 0; b < BAR_MMA; ++b)
        if (pending & (1u << b)) mbar_wait_bounded(&bars[b], (ph >> b) & 1u, never_flag, limit);
      atomicExch(p.status, static_cast<uint32_t>(TTT_B200_ERR_TIMEOUT));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace

uint64_t ttt_linear_backward_scratch_bytes(int B, int H, int cgs) {
  return static_cast<uint64_t>(B) * H * cgs * SLOT_BYTES;
}

int ttt_launch_linear_backward(const ttt_b200_linear_bwd_args* a, cudaStream_t stream, uint32_t* status,
                               uint64_t limit_ns, int drop_load) {
  const uint64_t rows = static_cast<uint64_t>(a->B) * a->H * a->NC * 64;
  CUtensorMap tmQ, tmK, tmV, tmGo;
  if (int rc = ttt_make_tile_map(&tmQ, a->XQ, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmK, a->XK, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmV, a->XV, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmGo, a->grad_L_XQW_mini_batch, rows)) return rc;
  LinBwdParams p;
  p.eta = static_cast<const __nv_bfloat16*>(a->last_eta);
  p.gamma = a->ttt_norm_weight;
  p.beta = a->ttt_norm_bias;
  p.Wc = a->W1_checkpoints; p.bc = a->b1_checkpoints;
  p.gW_last = a->grad_L_W1_last; p.gb_last = a->grad_L_b1_last;
  p.scratch = static_cast<uint8_t*>(a->scratch);
  p.d_gamma = a->grad_L_ttt_norm_weight; p.d_beta = a->grad_L_ttt_norm_bias;
  p.gW = a->grad_L_W1_init; p.gb = a->grad_L_b1_init;
  p.d_eta = static_cast<__nv_bfloat16*>(a->grad_L_last_eta);
  p.dXQ = static_cast<__nv_bfloat16*>(a->grad_L_XQ);
  p.dXK = static_cast<__nv_bfloat16*>(a->grad_L_XK);
  p.dXV = static_cast<__nv_bfloat16*>(a->grad_L_XV);
  p.H = a->H; p.NC = a->NC; p.cgs = a->checkpoint_group_size; p.nck = a->num_checkpoints;
  p.drop_load = drop_load;
  p.status = status;
  p.wait_limit_ns = limit_ns;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  static int sms[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ttt_set_error(TTT_B200_ERR_LAUNCH, "device index out of range");
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(ttt_linear_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Lay<1>::SMEM_BYTES);
    if (attr_err[dev] == cudaSuccess)
      attr_err[dev] = cudaFuncSetAttribute(ttt_linear_bwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           Lay<2>::SMEM_BYTES);
    sms[dev] = 148;
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  });
  if (attr_err[dev] != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(attr_err[dev]));
  // more streams than SMs: the form of which two CTAs fit on an SM; else the one that prefetches a step ahead
  // (TTT_B200_LINEAR_BWD_STAGES = 1 or 2 overrides, for measurements)
  static const int forced = [] {
    const char* e = std::getenv("TTT_B200_LINEAR_BWD_STAGES");
    return e ? std::atoi(e) : 0;
  }();
  const int streams = a->B * a->H;
  const bool two_per_sm = forced == 1 || (forced != 2 && streams > sms[dev]);
  if (two_per_sm)
    ttt_linear_bwd_kernel<1><<<dim3(streams), dim3(kThreads), Lay<1>::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmGo, p);
  else
    ttt_linear_bwd_kernel<2><<<dim3(streams), dim3(kThreads), Lay<2>::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmGo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}
