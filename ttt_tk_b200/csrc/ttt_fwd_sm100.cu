// TTT-MLP forward for sm_100a: one persistent CTA per (batch, head) stream.
//
// Replaces the reference's fwd_ttt_mlp_ker (kernels/ttt/ttt.cu:85-586); the per-mini-batch
// math is that of kernels/ttt/matching.py:30-125.
//
// Orientation.  Every 64x256 / 256x64 quantity is kept "hidden-major": the 256 hidden units
// run along the M dimension of the tensor-core tile (= TMEM lanes, = one thread per hidden
// unit in the epilogues) and the 64 tokens or 64 features along N.  The fp32 master state
//   W1^T [256 x 64]  and  W2 [256 x 64]
// lives in tensor memory as the accumulator of its own update MMA; a bf16 copy in shared
// memory, refreshed once per mini-batch, feeds the other MMAs.  b1 lives in registers (one
// hidden unit per thread), b2 in shared memory.
//
// Per mini-batch (K, V, Q: 64x64 bf16 tiles brought in by TMA, eta: 64 bf16):
//   MMA1  Z1^T  = W1^T K^T                    [256 x 64 tok]   (2 x M128, N64, K64)
//   EPI1  X2^T = gelu(Z1^T + b1), G' = gelu'(.)  -> smem bf16
//   MMA2  Z2    = X2 W2                       [64 tok x 64]    (M64, N64, K256)
//   LN    fused LayerNorm + L2-gradient: U2 = -eta * dl/dZ2    -> smem bf16;  b2 += colsum(U2)
//   MMA3  R^T   = W2 U2^T                     [256 x 64 tok]
//   EPI3  U1^T = R^T * G'  (= -eta * dl/dZ1)   -> smem bf16;  b1 += rowsum
//   MMA4  W1^T += U1^T K ;  W2 += X2^T U2     (accumulate into the TMEM state)
//   EPI4  bf16 copies of the new W1^T, W2     -> smem
//   MMA5  Z1b^T = W1^T Q^T ;  EPI5  X2b^T = gelu(. + b1)
//   MMA6  Z2b   = X2b W2   ;  OUT   Out = Q + gamma * LN(Z2b + b2) + beta  -> TMA store
//
// All waits are bounded (see sm100_ptx.cuh); on expiry the CTA reports through the status
// word, drains its own copies, frees its tensor memory and returns.
#include <mutex>

#include "ttt_device.cuh"
#include "ttt_internal.h"

using namespace tttdev;

namespace {

constexpr int kStages = 3;
constexpr int kThreads = 256;
// The thread that issues the bulk copies and waits for their completion is not one of the four MMA issuers
// (lane 0 of warps 0..3): its bookkeeping between a barrier and the next MMA group stays off the issue path.
constexpr int kProd = 128;

constexpr uint32_t OFF_K = 0;
constexpr uint32_t OFF_V = OFF_K + kStages * TILE;
constexpr uint32_t OFF_Q = OFF_V + kStages * TILE;
constexpr uint32_t OFF_OUT = OFF_Q + kStages * TILE;
constexpr uint32_t OFF_W1 = OFF_OUT + TILE;
constexpr uint32_t OFF_W2 = OFF_W1 + BIG;
constexpr uint32_t OFF_X2 = OFF_W2 + BIG;
constexpr uint32_t OFF_GP = OFF_X2 + BIG;
constexpr uint32_t OFF_U2 = OFF_GP + BIG;
constexpr uint32_t OFF_ETA = OFF_U2 + TILE;
constexpr uint32_t OFF_B2 = OFF_ETA + kStages * 128;
constexpr uint32_t OFF_GAMMA = OFF_B2 + 256;
constexpr uint32_t OFF_BETA = OFF_GAMMA + 256;
constexpr uint32_t OFF_BAR = OFF_BETA + 256;
constexpr uint32_t OFF_MISC = OFF_BAR + 64;
constexpr uint32_t OFF_XCH = OFF_MISC + 64;       // fp32[2][64][8] row-sum exchange between warp pairs
constexpr uint32_t SMEM_USED = OFF_XCH + 4096;
constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;  // slack for the 1024-byte alignment
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB per-CTA shared memory of sm_100");

// tensor-memory columns (fp32): two 128-lane blocks of 64 columns per 256-row matrix
constexpr uint32_t TM_W1 = 0;
constexpr uint32_t TM_W2 = 128;
constexpr uint32_t TM_A = 256;
constexpr uint32_t TM_Z = 384;
constexpr uint32_t TM_COLS = 512;

struct FwdParams {
  const __nv_bfloat16* eta;
  const float* gamma;
  const float* beta;
  const float* W1;
  const float* b1;
  const float* W2;
  const float* b2;
  float* W1c;
  float* b1c;
  float* W2c;
  float* b2c;
  float* W1f;
  float* b1f;
  float* W2f;
  float* b2f;
  int H, NC, cgs, nck;
  int drop_load;            // test only: mini-batch whose loads stream 0 never issues (-1: none)
  uint32_t* status;
  uint64_t wait_limit_ns;
};

// The MMAs of one phase are issued by lane 0 of warps 0..3: four instruction streams on four
// schedulers instead of one.  Every issuer commits (an issuer without work too), so the MMA
// barrier counts four arrivals per phase.
#define TTT_ISSUE(W0, W1, W2, W3)   \
  if (warp < 4) {                   \
    if (elect_one()) {              \
      tc_fence_after_sync();        \
      if (warp == 0) { W0; }        \
      else if (warp == 1) { W1; }   \
      else if (warp == 2) { W2; }   \
      else { W3; }                  \
      umma_commit(mma_bar);         \
    }                               \
    __syncwarp();                   \
  }

__global__ void __launch_bounds__(kThreads, 1)
ttt_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmOut,
               const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // same value, known to be warp-uniform
  const int quad = warp & 3, wg = warp >> 2;
  const int hrow = wg * 128 + quad * 32 + lane;          // hidden unit owned in the 256-row epilogues
  const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
  const TokMap tm(warp, lane);                           // fragment of the 64 x 64 token-major tiles
  const long stream_id = blockIdx.x;
  const int head = static_cast<int>(stream_id % p.H);

  uint8_t* sW1 = smem + OFF_W1;
  uint8_t* sW2 = smem + OFF_W2;
  uint8_t* sX2 = smem + OFF_X2;
  uint8_t* sGP = smem + OFF_GP;
  uint8_t* sU2 = smem + OFF_U2;
  uint8_t* sOut = smem + OFF_OUT;
  float* sB2 = reinterpret_cast<float*>(smem + OFF_B2);
  float* sGamma = reinterpret_cast<float*>(smem + OFF_GAMMA);
  float* sBeta = reinterpret_cast<float*>(smem + OFF_BETA);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);   // [kStages]
  uint64_t* mma_bar = full + kStages;
  uint64_t* drain_bar = mma_bar + 1;        // abort path only
  float* sXch = reinterpret_cast<float*>(smem + OFF_XCH);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 4);
  volatile uint32_t* never_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 8);   // stays 0

  const uint64_t limit = p.wait_limit_ns;
  const int NC = p.NC;

  if (tid == kProd) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    mbar_init(mma_bar, 4);
    mbar_init(drain_bar, 4);
    fence_mbar_init();
    *abort_flag = 0;
    *never_flag = 0;
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmOut);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  if (tid < 64) {
    sGamma[tid] = p.gamma[head * 64 + tid];
    sBeta[tid] = p.beta[head * 64 + tid];
    sB2[tid] = p.b2[stream_id * 64 + tid];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  auto issue_loads = [&](int i) {   // thread 0 only
    if (i == p.drop_load && stream_id == 0) return;
    const int s = i % kStages;
    const int row0 = static_cast<int>((stream_id * NC + i) * 64);
    mbar_expect_tx(&full[s], 3 * TILE + 128);
    tma_load_2d(smem + OFF_K + s * TILE, &tmK, &full[s], 0, row0);
    tma_load_2d(smem + OFF_V + s * TILE, &tmV, &full[s], 0, row0);
    tma_load_2d(smem + OFF_Q + s * TILE, &tmQ, &full[s], 0, row0);
    bulk_load_1d(smem + OFF_ETA + s * 128, p.eta + (stream_id * NC + i) * 64, 128, &full[s]);
  };
  int loads_issued = 0;
  if (tid == kProd) {
    for (; loads_issued < kStages && loads_issued < NC; ++loads_issued) issue_loads(loads_issued);
  }

  // ---- initial state: global fp32 -> tensor memory (master) + shared memory (bf16 operand copy)
  float b1v = p.b1[stream_id * 256 + hrow];
  {
    const float* W1g = p.W1 + stream_id * (64 * 256);
    const float* W2g = p.W2 + stream_id * (256 * 64) + hrow * 64;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        f[j] = W1g[(half * 32 + j) * 256 + hrow];
        v[j] = __float_as_uint(f[j]);
      }
      tmem_st32(tmem + lane_base + TM_W1 + wg * 64 + half * 32, v);
#pragma unroll
      for (int c = 0; c < 4; ++c) st_chunk(sW1, hrow, half * 4 + c, f + c * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 q4 = reinterpret_cast<const float4*>(W2g)[half * 8 + j];
        f[j * 4 + 0] = q4.x; f[j * 4 + 1] = q4.y; f[j * 4 + 2] = q4.z; f[j * 4 + 3] = q4.w;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(f[j]);
      tmem_st32(tmem + lane_base + TM_W2 + wg * 64 + half * 32, v);
#pragma unroll
      for (int c = 0; c < 4; ++c) st_chunk(sW2, hrow, half * 4 + c, f + c * 8);
    }
    tmem_wait_st();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  // fp32 state (tensor memory, registers, shared memory) -> global, reference layouts
  // Quarter q of the state: 0, 2 = the two 32-column halves of W1^T; 1, 3 = those of W2.
  auto store_state_quarter = [&](int q, float* W1o, float* W2o) {
    const int half = q >> 1;
    uint32_t v[32];
    __syncwarp();
    if ((q & 1) == 0) {
      tmem_ld32(tmem + lane_base + TM_W1 + wg * 64 + half * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) W1o[(half * 32 + j) * 256 + hrow] = __uint_as_float(v[j]);
    } else {
      // through a staging area in the X2 / G' buffers: only called while those are free (before EPI1
      // writes them: the first MMA window of a mini-batch, or after the last mini-batch)
      tmem_ld32(tmem + lane_base + TM_W2 + wg * 64 + half * 32, v);
      tmem_wait_ld();
      store_rows_coalesced(W2o + (hrow - lane) * 64 + half * 32, 64, v, sX2 + warp * kRowStageBytes, lane);
    }
  };
  auto store_state = [&](float* W1o, float* b1o, float* W2o, float* b2o) {
#pragma unroll 1
    for (int q = 0; q < 4; ++q) store_state_quarter(q, W1o, W2o);
    b1o[hrow] = b1v;
    if (tid < 64) b2o[tid] = sB2[tid];
  };

  uint32_t mma_phase = 0;
  auto wait_mma = [&]() {
    mbar_wait_bounded(mma_bar, mma_phase, abort_flag, limit);
    mma_phase ^= 1;
    __syncwarp();
    tc_fence_after_sync();
  };
  // generic-proxy smem writes + TMEM reads done -> next MMA may be issued
  auto publish = [&]() {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
  };

  int it = 0;
  for (; it < NC; ++it) {
    const int s = it % kStages;
    const uint8_t* sK = smem + OFF_K + s * TILE;
    const uint8_t* sV = smem + OFF_V + s * TILE;
    const uint8_t* sQ = smem + OFF_Q + s * TILE;
    const __nv_bfloat16* sEta = reinterpret_cast<const __nv_bfloat16*>(smem + OFF_ETA + s * 128);

    // A checkpoint (the state before this mini-batch) is written while the first three MMA groups of the
    // mini-batch run: they leave the state columns alone (the update is the fourth), and the stores use
    // neither shared memory nor the tensor pipe.
    const bool ckpt = it % p.cgs == 0;
    const long ckc = stream_id * p.nck + it / p.cgs;
    float* ckW1 = p.W1c + ckc * (64 * 256);
    float* ckW2 = p.W2c + ckc * (256 * 64);
    mbar_wait_bounded(&full[s], (it / kStages) & 1, abort_flag, limit);

    // ---- MMA1: Z1^T = W1^T K^T
    TTT_ISSUE(mma_hidden_half(tmem + TM_A, smem_u32(sW1), smem_u32(sK), false, false, 0),
              mma_hidden_half(tmem + TM_A, smem_u32(sW1), smem_u32(sK), false, false, 1),
              ,
              )
    if (ckpt) {
      store_state_quarter(1, ckW1, ckW2);
      store_state_quarter(3, ckW1, ckW2);
      p.b1c[ckc * 256 + hrow] = b1v;
      if (tid < 64) p.b2c[ckc * 64 + tid] = sB2[tid];     // before this mini-batch's column sums reach b2
      // a warp's staging area reaches into the X2 rows its neighbour writes in EPI1: nobody goes on to EPI1
      // before every warp is done with its area
      __syncthreads();
    }
    wait_mma();
    // ---- EPI1: X2^T = gelu(Z1^T + b1), G' = gelu'(Z1^T + b1)
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      tmem_ld32(tmem + lane_base + TM_A + wg * 64 + half * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float g[8], gp[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) gelu_pair(__uint_as_float(v[c * 8 + k]) + b1v, g[k], gp[k]);
        st_chunk(sX2, hrow, half * 4 + c, g);
        st_chunk(sGP, hrow, half * 4 + c, gp);
      }
    }
    publish();

    // ---- MMA2: Z2 = X2 W2
    TTT_ISSUE(mma_token_major(tmem + TM_Z, smem_u32(sX2), smem_u32(sW2)),
              ,
              ,
              )
    if (ckpt) store_state_quarter(0, ckW1, ckW2);
    wait_mma();
    // ---- LN: fused LayerNorm + L2 gradient, U2 = -eta * dl/dZ2 (all 8 warps, 16 values each)
    {
      float xh[16], b2c[8], gam[8], bet[8];
      tok_ld(tm, tmem + TM_Z, xh);
      tok_ld_cols(tm, sB2, b2c);
      tok_ld_cols(tm, sGamma, gam);
      tok_ld_cols(tm, sBeta, bet);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[4 * j] += b2c[2 * j]; xh[4 * j + 1] += b2c[2 * j + 1];
        xh[4 * j + 2] += b2c[2 * j]; xh[4 * j + 3] += b2c[2 * j + 1];
      }
      float rs0, rs1;
      float kk[16], vv[16], g[16];
      tok_ld_tile(tm, sK, kk);          // requested before the all-reduces of the LayerNorm, used after them
      tok_ld_tile(tm, sV, vv);
      tok_layernorm(tm, xh, TTT_LN_EPS, sXch, rs0, rs1);
      float a[2] = {0.f, 0.f}, b[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i0 = 4 * j + e, i1 = 4 * j + 2 + e, c = 2 * j + e;
          xh[i0] *= rs0;
          xh[i1] *= rs1;
          g[i0] = (fmaf(gam[c], xh[i0], bet[c]) - (vv[i0] - kk[i0])) * gam[c];
          g[i1] = (fmaf(gam[c], xh[i1], bet[c]) - (vv[i1] - kk[i1])) * gam[c];
          a[0] += g[i0]; a[1] = fmaf(g[i0], xh[i0], a[1]);
          b[0] += g[i1]; b[1] = fmaf(g[i1], xh[i1], b[1]);
        }
      }
      tok_row_allreduce<2, 2>(tm, a, b, sXch);
      const float sc0 = -__bfloat162float(sEta[tm.r0]) * rs0 * (1.f / 64.f);
      const float sc1 = -__bfloat162float(sEta[tm.r1]) * rs1 * (1.f / 64.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i0 = 4 * j + e, i1 = 4 * j + 2 + e;
          g[i0] = (64.f * g[i0] - a[0] - xh[i0] * a[1]) * sc0;
          g[i1] = (64.f * g[i1] - b[0] - xh[i1] * b[1]) * sc1;
        }
      }
      tok_st_tile(tm, sU2, g);
    }
    publish();

    // ---- MMA3: R^T = W2 U2^T
    TTT_ISSUE(mma_hidden_half(tmem + TM_A, smem_u32(sW2), smem_u32(sU2), false, false, 0),
              mma_hidden_half(tmem + TM_A, smem_u32(sW2), smem_u32(sU2), false, false, 1),
              ,
              )
    // b2 += column sums of U2 (bf16 values, the operand the W2 update sees), fp32 accumulate: every
    // thread sums 16 rows of one column while the MMA runs, threads 0..63 add the four parts
    {
      const int q = tid >> 6, f = tid & 63;
      float acc = 0.f;
#pragma unroll 8
      for (int t = q * 16; t < q * 16 + 16; ++t) acc += ld_elem(sU2, t, f);
      sXch[tid] = acc;     // the exchange buffer of the token-major epilogues is idle here
      __syncthreads();
      if (tid < 64) sB2[tid] += (sXch[tid] + sXch[64 + tid]) + (sXch[128 + tid] + sXch[192 + tid]);
    }
    if (ckpt) {
      store_state_quarter(2, ckW1, ckW2);
      tc_fence_before_sync();      // the state columns are written by the next MMA group
    }
    wait_mma();
    // ---- EPI3: U1^T = R^T * G' (= -eta dl/dZ1), b1 += row sum
    {
      float bsum = 0.f;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld32(tmem + lane_base + TM_A + wg * 64 + half * 32, v);
        const uint4 gr[4] = {ld_chunk_raw(sGP, hrow, half * 4), ld_chunk_raw(sGP, hrow, half * 4 + 1),
                             ld_chunk_raw(sGP, hrow, half * 4 + 2), ld_chunk_raw(sGP, hrow, half * 4 + 3)};
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float gp[8];
          unpack_chunk(gr[c], gp);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            gp[k] *= __uint_as_float(v[c * 8 + k]);
            bsum += gp[k];
          }
          st_chunk(sGP, hrow, half * 4 + c, gp);
        }
      }
      b1v += bsum;
    }
    publish();

    // ---- MMA4: W1^T += U1^T K ;  W2 += X2^T U2
    TTT_ISSUE(mma_hidden_half(tmem + TM_W1, smem_u32(sGP), smem_u32(sK), true, true, 0),
              mma_hidden_half(tmem + TM_W1, smem_u32(sGP), smem_u32(sK), true, true, 1),
              mma_hidden_half(tmem + TM_W2, smem_u32(sX2), smem_u32(sU2), true, true, 0),
              mma_hidden_half(tmem + TM_W2, smem_u32(sX2), smem_u32(sU2), true, true, 1))
    wait_mma();
    // ---- EPI4: refresh the bf16 operand copies of the state
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      float f[32];
      tmem_ld32(tmem + lane_base + TM_W1 + wg * 64 + half * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
#pragma unroll
      for (int c = 0; c < 4; ++c) st_chunk(sW1, hrow, half * 4 + c, f + c * 8);
      tmem_ld32(tmem + lane_base + TM_W2 + wg * 64 + half * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
#pragma unroll
      for (int c = 0; c < 4; ++c) st_chunk(sW2, hrow, half * 4 + c, f + c * 8);
    }
    publish();

    // ---- MMA5: Z1b^T = W1^T Q^T
    TTT_ISSUE(mma_hidden_half(tmem + TM_A, smem_u32(sW1), smem_u32(sQ), false, false, 0),
              mma_hidden_half(tmem + TM_A, smem_u32(sW1), smem_u32(sQ), false, false, 1),
              ,
              )
    wait_mma();
    // ---- EPI5: X2b^T = gelu(Z1b^T + b1)
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      tmem_ld32(tmem + lane_base + TM_A + wg * 64 + half * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float g[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = gelu_only(__uint_as_float(v[c * 8 + k]) + b1v);
        st_chunk(sX2, hrow, half * 4 + c, g);
      }
    }
    // the Out tile stored earlier has long left shared memory: confirmed here, off the critical path,
    // before the barrier after which the tile is written again
    if (tid == kProd) tma_wait_group_read<0>();
    publish();

    // ---- MMA6: Z2b = X2b W2
    TTT_ISSUE(mma_token_major(tmem + TM_Z, smem_u32(sX2), smem_u32(sW2)),
              ,
              ,
              )
    wait_mma();
    // ---- OUT: Q + gamma * LN(Z2b + b2) + beta
    {
      float z[16], b2c[8], gam[8], bet[8], q[16];
      tok_ld(tm, tmem + TM_Z, z);
      tok_ld_cols(tm, sB2, b2c);
      tok_ld_cols(tm, sGamma, gam);
      tok_ld_cols(tm, sBeta, bet);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        z[4 * j] += b2c[2 * j]; z[4 * j + 1] += b2c[2 * j + 1];
        z[4 * j + 2] += b2c[2 * j]; z[4 * j + 3] += b2c[2 * j + 1];
      }
      float rs0, rs1;
      tok_ld_tile(tm, sQ, q);           // requested before the all-reduces of the LayerNorm, used after them
      tok_layernorm(tm, z, TTT_LN_EPS, sXch, rs0, rs1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i0 = 4 * j + e, i1 = 4 * j + 2 + e, c = 2 * j + e;
          q[i0] += fmaf(gam[c], z[i0] * rs0, bet[c]);
          q[i1] += fmaf(gam[c], z[i1] * rs1, bet[c]);
        }
      }
      tok_st_tile(tm, sOut, q);
    }
    publish();
    if (tid == kProd) {
      tma_store_2d(&tmOut, sOut, 0, static_cast<int>((stream_id * NC + it) * 64));
      tma_commit_group();
      if (!*abort_flag && loads_issued < NC && loads_issued == it + kStages) {
        issue_loads(loads_issued);
        ++loads_issued;
      }
    }
    if (*abort_flag) break;
  }

  // ---- epilogue: optional final state, then teardown
  const bool aborted = *abort_flag != 0;
  if (!aborted && p.W1f != nullptr) {
    store_state(p.W1f + stream_id * (64 * 256), p.b1f + stream_id * 256, p.W2f + stream_id * (256 * 64),
                p.b2f + stream_id * 64);
  }
  if (aborted) {
    // everything this CTA still has in flight is waited for (bounded, not cut short by the abort flag)
    // before its shared and tensor memory go away: the tensor-core work of the four issuers ...
    if (warp < 4) {
      if (elect_one()) umma_commit(drain_bar);
      __syncwarp();
    }
    if (tid == kProd) {
      mbar_wait_bounded(drain_bar, 0, never_flag, limit);
      // ... and its own loads
      for (int j = it; j < loads_issued; ++j) {
        if (j == p.drop_load && stream_id == 0) continue;
        mbar_wait_bounded(&full[j % kStages], (j / kStages) & 1, never_flag, limit);
      }
      atomicExch(p.status, static_cast<uint32_t>(TTT_B200_ERR_TIMEOUT));
    }
  }
  if (tid == kProd) tma_wait_group<0>();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace

int ttt_launch_forward(const ttt_b200_fwd_args* a, cudaStream_t stream, uint32_t* status, uint64_t limit_ns,
                       int drop_load) {
  const uint64_t rows = static_cast<uint64_t>(a->B) * a->H * a->NC * 64;
  CUtensorMap tmQ, tmK, tmV, tmOut;
  if (int rc = ttt_make_tile_map(&tmQ, a->XQ, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmK, a->XK, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmV, a->XV, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmOut, a->Out, rows)) return rc;
  FwdParams p;
  p.eta = static_cast<const __nv_bfloat16*>(a->last_eta);
  p.gamma = a->ttt_norm_weight;
  p.beta = a->ttt_norm_bias;
  p.W1 = a->W1; p.b1 = a->b1; p.W2 = a->W2; p.b2 = a->b2;
  p.W1c = a->W1_checkpoints; p.b1c = a->b1_checkpoints; p.W2c = a->W2_checkpoints; p.b2c = a->b2_checkpoints;
  const bool want_final = a->W1_final && a->b1_final && a->W2_final && a->b2_final;
  p.W1f = want_final ? a->W1_final : nullptr;
  p.b1f = a->b1_final; p.W2f = a->W2_final; p.b2f = a->b2_final;
  p.H = a->H; p.NC = a->NC; p.cgs = a->checkpoint_group_size; p.nck = a->num_checkpoints;
  p.drop_load = drop_load;
  p.status = status;
  p.wait_limit_ns = limit_ns;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ttt_set_error(TTT_B200_ERR_LAUNCH, "device index out of range");
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(ttt_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (attr_err[dev] != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(attr_err[dev]));
  ttt_fwd_kernel<<<dim3(a->B * a->H), dim3(kThreads), SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmOut, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}
