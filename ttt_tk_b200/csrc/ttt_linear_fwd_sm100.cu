// TTT-Linear forward for sm_100a: the operator's mini-batch step with the inner model reduced from the
// two-layer MLP to one linear layer, f(x) = x W + b with W [64 x 64].
//
// The reference ships the TTT-MLP operator only (README.md:18: non-causal, head dimension 64); this
// variant keeps its interface, tensor layouts, checkpoint rule (kernels/ttt/matching.py:223-228) and the
// fused LayerNorm + L2 step of kernels/ttt/matching.py:67-101, and drops the hidden layer.  Per mini-batch
// (K, V, Q: 64 x 64 bf16 tiles, eta: 64 bf16):
//
//   MMA1  Z  = K W                              [64 tok x 64]
//   LN    x = LN(Z + b); e = gamma x + beta - (V - K); U = -eta * dl/dZ (the LayerNorm backward of
//         e * gamma)                            -> smem bf16;  b += column sums of U
//   MMA2  W^T += U^T K                          (accumulated into the fp32 state in tensor memory)
//   EPI   bf16 operand copy of the new W^T      -> smem
//   MMA3  Zb = Q W
//   OUT   Out = Q + gamma * LN(Zb + b) + beta   -> global
//
// Before mini-batch i with i % checkpoint_group_size == 0 the state (W, b) is stored as checkpoint
// i / checkpoint_group_size.  One CTA of 256 threads per (batch, head) stream; every tile is 64 x 64, read
// out of tensor memory as the 16x256b fragments of TokMap by all eight warps; up to three CTAs share an SM
// when there are more streams than SMs (72 KB of shared memory with a two-stage input ring, 128
// tensor-memory columns, 80 registers per thread each), which hides the latency of the three dependent MMA
// phases (measured at 1536 streams: 1.43 ms with two CTAs per SM and a three-stage ring, 1.34 ms with three).  All waits are bounded; on expiry the CTA reports through
// the status word, drains its own copies, frees its tensor memory and returns.
#include <mutex>

#include "ttt_cluster.cuh"
#include "ttt_internal.h"

using namespace tttcl;

namespace {

constexpr int kStages = 2;
constexpr int kThreads = 256;
constexpr int kProd = 128;     // issues the bulk copies; not the MMA issuer (lane 0 of warp 0)

constexpr uint32_t OFF_K = 0;
constexpr uint32_t OFF_V = OFF_K + kStages * TILE;
constexpr uint32_t OFF_Q = OFF_V + kStages * TILE;
constexpr uint32_t OFF_W = OFF_Q + kStages * TILE;      // bf16 W^T: row = output feature, column = input feature
constexpr uint32_t OFF_U = OFF_W + TILE;                // bf16 U: row = token
constexpr uint32_t OFF_ETA = OFF_U + TILE;
constexpr uint32_t OFF_B = OFF_ETA + kStages * 128;
constexpr uint32_t OFF_GAMMA = OFF_B + 256;
constexpr uint32_t OFF_BETA = OFF_GAMMA + 256;
constexpr uint32_t OFF_BAR = OFF_BETA + 256;
constexpr uint32_t OFF_MISC = OFF_BAR + 64;
constexpr uint32_t OFF_XCH = OFF_MISC + 64;             // fp32[2][64][8] row-sum exchange between warp pairs
constexpr uint32_t OFF_ONES = (OFF_XCH + 4096 + 1023) & ~1023u;   // bf16[8][64] ones: B operand of the column sums
constexpr uint32_t SMEM_USED = OFF_ONES + 1024;
constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;       // slack for the 1024-byte alignment
static_assert(3 * (SMEM_BYTES + 1024) <= 233472, "three CTAs per SM");

constexpr uint32_t TM_W = 0;
constexpr uint32_t TM_Z = 64;
constexpr uint32_t TM_COLS = 128;

struct LinParams {
  const __nv_bfloat16* eta;
  const float* gamma;
  const float* beta;
  const float* W;
  const float* b;
  float* Wc;
  float* bc;
  float* Wf;
  float* bf;
  __nv_bfloat16* out;
  int H, NC, cgs, nck;
  int drop_load;            // test only: mini-batch whose loads stream 0 never issues (-1: none)
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

__global__ void __launch_bounds__(kThreads, 3)
ttt_linear_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const LinParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const TokMap tm(warp, lane);
  const long stream_id = blockIdx.x;
  const int head = static_cast<int>(stream_id % p.H);

  uint8_t* sW = smem + OFF_W;
  uint8_t* sU = smem + OFF_U;
  float* sB = reinterpret_cast<float*>(smem + OFF_B);
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
    mbar_init(mma_bar, 1);
    mbar_init(drain_bar, 1);
    fence_mbar_init();
    *abort_flag = 0;
    *never_flag = 0;
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TM_COLS);
    tmem_relinquish();
  }
  if (tid < 64) {
    sGamma[tid] = p.gamma[head * 64 + tid];
    sBeta[tid] = p.beta[head * 64 + tid];
    sB[tid] = p.b[stream_id * 64 + tid];
  }
  reinterpret_cast<uint32_t*>(smem + OFF_ONES)[tid] = 0x3F803F80u;     // 256 x two bf16 ones
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  auto issue_loads = [&](int i) {   // thread kProd only
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

  // ---- state <-> global memory.  W is [64 in][64 out] in global memory; the fragment of W^T holds output
  // features r0 / r1 (rows) and, for j = 0..3, the input-feature pair col(j), col(j) + 1.
  auto load_state = [&](const float* Wg) {
    float w[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      w[4 * j] = Wg[c * 64 + tm.r0];
      w[4 * j + 1] = Wg[(c + 1) * 64 + tm.r0];
      w[4 * j + 2] = Wg[c * 64 + tm.r1];
      w[4 * j + 3] = Wg[(c + 1) * 64 + tm.r1];
    }
    tok_st_tmem(tm, tmem + TM_W, w);
    tok_st_tile(tm, sW, w);
  };
  auto store_state = [&](float* Wo, float* bo) {
    float w[16];
    tok_ld(tm, tmem + TM_W, w);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      Wo[c * 64 + tm.r0] = w[4 * j];
      Wo[(c + 1) * 64 + tm.r0] = w[4 * j + 1];
      Wo[c * 64 + tm.r1] = w[4 * j + 2];
      Wo[(c + 1) * 64 + tm.r1] = w[4 * j + 3];
    }
    if (tid < 64) bo[tid] = sB[tid];
  };
  load_state(p.W + stream_id * 4096);
  tmem_wait_st();
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  uint32_t mma_phase = 0;
  auto wait_mma = [&]() {
    mbar_wait_bounded(mma_bar, mma_phase, abort_flag, limit);
    mma_phase ^= 1;
    __syncwarp();
    tc_fence_after_sync();
  };
  auto publish = [&]() {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
  };
#define TTT_ISSUE1(WORK)            \
  if (warp == 0) {                  \
    if (elect_one()) {              \
      tc_fence_after_sync();        \
      WORK;                         \
      umma_commit(mma_bar);         \
    }                               \
    __syncwarp();                   \
  }

  int it = 0;
  for (; it < NC; ++it) {
    const int s = it % kStages;
    const uint8_t* sK = smem + OFF_K + s * TILE;
    const uint8_t* sV = smem + OFF_V + s * TILE;
    const uint8_t* sQ = smem + OFF_Q + s * TILE;
    const __nv_bfloat16* sEta = reinterpret_cast<const __nv_bfloat16*>(smem + OFF_ETA + s * 128);
    mbar_wait_bounded(&full[s], (it / kStages) & 1, abort_flag, limit);

    // ---- MMA1: Z = K W
    TTT_ISSUE1(mma_hid64<false>(tmem + TM_Z, smem_u32(sK), smem_u32(sW), 0u))
    // a checkpoint (the state before this mini-batch) leaves while MMA1 runs: it only reads the state
    if (it % p.cgs == 0) {
      const long ckc = stream_id * p.nck + it / p.cgs;
      store_state(p.Wc + ckc * 4096, p.bc + ckc * 64);
      tc_fence_before_sync();      // the state columns are written by the second MMA group
    }
    wait_mma();
    // ---- LN: fused LayerNorm + L2 gradient, U = -eta * dl/dZ
    {
      float xh[16], bc[8], gam[8], bet[8];
      tok_ld(tm, tmem + TM_Z, xh);
      tok_ld_cols(tm, sB, bc);
      tok_ld_cols(tm, sGamma, gam);
      tok_ld_cols(tm, sBeta, bet);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[4 * j] += bc[2 * j]; xh[4 * j + 1] += bc[2 * j + 1];
        xh[4 * j + 2] += bc[2 * j]; xh[4 * j + 3] += bc[2 * j + 1];
      }
      float rs0, rs1;
      float kk[16], vv[16], g[16];
      tok_ld_tile(tm, sK, kk);
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
      tok_st_tile(tm, sU, g);
    }
    publish();

    // ---- MMA2: W^T += U^T K; the column sums of U (the bf16 operand the update sees) for b are taken by the
    // tensor pipe in the same phase, into the accumulator columns that are free between Z and Zb
    TTT_ISSUE1(mma_mn_accumulate(tmem + TM_W, smem_u32(sU), smem_u32(sK));
               mma_colsum(tmem + TM_Z, smem_u32(sU), smem_u32(smem + OFF_ONES)))
    wait_mma();
    if (warp < 4) {
      const float cs = colsum_read(tmem + TM_Z, warp);
      if (lane < 16) sB[16 * warp + lane] += cs;       // its next reader comes after the barrier below
    }
    // ---- EPI: refresh the bf16 operand copy of the state
    {
      float w[16];
      tok_ld(tm, tmem + TM_W, w);
      tok_st_tile(tm, sW, w);
    }
    publish();

    // ---- MMA3: Zb = Q W
    TTT_ISSUE1(mma_hid64<false>(tmem + TM_Z, smem_u32(sQ), smem_u32(sW), 0u))
    wait_mma();
    // ---- OUT: Q + gamma * LN(Zb + b) + beta, straight to global memory
    {
      float z[16], bc[8], gam[8], bet[8], q[16];
      tok_ld(tm, tmem + TM_Z, z);
      tok_ld_cols(tm, sB, bc);
      tok_ld_cols(tm, sGamma, gam);
      tok_ld_cols(tm, sBeta, bet);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        z[4 * j] += bc[2 * j]; z[4 * j + 1] += bc[2 * j + 1];
        z[4 * j + 2] += bc[2 * j]; z[4 * j + 3] += bc[2 * j + 1];
      }
      float rs0, rs1;
      tok_ld_tile(tm, sQ, q);
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
      tok_st_global(tm, p.out + (stream_id * NC + it) * 4096, q);
    }
    // every warp has read this stage's tiles and the tensor-memory tile: the stage takes the loads of the
    // mini-batch kStages ahead, and all threads take the same decision on leaving the loop
    tc_fence_before_sync();
    const bool stop = __syncthreads_or(*abort_flag != 0) != 0;
    if (stop) break;
    if (tid == kProd && loads_issued < NC && loads_issued == it + kStages) {
      issue_loads(loads_issued);
      ++loads_issued;
    }
  }
#undef TTT_ISSUE1

  // ---- epilogue: optional final state, then teardown
  const bool aborted = __syncthreads_or(*abort_flag != 0) != 0;
  if (!aborted && p.Wf != nullptr) store_state(p.Wf + stream_id * 4096, p.bf + stream_id * 64);
  if (aborted) {
    // everything this CTA still has in flight is waited for (bounded, not cut short by the abort flag)
    // before its shared and tensor memory go away: the issuer's tensor-core work ...
    if (warp == 0) {
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
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

}  // namespace

int ttt_launch_linear_forward(const ttt_b200_linear_fwd_args* a, cudaStream_t stream, uint32_t* status,
                              uint64_t limit_ns, int drop_load) {
  const uint64_t rows = static_cast<uint64_t>(a->B) * a->H * a->NC * 64;
  CUtensorMap tmQ, tmK, tmV;
  if (int rc = ttt_make_tile_map(&tmQ, a->XQ, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmK, a->XK, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmV, a->XV, rows)) return rc;
  LinParams p;
  p.eta = static_cast<const __nv_bfloat16*>(a->last_eta);
  p.gamma = a->ttt_norm_weight;
  p.beta = a->ttt_norm_bias;
  p.W = a->W1; p.b = a->b1;
  p.Wc = a->W1_checkpoints; p.bc = a->b1_checkpoints;
  const bool want_final = a->W1_final && a->b1_final;
  p.Wf = want_final ? a->W1_final : nullptr;
  p.bf = a->b1_final;
  p.out = static_cast<__nv_bfloat16*>(a->Out);
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
    attr_err[dev] = cudaFuncSetAttribute(ttt_linear_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (attr_err[dev] != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(attr_err[dev]));
  ttt_linear_fwd_kernel<<<dim3(a->B * a->H), dim3(kThreads), SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}
