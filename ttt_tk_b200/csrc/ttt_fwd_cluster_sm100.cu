// TTT-MLP forward for sm_100a, cluster-sharded: one thread-block cluster of kC = 2 or 4 CTAs per
// (batch, head) stream, each CTA owning 256 / kC of the hidden units.
//
// Replaces the reference's fwd_ttt_mlp_ker with its hidden dimension split over a cluster
// (kernels/ttt/ttt.cu:11-12, 85-586; the Z2 reductions at :332-348 and :506-522); the
// per-mini-batch math is that of kernels/ttt/matching.py:30-125.  The launcher uses it when a GPU
// has fewer streams than SMs: the mini-batches of a stream are strictly sequential, so splitting a
// stream over several SMs is the only way to put idle SMs to work on it.
//
// What is local and what is exchanged (ttt_cluster.cuh: RowSplit).  Everything indexed by a hidden unit is local to the CTA that
// owns the unit: its rows of W1^T and W2 (fp32 master copy in tensor memory as the accumulator of
// their own update MMA, bf16 operand copy in shared memory), its b1 entries, Z1^T, X2^T, gelu', U1^T
// and the state updates.  The two contractions over the hidden units, Z2 = X2 W2 and Z2b = X2b W2,
// leave a partial 64 x 64 fp32 tile per CTA; the partial tiles are summed across the cluster through
// distributed shared memory by reduce-scatter: CTA r receives the token rows 64 r / kC .. of every peer's
// tile, runs the LayerNorm stage on those rows with all of its threads, and (for the fused LayerNorm,
// whose result U2 every CTA needs as an MMA operand) copies its rows of the bf16 result into the peers'
// shared memories.  Every CTA loads its own copy of the K, V, Q
// tiles (plain TMA loads; after the first CTA they hit in L2).  b2 is kept, identically, by every CTA.
// Z2b is needed only for the output: every CTA normalises and stores the Out rows it owns.
//
// All accumulators are M = 64 tiles read with the 16x256b fragments (TokMap): a CTA's hidden units are
// NB = 4 / kC blocks of 64 rows.  Per mini-batch the steps are those of the one-CTA kernel
// (ttt_fwd_sm100.cu).  Every wait is bounded; a wait that runs out raises the abort flag of the whole
// cluster, and every CTA stays resident until its peers have reached the exit barrier.
#include <mutex>

#include "ttt_cluster.cuh"
#include "ttt_internal.h"

using namespace tttcl;

namespace {

constexpr int kStages = 3;
constexpr int kThreads = 256;
// The thread that issues the bulk copies and waits for their completion is not one of the four MMA issuers
// (lane 0 of warps 0..3): its bookkeeping between a barrier and the next MMA group stays off the issue path.
constexpr int kProd = 128;

template <int kC>
struct Cfg {
  static constexpr int NB = 4 / kC;                  // 64-row blocks of hidden units per CTA
  static constexpr int R = 64 * NB;                  // hidden units per CTA
  static constexpr uint32_t HB = NB * TILE;          // bytes of an [R][64] bf16 tile
  using RS = RowSplit<kC>;                     // kC = 4: row-split LayerNorm stages
  using Sum = ClusterSum<kC, 16384>;           // kC = 2: all-reduce, stages on the whole tile in both CTAs
  static constexpr bool kRowSplit = kC == 4;   // measured: at kC = 2 the second hop costs more than the halved stage saves
  static constexpr uint32_t OFF_K = 0;
  static constexpr uint32_t OFF_V = OFF_K + kStages * TILE;
  static constexpr uint32_t OFF_Q = OFF_V + kStages * TILE;
  static constexpr uint32_t OFF_OUT = OFF_Q + kStages * TILE;
  static constexpr uint32_t OFF_U2 = OFF_OUT + TILE;
  static constexpr uint32_t OFF_W1 = OFF_U2 + TILE;
  static constexpr uint32_t OFF_W2 = OFF_W1 + HB;
  static constexpr uint32_t OFF_X2 = OFF_W2 + HB;
  static constexpr uint32_t OFF_GP = OFF_X2 + HB;
  static constexpr uint32_t OFF_SUM = OFF_GP + HB;                 // cluster exchange area
  static constexpr uint32_t OFF_ETA = OFF_SUM + (kRowSplit ? RS::kBytes : Sum::kBytes);
  static constexpr uint32_t OFF_B2 = OFF_ETA + kStages * 128;
  static constexpr uint32_t OFF_GAMMA = OFF_B2 + 256;
  static constexpr uint32_t OFF_BETA = OFF_GAMMA + 256;
  static constexpr uint32_t OFF_BAR = OFF_BETA + 256;              // kStages + 1 + 4 + 1 + 1 mbarriers
  static constexpr uint32_t OFF_MISC = OFF_BAR + 128;
  static constexpr uint32_t OFF_PART = OFF_MISC + 64;              // fp32[4][64] column-sum partials
  static constexpr uint32_t OFF_XCH = OFF_PART + 1024;             // fp32[2][64][8] row-sum exchange between warp pairs
  static constexpr uint32_t OFF_ONES = (OFF_XCH + 4096 + 1023) & ~1023u;   // bf16[8][64] ones: B operand of the column sums
  static constexpr uint32_t SMEM_USED = OFF_ONES + 1024;
  static constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;         // slack for the 1024-byte alignment
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB per-CTA shared memory of sm_100");
  // tensor-memory columns (fp32), one 64-column M = 64 accumulator per block
  static constexpr uint32_t TM_W1 = 0;
  static constexpr uint32_t TM_W2 = 64 * NB;
  static constexpr uint32_t TM_A = 128 * NB;
  static constexpr uint32_t TM_Z = 192 * NB;
  static constexpr uint32_t TM_S = 192 * NB + 64;                  // 8 columns: column sums of U2
  static constexpr uint32_t TM_COLS = 512;
};

struct FwdClParams {
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
  __nv_bfloat16* out;
  int H, NC, cgs, nck;
  int drop_load;            // test only: mini-batch whose loads stream 0 never issues (-1: none)
  uint32_t* status;
  uint64_t wait_limit_ns;
};

template <int kC>
__global__ void __launch_bounds__(kThreads, 1)
ttt_fwd_cluster_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmOut,
                       const FwdClParams p) {
  using C = Cfg<kC>;
  constexpr int NB = C::NB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const TokMap tm(warp, lane);
  const uint32_t rank = cluster_ctarank();
  const long stream_id = blockIdx.x / kC;
  const int head = static_cast<int>(stream_id % p.H);
  const int hid0 = static_cast<int>(rank) * C::R;          // first hidden unit of this CTA

  uint8_t* sW1 = smem + C::OFF_W1;
  uint8_t* sW2 = smem + C::OFF_W2;
  uint8_t* sX2 = smem + C::OFF_X2;
  uint8_t* sGP = smem + C::OFF_GP;
  uint8_t* sU2 = smem + C::OFF_U2;
  uint8_t* sOut = smem + C::OFF_OUT;
  float* sB2 = reinterpret_cast<float*>(smem + C::OFF_B2);
  float* sGamma = reinterpret_cast<float*>(smem + C::OFF_GAMMA);
  float* sBeta = reinterpret_cast<float*>(smem + C::OFF_BETA);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);   // [kStages]
  uint64_t* mma_bar = full + kStages;
  uint64_t* sum_bars = mma_bar + 1;                                  // [4]
  uint64_t* drain_bar = sum_bars + 4;                                // abort path only
  uint64_t* ag_bar = drain_bar + 1;                                  // all-gather of the U2 rows
  float* sPart = reinterpret_cast<float*>(smem + C::OFF_PART);
  float* sXch = reinterpret_cast<float*>(smem + C::OFF_XCH);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 4);
  volatile uint32_t* never_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 8);   // stays 0

  const uint64_t limit = p.wait_limit_ns;
  const int NC = p.NC;

  if (tid == kProd) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    mbar_init(mma_bar, 4);
    for (int i = 0; i < C::RS::kBufs; ++i) mbar_init(&sum_bars[i], C::kRowSplit ? C::RS::kBarCount : C::Sum::kArrivals);
    mbar_init(drain_bar, 4);
    mbar_init(ag_bar, 1);
    fence_mbar_init();
    *abort_flag = 0;
    *never_flag = 0;
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmOut);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TM_COLS);
    tmem_relinquish();
  }
  if (tid < 64) {
    sGamma[tid] = p.gamma[head * 64 + tid];
    sBeta[tid] = p.beta[head * 64 + tid];
    sB2[tid] = p.b2[stream_id * 64 + tid];
  }
  reinterpret_cast<uint32_t*>(smem + C::OFF_ONES)[tid] = 0x3F803F80u;     // 256 x two bf16 ones
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // the peers' mbarriers and abort flags are initialised before anything is sent to them
  cluster_arrive();
  cluster_wait();
  const uint32_t tmem = *tmem_slot;

  typename C::RS rs;
  rs.bufp = smem + C::OFF_SUM;
  rs.bars = sum_bars;
  rs.n = 0;
  rs.rank = rank;
  rs.abort_flag = abort_flag;
  rs.limit = limit;
  constexpr int NR = C::RS::NR;                     // rows per thread in the row-split stages
  uint32_t ag_phase = 0;
  typename C::Sum csum;
  csum.bufp = smem + C::OFF_SUM;
  csum.bars = sum_bars;
  csum.n = 0;
  csum.rank = rank;
  csum.abort_flag = abort_flag;
  csum.limit = limit;

  auto issue_loads = [&](int i) {   // thread 0 only
    if (i == p.drop_load && stream_id == 0) return;
    const int s = i % kStages;
    const int row0 = static_cast<int>((stream_id * NC + i) * 64);
    mbar_expect_tx(&full[s], 3 * TILE + 128);
    tma_load_2d(smem + C::OFF_K + s * TILE, &tmK, &full[s], 0, row0);
    tma_load_2d(smem + C::OFF_V + s * TILE, &tmV, &full[s], 0, row0);
    tma_load_2d(smem + C::OFF_Q + s * TILE, &tmQ, &full[s], 0, row0);
    bulk_load_1d(smem + C::OFF_ETA + s * 128, p.eta + (stream_id * NC + i) * 64, 128, &full[s]);
  };
  int loads_issued = 0;
  if (tid == kProd) {
    for (; loads_issued < kStages && loads_issued < NC; ++loads_issued) issue_loads(loads_issued);
  }

  // ---- state <-> global memory.  In the fragment of block b a thread holds hidden units
  // hid0 + 64 b + r0 / r1 (rows) and, for j = 0..3, the feature pair col(j), col(j) + 1.
  // W1 is [64 feat][256 hid] in global memory, W2 [256 hid][64 feat].
  auto w1_index = [&](int b, int r, int c) { return c * 256 + hid0 + 64 * b + r; };
  auto w2_index = [&](int b, int r, int c) { return (hid0 + 64 * b + r) * 64 + c; };
  auto load_state_block = [&](const float* W1g, const float* W2g, int b) {
    float w1[16], w2[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      w1[4 * j] = W1g[w1_index(b, tm.r0, c)];
      w1[4 * j + 1] = W1g[w1_index(b, tm.r0, c + 1)];
      w1[4 * j + 2] = W1g[w1_index(b, tm.r1, c)];
      w1[4 * j + 3] = W1g[w1_index(b, tm.r1, c + 1)];
      const float2 a = *reinterpret_cast<const float2*>(W2g + w2_index(b, tm.r0, c));
      const float2 d = *reinterpret_cast<const float2*>(W2g + w2_index(b, tm.r1, c));
      w2[4 * j] = a.x; w2[4 * j + 1] = a.y; w2[4 * j + 2] = d.x; w2[4 * j + 3] = d.y;
    }
    tok_st_tmem(tm, tmem + C::TM_W1 + b * 64, w1);
    tok_st_tmem(tm, tmem + C::TM_W2 + b * 64, w2);
    tok_st_tile(tm, sW1 + b * TILE, w1);
    tok_st_tile(tm, sW2 + b * TILE, w2);
  };
  auto store_w1_block = [&](float* W1o, int b) {
    float w1[16];
    tok_ld(tm, tmem + C::TM_W1 + b * 64, w1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      W1o[w1_index(b, tm.r0, c)] = w1[4 * j];
      W1o[w1_index(b, tm.r0, c + 1)] = w1[4 * j + 1];
      W1o[w1_index(b, tm.r1, c)] = w1[4 * j + 2];
      W1o[w1_index(b, tm.r1, c + 1)] = w1[4 * j + 3];
    }
  };
  auto store_w2_block = [&](float* W2o, int b) {
    float w2[16];
    tok_ld(tm, tmem + C::TM_W2 + b * 64, w2);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      *reinterpret_cast<float2*>(W2o + w2_index(b, tm.r0, c)) = make_float2(w2[4 * j], w2[4 * j + 1]);
      *reinterpret_cast<float2*>(W2o + w2_index(b, tm.r1, c)) = make_float2(w2[4 * j + 2], w2[4 * j + 3]);
    }
  };

  float b1v[NB][2];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    b1v[b][0] = p.b1[stream_id * 256 + hid0 + 64 * b + tm.r0];
    b1v[b][1] = p.b1[stream_id * 256 + hid0 + 64 * b + tm.r1];
  }
  // of the 8 threads that hold a row's bias, this one writes it out
  const bool b1_writer = tm.colhalf == 0 && tm.l3 == 0;
  auto store_b1 = [&](float* b1o) {
    if (b1_writer) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        b1o[hid0 + 64 * b + tm.r0] = b1v[b][0];
        b1o[hid0 + 64 * b + tm.r1] = b1v[b][1];
      }
    }
  };
#pragma unroll
  for (int b = 0; b < NB; ++b)
    load_state_block(p.W1 + stream_id * (64 * 256), p.W2 + stream_id * (256 * 64), b);
  tmem_wait_st();
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  uint32_t mma_phase = 0;
  auto wait_mma = [&]() {
    mbar_wait_cl(mma_bar, mma_phase, abort_flag, limit, kC);
    mma_phase ^= 1;
    __syncwarp();
    tc_fence_after_sync();
  };
  auto publish = [&]() {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
  };
  // The MMAs of a phase are issued by lane 0 of warps 0..3, every one of which commits (an issuer
  // without work too): the MMA barrier counts four arrivals per phase.
#define TTT_ISSUE4(W0, W1_, W2_, W3)  \
  if (warp < 4) {                     \
    if (elect_one()) {                \
      tc_fence_after_sync();          \
      if (warp == 0) { W0; }          \
      else if (warp == 1) { W1_; }    \
      else if (warp == 2) { W2_; }    \
      else { W3; }                    \
      umma_commit(mma_bar);           \
    }                                 \
    __syncwarp();                     \
  }

  // The output of a mini-batch: its partial Z2b tile is sent at the end of the mini-batch (reduce-scatter);
  // the sums are received, normalised and stored, by the CTA that owns the rows, in the next mini-batch while
  // that one waits for its own Z2 sum.
  uint32_t zo_tag = 0;
  int zo_it = -1;
  float zo[16];          // kC = 2: the partial tile between the send and the receive of its reduce-scatter
  auto finish_out_whole = [&]() {
    const bool mine = csum.reduce_scatter_recv(zo, tid, zo_tag);
    if (mine) {       // whole warp pairs (the two warps of a fragment quadrant) take this branch together
      const uint8_t* sQp = smem + C::OFF_Q + (zo_it % kStages) * TILE;
      float b2c[8], gam[8], bet[8], q[16];
      tok_ld_cols(tm, sB2, b2c);
      tok_ld_cols(tm, sGamma, gam);
      tok_ld_cols(tm, sBeta, bet);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        zo[4 * j] += b2c[2 * j]; zo[4 * j + 1] += b2c[2 * j + 1];
        zo[4 * j + 2] += b2c[2 * j]; zo[4 * j + 3] += b2c[2 * j + 1];
      }
      float rs0, rs1;
      tok_ld_tile(tm, sQp, q);
      tok_layernorm(tm, zo, TTT_LN_EPS, sXch, rs0, rs1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i0 = 4 * j + e, i1 = 4 * j + 2 + e, c = 2 * j + e;
          q[i0] += fmaf(gam[c], zo[i0] * rs0, bet[c]);
          q[i1] += fmaf(gam[c], zo[i1] * rs1, bet[c]);
        }
      }
      tok_st_global(tm, p.out + (stream_id * NC + zo_it) * 4096, q);
    }
    zo_it = -1;
  };

  auto finish_out = [&]() {
    const uint8_t* sQp = smem + C::OFF_Q + (zo_it % kStages) * TILE;
    const float2 b2c = *reinterpret_cast<const float2*>(sB2 + 2 * lane);
    const float2 gam = *reinterpret_cast<const float2*>(sGamma + 2 * lane);
    const float2 bet = *reinterpret_cast<const float2*>(sBeta + 2 * lane);
    float2 q[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) q[i] = C::RS::ld_pair(sQp, rs.row(i, warp), lane);
    float z[NR][2];
    rs.recv(z, warp, lane, zo_tag);
    __nv_bfloat16* out_tile = p.out + (stream_id * NC + zo_it) * 4096;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      z[i][0] += b2c.x;
      z[i][1] += b2c.y;
      const float mu = C::RS::row_sum(z[i][0] + z[i][1]) * (1.f / 64.f);
      z[i][0] -= mu;
      z[i][1] -= mu;
      const float rstd = rsqrtf(C::RS::row_sum(fmaf(z[i][0], z[i][0], z[i][1] * z[i][1])) * (1.f / 64.f) + TTT_LN_EPS);
      C::RS::st_pair_global(out_tile, rs.row(i, warp), lane, q[i].x + fmaf(gam.x, z[i][0] * rstd, bet.x),
                            q[i].y + fmaf(gam.y, z[i][1] * rstd, bet.y));
    }
    zo_it = -1;
  };

  int it = 0;
  bool aborted = false;
  for (; it < NC; ++it) {
    const int s = it % kStages;
    const uint8_t* sK = smem + C::OFF_K + s * TILE;
    const uint8_t* sV = smem + C::OFF_V + s * TILE;
    const uint8_t* sQ = smem + C::OFF_Q + s * TILE;
    const __nv_bfloat16* sEta = reinterpret_cast<const __nv_bfloat16*>(smem + C::OFF_ETA + s * 128);

    // A checkpoint (the state before this mini-batch) leaves while the first three MMA groups of the
    // mini-batch run: they do not write the state columns (the update is the fourth).
    const bool ckpt = it % p.cgs == 0;
    const long ckc = stream_id * p.nck + it / p.cgs;
    float* ckW1 = p.W1c + ckc * (64 * 256);
    float* ckW2 = p.W2c + ckc * (256 * 64);
    mbar_wait_cl(&full[s], (it / kStages) & 1, abort_flag, limit, kC);

    // ---- MMA1: Z1^T = W1^T K^T (one block per issuer)
    TTT_ISSUE4(mma_hid64<false>(tmem + C::TM_A, smem_u32(sW1), smem_u32(sK), 0u),
               if (NB > 1) mma_hid64<false>(tmem + C::TM_A + 64, smem_u32(sW1 + TILE), smem_u32(sK), 0u),
               ,
               )
    if (ckpt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) store_w2_block(ckW2, b);
      store_b1(p.b1c + ckc * 256);
      if (rank == 0 && tid < 64) p.b2c[ckc * 64 + tid] = sB2[tid];   // before this mini-batch's column sums reach b2
    }
    if constexpr (!C::kRowSplit) {
      if (zo_it >= 0) finish_out_whole();    // the previous mini-batch's output, with the b2 it saw
    }
    wait_mma();
    // ---- EPI1: X2^T = gelu(Z1^T + b1), G' = gelu'(Z1^T + b1)
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float z[16], g[16], gp[16];
      tok_ld(tm, tmem + C::TM_A + b * 64, z);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          gelu_pair(z[4 * j + e] + b1v[b][0], g[4 * j + e], gp[4 * j + e]);
          gelu_pair(z[4 * j + 2 + e] + b1v[b][1], g[4 * j + 2 + e], gp[4 * j + 2 + e]);
        }
      }
      tok_st_tile(tm, sX2 + b * TILE, g);
      tok_st_tile(tm, sGP + b * TILE, gp);
    }
    publish();

    // ---- MMA2: partial Z2 = X2 W2 over this CTA's hidden units
    TTT_ISSUE4(mma_tok_partial(tmem + C::TM_Z, smem_u32(sX2), smem_u32(sW2), NB),
               ,
               ,
               )
    if (ckpt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) store_w1_block(ckW1, b);
      tc_fence_before_sync();      // the state columns are written by the fourth MMA group
    }
    wait_mma();
    // ---- LN: the partial Z2 tiles are summed by reduce-scatter; every CTA runs the fused LayerNorm + L2
    // gradient, U2 = -eta * dl/dZ2, on the token rows it owns (all 256 threads, CPT columns of one row each)
    // and hands its rows of U2 to the other CTAs' shared memories.
    if constexpr (C::kRowSplit) {
    {
      float frag[16];
      tok_ld(tm, tmem + C::TM_Z, frag);
      const uint32_t tag = rs.send(frag, tid, warp, lane);
      if (tid == 0) rs.arm_all_gather(ag_bar, 1);
      const float2 b2c = *reinterpret_cast<const float2*>(sB2 + 2 * lane);
      const float2 gam = *reinterpret_cast<const float2*>(sGamma + 2 * lane);
      const float2 bet = *reinterpret_cast<const float2*>(sBeta + 2 * lane);
      float2 kk[NR], vv[NR];
      float neta[NR];
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rs.row(i, warp);
        kk[i] = C::RS::ld_pair(sK, r, lane);
        vv[i] = C::RS::ld_pair(sV, r, lane);
        neta[i] = -__bfloat162float(sEta[r]);
      }
      // while this sum is under way: the previous mini-batch's output, whose sum arrived long ago (b2 has
      // not changed since: its update follows in the next MMA window)
      if (zo_it >= 0) finish_out();
      float z[NR][2];
      rs.recv(z, warp, lane, tag);
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        z[i][0] += b2c.x;
        z[i][1] += b2c.y;
        const float mu = C::RS::row_sum(z[i][0] + z[i][1]) * (1.f / 64.f);
        z[i][0] -= mu;
        z[i][1] -= mu;
        const float rstd = rsqrtf(C::RS::row_sum(fmaf(z[i][0], z[i][0], z[i][1] * z[i][1])) * (1.f / 64.f) + TTT_LN_EPS);
        const float x0 = z[i][0] * rstd, x1 = z[i][1] * rstd;
        const float g0 = (fmaf(gam.x, x0, bet.x) - (vv[i].x - kk[i].x)) * gam.x;
        const float g1 = (fmaf(gam.y, x1, bet.y) - (vv[i].y - kk[i].y)) * gam.y;
        const float a0 = C::RS::row_sum(g0 + g1);
        const float a1 = C::RS::row_sum(fmaf(g0, x0, g1 * x1));
        const float sc = neta[i] * rstd * (1.f / 64.f);
        rs.all_gather_store(sU2, ag_bar, rs.row(i, warp), lane, (64.f * g0 - a0 - x0 * a1) * sc,
                            (64.f * g1 - a0 - x1 * a1) * sc);
      }
    }
    mbar_wait_cl(ag_bar, ag_phase, abort_flag, limit, kC);
    ag_phase ^= 1u;
    } else {
    {
      float xh[16], b2c[8], gam[8], bet[8];
      tok_ld(tm, tmem + C::TM_Z, xh);
      csum.run(xh, tid, lane);
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
      tok_ld_tile(tm, sK, kk);
      tok_ld_tile(tm, sV, vv);
      tok_layernorm(tm, xh, TTT_LN_EPS, sXch, rs0, rs1);
      float a[2] = {0.f, 0.f}, bb[2] = {0.f, 0.f};
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
          bb[0] += g[i1]; bb[1] = fmaf(g[i1], xh[i1], bb[1]);
        }
      }
      tok_row_allreduce<2, 2>(tm, a, bb, sXch);
      const float sc0 = -__bfloat162float(sEta[tm.r0]) * rs0 * (1.f / 64.f);
      const float sc1 = -__bfloat162float(sEta[tm.r1]) * rs1 * (1.f / 64.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i0 = 4 * j + e, i1 = 4 * j + 2 + e;
          g[i0] = (64.f * g[i0] - a[0] - xh[i0] * a[1]) * sc0;
          g[i1] = (64.f * g[i1] - bb[0] - xh[i1] * bb[1]) * sc1;
        }
      }
      tok_st_tile(tm, sU2, g);
    }
    }
    publish();
    // the previous mini-batch's Q tile has been read by every warp (its output is finished): its stage takes
    // the loads of the mini-batch two ahead
    if (tid == kProd && it >= 1 && loads_issued < NC && loads_issued == it - 1 + kStages) {
      issue_loads(loads_issued);
      ++loads_issued;
    }

    // ---- MMA3: R^T = W2 U2^T
    // the column sums of U2 (the bf16 operand the W2 update sees) for b2 are taken by the tensor pipe in the same
    // phase: the window of these small MMAs is too short to hide a pass over the tile by the warps
    TTT_ISSUE4(mma_hid64<false>(tmem + C::TM_A, smem_u32(sW2), smem_u32(sU2), 0u),
               if (NB > 1) mma_hid64<false>(tmem + C::TM_A + 64, smem_u32(sW2 + TILE), smem_u32(sU2), 0u),
               mma_colsum(tmem + C::TM_S, smem_u32(sU2), smem_u32(smem + C::OFF_ONES)),
               )
    wait_mma();
    // b2 += column sums, the same in every CTA of the cluster (its next reader comes after the barrier below)
    if (warp < 4) {
      const float cs = colsum_read(tmem + C::TM_S, warp);
      if (lane < 16) sB2[16 * warp + lane] += cs;
    }
    // ---- EPI3: U1^T = R^T * G' (= -eta dl/dZ1), b1 += row sums
    {
      float ra[NB], rb[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float r[16], gp[16];
        tok_ld(tm, tmem + C::TM_A + b * 64, r);
        tok_ld_tile(tm, sGP + b * TILE, gp);
        ra[b] = 0.f; rb[b] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            gp[4 * j + e] *= r[4 * j + e];
            gp[4 * j + 2 + e] *= r[4 * j + 2 + e];
            ra[b] += gp[4 * j + e];
            rb[b] += gp[4 * j + 2 + e];
          }
        }
        tok_st_tile(tm, sGP + b * TILE, gp);
      }
      tok_row_allreduce<NB, 4>(tm, ra, rb, sXch);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        b1v[b][0] += ra[b];
        b1v[b][1] += rb[b];
      }
    }
    publish();

    // ---- MMA4: W1^T += U1^T K ;  W2 += X2^T U2
    TTT_ISSUE4(mma_hid64<true>(tmem + C::TM_W1, smem_u32(sGP), smem_u32(sK), 1u),
               mma_hid64<true>(tmem + C::TM_W2, smem_u32(sX2), smem_u32(sU2), 1u),
               if (NB > 1) mma_hid64<true>(tmem + C::TM_W1 + 64, smem_u32(sGP + TILE), smem_u32(sK), 1u),
               if (NB > 1) mma_hid64<true>(tmem + C::TM_W2 + 64, smem_u32(sX2 + TILE), smem_u32(sU2), 1u))
    wait_mma();
    // ---- EPI4: refresh the bf16 operand copies of the state
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float w[16];
      tok_ld(tm, tmem + C::TM_W1 + b * 64, w);
      tok_st_tile(tm, sW1 + b * TILE, w);
      tok_ld(tm, tmem + C::TM_W2 + b * 64, w);
      tok_st_tile(tm, sW2 + b * TILE, w);
    }
    publish();

    // ---- MMA5: Z1b^T = W1^T Q^T
    TTT_ISSUE4(mma_hid64<false>(tmem + C::TM_A, smem_u32(sW1), smem_u32(sQ), 0u),
               if (NB > 1) mma_hid64<false>(tmem + C::TM_A + 64, smem_u32(sW1 + TILE), smem_u32(sQ), 0u),
               ,
               )
    wait_mma();
    // ---- EPI5: X2b^T = gelu(Z1b^T + b1)
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float z[16];
      tok_ld(tm, tmem + C::TM_A + b * 64, z);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          z[4 * j + e] = gelu_only(z[4 * j + e] + b1v[b][0]);
          z[4 * j + 2 + e] = gelu_only(z[4 * j + 2 + e] + b1v[b][1]);
        }
      }
      tok_st_tile(tm, sX2 + b * TILE, z);
    }
    publish();

    // ---- MMA6: partial Z2b = X2b W2
    TTT_ISSUE4(mma_tok_partial(tmem + C::TM_Z, smem_u32(sX2), smem_u32(sW2), NB),
               ,
               ,
               )
    wait_mma();
    // ---- OUT: Q + gamma * LN(Z2b + b2) + beta.  Z2b is an output only: its partial tiles are summed by
    // reduce-scatter, and every CTA normalises and stores the token rows it owns.  The partial tile is
    // sent now; it is received, normalised and stored inside the first MMA window of the next mini-batch.
    if constexpr (C::kRowSplit) {
      float frag[16];
      tok_ld(tm, tmem + C::TM_Z, frag);
      zo_tag = rs.send(frag, tid, warp, lane);
    } else {
      tok_ld(tm, tmem + C::TM_Z, zo);
      zo_tag = csum.reduce_scatter_send(zo, tid);
    }
    zo_it = it;
    // the last CTA barrier of the mini-batch also takes the vote on leaving the loop: a peer can raise
    // this CTA's abort flag at any moment, and all 256 threads must see the same answer
    fence_proxy_async_smem();
    tc_fence_before_sync();
    aborted = __syncthreads_or(*abort_flag != 0) != 0;
    if (aborted) break;
  }
#undef TTT_ISSUE4
  if (!aborted && zo_it >= 0) {                  // the last mini-batch's output
    if constexpr (C::kRowSplit) finish_out();
    else finish_out_whole();
  }

  // ---- epilogue: optional final state, then teardown
  if (!aborted && p.W1f != nullptr) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      store_w1_block(p.W1f + stream_id * (64 * 256), b);
      store_w2_block(p.W2f + stream_id * (256 * 64), b);
    }
    store_b1(p.b1f + stream_id * 256);
    if (rank == 0 && tid < 64) p.b2f[stream_id * 64 + tid] = sB2[tid];
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
  // no CTA leaves while a peer may still write into its shared memory (exchange area, abort flag)
  cluster_exit(abort_flag);
  if (warp == 0) tmem_dealloc(tmem, C::TM_COLS);
}

// Once per device: the kernel's dynamic shared memory limit.
template <int kC>
int prepare_kernel() {
  using C = Cfg<kC>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return ttt_set_error(TTT_B200_ERR_LAUNCH, "device index out of range");
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(ttt_fwd_cluster_kernel<kC>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  });
  if (attr_err[dev] != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(attr_err[dev]));
  return TTT_B200_OK;
}

// How many clusters of kC CTAs the device runs at once (a cluster lives inside one GPC, and the GPCs' SM counts
// are not all multiples of kC: fewer than SMs / kC).  0 if the query fails.
template <int kC>
int cluster_capacity() {
  using C = Cfg<kC>;
  static std::once_flag once[64];
  static int cap[64];
  if (prepare_kernel<kC>()) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  std::call_once(once[dev], [&] {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kC * 64);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kC;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, ttt_fwd_cluster_kernel<kC>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cap[dev] = n;
  });
  return cap[dev];
}

template <int kC>
int launch_cluster(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmOut,
                   const FwdClParams& p, int streams, cudaStream_t stream) {
  using C = Cfg<kC>;
  if (int rc = prepare_kernel<kC>()) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(streams) * kC);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kC;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, ttt_fwd_cluster_kernel<kC>, tmQ, tmK, tmV, tmOut, p);
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}

}  // namespace

int ttt_launch_forward_cluster(const ttt_b200_fwd_args* a, int cluster, cudaStream_t stream, uint32_t* status,
                               uint64_t limit_ns, int drop_load) {
  const uint64_t rows = static_cast<uint64_t>(a->B) * a->H * a->NC * 64;
  CUtensorMap tmQ, tmK, tmV, tmOut;
  if (int rc = ttt_make_tile_map(&tmQ, a->XQ, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmK, a->XK, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmV, a->XV, rows)) return rc;
  if (int rc = ttt_make_tile_map(&tmOut, a->Out, rows)) return rc;
  FwdClParams p;
  p.eta = static_cast<const __nv_bfloat16*>(a->last_eta);
  p.gamma = a->ttt_norm_weight;
  p.beta = a->ttt_norm_bias;
  p.W1 = a->W1; p.b1 = a->b1; p.W2 = a->W2; p.b2 = a->b2;
  p.W1c = a->W1_checkpoints; p.b1c = a->b1_checkpoints; p.W2c = a->W2_checkpoints; p.b2c = a->b2_checkpoints;
  const bool want_final = a->W1_final && a->b1_final && a->W2_final && a->b2_final;
  p.W1f = want_final ? a->W1_final : nullptr;
  p.b1f = a->b1_final; p.W2f = a->W2_final; p.b2f = a->b2_final;
  p.out = static_cast<__nv_bfloat16*>(a->Out);
  p.H = a->H; p.NC = a->NC; p.cgs = a->checkpoint_group_size; p.nck = a->num_checkpoints;
  p.drop_load = drop_load;
  p.status = status;
  p.wait_limit_ns = limit_ns;
  const int streams = a->B * a->H;
  if (cluster == 2) return launch_cluster<2>(tmQ, tmK, tmV, tmOut, p, streams, stream);
  if (cluster == 4) return launch_cluster<4>(tmQ, tmK, tmV, tmOut, p, streams, stream);
  return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "cluster size must be 2 or 4");
}

int ttt_forward_cluster_capacity(int cluster) {
  return cluster == 2 ? cluster_capacity<2>() : cluster == 4 ? cluster_capacity<4>() : 0;
}
