// TTT-MLP backward for sm_100a, cluster-sharded: one thread-block cluster of kC = 2 or 4 CTAs per
// (batch, head) stream, each CTA owning 256 / kC of the hidden units.
//
// Replaces the reference's bwd_ttt_mlp_ker with its hidden dimension split over a cluster of four
// CTAs and its tp_reduce (kernels/ttt_backward/ttt.cu:21-69, 179-1443; reductions at :574, :766,
// :1160); the math is that of kernels/ttt_backward/matching.py:57-342.  Structure, phase order,
// buffer rotation and scratch layout are those of the one-CTA kernel (ttt_bwd_sm100.cu), whose
// header lists the reverse step G1..G15 / E1..E6; what changes is the ownership:
//
//   local to the CTA that owns a hidden unit: its rows of W1^T / W2 and of the gradient state
//   dL/dW1^T / dL/dW2 (tensor memory), b1 and dL/db1 (registers), and every [256][64 tok] quantity
//   (Z1, X2, dl/dZ1, gelu', P, S, ... : NB = 4 / kC blocks of 64 rows).  In the scratch slots a CTA
//   writes and reads back only its own rows of the [256][64] images, so scratch written by this
//   kernel has the layout of the one-CTA kernel's.
//
//   summed over the cluster (ttt_cluster.cuh), as fp32 64 x 64 tiles: Z2 and Z2_bar in the
//   recompute; in the reverse step the hidden-unit contractions G7 (dQ), G5 / G6 / G8 (merged into
//   one tile: A2 = -eta acc1 + acc2, plus the two d_eta row sums that are linear in acc1 and T1) and
//   G13 (dK, together with the -eta T1 term).  Three sums per reverse step, two per recomputed
//   mini-batch.  dQ and dK are outputs only: they are summed by reduce-scatter (every CTA finishes and
//   stores the token rows it owns), which sends kC times fewer bytes than an all-reduce.
//
//   the 64 x 64 token stages (LayerNorm stages, second-order terms), in one of two forms:
//
//   kC = 2, replicated: every CTA computes them from the same summed tiles, bit for bit, together with b2,
//   dL/db2, d_gamma, d_beta.  The token-tile scratch (x_hat_fused, dl/dZ2, x_hat_ln, 1/std) is written by
//   every CTA with the same bytes, so that a CTA only ever reads back what it has written itself.  The CTAs
//   take turns storing dV; rank 0 stores d_eta and the per-stream vectors.
//
//   kC = 4, split by rows (RowSplit in ttt_cluster.cuh): every sum is a reduce-scatter to the CTA that owns
//   the 16 token rows, which runs the stage on them (warp = row pair, lane = column pair) and hands the bf16
//   rows that feed MMAs (dl/dZ2, U2, x_hat_ln, gZ2in) to every peer's operand tile.  x_hat_fused and the
//   1/std vectors are needed by the row's owner only: a CTA writes and reads back its own rows of those
//   scratch tiles.  dQ, dK, dV, d_eta are stored by the owner of the row.  b2 and dL/db2 stay replicated
//   (column sums of gathered tiles); the d_gamma / d_beta addends of the second-order stage are summed per
//   CTA over its own rows and added up by rank 0, in rank order, at the end.
//
// Every wait is bounded; a wait that runs out raises the abort flag of the whole cluster, the vote on
// leaving a loop is taken CTA-wide at a barrier, and no CTA exits before its peers have reached the
// exit barrier.
#include <mutex>

#include "ttt_cluster.cuh"
#include "ttt_internal.h"

using namespace tttcl;

namespace {

constexpr int kThreads = 256;
// The thread that issues the bulk copies and waits for their completion is not one of the four MMA issuers
// (lane 0 of warps 0..3): its bookkeeping between a barrier and the next MMA group stays off the issue path.
constexpr int kProd = 128;

// barrier indices
constexpr int BAR_BIG = 0;     // +buffer index (0..4)
constexpr int BAR_T = 5;       // +tile index (0..6)
constexpr int BAR_IN = 12;     // +stage (0..1), recompute inputs
constexpr int BAR_MMA = 14;
constexpr int BAR_V = 15;      // recompute: the single V tile
constexpr int BAR_SUM = 16;    // +buffer (0..3; the all-reduce form uses two), cluster sums
constexpr int BAR_DRAIN = 20;  // abort path only
constexpr int BAR_AG = 21;     // row-split form: rows of a stage's result arriving from the peers
constexpr int BAR_AG2 = 22;    // the same for the deferred x_hat_ln
constexpr int NUM_BARS = 23;

template <int kC>
struct Cfg {
  static constexpr int NB = 4 / kC;
  static constexpr int R = 64 * NB;
  static constexpr uint32_t HB = NB * TILE;            // bytes of an [R][64] bf16 tile
  using Sum = ClusterSum<kC, 18432>;                   // a 64 x 64 tile, optionally with two extra values per thread
  // Four CTAs: the token stages are split by rows as well (every CTA runs them on the 16 token rows it owns
  // and hands the bf16 results to its peers).  At two CTAs the row-split form works too (set this to true) but
  // was measured slower than the all-reduce form: 22.9 against 21.2 us per mini-batch at 32 streams.
  static constexpr bool kRowSplit = kC == 4;
  using RS = RowSplit<kC, true>;
  static constexpr uint32_t OFF_BIG = 0;               // 5 hidden-major buffers
  static constexpr uint32_t OFF_T = 5 * HB;            // 8 token tiles of 8 KB
  static constexpr uint32_t OFF_SUM = OFF_T + 8 * TILE;
  static constexpr uint32_t OFF_B2 = OFF_SUM + (kRowSplit ? RS::kBytes : Sum::kBytes);
  static constexpr uint32_t OFF_GB2 = OFF_B2 + 256;
  static constexpr uint32_t OFF_GAMMA = OFF_GB2 + 256;
  static constexpr uint32_t OFF_BETA = OFF_GAMMA + 256;
  static constexpr uint32_t OFF_DG = OFF_BETA + 256;
  static constexpr uint32_t OFF_DB = OFF_DG + 256;
  static constexpr uint32_t OFF_SIGLN = OFF_DB + 256;
  static constexpr uint32_t OFF_SIGF = OFF_SIGLN + 256;
  static constexpr uint32_t OFF_GB1 = OFF_SIGF + 256;       // fp32[R] copy of the per-thread dL/db1
  static constexpr uint32_t OFF_PART = OFF_GB1 + 1024;      // fp32[8][64] partial sums for d_eta (one row per warp)
  // fp32[3][4][64] column-sum partials (the row-split form keeps the second-order stage's own-row partials,
  // 2 x [8][64], in the row-sum exchange area, which is not in use between that stage and their sum)
  static constexpr uint32_t OFF_CSUM = OFF_PART + 2048;
  static constexpr uint32_t OFF_ETA = OFF_CSUM + 3072;      // bf16[2][64]
  static constexpr uint32_t OFF_BAR = OFF_ETA + 256;
  static constexpr uint32_t OFF_MISC = OFF_BAR + 192;
  static constexpr uint32_t OFF_XCH = OFF_MISC + 64;        // fp32[2][64][8] row-sum exchange between warp pairs
  // row-split form only: 1/std of x_hat_ln gathered from the row owners; d_gamma / d_beta addends of this
  // CTA's own rows ([2][64])
  static constexpr uint32_t OFF_SIGAG = OFF_XCH + 4096;
  static constexpr uint32_t OFF_DGP = OFF_SIGAG + 256;
  static constexpr uint32_t OFF_ONES = (OFF_DGP + 512 + 1023) & ~1023u;   // bf16[8][64] ones: B operand of the column sums
  static constexpr uint32_t SMEM_USED = OFF_ONES + (NB == 1 ? 1024 : 0);
  static constexpr uint32_t SMEM_BYTES = SMEM_USED + 1024;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB per-CTA shared memory of sm_100");
  static_assert(NUM_BARS * 8 <= 192, "barrier area");
  // tensor memory: state blocks, accumulator A (NB hidden blocks or one token tile), accumulator B (NB
  // hidden blocks or two token tiles)
  static constexpr uint32_t TM_S1 = 0;
  static constexpr uint32_t TM_S2 = 64 * NB;
  static constexpr uint32_t TM_A = 128 * NB;
  static constexpr uint32_t TM_B = 128 * NB + (NB > 1 ? 64 * NB : 64);
  // four CTAs per stream only (tensor memory is full at two): 8 columns each for column sums taken by the tensor pipe
  static constexpr bool kMmaColsum = NB == 1;
  static constexpr uint32_t TM_CS = TM_B + 128;
  static constexpr uint32_t TM_COLS = 512;
  static_assert(TM_B + 128 + (kMmaColsum ? 16 : 0) <= 512, "tensor memory");
};

struct BwdClParams {
  const __nv_bfloat16* eta;
  const float* gamma;
  const float* beta;
  const float* W1c; const float* b1c; const float* W2c; const float* b2c;
  uint8_t* sc_W1; uint8_t* sc_W2;                       // 64 KB per slot, first 32 KB used
  uint8_t* sc_Z1; uint8_t* sc_X2; uint8_t* sc_gZ1; uint8_t* sc_Z1b; uint8_t* sc_X2b;   // 32 KB per slot
  uint8_t* sc_xhf; uint8_t* sc_gZ2; uint8_t* sc_xhln;                                  // 8 KB per slot
  float* sc_sigf; float* sc_sigln;                      // 64 floats per slot
  const float* gW1_last; const float* gb1_last; const float* gW2_last; const float* gb2_last;
  float* d_gamma; float* d_beta;
  float* gW1; float* gb1; float* gW2; float* gb2;
  __nv_bfloat16* d_eta;
  __nv_bfloat16* dXQ; __nv_bfloat16* dXK; __nv_bfloat16* dXV;   // bf16 [rows][64], row-major
  int H, NC, cgs, nck;
  int drop_load;            // test only: mini-batch whose recompute inputs stream 0 never loads (-1: none)
  uint32_t* status;
  uint64_t wait_limit_ns;
};

template <int kC>
__global__ void __launch_bounds__(kThreads, 1)
ttt_bwd_cluster_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmGo,
                       const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                       const __grid_constant__ CUtensorMap tmDV, const BwdClParams p) {
  using C = Cfg<kC>;
  constexpr int NB = C::NB;
  constexpr uint32_t HB = C::HB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const TokMap tm(warp, lane);
  const uint32_t rank = cluster_ctarank();
  const long sid = blockIdx.x / kC;
  const int head = static_cast<int>(sid % p.H);
  const int NC = p.NC, cgs = p.cgs;
  const int hid0 = static_cast<int>(rank) * C::R;
  const uint32_t img0 = rank * HB;            // this CTA's rows inside a [256][64] scratch image
  const bool kp_owner = C::Sum::row_owner(tid) == rank;     // this thread's token rows are this CTA's to finish
  const bool row_writer = tm.colhalf == 0 && tm.l3 == 0;   // of the 8 threads that share a row, the one that stores per-row values

  auto big = [&](int i) -> uint8_t* { return smem + C::OFF_BIG + i * HB; };
  auto tile = [&](int i) -> uint8_t* { return smem + C::OFF_T + i * TILE; };
  float* sB2 = reinterpret_cast<float*>(smem + C::OFF_B2);
  float* sGb2 = reinterpret_cast<float*>(smem + C::OFF_GB2);
  float* sGamma = reinterpret_cast<float*>(smem + C::OFF_GAMMA);
  float* sBeta = reinterpret_cast<float*>(smem + C::OFF_BETA);
  float* sDG = reinterpret_cast<float*>(smem + C::OFF_DG);
  float* sDB = reinterpret_cast<float*>(smem + C::OFF_DB);
  float* sSigLn = reinterpret_cast<float*>(smem + C::OFF_SIGLN);
  float* sSigF = reinterpret_cast<float*>(smem + C::OFF_SIGF);
  float* sGb1 = reinterpret_cast<float*>(smem + C::OFF_GB1);
  float* sPart = reinterpret_cast<float*>(smem + C::OFF_PART);
  float* part = reinterpret_cast<float*>(smem + C::OFF_CSUM);
  __nv_bfloat16* sEta = reinterpret_cast<__nv_bfloat16*>(smem + C::OFF_ETA);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  float* sXch = reinterpret_cast<float*>(smem + C::OFF_XCH);
  float* sSigAG = reinterpret_cast<float*>(smem + C::OFF_SIGAG);
  float* sDGp = reinterpret_cast<float*>(smem + C::OFF_DGP);       // [0..63] d_gamma, [64..127] d_beta addends of the own rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 4);
  volatile uint32_t* never_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 8);   // stays 0
  const uint64_t limit = p.wait_limit_ns;

  if (tid == kProd) {
    for (int i = 0; i < NUM_BARS; ++i) {
      uint32_t cnt = 1;
      if (i == BAR_MMA || i == BAR_DRAIN) cnt = 4;
      if (i >= BAR_SUM && i < BAR_SUM + 4) cnt = C::kRowSplit ? C::RS::kBarCount : C::Sum::kArrivals;
      mbar_init(&bars[i], cnt);
    }
    fence_mbar_init();
    *abort_flag = 0;
    *never_flag = 0;
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmGo);
    prefetch_tmap(&tmDQ);
    prefetch_tmap(&tmDK);
    prefetch_tmap(&tmDV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TM_COLS);
    tmem_relinquish();
  }
  if (tid < 64) {
    sGamma[tid] = p.gamma[head * 64 + tid];
    sBeta[tid] = p.beta[head * 64 + tid];
    sGb2[tid] = p.gb2_last[sid * 64 + tid];
    sDG[tid] = 0.f;
    sDB[tid] = 0.f;
    sDGp[tid] = 0.f;
    sDGp[64 + tid] = 0.f;
  }
  if constexpr (C::kMmaColsum) reinterpret_cast<uint32_t*>(smem + C::OFF_ONES)[tid] = 0x3F803F80u;     // 256 x two bf16 ones
  float Gb1[NB][2];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    Gb1[b][0] = p.gb1_last[sid * 256 + hid0 + 64 * b + tm.r0];
    Gb1[b][1] = p.gb1_last[sid * 256 + hid0 + 64 * b + tm.r1];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  cluster_arrive();     // the peers' mbarriers and abort flags are initialised before anything is sent to them
  cluster_wait();
  const uint32_t tmem = *tmem_slot;

  typename C::Sum csum;
  csum.bufp = smem + C::OFF_SUM;
  csum.bars = &bars[BAR_SUM];
  csum.n = 0;
  csum.rank = rank;
  csum.abort_flag = abort_flag;
  csum.limit = limit;
  auto cluster_sum = [&](float (&v)[16]) { csum.run(v, tid, lane); };
  typename C::RS rs;
  rs.bufp = smem + C::OFF_SUM;
  rs.bars = &bars[BAR_SUM];
  rs.n = 0;
  rs.rank = rank;
  rs.abort_flag = abort_flag;
  rs.limit = limit;
  constexpr int NR = C::RS::NR;
  using RSx = typename C::RS;

  // ---- barrier bookkeeping: every thread waits on every barrier use, in program order
  uint32_t ph = 0;        // expected parity per barrier (indices 0..15)
  uint32_t pending = 0;   // thread 0: loads issued and not yet waited for
  auto wait_bar = [&](int b) {
    if (mbar_wait_cl(&bars[b], (ph >> b) & 1u, abort_flag, limit, kC)) {
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
  // the same barrier, also taking the CTA-wide vote on the abort flag (a peer can raise it at any moment)
  auto publish_vote = [&]() -> bool {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    return __syncthreads_or(*abort_flag != 0) != 0;
  };
  auto load_big = [&](int buf, const uint8_t* slot_image) {     // thread 0: this CTA's rows of a scratch image
    mbar_expect_tx(&bars[BAR_BIG + buf], HB);
    bulk_load_1d(big(buf), slot_image + img0, HB, &bars[BAR_BIG + buf]);
    pending |= 1u << (BAR_BIG + buf);
  };
  auto store_big = [&](uint8_t* slot_image, const uint8_t* src) {   // thread 0
    bulk_store_1d(slot_image + img0, src, HB);
  };
#define TTT_ISSUE4(W0, W1_, W2_, W3)  \
  if (warp < 4) {                     \
    if (elect_one()) {                \
      tc_fence_after_sync();          \
      if (warp == 0) { W0; }          \
      else if (warp == 1) { W1_; }    \
      else if (warp == 2) { W2_; }    \
      else { W3; }                    \
      umma_commit(&bars[BAR_MMA]);    \
    }                                 \
    __syncwarp();                     \
  }
  // hidden-major block products over this CTA's NB blocks: D[b] (+)= A[b] * Bt
#define HID_ALL(KBMN, D, A, BT, ACC)                                                          \
  do {                                                                                        \
    _Pragma("unroll") for (int b_ = 0; b_ < NB; ++b_)                                         \
      mma_hid64<KBMN>(tmem + (D) + b_ * 64, smem_u32(A) + b_ * TILE, smem_u32(BT), (ACC));    \
  } while (0)
#define HID_ONE(KBMN, D, A, BT, ACC, B_)                                                      \
  mma_hid64<KBMN>(tmem + (D) + (B_) * 64, smem_u32(A) + (B_) * TILE, smem_u32(BT), (ACC))

  const long tok_rows0 = sid * NC * 64;

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
  // the thread's eight token columns of the bf16 eta vector
  auto ld_eta_cols = [&](const __nv_bfloat16* e, float (&c)[8]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 w = *reinterpret_cast<const __nv_bfloat162*>(e + tm.col(j));
      c[2 * j] = __bfloat162float(w.x);
      c[2 * j + 1] = __bfloat162float(w.y);
    }
  };

  // ---- state <-> global memory (this CTA's rows): W1-shaped matrices are [64 feat][256 hid], W2-shaped
  // ones [256 hid][64 feat]; in the fragment of block b a thread holds hidden units hid0 + 64 b + r0 / r1
  // and, for j = 0..3, the feature pair col(j), col(j) + 1.
  auto w1_index = [&](int b, int r, int c) { return c * 256 + hid0 + 64 * b + r; };
  auto w2_index = [&](int b, int r, int c) { return (hid0 + 64 * b + r) * 64 + c; };
  auto load_w1_frag = [&](const float* W1g, int b, float (&w)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      w[4 * j] = W1g[w1_index(b, tm.r0, c)];
      w[4 * j + 1] = W1g[w1_index(b, tm.r0, c + 1)];
      w[4 * j + 2] = W1g[w1_index(b, tm.r1, c)];
      w[4 * j + 3] = W1g[w1_index(b, tm.r1, c + 1)];
    }
  };
  auto load_w2_frag = [&](const float* W2g, int b, float (&w)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      const float2 a = *reinterpret_cast<const float2*>(W2g + w2_index(b, tm.r0, c));
      const float2 d = *reinterpret_cast<const float2*>(W2g + w2_index(b, tm.r1, c));
      w[4 * j] = a.x; w[4 * j + 1] = a.y; w[4 * j + 2] = d.x; w[4 * j + 3] = d.y;
    }
  };
  auto store_w1_frag = [&](float* W1o, int b, const float (&w)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      W1o[w1_index(b, tm.r0, c)] = w[4 * j];
      W1o[w1_index(b, tm.r0, c + 1)] = w[4 * j + 1];
      W1o[w1_index(b, tm.r1, c)] = w[4 * j + 2];
      W1o[w1_index(b, tm.r1, c + 1)] = w[4 * j + 3];
    }
  };
  auto store_w2_frag = [&](float* W2o, int b, const float (&w)[16]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tm.col(j);
      *reinterpret_cast<float2*>(W2o + w2_index(b, tm.r0, c)) = make_float2(w[4 * j], w[4 * j + 1]);
      *reinterpret_cast<float2*>(W2o + w2_index(b, tm.r1, c)) = make_float2(w[4 * j + 2], w[4 * j + 3]);
    }
  };

  // =====================================================================================
  const float* Gsrc_W1 = p.gW1_last + sid * (64 * 256);
  const float* Gsrc_W2 = p.gW2_last + sid * (256 * 64);
  float* Gdst_W1 = p.gW1 + sid * (64 * 256);
  float* Gdst_W2 = p.gW2 + sid * (256 * 64);
  bool aborted = false;

  for (int ck = p.nck - 1; ck >= 0 && !aborted; --ck) {
    const int i0 = ck * cgs;
    const int gsz = min(cgs, NC - i0);
    const long slot0 = sid * cgs;           // scratch slot of the group's first mini-batch
    // buffer roles during recompute: 0 = W1^T bf16, 1 = W2 bf16, 2 = X2^T / X2_bar^T,
    // 3 = Z1^T -> U1^T -> gelu'(Z1_bar^T), 4 = G' -> dl/dZ1^T.  Token tiles: 0..3 = K, Q of two stages,
    // 4 = V, 5 = gZ2, 6 = U2.
    uint8_t* bW1 = big(0);
    uint8_t* bW2 = big(1);
    uint8_t* bX2 = big(2);
    uint8_t* bZ1 = big(3);
    uint8_t* bGP = big(4);
    uint8_t* tV = tile(4);
    uint8_t* tGZ2 = tile(5);
    uint8_t* tU2 = tile(6);

    auto issue_inputs = [&](int j) {   // thread 0
      if (i0 + j == p.drop_load && sid == 0) return;
      const int s = j & 1;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      mbar_expect_tx(&bars[BAR_IN + s], 2 * TILE + 128);
      tma_load_2d(tile(2 * s + 0), &tmK, &bars[BAR_IN + s], 0, row0);
      tma_load_2d(tile(2 * s + 1), &tmQ, &bars[BAR_IN + s], 0, row0);
      bulk_load_1d(sEta + s * 64, p.eta + (sid * NC + i0 + j) * 64, 128, &bars[BAR_IN + s]);
      pending |= 1u << (BAR_IN + s);
    };
    auto issue_v = [&](int j) {        // thread 0
      mbar_expect_tx(&bars[BAR_V], TILE);
      tma_load_2d(tV, &tmV, &bars[BAR_V], 0, static_cast<int>(tok_rows0 + (long)(i0 + j) * 64));
      pending |= 1u << BAR_V;
    };
    if (tid == kProd) {
      issue_inputs(0);
      issue_v(0);
      if (gsz > 1) issue_inputs(1);
    }

    // ---- checkpoint -> tensor memory (fp32) + shared memory (bf16) + scratch slot 0 (bf16)
    float b1v[NB][2];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      b1v[b][0] = p.b1c[(sid * p.nck + ck) * 256 + hid0 + 64 * b + tm.r0];
      b1v[b][1] = p.b1c[(sid * p.nck + ck) * 256 + hid0 + 64 * b + tm.r1];
    }
    if (tid < 64) sB2[tid] = p.b2c[(sid * p.nck + ck) * 64 + tid];
    {
      const float* W1g = p.W1c + (sid * p.nck + ck) * (64 * 256);
      const float* W2g = p.W2c + (sid * p.nck + ck) * (256 * 64);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float w1[16], w2[16];
        load_w1_frag(W1g, b, w1);
        load_w2_frag(W2g, b, w2);
        tok_st_tmem(tm, tmem + C::TM_S1 + b * 64, w1);
        tok_st_tmem(tm, tmem + C::TM_S2 + b * 64, w2);
        tok_st_tile(tm, bW1 + b * TILE, w1);
        tok_st_tile(tm, bW2 + b * TILE, w2);
      }
      tmem_wait_st();
    }
    publish();
    if (tid == kProd) {   // bf16 images of the checkpoint = pre-update weights of the group's first mini-batch
      store_big(p.sc_W1 + slot0 * 65536, bW1);
      store_big(p.sc_W2 + slot0 * 65536, bW2);
      tma_commit_group();
    }

    // ================================================================== recompute the group
    float zb[16];             // a mini-batch's partial Z2b between the send and the receive of its sum
    uint32_t zb_tag = 0;
    long zb_slot = -1;
    uint8_t* tXln = tile(7);  // x_hat_ln on its way to the scratch slot
    auto finish_xhln = [&]() {
      csum.allreduce_recv(zb, tid, zb_tag);
      float b2c[8];
      tok_ld_cols(tm, sB2, b2c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        zb[4 * q] += b2c[2 * q]; zb[4 * q + 1] += b2c[2 * q + 1];
        zb[4 * q + 2] += b2c[2 * q]; zb[4 * q + 3] += b2c[2 * q + 1];
      }
      float rs0, rs1;
      tok_layernorm(tm, zb, TTT_LN_EPS, sXch, rs0, rs1);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        zb[4 * q] *= rs0; zb[4 * q + 1] *= rs0;
        zb[4 * q + 2] *= rs1; zb[4 * q + 3] *= rs1;
      }
      tok_st_tile(tm, tXln, zb);
      if (row_writer) {
        p.sc_sigln[zb_slot * 64 + tm.r0] = rs0;
        p.sc_sigln[zb_slot * 64 + tm.r1] = rs1;
      }
    };
    // Row-split form: the sums of the rows this CTA owns are normalised here; the bf16 rows and their 1/std go
    // to every CTA of the cluster (each keeps a whole tile for its scratch slot).
    auto finish_xhln_rows = [&]() {
      if (tid == 0) rs.arm_all_gather(&bars[BAR_AG2], 1, C::RS::ROWS * 4u);
      const float2 b2c = *reinterpret_cast<const float2*>(sB2 + 2 * lane);
      float z[NR][2];
      rs.recv(z, warp, lane, zb_tag);
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rs.row(i, warp);
        z[i][0] += b2c.x;
        z[i][1] += b2c.y;
        const float mu = RSx::row_sum(z[i][0] + z[i][1]) * (1.f / 64.f);
        z[i][0] -= mu;
        z[i][1] -= mu;
        const float rstd = rsqrtf(RSx::row_sum(fmaf(z[i][0], z[i][0], z[i][1] * z[i][1])) * (1.f / 64.f) + TTT_LN_EPS);
        rs.all_gather_store(tXln, &bars[BAR_AG2], r, lane, z[i][0] * rstd, z[i][1] * rstd);
        if (lane == 0) sSigAG[r] = rstd;
        else if (lane < kC)
          st_async_f1(mapa(smem_u32(sSigAG + r), rank ^ static_cast<uint32_t>(lane)),
                      mapa(smem_u32(&bars[BAR_AG2]), rank ^ static_cast<uint32_t>(lane)), rstd);
      }
    };
    // after the barrier that follows the wait on BAR_AG2: the gathered tile and its 1/std leave for the slot
    auto store_xhln_rows = [&](long xslot) {
      if (tid < 64) p.sc_sigln[xslot * 64 + tid] = sSigAG[tid];
      if (tid == kProd) bulk_store_1d(p.sc_xhln + xslot * TILE, tXln, TILE);
    };
    for (int j = 0; j < gsz; ++j) {
      const int s = j & 1;
      const long slot = slot0 + j;
      const uint8_t* sK = tile(2 * s + 0);
      const uint8_t* sQ = tile(2 * s + 1);
      const uint8_t* sV = tV;
      const __nv_bfloat16* eta = sEta + s * 64;
      wait_bar(BAR_IN + s);

      // MMA1: Z1^T = W1^T K^T
      TTT_ISSUE4(HID_ONE(false, C::TM_A, bW1, sK, 0u, 0),
                 if (NB > 1) HID_ONE(false, C::TM_A, bW1, sK, 0u, NB - 1),
                 ,
                 )
      long xhln_slot = -1;                     // the previous mini-batch's x_hat_ln, with the b2 it saw
      if constexpr (!C::kRowSplit) {
        xhln_slot = zb_slot;
        if (zb_slot >= 0) {
          finish_xhln();
          zb_slot = -1;
        }
      }
      wait_mma();
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float z[16], g[16], gp[16];
        tok_ld(tm, tmem + C::TM_A + b * 64, z);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            z[4 * q + h] += b1v[b][0];
            z[4 * q + 2 + h] += b1v[b][1];
            gelu_pair(z[4 * q + h], g[4 * q + h], gp[4 * q + h]);
            gelu_pair(z[4 * q + 2 + h], g[4 * q + 2 + h], gp[4 * q + 2 + h]);
          }
        }
        tok_st_tile(tm, bX2 + b * TILE, g);
        tok_st_tile(tm, bGP + b * TILE, gp);
        tok_st_tile(tm, bZ1 + b * TILE, z);
      }
      publish();
      if (tid == kProd) {
        if (xhln_slot >= 0) bulk_store_1d(p.sc_xhln + xhln_slot * TILE, tXln, TILE);
        store_big(p.sc_X2 + slot * BIG, bX2);
        store_big(p.sc_Z1 + slot * BIG, bZ1);
        tma_commit_group();
      }

      // MMA2: partial Z2 = X2 W2
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_B, smem_u32(bX2), smem_u32(bW2), NB),
                 ,
                 ,
                 )
      wait_mma();
      wait_bar(BAR_V);
      long xrow_slot = -1;      // row-split form: the x_hat_ln gathered during this phase
      if constexpr (C::kRowSplit) {
        // the partial Z2 tiles are summed by reduce-scatter; the fused LayerNorm + L2 gradient runs on the token
        // rows this CTA owns (warp = row pair, lane = column pair) and its rows of dl/dZ2 and U2 go to every CTA
        float frag[16];
        tok_ld(tm, tmem + C::TM_B, frag);
        const uint32_t tag = rs.send(frag, tid, warp, lane);
        if (tid == 0) rs.arm_all_gather(&bars[BAR_AG], 2);
        const float2 b2c = *reinterpret_cast<const float2*>(sB2 + 2 * lane);
        const float2 gam = *reinterpret_cast<const float2*>(sGamma + 2 * lane);
        const float2 bet = *reinterpret_cast<const float2*>(sBeta + 2 * lane);
        float2 kk[NR], vv[NR];
        float neta[NR];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = rs.row(i, warp);
          kk[i] = RSx::ld_pair(sK, r, lane);
          vv[i] = RSx::ld_pair(sV, r, lane);
          neta[i] = -__bfloat162float(eta[r]);
        }
        // while this sum is under way: the previous mini-batch's x_hat_ln, whose sum arrived long ago (b2 has
        // not changed since: its update follows in the next MMA window)
        if (zb_slot >= 0) {
          xrow_slot = zb_slot;
          finish_xhln_rows();
          zb_slot = -1;
        }
        float z[NR][2];
        rs.recv(z, warp, lane, tag);
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = rs.row(i, warp);
          z[i][0] += b2c.x;
          z[i][1] += b2c.y;
          const float mu = RSx::row_sum(z[i][0] + z[i][1]) * (1.f / 64.f);
          z[i][0] -= mu;
          z[i][1] -= mu;
          const float rstd = rsqrtf(RSx::row_sum(fmaf(z[i][0], z[i][0], z[i][1] * z[i][1])) * (1.f / 64.f) + TTT_LN_EPS);
          const float x0 = z[i][0] * rstd, x1 = z[i][1] * rstd;
          const float g0 = (fmaf(gam.x, x0, bet.x) - (vv[i].x - kk[i].x)) * gam.x;
          const float g1 = (fmaf(gam.y, x1, bet.y) - (vv[i].y - kk[i].y)) * gam.y;
          const float a0 = RSx::row_sum(g0 + g1);
          const float a1 = RSx::row_sum(fmaf(g0, x0, g1 * x1));
          const float sc = rstd * (1.f / 64.f);
          // x_hat_fused leaves through this CTA's rows of the V tile; dl/dZ2 is rounded to bf16 once (the update
          // uses -eta times the rounded value)
          RSx::st_pair(tV, r, lane, x0, x1);
          const float d0 = __bfloat162float(__float2bfloat16((64.f * g0 - a0 - x0 * a1) * sc));
          const float d1 = __bfloat162float(__float2bfloat16((64.f * g1 - a0 - x1 * a1) * sc));
          rs.all_gather_store(tGZ2, &bars[BAR_AG], r, lane, d0, d1);
          rs.all_gather_store(tU2, &bars[BAR_AG], r, lane, neta[i] * d0, neta[i] * d1);
          if (lane == 0) p.sc_sigf[slot * 64 + r] = rstd;
        }
        wait_bar(BAR_AG);
        if (xrow_slot >= 0) wait_bar(BAR_AG2);
      } else {
        float xh[16], b2c[8], gam[8], bet[8];
        tok_ld(tm, tmem + C::TM_B, xh);
        cluster_sum(xh);
        tok_ld_cols(tm, sB2, b2c);
        tok_ld_cols(tm, sGamma, gam);
        tok_ld_cols(tm, sBeta, bet);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          xh[4 * q] += b2c[2 * q]; xh[4 * q + 1] += b2c[2 * q + 1];
          xh[4 * q + 2] += b2c[2 * q]; xh[4 * q + 3] += b2c[2 * q + 1];
        }
        float rs0, rs1;
        float kk[16], vv[16], g[16], e[16];
        tok_ld_tile(tm, sK, kk);
        tok_ld_tile(tm, sV, vv);
        tok_layernorm(tm, xh, TTT_LN_EPS, sXch, rs0, rs1);
        float a[2] = {0.f, 0.f}, bb[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h, c = 2 * q + h;
            xh[x0] *= rs0;
            xh[x1] *= rs1;
            e[x0] = fmaf(gam[c], xh[x0], bet[c]) - (vv[x0] - kk[x0]);
            e[x1] = fmaf(gam[c], xh[x1], bet[c]) - (vv[x1] - kk[x1]);
            g[x0] = e[x0] * gam[c];
            g[x1] = e[x1] * gam[c];
            a[0] += g[x0]; a[1] = fmaf(g[x0], xh[x0], a[1]);
            bb[0] += g[x1]; bb[1] = fmaf(g[x1], xh[x1], bb[1]);
          }
        }
        // x_hat_fused leaves through the V tile (every thread overwrites exactly the elements it has just
        // read) as a bulk store; grad_output_fused is rebuilt in the sweep from x_hat_fused, K, V
        tok_st_tile(tm, tV, xh);
        tok_row_allreduce<2, 2>(tm, a, bb, sXch);
        const float sc0 = rs0 * (1.f / 64.f), sc1 = rs1 * (1.f / 64.f);
        const float ne0 = -__bfloat162float(eta[tm.r0]), ne1 = -__bfloat162float(eta[tm.r1]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            // dl/dZ2, rounded to bf16 once: the update below uses -eta times the rounded value
            g[x0] = __bfloat162float(__float2bfloat16((64.f * g[x0] - a[0] - xh[x0] * a[1]) * sc0));
            g[x1] = __bfloat162float(__float2bfloat16((64.f * g[x1] - bb[0] - xh[x1] * bb[1]) * sc1));
          }
        }
        tok_st_tile(tm, tGZ2, g);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          g[4 * q] *= ne0; g[4 * q + 1] *= ne0;
          g[4 * q + 2] *= ne1; g[4 * q + 3] *= ne1;
        }
        tok_st_tile(tm, tU2, g);
        if (row_writer) {
          p.sc_sigf[slot * 64 + tm.r0] = rs0;     // the slot keeps 1/std: the sweep only ever divides by std
          p.sc_sigf[slot * 64 + tm.r1] = rs1;
        }
      }
      if (tid == kProd) tma_wait_group_read<0>();   // Z1 / X2 images have left shared memory
      publish();

      // MMA3: R^T = W2 gZ2^T
      if constexpr (C::kRowSplit) {
        if (xrow_slot >= 0) store_xhln_rows(xrow_slot);
      }
      if (tid == kProd) {
        if constexpr (C::kRowSplit) {   // only the rows this CTA owns hold x_hat_fused (the others still hold V)
          constexpr uint32_t RB = C::RS::ROWS * 128u;
          bulk_store_1d(p.sc_xhf + slot * TILE + rank * RB, tV + rank * RB, RB);
        } else {
          bulk_store_1d(p.sc_xhf + slot * TILE, tV, TILE);
        }
        bulk_store_1d(p.sc_gZ2 + slot * TILE, tGZ2, TILE);
        tma_commit_group();
      }
      if constexpr (C::kMmaColsum) {
        // b2 += column sums of U2, taken by the tensor pipe in the same phase (the window of these small MMAs is
        // too short to hide a pass over the tile by the warps)
        TTT_ISSUE4(HID_ONE(false, C::TM_A, bW2, tGZ2, 0u, 0),
                   mma_colsum(tmem + C::TM_CS, smem_u32(tU2), smem_u32(smem + C::OFF_ONES)),
                   ,
                   )
        wait_mma();
        if (warp < 4) {
          const float cs = colsum_read(tmem + C::TM_CS, warp);
          if (lane < 16) sB2[16 * warp + lane] += cs;
        }
      } else {
        TTT_ISSUE4(HID_ONE(false, C::TM_A, bW2, tGZ2, 0u, 0),
                   if (NB > 1) HID_ONE(false, C::TM_A, bW2, tGZ2, 0u, NB - 1),
                   ,
                   )
        part[tid] = colsum16(tU2);
        __syncthreads();
        if (tid < 64) sB2[tid] += part_sum(0);
        wait_mma();
      }
      {
        float et[8];
        ld_eta_cols(eta, et);
        float ra[NB], rb[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float r[16], gp[16], u[16];
          tok_ld(tm, tmem + C::TM_A + b * 64, r);
          tok_ld_tile(tm, bGP + b * TILE, gp);
          ra[b] = 0.f; rb[b] = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int x0 = 4 * q + h, x1 = 4 * q + 2 + h, c = 2 * q + h;
              // dl/dZ1 rounded to bf16 (the value the scratch slot and the sweep see); U1 = -eta dl/dZ1
              gp[x0] = __bfloat162float(__float2bfloat16(gp[x0] * r[x0]));
              gp[x1] = __bfloat162float(__float2bfloat16(gp[x1] * r[x1]));
              u[x0] = -et[c] * gp[x0];
              u[x1] = -et[c] * gp[x1];
              ra[b] += u[x0];
              rb[b] += u[x1];
            }
          }
          tok_st_tile(tm, bGP + b * TILE, gp);     // dl/dZ1, in place over G'
          tok_st_tile(tm, bZ1 + b * TILE, u);      // U1, over Z1
        }
        tok_row_allreduce<NB, 4>(tm, ra, rb, sXch);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          b1v[b][0] += ra[b];
          b1v[b][1] += rb[b];
        }
      }
      publish();

      // MMA4: W1^T += U1^T K ; W2 += X2^T U2
      if (tid == kProd) {
        tma_wait_group_read<0>();               // x_hat_fused has left the V tile
        if (j + 1 < gsz) issue_v(j + 1);
        store_big(p.sc_gZ1 + slot * BIG, bGP);
        tma_commit_group();
      }
      TTT_ISSUE4(HID_ONE(true, C::TM_S1, bZ1, sK, 1u, 0),
                 HID_ONE(true, C::TM_S2, bX2, tU2, 1u, 0),
                 if (NB > 1) HID_ONE(true, C::TM_S1, bZ1, sK, 1u, NB - 1),
                 if (NB > 1) HID_ONE(true, C::TM_S2, bX2, tU2, 1u, NB - 1))
      wait_mma();
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float w[16];
        tok_ld(tm, tmem + C::TM_S1 + b * 64, w);
        tok_st_tile(tm, bW1 + b * TILE, w);
        tok_ld(tm, tmem + C::TM_S2 + b * 64, w);
        tok_st_tile(tm, bW2 + b * TILE, w);
      }
      publish();

      // MMA5: Z1b^T = W1+^T Q^T
      if (tid == kProd) {
        if (j + 1 < gsz) {   // the new weights are the next mini-batch's pre-update weights
          store_big(p.sc_W1 + (slot + 1) * 65536, bW1);
          store_big(p.sc_W2 + (slot + 1) * 65536, bW2);
          tma_commit_group();
        }
      }
      TTT_ISSUE4(HID_ONE(false, C::TM_A, bW1, sQ, 0u, 0),
                 if (NB > 1) HID_ONE(false, C::TM_A, bW1, sQ, 0u, NB - 1),
                 ,
                 )
      wait_mma();
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float z[16], g[16];
        tok_ld(tm, tmem + C::TM_A + b * 64, z);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            // the sweep needs gelu'(Z1_bar) only: it is cheaper here, next to gelu, than there from a bf16 copy
            gelu_pair(z[4 * q + h] + b1v[b][0], g[4 * q + h], z[4 * q + h]);
            gelu_pair(z[4 * q + 2 + h] + b1v[b][1], g[4 * q + 2 + h], z[4 * q + 2 + h]);
          }
        }
        tok_st_tile(tm, bX2 + b * TILE, g);
        tok_st_tile(tm, bZ1 + b * TILE, z);
      }
      publish();

      // MMA6: partial Z2b = X2b W2+ ; output LayerNorm statistics
      if (tid == kProd) {
        store_big(p.sc_X2b + slot * BIG, bX2);
        store_big(p.sc_Z1b + slot * BIG, bZ1);
        tma_commit_group();
      }
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_B, smem_u32(bX2), smem_u32(bW2), NB),
                 ,
                 ,
                 )
      wait_mma();
      // Z2b only feeds the output LayerNorm statistics the sweep will read back from scratch: nothing in the
      // recompute waits for it.  Its partial tile is sent now; the sum is received and normalised inside the
      // first MMA window of the next mini-batch (or right after the group's last one).
      tok_ld(tm, tmem + C::TM_B, zb);
      if constexpr (C::kRowSplit) zb_tag = rs.send(zb, tid, warp, lane);
      else zb_tag = csum.allreduce_send(zb, tid);
      zb_slot = slot;
      if (tid == kProd) tma_wait_group_read<0>();   // every big image of this mini-batch has left shared memory
      aborted = publish_vote();
      if (tid == kProd && j + 2 < gsz && !aborted) issue_inputs(j + 2);
      if (aborted) break;
    }
    if (aborted) break;
    if constexpr (C::kRowSplit) {   // the group's last x_hat_ln
      finish_xhln_rows();
      wait_bar(BAR_AG2);
      publish();
      store_xhln_rows(zb_slot);
      if (tid == kProd) tma_commit_group();
    } else {
      finish_xhln();
      publish();
      if (tid == kProd) {
        bulk_store_1d(p.sc_xhln + zb_slot * TILE, tXln, TILE);
        tma_commit_group();
      }
    }

    // ================================================================== reverse sweep
    // buffer roles: ib0 = W1+ (bf16), ib1 = W2+, the other three free
    int ib0 = 0, ib1 = 1, ib2 = 2, ib3 = 3, ib4 = 4;
    uint8_t* t_go = tile(0);
    uint8_t* t_a = tile(1);     // x_hat_ln -> V -> d_gamma addends
    uint8_t* t_q = tile(2);     // Q -> gZ2in
    uint8_t* t_g = tile(3);     // gZ2b -> U2 = -eta gZ2
    uint8_t* t_k = tile(4);
    uint8_t* t_gz2 = tile(5);
    uint8_t* t_xf = tile(6);    // x_hat_fused
    auto issue_tiles_a = [&](int j) {          // dL/dOut, x_hat_ln + std_ln, x_hat_fused + std_fused
      const long slot = slot0 + j;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      mbar_expect_tx(&bars[BAR_T + 0], TILE);
      tma_load_2d(t_go, &tmGo, &bars[BAR_T + 0], 0, row0);
      mbar_expect_tx(&bars[BAR_T + 1], TILE + 256);
      bulk_load_1d(t_a, p.sc_xhln + slot * TILE, TILE, &bars[BAR_T + 1]);
      bulk_load_1d(sSigLn, p.sc_sigln + slot * 64, 256, &bars[BAR_T + 1]);
      mbar_expect_tx(&bars[BAR_T + 6], TILE + 256);
      bulk_load_1d(t_xf, p.sc_xhf + slot * TILE, TILE, &bars[BAR_T + 6]);
      bulk_load_1d(sSigF, p.sc_sigf + slot * 64, 256, &bars[BAR_T + 6]);
      pending |= (1u << (BAR_T + 0)) | (1u << (BAR_T + 1)) | (1u << (BAR_T + 6));
    };
    auto issue_rest = [&](int j) {             // Q, K + eta tiles; X2_bar and dl/dZ1
      const long slot = slot0 + j;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      mbar_expect_tx(&bars[BAR_T + 2], TILE);
      tma_load_2d(t_q, &tmQ, &bars[BAR_T + 2], 0, row0);
      load_big(ib3, p.sc_X2b + slot * BIG);
      mbar_expect_tx(&bars[BAR_T + 4], TILE + 128);
      tma_load_2d(t_k, &tmK, &bars[BAR_T + 4], 0, row0);
      bulk_load_1d(sEta, p.eta + (sid * NC + i0 + j) * 64, 128, &bars[BAR_T + 4]);
      load_big(ib4, p.sc_gZ1 + slot * BIG);
      pending |= (1u << (BAR_T + 2)) | (1u << (BAR_T + 4));
    };
    auto issue_gz2 = [&](int j) {
      tma_wait_group_read<0>();
      mbar_expect_tx(&bars[BAR_T + 5], TILE);
      bulk_load_1d(t_gz2, p.sc_gZ2 + (slot0 + j) * TILE, TILE, &bars[BAR_T + 5]);
      pending |= 1u << (BAR_T + 5);
    };
    // scratch was written partly with generic-proxy stores by all threads, partly with bulk
    // stores by thread 0: order both before the bulk (async-proxy) copies that read it back
    asm volatile("fence.proxy.async;" ::: "memory");
    if (tid == kProd) tma_wait_group<0>();
    publish();
    if (tid == kProd) {
      issue_tiles_a(gsz - 1);
      load_big(ib2, p.sc_Z1b + (slot0 + gsz - 1) * BIG);
      issue_rest(gsz - 1);
    }
    // dL/dW state: global (fp32) -> tensor memory
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float w1[16], w2[16];
      load_w1_frag(Gsrc_W1, b, w1);
      load_w2_frag(Gsrc_W2, b, w2);
      tok_st_tmem(tm, tmem + C::TM_S1 + b * 64, w1);
      tok_st_tmem(tm, tmem + C::TM_S2 + b * 64, w2);
    }
    tmem_wait_st();
    tc_fence_before_sync();   // the state columns are read by the MMAs of the first step

    float dk_pend[16];          // a step's share of dK between its send and its receive
    uint32_t dk_tag = 0;
    int dk_row0 = -1;
    float dk_gly[NR][2];        // row-split form: the LayerNorm term of dK for the rows this CTA owns
    auto finish_dk_rows = [&]() {
      float z[NR][2];
      rs.recv(z, warp, lane, dk_tag);
#pragma unroll
      for (int i = 0; i < NR; ++i)
        RSx::st_pair_global(p.dXK + static_cast<long>(dk_row0) * 64, rs.row(i, warp), lane, z[i][0] + dk_gly[i][0],
                            z[i][1] + dk_gly[i][1]);
    };
    for (int j = gsz - 1; j >= 0; --j) {
      const long slot = slot0 + j;
      const int row0 = static_cast<int>(tok_rows0 + (long)(i0 + j) * 64);
      const uint32_t turn = static_cast<uint32_t>(i0 + j);     // whose turn it is to store dQ / dV / dK
      float kp[16];                                            // this CTA's share of dK, completed in E6

      // ---- S4: backward of the output LayerNorm
      wait_bar(BAR_T + 0);
      wait_bar(BAR_T + 1);
      {
        float go[16], xl[16], gam[8];
        tok_ld_tile(tm, t_go, go);
        tok_ld_tile(tm, t_a, xl);
        tok_ld_cols(tm, sGamma, gam);
        float a[2] = {0.f, 0.f}, bb[2] = {0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            go[x0] *= gam[2 * q + h];
            go[x1] *= gam[2 * q + h];
            a[0] += go[x0]; a[1] = fmaf(go[x0], xl[x0], a[1]);
            bb[0] += go[x1]; bb[1] = fmaf(go[x1], xl[x1], bb[1]);
          }
        }
        tok_row_allreduce<2, 2>(tm, a, bb, sXch);
        const float q0 = sSigLn[tm.r0] * (1.f / 64.f), q1 = sSigLn[tm.r1] * (1.f / 64.f);   // 1 / (64 std)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            go[x0] = (64.f * go[x0] - a[0] - xl[x0] * a[1]) * q0;
            go[x1] = (64.f * go[x1] - bb[0] - xl[x1] * bb[1]) * q1;
          }
        }
        tok_st_tile(tm, t_g, go);
      }
      publish();
      // G1: gX2b^T = W2+ gZ2b^T
      TTT_ISSUE4(HID_ONE(false, C::TM_A, big(ib1), t_g, 0u, 0),
                 if (NB > 1) HID_ONE(false, C::TM_A, big(ib1), t_g, 0u, NB - 1),
                 ,
                 )
      {
        // column sums over the tokens: d_beta += sum go, d_gamma += sum go * x_hat_ln, G_b2 += sum gZ2b
        float a = 0.f, bsum = 0.f;
#pragma unroll 8
        for (int r = cs_q * 16; r < cs_q * 16 + 16; ++r) {
          const float go = ld_elem(t_go, r, cs_f);
          bsum += go;
          a = fmaf(go, ld_elem(t_a, r, cs_f), a);
        }
        part[tid] = bsum;
        part[256 + tid] = a;
        part[512 + tid] = colsum16(t_g);
        __syncthreads();
        if (tid < 64) {
          sDB[tid] += part_sum(0);
          sDG[tid] += part_sum(1);
          sGb2[tid] += part_sum(2);
        }
      }
      if (dk_row0 >= 0) {     // the previous step's dK
        if constexpr (C::kRowSplit) {
          finish_dk_rows();
        } else {
          if (csum.reduce_scatter_recv(dk_pend, tid, dk_tag)) tok_st_global(tm, p.dXK + static_cast<long>(dk_row0) * 64, dk_pend);
        }
        dk_row0 = -1;
      }
      wait_mma();
      if (tid == kProd) load_big(ib1, p.sc_X2 + slot * BIG);   // W2+ is consumed (G1 was its only use): X2 for G5
      wait_bar(BAR_BIG + ib2);
      // ---- E1: gZ1b^T = gX2b^T * gelu'(Z1b^T), in place over the gelu'(Z1_bar) tile
      {
        uint8_t* bz = big(ib2);
        float ra[NB], rb[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float v[16], z[16];
          tok_ld(tm, tmem + C::TM_A + b * 64, v);
          tok_ld_tile(tm, bz + b * TILE, z);
          ra[b] = 0.f; rb[b] = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              z[4 * q + h] *= v[4 * q + h];
              z[4 * q + 2 + h] *= v[4 * q + 2 + h];
              ra[b] += z[4 * q + h];
              rb[b] += z[4 * q + 2 + h];
            }
          }
          tok_st_tile(tm, bz + b * TILE, z);
        }
        tok_row_allreduce<NB, 4>(tm, ra, rb, sXch);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          Gb1[b][0] += ra[b];
          Gb1[b][1] += rb[b];
        }
      }
      publish();
      if (tid == kProd) {   // x_hat_ln and its column sums are consumed: bring V into that tile (E4 rebuilds
                        // grad_output_fused = gamma x_hat_fused + beta - (V - K) from it)
        mbar_expect_tx(&bars[BAR_T + 1], TILE);
        tma_load_2d(t_a, &tmV, &bars[BAR_T + 1], 0, row0);
        pending |= 1u << (BAR_T + 1);
        issue_gz2(j);
      }
      wait_bar(BAR_BIG + ib3);
      wait_bar(BAR_T + 2);
      // G7 (partial dQ) // G2 // G3
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_B, smem_u32(big(ib2)), smem_u32(big(ib0)), NB),
                 HID_ALL(true, C::TM_S2, big(ib3), t_g, 1u),
                 HID_ONE(true, C::TM_S1, big(ib2), t_q, 1u, 0),
                 if (NB > 1) HID_ONE(true, C::TM_S1, big(ib2), t_q, 1u, NB - 1))
      wait_mma();
      // gZ1b is consumed: Z1 of this step comes in while E2 runs (X2_bar's buffer takes the W2 snapshot)
      if (tid == kProd) load_big(ib2, p.sc_Z1 + slot * BIG);
      // ---- E2: bf16 snapshots of the gradient state; dQ
      {
        uint8_t* s1b = big(ib0);
        uint8_t* s2b = big(ib3);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float w[16];
          tok_ld(tm, tmem + C::TM_S1 + b * 64, w);
          tok_st_tile(tm, s1b + b * TILE, w);
          tok_ld(tm, tmem + C::TM_S2 + b * 64, w);
          tok_st_tile(tm, s2b + b * TILE, w);
          if (row_writer) {
            sGb1[64 * b + tm.r0] = Gb1[b][0];
            sGb1[64 * b + tm.r1] = Gb1[b][1];
          }
        }
      }
      // dQ = go + sum over the cluster of gZ1b W1+^T: an output only, so the partial tiles are summed by
      // reduce-scatter and every CTA stores the token rows it owns.  The partial tile is sent now and
      // received inside the next MMA window: nobody waits for the exchange.
      float dq[16];
      tok_ld(tm, tmem + C::TM_B, dq);
      uint32_t dq_tag;
      if constexpr (C::kRowSplit) dq_tag = rs.send(dq, tid, warp, lane);
      else dq_tag = csum.reduce_scatter_send(dq, tid);
      publish();
      wait_bar(BAR_BIG + ib4);
      wait_bar(BAR_T + 4);
      wait_bar(BAR_BIG + ib1);      // X2, requested two phases ago
      // G8 (partial T1) // G5 (partial acc1) // G4
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_B, smem_u32(big(ib4)), smem_u32(big(ib0)), NB),
                 mma_tok_partial(tmem + C::TM_B + 64, smem_u32(big(ib1)), smem_u32(big(ib3)), NB),
                 HID_ONE(false, C::TM_A, big(ib0), t_k, 0u, 0),
                 if (NB > 1) HID_ONE(false, C::TM_A, big(ib0), t_k, 0u, NB - 1))
      // ---- while the MMAs run: partial sums over this CTA's hidden units of gZ1 * G_b1 (fourth term of d_eta)
      {
        // warp w takes hidden units (R / 8) w .., lane l the token pair (2 l, 2 l + 1)
        constexpr int RW = C::R / 8;
        const uint8_t* bg = big(ib4) + (lane & 3) * 4;
        const uint32_t chunk = lane >> 2;
        float a0 = 0.f, a1 = 0.f, c0 = 0.f, c1 = 0.f;
#pragma unroll
        for (int hh = 0; hh < RW; hh += 4) {
          const int h = warp * RW + hh;
          const float4 g = *reinterpret_cast<const float4*>(sGb1 + h);
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(bg + sw128_off(h, chunk));
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(bg + sw128_off(h + 1, chunk));
          const uint32_t w2 = *reinterpret_cast<const uint32_t*>(bg + sw128_off(h + 2, chunk));
          const uint32_t w3 = *reinterpret_cast<const uint32_t*>(bg + sw128_off(h + 3, chunk));
          a0 = fmaf(bf16_lo(w0), g.x, a0); a1 = fmaf(bf16_hi(w0), g.x, a1);
          c0 = fmaf(bf16_lo(w1), g.y, c0); c1 = fmaf(bf16_hi(w1), g.y, c1);
          a0 = fmaf(bf16_lo(w2), g.z, a0); a1 = fmaf(bf16_hi(w2), g.z, a1);
          c0 = fmaf(bf16_lo(w3), g.w, c0); c1 = fmaf(bf16_hi(w3), g.w, c1);
        }
        *reinterpret_cast<float2*>(sPart + warp * 64 + 2 * lane) = make_float2(a0 + c0, a1 + c1);
      }
      if constexpr (C::kRowSplit) {
        // finished inside E4's wait for its own sum
      } else if (csum.reduce_scatter_recv(dq, tid, dq_tag)) {
        float go[16];
        tok_ld_tile(tm, t_go, go);
#pragma unroll
        for (int q = 0; q < 16; ++q) go[q] += dq[q];
        tok_st_global(tm, p.dXQ + static_cast<long>(row0) * 64, go);
      }
      wait_mma();
      if (tid == kProd) {
        load_big(ib1, p.sc_W2 + slot * 65536);      // X2 is consumed until G14: W2 takes its buffer
        tma_wait_group_read<0>();     // dQ has left the dL/dOut tile (E4 reuses it for dV)
      }
      wait_bar(BAR_BIG + ib2);
      // ---- E3: A1, P = A1 gelu'(Z1), S = A1 gelu''(Z1), gelu'(Z1)
      {
        uint8_t* bz = big(ib2);
        uint8_t* bp = big(ib4);
        uint8_t* bgp = big(ib0);
        float et[8];
        ld_eta_cols(sEta, et);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float v[16], z[16], pp[16], gp[16];
          tok_ld(tm, tmem + C::TM_A + b * 64, v);
          tok_ld_tile(tm, bz + b * TILE, z);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {       // h = 0: the pair of row r0, h = 1: the pair of row r1
              const int x = 4 * q + 2 * h;
              const float gb = Gb1[b][h];
              const float a10 = -et[2 * q] * (v[x] + gb);
              const float a11 = -et[2 * q + 1] * (v[x + 1] + gb);
              float gpp0, gpp1;
              gelu_grad_pair2(z[x], z[x + 1], gp[x], gp[x + 1], gpp0, gpp1);
              pp[x] = a10 * gp[x];
              pp[x + 1] = a11 * gp[x + 1];
              z[x] = a10 * gpp0;
              z[x + 1] = a11 * gpp1;
            }
          }
          tok_st_tile(tm, bp + b * TILE, pp);
          tok_st_tile(tm, bz + b * TILE, z);
          tok_st_tile(tm, bgp + b * TILE, gp);
        }
      }
      publish();
      wait_bar(BAR_BIG + ib1);
      wait_bar(BAR_T + 5);
      // G6 (partial acc2) // G10
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_A, smem_u32(big(ib4)), smem_u32(big(ib1)), NB),
                 HID_ONE(true, C::TM_S2, big(ib4), t_gz2, 1u, 0),
                 if (NB > 1) HID_ONE(true, C::TM_S2, big(ib4), t_gz2, 1u, NB - 1),
                 )
      wait_mma();
      if (tid == kProd) load_big(ib4, p.sc_W1 + slot * 65536);
      wait_bar(BAR_T + 6);
      wait_bar(BAR_T + 1);   // V
      // ---- E4: second order through the fused LayerNorm + L2 gradient (token-major, all 8 warps)
      if constexpr (C::kRowSplit) {
        // Row-split form.  Fragment side: this CTA's shares X2 G_W2 (acc1), P W2 (acc2), gZ1 G_W1 (t1); what the
        // step needs from them is linear: A2 = -eta acc1 + acc2 and the d_eta row sums of gz acc1 + t1 K travel
        // to the owner of the rows, -eta t1 stays for dK.  U2 = -eta gZ2 needs no sum: every CTA writes all of it.
        uint32_t a2_tag;
        {
          float A2[16], gz[16], kk[16], acc1[16], acc2[16], t1[16];
          const float eta0 = __bfloat162float(sEta[tm.r0]), eta1 = __bfloat162float(sEta[tm.r1]);
          tok_ld_tile(tm, t_gz2, gz);
          tok_ld_tile(tm, t_k, kk);
          tok_ld3(tm, tmem + C::TM_B + 64, acc1, tmem + C::TM_A, acc2, tmem + C::TM_B, t1);
          float de0 = 0.f, de1 = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
              A2[x0] = fmaf(-eta0, acc1[x0], acc2[x0]);
              A2[x1] = fmaf(-eta1, acc1[x1], acc2[x1]);
              de0 = fmaf(gz[x0], acc1[x0], fmaf(t1[x0], kk[x0], de0));
              de1 = fmaf(gz[x1], acc1[x1], fmaf(t1[x1], kk[x1], de1));
              kp[x0] = -eta0 * t1[x0];
              kp[x1] = -eta1 * t1[x1];
              gz[x0] *= -eta0;
              gz[x1] *= -eta1;
            }
          }
          if (row_writer) {     // the partial sums over this CTA's hidden units of gZ1 * G_b1, once per row
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              de0 += sPart[w * 64 + tm.r0];
              de1 += sPart[w * 64 + tm.r1];
            }
          }
          a2_tag = rs.send_x(A2, de0, de1, tid, warp, lane);
          if (tid == 0) rs.arm_all_gather(&bars[BAR_AG], 1);
          tok_st_tile(tm, t_g, gz);
        }
        // Row side: the rows this CTA owns (warp = row pair, lane = column pair)
        const float2 gam = *reinterpret_cast<const float2*>(sGamma + 2 * lane);
        const float2 bet = *reinterpret_cast<const float2*>(sBeta + 2 * lane);
        const float2 gb2 = *reinterpret_cast<const float2*>(sGb2 + 2 * lane);
        float2 gzr[NR], xh[NR], vv[NR], kr[NR];
        float etar[NR], rsd[NR];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = rs.row(i, warp);
          gzr[i] = RSx::ld_pair(t_gz2, r, lane);
          xh[i] = RSx::ld_pair(t_xf, r, lane);
          vv[i] = RSx::ld_pair(t_a, r, lane);
          kr[i] = RSx::ld_pair(t_k, r, lane);
          etar[i] = __bfloat162float(sEta[r]);
          rsd[i] = sSigF[r];       // 1 / std
        }
        {   // while the A2 sum is under way: dQ = dL/dOut + the sum sent in E2, on the rows this CTA owns
          float2 go[NR];
#pragma unroll
          for (int i = 0; i < NR; ++i) go[i] = RSx::ld_pair(t_go, rs.row(i, warp), lane);
          float zq[NR][2];
          rs.recv(zq, warp, lane, dq_tag);
#pragma unroll
          for (int i = 0; i < NR; ++i)
            RSx::st_pair_global(p.dXQ + static_cast<long>(row0) * 64, rs.row(i, warp), lane, go[i].x + zq[i][0],
                                go[i].y + zq[i][1]);
        }
        float z[NR][2], ex[NR];
        rs.recv_x(z, ex, warp, lane, a2_tag);
        float ca0 = 0.f, ca1 = 0.f, cv0 = 0.f, cv1 = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = rs.row(i, warp);
          const float rstd = rsd[i];
          // grad_output_fused = gamma x_hat_fused + beta - (V - K)
          const float go0 = fmaf(gam.x, xh[i].x, bet.x) - (vv[i].x - kr[i].x);
          const float go1 = fmaf(gam.y, xh[i].y, bet.y) - (vv[i].y - kr[i].y);
          // the G_b2 parts of u = acc1 + G_b2
          const float A0 = fmaf(-etar[i], gb2.x, z[i][0]), A1 = fmaf(-etar[i], gb2.y, z[i][1]);
          const float de = ex[i] + RSx::row_sum(fmaf(gzr[i].x, gb2.x, gzr[i].y * gb2.y));
          const float s2 = RSx::row_sum(A0 + A1);
          const float s3 = RSx::row_sum(fmaf(A0, xh[i].x, A1 * xh[i].y));
          const float s4 = RSx::row_sum(fmaf(go0 * gam.x, xh[i].x, go1 * gam.y * xh[i].y));
          const float bt0 = (A0 - (s2 + xh[i].x * s3) * (1.f / 64.f)) * rstd;
          const float bt1 = (A1 - (s2 + xh[i].y * s3) * (1.f / 64.f)) * rstd;
          const float gly0 = gam.x * bt0, gly1 = gam.y * bt1;
          ca0 += fmaf(go0, bt0, gly0 * xh[i].x);      // d_gamma addends
          ca1 += fmaf(go1, bt1, gly1 * xh[i].y);
          cv0 += gly0;                                // d_beta addends
          cv1 += gly1;
          dk_gly[i][0] = gly0;
          dk_gly[i][1] = gly1;
          RSx::st_pair_global(p.dXV + static_cast<long>(row0) * 64, r, lane, -gly0, -gly1);
          const float gx0 = fmaf(gly0, gam.x, -(go0 * gam.x * s3 + A0 * s4) * rstd * (1.f / 64.f));
          const float gx1 = fmaf(gly1, gam.y, -(go1 * gam.y * s3 + A1 * s4) * rstd * (1.f / 64.f));
          const float sa0 = RSx::row_sum(((-gx0 * xh[i].x - A0 * gzr[i].x) + (-gx1 * xh[i].y - A1 * gzr[i].y)) * rstd);
          const float sa1 = RSx::row_sum(gx0 + gx1);
          rs.all_gather_store(t_q, &bars[BAR_AG], r, lane,
                              fmaf(gx0, rstd, (sa0 * xh[i].x - sa1 * rstd) * (1.f / 64.f)),      // gZ2in
                              fmaf(gx1, rstd, (sa0 * xh[i].y - sa1 * rstd) * (1.f / 64.f)));
          if (lane == 0) p.d_eta[(sid * NC + i0 + j) * 64 + r] = __float2bfloat16(-de);
        }
        *reinterpret_cast<float2*>(sXch + warp * 64 + 2 * lane) = make_float2(ca0, ca1);
        *reinterpret_cast<float2*>(sXch + 512 + warp * 64 + 2 * lane) = make_float2(cv0, cv1);
        wait_bar(BAR_AG);
      } else {
        float A2[16], gz[16], xh[16], go[16];
        float gam[8];
        tok_ld_cols(tm, sGamma, gam);
        const float eta0 = __bfloat162float(sEta[tm.r0]), eta1 = __bfloat162float(sEta[tm.r1]);
        const float rs0 = sSigF[tm.r0], rs1 = sSigF[tm.r1];      // 1 / std
        tok_ld_tile(tm, t_gz2, gz);
        tok_ld_tile(tm, t_xf, xh);
        tok_ld_tile(tm, t_a, go);
        float ra[5] = {0.f, 0.f, 0.f, 0.f, 0.f}, rb[5] = {0.f, 0.f, 0.f, 0.f, 0.f};   // d_eta terms, (unused), sum A2, sum A2 xh, sum gxf xh
        {
          float kk[16], gb2[8], bet[8];
          tok_ld_tile(tm, t_k, kk);
          {
            // this CTA's shares: X2 G_W2 (acc1), P W2 (acc2), gZ1 G_W1 (t1).  Everything the step needs
            // from them is linear: A2 = -eta acc1 + acc2, the d_eta row sums of gz acc1 and of t1 K, and
            // -eta t1 inside dK; one cluster sum carries the first three, the dK sum the last.
            float acc1[16], acc2[16], t1[16];
            tok_ld3(tm, tmem + C::TM_B + 64, acc1, tmem + C::TM_A, acc2, tmem + C::TM_B, t1);
            float de0 = 0.f, de1 = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
                A2[x0] = fmaf(-eta0, acc1[x0], acc2[x0]);
                A2[x1] = fmaf(-eta1, acc1[x1], acc2[x1]);
                de0 = fmaf(gz[x0], acc1[x0], fmaf(t1[x0], kk[x0], de0));
                de1 = fmaf(gz[x1], acc1[x1], fmaf(t1[x1], kk[x1], de1));
                kp[x0] = -eta0 * t1[x0];
                kp[x1] = -eta1 * t1[x1];
              }
            }
            if (row_writer) {     // the partial sums over this CTA's hidden units of gZ1 * G_b1, once per row
#pragma unroll
              for (int w = 0; w < 8; ++w) {
                de0 += sPart[w * 64 + tm.r0];
                de1 += sPart[w * 64 + tm.r1];
              }
            }
            csum.run_with_extras(A2, de0, de1, tid, lane);
            ra[0] = de0;
            rb[0] = de1;
          }
          tok_ld_cols(tm, sGb2, gb2);
          tok_ld_cols(tm, sBeta, bet);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int x0 = 4 * q + h, x1 = 4 * q + 2 + h, c = 2 * q + h;
              // go[] arrives holding V: grad_output_fused = gamma x_hat_fused + beta - (V - K)
              go[x0] = fmaf(gam[c], xh[x0], bet[c]) - (go[x0] - kk[x0]);
              go[x1] = fmaf(gam[c], xh[x1], bet[c]) - (go[x1] - kk[x1]);
              // the G_b2 parts of u = acc1 + G_b2
              ra[0] = fmaf(gz[x0], gb2[c], ra[0]);
              rb[0] = fmaf(gz[x1], gb2[c], rb[0]);
              A2[x0] = fmaf(-eta0, gb2[c], A2[x0]);
              A2[x1] = fmaf(-eta1, gb2[c], A2[x1]);
              ra[2] += A2[x0];
              rb[2] += A2[x1];
              ra[3] = fmaf(A2[x0], xh[x0], ra[3]);
              rb[3] = fmaf(A2[x1], xh[x1], rb[3]);
              ra[4] = fmaf(go[x0] * gam[c], xh[x0], ra[4]);
              rb[4] = fmaf(go[x1] * gam[c], xh[x1], rb[4]);
            }
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
              const float bt = (A2[x] - (ra[2] + xh[x] * ra[3]) * (1.f / 64.f)) * rs0;
              const float gly = gm * bt;
              dga[x] = fmaf(go[x], bt, gly * xh[x]);
              dv[x] = -gly;
              if (kp_owner) kp[x] += gly;         // added once across the cluster: by the CTA that owns the row
              const float gxh = fmaf(gly, gm, -(go[x] * gm * ra[3] + A2[x] * ra[4]) * rs0 * (1.f / 64.f));
              sa[0] += (-gxh * xh[x] - A2[x] * gz[x]) * rs0;
              sa[1] += gxh;
              A2[x] = gxh;
            }
            {
              const int x = 4 * q + 2 + h;
              const float bt = (A2[x] - (rb[2] + xh[x] * rb[3]) * (1.f / 64.f)) * rs1;
              const float gly = gm * bt;
              dga[x] = fmaf(go[x], bt, gly * xh[x]);
              dv[x] = -gly;
              if (kp_owner) kp[x] += gly;
              const float gxh = fmaf(gly, gm, -(go[x] * gm * rb[3] + A2[x] * rb[4]) * rs1 * (1.f / 64.f));
              sb[0] += (-gxh * xh[x] - A2[x] * gz[x]) * rs1;
              sb[1] += gxh;
              A2[x] = gxh;
            }
          }
        }
        tok_st_tile(tm, t_a, dga);       // d_gamma addends, over V
        tok_st_tile(tm, t_go, dv);       // dV: stored by TMA, and column-summed for d_beta
        tok_row_allreduce<2, 5>(tm, sa, sb, sXch);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
            A2[x0] = fmaf(A2[x0], rs0, (sa[0] * xh[x0] - sa[1] * rs0) * (1.f / 64.f));   // gZ2in
            A2[x1] = fmaf(A2[x1], rs1, (sb[0] * xh[x1] - sb[1] * rs1) * (1.f / 64.f));
            gz[x0] *= -eta0;                                                            // U2 = -eta gZ2
            gz[x1] *= -eta1;
          }
        }
        tok_st_tile(tm, t_q, A2);
        tok_st_tile(tm, t_g, gz);
        if (row_writer && rank == 0) {
          p.d_eta[(sid * NC + i0 + j) * 64 + tm.r0] = __float2bfloat16(-ra[0]);
          p.d_eta[(sid * NC + i0 + j) * 64 + tm.r1] = __float2bfloat16(-rb[0]);
        }
      }
      publish();
      // G11 (+ G_W2snap U2^T) // G12
      if constexpr (!C::kRowSplit) {
        if (tid == kProd && (turn + 1) % kC == rank) {
          tma_store_2d(&tmDV, t_go, 0, row0);
          tma_commit_group();
        }
      }
      TTT_ISSUE4(HID_ONE(false, C::TM_B, big(ib1), t_q, 0u, 0); HID_ONE(false, C::TM_B, big(ib3), t_g, 1u, 0),
                 if (NB > 1) { HID_ONE(false, C::TM_B, big(ib1), t_q, 0u, NB - 1); HID_ONE(false, C::TM_B, big(ib3), t_g, 1u, NB - 1); }
                 else if (C::kMmaColsum) mma_colsum(tmem + C::TM_CS + 8, smem_u32(t_q), smem_u32(smem + C::OFF_ONES)),
                 HID_ONE(false, C::TM_A, big(ib1), t_gz2, 0u, 0),
                 if (NB > 1) HID_ONE(false, C::TM_A, big(ib1), t_gz2, 0u, NB - 1))
      if constexpr (C::kRowSplit && C::kMmaColsum) {
        // the second-order stage's d_gamma / d_beta partials (this CTA's rows only: summed over the cluster at
        // the end) are read out of the row-sum exchange area before the barrier below; the next epilogue, which
        // uses that area again, comes after it.  The column sums of the gathered gZ2in tile (G_b2 stays
        // replicated) come from the tensor pipe after the phase.
        if (tid < 64) {
          float a = 0.f, v = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            a += sXch[w * 64 + tid];
            v += sXch[512 + w * 64 + tid];
          }
          sDGp[tid] += a;
          sDGp[64 + tid] += v;
        }
        __syncthreads();
      } else if constexpr (C::kRowSplit) {
        // the second-order stage's d_gamma / d_beta partials (this CTA's rows only: summed over the cluster at
        // the end) are read out of the row-sum exchange area before the barrier below; the next epilogue, which
        // uses that area again, comes after it
        float a = 0.f, v = 0.f;
        if (tid < 64) {
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            a += sXch[w * 64 + tid];
            v += sXch[512 + w * 64 + tid];
          }
        }
        part[tid] = colsum16(t_q);      // the gathered gZ2in tile: G_b2 stays replicated
        __syncthreads();
        if (tid < 64) {
          sGb2[tid] += part_sum(0);
          sDGp[tid] += a;
          sDGp[64 + tid] += v;
        }
      } else {
        part[tid] = colsum16(t_q);
        part[256 + tid] = colsum16(t_a);
        part[512 + tid] = colsum16(t_go);
        __syncthreads();
        if (tid < 64) {
          sGb2[tid] += part_sum(0);
          sDG[tid] += part_sum(1);
          sDB[tid] -= part_sum(2);
        }
      }
      wait_mma();
      if constexpr (C::kRowSplit && C::kMmaColsum) {
        if (warp < 4) {
          const float cs = colsum_read(tmem + C::TM_CS + 8, warp);
          if (lane < 16) sGb2[16 * warp + lane] += cs;
        }
      }
      if (tid == kProd) {
        // the W2 state-gradient snapshot is consumed: X2 comes back into its buffer for G14; dV has left
        // its tile, the d_gamma addends and x_hat_fused are consumed: the next step's first tiles are
        // requested now, two phases before they are needed
        load_big(ib3, p.sc_X2 + slot * BIG);
        tma_wait_group_read<0>();
        if (j > 0) issue_tiles_a(j - 1);
      }
      // ---- E5: gZ1in^T = gX2^T gelu'(Z1^T) + R^T S^T, in place over S^T
      {
        uint8_t* bs = big(ib2);
        const uint8_t* bgp = big(ib0);
        float ra[NB], rb[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float v[16], w[16], gp[16], sv[16];
          tok_ld(tm, tmem + C::TM_B + b * 64, v);
          tok_ld(tm, tmem + C::TM_A + b * 64, w);
          tok_ld_tile(tm, bgp + b * TILE, gp);
          tok_ld_tile(tm, bs + b * TILE, sv);
          ra[b] = 0.f; rb[b] = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int x0 = 4 * q + h, x1 = 4 * q + 2 + h;
              sv[x0] = fmaf(v[x0], gp[x0], w[x0] * sv[x0]);
              sv[x1] = fmaf(v[x1], gp[x1], w[x1] * sv[x1]);
              ra[b] += sv[x0];
              rb[b] += sv[x1];
            }
          }
          tok_st_tile(tm, bs + b * TILE, sv);
        }
        tok_row_allreduce<NB, 0>(tm, ra, rb, sXch);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          Gb1[b][0] += ra[b];
          Gb1[b][1] += rb[b];
        }
      }
      publish();
      // gelu'(Z1) is consumed: the next step's gelu'(Z1_bar) comes into its buffer
      if (tid == kProd && j > 0) load_big(ib0, p.sc_Z1b + (slot - 1) * BIG);
      wait_bar(BAR_BIG + ib4);
      wait_bar(BAR_BIG + ib3);
      // G13 (partial dK) // G15 // G14
      TTT_ISSUE4(mma_tok_partial(tmem + C::TM_A, smem_u32(big(ib2)), smem_u32(big(ib4)), NB),
                 HID_ALL(true, C::TM_S1, big(ib2), t_k, 1u),
                 HID_ONE(true, C::TM_S2, big(ib3), t_q, 1u, 0),
                 if (NB > 1) HID_ONE(true, C::TM_S2, big(ib3), t_q, 1u, NB - 1))
      wait_mma();
      // ---- E6: dK = sum over the cluster of (share of dK + gZ1in W1^T): an output only, summed by
      // reduce-scatter; every CTA stores the token rows it owns.  Sent now, received inside the first MMA
      // window of the next step (or right after the group's last step).
      {
        float acc[16];
        tok_ld(tm, tmem + C::TM_A, acc);
#pragma unroll
        for (int q = 0; q < 16; ++q) dk_pend[q] = kp[q] + acc[q];
        if constexpr (C::kRowSplit) dk_tag = rs.send(dk_pend, tid, warp, lane);
        else dk_tag = csum.reduce_scatter_send(dk_pend, tid);
        dk_row0 = row0;
      }
      aborted = publish_vote();
      // pre-update weights of this mini-batch are the post-update weights of the previous one
      {
        const int n0 = ib4, n1 = ib1, n2 = ib0, n3 = ib2, n4 = ib3;
        ib0 = n0; ib1 = n1; ib2 = n2; ib3 = n3; ib4 = n4;
      }
      if (tid == kProd && j > 0 && !aborted) issue_rest(j - 1);
      if (aborted) break;
    }
    if (aborted) break;
    if constexpr (C::kRowSplit) {      // the group's last dK
      if (dk_row0 >= 0) finish_dk_rows();
    } else {
      if (dk_row0 >= 0 && csum.reduce_scatter_recv(dk_pend, tid, dk_tag))
        tok_st_global(tm, p.dXK + static_cast<long>(dk_row0) * 64, dk_pend);
    }
    if (tid == kProd) tma_wait_group_read<0>();   // the last dV has left its tile (the recompute writes it again)

    // ---- park the gradient state (tensor memory -> grad_L_W*_init); the last group leaves the result
    __syncwarp();
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float w[16];
      tok_ld(tm, tmem + C::TM_S1 + b * 64, w);
      store_w1_frag(Gdst_W1, b, w);
      tok_ld(tm, tmem + C::TM_S2 + b * 64, w);
      store_w2_frag(Gdst_W2, b, w);
    }
    Gsrc_W1 = Gdst_W1;
    Gsrc_W2 = Gdst_W2;
    publish();
  }
#undef TTT_ISSUE4
#undef HID_ALL
#undef HID_ONE

  // ---- final vector outputs
  if (!aborted) {
    if (row_writer) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        p.gb1[sid * 256 + hid0 + 64 * b + tm.r0] = Gb1[b][0];
        p.gb1[sid * 256 + hid0 + 64 * b + tm.r1] = Gb1[b][1];
      }
    }
    if constexpr (C::kRowSplit) {
      // d_gamma / d_beta: the replicated addends (output LayerNorm) plus every CTA's own-row addends, summed by
      // rank 0 in rank order.  The peers' addends ([kC][2][64]) land in the exchange buffer after next: the last
      // sum that used it was received by every CTA before the last-but-one was sent.
      float* sFin = reinterpret_cast<float*>(rs.bufp + ((rs.n + 1u) & 3u) * C::RS::kBufBytes);
      if (rank == 0) {
        if (tid == 0) mbar_expect_tx(&bars[BAR_AG], (kC - 1) * 512u);
      } else if (tid < 32) {
        const float4 v = reinterpret_cast<const float4*>(sDGp)[tid];
        st_async_f4(mapa(smem_u32(sFin + rank * 128 + tid * 4), 0), mapa(smem_u32(&bars[BAR_AG]), 0), v.x, v.y, v.z, v.w);
      }
      if (rank == 0) {
        wait_bar(BAR_AG);
        if (tid < 64) {
          float dg = sDG[tid] + sDGp[tid], db = sDB[tid] + sDGp[64 + tid];
#pragma unroll
          for (int r = 1; r < kC; ++r) {
            dg += sFin[r * 128 + tid];
            db += sFin[r * 128 + 64 + tid];
          }
          p.gb2[sid * 64 + tid] = sGb2[tid];
          p.d_gamma[sid * 64 + tid] = dg;
          p.d_beta[sid * 64 + tid] = db;
        }
      }
    } else if (rank == 0 && tid < 64) {
      p.gb2[sid * 64 + tid] = sGb2[tid];
      p.d_gamma[sid * 64 + tid] = sDG[tid];
      p.d_beta[sid * 64 + tid] = sDB[tid];
    }
  }
  if (tid == kProd) tma_wait_group<0>();
  if (aborted) {
    // everything this CTA still has in flight is waited for (bounded, not cut short by the abort flag)
    // before its shared and tensor memory go away: the tensor-core work of the four issuers ...
    if (warp < 4) {
      if (elect_one()) umma_commit(&bars[BAR_DRAIN]);
      __syncwarp();
    }
    if (tid == kProd) {
      mbar_wait_bounded(&bars[BAR_DRAIN], 0, never_flag, limit);
      // ... and its own loads
      for (int b = 0; b < 16; ++b)
        if (pending & (1u << b)) mbar_wait_bounded(&bars[b], (ph >> b) & 1u, never_flag, limit);
      atomicExch(p.status, static_cast<uint32_t>(TTT_B200_ERR_TIMEOUT));
    }
  }
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
    attr_err[dev] = cudaFuncSetAttribute(ttt_bwd_cluster_kernel<kC>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
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
    if (cudaOccupancyMaxActiveClusters(&n, ttt_bwd_cluster_kernel<kC>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cap[dev] = n;
  });
  return cap[dev];
}

template <int kC>
int launch_cluster(const CUtensorMap* tm, const BwdClParams& p, int streams, cudaStream_t stream) {
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, ttt_bwd_cluster_kernel<kC>, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6], p);
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}

}  // namespace

int ttt_launch_backward_cluster(const ttt_b200_bwd_args* a, int cluster, cudaStream_t stream, uint32_t* status,
                                uint64_t limit_ns, int drop_load) {
  const uint64_t rows = static_cast<uint64_t>(a->B) * a->H * a->NC * 64;
  CUtensorMap tm[7];
  const void* bases[7] = {a->XQ, a->XK, a->XV, a->grad_L_XQW_mini_batch, a->grad_L_XQ, a->grad_L_XK, a->grad_L_XV};
  for (int i = 0; i < 7; ++i)
    if (int rc = ttt_make_tile_map(&tm[i], bases[i], rows)) return rc;
  BwdClParams p;
  p.eta = static_cast<const __nv_bfloat16*>(a->last_eta);
  p.gamma = a->ttt_norm_weight;
  p.beta = a->ttt_norm_bias;
  p.W1c = a->W1_checkpoints; p.b1c = a->b1_checkpoints; p.W2c = a->W2_checkpoints; p.b2c = a->b2_checkpoints;
  p.sc_W1 = reinterpret_cast<uint8_t*>(a->W1_init_group);
  p.sc_W2 = reinterpret_cast<uint8_t*>(a->W2_init_group);
  p.sc_Z1 = static_cast<uint8_t*>(a->Z1_group);
  p.sc_X2 = static_cast<uint8_t*>(a->X2_group);
  p.sc_gZ1 = static_cast<uint8_t*>(a->grad_l_wrt_Z1_group);
  p.sc_Z1b = static_cast<uint8_t*>(a->Z1_bar_group);
  p.sc_X2b = static_cast<uint8_t*>(a->X2_bar_group);
  p.sc_xhf = static_cast<uint8_t*>(a->x_hat_fused_group);
  p.sc_gZ2 = static_cast<uint8_t*>(a->grad_l_wrt_Z2_group);
  p.sc_xhln = static_cast<uint8_t*>(a->x_hat_ln_group);
  p.sc_sigf = a->std_fused_group;
  p.sc_sigln = a->std_ln_group;
  p.gW1_last = a->grad_L_W1_last; p.gb1_last = a->grad_L_b1_last;
  p.gW2_last = a->grad_L_W2_last; p.gb2_last = a->grad_L_b2_last;
  p.d_gamma = a->grad_L_ttt_norm_weight; p.d_beta = a->grad_L_ttt_norm_bias;
  p.gW1 = a->grad_L_W1_init; p.gb1 = a->grad_L_b1_init; p.gW2 = a->grad_L_W2_init; p.gb2 = a->grad_L_b2_init;
  p.d_eta = static_cast<__nv_bfloat16*>(a->grad_L_last_eta);
  p.dXQ = static_cast<__nv_bfloat16*>(a->grad_L_XQ);
  p.dXK = static_cast<__nv_bfloat16*>(a->grad_L_XK);
  p.dXV = static_cast<__nv_bfloat16*>(a->grad_L_XV);
  p.H = a->H; p.NC = a->NC; p.cgs = a->checkpoint_group_size; p.nck = a->num_checkpoints;
  p.drop_load = drop_load;
  p.status = status;
  p.wait_limit_ns = limit_ns;
  const int streams = a->B * a->H;
  if (cluster == 2) return launch_cluster<2>(tm, p, streams, stream);
  if (cluster == 4) return launch_cluster<4>(tm, p, streams, stream);
  return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "cluster size must be 2 or 4");
}

int ttt_backward_cluster_capacity(int cluster) {
  return cluster == 2 ? cluster_capacity<2>() : cluster == 4 ? cluster_capacity<4>() : 0;
}
