// Thread-block-cluster layer of the cluster-sharded TTT-MLP kernels: the 256 hidden units of one
// (batch, head) stream are split over the kC CTAs of a cluster (kC = 2 or 4), and every
// contraction over the hidden units leaves each CTA with a partial 64 x 64 fp32 tile that is summed
// across the cluster through distributed shared memory.
//
// Replaces the reference's tp_reduce / tp_reduce_arrive (kernels/ttt_backward/ttt.cu:21-69) and the
// forward's Z2 reduction (kernels/ttt/ttt.cu:332-348, 506-522), which exchange bf16 tiles between
// hardware cluster barriers.  Here the partial tiles travel in fp32, straight from the registers of
// the thread that read them out of tensor memory into the peers' shared memory as asynchronous stores
// (st.async) that complete a transaction count on the receiver's mbarrier: data and signal travel
// together, nobody waits for an acknowledgement (plain remote stores followed by a release-arrive
// cost a further round trip over the SM-to-SM network: measured 0.3 us per exchange).  The receiver
// arms its mbarrier with the byte count it expects and polls it with a bounded try_wait.  The hardware
// cluster barrier, which cannot time out, is used only after the mbarriers are initialised and before
// the CTAs exit.
#pragma once

#include "ttt_device.cuh"

namespace tttcl {

using namespace tttdev;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cta address -> shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// arrive on an mbarrier of another CTA of the cluster; orders this thread's earlier stores (and, after
// a __syncwarp, its warp's) before the arrival
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Bounded wait of the cluster kernels.  A thread whose wait runs out raises the abort flag of its own
// CTA and of every peer (the flag lives at the same shared-memory offset in all of them), so that the
// whole cluster leaves its waits within a few polls and walks to the exit barrier together.
static __device__ __noinline__ bool mbar_wait_slow_cl(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                      uint64_t limit_ns, uint32_t cluster_size) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        const uint32_t a = smem_u32(const_cast<uint32_t*>(abort_flag));
        for (uint32_t r = 0; r < cluster_size; ++r) st_cluster_u32(mapa(a, r), 1u);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_cl(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             uint64_t limit_ns, uint32_t cluster_size) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  return mbar_wait_slow_cl(bar, parity, abort_flag, limit_ns, cluster_size);
}

// tcgen05.st counterpart of tmem_ld_16x256b_x4 (same thread <-> element mapping)
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tok_st_tmem(const TokMap& m, uint32_t tmem_acc, const float (&v)[16]) {
  uint32_t u[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) u[i] = __float_as_uint(v[i]);
  tmem_st_16x256b_x4(tmem_acc + m.taddr, u);
}

// ---- MMA forms of the cluster kernels.  A CTA owns R = 256 / kC hidden units, kept as NB = R / 64
// blocks of 64 rows: every accumulator is an M = 64 tile (row r in TMEM lane r % 16 + 32 (r / 16)) read
// back with the 16x256b fragments of TokMap, whether its rows are hidden units or tokens.
//
// "Hidden-major" block product: D[64 hid x 64] (+)= A * B with A one [64][64] bf16 block read K-major
// (row = hidden unit) and B a [64][64] tile read K-major (row = N index) or MN-major (row = K index).
template <bool kBMn>
__device__ __forceinline__ void mma_hid64(uint32_t tmem_d, uint32_t a_smem, uint32_t b_smem, uint32_t accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(64, 64, false, kBMn, false);
  const uint32_t a0 = desc_lo(a_smem, 16);
  const uint32_t b0 = desc_lo(b_smem, kBMn ? 8192 : 16);
  constexpr uint32_t bstep = kBMn ? (2048u >> 4) : (32u >> 4);
  mma_issue_rt(tmem_d, a0, b0, idesc, accumulate);
#pragma unroll
  for (int j = 1; j < 4; ++j) mma_issue_rt(tmem_d, a0 + j * 2, b0 + j * bstep, idesc, 1u);
}
// Partial "token-major" product over this CTA's hidden units: D[64 tok x 64] = X[64 x R] * W[R x 64], both
// operands [R][64] tiles read MN-major (row = hidden unit), R = 64 nblk.
__device__ __forceinline__ void mma_tok_partial(uint32_t tmem_d, uint32_t x_smem, uint32_t w_smem, int nblk) {
  constexpr uint32_t idesc = umma_idesc_bf16(64, 64, true, true, false);
  const uint32_t a0 = desc_lo(x_smem, TILE);
  const uint32_t b0 = desc_lo(w_smem, TILE);
  mma_issue_rt(tmem_d, a0, b0, idesc, 0u);
#pragma unroll 1
  for (int j = 1; j < 4 * nblk; ++j) mma_issue_rt(tmem_d, a0 + j * (2048u >> 4), b0 + j * (2048u >> 4), idesc, 1u);
}

// Column sums of a [64 tok][64] bf16 tile on the (otherwise idle) tensor pipe: D[64 feat x 8] = T^T * ones, the
// tile read MN-major (row = token = contraction index) against 8 rows of bf16 ones (1 KB, 1024-byte aligned,
// read K-major); every one of the 8 columns of D holds the sums.  Read back with colsum_read by warps 0..3.
__device__ __forceinline__ void mma_colsum(uint32_t tmem_d, uint32_t tile_smem, uint32_t ones_smem) {
  constexpr uint32_t idesc = umma_idesc_bf16(64, 8, true, false, false);
  const uint32_t a0 = desc_lo(tile_smem, TILE);
  const uint32_t b0 = desc_lo(ones_smem, 16);
  mma_issue_rt(tmem_d, a0, b0, idesc, 0u);
#pragma unroll
  for (int j = 1; j < 4; ++j) mma_issue_rt(tmem_d, a0 + j * (2048u >> 4), b0 + j * (32u >> 4), idesc, 1u);
}
// Warp q of warps 0..3 (all 32 lanes call): lanes 0..15 return the sum of column 16 q + lane (row r of an M = 64
// accumulator sits in tensor-memory lane r % 16 + 32 (r / 16)); the other lanes return garbage.
__device__ __forceinline__ float colsum_read(uint32_t tmem_d, int warp) {
  uint32_t v[8];
  tmem_ld8(tmem_d + (static_cast<uint32_t>(warp * 32) << 16), v);
  tmem_wait_ld();
  return __uint_as_float(v[0]);
}

// the thread's 16 values of a token-major fragment, rounded to bf16, straight to a row-major [64][64] bf16
// tile in global memory (`tile` = its first element): used by the CTA that owns the rows after a
// reduce-scatter, where only a quarter or half of the tile is this CTA's to store
__device__ __forceinline__ void tok_st_global(const TokMap& m, __nv_bfloat16* tile, const float (&v)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = m.col(j);
    *reinterpret_cast<uint32_t*>(tile + m.r0 * 64 + c) = pack_bf16(v[4 * j], v[4 * j + 1]);
    *reinterpret_cast<uint32_t*>(tile + m.r1 * 64 + c) = pack_bf16(v[4 * j + 2], v[4 * j + 3]);
  }
}

// ---- Sum of a partial 64 x 64 fp32 tile (the TokMap fragment: 16 values per thread, optionally with
// two further per-thread values) over the CTAs of the cluster.  Every CTA ends with the same bits: the
// additions are arranged as a butterfly over the rank bits, (own + [rank^1]) + ([rank^2] + [rank^3]),
// which is the same expression in every CTA up to the commutativity of each addition.
//
// Exchange area per CTA: 2 buffers x (kC - 1) slots (slot s holds the values of rank ^ (s + 1)) of
// kSlotBytes each: 256 x 4 float4 for the tile, then 256 x float2 for the extra values when a kernel
// uses them (kSlotBytes = 16384 or 18432); one mbarrier per buffer counting (kC - 1) x 8 arrivals (one
// per warp and peer).  Successive reductions alternate between the buffers.  That is enough: a CTA
// sends reduction n + 2 only after it has received reduction n + 1 from every warp of every peer, and
// a peer's warp sends n + 1 only after it has read its part of buffer n.
// asynchronous remote stores: the bytes are counted on the mbarrier `bar` (a shared::cluster address in
// the same CTA as `addr`) when they have landed
__device__ __forceinline__ void st_async_f4(uint32_t addr, uint32_t bar, float a, float b, float c, float d) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%2, %3, %4, %5}, [%1];" ::"r"(addr),
               "r"(bar), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void st_async_f1(uint32_t cluster_addr, uint32_t cluster_bar, float a) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %2, [%1];" ::"r"(cluster_addr),
               "r"(cluster_bar), "f"(a)
               : "memory");
}
__device__ __forceinline__ void st_async_f2(uint32_t addr, uint32_t bar, float a, float b) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%2, %3}, [%1];" ::"r"(addr),
               "r"(bar), "f"(a), "f"(b)
               : "memory");
}
template <int kC, uint32_t kSlotBytes_>
struct ClusterSum {
  uint8_t* bufp;         // the exchange area (this CTA's shared memory)
  uint64_t* bars;        // [2], initialised with count 1 (the arming arrival of this CTA's thread 0)
  uint32_t n;            // reductions done
  uint32_t rank;
  volatile uint32_t* abort_flag;
  uint64_t limit;

  static constexpr uint32_t kSlotBytes = kSlotBytes_;
  static constexpr uint32_t kBufBytes = (kC - 1) * kSlotBytes;
  static constexpr uint32_t kBytes = 2 * kBufBytes;
  static constexpr uint32_t kArrivals = 1;
  static_assert(kSlotBytes == 16384 || kSlotBytes == 18432, "slot = tile, or tile + extras");

  // v: the thread's 16 tile values; e0, e1: its two extra values (kExtra).  Returns with all of them
  // summed over the cluster.
  //
  // Order on one buffer: this CTA arms phase k of barrier b (reduction n = 2 k + b) after it has left
  // the wait of reduction n - 2 in program order, and a peer's bytes for reduction n can only be sent
  // after that peer has received this CTA's reduction n - 1, which every thread sends after its own wait
  // of n - 2: no byte of phase k is counted on phase k - 1.  Bytes that arrive before the arming only
  // take the transaction count below zero for a moment.
  template <bool kExtra>
  __device__ __forceinline__ void run_impl(float (&v)[16], float& e0, float& e1, int tid, int lane) {
    static_assert(!kExtra || kSlotBytes == 18432, "the exchange area has no room for extra values");
    const uint32_t b = n & 1u, par = (n >> 1) & 1u;
    ++n;
    const uint32_t boff = b * kBufBytes + static_cast<uint32_t>(tid) * 16u;
    const uint32_t eoff = b * kBufBytes + 16384u + static_cast<uint32_t>(tid) * 8u;
    const uint32_t base = smem_u32(bufp);
    const uint32_t ba = smem_u32(&bars[b]);
    if (tid == 0) mbar_expect_tx(&bars[b], (kC - 1) * (kExtra ? 18432u : 16384u));
#pragma unroll
    for (int s = 0; s < kC - 1; ++s) {
      const uint32_t peer = rank ^ static_cast<uint32_t>(s + 1);
      // at the peer, this CTA is rank ^ (s + 1) as well: the slot index is the same on both sides
      const uint32_t dst = mapa(base + boff + s * kSlotBytes, peer);
      const uint32_t rbar = mapa(ba, peer);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st_async_f4(dst + j * 4096u, rbar, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      if constexpr (kExtra) st_async_f2(mapa(base + eoff + s * kSlotBytes, peer), rbar, e0, e1);
    }
    mbar_wait_cl(&bars[b], par, abort_flag, limit, kC);
    const float4* src = reinterpret_cast<const float4*>(bufp + boff);
    const float2* esrc = reinterpret_cast<const float2*>(bufp + eoff);
    if constexpr (kC == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p = src[j * 256];
        v[4 * j] += p.x; v[4 * j + 1] += p.y; v[4 * j + 2] += p.z; v[4 * j + 3] += p.w;
      }
      if constexpr (kExtra) {
        const float2 q = esrc[0];
        e0 += q.x; e1 += q.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p1 = src[j * 256];
        const float4 p2 = src[(kSlotBytes / 16) + j * 256];
        const float4 p3 = src[2 * (kSlotBytes / 16) + j * 256];
        v[4 * j] = (v[4 * j] + p1.x) + (p2.x + p3.x);
        v[4 * j + 1] = (v[4 * j + 1] + p1.y) + (p2.y + p3.y);
        v[4 * j + 2] = (v[4 * j + 2] + p1.z) + (p2.z + p3.z);
        v[4 * j + 3] = (v[4 * j + 3] + p1.w) + (p2.w + p3.w);
      }
      if constexpr (kExtra) {
        const float2 q1 = esrc[0], q2 = esrc[kSlotBytes / 8], q3 = esrc[2 * (kSlotBytes / 8)];
        e0 = (e0 + q1.x) + (q2.x + q3.x);
        e1 = (e1 + q1.y) + (q2.y + q3.y);
      }
    }
  }
  __device__ __forceinline__ void run(float (&v)[16], int tid, int lane) {
    float d0 = 0.f, d1 = 0.f;
    run_impl<false>(v, d0, d1, tid, lane);
  }

  // The same sum, delivered only where it is needed when a tile is an output and not an operand of
  // later steps: the token rows of the tile are dealt out to the CTAs of the cluster (the rows of
  // fragment quadrant q = warp % 4, i.e. tokens 16 q .. 16 q + 15, belong to CTA q kC / 4), every thread
  // sends its 16 values to the owner of its rows only, and the owner's threads add what arrives.  A CTA
  // sends (kC - 1) / kC of a tile instead of kC - 1 tiles: the exchange is bound by the bytes that cross
  // the SM-to-SM network.  Uses the same buffers, barriers and reduction counter as run().
  // Returns true in the threads that now hold finished rows.
  static __device__ __forceinline__ uint32_t row_owner(int tid) { return (static_cast<uint32_t>(tid >> 5) & 3u) * kC / 4u; }
  // The two halves may be separated by other work (the result of such a sum is only stored): the send
  // right after the partial tile has been read, the receive inside a later MMA window.  `tag` carries
  // the buffer and parity from one to the other.  No other reduction may start in between (the buffers
  // alternate per reduction).
  __device__ __forceinline__ uint32_t reduce_scatter_send(const float (&v)[16], int tid) {
    const uint32_t b = n & 1u, par = (n >> 1) & 1u;
    ++n;
    const uint32_t boff = b * kBufBytes + static_cast<uint32_t>(tid) * 16u;
    const uint32_t owner = row_owner(tid);
    if (tid == 0) mbar_expect_tx(&bars[b], (kC - 1) * (16384u / kC));
    if (owner != rank) {
      const uint32_t s = (rank ^ owner) - 1u;
      const uint32_t dst = mapa(smem_u32(bufp) + boff + s * kSlotBytes, owner);
      const uint32_t rbar = mapa(smem_u32(&bars[b]), owner);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st_async_f4(dst + j * 4096u, rbar, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    return b | (par << 1);
  }
  __device__ __forceinline__ bool reduce_scatter_recv(float (&v)[16], int tid, uint32_t tag) {
    const uint32_t b = tag & 1u, par = tag >> 1;
    const uint32_t boff = b * kBufBytes + static_cast<uint32_t>(tid) * 16u;
    mbar_wait_cl(&bars[b], par, abort_flag, limit, kC);
    if (row_owner(tid) != rank) return false;
    const float4* src = reinterpret_cast<const float4*>(bufp + boff);
    if constexpr (kC == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p = src[j * 256];
        v[4 * j] += p.x; v[4 * j + 1] += p.y; v[4 * j + 2] += p.z; v[4 * j + 3] += p.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p1 = src[j * 256];
        const float4 p2 = src[(kSlotBytes / 16) + j * 256];
        const float4 p3 = src[2 * (kSlotBytes / 16) + j * 256];
        v[4 * j] = (v[4 * j] + p1.x) + (p2.x + p3.x);
        v[4 * j + 1] = (v[4 * j + 1] + p1.y) + (p2.y + p3.y);
        v[4 * j + 2] = (v[4 * j + 2] + p1.z) + (p2.z + p3.z);
        v[4 * j + 3] = (v[4 * j + 3] + p1.w) + (p2.w + p3.w);
      }
    }
    return true;
  }
  __device__ __forceinline__ bool reduce_scatter(float (&v)[16], int tid) {
    const uint32_t tag = reduce_scatter_send(v, tid);
    return reduce_scatter_recv(v, tid, tag);
  }
  __device__ __forceinline__ void run_with_extras(float (&v)[16], float& e0, float& e1, int tid, int lane) {
    run_impl<true>(v, e0, e1, tid, lane);
  }
  // run() in two halves, for a sum whose result nothing on the critical path waits for (same rules as
  // the halves of reduce_scatter)
  __device__ __forceinline__ uint32_t allreduce_send(const float (&v)[16], int tid) {
    const uint32_t b = n & 1u, par = (n >> 1) & 1u;
    ++n;
    const uint32_t boff = b * kBufBytes + static_cast<uint32_t>(tid) * 16u;
    if (tid == 0) mbar_expect_tx(&bars[b], (kC - 1) * 16384u);
#pragma unroll
    for (int s = 0; s < kC - 1; ++s) {
      const uint32_t peer = rank ^ static_cast<uint32_t>(s + 1);
      const uint32_t dst = mapa(smem_u32(bufp) + boff + s * kSlotBytes, peer);
      const uint32_t rbar = mapa(smem_u32(&bars[b]), peer);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st_async_f4(dst + j * 4096u, rbar, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    return b | (par << 1);
  }
  __device__ __forceinline__ void allreduce_recv(float (&v)[16], int tid, uint32_t tag) {
    const uint32_t b = tag & 1u, par = tag >> 1;
    const uint32_t boff = b * kBufBytes + static_cast<uint32_t>(tid) * 16u;
    mbar_wait_cl(&bars[b], par, abort_flag, limit, kC);
    const float4* src = reinterpret_cast<const float4*>(bufp + boff);
    if constexpr (kC == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p = src[j * 256];
        v[4 * j] += p.x; v[4 * j + 1] += p.y; v[4 * j + 2] += p.z; v[4 * j + 3] += p.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 p1 = src[j * 256];
        const float4 p2 = src[(kSlotBytes / 16) + j * 256];
        const float4 p3 = src[2 * (kSlotBytes / 16) + j * 256];
        v[4 * j] = (v[4 * j] + p1.x) + (p2.x + p3.x);
        v[4 * j + 1] = (v[4 * j + 1] + p1.y) + (p2.y + p3.y);
        v[4 * j + 2] = (v[4 * j + 2] + p1.z) + (p2.z + p3.z);
        v[4 * j + 3] = (v[4 * j + 3] + p1.w) + (p2.w + p3.w);
      }
    }
  }
};

// ---- Row-split stages.  A 64 x 64 stage that follows a contraction over the hidden units (the fused
// LayerNorm, the output LayerNorm) does not have to be repeated by every CTA of the cluster on the whole
// tile: the token rows are dealt out (CTA r owns the rows of fragment quadrants QPC r .. QPC r + QPC - 1,
// QPC = 4 / kC, i.e. rows 64 r / kC .. 64 (r + 1) / kC - 1), the partial tiles are summed by reduce-scatter,
// every CTA runs the stage on its own rows with ALL of its 256 threads, and the bf16 results that the
// other CTAs need as MMA operands are written into the peers' shared memories as well (all-gather).
// Against an all-reduce followed by the stage on the whole tile in every CTA this sends (kC - 1) / kC of a
// tile in fp32 plus the bf16 rows instead of kC - 1 tiles, and does 1 / kC of the arithmetic per CTA.
//
// Reduce-scatter buffers: kBufs = 4 (taken in turn per use) x kC slots (slot s = the partial of rank s, this
// CTA's own included).  A slot holds the owner's rows as [quadrant lq][row pair w = 0..7][column pair
// 0..31] float4 = {(r, c), (r, c+1), (r+8, c), (r+8, c+1)}, r = 16 (QPC rank + lq) + w, c = 2 x column pair:
// the float4 a fragment thread holds for j = 0..3, so the sender stores 16 bytes at a time, and one row
// pair is 512 contiguous bytes, so the 32 lanes of the warp that works on it read them without bank
// conflicts (an earlier layout indexed by sending thread cost 0.5 us per receive in 8-way conflicts).
// One mbarrier per buffer: the arming arrival of thread 0 (expect_tx of the peers' bytes) plus one arrival
// per warp that wrote this CTA's own partial with plain stores.  Four buffers, because a kernel may send
// use n + 1 before it receives use n (it receives a deferred sum while it waits for the next one): a peer
// writes use n + 4 into the buffer of use n only after it has received n + 3 from this CTA, which this CTA
// sends after its receive of n in program order.
//
// Row layout of the stage: warp w works on row pair w of each of the CTA's QPC quadrants, lane l on the
// column pair l: NR = 2 QPC rows x 2 columns per thread; a row lives in one warp, so row sums are five
// xor-shuffles.
// kExtras: a second, smaller exchange area (two alternating buffers of one slot per CTA) takes two extra per-row
// values from each of the 8 fragment threads that share a row pair ([quadrant][row pair][colhalf x 4 + lane % 4]
// float2), which send_x / recv_x sum over the contributors as well: per-row scalars that are linear in the
// partial tiles travel with them, counted on the same mbarrier.  Two buffers are enough when sums with extras
// are separated by other sums, as they are here (one per reverse step).
template <int kC, bool kExtras = false>
struct RowSplit {
  static constexpr int QPC = 4 / kC;                          // fragment quadrants per CTA
  static constexpr int ROWS = 16 * QPC;
  static constexpr int NR = 2 * QPC;                          // rows per thread in the row layout
  static constexpr uint32_t kTileBytes = QPC * 4096u;
  static constexpr uint32_t kSlotBytes = kTileBytes;
  static constexpr uint32_t kBufBytes = kC * kSlotBytes;      // 16 KB
  static constexpr int kBufs = 4;
  static constexpr uint32_t kXSlotBytes = QPC * 512u;
  static constexpr uint32_t kXBufBytes = kC * kXSlotBytes;
  static constexpr uint32_t kBytes = kBufs * kBufBytes + (kExtras ? 2 * kXBufBytes : 0u);   // tiles, then extras
  static constexpr uint32_t kBarCount = 1 + 2 * QPC;          // arming thread + the warps of the own quadrants

  uint8_t* bufp;
  uint64_t* bars;        // [kBufs]
  uint32_t n;
  uint32_t nx = 0;       // sums with extras so far
  uint32_t rank;
  volatile uint32_t* abort_flag;
  uint64_t limit;

  // ---- fragment side (TokMap layout)
  static __device__ __forceinline__ uint32_t owner_of(int warp) { return static_cast<uint32_t>(warp & 3) / QPC; }
  // Send this thread's 16 partial values to the owner of its rows (or file them in this CTA's own slot).
  // Returns the tag for recv().
  template <bool kX>
  __device__ __forceinline__ uint32_t send_impl(const float (&v)[16], float e0, float e1, int tid, int warp, int lane) {
    static_assert(!kX || kExtras, "this exchange area has no room for extra values");
    const uint32_t b = n & 3u, par = (n >> 2) & 1u;
    ++n;
    const uint32_t xb = nx & 1u;
    if constexpr (kX) ++nx;
    const uint32_t owner = owner_of(warp);
    const uint32_t lq = static_cast<uint32_t>(warp & 3) % QPC, colhalf = static_cast<uint32_t>(warp >> 2);
    const uint32_t slot = b * kBufBytes + rank * kSlotBytes;
    const uint32_t off = slot + lq * 4096u + static_cast<uint32_t>(lane >> 2) * 512u +
                         (colhalf * 16u + static_cast<uint32_t>(lane & 3)) * 16u;
    const uint32_t xoff = kBufs * kBufBytes + xb * kXBufBytes + rank * kXSlotBytes + lq * 512u +
                          static_cast<uint32_t>(lane >> 2) * 64u + (colhalf * 4u + static_cast<uint32_t>(lane & 3)) * 8u;
    if (tid == 0) mbar_expect_tx(&bars[b], (kC - 1) * (kTileBytes + (kX ? kXSlotBytes : 0u)));
    if (owner != rank) {
      const uint32_t dst = mapa(smem_u32(bufp) + off, owner);
      const uint32_t rbar = mapa(smem_u32(&bars[b]), owner);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st_async_f4(dst + j * 64u, rbar, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      if constexpr (kX) st_async_f2(mapa(smem_u32(bufp) + xoff, owner), rbar, e0, e1);
    } else {
      float4* dst = reinterpret_cast<float4*>(bufp + off);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[j * 4] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      if constexpr (kX) *reinterpret_cast<float2*>(bufp + xoff) = make_float2(e0, e1);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[b]);
    }
    return b | (par << 2) | (xb << 3);
  }
  __device__ __forceinline__ uint32_t send(const float (&v)[16], int tid, int warp, int lane) {
    return send_impl<false>(v, 0.f, 0.f, tid, warp, lane);
  }
  // e0 / e1: this thread's contributions to the extra value of its rows r0 / r1
  __device__ __forceinline__ uint32_t send_x(const float (&v)[16], float e0, float e1, int tid, int warp, int lane) {
    return send_impl<true>(v, e0, e1, tid, warp, lane);
  }

  // ---- row side: row i of the thread (i = 2 lq + h) is token row 16 (QPC rank + lq) + warp + 8 h of the tile
  __device__ __forceinline__ int row(int i, int warp) const {
    return 16 * (QPC * static_cast<int>(rank) + (i >> 1)) + warp + 8 * (i & 1);
  }
  // Wait for the partial tiles and return their sums (rank order): z[i][0..1] = row i, columns 2 lane, 2 lane + 1.
  __device__ __forceinline__ void recv(float (&z)[NR][2], int warp, int lane, uint32_t tag) {
    const uint32_t b = tag & 3u, par = (tag >> 2) & 1u;
    mbar_wait_cl(&bars[b], par, abort_flag, limit, kC);
    const uint8_t* base = bufp + b * kBufBytes + static_cast<uint32_t>(warp) * 512u + static_cast<uint32_t>(lane) * 16u;
#pragma unroll
    for (int lq = 0; lq < QPC; ++lq) {
      float4 acc = *reinterpret_cast<const float4*>(base + lq * 4096u);
#pragma unroll
      for (int s = 1; s < kC; ++s) {
        const float4 f = *reinterpret_cast<const float4*>(base + s * kSlotBytes + lq * 4096u);
        acc.x += f.x; acc.y += f.y; acc.z += f.z; acc.w += f.w;
      }
      z[2 * lq][0] = acc.x; z[2 * lq][1] = acc.y;
      z[2 * lq + 1][0] = acc.z; z[2 * lq + 1][1] = acc.w;
    }
  }
  // recv() plus the extra values: e[i] = the sum over all CTAs and contributors for row i (all lanes get it)
  __device__ __forceinline__ void recv_x(float (&z)[NR][2], float (&e)[NR], int warp, int lane, uint32_t tag) {
    recv(z, warp, lane, tag);
    const uint32_t xb = (tag >> 3) & 1u;
    const uint8_t* base = bufp + kBufs * kBufBytes + xb * kXBufBytes + static_cast<uint32_t>(warp) * 64u +
                          static_cast<uint32_t>(lane & 7) * 8u;
#pragma unroll
    for (int lq = 0; lq < QPC; ++lq) {
      float2 acc = *reinterpret_cast<const float2*>(base + lq * 512u);
#pragma unroll
      for (int s = 1; s < kC; ++s) {
        const float2 f = *reinterpret_cast<const float2*>(base + s * kXSlotBytes + lq * 512u);
        acc.x += f.x; acc.y += f.y;
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {       // lanes 0..7 hold the eight contributors (the others repeat them)
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
      }
      e[2 * lq] = acc.x;
      e[2 * lq + 1] = acc.y;
    }
  }
  static __device__ __forceinline__ float row_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
  }
  // the thread's column pair of row r of a swizzled bf16 tile
  static __device__ __forceinline__ float2 ld_pair(const uint8_t* tile, int r, int lane) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(tile + sw128_off(r, lane >> 2) + (lane & 3) * 4);
    return make_float2(bf16_lo(w), bf16_hi(w));
  }
  static __device__ __forceinline__ void st_pair(uint8_t* tile, int r, int lane, float a, float b) {
    *reinterpret_cast<uint32_t*>(tile + sw128_off(r, lane >> 2) + (lane & 3) * 4) = pack_bf16(a, b);
  }
  static __device__ __forceinline__ void st_pair_global(__nv_bfloat16* tile, int r, int lane, float a, float b) {
    *reinterpret_cast<uint32_t*>(tile + r * 64 + 2 * lane) = pack_bf16(a, b);
  }

  // ---- all-gather of a stage's bf16 result: row r of `tile`, of which this thread holds the column pair
  // (a, b), is written into this CTA's tile and, as 16-byte asynchronous stores counted on the peers'
  // `ag_bar`, into the same place of every peer's tile (four neighbouring lanes make up one 16-byte chunk;
  // all 32 lanes call this).  The receiver waits on its `ag_bar` (armed by arm_all_gather) and runs the usual
  // proxy fence + CTA barrier before an MMA reads the tile.
  __device__ __forceinline__ void arm_all_gather(uint64_t* ag_bar, int ntiles, uint32_t extra_bytes = 0) const {
    mbar_expect_tx(ag_bar, (kC - 1) * (ROWS * 128u * static_cast<uint32_t>(ntiles) + extra_bytes));
  }
  // four fp32 values (16 bytes at `dst`, the same address in every CTA) to this CTA and every peer, counted on
  // the peers' `ag_bar` like the tiles of an all-gather
  __device__ __forceinline__ void all_gather_f4(float* dst, uint64_t* ag_bar, float a, float b, float c, float d) const {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
    const uint32_t adr = smem_u32(dst), ba = smem_u32(ag_bar);
#pragma unroll
    for (int s = 1; s < kC; ++s) {
      const uint32_t peer = rank ^ static_cast<uint32_t>(s);
      st_async_f4(mapa(adr, peer), mapa(ba, peer), a, b, c, d);
    }
  }
  __device__ __forceinline__ void all_gather_store(uint8_t* tile, uint64_t* ag_bar, int r, int lane, float a, float b) const {
    const uint32_t w0 = pack_bf16(a, b);
    const uint32_t w1 = __shfl_down_sync(0xffffffffu, w0, 1), w2 = __shfl_down_sync(0xffffffffu, w0, 2),
                   w3 = __shfl_down_sync(0xffffffffu, w0, 3);
    if ((lane & 3) == 0) {
      const uint32_t off = sw128_off(r, lane >> 2);
      *reinterpret_cast<uint4*>(tile + off) = make_uint4(w0, w1, w2, w3);
      const uint32_t adr = smem_u32(tile) + off, ba = smem_u32(ag_bar);
#pragma unroll
      for (int s = 1; s < kC; ++s) {
        const uint32_t peer = rank ^ static_cast<uint32_t>(s);
        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%2, %3, %4, %5}, [%1];" ::"r"(
                         mapa(adr, peer)),
                     "r"(mapa(ba, peer)), "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                     : "memory");
      }
    }
  }
};

// Exit of a cluster kernel (all threads of all CTAs call it).  On the ordinary path every byte a peer
// has sent to this CTA has been waited for, so one cluster barrier is enough before the shared memory
// goes away.  After an abort the CTAs may have skipped waits: all of them first meet (nobody sends any
// more), then let the asynchronous stores already under way land (they take well under a microsecond;
// 50 us are allowed), then meet again.  Whether the cluster aborted is read after the first barrier: a
// CTA raises the flag in every CTA of the cluster before it arrives there, so all of them read the same
// answer and run the same number of barriers.
__device__ __forceinline__ void cluster_exit(volatile uint32_t* abort_flag) {
  cluster_arrive();
  cluster_wait();
  if (__syncthreads_or(*abort_flag != 0)) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) {
    }
    cluster_arrive();
    cluster_wait();
  }
}

}  // namespace tttcl
