// Self-test of the tcgen05 building blocks the TTT-MLP kernels rely on: one CTA computes
// D[M x N] = (+/-) A[M x K] * B[N x K]^T (+ D) with bf16 operands written to shared memory in
// the 128-byte-swizzled layout by plain stores, in either operand majorness, and reads the
// fp32 result back from tensor memory.  The GPU tests compare it with a host matmul, which
// pins the shared-memory descriptors, the instruction descriptor and the TMEM lane mapping
// for M = 64 and M = 128 independently of the TTT kernels.
#include "sm100_ptx.cuh"
#include "ttt_internal.h"

using namespace sm100;

namespace {

struct ProbeParams {
  const float* A;   // [M][K] row-major
  const float* B;   // [N][K] row-major
  float* D;         // [M][N] row-major
  int M, N, K;      // M in {64,128}; N multiple of 16, <= 256; K multiple of 64, <= 256
  int a_mn, b_mn;   // operand stored MN-major (else K-major)
  int neg_a;        // use -A
  int repeat;       // run the product `repeat` times, accumulating
  int frag_ld;      // read the result back with the 16x256b fragment loads (M = 64 only)
  uint32_t* status;
};

__global__ void __launch_bounds__(128, 1) umma_probe_kernel(ProbeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int M = p.M, N = p.N, K = p.K;
  uint8_t* sA = smem;                                  // <= 128 x 256 bf16 = 64 KB
  uint8_t* sB = smem + 65536;                          // <= 256 x 256 bf16 = 128 KB

  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  // operand fill (element-wise; speed is irrelevant here)
  for (int i = tid; i < M * K; i += blockDim.x) {
    const int r = i / K, k = i % K;
    uint32_t tile, row, col;
    if (p.a_mn) { tile = (r / 64) * (K * 128); row = k; col = r % 64; }
    else        { tile = (k / 64) * (M * 128); row = r; col = k % 64; }
    *reinterpret_cast<__nv_bfloat16*>(sA + tile + sw128_off(row, col >> 3) + (col & 7) * 2) =
        __float2bfloat16(p.A[i]);
  }
  for (int i = tid; i < N * K; i += blockDim.x) {
    const int r = i / K, k = i % K;
    uint32_t tile, row, col;
    if (p.b_mn) { tile = (r / 64) * (K * 128); row = k; col = r % 64; }
    else        { tile = (k / 64) * (N * 128); row = r; col = k % 64; }
    *reinterpret_cast<__nv_bfloat16*>(sB + tile + sw128_off(row, col >> 3) + (col & 7) * 2) =
        __float2bfloat16(p.B[i]);
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;

  if (tid == 0) {
    const uint32_t idesc = umma_idesc_bf16(M, N, p.a_mn != 0, p.b_mn != 0, p.neg_a != 0);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
    for (int rep = 0; rep < p.repeat; ++rep) {
      for (int j = 0; j < K / 16; ++j) {
        const uint32_t aoff = p.a_mn ? j * 2048 : (j / 4) * (M * 128) + (j % 4) * 32;
        const uint32_t boff = p.b_mn ? j * 2048 : (j / 4) * (N * 128) + (j % 4) * 32;
        const uint64_t ad = umma_desc_sw128(a0 + aoff, p.a_mn ? K * 128 : 16);
        const uint64_t bd = umma_desc_sw128(b0 + boff, p.b_mn ? K * 128 : 16);
        umma_bf16_ss(tmem, ad, bd, idesc, (rep | j) ? 1u : 0u);
      }
    }
    umma_commit(&bar);
  }
  const bool ok = mbar_wait_bounded(&bar, 0, &abort_flag, 200ull * 1000 * 1000);
  tc_fence_after_sync();
  if (ok && p.frag_ld) {
    // 16x256b fragments of the M = 64 layout: rows 16*warp + lane/4 (+8), column pairs 8j + 2(lane%4)
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t v[16];
      tmem_ld_16x256b_x4(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      tmem_wait_ld();
      const int r0 = warp * 16 + (lane >> 2);
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + 8 * j + 2 * (lane & 3);
        if (c + 1 < N) {
          p.D[r0 * N + c] = __uint_as_float(v[4 * j]);
          p.D[r0 * N + c + 1] = __uint_as_float(v[4 * j + 1]);
          p.D[(r0 + 8) * N + c] = __uint_as_float(v[4 * j + 2]);
          p.D[(r0 + 8) * N + c + 1] = __uint_as_float(v[4 * j + 3]);
        }
      }
    }
  } else if (ok) {
    // M = 128: row = TMEM lane.  M = 64: row r sits in lane (r % 16) + 32 * (r / 16).
    const int row = (M == 128) ? tid : (lane < 16 ? warp * 16 + lane : -1);
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t v[32];
      tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      tmem_wait_ld();
      if (row >= 0)
        for (int j = 0; j < 32 && c0 + j < N; ++j) p.D[row * N + c0 + j] = __uint_as_float(v[j]);
    }
  } else if (tid == 0) {
    atomicExch(p.status, TTT_B200_ERR_TIMEOUT);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

extern "C" int ttt_b200_umma_selftest(const float* A, const float* B, float* D, int M, int N, int K, int a_mn,
                                      int b_mn, int neg_a, int repeat_and_mode, void* stream_) {
  // bits 0..7: repeat count; bit 8: read back through the 16x256b fragment loads (M = 64, N % 32 == 0)
  const int repeat = repeat_and_mode & 0xff;
  const int frag_ld = (repeat_and_mode >> 8) & 1;
  if (frag_ld && (M != 64 || (N % 32) != 0))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "umma_selftest: fragment read-back needs M = 64 and N % 32 == 0");
  // N: a multiple of 8 from 8 up with M = 64, a multiple of 16 from 16 up with M = 128
  if (!(M == 64 || M == 128) || N < (M == 64 ? 8 : 16) || N > 256 || (N % (M == 64 ? 8 : 16)) || K < 64 || K > 256 ||
      (K % 64) || repeat < 1)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "umma_selftest: unsupported shape");
  if ((a_mn && M > 128) || N * K * 2 > 131072)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "umma_selftest: operand too large");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = ttt_status_word(&status)) return rc;
  ProbeParams p{A, B, D, M, N, K, a_mn, b_mn, neg_a, repeat, frag_ld, status};
  const int smem = 65536 + 131072 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  umma_probe_kernel<<<1, 128, smem, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return ttt_check_status(stream);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the failure path: one CTA waits, with the kernels' own bounded wait, on a barrier
// that nothing ever arrives on.  The wait must run out after `limit_us`, the CTA must report
// through the status word and exit normally, and the context must stay usable.
namespace {
__global__ void wait_probe_kernel(uint32_t* status, uint64_t limit_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  __syncthreads();
  const uint64_t t0 = globaltimer_ns();
  const bool ok = mbar_wait_bounded(&bar, 0, &abort_flag, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0) {
    *waited_ns = globaltimer_ns() - t0;
    if (!ok) atomicExch(status, TTT_B200_ERR_TIMEOUT);
  }
}
}  // namespace

extern "C" int ttt_b200_wait_selftest(int limit_us, unsigned long long* waited_ns_host, void* stream_) {
  if (limit_us < 1 || limit_us > 1000000)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "wait_selftest: limit must be 1 us .. 1 s");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = ttt_status_word(&status)) return rc;
  unsigned long long* d_waited = nullptr;
  cudaError_t e = cudaMalloc(&d_waited, sizeof(unsigned long long));
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  wait_probe_kernel<<<1, 64, 0, stream>>>(status, static_cast<uint64_t>(limit_us) * 1000ull, d_waited);
  e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  unsigned long long waited = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&waited, d_waited, sizeof(waited), cudaMemcpyDeviceToHost);
  cudaFree(d_waited);
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  if (waited_ns_host) *waited_ns_host = waited;
  if (ttt_take_status() != 0)
    return ttt_set_error(TTT_B200_ERR_TIMEOUT, "a device-side bounded wait ran out; results are invalid");
  return TTT_B200_OK;
}
