// Layer-side kernels around the TTT-MLP operator: the learning-rate gate that produces `last_eta`,
// and the output LayerNorm that follows the operator, each fused with the layout change the operator's
// interface forces (a model's activations are token-major [B][T][H*64]; the operator wants contiguous
// head-major [B][H][T][..] tensors: README.md:98 of the reference).  The reference leaves all of this
// to its callers (README.md:22-98: the caller passes `last_eta` and receives `XQW_batch`); the
// statements these kernels must match are the torch expressions in oracle/glue.py.
//
//   eta gate       last_eta[b][h][t] = scale * sigmoid(logit[b][t][h])             bf16 in, bf16 out
//   its backward   d_logit[b][t][h]  = d_last_eta[b][h][t] * scale * s (1 - s)
//   output norm    y[b][t][:] = gamma * LayerNorm_{H*64}(x[b][:][t][:]) + beta     x = Out [B][H][T][64] bf16
//   its backward   dx (head-major: the operator's grad_L_XQW_mini_batch), d_gamma, d_beta from dy (token-major)
//
// All of them are HBM-bound byte movers with a little fp32 arithmetic: algorithmic bytes = input + output.
#include <cuda_bf16.h>

#include <cstdio>

#include "ttt_internal.h"

namespace {

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.f / (1.f + __expf(-x)); }

// ---- eta gate.  One CTA per (b, block of 64 tokens): the [64 tok][H] block of the logits is one
// contiguous run of 128 H bytes; it is turned through shared memory and leaves as H runs of 128 bytes
// (64 tokens of one head).  kBackward: `other` is d_last_eta [B][H][T] and the result d_logit [B][T][H].
template <bool kBackward>
__global__ void __launch_bounds__(256) eta_gate_kernel(const __nv_bfloat16* __restrict__ logits,
                                                       const __nv_bfloat16* __restrict__ other,
                                                       __nv_bfloat16* __restrict__ out, float scale, int T, int H) {
  extern __shared__ float tile[];                 // [64][H + 1]
  const int nblk = T / 64;
  const int b = blockIdx.x / nblk, t0 = (blockIdx.x % nblk) * 64;
  const int n = 64 * H;
  const long tm0 = (static_cast<long>(b) * T + t0) * H;             // first element of the token-major block
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int t = i / H, h = i - t * H;
    const float s = sigmoidf_fast(__bfloat162float(logits[tm0 + i]));
    tile[t * (H + 1) + h] = kBackward ? scale * s * (1.f - s) : scale * s;
  }
  __syncthreads();
  if (!kBackward) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int h = i >> 6, t = i & 63;
      out[(static_cast<long>(b) * H + h) * T + t0 + t] = __float2bfloat16(tile[t * (H + 1) + h]);
    }
  } else {
    // d_last_eta is head-major: read it along t, multiply, and leave token-major
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int h = i >> 6, t = i & 63;
      tile[t * (H + 1) + h] *= __bfloat162float(other[(static_cast<long>(b) * H + h) * T + t0 + t]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int t = i / H, h = i - t * H;
      out[tm0 + i] = __float2bfloat16(tile[t * (H + 1) + h]);
    }
  }
}

// ---- output LayerNorm over the H*64 features of a token, fused with the head-major -> token-major
// turn.  One warp per token: 8 lanes take one head's 128-byte row as 16-byte pieces, so one warp-wide
// load covers 4 heads; a token's values stay in registers (packed bf16) between the statistics and the
// normalisation; the result leaves as whole 512-byte runs of the token's row.
// kChunks = groups of 4 heads (compile time: a token's values must stay in registers, and the kernel is
// latency-bound unless enough warps are resident, so the register count follows the head count).
constexpr int kMaxChunks = 16;     // H <= 64
template <int kChunks>
__global__ void __launch_bounds__(256, (kChunks <= 8 ? 4 : 2)) unpack_layernorm_kernel(const uint4* __restrict__ src, const float* __restrict__ gamma,
                                                               const float* __restrict__ beta, uint4* __restrict__ dst,
                                                               float2* __restrict__ stats, float eps, long tokens, int T, int H) {
  const int lane = threadIdx.x & 31;
  const int sub = lane >> 3, piece = lane & 7;          // head within a group of 4, 16-byte piece of the row
  const long warp0 = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long nwarps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  const float inv_n = 1.f / static_cast<float>(H * 64);
  for (long tok = warp0; tok < tokens; tok += nwarps) {
    const long b = tok / T, t = tok - b * T;
    uint4 raw[kChunks];
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int h = 4 * c + sub;
      if (h < H) raw[c] = __ldcs(src + (((b * H + h) * T + t) << 3) + piece);
    }
    // One pass over the values for both moments, taken about a pivot (the token's first value) so that
    // the variance does not come out of the difference of two large numbers: with d = x - pivot,
    // mean = pivot + sum(d) / n and var = sum(d^2) / n - (sum(d) / n)^2.
    const float pivot = __shfl_sync(0xffffffffu, __uint_as_float(raw[0].x << 16), 0);
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int h = 4 * c + sub;
      if (h < H) {
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw[c]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(v[k]);
          const float d0 = f.x - pivot, d1 = f.y - pivot;
          sum += d0 + d1;
          sq = fmaf(d0, d0, fmaf(d1, d1, sq));
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
    }
    const float dm = sum * inv_n;
    const float mean = pivot + dm;
    sq = fmaxf(sq - sum * dm, 0.f);           // n * variance
    const float rstd = rsqrtf(sq * inv_n + eps);
    if (stats != nullptr && lane == 0) stats[tok] = make_float2(mean, rstd);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int h = 4 * c + sub;
      if (h < H) {
        const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw[c]);
        const int f0 = h * 64 + piece * 8;
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + f0), g1 = *reinterpret_cast<const float4*>(gamma + f0 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(beta + f0), b1 = *reinterpret_cast<const float4*>(beta + f0 + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint4 o4;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(v[k]);
          o[k] = __floats2bfloat162_rn(fmaf((f.x - mean) * rstd, gg[2 * k], bb[2 * k]),
                                       fmaf((f.y - mean) * rstd, gg[2 * k + 1], bb[2 * k + 1]));
        }
        __stcs(dst + ((tok * H + h) << 3) + piece, o4);
      }
    }
  }
}

// ---- backward of the output norm, fused with the token-major -> head-major turn of the gradient: the
// result is the operator's grad_L_XQW_mini_batch.  With xhat = (x - mean) rstd and g = dy gamma:
//   dx = rstd (g - mean(g) - xhat mean(g xhat)),   d_gamma[f] += sum over tokens of dy xhat,   d_beta[f] += sum of dy.
// One pass over x and dy.  A lane owns 8 features (one 16-byte piece of a head row) for every token its CTA
// works on: warp w takes the heads 4 w .. 4 w + 3 (and 4 (w + 8) .. when H > 32), so the parameter gradients
// accumulate in 16 registers per head group with no traffic at all, and a token's two row means are put
// together from the eight warps' partial sums through shared memory, kTokBatch tokens per CTA barrier.  When
// the CTA has run out of tokens every lane adds its sums to the global ones with fp32 atomics (the order of
// the CTAs is not fixed: the last bits of the result can differ from run to run).
constexpr int kTokBatch = 2;
template <int kGroups>
__global__ void __launch_bounds__(256, (kGroups == 1 ? 3 : 1))
pack_layernorm_backward_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, const float* __restrict__ gamma,
                               const float2* __restrict__ stats, uint4* __restrict__ dx, float* __restrict__ d_gamma,
                               float* __restrict__ d_beta, long tokens, int T, int H) {
  __shared__ float2 part[2][kTokBatch][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane >> 3, piece = lane & 7;
  const float inv_n = 1.f / static_cast<float>(H * 64);
  int hh[kGroups];
  float gg[kGroups][8], ag[kGroups][8], ab[kGroups][8];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    hh[g] = 4 * (warp + 8 * g) + sub;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      gg[g][k] = hh[g] < H ? gamma[hh[g] * 64 + piece * 8 + k] : 0.f;
      ag[g][k] = 0.f;
      ab[g][k] = 0.f;
    }
  }
  const long nbatch = (tokens + kTokBatch - 1) / kTokBatch;
  int buf = 0;
  for (long bt = blockIdx.x; bt < nbatch; bt += gridDim.x, buf ^= 1) {
    uint4 rx[kTokBatch][kGroups], rg[kTokBatch][kGroups];
    float2 st[kTokBatch];
    long xrow[kTokBatch];
#pragma unroll
    for (int q = 0; q < kTokBatch; ++q) {
      const long tok = bt * kTokBatch + q;
      const bool live = tok < tokens;
      const long b = live ? tok / T : 0, t = live ? tok - b * T : 0;
      xrow[q] = b * H * T + t;                      // row of head 0; head h is h * T rows further
      st[q] = live ? stats[tok] : make_float2(0.f, 0.f);
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        if (live && hh[g] < H) {
          rx[q][g] = __ldcs(x + ((xrow[q] + static_cast<long>(hh[g]) * T) << 3) + piece);
          rg[q][g] = __ldcs(dy + ((tok * H + hh[g]) << 3) + piece);
        } else {
          rx[q][g] = make_uint4(0u, 0u, 0u, 0u);    // dy = 0: no contribution to any sum
          rg[q][g] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    float s1[kTokBatch], s2[kTokBatch];
#pragma unroll
    for (int q = 0; q < kTokBatch; ++q) {
      s1[q] = 0.f;
      s2[q] = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const __nv_bfloat162* vx = reinterpret_cast<const __nv_bfloat162*>(&rx[q][g]);
        const __nv_bfloat162* vg = reinterpret_cast<const __nv_bfloat162*>(&rg[q][g]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 fx = __bfloat1622float2(vx[k]), fg = __bfloat1622float2(vg[k]);
          const float x0 = (fx.x - st[q].x) * st[q].y, x1 = (fx.y - st[q].x) * st[q].y;
          const float a0 = fg.x * gg[g][2 * k], a1 = fg.y * gg[g][2 * k + 1];
          s1[q] += a0 + a1;
          s2[q] = fmaf(a0, x0, fmaf(a1, x1, s2[q]));
          ag[g][2 * k] = fmaf(fg.x, x0, ag[g][2 * k]);
          ag[g][2 * k + 1] = fmaf(fg.y, x1, ag[g][2 * k + 1]);
          ab[g][2 * k] += fg.x;
          ab[g][2 * k + 1] += fg.y;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int q = 0; q < kTokBatch; ++q) {
        s1[q] += __shfl_xor_sync(0xffffffffu, s1[q], o);
        s2[q] += __shfl_xor_sync(0xffffffffu, s2[q], o);
      }
    }
    if (lane < kTokBatch) {
      float a = s1[0], c = s2[0];
#pragma unroll
      for (int q = 1; q < kTokBatch; ++q)
        if (lane == q) { a = s1[q]; c = s2[q]; }
      part[buf][lane][warp] = make_float2(a, c);
    }
    // one barrier per batch: the other buffer is written again only after the next barrier, which every thread
    // passes after it has read this one
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kTokBatch; ++q) {
      const long tok = bt * kTokBatch + q;
      if (tok >= tokens) break;
      float m1 = 0.f, m2 = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float2 pw = part[buf][q][w];
        m1 += pw.x;
        m2 += pw.y;
      }
      m1 *= inv_n;
      m2 *= inv_n;
      const float mean = st[q].x, rstd = st[q].y;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        if (hh[g] < H) {
          const __nv_bfloat162* vx = reinterpret_cast<const __nv_bfloat162*>(&rx[q][g]);
          const __nv_bfloat162* vg = reinterpret_cast<const __nv_bfloat162*>(&rg[q][g]);
          uint4 o4;
          __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 fx = __bfloat1622float2(vx[k]), fg = __bfloat1622float2(vg[k]);
            const float x0 = (fx.x - mean) * rstd, x1 = (fx.y - mean) * rstd;
            o[k] = __floats2bfloat162_rn(rstd * (fmaf(fg.x, gg[g][2 * k], -m1) - x0 * m2),
                                         rstd * (fmaf(fg.y, gg[g][2 * k + 1], -m1) - x1 * m2));
          }
          __stcs(dx + ((xrow[q] + static_cast<long>(hh[g]) * T) << 3) + piece, o4);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    if (hh[g] < H) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        atomicAdd(d_gamma + hh[g] * 64 + piece * 8 + k, ag[g][k]);
        atomicAdd(d_beta + hh[g] * 64 + piece * 8 + k, ab[g][k]);
      }
    }
  }
}

int check_common(const char* what, int B, int T, int H) {
  if (B < 1 || T < 1 || H < 1 || (T % TTT_CS) != 0) {
    static thread_local char buf[128];
    snprintf(buf, sizeof buf, "%s: B, T, H >= 1 and T a multiple of the mini-batch size 64", what);
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, buf);
  }
  if (static_cast<long>(B) * T * H >= (1L << 31))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "B * T * H must stay below 2^31");
  return TTT_B200_OK;
}
bool bad_ptr(const void* p, uintptr_t align) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & (align - 1)); }

int launch_eta(bool backward, const void* logits, const void* other, void* out, float scale, int B, int T, int H,
               void* stream_) {
  if (int rc = check_common("eta gate", B, T, H)) return rc;
  if (H > 256) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "eta gate: H must not exceed 256");
  if (bad_ptr(logits, 2) || bad_ptr(out, 2) || (backward && bad_ptr(other, 2)))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "eta gate: null or misaligned tensor pointer");
  const unsigned grid = static_cast<unsigned>(B) * (T / 64);
  const size_t smem = 64 * (H + 1) * sizeof(float);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (backward) {
    eta_gate_kernel<true><<<grid, 256, smem, stream>>>(static_cast<const __nv_bfloat16*>(logits),
                                                       static_cast<const __nv_bfloat16*>(other),
                                                       static_cast<__nv_bfloat16*>(out), scale, T, H);
  } else {
    eta_gate_kernel<false><<<grid, 256, smem, stream>>>(static_cast<const __nv_bfloat16*>(logits), nullptr,
                                                        static_cast<__nv_bfloat16*>(out), scale, T, H);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}

}  // namespace

extern "C" int ttt_b200_eta_gate(const void* logits, void* last_eta, float scale, int B, int T, int H, void* stream) {
  return launch_eta(false, logits, nullptr, last_eta, scale, B, T, H, stream);
}

extern "C" int ttt_b200_eta_gate_backward(const void* logits, const void* grad_last_eta, void* grad_logits, float scale,
                                          int B, int T, int H, void* stream) {
  return launch_eta(true, logits, grad_last_eta, grad_logits, scale, B, T, H, stream);
}

extern "C" int ttt_b200_unpack_layernorm(const void* src, const float* gamma, const float* beta, void* dst, float* stats,
                                         float eps, int B, int T, int H, void* stream_) {
  if (int rc = check_common("output norm", B, T, H)) return rc;
  if (H > 4 * kMaxChunks) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm: H must not exceed 64");
  if (bad_ptr(src, 16) || bad_ptr(dst, 16) || bad_ptr(gamma, 16) || bad_ptr(beta, 16))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm: null or not 16-byte aligned tensor pointer");
  if (src == dst) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm: the transform is out of place");
  if (stats != nullptr && (reinterpret_cast<uintptr_t>(stats) & 7))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm: stats must be 8-byte aligned");
  if (!(eps >= 0.f)) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm: eps must be >= 0");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long tokens = static_cast<long>(B) * T;
  long blocks = (tokens + 7) / 8;                     // 8 warps = 8 tokens per CTA pass
  const long cap = static_cast<long>(sms) * 8;        // a whole number of CTAs per SM
  if (blocks > cap) blocks = cap;
  const int chunks = (H + 3) / 4;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
#define TTT_LN_LAUNCH(CH)                                                                                  \
  unpack_layernorm_kernel<CH><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                          \
      static_cast<const uint4*>(src), gamma, beta, static_cast<uint4*>(dst), reinterpret_cast<float2*>(stats), eps, \
      tokens, T, H)
  if (chunks <= 1) TTT_LN_LAUNCH(1);
  else if (chunks <= 2) TTT_LN_LAUNCH(2);
  else if (chunks <= 3) TTT_LN_LAUNCH(3);
  else if (chunks <= 4) TTT_LN_LAUNCH(4);
  else if (chunks <= 6) TTT_LN_LAUNCH(6);
  else if (chunks <= 8) TTT_LN_LAUNCH(8);
  else if (chunks <= 12) TTT_LN_LAUNCH(12);
  else TTT_LN_LAUNCH(16);
#undef TTT_LN_LAUNCH
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}

extern "C" int ttt_b200_pack_layernorm_backward(const void* grad_y, const void* x, const float* gamma, const float* stats,
                                                void* grad_x, float* grad_gamma, float* grad_beta, int B, int T, int H,
                                                void* stream_) {
  if (int rc = check_common("output norm backward", B, T, H)) return rc;
  if (H > 4 * kMaxChunks) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm backward: H must not exceed 64");
  if (bad_ptr(grad_y, 16) || bad_ptr(x, 16) || bad_ptr(grad_x, 16) || bad_ptr(gamma, 16) || bad_ptr(stats, 8) ||
      bad_ptr(grad_gamma, 4) || bad_ptr(grad_beta, 4))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm backward: null or misaligned tensor pointer");
  if (grad_x == x || grad_x == grad_y)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "output norm backward: the transform is out of place");
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long tokens = static_cast<long>(B) * T;
  // one wave of CTAs (as many as are resident at once), each looping over its token batches: every CTA ends
  // with 2 x 64 H atomic adds for the parameter gradients, so there should be no more of them than can run
  long blocks = (tokens + kTokBatch - 1) / kTokBatch;
  const long cap = static_cast<long>(sms) * (H <= 32 ? 3 : 1);
  if (blocks > cap) blocks = cap;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
#define TTT_LNB_LAUNCH(G)                                                                                        \
  pack_layernorm_backward_kernel<G><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                          \
      static_cast<const uint4*>(grad_y), static_cast<const uint4*>(x), gamma, reinterpret_cast<const float2*>(stats), \
      static_cast<uint4*>(grad_x), grad_gamma, grad_beta, tokens, T, H)
  if (H <= 32) TTT_LNB_LAUNCH(1);
  else TTT_LNB_LAUNCH(2);
#undef TTT_LNB_LAUNCH
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}
