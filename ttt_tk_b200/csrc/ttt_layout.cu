// Token layout transforms either side of the TTT-MLP operator.  A model keeps its activations
// token-major, [B][T][H][64] (= [B, T, H*64]); the operator, like the reference's (README.md:98 of
// the reference asks for contiguous [B, H, NC, 64, 64] inputs), wants them head-major,
// [B][H][T][64].  `pack` goes model -> operator for up to four tensors in one launch (Q, K, V and
// the upstream gradient), `unpack` the other way (Out, dQ, dK, dV).  Pure byte movement: every
// (b, t, h) row of 64 bf16 = 128 bytes is one cache line on both sides, moved by 8 threads as
// 16-byte pieces.  HBM-bound; algorithmic bytes = 2 x tensor size.
#include "ttt_internal.h"

namespace {

constexpr int kMaxTensors = 4;

struct LayoutParams {
  const uint4* src[kMaxTensors];
  uint4* dst[kMaxTensors];
  uint32_t T, H;    // tokens per sequence, heads
  long pieces;      // B * T * H * 8 sixteen-byte pieces per tensor (B * T * H < 2^31)
};

// kPack: src [B][T][H][8 pieces] -> dst [B][H][T][8 pieces]; else the inverse.  The pieces are
// enumerated in the token-major order, so that side is one sequential stream per CTA wave; the
// head-major side is touched in whole 128-byte lines, 4 KB apart for neighbouring heads, which
// the L2 merges (a CTA wave covers the neighbouring tokens of each line's 8 KB tile at once).
template <bool kPack>
__global__ void __launch_bounds__(256) layout_kernel(LayoutParams p) {
  const uint4* __restrict__ src = p.src[blockIdx.y];
  uint4* __restrict__ dst = p.dst[blockIdx.y];
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.pieces; i += stride) {
    const uint32_t row = static_cast<uint32_t>(i >> 3), q = static_cast<uint32_t>(i) & 7u;   // token-major row (b, t, h)
    const uint32_t bt = row / p.H, h = row - bt * p.H;
    const uint32_t b = bt / p.T, t = bt - b * p.T;
    const long hm = (static_cast<long>((b * p.H + h) * p.T + t) << 3) + q;     // the same piece, head-major
    if (kPack) __stcs(dst + hm, __ldcs(src + i));
    else       __stcs(dst + i, __ldcs(src + hm));
  }
}

int launch_layout(bool pack, const void* const* src, void* const* dst, int n, int B, int T, int H, void* stream_) {
  if (!src || !dst || n < 1 || n > kMaxTensors)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "layout: 1 to 4 tensors, non-null pointer arrays");
  if (B < 1 || T < 1 || H < 1 || (T % TTT_CS) != 0)
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "layout: B, T, H >= 1 and T a multiple of the mini-batch size 64");
  LayoutParams p{};
  for (int k = 0; k < n; ++k) {
    if (!src[k] || !dst[k] || (reinterpret_cast<uintptr_t>(src[k]) & 15) || (reinterpret_cast<uintptr_t>(dst[k]) & 15))
      return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "layout: null or not 16-byte aligned tensor pointer");
    if (src[k] == dst[k]) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "layout: the transform is out of place");
    p.src[k] = static_cast<const uint4*>(src[k]);
    p.dst[k] = static_cast<uint4*>(dst[k]);
  }
  if (static_cast<long>(B) * T * H >= (1L << 31))
    return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "layout: B * T * H must stay below 2^31");
  p.T = static_cast<uint32_t>(T);
  p.H = static_cast<uint32_t>(H);
  p.pieces = static_cast<long>(B) * T * H * 8;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // a whole number of CTAs per SM (8 x 256 threads are resident), no more than the work needs
  long blocks = (p.pieces + 255) / 256;
  const long cap = static_cast<long>(sms) * 8;
  if (blocks > cap) blocks = cap;
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(n));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (pack) layout_kernel<true><<<grid, 256, 0, stream>>>(p);
  else      layout_kernel<false><<<grid, 256, 0, stream>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  return TTT_B200_OK;
}

}  // namespace

extern "C" int ttt_b200_pack_tokens(const void* const* src, void* const* dst, int n_tensors, int B, int T, int H,
                                    void* stream) {
  return launch_layout(true, src, dst, n_tensors, B, T, H, stream);
}

extern "C" int ttt_b200_unpack_tokens(const void* const* src, void* const* dst, int n_tensors, int B, int T, int H,
                                      void* stream) {
  return launch_layout(false, src, dst, n_tensors, B, T, H, stream);
}
