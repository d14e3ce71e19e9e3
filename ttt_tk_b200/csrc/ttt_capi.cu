// Host side of the C ABI: argument validation, tensor-map construction, status word,
// error text.  Replaces the host launchers of the reference
// (kernels/ttt/ttt.cu:594-721, kernels/ttt_backward/ttt.cu:1451-1917): same checks, made on
// every call (the reference's backward checks only on the first call of the process,
// kernels/ttt_backward/ttt.cu:1507-1508), and errors are returned instead of printed
// (kernels/ttt/ttt.cu:708-718).
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "ttt_internal.h"

int ttt_launch_forward(const ttt_b200_fwd_args* a, cudaStream_t stream, uint32_t* status, uint64_t limit_ns,
                       int drop_load);
int ttt_launch_backward(const ttt_b200_bwd_args* a, cudaStream_t stream, uint32_t* status, uint64_t limit_ns,
                        int drop_load);
int ttt_launch_backward_cluster(const ttt_b200_bwd_args* a, int cluster, cudaStream_t stream, uint32_t* status,
                                uint64_t limit_ns, int drop_load);
int ttt_launch_linear_forward(const ttt_b200_linear_fwd_args* a, cudaStream_t stream, uint32_t* status,
                              uint64_t limit_ns, int drop_load);
int ttt_launch_linear_backward(const ttt_b200_linear_bwd_args* a, cudaStream_t stream, uint32_t* status,
                               uint64_t limit_ns, int drop_load);
uint64_t ttt_linear_backward_scratch_bytes(int B, int H, int cgs);
int ttt_forward_cluster_capacity(int cluster);
int ttt_backward_cluster_capacity(int cluster);
int ttt_launch_forward_cluster(const ttt_b200_fwd_args* a, int cluster, cudaStream_t stream, uint32_t* status,
                               uint64_t limit_ns, int drop_load);

namespace {

thread_local std::string g_last_error;

std::mutex g_mu;
uint32_t* g_status_host = nullptr;   // pinned, device-visible
uint32_t* g_status_dev = nullptr;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

uint64_t wait_limit_ns() { return ttt_wait_limit_ns(); }

}  // namespace

// Device-side waits give up after this long (nanoseconds).  A healthy launch never waits
// more than microseconds; the limit only decides how fast a lost signal is reported.
uint64_t ttt_wait_limit_ns() {
  static uint64_t v = [] {
    const char* e = std::getenv("TTT_B200_WAIT_LIMIT_MS");
    long ms = e ? std::atol(e) : 2000;
    if (ms < 1) ms = 1;
    return static_cast<uint64_t>(ms) * 1000000ull;
  }();
  return v;
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// How many CTAs share one stream.  The mini-batches of a stream are strictly sequential, so with fewer
// streams than SMs the idle SMs can only help by taking a share of every stream's hidden units.  The
// thresholds are measured (B200, 148 SMs): four CTAs per stream win whenever they all fit on the GPU at
// once (forward 18 %, backward 17-20 % per mini-batch over one CTA).  Two CTAs per stream win in the
// forward whenever they fit (12-17 %).  In the backward they gain 6-11 % up to 32 streams, where four CTAs
// are the better choice anyway, and nothing beyond 37 streams (more than 74 CTAs: both SMs of a TPC are
// then busy, and the backward, whose scratch traffic goes through the port the two share, slows down by
// as much as the split gained), so the backward is never given two.
int ttt_pick_cluster(int streams, uint32_t flags, bool backward, int* cluster) {
  int forced = static_cast<int>((flags & TTT_B200_FLAG_CLUSTER_MASK) >> TTT_B200_FLAG_CLUSTER_SHIFT);
  if (forced == 0) {
    static const int env = [] {
      const char* e = std::getenv("TTT_B200_CLUSTER");
      return e ? std::atoi(e) : 0;
    }();
    forced = env;
  }
  if (forced != 0) {
    if (forced != 1 && forced != 2 && forced != 4)
      return ttt_set_error(TTT_B200_ERR_BAD_ARGS, "cluster size must be 1, 2 or 4");
    *cluster = forced;
    return TTT_B200_OK;
  }
  // all streams must be resident at once for the sharding to pay: the widest cluster size whose capacity
  // (clusters the device runs at the same time) covers them.  The backward gains nothing from two CTAs per
  // stream beyond the stream counts four CTAs cover (measured), so it never picks two.
  auto capacity = [&](int c) { return backward ? ttt_backward_cluster_capacity(c) : ttt_forward_cluster_capacity(c); };
  if (streams <= capacity(4)) *cluster = 4;
  else if (!backward && streams <= capacity(2)) *cluster = 2;
  else *cluster = 1;
  return TTT_B200_OK;
}

int ttt_set_error(int code, const char* msg) {
  g_last_error = msg ? msg : "";
  return code;
}

int ttt_status_word(uint32_t** dev_ptr) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_host) {
    cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), sizeof(uint32_t),
                                  cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
    *g_status_host = 0;
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0);
    if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  }
  *dev_ptr = g_status_dev;
  return TTT_B200_OK;
}

uint32_t ttt_take_status() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_host) return 0;
  volatile uint32_t* w = g_status_host;
  const uint32_t v = *w;
  *w = 0;
  return v;
}

int ttt_check_status(cudaStream_t stream) {
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return ttt_set_error(TTT_B200_ERR_LAUNCH, cudaGetErrorString(e));
  if (ttt_take_status() != 0)
    return ttt_set_error(TTT_B200_ERR_TIMEOUT, "a device-side bounded wait ran out; results are invalid");
  return TTT_B200_OK;
}

// Encoded maps are kept in a small cache keyed on (base pointer, rows): a training loop calls the
// operator with the same buffers step after step, and an encode costs about a hundred microseconds of
// host time per map (the reference re-encodes 15 / 44 maps on every call: kernels/ttt/ttt.cu:655-673).
// A map depends on nothing but its key, so a stale entry cannot exist; the cache is bounded and simply
// overwrites its oldest entry.
int ttt_make_tile_map(CUtensorMap* map, const void* base, uint64_t rows) {
  struct Entry { const void* base; uint64_t rows; CUtensorMap map; };
  constexpr int kEntries = 64;
  static Entry cache[kEntries];
  static int used = 0, next = 0;
  std::lock_guard<std::mutex> lk(g_mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].rows == rows) {
      *map = cache[i].map;
      return TTT_B200_OK;
    }
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return ttt_set_error(TTT_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from the driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t dims[2] = {64, rows};
  const cuuint64_t strides[1] = {128};           // bytes between rows
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    std::snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return ttt_set_error(TTT_B200_ERR_LAUNCH, buf);
  }
  Entry& e = cache[next];
  e.base = base; e.rows = rows; e.map = *map;
  next = (next + 1) % kEntries;
  if (used < kEntries) ++used;
  return TTT_B200_OK;
}

namespace {

#define TTT_REQUIRE(cond, msg) \
  do {                         \
    if (!(cond)) return ttt_set_error(TTT_B200_ERR_BAD_ARGS, msg); \
  } while (0)

int check_dims(int B, int H, int NC, int cgs, int nck) {
  TTT_REQUIRE(B >= 1 && H >= 1, "B and H must be >= 1");
  TTT_REQUIRE(NC >= 1, "NC (sequence length / 64) must be >= 1");
  TTT_REQUIRE(cgs >= 1, "checkpoint_group_size must be >= 1");
  TTT_REQUIRE(nck == (NC + cgs - 1) / cgs, "checkpoint tensors must hold ceil(NC / checkpoint_group_size) states");
  TTT_REQUIRE(static_cast<uint64_t>(B) * H * NC * 64 < (1ull << 31), "B*H*NC*64 must be below 2^31");
  return TTT_B200_OK;
}

int pre_launch(uint32_t** status) {
  if (int rc = ttt_status_word(status)) return rc;
  if (ttt_take_status() != 0)
    return ttt_set_error(TTT_B200_ERR_TIMEOUT,
                         "an earlier launch reported a device-side wait that ran out; its results are invalid");
  return TTT_B200_OK;
}

}  // namespace

extern "C" int ttt_b200_forward(const ttt_b200_fwd_args* a, void* stream_) {
  TTT_REQUIRE(a != nullptr, "args is NULL");
  if (int rc = check_dims(a->B, a->H, a->NC, a->checkpoint_group_size, a->num_checkpoints)) return rc;
  const void* ptrs[] = {a->XQ, a->XK, a->XV, a->last_eta, a->ttt_norm_weight, a->ttt_norm_bias, a->W1, a->b1,
                        a->W2, a->b2, a->W1_checkpoints, a->b1_checkpoints, a->W2_checkpoints, a->b2_checkpoints,
                        a->Out};
  for (const void* q : ptrs) {
    TTT_REQUIRE(q != nullptr, "a required tensor pointer is NULL");
    TTT_REQUIRE(aligned16(q), "tensor pointers must be 16-byte aligned");
  }
  const int nfinal = (a->W1_final != nullptr) + (a->b1_final != nullptr) + (a->W2_final != nullptr) +
                     (a->b2_final != nullptr);
  TTT_REQUIRE(nfinal == 0 || nfinal == 4, "W1/b1/W2/b2_final must be given together or not at all");
  if (nfinal == 4)
    TTT_REQUIRE(aligned16(a->W1_final) && aligned16(a->b1_final) && aligned16(a->W2_final) && aligned16(a->b2_final),
                "tensor pointers must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = pre_launch(&status)) return rc;
  int cluster = 1;
  if (int rc = ttt_pick_cluster(a->B * a->H, a->flags, false, &cluster)) return rc;
  const int drop = (a->flags & TTT_B200_FLAG_TEST_LOST_LOAD) ? (a->NC > 1 ? 1 : 0) : -1;
  if (int rc = cluster == 1 ? ttt_launch_forward(a, stream, status, wait_limit_ns(), drop)
                            : ttt_launch_forward_cluster(a, cluster, stream, status, wait_limit_ns(), drop))
    return rc;
  if (a->flags & TTT_B200_FLAG_SYNC) return ttt_check_status(stream);
  return TTT_B200_OK;
}

extern "C" int ttt_b200_linear_forward(const ttt_b200_linear_fwd_args* a, void* stream_) {
  TTT_REQUIRE(a != nullptr, "args is NULL");
  if (int rc = check_dims(a->B, a->H, a->NC, a->checkpoint_group_size, a->num_checkpoints)) return rc;
  const void* ptrs[] = {a->XQ, a->XK, a->XV, a->last_eta, a->ttt_norm_weight, a->ttt_norm_bias, a->W1, a->b1,
                        a->W1_checkpoints, a->b1_checkpoints, a->Out};
  for (const void* q : ptrs) {
    TTT_REQUIRE(q != nullptr, "a required tensor pointer is NULL");
    TTT_REQUIRE(aligned16(q), "tensor pointers must be 16-byte aligned");
  }
  TTT_REQUIRE((a->W1_final != nullptr) == (a->b1_final != nullptr), "W1_final and b1_final must be given together or not at all");
  if (a->W1_final != nullptr)
    TTT_REQUIRE(aligned16(a->W1_final) && aligned16(a->b1_final), "tensor pointers must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = pre_launch(&status)) return rc;
  const int drop = (a->flags & TTT_B200_FLAG_TEST_LOST_LOAD) ? (a->NC > 1 ? 1 : 0) : -1;
  if (int rc = ttt_launch_linear_forward(a, stream, status, wait_limit_ns(), drop)) return rc;
  if (a->flags & TTT_B200_FLAG_SYNC) return ttt_check_status(stream);
  return TTT_B200_OK;
}

extern "C" uint64_t ttt_b200_linear_backward_scratch_bytes(int B, int H, int checkpoint_group_size) {
  if (B < 1 || H < 1 || checkpoint_group_size < 1) return 0;
  return ttt_linear_backward_scratch_bytes(B, H, checkpoint_group_size);
}

extern "C" int ttt_b200_linear_backward(const ttt_b200_linear_bwd_args* a, void* stream_) {
  TTT_REQUIRE(a != nullptr, "args is NULL");
  if (int rc = check_dims(a->B, a->H, a->NC, a->checkpoint_group_size, a->num_checkpoints)) return rc;
  const void* ptrs[] = {a->XQ, a->XK, a->XV, a->last_eta, a->ttt_norm_weight, a->ttt_norm_bias, a->W1_checkpoints,
                        a->b1_checkpoints, a->grad_L_W1_last, a->grad_L_b1_last, a->grad_L_XQW_mini_batch, a->scratch,
                        a->grad_L_ttt_norm_weight, a->grad_L_ttt_norm_bias, a->grad_L_W1_init, a->grad_L_b1_init,
                        a->grad_L_last_eta, a->grad_L_XQ, a->grad_L_XK, a->grad_L_XV};
  for (const void* q : ptrs) {
    TTT_REQUIRE(q != nullptr, "a required tensor pointer is NULL");
    TTT_REQUIRE(aligned16(q), "tensor pointers must be 16-byte aligned");
  }
  TTT_REQUIRE(a->scratch_bytes >= ttt_linear_backward_scratch_bytes(a->B, a->H, a->checkpoint_group_size),
              "scratch is smaller than ttt_b200_linear_backward_scratch_bytes(B, H, checkpoint_group_size)");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = pre_launch(&status)) return rc;
  // the hook drops the recompute inputs of the last group's second mini-batch (its only one if it has one)
  const int last0 = (a->num_checkpoints - 1) * a->checkpoint_group_size;
  const int drop = (a->flags & TTT_B200_FLAG_TEST_LOST_LOAD) ? (last0 + 1 < a->NC ? last0 + 1 : last0) : -1;
  if (int rc = ttt_launch_linear_backward(a, stream, status, wait_limit_ns(), drop)) return rc;
  if (a->flags & TTT_B200_FLAG_SYNC) return ttt_check_status(stream);
  return TTT_B200_OK;
}

extern "C" int ttt_b200_backward(const ttt_b200_bwd_args* a, void* stream_) {
  TTT_REQUIRE(a != nullptr, "args is NULL");
  if (int rc = check_dims(a->B, a->H, a->NC, a->checkpoint_group_size, a->num_checkpoints)) return rc;
  const void* ptrs[] = {a->XQ, a->XK, a->XV, a->last_eta, a->ttt_norm_weight, a->ttt_norm_bias,
                        a->W1_checkpoints, a->b1_checkpoints, a->W2_checkpoints, a->b2_checkpoints,
                        a->W1_init_group, a->b1_init_group, a->W2_init_group, a->b2_init_group,
                        a->x_hat_ln_group, a->std_ln_group, a->X2_group, a->Z1_group, a->Z1_bar_group,
                        a->X2_bar_group, a->grad_l_wrt_Z2_group, a->grad_l_wrt_Z1_group, a->x_hat_fused_group,
                        a->grad_x_hat_fused_group, a->grad_output_fused_group, a->std_fused_group,
                        a->grad_L_W1_last, a->grad_L_b1_last, a->grad_L_W2_last, a->grad_L_b2_last,
                        a->grad_L_XQW_mini_batch, a->grad_L_ttt_norm_weight, a->grad_L_ttt_norm_bias,
                        a->grad_L_W1_init, a->grad_L_b1_init, a->grad_L_W2_init, a->grad_L_b2_init,
                        a->grad_L_last_eta, a->grad_L_XQ, a->grad_L_XK, a->grad_L_XV};
  for (const void* q : ptrs) {
    TTT_REQUIRE(q != nullptr, "a required tensor pointer is NULL");
    TTT_REQUIRE(aligned16(q), "tensor pointers must be 16-byte aligned");
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint32_t* status = nullptr;
  if (int rc = pre_launch(&status)) return rc;
  int cluster = 1;
  if (int rc = ttt_pick_cluster(a->B * a->H, a->flags, true, &cluster)) return rc;
  // the hook drops the recompute inputs of the last group's second mini-batch (its only one if it has one)
  const int last0 = (a->num_checkpoints - 1) * a->checkpoint_group_size;
  const int drop = (a->flags & TTT_B200_FLAG_TEST_LOST_LOAD) ? (last0 + 1 < a->NC ? last0 + 1 : last0) : -1;
  if (int rc = cluster == 1 ? ttt_launch_backward(a, stream, status, wait_limit_ns(), drop)
                            : ttt_launch_backward_cluster(a, cluster, stream, status, wait_limit_ns(), drop))
    return rc;
  if (a->flags & TTT_B200_FLAG_SYNC) return ttt_check_status(stream);
  return TTT_B200_OK;
}

extern "C" const char* ttt_b200_last_error(void) { return g_last_error.c_str(); }

extern "C" int ttt_b200_take_status(void) {
  const uint32_t a = ttt_take_status();
  const uint32_t b = ttt_noalloc_take_status();
  return (a | b) ? TTT_B200_ERR_TIMEOUT : TTT_B200_OK;
}

extern "C" int ttt_b200_version(void) { return 1001; }

extern "C" int ttt_b200_cluster_capacity(int cluster, int backward) {
  return backward ? ttt_backward_cluster_capacity(cluster) : ttt_forward_cluster_capacity(cluster);
}

extern "C" int ttt_b200_pick_cluster(int streams, int backward) {
  int c = 1;
  if (streams < 1 || ttt_pick_cluster(streams, 0u, backward != 0, &c) != TTT_B200_OK) return -1;
  return c;
}
