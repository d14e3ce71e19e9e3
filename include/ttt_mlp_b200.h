/* C ABI of libttt_mlp_b200.so: the TTT-MLP forward / backward operator for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; every pointer is a DEVICE pointer to a
 * contiguous array unless stated otherwise; `stream` is a cudaStream_t passed as void*.
 *
 * The two operator entry points stand behind the reference's PyTorch extension
 * `test_time_training` (test_time_training.cpp:24-104) and replace its two host launchers
 *   ttt_forward   kernels/ttt/ttt.cu:594-721
 *   ttt_backward  kernels/ttt_backward/ttt.cu:1451-1917
 * one struct field per positional tensor of those functions, in the same order.
 *
 * Fixed sizes (reference: kernels/ttt/ttt.cu:612-613, 621-630): mini-batch CS = 64 tokens,
 * head dimension F = 64, MLP hidden width 256.  NC = sequence length / 64.
 *
 * Return codes: 0 ok; 1 bad arguments (nothing launched); 2 CUDA launch / runtime error;
 * 3 a device-side bounded wait ran out (the kernel exited cleanly, results are invalid).
 * ttt_b200_last_error() returns the calling thread's last message.
 *
 * Calls are stream-ordered and do not synchronise unless TTT_B200_FLAG_SYNC is set (the
 * reference blocks on the stream and the device after every call, kernels/ttt/ttt.cu:714-715).
 * A code-3 condition of an asynchronous call is reported by the next call on any stream, or by
 * ttt_b200_take_status() after the caller has synchronised.
 */
#ifndef TTT_MLP_B200_H_
#define TTT_MLP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TTT_B200_OK = 0,
  TTT_B200_ERR_BAD_ARGS = 1,
  TTT_B200_ERR_LAUNCH = 2,
  TTT_B200_ERR_TIMEOUT = 3
};

enum {
  TTT_B200_FLAG_SYNC = 1u, /* synchronise the stream and report device-side status before returning */
  /* Test hook for the failure path (no counterpart in the reference): stream 0 never issues the loads
   * of its second mini-batch (its only one when NC = 1), so that the kernel's bounded wait for them
   * runs out; the kernel reports code 3 through the status word and exits normally. */
  TTT_B200_FLAG_TEST_LOST_LOAD = 2u,
  /* Bits 8..11: how many CTAs (a thread-block cluster) share one (batch, head) stream, each owning
   * 256 / n hidden units; the reference fixes this at compile time (TP = 2 in kernels/ttt/ttt.cu:11-12,
   * 4 in kernels/ttt_backward/ttt.cu:12-16).  0 = chosen per launch from B*H and the number of clusters the GPU runs at once
   * (overridable with the environment variable TTT_B200_CLUSTER); 1, 2 or 4 = forced. */
  TTT_B200_FLAG_CLUSTER_SHIFT = 8,
  TTT_B200_FLAG_CLUSTER_MASK = 0xFu << 8
};

/* Arguments of the forward.  Replaces ttt_forward(XQ, XK, XV, last_eta, ttt_norm_weight,
 * ttt_norm_bias, W1, b1, W2, b2, W1_checkpoints, b1_checkpoints, W2_checkpoints,
 * b2_checkpoints, Out, checkpoint_group_size)  -- kernels/ttt/ttt.cu:594-611.
 * bf16: XQ XK XV last_eta Out.  fp32: everything else. */
typedef struct ttt_b200_fwd_args {
  const void* XQ;                /* bf16 [B,H,NC,64,64] */
  const void* XK;                /* bf16 [B,H,NC,64,64] */
  const void* XV;                /* bf16 [B,H,NC,64,64] */
  const void* last_eta;          /* bf16 [B,H,NC,64] */
  const float* ttt_norm_weight;  /* [H,64] */
  const float* ttt_norm_bias;    /* [H,64] */
  const float* W1;               /* [B,H,64,256] */
  const float* b1;               /* [B,H,256] */
  const float* W2;               /* [B,H,256,64] */
  const float* b2;               /* [B,H,64] */
  float* W1_checkpoints;         /* [B,H,n,64,256], n = ceil(NC / checkpoint_group_size) */
  float* b1_checkpoints;         /* [B,H,n,256] */
  float* W2_checkpoints;         /* [B,H,n,256,64] */
  float* b2_checkpoints;         /* [B,H,n,64] */
  void* Out;                     /* bf16 [B,H,NC,64,64] */
  int32_t B, H, NC;
  int32_t checkpoint_group_size;
  int32_t num_checkpoints;       /* size(2) of the checkpoint tensors; must equal n */
  uint32_t flags;
  /* Optional (may be NULL): state after the last mini-batch, which the reference computes
   * but never stores (kernels/ttt/ttt.cu:276-584).  Shapes as W1/b1/W2/b2. */
  float* W1_final;
  float* b1_final;
  float* W2_final;
  float* b2_final;
} ttt_b200_fwd_args;

/* Arguments of the TTT-Linear forward: the same operator with the inner model reduced to one linear layer,
 * f(x) = x W1 + b1 with W1 [64 x 64] (the hidden layer, W2 and b2 dropped; everything else, the checkpoint
 * rule included, as in ttt_b200_fwd_args).  The reference has no counterpart: it ships the TTT-MLP operator
 * only (README.md:18).  Its backward: ttt_b200_linear_bwd_args. */
typedef struct ttt_b200_linear_fwd_args {
  const void* XQ;                /* bf16 [B,H,NC,64,64] */
  const void* XK;                /* bf16 [B,H,NC,64,64] */
  const void* XV;                /* bf16 [B,H,NC,64,64] */
  const void* last_eta;          /* bf16 [B,H,NC,64] */
  const float* ttt_norm_weight;  /* [H,64] */
  const float* ttt_norm_bias;    /* [H,64] */
  const float* W1;               /* [B,H,64,64] (input feature x output feature) */
  const float* b1;               /* [B,H,64] */
  float* W1_checkpoints;         /* [B,H,n,64,64], n = ceil(NC / checkpoint_group_size) */
  float* b1_checkpoints;         /* [B,H,n,64] */
  void* Out;                     /* bf16 [B,H,NC,64,64] */
  int32_t B, H, NC;
  int32_t checkpoint_group_size;
  int32_t num_checkpoints;       /* size(2) of the checkpoint tensors; must equal n */
  uint32_t flags;                /* TTT_B200_FLAG_SYNC, TTT_B200_FLAG_TEST_LOST_LOAD; the cluster bits are ignored */
  float* W1_final;               /* optional (both or neither): state after the last mini-batch */
  float* b1_final;
} ttt_b200_linear_fwd_args;

/* Arguments of the TTT-Linear backward: gradients of ttt_b200_linear_forward from its checkpoints (per
 * checkpoint group: recompute, then reverse sweep).  `scratch` is caller-provided working memory of at least
 * ttt_b200_linear_backward_scratch_bytes(B, H, checkpoint_group_size) bytes, 16-byte aligned, contents
 * unspecified before and after.  Outputs are overwritten; the norm gradients come per batch element
 * ([B,H,64]: the caller sums over B), like the MLP operator's.  No counterpart in the reference. */
typedef struct ttt_b200_linear_bwd_args {
  const void* XQ;                    /* bf16 [B,H,NC,64,64] */
  const void* XK;
  const void* XV;
  const void* last_eta;              /* bf16 [B,H,NC,64] */
  const float* ttt_norm_weight;      /* [H,64] */
  const float* ttt_norm_bias;        /* [H,64] */
  const float* W1_checkpoints;       /* [B,H,n,64,64] written by the forward */
  const float* b1_checkpoints;       /* [B,H,n,64] */
  const float* grad_L_W1_last;       /* [B,H,64,64] dL/d(state after the last mini-batch) */
  const float* grad_L_b1_last;       /* [B,H,64] */
  const void* grad_L_XQW_mini_batch; /* bf16 [B,H,NC,64,64] dL/dOut */
  void* scratch;
  float* grad_L_ttt_norm_weight;     /* [B,H,64] */
  float* grad_L_ttt_norm_bias;       /* [B,H,64] */
  float* grad_L_W1_init;             /* [B,H,64,64] */
  float* grad_L_b1_init;             /* [B,H,64] */
  void* grad_L_last_eta;             /* bf16 [B,H,NC,64] */
  void* grad_L_XQ;                   /* bf16 [B,H,NC,64,64] */
  void* grad_L_XK;
  void* grad_L_XV;
  int32_t B, H, NC;
  int32_t checkpoint_group_size;
  int32_t num_checkpoints;
  uint32_t flags;                    /* TTT_B200_FLAG_SYNC, TTT_B200_FLAG_TEST_LOST_LOAD */
  uint64_t scratch_bytes;            /* size of `scratch`, checked against the requirement */
} ttt_b200_linear_bwd_args;

/* Arguments of the backward.  Replaces ttt_backward(...43 positional arguments...)
 * -- kernels/ttt_backward/ttt.cu:1451-1495; same order.  The sixteen `*_group` tensors are
 * caller-provided scratch of the reference's shapes; this implementation uses a subset of
 * them, in its own layout (their contents after the call are unspecified).
 * Deviations from the reference, all towards the documented usage:
 *   - grad_L_XQ / XK / XV / last_eta are OVERWRITTEN (the reference accumulates into them and
 *     requires zero-filled buffers: kernels/ttt_backward/matching.py:412-415);
 *   - `Out` is never written (the reference adds a debug term into it,
 *     kernels/ttt_backward/ttt.cu:1313). */
typedef struct ttt_b200_bwd_args {
  const void* XQ;                    /* bf16 [B,H,NC,64,64] */
  const void* XK;
  const void* XV;
  const void* last_eta;              /* bf16 [B,H,NC,64(,1)] */
  const float* ttt_norm_weight;      /* [H,64] */
  const float* ttt_norm_bias;        /* [H,64] */
  const float* W1_checkpoints;       /* [B,H,n,64,256] */
  const float* b1_checkpoints;       /* [B,H,n,256] */
  const float* W2_checkpoints;       /* [B,H,n,256,64] */
  const float* b2_checkpoints;       /* [B,H,n,64] */
  const void* Out;                   /* bf16, unused */
  /* scratch, one slot per mini-batch of a checkpoint group (cgs slots per (b,h)) */
  float* W1_init_group;              /* fp32 [B,H,cgs,64,256] */
  float* b1_init_group;              /* fp32 [B,H,cgs,256] */
  float* W2_init_group;              /* fp32 [B,H,cgs,256,64] */
  float* b2_init_group;              /* fp32 [B,H,cgs,64] */
  void* x_hat_ln_group;              /* bf16 [B,H,cgs,64,64] */
  float* std_ln_group;               /* fp32 [B,H,cgs,64] */
  void* X2_group;                    /* bf16 [B,H,cgs,64,256] */
  void* Z1_group;                    /* bf16 [B,H,cgs,64,256] */
  void* Z1_bar_group;                /* bf16 [B,H,cgs,64,256] */
  void* X2_bar_group;                /* bf16 [B,H,cgs,64,256] */
  void* grad_l_wrt_Z2_group;         /* bf16 [B,H,cgs,64,64] */
  void* grad_l_wrt_Z1_group;         /* bf16 [B,H,cgs,64,256] */
  void* x_hat_fused_group;           /* bf16 [B,H,cgs,64,64] */
  void* grad_x_hat_fused_group;      /* bf16 [B,H,cgs,64,64]; validated, never touched */
  void* grad_output_fused_group;     /* bf16 [B,H,cgs,64,64]; validated, never touched (rebuilt from x_hat_fused, K, V) */
  float* std_fused_group;            /* fp32 [B,H,cgs,64] */
  /* upstream gradients */
  const float* grad_L_W1_last;       /* [B,H,64,256] */
  const float* grad_L_b1_last;       /* [B,H,256] */
  const float* grad_L_W2_last;       /* [B,H,256,64] */
  const float* grad_L_b2_last;       /* [B,H,64] */
  const void* grad_L_XQW_mini_batch; /* bf16 [B,H,NC,64,64] */
  /* outputs */
  float* grad_L_ttt_norm_weight;     /* [B,H,64]: one row per batch element, caller sums dim 0 */
  float* grad_L_ttt_norm_bias;       /* [B,H,64] */
  float* grad_L_W1_init;             /* [B,H,64,256] */
  float* grad_L_b1_init;             /* [B,H,256] */
  float* grad_L_W2_init;             /* [B,H,256,64] */
  float* grad_L_b2_init;             /* [B,H,64] */
  void* grad_L_last_eta;             /* bf16 [B,H,NC,64] */
  void* grad_L_XQ;                   /* bf16 [B,H,NC,64,64] */
  void* grad_L_XK;
  void* grad_L_XV;
  int32_t B, H, NC;
  int32_t checkpoint_group_size;
  int32_t num_checkpoints;
  uint32_t flags;
} ttt_b200_bwd_args;

/* Forward: replaces kernels/ttt/ttt.cu:594-721 (validation, launch) and the device kernel
 * fwd_ttt_mlp_ker (kernels/ttt/ttt.cu:85-586). */
int ttt_b200_forward(const ttt_b200_fwd_args* args, void* stream);

/* Backward: replaces kernels/ttt_backward/ttt.cu:1451-1917 and bwd_ttt_mlp_ker (:179-1443). */
int ttt_b200_backward(const ttt_b200_bwd_args* args, void* stream);

/* Backward for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Hosts that commit all of HBM to their own pools at start-up (so that a later
 * cudaMalloc fails or fragments the pool), or that cannot afford the implicit device
 * synchronisation of an allocation inside a latency-critical loop, cannot provide the sixteen
 * `*_group` scratch tensors on demand; for them the scratch is a fixed array inside the library
 * (about 32 MiB, held by every GPU that loads the library's kernels until the process exits).
 * Inputs, checkpoints, upstream gradients and outputs are passed as for ttt_b200_backward and
 * the results are the same.
 *   - Limit: B * H * checkpoint_group_size <= TTT_B200_NOALLOC_MAX_SLOTS; larger problems
 *     return code 1.
 *   - The call performs no cudaMalloc / cudaFree / allocating library call.  The first call on
 *     each device also resolves the array's device address and raises the kernel's
 *     shared-memory limit: make that first call before any stream capture begins.
 *   - All calls on a device share the array, which keeps the previous call's contents (nothing
 *     in it needs to start at zero); calls that overlap on the GPU race on it: serialise them.
 *   - A device-side wait that ran out (code 3) is reported by the call itself when
 *     TTT_B200_FLAG_SYNC is set; without the flag the call returns once the kernel is launched and
 *     the condition stays recorded (no later launch clears it) until ttt_b200_take_status() is
 *     called after the caller has synchronised.  The wait limit is TTT_B200_WAIT_LIMIT_MS, as for
 *     the other entry points. */
#define TTT_B200_NOALLOC_MAX_SLOTS 128
typedef struct ttt_b200_bwd_noalloc_args {
  const void* XQ;                    /* bf16 [B,H,NC,64,64] */
  const void* XK;
  const void* XV;
  const void* last_eta;              /* bf16 [B,H,NC,64(,1)] */
  const float* ttt_norm_weight;      /* [H,64] */
  const float* ttt_norm_bias;        /* [H,64] */
  const float* W1_checkpoints;       /* [B,H,n,64,256] */
  const float* b1_checkpoints;       /* [B,H,n,256] */
  const float* W2_checkpoints;       /* [B,H,n,256,64] */
  const float* b2_checkpoints;       /* [B,H,n,64] */
  const float* grad_L_W1_last;       /* [B,H,64,256] */
  const float* grad_L_b1_last;       /* [B,H,256] */
  const float* grad_L_W2_last;       /* [B,H,256,64] */
  const float* grad_L_b2_last;       /* [B,H,64] */
  const void* grad_L_XQW_mini_batch; /* bf16 [B,H,NC,64,64] */
  float* grad_L_ttt_norm_weight;     /* [B,H,64] */
  float* grad_L_ttt_norm_bias;       /* [B,H,64] */
  float* grad_L_W1_init;             /* [B,H,64,256] */
  float* grad_L_b1_init;             /* [B,H,256] */
  float* grad_L_W2_init;             /* [B,H,256,64] */
  float* grad_L_b2_init;             /* [B,H,64] */
  void* grad_L_last_eta;             /* bf16 [B,H,NC,64] */
  void* grad_L_XQ;                   /* bf16 [B,H,NC,64,64] */
  void* grad_L_XK;
  void* grad_L_XV;
  int32_t B, H, NC;
  int32_t checkpoint_group_size;
  int32_t num_checkpoints;
  uint32_t flags;
} ttt_b200_bwd_noalloc_args;
int ttt_b200_backward_noalloc(const ttt_b200_bwd_noalloc_args* args, void* stream);

/* Last error text of the calling thread ("" if none). */
const char* ttt_b200_last_error(void);

/* TTT-Linear forward (see ttt_b200_linear_fwd_args): one CTA per (batch, head) stream, stream-ordered,
 * same status codes and status-word protocol as ttt_b200_forward. */
int ttt_b200_linear_forward(const ttt_b200_linear_fwd_args* args, void* cuda_stream);

/* TTT-Linear backward (see ttt_b200_linear_bwd_args): one CTA per (batch, head) stream, stream-ordered, same
 * status codes and status-word protocol as ttt_b200_backward. */
int ttt_b200_linear_backward(const ttt_b200_linear_bwd_args* args, void* cuda_stream);
/* Bytes of scratch ttt_b200_linear_backward needs (33 280 per stream and mini-batch of a checkpoint group). */
uint64_t ttt_b200_linear_backward_scratch_bytes(int B, int H, int checkpoint_group_size);

/* Take (read and clear) the device-side status word: 0, or TTT_B200_ERR_TIMEOUT if a kernel of
 * this process gave up on a bounded wait since the last take.  Call after synchronising. */
int ttt_b200_take_status(void);

/* Library / ABI version (major * 1000 + minor). */
int ttt_b200_version(void);

/* How many CTAs (1, 2 or 4) the forward (backward = 0) or backward (backward != 0) launcher gives each
 * (batch, head) stream of a problem with `streams` = B*H streams on the current device when the flags leave
 * the choice to it: four when the device runs that many clusters of four at once
 * (ttt_b200_cluster_capacity), else (forward only) two when those fit, else one (measured thresholds);
 * TTT_B200_CLUSTER overrides.  The reference fixes the split at compile time
 * (kernels/ttt/ttt.cu:11-12, kernels/ttt_backward/ttt.cu:12-16).  Returns -1 on error. */
int ttt_b200_pick_cluster(int streams, int backward);

/* How many clusters of `cluster` (2 or 4) CTAs of the forward (backward = 0) or backward kernel the current
 * device runs at the same time, from the CUDA occupancy query (a cluster lives inside one GPC, so this is
 * less than SMs / cluster when the GPCs' SM counts are not multiples of it: 32 clusters of four on a 148-SM
 * B200).  0 for other sizes or if the query fails.  No counterpart in the reference. */
int ttt_b200_cluster_capacity(int cluster, int backward);

/* Diagnostics (no counterpart in the reference): one CTA computes
 * D[M,N] = (+/-)A[M,K] * B[N,K]^T, `repeat` times accumulated, through the same shared-memory
 * descriptors, instruction descriptors and tensor-memory mapping as the operator kernels.
 * A, B, D are fp32 device arrays (operands are rounded to bf16).  repeat_and_mode: bits 0..7 the
 * repeat count, bit 8 = read the M = 64 result back with the 16x256b fragment loads.  Synchronises. */
int ttt_b200_umma_selftest(const float* A, const float* B, float* D, int M, int N, int K, int a_mn, int b_mn,
                           int neg_a, int repeat_and_mode, void* stream);

/* Diagnostics (no counterpart in the reference): exercise the failure path.  One CTA waits, with
 * the operator kernels' bounded wait, on a barrier nothing arrives on; after `limit_us` it gives
 * up, reports through the status word and exits normally.  Returns code 3 (the expected outcome)
 * and stores the time the kernel waited in *waited_ns (host pointer, may be NULL).  The context
 * stays usable.  Synchronises. */
int ttt_b200_wait_selftest(int limit_us, unsigned long long* waited_ns, void* stream);

/* Token layout transforms either side of the operator (no counterpart in the reference, which
 * asks its callers for contiguous [B, H, NC, 64, 64] tensors: README.md:98; a model's activations
 * are [B, T, H*64]).  pack: src[k] is [B][T][H][64] bf16, dst[k] becomes [B][H][T][64]; unpack is
 * the inverse (src[k] [B][H][T][64] -> dst[k] [B][T][H][64]).  Up to 4 tensors of the same shape
 * move in one launch (Q, K, V, upstream gradient / Out, dQ, dK, dV).  Out of place, device
 * pointers 16-byte aligned, T a multiple of 64, B*T*H < 2^31.  Stream-ordered, does not
 * synchronise.  Returns a TTT_B200_* code. */
int ttt_b200_pack_tokens(const void* const* src, void* const* dst, int n_tensors, int B, int T, int H,
                         void* stream);
int ttt_b200_unpack_tokens(const void* const* src, void* const* dst, int n_tensors, int B, int T, int H,
                           void* stream);

/* Layer-side kernels around the operator (no counterpart in the reference, whose callers compute
 * `last_eta` and post-process `XQW_batch` themselves: README.md:22-98).  Token-major tensors are a
 * model's [B][T][H] / [B][T][H*64] activations, head-major ones the operator's [B][H][T] / [B][H][T][64].
 * T a multiple of 64; B*T*H < 2^31; device pointers; stream-ordered, no synchronisation; TTT_B200_* codes.
 *
 * eta gate: last_eta[b][h][t] = scale * sigmoid(logits[b][t][h]), bf16 -> bf16 (H <= 256).  `scale` carries
 * the base learning rate, the 1 / 64 of the head dimension and the last row's token weight.  Its
 * backward: grad_logits[b][t][h] = grad_last_eta[b][h][t] * scale * s (1 - s), s = sigmoid(logits[b][t][h]). */
int ttt_b200_eta_gate(const void* logits, void* last_eta, float scale, int B, int T, int H, void* stream);
int ttt_b200_eta_gate_backward(const void* logits, const void* grad_last_eta, void* grad_logits, float scale, int B,
                               int T, int H, void* stream);
/* Output norm fused with the unpack: dst[b][t][:] = gamma * LayerNorm(src[b][:][t][:]) + beta over the H*64
 * features of a token; src = the operator's Out, bf16 [B][H][T][64]; gamma, beta fp32 [H*64]; dst bf16
 * [B][T][H*64]; statistics in fp32 (biased variance, eps inside the square root); H <= 64; pointers 16-byte
 * aligned; out of place.  `stats` (may be NULL): fp32 [B][T][2] receives (mean, 1 / std) per token for the
 * backward. */
int ttt_b200_unpack_layernorm(const void* src, const float* gamma, const float* beta, void* dst, float* stats,
                              float eps, int B, int T, int H, void* stream);
/* Its backward, fused with the pack of the gradient: from grad_y (bf16 [B][T][H*64]), x = the operator's Out
 * (bf16 [B][H][T][64]), gamma and the forward's `stats`, writes grad_x (bf16 [B][H][T][64]: the operator's
 * grad_L_XQW_mini_batch) and ADDS the parameter gradients into grad_gamma / grad_beta (fp32 [H*64]; the caller
 * zero-fills them; blocks add with atomics, so their last bits can differ from run to run). */
int ttt_b200_pack_layernorm_backward(const void* grad_y, const void* x, const float* gamma, const float* stats,
                                     void* grad_x, float* grad_gamma, float* grad_beta, int B, int T, int H,
                                     void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TTT_MLP_B200_H_ */
