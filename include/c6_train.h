/*
 * c6_train.h -- C ABI of the training-side operators of the B200 (sm_100a) engine library: the
 * backward pass of backbone layers of the Connect6 policy/value CNN on tcgen05 tensor cores.
 *
 * The reference project (mgxmateusz/connect6) differentiates its network with PyTorch autograd inside
 * the PPO minibatch update (connect6/train.py:1032-1147: forward at 1047-1048, loss.backward() at
 * 1115-1119); per backbone layer y = silu(conv2d(x, W, b)) (connect6/model.py:104-106) autograd runs
 * cuDNN's data-gradient and weight-gradient convolutions plus elementwise kernels.  The entry points
 * below do that work, for one layer or for a stack of layers, with this library's own kernels.  Same conventions as c6_engine.h:
 * extern "C", plain DEVICE pointers and sizes, int status (0 = C6_OK), work enqueued on the stream
 * handed in (a cudaStream_t passed as void*), no synchronisation, no allocation.
 */
#ifndef C6_TRAIN_H_
#define C6_TRAIN_H_

#include <stdint.h>

#include "c6_engine.h" /* status codes */

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of workspace c6_conv_layer_backward needs for this shape (0 if the shape is not supported). */
int64_t c6_conv_layer_backward_workspace_bytes(int32_t board_size, int32_t kside, int32_t cin, int32_t cout,
                                               int64_t B);

/* Replaces: autograd's backward of one backbone layer y = silu(conv2d(x, W, b, padding = k/2))
 * (connect6/model.py:104-106, differentiated at connect6/train.py:1115-1119).
 *   x   fp32 [B, cin, n, n]   the layer's input (the previous layer's output)
 *   w   fp32 [cout, cin, k, k], bias fp32 [cout] (null = zeros)
 *   dy  fp32 [B, cout, n, n]  dL/dy
 * Outputs: dx fp32 [B, cin, n, n] (nullable: the first trainable layer needs none), dw fp32
 * [cout, cin, k, k], db fp32 [cout].
 * Arithmetic: bf16 operands, fp32 accumulation, like the forward engine's bf16 mode: the layer's
 * pre-activation is recomputed on the tensor cores and turned into dL/d(pre-activation) = dy * silu'(.)
 * in the same kernel's epilogue; dx is that gradient convolved with the flipped, transposed filter; dw is
 * a position-contracted GEMM summed over K slabs in a fixed order (reproducible, no atomics); db its
 * column sums.
 * Supported: k = 3, n <= 32, cin and cout <= 128 (C6_ERR_UNSUPPORTED otherwise).
 * workspace: c6_conv_layer_backward_workspace_bytes() bytes, 256-byte aligned, ZERO-FILLED before its
 * first use with a given (n, k, cin, cout, B); the call keeps the zero padding it relies on intact, so
 * the same buffer can be reused for the same shape without clearing.  The first 4 bytes are a status
 * word like the engine's (a bounded wait that ran out sets a bit; read it after synchronising). */
int c6_conv_layer_backward(int32_t device, int32_t board_size, int32_t kside, int32_t cin, int32_t cout,
                           int64_t B, const float* x, const float* w, const float* bias, const float* dy,
                           float* dx, float* dw, float* db, void* workspace, int64_t workspace_bytes,
                           void* stream);

/* ---- a whole stack of layers ------------------------------------------------------------------------
 * Replaces the grad-enabled forward of the PPO minibatch update through the backbone (the loop of
 * connect6/model.py:104-106 as run from connect6/train.py:1047-1048) and autograd's backward through it
 * (connect6/train.py:1115-1119).  Layer l (0-based, l < nlayers) maps channels[l] -> channels[l + 1] with a
 * "same" convolution, bias and SiLU.  stem_kside = 0: every layer is 3 x 3 (the layers after the stem; x is the
 * stem's output).  stem_kside = k > 0: layer 0 is the network's k x k first layer on the 3 input planes
 * (channels[0] = 3, connect6/model.py:22-23: k = 23), the others are 3 x 3; x is the network input.
 * The forward call keeps every layer's input as 16-bit channel-chunk planes inside the workspace (the stem's as
 * its x-expanded input planes); the backward call walks the stack from the top with the gradient staying in
 * that layout between layers, so only the stack's ends are NCHW fp32.  Arithmetic as in c6_conv_layer_backward
 * (bf16 operands, fp32 accumulation), except that no forward is recomputed: the forward call also keeps silu' of
 * every layer's pre-activation (one bf16 rounding), and a layer's data-gradient convolution multiplies by the
 * saved silu' of the layer below in its epilogue.  The stem's forward is the engine's direct stem, its weight
 * gradient the same position-contracted GEMM with 8 filter columns x 16 filter rows as the M side.
 * Supported: 1 <= nlayers <= C6_MAX_LAYERS, n <= 32, every 3 x 3 layer's channel counts <= 128; with a stem:
 * nlayers >= 2, k odd and <= 31, channels[1] <= 64.
 * workspace: c6_backbone_workspace_bytes() bytes (0: unsupported shape), 256-byte aligned, ZERO-FILLED before its
 * first use with a given shape; a forward call followed by its backward call must use the same workspace
 * with nothing else written to it in between; the pair keeps the zero padding intact, so the buffer can be
 * reused for the same shape without clearing.  The first 4 bytes are a status word like the engine's. */
int64_t c6_backbone_workspace_bytes(int32_t board_size, int32_t nlayers, const int32_t* channels /* HOST, nlayers + 1 */,
                                    int32_t stem_kside, int64_t B);

/* x fp32 [B, channels[0], n, n] -> y fp32 [B, channels[nlayers], n, n] (y nullable: the features then stay in the
 * workspace only, for c6_backbone_heads_forward).  w and bias are HOST arrays of
 * nlayers DEVICE pointers (w[l] fp32 [channels[l+1], channels[l], k_l, k_l]; bias[l] fp32 [channels[l+1]] or null). */
int c6_backbone_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                        int64_t B, const float* x, const float* const* w, const float* const* bias, float* y,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* c6_backbone_forward for a stack that starts with the stem (stem_kside > 0), fed with the environment's raw state
 * instead of network-input planes: boards int8 [num_envs, n, n], current_player and stones_left int8 [num_envs], and an
 * optional int64 index [B] selecting the boards (null: boards 0..B-1).  The planes of canonical_network_input
 * (connect6/vector_env.py:196-218; the PPO minibatch builds them at connect6/train.py:1038-1046 after gathering
 * buffer.boards[idx]) are formed inside the first kernel.  An index entry outside [0, num_envs) reads as an empty
 * board and raises C6_STATUS_BAD_INDEX in the workspace's status word. */
int c6_backbone_forward_boards(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels,
                               int32_t stem_kside, int64_t B, const int8_t* boards, const int8_t* current_player,
                               const int8_t* stones_left, int64_t num_envs, const int64_t* index, const float* const* w,
                               const float* const* bias, float* y, void* workspace, int64_t workspace_bytes, void* stream);

/* dy fp32 [B, channels[nlayers], n, n] = dL/dy of the preceding c6_backbone_forward on this workspace (null: the
 * gradient of the features is already in the workspace, left there by c6_backbone_heads_backward).
 * Outputs: dx fp32 [B, channels[0], n, n] (nullable; must be null with a stem: the network input has no gradient);
 * dw and db HOST arrays of nlayers DEVICE pointers (dw[l] fp32 like w[l], db[l] fp32 [channels[l+1]]). */
int c6_backbone_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                         int64_t B, const float* dy, float* dx, float* const* dw, float* const* db, void* workspace,
                         int64_t workspace_bytes, void* stream);

/* The two 1 x 1 heads on the features a preceding c6_backbone_forward left in the workspace
 * (connect6/model.py:70-75,108-110): logits fp32 [B, n*n] = policy_output(features) flattened, unmasked;
 * value fp32 [B] = tanh(mean over the board of value_output(features)).  wp, wv fp32 [channels[nlayers]]
 * (the [1, C, 1, 1] filters), bp, bv fp32 [1]; all DEVICE pointers. */
int c6_backbone_heads_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels,
                              int32_t stem_kside, int64_t B, const float* wp, const float* bp, const float* wv,
                              const float* bv, float* logits, float* value, void* workspace, int64_t workspace_bytes,
                              void* stream);

/* Backward of the heads: from dlogits fp32 [B, n*n], dvalue fp32 [B] and the forward's value fp32 [B] it writes the
 * gradient of the features into the workspace (where c6_backbone_backward with dy = null picks it up) and
 * dwp, dwv fp32 [channels[nlayers]], dbp, dbv fp32 [1] (fixed summation order: reproducible). */
int c6_backbone_heads_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels,
                               int32_t stem_kside, int64_t B, const float* wp, const float* wv, const float* dlogits,
                               const float* dvalue, const float* value, float* dwp, float* dbp, float* dwv, float* dbv,
                               void* workspace, int64_t workspace_bytes, void* stream);

/* Replaces: the loss of one PPO minibatch and autograd's backward from it to the network outputs
 * (connect6/train.py:1047-1086, 1115-1119): masked and temperature-scaled logits -> Categorical log-probability of
 * the taken action and entropy, clipped-ratio policy loss, squared-error value loss,
 *   loss = mean(policy) + value_coef * mean(value) - entropy_coef * mean(entropy),
 * plus the two statistics of connect6/train.py:1088-1094.
 *   logits fp32 [B, A] unmasked, legal uint8 [B, A] (non-zero = legal), actions int64 [B], old_logprob, advantages,
 *   returns, values fp32 [B]; temperature is floored at 1e-4 like the reference.
 * Outputs: stats fp32 [6] = {loss, policy loss, value loss, entropy, approx_kl, clipfrac}; dlogits fp32 [B, A] and
 * dvalues fp32 [B] = d loss / d logits, d loss / d values (zero at illegal actions).  Sums run in a fixed order.
 * A board without any legal action (a finished game: never part of a real minibatch) is given the uniform
 * distribution and no gradient.
 * workspace: 20 bytes per board.  All pointers DEVICE pointers. */
int c6_ppo_loss(int32_t device, int64_t B, int32_t A, const float* logits, const uint8_t* legal, const int64_t* actions,
                const float* old_logprob, const float* advantages, const float* returns, const float* values,
                float temperature, float clip_coef, float value_coef, float entropy_coef, float* stats, float* dlogits,
                float* dvalues, void* workspace, int64_t workspace_bytes, void* stream);

/* Replaces: nn.utils.clip_grad_norm_(model.parameters(), max_grad_norm) followed by torch.optim.AdamW.step()
 * (connect6/train.py:1121-1145, optimizer set up at connect6/train.py:476-481) for a whole parameter list, in two
 * launches.  sizes: HOST array of ntensors element counts; params, grads, exp_avg, exp_avg_sq: HOST arrays of
 * ntensors DEVICE pointers to fp32 tensors of those sizes (1 <= ntensors <= 48).  step: the 1-based number of this
 * update (bias corrections 1 - beta^step); or step_device (DEVICE, fp32 [1], nullable): the number of updates done so far,
 * kept on the device -- the call adds one and derives the bias corrections from it, `step` is ignored (for a call
 * sequence that is captured in a CUDA graph and replayed).  max_grad_norm <= 0: no clipping.
 * Effects: grads scaled in place by min(1, max_grad_norm / (total_norm + 1e-6)) like clip_grad_norm_; params and both
 * moments updated in place with PyTorch's AdamW arithmetic (decoupled weight decay); grad_norm (DEVICE, fp32 [1]) =
 * the total norm BEFORE clipping.  A non-finite norm leaves params and moments untouched (the reference raises there:
 * error_if_nonfinite=True); the caller sees it in grad_norm.  The sum of squares runs in a fixed order.
 * workspace: 592 bytes. */
int c6_clip_adamw_step(int32_t device, int32_t ntensors, const int64_t* sizes, float* const* params, float* const* grads,
                       float* const* exp_avg, float* const* exp_avg_sq, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float max_grad_norm, int64_t step, float* step_device, float* grad_norm,
                       void* workspace, int64_t workspace_bytes, void* stream);

/* Last error text of the calling thread's most recent failing call of this header. Never null. */
const char* c6_train_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* C6_TRAIN_H_ */
