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

/* ---- a whole stack of 3 x 3 layers -------------------------------------------------------------------
 * Replaces, for the backbone layers after the stem: the grad-enabled forward of the PPO minibatch update
 * (the loop of connect6/model.py:104-106 as run from connect6/train.py:1047-1048) and autograd's backward
 * through it (connect6/train.py:1115-1119).  Layer l (0-based, l < nlayers) maps channels[l] ->
 * channels[l + 1] with a 3 x 3 "same" convolution, bias and SiLU.  The forward call keeps every layer's
 * input as 16-bit channel-chunk planes inside the workspace; the backward call walks the stack from the top
 * with the gradient staying in that layout between layers, so only the stack's ends are converted from and
 * to NCHW fp32.  Per layer the arithmetic is c6_conv_layer_backward's.
 * Supported: 1 <= nlayers <= C6_MAX_LAYERS, n <= 32, every channel count <= 128.
 * workspace: c6_backbone_workspace_bytes() bytes (0: unsupported shape), 256-byte aligned, ZERO-FILLED before its
 * first use with a given shape; a forward call followed by its backward call must use the same workspace
 * with nothing else written to it in between; the pair keeps the zero padding intact, so the buffer can be
 * reused for the same shape without clearing.  The first 4 bytes are a status word like the engine's. */
int64_t c6_backbone_workspace_bytes(int32_t board_size, int32_t nlayers, const int32_t* channels /* HOST, nlayers + 1 */,
                                    int64_t B);

/* x fp32 [B, channels[0], n, n] -> y fp32 [B, channels[nlayers], n, n].  w and bias are HOST arrays of
 * nlayers DEVICE pointers (w[l] fp32 [channels[l+1], channels[l], 3, 3]; bias[l] fp32 [channels[l+1]] or null). */
int c6_backbone_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int64_t B,
                        const float* x, const float* const* w, const float* const* bias, float* y, void* workspace,
                        int64_t workspace_bytes, void* stream);

/* dy fp32 [B, channels[nlayers], n, n] = dL/dy of the preceding c6_backbone_forward on this workspace.
 * Outputs: dx fp32 [B, channels[0], n, n] (nullable); dw and db HOST arrays of nlayers DEVICE pointers
 * (dw[l] fp32 like w[l], db[l] fp32 [channels[l+1]]). */
int c6_backbone_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int64_t B,
                         const float* dy, float* dx, float* const* dw, float* const* db, void* workspace,
                         int64_t workspace_bytes, void* stream);

/* Last error text of the calling thread's most recent failing call of this header. Never null. */
const char* c6_train_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* C6_TRAIN_H_ */
