/*
 * c6_engine.h -- C ABI of the B200 (sm_100a) inference engine for the Connect6
 * policy/value CNN.
 *
 * The reference project (mgxmateusz/connect6) is pure Python on PyTorch and has
 * no native interface; the entry points below are what a Python binding of its
 * inference hot path needs, one per reference function that it replaces.  Every
 * function is extern "C", takes plain pointers and sizes, returns an int status
 * (0 = C6_OK), never throws, never exits the process and never traps the device.
 * All data pointers are DEVICE pointers on the engine's device unless a
 * parameter is documented as host memory.  The caller owns every input and
 * output buffer; the engine owns packed weights and activation workspace only.
 * Work is enqueued on the stream handed in (a cudaStream_t passed as void*);
 * the engine never synchronises that stream except where documented
 * (workspace growth).  One host thread at a time per engine handle.
 */
#ifndef C6_ENGINE_H_
#define C6_ENGINE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define C6_MAX_LAYERS 16

/* status codes */
enum {
  C6_OK = 0,
  C6_ERR_ARG = 1,         /* bad argument (null pointer, bad size, bad enum)          */
  C6_ERR_CUDA = 2,        /* a CUDA runtime call failed; see c6_last_error            */
  C6_ERR_UNSUPPORTED = 3, /* architecture outside what the kernels implement          */
  C6_ERR_WEIGHTS = 4,     /* forward called before every layer/head received weights  */
  C6_ERR_DEVICE = 5       /* the device status word is non-zero (see c6_status)         */
};

/* bits of the device status word read by c6_status */
enum {
  C6_STATUS_WAIT_MASK = 63,   /* bits 0..5: a bounded wait inside a kernel ran out (which one)            */
  C6_STATUS_BAD_INDEX = 64,   /* c6_forward_step_boards: an index entry outside [0, num_envs), read as an
                                 empty board                                                               */
  C6_STATUS_F16_RANGE = 128   /* C6_PREC_F16: an activation exceeded +-65504 and was clamped                */
};

/* arithmetic mode of an engine */
enum {
  C6_PREC_BF16 = 0, /* bf16 operands, fp32 accumulate, tcgen05 tensor cores            */
  C6_PREC_FP32 = 1, /* fp32 operands and accumulate on CUDA cores (reference-exact mode) */
  C6_PREC_F16 = 2   /* fp16 weights and activations, fp32 accumulate, tcgen05 tensor cores: the
                       speed of the bf16 mode with 11-bit significands (tf32's width) instead of 8, for
                       callers that need the fp32 network's moves; activations beyond +-65504 are clamped
                       and reported through C6_STATUS_F16_RANGE                                         */
};

/* dtype of the network-input tensor x */
enum { C6_X_F32 = 0, C6_X_BF16 = 1 };

/* ids for c6_set_weights beyond the backbone layers 0..n_layers-1 */
enum { C6_HEAD_POLICY = 100, C6_HEAD_VALUE = 101 };

/* flags of the forward entry points */
enum {
  C6_FLAG_MASK_LOGITS = 1, /* write finfo(float32).min at occupied cells (model.py:123-125)   */
  C6_FLAG_INVERSE_MAP = 2  /* with orient: return logits / actions in canonical cell indices   */
};

typedef struct C6Desc {
  int32_t device;                  /* CUDA device ordinal                                   */
  int32_t board_size;              /* n; the board is n x n (19)                             */
  int32_t n_layers;                /* backbone depth, 1..C6_MAX_LAYERS                       */
  int32_t kernels[C6_MAX_LAYERS];  /* odd kernel size per layer (connect6/model.py:22)       */
  int32_t channels[C6_MAX_LAYERS]; /* output channels per layer (connect6/model.py:23)       */
  int32_t groups;                  /* G stacked models; 1 = a single PolicyValueNet          */
  int32_t precision;               /* C6_PREC_*                                              */
  int32_t max_chunk;               /* boards per internal pass, 0 = default                  */
} C6Desc;

typedef struct C6Engine C6Engine;

/* Library version (major*10000 + minor*100 + patch). */
int c6_version(void);

/* Replaces: PolicyValueNet.__init__ / build_model (connect6/model.py:26-81, 114-120) and
 * HistoricalPolicyEnsemble.__init__ (connect6/history.py:195-232) as far as device state goes.
 * Validates the architecture the same way (odd positive kernels, positive channels). */
int c6_create(const C6Desc* desc, C6Engine** out);

/* Replaces: the parameter storage read by nn.Conv2d (connect6/model.py:56-75) and the weight
 * stacking of connect6/history.py:224-240.  Packs one layer (or head) of one group from the
 * reference state_dict layout: w is fp32 [Cout,Cin,K,K] (heads: [1,C,1,1]), bias fp32 [Cout]
 * (heads: [1]; may be null = zeros).  Enqueued on `stream`; engines with groups == 1 in bf16 mode
 * also copy the small bias / head vectors back to the host and wait for `stream` once per call. */
int c6_set_weights(C6Engine* eng, int group, int layer_or_head, const float* w_oihw,
                   const float* bias, void* stream);

/* Optional: grow the workspace for `boards` boards now (synchronises the device once).
 * Forward calls grow it on demand otherwise. */
int c6_reserve(C6Engine* eng, int64_t boards);

/* Replaces: PolicyValueNet.forward (connect6/model.py:96-111), optionally fused with
 * mask_logits (connect6/model.py:123-125) and the per-board D4 view of
 * connect6/train.py:222-252.
 *   x       [B,3,n,n] contiguous NCHW, dtype x_dtype
 *   orient  nullable uint8 [B], D4 phase 0..7 per board (phase -> (k,flip) as train.py:216-219);
 *           the planes are transformed on the fly before the network sees them
 *   logits  nullable fp32 [B,n*n]; value nullable fp32 [B]
 *   flags   C6_FLAG_* ; occupancy for masking is plane0|plane1 of x */
int c6_forward(C6Engine* eng, const void* x, int x_dtype, int64_t B, const uint8_t* orient,
               float* logits, float* value, int flags, void* stream);

/* Replaces: one self-play inference step, connect6/train.py:792-795 = forward + _sample_actions
 * (connect6/train.py:195-203): masked logits / max(T,1e-4), log-softmax, one categorical draw
 * per board from a Philox4x32-10 stream keyed (seed, offset, board_index0 + b).
 *   action int64 [B]; logprob nullable fp32 [B]; value nullable fp32 [B];
 *   masked_logits nullable fp32 [B,n*n] (the masked, un-tempered logits) */
int c6_forward_step(C6Engine* eng, const void* x, int x_dtype, int64_t B, const uint8_t* orient,
                    int flags, float temperature, uint64_t seed, uint64_t offset,
                    int64_t board_index0, int64_t* action, float* logprob, float* value,
                    float* masked_logits, void* stream);

/* Replaces: canonical_network_input (connect6/vector_env.py:196-218), the batch gather
 * network_input[current_idx] (connect6/train.py:793) and the self-play step above in one call: the
 * three input planes are derived from the environment's raw state inside the first kernel, so the
 * fp32 planes (4.3 KB per board) never exist in memory.
 *   boards int8 [num_envs,n,n] (+1/-1/0), current_player int8 [num_envs] (+1/-1), stones_left int8
 *   [num_envs]; index nullable int64 [B]: board b of the batch is environment index[b] (null: b
 *   itself, then B <= num_envs).  An index entry outside [0, num_envs) is never dereferenced: that
 *   board is evaluated as an empty one and C6_STATUS_BAD_INDEX is raised in the status word.
 *   occupancy for masking is boards != 0; outputs as in c6_forward_step. */
int c6_forward_step_boards(C6Engine* eng, const int8_t* boards, const int8_t* current_player,
                           const int8_t* stones_left, int64_t num_envs, const int64_t* index, int64_t B,
                           const uint8_t* orient, int flags, float temperature, uint64_t seed,
                           uint64_t offset, int64_t board_index0, int64_t* action, float* logprob,
                           float* value, float* masked_logits, void* stream);

/* Replaces: HistoricalPolicyEnsemble.forward_grouped (connect6/history.py:276-303): G
 * independent models, T boards each, one launch sequence for all groups.
 *   x [G,T,3,n,n]; logits fp32 [G,T,n*n]; value nullable fp32 [G,T] (the reference ensemble
 *   has no value output; per-model PolicyValueNet.forward defines it) */
int c6_forward_grouped(C6Engine* eng, const void* x, int x_dtype, int64_t T, float* logits,
                       float* value, int flags, void* stream);

/* No counterpart in the reference.  Same result as c6_forward for an fp32-mode engine with
 * groups == 1, for callers that must not trigger a device allocation while they run: a host
 * thread inside a latency-critical loop (cudaMalloc may synchronise the whole device), a process
 * whose device memory is already handed out to another allocator or pool, or code that runs
 * where the CUDA allocator must not be entered at all.  c6_forward may grow the engine's
 * workspace with cudaMalloc on the first call or on a larger batch; this entry point never calls
 * cudaMalloc, cudaFree or any allocating library routine.  Its activations live in a fixed
 * 2.5 MiB array that is part of the library image on every GPU that loads it.
 *   Limit: B * n*n * (3 + 2*max(channels) + 2) floats must fit in 2.5 MiB (9 boards of the
 *   default 19x19 network); larger calls are rejected with C6_ERR_ARG and a message.
 *   The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *   that first call before any stream capture begins.
 *   All calls share the one array and it keeps the previous call's contents (every buffer is
 *   rewritten before it is read, so nothing needs clearing); two calls whose kernels overlap on
 *   the GPU -- different streams, or different engines on one device -- race on it. */
int c6_forward_noalloc(C6Engine* eng, const void* x, int x_dtype, int64_t B, const uint8_t* orient,
                       float* logits, float* value, int flags, void* stream);

/* Replaces: _sample_actions / _sample_actions_only on logits that already exist
 * (connect6/train.py:195-213).  legal is uint8/bool [B,A]; logprob nullable. */
int c6_sample_actions(const float* logits, const uint8_t* legal, int64_t B, int32_t A,
                      float temperature, uint64_t seed, uint64_t offset, int64_t board_index0,
                      int64_t* action, float* logprob, void* stream);

/* Replaces: mask_logits (connect6/model.py:123-125) for fp32 logits; `fill` is the dtype
 * minimum the caller's dtype implies (float32: -3.4028235e38, bfloat16: -3.3895314e38). */
int c6_mask_logits(const float* logits, const uint8_t* legal, int64_t count, float fill,
                   float* out, void* stream);

/* Replaces: _transform_actions / _inverse_transform_actions (connect6/train.py:233-277).
 * phase nullable uint8 [B] per action; if null `phase_all` applies to every action. */
int c6_transform_actions(const int64_t* actions, int64_t B, int32_t n, const uint8_t* phase,
                         int32_t phase_all, int32_t inverse, int64_t* out, void* stream);

/* Replaces: _transform_boards (connect6/train.py:222-230) on int8 boards [B,n,n]. */
int c6_transform_boards(const int8_t* boards, int64_t B, int32_t n, const uint8_t* phase,
                        int32_t phase_all, int8_t* out, void* stream);

/* Replaces: canonical_network_input (connect6/vector_env.py:196-218): int8 boards [B,n,n],
 * current_player int8 [B], stones_left int8 [B] -> fp32 planes [B,3,n,n]. */
int c6_network_input(const int8_t* boards, const int8_t* current_player, const int8_t* stones_left,
                     int64_t B, int32_t n, float* out, void* stream);

/* Per-kernel timing (no reference counterpart; the reference only has wall-clock phase timers,
 * connect6/train.py:586-1191).  While enabled, every forward-path launch is bracketed by a CUDA
 * event pair on the caller's stream.  c6_profile_read waits for the recorded events, adds the
 * elapsed milliseconds and launch counts per kind into the caller's HOST arrays (length
 * n_kinds >= C6_KIND_COUNT) and clears the record. */
enum {
  C6_KIND_PACK = 0,   /* input packing / view copy                      */
  C6_KIND_STEM = 1,   /* first backbone layer                           */
  C6_KIND_FINISH = 2, /* mask + log-softmax + draw + value              */
  C6_KIND_OTHER = 3,  /* fp32 head maps                                 */
  C6_KIND_CONV0 = 8,  /* backbone layer l >= 1 is kind C6_KIND_CONV0+l  */
  C6_KIND_COUNT = 8 + C6_MAX_LAYERS
};
int c6_profile_enable(C6Engine* eng, int on); /* 0 off, 1 events, 2 events + in-kernel wait counters (c6_debug.h) */
int c6_profile_read(C6Engine* eng, float* ms_per_kind, int64_t* launches_per_kind, int n_kinds);

/* Reads the device status word (host int, C6_STATUS_* bits).  Non-zero returns C6_ERR_DEVICE: a
 * bounded wait inside a kernel ran out (the kernels then skip their work instead of hanging), a
 * gather index was out of range, or the fp16 mode clamped an activation.  The caller must have
 * synchronised the stream it used. */
int c6_status(C6Engine* eng, int* device_status);

/* Clears the device status word (synchronous) after the caller has dealt with a non-zero status. */
int c6_clear_status(C6Engine* eng);

/* Number of kernel launches the engine has enqueued since creation (host counter). */
int64_t c6_launch_count(const C6Engine* eng);

/* Bytes of device memory the engine currently owns (weights + workspace). */
int64_t c6_device_bytes(const C6Engine* eng);

/* Last error text of this engine (or of c6_create when eng is null). Never null. */
const char* c6_last_error(const C6Engine* eng);

/* Frees everything the engine owns. */
int c6_destroy(C6Engine* eng);

#ifdef __cplusplus
}
#endif
#endif /* C6_ENGINE_H_ */
