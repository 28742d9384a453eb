// Host side of the engine and its C ABI (see include/c6_engine.h for the contract).
//
// One engine = one architecture (board, kernels, channels), G stacked weight sets and one
// arithmetic mode.  A forward call is cut into passes of at most `chunk` boards; a pass is a
// fixed launch sequence on the caller's stream:
//   bf16 / fp16:  pack input -> stem GEMM (tcgen05) -> k x k conv layers (tcgen05, last one fused
//                 with both heads) -> finishing kernel; engines with several weight sets run the
//                 first layer of small calls straight from the filter instead (conv_tc_kernel's
//                 stem mode behind its own pack kernel)
//   fp32:         view copy -> direct conv layers (CUDA cores) -> head maps -> finishing kernel
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/c6_debug.h"
#include "../../include/c6_engine.h"
#include "c6_aux_kernels.cuh"
#include "c6_conv2_fused.cuh"
#include "c6_conv_tc.cuh"
#include "c6_fp32_kernels.cuh"
#include "c6_host_plan.h"
#include "c6_stem_tc.cuh"

using namespace c6;

namespace {

thread_local std::string g_create_error = "";

}  // namespace

struct C6Engine {
  C6Desc d{};
  int device = 0, sms = 148;
  int n = 0, cells = 0, pad = 1, wp = 0, slots = 0, halo = 0, halo_rows = 0, front = 0;
  int L = 0, G = 1, prec = 0, chunk = 0;
  int f16 = 0;                      // tensor-core modes: 16-bit operand type, 0 = bf16, 1 = fp16
  std::vector<LayerPlan> lp;
  int cmax_p = 0, cmax = 0;
  // stem GEMM plan
  int kc_short = 0;                 // stem K chunks of input planes 0 and 1; kc0 - kc_short chunks hold plane 2
  unsigned int stem_epoch = 0;      // pass counter: tells the stem whether THIS pass saw a non-constant third plane
  unsigned int* p2_epoch = nullptr; // device word written by the input pack kernel
  uint8_t* occ = nullptr;           // [kc_short][mrows] occupancy bits of planes 0/1 (workspace, written by the input pack kernel)
  int kc0 = 0, nt = 0, ntiles = 0, ntot = 0, stem_stages = 0, stem_smem = 0, stem_acc_stride = 0,
      stem_tmem_cols = 0, stem_kcs = 4, stem_pair = 0;
  // direct stem (conv_tc_kernel's stem mode), taken by passes of at most sd_max_boards boards per group
  int sd_ok = 0, sd_max_boards = 32, sd_min_groups = 2, sd_hx = 0, sd_wi = 0, sd_slots = 0, sd_halo_b = 0, sd_halo_a = 0, sd_front = 0;
  LayerPlan sdp;                    // its pipeline plan
  uint4* w_sd = nullptr;            // [G][ci][ky][kx block][2][cout_p] filter rows
  uint4* w_sd_pair = nullptr;       // the same split in two row halves for CTA pairs
  uint4* xe = nullptr;              // workspace: 3 x-expanded input planes
  long long xe_plane_rows = 0, sd_last_group_pos = -1;
  long long xk_rows = 0;              // rows per plane of xk / occ as allocated
  long long xe_cap = 0, xk_cap = 0;   // boards per group the stem operands of the two paths are sized for
  // weights
  uint4* wt = nullptr;              // [G][kc0][ntot] Toeplitz rows of the stem GEMM: 27 MB per model for the default
                                    // net, so they are allocated and expanded only when a pass first needs them
  float* w0_raw = nullptr;          // [G][cout*3*k0*k0] the first layer's filter as received (source of that expansion)
  std::vector<uint8_t> wt_fresh;    // [G] Toeplitz rows match w0_raw
  std::vector<uint4*> wconv;        // per layer [G][rows]
  std::vector<uint4*> wconv_pair;   // per layer, pair mode: [G][2 halves][rows/2]
  bool pair_mode = false;           // tile counts are kept even so that layers may run as CTA pairs
  std::vector<float*> bias;         // per layer [G][cout_p] (fp32 mode: [G][cout])
  std::vector<float*> wraw;         // fp32 mode: per layer [G][cout*cin*k*k]
  float *head_wp = nullptr, *head_wv = nullptr, *pol_bias = nullptr, *val_bias = nullptr;
  std::vector<uint8_t> have;        // [G][L+2]
  // host mirrors of bias / head vectors of single-model engines (passed to kernels by value)
  std::vector<std::vector<float>> h_bias;   // per layer, padded
  std::vector<float> h_wp, h_wv;
  // workspace (capacity in boards per group)
  long long cap = 0;
  long long plane_rows = 0, mrows = 0;
  uint4* xk = nullptr;
  uint4* act[2] = {nullptr, nullptr};
  float* f32buf[2] = {nullptr, nullptr};
  float* f32x = nullptr;
  float *logit_raw = nullptr, *vmap = nullptr;
  long long last_group_pos = -1;
  int* status_dev = nullptr;
  long long* wait_dev = nullptr;   // [4] pipeline wait counters of CTA 0 (conv kernel)
  long long launches = 0;
  // optional per-kernel timing: event pairs recorded around every launch
  bool profiling = false;
  int fuse12 = 0;                  // layers 1 and 2 run as one kernel (conv2_fused_kernel), the intermediate in shared memory
  int fuse12_smem = 0;
  bool dependent_launch = true;    // programmatic dependent launch along the kernel chain (C6_DEPENDENT_LAUNCH=0 turns it off)
  bool wait_counters = false;      // level 2: also the in-kernel pipeline wait counters
  struct ProfRec { int kind; cudaEvent_t a, b; };
  std::vector<ProfRec> prof;
  std::vector<cudaEvent_t> ev_pool;
  long long dev_bytes = 0;
  long long ws_bytes = 0;
  std::string err = "";
};

namespace {

int fail(C6Engine* e, int code, const std::string& msg) {
  if (e) e->err = msg; else g_create_error = msg;
  return code;
}

#define C6_CUDA(e, call)                                                                         \
  do {                                                                                           \
    cudaError_t _st = (call);                                                                    \
    if (_st != cudaSuccess)                                                                      \
      return fail((e), C6_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_st));        \
  } while (0)

#define C6_LAUNCHED(e, name)                                                                     \
  do {                                                                                           \
    cudaError_t _st = cudaGetLastError();                                                        \
    if (_st != cudaSuccess)                                                                      \
      return fail((e), C6_ERR_CUDA, std::string("launch ") + name + ": " + cudaGetErrorString(_st)); \
    (e)->launches++;                                                                             \
  } while (0)

cudaEvent_t prof_event(C6Engine* e) {
  if (!e->ev_pool.empty()) {
    cudaEvent_t ev = e->ev_pool.back();
    e->ev_pool.pop_back();
    return ev;
  }
  cudaEvent_t ev = nullptr;
  cudaEventCreate(&ev);
  return ev;
}
// Scope object: records an event pair on `st` around the launches made while it lives.
struct ProfScope {
  C6Engine* e;
  cudaStream_t st;
  cudaEvent_t b = nullptr;
  ProfScope(C6Engine* e_, int kind, cudaStream_t st_) : e(e_), st(st_) {
    if (!e->profiling) return;
    cudaEvent_t a = prof_event(e);
    b = prof_event(e);
    cudaEventRecord(a, st);
    e->prof.push_back({kind, a, b});
  }
  ~ProfScope() {
    if (b) cudaEventRecord(b, st);
  }
};

// Opt every instantiation of the k x k kernel for one filter side into the large dynamic shared memory.
template <int KS, bool F16, bool TIMED>
bool conv_smem_opt_in2() {
  return cudaFuncSetAttribute(conv_tc_kernel<KS, false, F16, TIMED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) == cudaSuccess &&
         cudaFuncSetAttribute(conv_tc_kernel<KS, true, F16, TIMED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) == cudaSuccess;
}
template <int KS>
bool conv_smem_opt_in() {
  bool ok = conv_smem_opt_in2<KS, false, false>() && conv_smem_opt_in2<KS, true, false>();
#ifdef C6_TIMED_BUILD
  ok = ok && conv_smem_opt_in2<KS, false, true>() && conv_smem_opt_in2<KS, true, true>();
#endif
  return ok;
}

// The instantiation for (clock counters, CTA pairs, fp16, filter side: 0 generic, 1, 3, 5).
using ConvKernel = void (*)(ConvTcParams);
template <bool PAIR, bool F16, bool TIMED>
ConvKernel conv_kernel_ks(int k) {
  return k == 1 ? conv_tc_kernel<1, PAIR, F16, TIMED> : k == 3 ? conv_tc_kernel<3, PAIR, F16, TIMED>
       : k == 5 ? conv_tc_kernel<5, PAIR, F16, TIMED> : conv_tc_kernel<0, PAIR, F16, TIMED>;
}
template <bool TIMED>
ConvKernel conv_kernel_pf(bool pair, bool f16, int k) {
  return pair ? (f16 ? conv_kernel_ks<true, true, TIMED>(k) : conv_kernel_ks<true, false, TIMED>(k))
              : (f16 ? conv_kernel_ks<false, true, TIMED>(k) : conv_kernel_ks<false, false, TIMED>(k));
}
ConvKernel conv_kernel_for(bool timed, bool pair, bool f16, int k) {
#ifdef C6_TIMED_BUILD
  if (timed) return conv_kernel_pf<true>(pair, f16, k);
#endif
  (void)timed;
  return conv_kernel_pf<false>(pair, f16, k);
}

template <typename T>
int dev_alloc(C6Engine* e, T** p, size_t count, bool zero, long long* tally) {
  *p = nullptr;
  if (count == 0) return C6_OK;
  C6_CUDA(e, cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)));
  if (zero) C6_CUDA(e, cudaMemset(*p, 0, count * sizeof(T)));
  e->dev_bytes += (long long)(count * sizeof(T));
  if (tally) *tally += (long long)(count * sizeof(T));
  return C6_OK;
}

struct Geometry {
  int tiles_per_group;
  int tiles_per_board;        // > 0: tiles are aligned to board images and skip each image's all-padding tail
  long long group_pos;        // positions reserved per group
  int mrows_per_group;
};

Geometry geometry(const C6Engine* e, long long nb) {
  Geometry g;
  // Positions of a board image that hold cells: rows 0..n-1 of pitch wp, i.e. (n-1)*wp + n of the
  // wp*wp slots.  When whole 128-position tiles cover them in fewer positions than the image has
  // (19x19: 3 tiles = 384 of 400), tiles are aligned to the images and the tail is never computed.
  const int used = (e->n - 1) * e->wp + e->n;
  const int tpb = (used + 127) / 128;
  g.tiles_per_board = tpb * 128 < e->slots ? tpb : 0;
  g.tiles_per_group = g.tiles_per_board ? (int)(nb * tpb) : (int)((nb * e->slots + 127) / 128);
  if (e->pair_mode) g.tiles_per_group += g.tiles_per_group & 1;   // CTA pairs take tiles two at a time
  // the odd tile added for a pair starts a board image of its own: reserve it
  g.group_pos = g.tiles_per_board
                    ? round_up_ll((long long)((g.tiles_per_group + tpb - 1) / tpb) * e->slots, 128)
                    : (long long)g.tiles_per_group * 128;
  g.mrows_per_group = (int)round_up_ll(nb, e->stem_pair ? 256 : 128);   // CTA pairs take 256 boards per tile
  return g;
}

// Tiles of the direct stem walk the INPUT geometry (pitch sd_wi, sd_slots per board image).
Geometry geometry_sd(const C6Engine* e, long long nb) {
  Geometry g;
  const int used = (e->n - 1) * e->sd_wi + e->n;
  const int tpb = (used + 127) / 128;
  g.tiles_per_board = tpb * 128 < e->sd_slots ? tpb : 0;
  g.tiles_per_group = g.tiles_per_board ? (int)(nb * tpb) : (int)((nb * e->sd_slots + 127) / 128);
  if (e->sdp.pair) g.tiles_per_group += g.tiles_per_group & 1;
  g.group_pos = g.tiles_per_board
                    ? round_up_ll((long long)((g.tiles_per_group + tpb - 1) / tpb) * e->sd_slots, 128)
                    : (long long)g.tiles_per_group * 128;
  g.mrows_per_group = 0;
  return g;
}

void free_workspace(C6Engine* e) {
  cudaFree(e->xe);
  e->xe = nullptr;
  cudaFree(e->xk);
  cudaFree(e->occ);
  e->occ = nullptr;
  cudaFree(e->act[0]);
  cudaFree(e->act[1]);
  cudaFree(e->f32buf[0]);
  cudaFree(e->f32buf[1]);
  cudaFree(e->f32x);
  cudaFree(e->logit_raw);
  cudaFree(e->vmap);
  e->xk = nullptr;
  e->act[0] = e->act[1] = nullptr;
  e->f32buf[0] = e->f32buf[1] = nullptr;
  e->f32x = nullptr;
  e->logit_raw = e->vmap = nullptr;
  e->dev_bytes -= e->ws_bytes;
  e->ws_bytes = 0;
  e->cap = 0;
  e->xe_cap = e->xk_cap = 0;
}

// Grow the workspace to hold `nb` boards per group; `direct` says which stem path the pass takes (its
// operand buffers are only allocated for the path in use).  Synchronises the device when anything grows.
int ensure_workspace(C6Engine* e, long long nb, bool direct) {
  const bool tc = e->prec != C6_PREC_FP32;
  if (nb <= e->cap && (!tc || (direct ? nb <= e->xe_cap : nb <= e->xk_cap))) return C6_OK;
  C6_CUDA(e, cudaDeviceSynchronize());
  int rc;
  if (nb > e->cap) {
    free_workspace(e);
    const Geometry g = geometry(e, nb);
    if (tc) {
      e->plane_rows = (long long)e->front + (long long)e->G * g.group_pos + e->halo_rows;
      e->mrows = (long long)e->G * g.mrows_per_group;
      const size_t act_rows = (size_t)(e->cmax_p / 8) * e->plane_rows;
      if ((rc = dev_alloc(e, &e->act[0], act_rows, true, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->act[1], act_rows, true, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->logit_raw, (size_t)e->G * g.group_pos, true, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->vmap, (size_t)e->G * g.group_pos, true, &e->ws_bytes))) return rc;
    } else {
      const size_t boards = (size_t)e->G * nb;
      if ((rc = dev_alloc(e, &e->f32x, boards * 3 * e->cells, false, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->f32buf[0], boards * e->cmax * e->cells, false, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->f32buf[1], boards * e->cmax * e->cells, false, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->logit_raw, boards * e->cells, false, &e->ws_bytes))) return rc;
      if ((rc = dev_alloc(e, &e->vmap, boards * e->cells, false, &e->ws_bytes))) return rc;
    }
    e->cap = nb;
    e->last_group_pos = -1;
  }
  if (tc && direct && nb > e->xe_cap) {
    // x-expanded input planes of the direct stem
    if (e->xe) { e->ws_bytes -= (long long)(3 * e->xe_plane_rows * sizeof(uint4)); e->dev_bytes -= (long long)(3 * e->xe_plane_rows * sizeof(uint4)); }
    cudaFree(e->xe);
    e->xe = nullptr;
    const Geometry gs = geometry_sd(e, nb);
    e->xe_plane_rows = (long long)e->sd_front + (long long)e->G * gs.group_pos + e->sd_halo_a + 128 + 16;
    if ((rc = dev_alloc(e, &e->xe, (size_t)3 * e->xe_plane_rows, true, &e->ws_bytes))) return rc;
    e->xe_cap = nb;
    e->sd_last_group_pos = -1;
  }
  if (tc && !direct && e->xk_cap < e->cap) {
    // operand rows and occupancy bits of the stem GEMM, sized like the activation planes
    if (e->xk) {
      const long long old = (long long)((size_t)e->kc0 * e->xk_rows * sizeof(uint4) + (size_t)e->kc_short * e->xk_rows);
      e->ws_bytes -= old;
      e->dev_bytes -= old;
    }
    cudaFree(e->xk);
    cudaFree(e->occ);
    e->xk = nullptr;
    e->occ = nullptr;
    e->xk_rows = e->mrows;
    if ((rc = dev_alloc(e, &e->xk, (size_t)e->kc0 * e->mrows, true, &e->ws_bytes))) return rc;
    if ((rc = dev_alloc(e, &e->occ, (size_t)e->kc_short * e->mrows, true, &e->ws_bytes))) return rc;
    e->xk_cap = e->cap;
  }
  return C6_OK;
}

int fp32_cit(const LayerPlan& l) { return l.k <= 5 ? std::min(l.cin, 16) : std::min(l.cin, 4); }
size_t fp32_smem(const C6Engine* e, const LayerPlan& l) {
  const int cit = fp32_cit(l), np = e->n + 2 * (l.k / 2);
  const size_t in_floats = ((size_t)cit * np * np + 3) & ~(size_t)3;  // weights start 16-byte aligned
  return (in_floats + (size_t)cit * l.k * l.k * kFp32CoT) * sizeof(float);
}

// ---- scratch for the entry point that must not allocate -------------------------------------------
// Held by every GPU that loads this library until the process exits.  In host code the symbol
// below is only a host-side stand-in; kernels get the device address from cudaGetSymbolAddress.
constexpr size_t kNoAllocScratchBytes = 2621440;  // 2.5 MiB
constexpr size_t kNoAllocScratchFloats = kNoAllocScratchBytes / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {nullptr};

InputSrc input_of(const struct RunArgs& a);

struct RunArgs {
  const void* x = nullptr;
  int x_bf16 = 0;
  const int8_t* boards = nullptr;       // board-input mode (x stays null)
  const int8_t* player = nullptr;
  const int8_t* stones_left = nullptr;
  const long long* index = nullptr;
  long long num_envs = 0;               // board-input mode: environments behind the state pointers
  long long T = 0;  // boards per group
  const uint8_t* orient = nullptr;
  float* logits = nullptr;
  float* value = nullptr;
  int flags = 0;
  int do_sample = 0;
  float temperature = 1.f;
  unsigned long long seed = 0, offset = 0;
  long long board_index0 = 0;
  long long* action = nullptr;
  float* logprob = nullptr;
  int direct_stem = 0;       // this call's first layer runs straight from the filter (set by run())
  int stop_layer = -1;       // debug: stop after this backbone layer
  float* layer_out = nullptr;  // debug: fp32 NCHW output of stop_layer
};

InputSrc input_of(const RunArgs& a) {
  InputSrc in{};
  in.x = a.x;
  in.x_bf16 = a.x_bf16;
  in.boards = a.boards;
  in.player = a.player;
  in.stones_left = a.stones_left;
  in.index = a.index;
  in.num_envs = a.num_envs;
  return in;
}

int launch_finish(C6Engine* e, const RunArgs& a, long long t0, int nb, long long group_stride,
                  int board_stride, int pitch, const uint8_t* occ, int mrows_per_group, cudaStream_t st) {
  FinishParams f{};
  f.occ = occ;
  f.occ_stride = e->mrows;
  f.mrows_per_group = mrows_per_group;
  f.logit_raw = e->logit_raw;
  f.vmap = a.value ? e->vmap : nullptr;
  f.group_stride = group_stride;
  f.board_stride = board_stride;
  f.pitch = pitch;
  f.pol_bias = e->pol_bias;
  f.val_bias = e->val_bias;
  f.in = input_of(a);
  f.orient = a.orient;
  f.x_group_stride = a.T;
  f.board0 = t0;
  f.n = e->n;
  f.n_magic = 65536 / e->n + 1;
  f.n_actions = e->cells;
  f.nb = nb;
  f.flags = a.flags;
  f.do_sample = a.do_sample;
  f.temperature = a.temperature;
  f.seed = a.seed;
  f.offset = a.offset;
  f.board_index0 = a.board_index0;
  f.logits_out = a.logits;
  f.value_out = a.value;
  f.action_out = a.action;
  f.logprob_out = a.logprob;
  {
    ProfScope _ps(e, C6_KIND_FINISH, st);
    launch_chain(finish_kernel_for(f.n_actions), finish_blocks(nb), (unsigned)e->G, kFinishThreads, 0, st, false,
                 e->dependent_launch, f);
  }
  C6_LAUNCHED(e, "finish_kernel");
  return C6_OK;
}

// Toeplitz rows of weight set `group` from its stored filter (enqueued on `st`).
int expand_toeplitz(C6Engine* e, int group, cudaStream_t st) {
  const LayerPlan& p = e->lp[0];
  const long long total = (long long)e->kc0 * e->ntot;
  pack_stem_toeplitz_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      e->w0_raw + (size_t)group * p.cout * 3 * p.k * p.k, e->wt + (size_t)group * e->kc0 * e->ntot, p.cout, p.k, e->n,
      p.cout_p, e->kc0, e->kc_short, e->ntot, e->nt, e->stem_pair ? 2 : 1, e->f16);
  C6_LAUNCHED(e, "pack_stem_toeplitz_kernel");
  e->wt_fresh[group] = 1;
  return C6_OK;
}

// The stem GEMM's operand exists and is current (allocates on first use; synchronises the device then).
int ensure_toeplitz(C6Engine* e, cudaStream_t st) {
  if (!e->wt) {
    C6_CUDA(e, cudaDeviceSynchronize());
    int rc = dev_alloc(e, &e->wt, (size_t)e->G * e->kc0 * e->ntot, true, nullptr);
    if (rc) return rc;
  }
  for (int g = 0; g < e->G; ++g)
    if (!e->wt_fresh[g]) {
      int rc = expand_toeplitz(e, g, st);
      if (rc) return rc;
    }
  return C6_OK;
}

// First backbone layer through conv_tc_kernel's stem mode: pack the x-expanded input planes, then one
// implicit GEMM straight from the filter into act[0].
int run_direct_stem(C6Engine* e, const RunArgs& a, long long t0, int nb, const Geometry& g, cudaStream_t st) {
  const Geometry gs = geometry_sd(e, nb);
  if (gs.group_pos != e->sd_last_group_pos) {
    // image bases moved: rows between and behind the images must read as zero padding again
    C6_CUDA(e, cudaMemsetAsync(e->xe, 0, (size_t)3 * e->xe_plane_rows * sizeof(uint4), st));
    e->sd_last_group_pos = gs.group_pos;
  }
  {
    ProfScope _ps(e, C6_KIND_PACK, st);
    pack_stem_direct_input_kernel<<<dim3((unsigned)nb, (unsigned)e->G), kPackDirectThreads, 0, st>>>(
        input_of(a), a.orient, e->xe, e->xe_plane_rows, e->sd_front, (int)gs.group_pos, e->sd_wi, e->sd_slots, e->n, nb,
        a.T, t0, e->f16, e->status_dev);
    C6_LAUNCHED(e, "pack_stem_direct_input_kernel");
  }
  const LayerPlan& lp = e->sdp;
  ConvTcParams p{};
  p.in = e->xe;
  p.in_plane_rows = e->xe_plane_rows;
  p.out = e->act[0];
  p.plane_rows = e->plane_rows;
  p.w = e->w_sd;
  p.w_pair = e->w_sd_pair;
  p.bias = e->bias[0];
  p.status = e->status_dev;
  p.front = e->sd_front;
  p.halo_rows = e->sd_halo_b;
  p.halo_after = e->sd_halo_a;
  p.cin = 48;                       // three pipeline steps, one input plane each
  p.n = lp.cout_p;
  p.kside = lp.k;
  p.ntaps = lp.k * e->sd_hx;
  p.planes_step = 1;
  p.stem = 1;
  p.stem_hx = e->sd_hx;
  p.a_lbo_rows = 8;
  p.wp = e->sd_wi;
  p.slots = e->sd_slots;
  p.bsize = e->n;
  p.nboards = nb;
  p.tiles_per_group = gs.tiles_per_group;
  p.tiles_per_board = gs.tiles_per_board;
  p.group_pos = (int)gs.group_pos;
  p.out_front = e->front;
  p.out_wp = e->wp;
  p.out_slots = e->slots;
  p.out_group_pos = (int)g.group_pos;
  p.ctas_per_group = std::max(1, std::min(e->sms / e->G, gs.tiles_per_group));
  if (lp.pair) p.ctas_per_group = std::max(2, p.ctas_per_group & ~1);
  p.resident = lp.resident;
  p.nstages = lp.nstages;
  p.nissue = lp.nissue;
  p.spi = lp.spi;
  p.qps = 1;
  p.use_const = e->G == 1 ? 1 : 0;
  if (p.use_const) std::memcpy(p.c_hbias, e->h_bias[0].data(), sizeof(p.c_hbias));
  p.acc_stride = lp.acc_stride;
  p.nacc = lp.nacc;
  p.tmem_cols = lp.tmem_cols;
  {
    ProfScope _ps(e, C6_KIND_STEM, st);
    launch_chain(conv_kernel_for(false, lp.pair != 0, e->f16 != 0, 0), (unsigned)(e->G * p.ctas_per_group), 1u, kConvThreads,
                 (size_t)lp.smem, st, lp.pair != 0, e->dependent_launch, p);
  }
  C6_LAUNCHED(e, "conv_tc_kernel (direct stem)");
  return C6_OK;
}

int run_pass_bf16(C6Engine* e, const RunArgs& a, long long t0, int nb, cudaStream_t st) {
  const Geometry g = geometry(e, nb);
  if (e->G > 1 && g.group_pos != e->last_group_pos) {
    // group bases moved: the zero padding between boards must be re-established
    const size_t bytes = (size_t)(e->cmax_p / 8) * e->plane_rows * sizeof(uint4);
    C6_CUDA(e, cudaMemsetAsync(e->act[0], 0, bytes, st));
    C6_CUDA(e, cudaMemsetAsync(e->act[1], 0, bytes, st));
  }
  e->last_group_pos = g.group_pos;

  // few boards per weight set: the first layer straight from the filter (conv_tc_kernel's stem mode);
  // otherwise the Toeplitz GEMM
  const bool direct_stem = a.direct_stem != 0;
  int cur = 0;
  if (direct_stem) {
    int rc = run_direct_stem(e, a, t0, nb, g, st);
    if (rc) return rc;
  } else {
    {
      int rc = ensure_toeplitz(e, st);
      if (rc) return rc;
    }
    {  // input planes
      const long long total = (long long)e->kc0 * nb;
      ProfScope _ps(e, C6_KIND_PACK, st);
      pack_stem_input_kernel<<<dim3((unsigned)((total + 255) / 256), (unsigned)e->G), 256, 0, st>>>(
          input_of(a), a.orient, e->xk, e->mrows, g.mrows_per_group, e->kc0, e->kc_short, e->n, nb, a.T, t0,
          ++e->stem_epoch, e->p2_epoch, e->occ, e->f16, e->status_dev);
      C6_LAUNCHED(e, "pack_stem_input_kernel");
    }
  }
  // stem GEMM -> act[0]
  auto launch_stem = [&]() -> int {
      StemTcParams p{};
      p.xk = e->xk;
      p.wt = e->wt;
      p.bias = e->bias[0];
      p.out = e->act[0];
      p.status = e->status_dev;
      p.wait_cycles = e->wait_counters ? e->wait_dev : nullptr;
      p.plane_rows = e->plane_rows;
      p.mrows = e->mrows;
      p.mrows_per_group = g.mrows_per_group;
      p.front = e->front;
      p.group_pos = (int)g.group_pos;
      p.kc = e->kc0;
      p.kc_short = e->kc_short;
      p.p2_epoch = e->p2_epoch;
      p.epoch = e->stem_epoch;
      p.kcs = e->stem_kcs;
      p.ntot = e->ntot;
      p.nt = e->nt;
      p.ntiles = e->ntiles;
      p.mtiles = g.mrows_per_group / 128;
      p.groups = e->G;
      p.c1 = e->lp[0].cout_p;
      p.bsize = e->n;
      p.wp = e->wp;
      p.slots = e->slots;
      p.nboards = nb;
      p.nstages = e->stem_stages;
      p.acc_stride = e->stem_acc_stride;
      p.tmem_cols = e->stem_tmem_cols;
      ProfScope _ps(e, C6_KIND_STEM, st);
      if (e->stem_pair) {
        const long long items = (long long)e->G * (p.mtiles / 2) * p.ntiles;
        const int grid = 2 * (int)std::min<long long>(e->sms / 2, items);
        launch_chain(e->f16 ? stem_tc_kernel<true, true> : stem_tc_kernel<true, false>, (unsigned)grid, 1u, kStemThreads,
                     (size_t)e->stem_smem, st, true, e->dependent_launch, p);
      } else {
        const long long items = (long long)e->G * p.mtiles * p.ntiles;
        const int grid = (int)std::min<long long>(e->sms, items);
        launch_chain(e->f16 ? stem_tc_kernel<false, true> : stem_tc_kernel<false, false>, (unsigned)grid, 1u, kStemThreads,
                     (size_t)e->stem_smem, st, false, e->dependent_launch, p);
      }
      C6_LAUNCHED(e, "stem_tc_kernel");
      return C6_OK;
  };
  // backbone layer l: act[cur] -> act[cur ^ 1]
  auto launch_layer = [&](int l) -> int {
    const LayerPlan& lp = e->lp[l];
    ConvTcParams p{};
    p.in = e->act[cur];
    p.out = e->act[cur ^ 1];
    p.w = e->wconv[l];
    p.bias = e->bias[l];
    p.head = (l == e->L - 1 && a.stop_layer < 0) ? 1 : 0;
    p.head_wp = e->head_wp;
    p.head_wv = e->head_wv;
    p.logit_raw = e->logit_raw;
    p.vmap = e->vmap;
    p.status = e->status_dev;
    p.wait_cycles = e->wait_counters ? e->wait_dev : nullptr;
    p.plane_rows = e->plane_rows;
    p.front = e->front;
    p.halo_rows = e->halo_rows;
    p.cin = lp.cin_p;
    p.n = lp.cout_p;
    p.kside = lp.k;
    p.in_plane_rows = e->plane_rows;
    p.ntaps = lp.k * lp.k;
    p.halo_after = e->halo_rows;
    p.planes_step = 2 * lp.qps;
    p.wp = e->wp;
    p.slots = e->slots;
    p.bsize = e->n;
    p.nboards = nb;
    p.tiles_per_group = g.tiles_per_group;
    p.tiles_per_board = g.tiles_per_board;
    p.group_pos = (int)g.group_pos;
    p.ctas_per_group = std::max(1, std::min(e->sms / e->G, g.tiles_per_group));
    if (lp.pair) p.ctas_per_group = std::max(2, p.ctas_per_group & ~1);   // whole pairs (tile counts are even)
    p.w_pair = e->wconv_pair[l];
    p.resident = lp.resident;
    p.nstages = lp.nstages;
    p.nissue = lp.nissue;
    p.spi = lp.spi;
    p.qps = lp.qps;
    p.use_const = e->G == 1 ? 1 : 0;
    if (p.use_const) {
      std::memcpy(p.c_hbias, e->h_bias[l].data(), sizeof(p.c_hbias));
      if (p.head) {
        std::memcpy(p.c_wp, e->h_wp.data(), sizeof(p.c_wp));
        std::memcpy(p.c_wv, e->h_wv.data(), sizeof(p.c_wv));
      }
    }
    p.acc_stride = lp.acc_stride;
    p.nacc = lp.nacc;
    p.tmem_cols = lp.tmem_cols;
    {
      ProfScope _ps(e, C6_KIND_CONV0 + l, st);
      const int grid = e->G * p.ctas_per_group;
      const bool dep = e->dependent_launch;
      launch_chain(conv_kernel_for(p.wait_cycles != nullptr, lp.pair != 0, e->f16 != 0, lp.k), (unsigned)grid, 1u,
                   kConvThreads, (size_t)lp.smem, st, lp.pair != 0, dep, p);
    }
    C6_LAUNCHED(e, "conv_tc_kernel");
    return C6_OK;
  };
  const int last = a.stop_layer >= 0 ? a.stop_layer : e->L - 1;
  if (!direct_stem) {
    int rc = launch_stem();
    if (rc) return rc;
  }
  int first_plain = 1;
  if (e->fuse12 && last >= 2 && g.tiles_per_board > 0) {
    // layers 1 and 2 in one kernel: act[0] -> act[1], the 32-channel intermediate stays in shared memory
    Conv2FusedParams p{};
    p.in = e->act[0];
    p.out = e->act[1];
    p.w1_pair = e->wconv_pair[1];
    p.w2_pair = e->wconv_pair[2];
    p.status = e->status_dev;
    p.plane_rows = e->plane_rows;
    p.front = e->front;
    p.halo_rows = e->halo_rows;
    p.cin = e->lp[1].cin_p;
    p.c1 = e->lp[1].cout_p;
    p.c2 = e->lp[2].cout_p;
    p.wp = e->wp;
    p.slots = e->slots;
    p.bsize = e->n;
    p.nboards = nb;
    p.tiles_per_board = g.tiles_per_board;
    p.board_pairs = (nb + 1) / 2;
    std::memcpy(p.c_hb1, e->h_bias[1].data(), sizeof(p.c_hb1));
    std::memcpy(p.c_hb2, e->h_bias[2].data(), sizeof(p.c_hb2));
    {
      ProfScope _ps(e, C6_KIND_CONV0 + 1, st);
      const int grid = 2 * std::max(1, std::min(e->sms / 2, p.board_pairs));
      launch_chain(e->f16 ? conv2_fused_kernel<true> : conv2_fused_kernel<false>, (unsigned)grid, 1u, kFusedThreads,
                   (size_t)e->fuse12_smem, st, true, e->dependent_launch, p);
    }
    C6_LAUNCHED(e, "conv2_fused_kernel");
    cur = 1;
    first_plain = 3;
  }
  for (int l = first_plain; l <= last; ++l) {
    int rc = launch_layer(l);
    if (rc) return rc;
    if (!(l == e->L - 1 && a.stop_layer < 0)) cur ^= 1;
  }
  if (a.stop_layer >= 0) {
    const LayerPlan& lp = e->lp[a.stop_layer];
    const long long total = (long long)nb * lp.cout * e->cells;
    unpack_activation_kernel<<<dim3((unsigned)((total + 255) / 256), (unsigned)e->G), 256, 0, st>>>(
        e->act[cur], e->plane_rows, e->front, (int)g.group_pos, e->slots, e->wp, e->n, lp.cout, nb,
        a.layer_out, e->f16);
    C6_LAUNCHED(e, "unpack_activation_kernel");
    return C6_OK;
  }
  return launch_finish(e, a, t0, nb, g.group_pos, e->slots, e->wp, direct_stem ? nullptr : e->occ, g.mrows_per_group, st);
}

int run_pass_fp32(C6Engine* e, const RunArgs& a, long long t0, int nb, cudaStream_t st) {
  const long long boards = (long long)e->G * nb;
  {
    const long long total = (long long)nb * 3 * e->cells;
    ProfScope _ps(e, C6_KIND_PACK, st);
    view_input_f32_kernel<<<dim3((unsigned)((total + 255) / 256), (unsigned)e->G), 256, 0, st>>>(
        input_of(a), a.orient, e->f32x, e->n, nb, a.T, t0);
    C6_LAUNCHED(e, "view_input_f32_kernel");
  }
  const float* in = e->f32x;
  int cur = 0;
  const int last = a.stop_layer >= 0 ? a.stop_layer : e->L - 1;
  for (int l = 0; l <= last; ++l) {
    const LayerPlan& lp = e->lp[l];
    const dim3 grid((unsigned)boards, (unsigned)((lp.cout + kFp32CoT - 1) / kFp32CoT));
    {
      ProfScope _ps(e, l == 0 ? C6_KIND_STEM : C6_KIND_CONV0 + l, st);
      conv_fp32_kernel<<<grid, kFp32Threads, fp32_smem(e, lp), st>>>(in, e->wraw[l], e->bias[l], e->f32buf[cur],
                                                                      lp.cin, lp.cout, lp.k, e->n, nb, fp32_cit(lp));
    }
    C6_LAUNCHED(e, "conv_fp32_kernel");
    in = e->f32buf[cur];
    cur ^= 1;
  }
  if (a.stop_layer >= 0) {
    const LayerPlan& lp = e->lp[a.stop_layer];
    C6_CUDA(e, cudaMemcpyAsync(a.layer_out, in, (size_t)boards * lp.cout * e->cells * sizeof(float),
                               cudaMemcpyDeviceToDevice, st));
    return C6_OK;
  }
  {
    ProfScope _ps(e, C6_KIND_OTHER, st);
    head_fp32_kernel<<<(unsigned)boards, kFp32Threads, 0, st>>>(in, e->head_wp, e->head_wv, e->logit_raw, e->vmap,
                                                                 e->lp[e->L - 1].cout, e->n, nb);
  }
  C6_LAUNCHED(e, "head_fp32_kernel");
  return launch_finish(e, a, t0, nb, (long long)nb * e->cells, e->cells, e->n, nullptr, 0, st);
}

int run(C6Engine* e, const RunArgs& a, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (a.T < 0) return fail(e, C6_ERR_ARG, "negative board count");
  if (a.T == 0) return C6_OK;
  if (!a.x && !a.boards) return fail(e, C6_ERR_ARG, "x is null");
  for (size_t i = 0; i < e->have.size(); ++i)
    if (!e->have[i]) return fail(e, C6_ERR_WEIGHTS, "forward before every layer and head of every group received weights");
  C6_CUDA(e, cudaSetDevice(e->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long per_pass = std::max<long long>(1, e->chunk / e->G);
  // The stem path is chosen once per call, from the call's boards per weight set, so that every pass of a
  // call sums in the same order: the direct stem for small calls, the stem GEMM otherwise.
  const bool direct = e->prec != C6_PREC_FP32 && e->sd_ok && a.T <= e->sd_max_boards && a.T <= per_pass;
  int rc = ensure_workspace(e, std::min(a.T, per_pass), direct);
  if (rc) return rc;
  for (long long t0 = 0; t0 < a.T; t0 += per_pass) {
    const int nb = (int)std::min<long long>(per_pass, a.T - t0);
    RunArgs b = a;
    b.direct_stem = direct ? 1 : 0;
    // outputs are indexed [g*T + t] by the kernels themselves (board0 = t0)
    rc = e->prec != C6_PREC_FP32 ? run_pass_bf16(e, b, t0, nb, st) : run_pass_fp32(e, b, t0, nb, st);
    if (rc) return rc;
  }
  return C6_OK;
}

}  // namespace

// =================================================================================================
// C ABI
// =================================================================================================
extern "C" {

int c6_version(void) { return kVersion; }

const char* c6_last_error(const C6Engine* eng) { return eng ? eng->err.c_str() : g_create_error.c_str(); }

int c6_destroy(C6Engine* e) {
  if (!e) return C6_OK;
  cudaSetDevice(e->device);
  cudaDeviceSynchronize();
  free_workspace(e);
  cudaFree(e->wt);
  cudaFree(e->w0_raw);
  cudaFree(e->w_sd);
  cudaFree(e->w_sd_pair);
  cudaFree(e->p2_epoch);
  for (auto p : e->wconv) cudaFree(p);
  for (auto p : e->wconv_pair) cudaFree(p);
  for (auto p : e->bias) cudaFree(p);
  for (auto p : e->wraw) cudaFree(p);
  cudaFree(e->head_wp);
  cudaFree(e->head_wv);
  cudaFree(e->pol_bias);
  cudaFree(e->val_bias);
  cudaFree(e->status_dev);
  cudaFree(e->wait_dev);
  for (auto& r : e->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (auto ev : e->ev_pool) cudaEventDestroy(ev);
  delete e;
  return C6_OK;
}

int c6_create(const C6Desc* d, C6Engine** out) {
  if (!d || !out) return fail(nullptr, C6_ERR_ARG, "null argument");
  *out = nullptr;
  if (d->n_layers < 1 || d->n_layers > C6_MAX_LAYERS) return fail(nullptr, C6_ERR_ARG, "n_layers out of range");
  if (d->board_size < 1 || d->board_size > 32) return fail(nullptr, C6_ERR_ARG, "board_size must be in 1..32");
  if (d->groups < 1) return fail(nullptr, C6_ERR_ARG, "groups must be >= 1");
  if (d->precision != C6_PREC_BF16 && d->precision != C6_PREC_FP32 && d->precision != C6_PREC_F16)
    return fail(nullptr, C6_ERR_ARG, "unknown precision");
  for (int i = 0; i < d->n_layers; ++i) {
    if (d->kernels[i] <= 0 || d->kernels[i] % 2 == 0) return fail(nullptr, C6_ERR_ARG, "every kernel must be a positive odd number");
    if (d->channels[i] <= 0) return fail(nullptr, C6_ERR_ARG, "channel counts must be positive");
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || d->device < 0 || d->device >= ndev)
    return fail(nullptr, C6_ERR_CUDA, "no such CUDA device (this engine has no CPU path)");

  C6Engine* e = new (std::nothrow) C6Engine();
  if (!e) return fail(nullptr, C6_ERR_ARG, "out of host memory");
  e->d = *d;
  e->device = d->device;
  e->n = d->board_size;
  e->cells = e->n * e->n;
  e->L = d->n_layers;
  e->G = d->groups;
  e->prec = d->precision;
  e->f16 = d->precision == C6_PREC_F16 ? 1 : 0;
  auto bail = [&](int code, const std::string& msg) {
    g_create_error = msg.empty() ? e->err : msg;
    c6_destroy(e);
    return code;
  };
  if (cudaSetDevice(e->device) != cudaSuccess) return bail(C6_ERR_CUDA, "cudaSetDevice failed");
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, e->device) != cudaSuccess) return bail(C6_ERR_CUDA, "cudaGetDeviceProperties failed");
  e->sms = prop.multiProcessorCount;
  if (e->prec != C6_PREC_FP32 && prop.major != 10)
    return bail(C6_ERR_UNSUPPORTED, "the bf16 and fp16 modes need an sm_100 GPU (tcgen05 tensor cores)");

  e->lp.resize(e->L);
  int cin = 3;
  for (int l = 0; l < e->L; ++l) {
    LayerPlan& p = e->lp[l];
    p.k = d->kernels[l];
    p.cin = cin;
    p.cout = d->channels[l];
    p.cin_p = l == 0 ? 3 : round_up(cin, 32);
    p.cout_p = round_up(p.cout, 32);
    cin = p.cout;
    e->cmax = std::max(e->cmax, p.cout);
    e->cmax_p = std::max(e->cmax_p, p.cout_p);
    if (l >= 1) e->pad = std::max(e->pad, p.k / 2);
  }
  e->wp = e->n + e->pad;
  e->slots = e->wp * e->wp;
  e->halo = e->pad * e->wp + e->pad;
  e->halo_rows = round_up(e->halo, 8);
  e->front = e->halo_rows;
  e->chunk = d->max_chunk > 0 ? d->max_chunk : (e->prec != C6_PREC_FP32 ? 8192 : 1024);
  e->have.assign((size_t)e->G * (e->L + 2), 0);
  e->h_bias.assign(e->L, std::vector<float>());

  int rc;
  if ((rc = dev_alloc(e, &e->status_dev, 1, true, nullptr))) return bail(rc, "");
  if ((rc = dev_alloc(e, &e->wait_dev, 8 + 2048, true, nullptr))) return bail(rc, "");
  if ((rc = dev_alloc(e, &e->pol_bias, e->G, true, nullptr))) return bail(rc, "");
  if ((rc = dev_alloc(e, &e->val_bias, e->G, true, nullptr))) return bail(rc, "");
  e->wconv.assign(e->L, nullptr);
  e->wconv_pair.assign(e->L, nullptr);
  e->bias.assign(e->L, nullptr);
  e->wraw.assign(e->L, nullptr);

  if (e->prec != C6_PREC_FP32) {
    if (e->L < 2) return bail(C6_ERR_UNSUPPORTED, "the tensor-core modes need at least two backbone layers");
    if (e->cmax_p > 256) return bail(C6_ERR_UNSUPPORTED, "the tensor-core modes support at most 256 channels per layer");
    // stem GEMM
    const int c1 = e->lp[0].cout_p;
    const int cpt = std::max(1, 256 / c1);
    e->nt = c1 * cpt;
    e->ntiles = (e->cells + cpt - 1) / cpt;
    e->ntot = e->ntiles * e->nt;
    // CTA pairs (each stages half of the Toeplitz rows, 64 K per stage) when at least one pair exists
    e->stem_pair = e->sms >= 2 ? 1 : 0;
    e->stem_kcs = e->stem_pair ? 8 : 4;
    // K = [planes 0 and 1 | plane 2], each part padded to whole pipeline stages
    e->kc_short = round_up(2 * e->cells + 2, 8 * e->stem_kcs) / 8;   // + the two level slots of the third plane
    e->kc0 = e->kc_short + round_up(e->cells, 8 * e->stem_kcs) / 8;
    const int sstage = e->stem_kcs * 128 * 16 + e->stem_kcs * (e->stem_pair ? e->nt / 2 : e->nt) * 16;
    e->stem_stages = std::min(kStemMaxStages, (kSmemLimit - 128 - kStemSmemHeader - kStemPatchBytes) / sstage);
    if (e->stem_stages < 2) return bail(C6_ERR_UNSUPPORTED, "the stem's pipeline stages do not fit shared memory");
    e->stem_smem = 128 + kStemSmemHeader + e->stem_stages * sstage + kStemPatchBytes;
    e->stem_acc_stride = pow2_ceil(e->nt);
    e->stem_tmem_cols = 2 * e->stem_acc_stride;
    e->wt_fresh.assign(e->G, 0);
    if ((rc = dev_alloc(e, &e->w0_raw, (size_t)e->G * e->lp[0].cout * 3 * e->lp[0].k * e->lp[0].k, true, nullptr))) return bail(rc, "");
    if ((rc = dev_alloc(e, &e->p2_epoch, 1, true, nullptr))) return bail(rc, "");
    if ((rc = dev_alloc(e, &e->bias[0], (size_t)e->G * c1, true, nullptr))) return bail(rc, "");
    // k x k layers
    e->pair_mode = e->sms / e->G >= 2;   // at least one CTA pair per group
    if (const char* v = std::getenv("C6_DEPENDENT_LAUNCH")) e->dependent_launch = std::strcmp(v, "0") != 0;
    const int rows = conv_stage_rows(e->halo_rows);
    for (int l = 1; l < e->L; ++l) {
      LayerPlan& p = e->lp[l];
      if (!plan_tc_layer(e->pair_mode, p, p.k * p.k, p.cin_p / 16, rows, 2, 2))
        return bail(C6_ERR_UNSUPPORTED, "a conv layer does not fit shared memory");
      if ((rc = dev_alloc(e, &e->wconv[l], (size_t)e->G * p.w_rows_per_group, true, nullptr))) return bail(rc, "");
      if (p.pair && (rc = dev_alloc(e, &e->wconv_pair[l], (size_t)e->G * p.w_rows_per_group, true, nullptr))) return bail(rc, "");
      if ((rc = dev_alloc(e, &e->bias[l], (size_t)e->G * p.cout_p, true, nullptr))) return bail(rc, "");
    }
    {
      // Layers 1 and 2 fused (narrow networks: 32 -> 32 -> at most 64 channels, 3 x 3 both, one weight set, CTA pairs,
      // board images of at most three tiles); C6_FUSE_PAIRS=0 turns it off.
      const int used = (e->n - 1) * e->wp + e->n, tpb = (used + 127) / 128;
      const bool shape_ok = e->L >= 4 && e->G == 1 && e->pair_mode && e->lp[1].k == 3 && e->lp[2].k == 3 && e->lp[1].cin_p == 32 &&
                            e->lp[1].cout_p == 32 && e->lp[2].cout_p <= 64 && tpb * 128 < e->slots && tpb <= kFusedMaxTiles &&
                            e->lp[1].pair && e->lp[2].pair;
      e->fuse12_smem = shape_ok ? fused_smem_bytes(32, 32, e->lp[2].cout_p, tpb, e->halo_rows) : 0;
      e->fuse12 = shape_ok && e->fuse12_smem <= kSmemLimit ? 1 : 0;
      if (const char* v = std::getenv("C6_FUSE_PAIRS")) e->fuse12 = e->fuse12 && std::strcmp(v, "0") != 0;
      if (e->fuse12 && (cudaFuncSetAttribute(conv2_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess ||
                        cudaFuncSetAttribute(conv2_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess))
        return bail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
    }
    {
      // Direct stem for passes with few boards per weight set.  Input images: pitch wi >= n + k0/2 so that the
      // pad columns serve both neighbours, n + k0/2 rows; taps are (filter row, 16-wide kx block).
      const int k0 = e->lp[0].k, kh = k0 / 2;
      e->sd_hx = (k0 + 15) / 16;
      e->sd_wi = round_up(e->n + kh, 8);
      e->sd_slots = e->sd_wi * (e->n + kh);
      e->sd_halo_b = round_up(kh * e->sd_wi + kh, 8);
      e->sd_halo_a = round_up(kh * e->sd_wi + 16 * e->sd_hx - 1 - kh + 8, 8);
      e->sd_front = e->sd_halo_b;
      e->sdp = e->lp[0];
      // Taken by engines with at least sd_min_groups weight sets for calls of at most sd_max_boards boards per
      // set: that is where the stem GEMM's 27 MB of expanded weights per model cost more than they save.  For a
      // single model the two paths tie up to about 16 boards and the GEMM wins beyond (measured), so it keeps
      // the GEMM.  C6_STEM_DIRECT_MAX / C6_STEM_DIRECT_GROUPS override the two thresholds.
      if (const char* v = std::getenv("C6_STEM_DIRECT_MAX")) e->sd_max_boards = std::max(0, std::atoi(v));
      if (const char* v = std::getenv("C6_STEM_DIRECT_GROUPS")) e->sd_min_groups = std::max(1, std::atoi(v));
      e->sd_ok = e->sd_max_boards > 0 && e->G >= e->sd_min_groups &&
                 plan_tc_layer(e->pair_mode, e->sdp, k0 * e->sd_hx, 3, 128 + e->sd_halo_b + e->sd_halo_a, 1, 1) ? 1 : 0;
      if (e->sd_ok) {
        if ((rc = dev_alloc(e, &e->w_sd, (size_t)e->G * e->sdp.w_rows_per_group, true, nullptr))) return bail(rc, "");
        if (e->sdp.pair && (rc = dev_alloc(e, &e->w_sd_pair, (size_t)e->G * e->sdp.w_rows_per_group, true, nullptr))) return bail(rc, "");
      }
    }
    const int cl = e->lp[e->L - 1].cout_p;
    if ((rc = dev_alloc(e, &e->head_wp, (size_t)e->G * cl, true, nullptr))) return bail(rc, "");
    if ((rc = dev_alloc(e, &e->head_wv, (size_t)e->G * cl, true, nullptr))) return bail(rc, "");
    if (!conv_smem_opt_in<0>() || !conv_smem_opt_in<1>() || !conv_smem_opt_in<3>() || !conv_smem_opt_in<5>() ||
        cudaFuncSetAttribute(stem_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess ||
        cudaFuncSetAttribute(stem_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess ||
        cudaFuncSetAttribute(stem_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess ||
        cudaFuncSetAttribute(stem_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
      return bail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  } else {
    size_t max_smem = 0;
    for (int l = 0; l < e->L; ++l) {
      const LayerPlan& p = e->lp[l];
      if ((rc = dev_alloc(e, &e->wraw[l], (size_t)e->G * p.cout * p.cin * p.k * p.k, true, nullptr))) return bail(rc, "");
      if ((rc = dev_alloc(e, &e->bias[l], (size_t)e->G * p.cout, true, nullptr))) return bail(rc, "");
      max_smem = std::max(max_smem, fp32_smem(e, p));
    }
    if (max_smem > (size_t)kSmemLimit) return bail(C6_ERR_UNSUPPORTED, "fp32 mode: layer does not fit shared memory");
    const int cl = e->lp[e->L - 1].cout;
    if ((rc = dev_alloc(e, &e->head_wp, (size_t)e->G * cl, true, nullptr))) return bail(rc, "");
    if ((rc = dev_alloc(e, &e->head_wv, (size_t)e->G * cl, true, nullptr))) return bail(rc, "");
    // The attribute belongs to the function on this device, not to this engine: always the full limit, so
    // that a second engine with smaller layers never lowers it under the first one's needs.
    if (cudaFuncSetAttribute(conv_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
      return bail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  }
  *out = e;
  return C6_OK;
}

int c6_set_weights(C6Engine* e, int group, int layer, const float* w, const float* bias, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (group < 0 || group >= e->G) return fail(e, C6_ERR_ARG, "group out of range");
  if (!w) return fail(e, C6_ERR_ARG, "weight pointer is null");
  C6_CUDA(e, cudaSetDevice(e->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf16 = e->prec != C6_PREC_FP32;   // tensor-core mode (bf16 or fp16 operands)
  if (layer == C6_HEAD_POLICY || layer == C6_HEAD_VALUE) {
    const LayerPlan& last = e->lp[e->L - 1];
    const int cl = bf16 ? last.cout_p : last.cout;
    float* dst = (layer == C6_HEAD_POLICY ? e->head_wp : e->head_wv) + (size_t)group * cl;
    float* bdst = (layer == C6_HEAD_POLICY ? e->pol_bias : e->val_bias) + group;
    copy_pad_f32_kernel<<<(cl + 127) / 128, 128, 0, st>>>(w, dst, last.cout, cl);
    C6_LAUNCHED(e, "copy_pad_f32_kernel");
    copy_pad_f32_kernel<<<1, 32, 0, st>>>(bias, bdst, 1, 1);
    C6_LAUNCHED(e, "copy_pad_f32_kernel");
    if (bf16 && e->G == 1) {
      // single-model engines keep a host copy: the conv kernel takes these vectors by value
      std::vector<float>& h = layer == C6_HEAD_POLICY ? e->h_wp : e->h_wv;
      h.assign(256, 0.f);
      C6_CUDA(e, cudaMemcpyAsync(h.data(), dst, (size_t)cl * sizeof(float), cudaMemcpyDeviceToHost, st));
      C6_CUDA(e, cudaStreamSynchronize(st));
    }
    e->have[(size_t)group * (e->L + 2) + e->L + (layer == C6_HEAD_POLICY ? 0 : 1)] = 1;
    return C6_OK;
  }
  if (layer < 0 || layer >= e->L) return fail(e, C6_ERR_ARG, "layer out of range");
  const LayerPlan& p = e->lp[layer];
  if (bf16) {
    if (layer == 0) {
      const size_t wn = (size_t)p.cout * 3 * p.k * p.k;
      C6_CUDA(e, cudaMemcpyAsync(e->w0_raw + (size_t)group * wn, w, wn * sizeof(float), cudaMemcpyDeviceToDevice, st));
      e->wt_fresh[group] = 0;
      if (e->wt) {
        int rc = expand_toeplitz(e, group, st);
        if (rc) return rc;
      }
      if (e->sd_ok) {
        const long long rows = (long long)e->sdp.w_rows_per_group;
        pack_stem_direct_weights_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
            w, e->w_sd + (size_t)group * rows, p.cout, p.k, p.cout_p, e->sd_hx, 1, e->f16);
        C6_LAUNCHED(e, "pack_stem_direct_weights_kernel");
        if (e->sdp.pair) {
          pack_stem_direct_weights_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
              w, e->w_sd_pair + (size_t)group * rows, p.cout, p.k, p.cout_p, e->sd_hx, 2, e->f16);
          C6_LAUNCHED(e, "pack_stem_direct_weights_kernel");
        }
      }
    } else {
      const long long total = (long long)p.w_rows_per_group;
      pack_conv_weights_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
          w, e->wconv[layer] + (size_t)group * p.w_rows_per_group, p.cout, p.cin, p.k, p.cout_p, p.cin_p, e->f16);
      C6_LAUNCHED(e, "pack_conv_weights_kernel");
      if (p.pair) {
        pack_conv_weights_pair_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            w, e->wconv_pair[layer] + (size_t)group * p.w_rows_per_group, p.cout, p.cin, p.k, p.cout_p, p.cin_p, e->f16);
        C6_LAUNCHED(e, "pack_conv_weights_pair_kernel");
      }
    }
    copy_pad_f32_kernel<<<(p.cout_p + 127) / 128, 128, 0, st>>>(bias, e->bias[layer] + (size_t)group * p.cout_p,
                                                                 p.cout, p.cout_p);
    C6_LAUNCHED(e, "copy_pad_f32_kernel");
    if (e->G == 1) {
      e->h_bias[layer].assign(256, 0.f);
      C6_CUDA(e, cudaMemcpyAsync(e->h_bias[layer].data(), e->bias[layer], (size_t)p.cout_p * sizeof(float),
                                 cudaMemcpyDeviceToHost, st));
      C6_CUDA(e, cudaStreamSynchronize(st));
      for (auto& v : e->h_bias[layer]) v *= 0.5f;   // the epilogue works on h = x/2
    }
  } else {
    const size_t wn = (size_t)p.cout * p.cin * p.k * p.k;
    C6_CUDA(e, cudaMemcpyAsync(e->wraw[layer] + (size_t)group * wn, w, wn * sizeof(float), cudaMemcpyDeviceToDevice, st));
    copy_pad_f32_kernel<<<(p.cout + 127) / 128, 128, 0, st>>>(bias, e->bias[layer] + (size_t)group * p.cout, p.cout, p.cout);
    C6_LAUNCHED(e, "copy_pad_f32_kernel");
  }
  e->have[(size_t)group * (e->L + 2) + layer] = 1;
  return C6_OK;
}

int c6_reserve(C6Engine* e, int64_t boards) {
  if (!e) return C6_ERR_ARG;
  if (boards <= 0) return fail(e, C6_ERR_ARG, "boards must be positive");
  C6_CUDA(e, cudaSetDevice(e->device));
  const long long per_pass = std::max<long long>(1, e->chunk / e->G);
  const long long nb = std::min<long long>(boards, per_pass);
  const bool direct = e->prec != C6_PREC_FP32 && e->sd_ok && boards <= e->sd_max_boards && boards <= per_pass;
  if (e->prec != C6_PREC_FP32 && !e->wt && !direct) {
    // calls of this size go through the stem GEMM: allocate its operand now (expanded by the first pass)
    C6_CUDA(e, cudaDeviceSynchronize());
    int rc = dev_alloc(e, &e->wt, (size_t)e->G * e->kc0 * e->ntot, true, nullptr);
    if (rc) return rc;
  }
  return ensure_workspace(e, nb, direct);
}

int c6_forward(C6Engine* e, const void* x, int x_dtype, int64_t B, const uint8_t* orient, float* logits,
               float* value, int flags, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (e->G != 1) return fail(e, C6_ERR_ARG, "c6_forward needs an engine with groups == 1");
  if (x_dtype != C6_X_F32 && x_dtype != C6_X_BF16) return fail(e, C6_ERR_ARG, "unknown x dtype");
  RunArgs a;
  a.x = x;
  a.x_bf16 = x_dtype == C6_X_BF16;
  a.T = B;
  a.orient = orient;
  a.logits = logits;
  a.value = value;
  a.flags = flags;
  return run(e, a, stream);
}

int c6_forward_step(C6Engine* e, const void* x, int x_dtype, int64_t B, const uint8_t* orient, int flags,
                    float temperature, uint64_t seed, uint64_t offset, int64_t board_index0, int64_t* action,
                    float* logprob, float* value, float* masked_logits, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (e->G != 1) return fail(e, C6_ERR_ARG, "c6_forward_step needs an engine with groups == 1");
  if (x_dtype != C6_X_F32 && x_dtype != C6_X_BF16) return fail(e, C6_ERR_ARG, "unknown x dtype");
  if (B > 0 && !action) return fail(e, C6_ERR_ARG, "action pointer is null");
  RunArgs a;
  a.x = x;
  a.x_bf16 = x_dtype == C6_X_BF16;
  a.T = B;
  a.orient = orient;
  a.logits = masked_logits;
  a.value = value;
  a.flags = flags | C6_FLAG_MASK_LOGITS;
  a.do_sample = 1;
  a.temperature = temperature;
  a.seed = seed;
  a.offset = offset;
  a.board_index0 = board_index0;
  a.action = reinterpret_cast<long long*>(action);
  a.logprob = logprob;
  return run(e, a, stream);
}

int c6_forward_step_boards(C6Engine* e, const int8_t* boards, const int8_t* current_player, const int8_t* stones_left,
                           int64_t num_envs, const int64_t* index, int64_t B, const uint8_t* orient, int flags, float temperature,
                           uint64_t seed, uint64_t offset, int64_t board_index0, int64_t* action, float* logprob,
                           float* value, float* masked_logits, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (e->G != 1) return fail(e, C6_ERR_ARG, "c6_forward_step_boards needs an engine with groups == 1");
  if (B > 0 && (!boards || !current_player || !stones_left)) return fail(e, C6_ERR_ARG, "board state pointer is null");
  if (B > 0 && !action) return fail(e, C6_ERR_ARG, "action pointer is null");
  if (num_envs < 0 || (!index && B > num_envs)) return fail(e, C6_ERR_ARG, "more boards than environments and no index vector");
  RunArgs a;
  a.num_envs = num_envs;
  a.boards = boards;
  a.player = current_player;
  a.stones_left = stones_left;
  a.index = reinterpret_cast<const long long*>(index);
  a.T = B;
  a.orient = orient;
  a.logits = masked_logits;
  a.value = value;
  a.flags = flags | C6_FLAG_MASK_LOGITS;
  a.do_sample = 1;
  a.temperature = temperature;
  a.seed = seed;
  a.offset = offset;
  a.board_index0 = board_index0;
  a.action = reinterpret_cast<long long*>(action);
  a.logprob = logprob;
  return run(e, a, stream);
}

int c6_forward_grouped(C6Engine* e, const void* x, int x_dtype, int64_t T, float* logits, float* value, int flags,
                       void* stream) {
  if (!e) return C6_ERR_ARG;
  if (x_dtype != C6_X_F32 && x_dtype != C6_X_BF16) return fail(e, C6_ERR_ARG, "unknown x dtype");
  RunArgs a;
  a.x = x;
  a.x_bf16 = x_dtype == C6_X_BF16;
  a.T = T;
  a.logits = logits;
  a.value = value;
  a.flags = flags;
  return run(e, a, stream);
}

int c6_forward_noalloc(C6Engine* e, const void* x, int x_dtype, int64_t B, const uint8_t* orient, float* logits,
                       float* value, int flags, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (e->prec != C6_PREC_FP32 || e->G != 1)
    return fail(e, C6_ERR_UNSUPPORTED, "c6_forward_noalloc needs an fp32-mode engine with groups == 1");
  if (x_dtype != C6_X_F32 && x_dtype != C6_X_BF16) return fail(e, C6_ERR_ARG, "unknown x dtype");
  if (B < 0) return fail(e, C6_ERR_ARG, "negative board count");
  if (B == 0) return C6_OK;
  if (!x) return fail(e, C6_ERR_ARG, "x is null");
  if (e->device < 0 || e->device >= kNoAllocMaxDevices) return fail(e, C6_ERR_UNSUPPORTED, "device ordinal too large");
  for (size_t i = 0; i < e->have.size(); ++i)
    if (!e->have[i]) return fail(e, C6_ERR_WEIGHTS, "forward before every layer and head received weights");
  // floats needed: view of x, two ping-pong activations, the two raw head maps
  const size_t per_board = (size_t)e->cells * (3 + 2 * (size_t)e->cmax + 2);
  const size_t need = per_board * (size_t)B;
  if (need > kNoAllocScratchFloats) {
    char buf[200];
    snprintf(buf, sizeof(buf), "c6_forward_noalloc: %lld boards need %zu bytes of scratch, the fixed scratch holds %zu "
             "(at most %zu boards of this architecture)", (long long)B, need * sizeof(float), kNoAllocScratchBytes,
             kNoAllocScratchFloats / per_board);
    return fail(e, C6_ERR_ARG, buf);
  }
  C6_CUDA(e, cudaSetDevice(e->device));
  if (!g_noalloc_scratch_ptr[e->device]) {
    // once per device, with that device current: resolve the device address of the static array
    float* ptr = nullptr;
    C6_CUDA(e, cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch));
    g_noalloc_scratch_ptr[e->device] = ptr;
  }
  float* base = g_noalloc_scratch_ptr[e->device];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nb = (int)B;
  float* xview = base;
  float* buf[2] = {xview + (size_t)nb * 3 * e->cells, xview + (size_t)nb * (3 + e->cmax) * e->cells};
  float* raw_pol = buf[1] + (size_t)nb * e->cmax * e->cells;
  float* raw_val = raw_pol + (size_t)nb * e->cells;
  // every buffer below is fully written before it is read, so nothing has to be cleared
  {
    const long long total = (long long)nb * 3 * e->cells;
    InputSrc in{};
    in.x = x;
    in.x_bf16 = x_dtype == C6_X_BF16;
    view_input_f32_kernel<<<dim3((unsigned)((total + 255) / 256), 1), 256, 0, st>>>(in, orient, xview, e->n, nb, B, 0);
    C6_LAUNCHED(e, "view_input_f32_kernel");
  }
  const float* in = xview;
  int cur = 0;
  for (int l = 0; l < e->L; ++l) {
    const LayerPlan& lp = e->lp[l];
    const dim3 grid((unsigned)nb, (unsigned)((lp.cout + kFp32CoT - 1) / kFp32CoT));
    conv_fp32_kernel<<<grid, kFp32Threads, fp32_smem(e, lp), st>>>(in, e->wraw[l], e->bias[l], buf[cur], lp.cin, lp.cout,
                                                                    lp.k, e->n, nb, fp32_cit(lp));
    C6_LAUNCHED(e, "conv_fp32_kernel");
    in = buf[cur];
    cur ^= 1;
  }
  head_fp32_kernel<<<(unsigned)nb, kFp32Threads, 0, st>>>(in, e->head_wp, e->head_wv, raw_pol, raw_val,
                                                           e->lp[e->L - 1].cout, e->n, nb);
  C6_LAUNCHED(e, "head_fp32_kernel");
  FinishParams f{};
  f.logit_raw = raw_pol;
  f.vmap = value ? raw_val : nullptr;
  f.group_stride = (long long)nb * e->cells;
  f.board_stride = e->cells;
  f.pitch = e->n;
  f.pol_bias = e->pol_bias;
  f.val_bias = e->val_bias;
  f.in.x = x;
  f.in.x_bf16 = x_dtype == C6_X_BF16;
  f.orient = orient;
  f.x_group_stride = B;
  f.board0 = 0;
  f.n = e->n;
  f.n_magic = 65536 / e->n + 1;
  f.n_actions = e->cells;
  f.nb = nb;
  f.flags = flags;
  f.logits_out = logits;
  f.value_out = value;
  finish_kernel_for(f.n_actions)<<<dim3(finish_blocks(nb), 1), kFinishThreads, 0, st>>>(f);
  C6_LAUNCHED(e, "finish_kernel");
  return C6_OK;
}

int c6_debug_layer_output(C6Engine* e, const void* x, int x_dtype, int64_t T, const uint8_t* orient, int layer,
                          float* out_nchw, void* stream) {
  if (!e) return C6_ERR_ARG;
  if (layer < 0 || layer >= e->L) return fail(e, C6_ERR_ARG, "layer out of range");
  if (!out_nchw) return fail(e, C6_ERR_ARG, "output pointer is null");
  if (T > std::max<long long>(1, e->chunk / e->G)) return fail(e, C6_ERR_ARG, "debug output is limited to one pass");
  RunArgs a;
  a.x = x;
  a.x_bf16 = x_dtype == C6_X_BF16;
  a.T = T;
  a.orient = orient;
  a.stop_layer = layer;
  a.layer_out = out_nchw;
  return run(e, a, stream);
}

int c6_sample_actions(const float* logits, const uint8_t* legal, int64_t B, int32_t A, float temperature,
                      uint64_t seed, uint64_t offset, int64_t board_index0, int64_t* action, float* logprob,
                      void* stream) {
  if (B < 0 || A <= 0 || A > kFinishMaxActions) return C6_ERR_ARG;
  if (B == 0) return C6_OK;
  if (!logits || !legal || !action) return C6_ERR_ARG;
  FinishParams f{};
  f.logits_in = logits;
  f.legal_in = legal;
  f.x_group_stride = B;
  f.n = 1;
  f.n_magic = 65537;
  f.n_actions = A;
  f.nb = (int)B;
  f.do_sample = 1;
  f.temperature = temperature;
  f.seed = seed;
  f.offset = offset;
  f.board_index0 = board_index0;
  f.action_out = reinterpret_cast<long long*>(action);
  f.logprob_out = logprob;
  finish_kernel_for(f.n_actions)<<<dim3(finish_blocks(B), 1), kFinishThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(f);
  return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA;
}

int c6_mask_logits(const float* logits, const uint8_t* legal, int64_t count, float fill, float* out, void* stream) {
  if (count < 0) return C6_ERR_ARG;
  if (count == 0) return C6_OK;
  if (!logits || !legal || !out) return C6_ERR_ARG;
  mask_logits_kernel<<<(unsigned)((count + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, legal, count, fill, out);
  return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA;
}

int c6_transform_actions(const int64_t* actions, int64_t B, int32_t n, const uint8_t* phase, int32_t phase_all,
                         int32_t inverse, int64_t* out, void* stream) {
  if (B < 0 || n <= 0) return C6_ERR_ARG;
  if (B == 0) return C6_OK;
  if (!actions || !out) return C6_ERR_ARG;
  transform_actions_kernel<<<(unsigned)((B + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(actions), B, n, phase, phase_all, inverse, reinterpret_cast<long long*>(out));
  return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA;
}

int c6_transform_boards(const int8_t* boards, int64_t B, int32_t n, const uint8_t* phase, int32_t phase_all,
                        int8_t* out, void* stream) {
  if (B < 0 || n <= 0) return C6_ERR_ARG;
  if (B == 0) return C6_OK;
  if (!boards || !out) return C6_ERR_ARG;
  const long long total = (long long)B * n * n;
  transform_boards_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      boards, B, n, phase, phase_all, out);
  return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA;
}

int c6_network_input(const int8_t* boards, const int8_t* current_player, const int8_t* stones_left, int64_t B,
                     int32_t n, float* out, void* stream) {
  if (B < 0 || n <= 0) return C6_ERR_ARG;
  if (B == 0) return C6_OK;
  if (!boards || !current_player || !stones_left || !out) return C6_ERR_ARG;
  const long long total = (long long)B * n * n;
  network_input_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      boards, current_player, stones_left, B, n, out);
  return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA;
}

int c6_status(C6Engine* e, int* device_status) {
  if (!e || !device_status) return C6_ERR_ARG;
  C6_CUDA(e, cudaSetDevice(e->device));
  C6_CUDA(e, cudaMemcpy(device_status, e->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  if (*device_status != 0) {
    char buf[200];
    const int st = *device_status;
    snprintf(buf, sizeof(buf), "device status word 0x%x:%s%s%s", st,
             (st & 63) ? " a bounded wait inside a kernel ran out;" : "",
             (st & kStatBadIndex) ? " a gather index lay outside the environments (read as an empty board);" : "",
             (st & kStatF16Range) ? " fp16 mode: an activation exceeded +-65504 and was clamped;" : "");
    return fail(e, C6_ERR_DEVICE, buf);
  }
  return C6_OK;
}

int c6_profile_enable(C6Engine* e, int on) {
  if (!e) return C6_ERR_ARG;
  e->profiling = on != 0;
  e->wait_counters = on >= 2 && kTimedBuild;
  return C6_OK;
}

int c6_profile_read(C6Engine* e, float* ms_per_kind, int64_t* launches_per_kind, int n_kinds) {
  if (!e || !ms_per_kind || !launches_per_kind || n_kinds < C6_KIND_COUNT) return C6_ERR_ARG;
  C6_CUDA(e, cudaSetDevice(e->device));
  for (int i = 0; i < n_kinds; ++i) { ms_per_kind[i] = 0.f; launches_per_kind[i] = 0; }
  for (auto& r : e->prof) {
    C6_CUDA(e, cudaEventSynchronize(r.b));
    float ms = 0.f;
    C6_CUDA(e, cudaEventElapsedTime(&ms, r.a, r.b));
    ms_per_kind[r.kind] += ms;
    launches_per_kind[r.kind] += 1;
    e->ev_pool.push_back(r.a);
    e->ev_pool.push_back(r.b);
  }
  e->prof.clear();
  return C6_OK;
}

int c6_debug_wait_cycles(C6Engine* e, int64_t* out8, int reset) {
  if (!e || !out8) return C6_ERR_ARG;
#ifdef C6_TIMED_BUILD
  C6_CUDA(e, cudaSetDevice(e->device));
  C6_CUDA(e, cudaMemcpy(out8, e->wait_dev, 8 * sizeof(long long), cudaMemcpyDeviceToHost));
  if (reset) C6_CUDA(e, cudaMemset(e->wait_dev, 0, 8 * sizeof(long long)));
  return C6_OK;
#else
  (void)reset;
  return fail(e, C6_ERR_UNSUPPORTED, "the library was built without -DC6_TIMED_BUILD: no in-kernel clock counters");
#endif
}

int c6_debug_cta_times(C6Engine* e, int64_t* out, int n_ctas) {
  if (!e || !out || n_ctas < 1 || n_ctas > 512) return C6_ERR_ARG;
#ifdef C6_TIMED_BUILD
  C6_CUDA(e, cudaSetDevice(e->device));
  C6_CUDA(e, cudaMemcpy(out, e->wait_dev + 8, (size_t)n_ctas * 4 * sizeof(long long), cudaMemcpyDeviceToHost));
  return C6_OK;
#else
  return fail(e, C6_ERR_UNSUPPORTED, "the library was built without -DC6_TIMED_BUILD: no in-kernel clock counters");
#endif
}

int c6_debug_expire_wait(C6Engine* e, void* stream) {
  if (!e) return C6_ERR_ARG;
  C6_CUDA(e, cudaSetDevice(e->device));
  expire_wait_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(e->status_dev, 1000000LL);
  C6_LAUNCHED(e, "expire_wait_kernel");
  return C6_OK;
}

int c6_clear_status(C6Engine* e) {
  if (!e) return C6_ERR_ARG;
  C6_CUDA(e, cudaSetDevice(e->device));
  C6_CUDA(e, cudaMemset(e->status_dev, 0, sizeof(int)));
  e->err.clear();
  return C6_OK;
}

int64_t c6_launch_count(const C6Engine* e) { return e ? e->launches : 0; }
int64_t c6_device_bytes(const C6Engine* e) { return e ? e->dev_bytes : 0; }

}  // extern "C"

// the training-side operators (include/c6_train.h) share this translation unit's kernels
#include "c6_train_ops.cuh"
