// Training-side operators (include/c6_train.h): the backward pass of one backbone layer, and forward + backward of
// a whole stack of 3 x 3 layers with the activations and gradients kept in the kernels' own plane layout between
// layers.  Host code, compiled as part of c6_engine.cu (one translation unit: the helper kernels are shared).
//
// Launch sequence of c6_conv_layer_backward on the caller's stream:
//   pack filter (forward layout and the flipped / transposed one), pack x and dy into channel-chunk planes
//   -> conv_tc_kernel<kEpiDsilu>: dPre = dy * silu'(conv(x, W) + b)      (forward recomputed on tensor cores)
//   -> column sums of dPre                                              = db
//   -> conv_tc_kernel<kEpiLinear>: dX = conv(dPre, W flipped/transposed)   -> unpack to NCHW
//   -> wgrad_tc_kernel + wgrad_reduce_kernel                            = dW
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/c6_train.h"
#include "c6_aux_kernels.cuh"
#include "c6_conv_tc.cuh"
#include "c6_host_plan.h"
#include "c6_train_kernels.cuh"
#include "c6_wgrad_tc.cuh"

using namespace c6;

namespace {

thread_local std::string g_train_error = "";

int tfail(int code, const std::string& msg) {
  g_train_error = msg;
  return code;
}

#define C6T_CUDA(call)                                                                         \
  do {                                                                                         \
    cudaError_t _st = (call);                                                                  \
    if (_st != cudaSuccess) return tfail(C6_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_st)); \
  } while (0)

#define C6T_LAUNCHED(name)                                                                     \
  do {                                                                                         \
    cudaError_t _st = cudaGetLastError();                                                      \
    if (_st != cudaSuccess) return tfail(C6_ERR_CUDA, std::string("launch ") + name + ": " + cudaGetErrorString(_st)); \
  } while (0)

constexpr int kColsumSlices = 64;

// Shape-derived layout of one call: the forward kernels' padded linear board geometry and the carve-up of
// the workspace.
struct BackwardLayout {
  bool ok = false;
  int n = 0, k = 0, cin = 0, cout = 0, cin_p = 0, cout_p = 0;
  int wp = 0, slots = 0, halo_rows = 0, front = 0, tiles = 0, tiles_per_board = 0;
  long long B = 0, total_pos = 0, plane_rows = 0;
  LayerPlan fwd, dgrad;           // pipeline plans of the two conv_tc_kernel launches
  int wg_taps_per_cta = 0, wg_groups = 0, wg_slabs = 0, wg_stages = 0, wg_smem = 0, wg_tile_rows = 128, wg_tiles = 0;
  // workspace offsets in bytes
  size_t off_bias = 0, off_zero = 0, off_wf = 0, off_wf_pair = 0, off_wd = 0, off_wd_pair = 0, off_x = 0, off_dy = 0,
         off_dpre = 0, off_dx = 0, off_partial = 0, off_colsum = 0, total = 0;
};

BackwardLayout make_layout(int n, int k, int cin, int cout, long long B, int sms) {
  BackwardLayout L;
  if (n < 1 || n > 32 || k != 3 || cin < 1 || cout < 1 || B < 1) return L;
  L.n = n; L.k = k; L.cin = cin; L.cout = cout; L.B = B;
  L.cin_p = round_up(cin, 32);
  L.cout_p = round_up(cout, 32);
  if (L.cin_p > 128 || L.cout_p > 128) return L;
  const int pad = k / 2;
  L.wp = n + pad;
  L.slots = L.wp * L.wp;
  L.halo_rows = round_up(pad * L.wp + pad, 8);
  L.front = L.halo_rows;
  const int used = (n - 1) * L.wp + n, tpb = (used + 127) / 128;
  L.tiles_per_board = tpb * 128 < L.slots ? tpb : 0;
  long long tiles = L.tiles_per_board ? B * tpb : (B * L.slots + 127) / 128;
  tiles += tiles & 1;                                      // CTA pairs take tiles two at a time
  if (tiles > 0x7fffffffLL / 128) return L;
  L.tiles = (int)tiles;
  L.total_pos = L.tiles_per_board ? round_up_ll((long long)((tiles + tpb - 1) / tpb) * L.slots, 128) : tiles * 128;
  L.plane_rows = (long long)L.front + L.total_pos + L.halo_rows + 256;   // + one K tile of the weight-gradient kernel
  const int rows = conv_stage_rows(L.halo_rows);
  L.fwd.k = k; L.fwd.cin = cin; L.fwd.cout = cout; L.fwd.cin_p = L.cin_p; L.fwd.cout_p = L.cout_p;
  L.dgrad.k = k; L.dgrad.cin = cout; L.dgrad.cout = cin; L.dgrad.cin_p = L.cout_p; L.dgrad.cout_p = L.cin_p;
  if (!plan_tc_layer(sms >= 2, L.fwd, k * k, L.cin_p / 16, rows, 2, 2)) return L;
  if (!plan_tc_layer(sms >= 2, L.dgrad, k * k, L.cout_p / 16, rows, 2, 2)) return L;
  L.wg_taps_per_cta = std::min(std::min(k * k, kWgradMaxTaps), 512 / L.cin_p);
  L.wg_groups = (k * k + L.wg_taps_per_cta - 1) / L.wg_taps_per_cta;
  L.wg_slabs = std::max(1, sms / L.wg_groups);
  // 32 KB of slack behind the last stage: the M = 128 operand descriptor addresses 16 channel groups even
  // when fewer gradient planes exist (those accumulator rows are never read).  K tiles of 256 positions when
  // two stages of that size fit, else 128.
  const int room = kSmemLimit - 128 - kWgradSmemHeader - 32768;
  L.wg_tile_rows = 2 * wgrad_stage_bytes(L.cin_p, L.cout_p, L.halo_rows, 256) <= room ? 256 : 128;
  const int stage = wgrad_stage_bytes(L.cin_p, L.cout_p, L.halo_rows, L.wg_tile_rows);
  L.wg_stages = std::min(kWgradMaxStages, room / stage);
  if (L.wg_stages < 2) return L;
  L.wg_smem = 128 + kWgradSmemHeader + L.wg_stages * stage + 32768;
  L.wg_tiles = (int)((L.total_pos + L.wg_tile_rows - 1) / L.wg_tile_rows);
  auto take = [&](size_t bytes) { size_t o = L.total; L.total += (bytes + 255) & ~(size_t)255; return o; };
  take(256);                                                // status word
  L.off_bias = take((size_t)L.cout_p * 4);
  L.off_zero = take((size_t)L.cin_p * 4);
  L.off_wf = take(L.fwd.w_rows_per_group * 16);
  L.off_wf_pair = take(L.fwd.w_rows_per_group * 16);
  L.off_wd = take(L.dgrad.w_rows_per_group * 16);
  L.off_wd_pair = take(L.dgrad.w_rows_per_group * 16);
  L.off_x = take((size_t)(L.cin_p / 8) * L.plane_rows * 16);
  L.off_dy = take((size_t)(L.cout_p / 8) * L.plane_rows * 16);
  L.off_dpre = take((size_t)(L.cout_p / 8) * L.plane_rows * 16);
  L.off_dx = take((size_t)(L.cin_p / 8) * L.plane_rows * 16);
  L.off_partial = take((size_t)L.wg_slabs * k * k * 128 * L.cin_p * 4);
  L.off_colsum = take((size_t)(L.cout_p / 8) * kColsumSlices * 8 * 4);
  L.ok = true;
  return L;
}

using ConvKernel = void (*)(ConvTcParams);

int launch_conv(const BackwardLayout& L, const LayerPlan& lp, int epi, const uint4* in, uint4* out, const uint4* aux,
                const uint4* w, const uint4* w_pair, const float* bias, int* status, int sms, cudaStream_t st) {
  ConvTcParams p{};
  p.in = in;
  p.out = out;
  p.aux = aux;
  p.w = w;
  p.w_pair = w_pair;
  p.bias = bias;
  p.status = status;
  p.plane_rows = L.plane_rows;
  p.in_plane_rows = L.plane_rows;
  p.front = L.front;
  p.halo_rows = L.halo_rows;
  p.halo_after = L.halo_rows;
  p.cin = lp.cin_p;
  p.n = lp.cout_p;
  p.kside = lp.k;
  p.ntaps = lp.k * lp.k;
  p.planes_step = 2 * lp.qps;
  p.wp = L.wp;
  p.slots = L.slots;
  p.bsize = L.n;
  p.nboards = (int)L.B;
  p.tiles_per_group = L.tiles;
  p.tiles_per_board = L.tiles_per_board;
  p.group_pos = (int)L.total_pos;
  p.ctas_per_group = std::max(1, std::min(sms, L.tiles));
  if (lp.pair) p.ctas_per_group = std::max(2, p.ctas_per_group & ~1);
  p.resident = lp.resident;
  p.nstages = lp.nstages;
  p.nissue = lp.nissue;
  p.spi = lp.spi;
  p.qps = lp.qps;
  p.acc_stride = lp.acc_stride;
  p.nacc = lp.nacc;
  p.tmem_cols = lp.tmem_cols;
  ConvKernel kernel = lp.pair ? (epi == kEpiDsilu   ? conv_tc_kernel<3, true, false, false, kEpiDsilu>
                                 : epi == kEpiLinear ? conv_tc_kernel<3, true, false, false, kEpiLinear>
                                                     : conv_tc_kernel<3, true, false, false, kEpiSilu>)
                              : (epi == kEpiDsilu   ? conv_tc_kernel<3, false, false, false, kEpiDsilu>
                                 : epi == kEpiLinear ? conv_tc_kernel<3, false, false, false, kEpiLinear>
                                                     : conv_tc_kernel<3, false, false, false, kEpiSilu>);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
    return tfail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  // programmatic dependent launch: the kernel's prologue (barriers, TMEM, weight copies) overlaps the tail of the launch
  // before it; every role that touches activations waits for that launch to complete (griddepcontrol.wait) first.  The
  // weights were packed at least two launches earlier.
  launch_chain(kernel, (unsigned)p.ctas_per_group, 1u, kConvThreads, (size_t)lp.smem, st, lp.pair != 0, true, p);
  C6T_LAUNCHED("conv_tc_kernel (backward)");
  return C6_OK;
}


// dW = sum over positions of dPre (x) shifted x: wgrad_tc_kernel into per-slab partial sums, then the fixed-order reduction.
int launch_wgrad(const BackwardLayout& L, const uint4* xp, const uint4* dpre, float* partial, float* dw, int* status,
                 cudaStream_t st) {
  const int taps = L.k * L.k;
  WgradParams p{};
  p.x = xp;
  p.dpre = dpre;
  p.partial = partial;
  p.status = status;
  p.plane_rows = L.plane_rows;
  p.front = L.front;
  p.halo_rows = L.halo_rows;
  p.cin = L.cin_p;
  p.cout = L.cout_p;
  p.kside = L.k;
  p.wp = L.wp;
  p.tile_rows = L.wg_tile_rows;
  p.ntiles = L.wg_tiles;
  p.ntaps = taps;
  p.taps_per_cta = L.wg_taps_per_cta;
  p.ngroups = L.wg_groups;
  p.nslabs = L.wg_slabs;          // planned for 148 SMs: the partial-sum buffer is sized for it
  p.nstages = L.wg_stages;
  if (cudaFuncSetAttribute(wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
    return tfail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  wgrad_tc_kernel<<<(unsigned)(p.ngroups * p.nslabs), kWgradThreads, (size_t)L.wg_smem, st>>>(p);
  C6T_LAUNCHED("wgrad_tc_kernel");
  const long long total = (long long)L.cout * L.cin * taps;
  wgrad_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(partial, dw, p.nslabs, taps, L.cin_p, L.cin, L.cout);
  C6T_LAUNCHED("wgrad_reduce_kernel");
  return C6_OK;
}

// A stack of consecutive 3 x 3 layers (the backbone after the stem) differentiated as a whole: every layer's input
// activation is kept as channel-chunk planes by the forward call, gradients travel between layers in the same layout.
struct StackLayout {
  bool ok = false;
  int L = 0, cmax_p = 0;
  BackwardLayout lay[C6_MAX_LAYERS];      // per layer: pipeline plans; the board geometry is the same for all
  size_t off_bias[C6_MAX_LAYERS] = {}, off_wf[C6_MAX_LAYERS] = {}, off_wf_pair[C6_MAX_LAYERS] = {}, off_wd[C6_MAX_LAYERS] = {},
         off_wd_pair[C6_MAX_LAYERS] = {}, off_act[C6_MAX_LAYERS + 1] = {};
  size_t off_zero = 0, off_grad[2] = {}, off_dpre = 0, off_partial = 0, off_colsum = 0, total = 0;
};

StackLayout make_stack_layout(int n, int nlayers, const int32_t* channels, long long B) {
  StackLayout S;
  if (nlayers < 1 || nlayers > C6_MAX_LAYERS || !channels) return S;
  S.L = nlayers;
  size_t partial_max = 0, colsum_max = 0;
  for (int l = 0; l < nlayers; ++l) {
    S.lay[l] = make_layout(n, 3, channels[l], channels[l + 1], B, 148);
    if (!S.lay[l].ok) return S;
    S.cmax_p = std::max(S.cmax_p, std::max(S.lay[l].cin_p, S.lay[l].cout_p));
    partial_max = std::max(partial_max, (size_t)S.lay[l].wg_slabs * 9 * 128 * S.lay[l].cin_p * 4);
    colsum_max = std::max(colsum_max, (size_t)(S.lay[l].cout_p / 8) * kColsumSlices * 8 * 4);
  }
  const long long plane_rows = S.lay[0].plane_rows;
  auto take = [&](size_t bytes) { size_t o = S.total; S.total += (bytes + 255) & ~(size_t)255; return o; };
  take(256);                                                // status word
  S.off_zero = take((size_t)S.cmax_p * 4);
  for (int l = 0; l < nlayers; ++l) {
    const BackwardLayout& L = S.lay[l];
    S.off_bias[l] = take((size_t)L.cout_p * 4);
    S.off_wf[l] = take(L.fwd.w_rows_per_group * 16);
    S.off_wf_pair[l] = take(L.fwd.w_rows_per_group * 16);
    S.off_wd[l] = take(L.dgrad.w_rows_per_group * 16);
    S.off_wd_pair[l] = take(L.dgrad.w_rows_per_group * 16);
  }
  for (int l = 0; l <= nlayers; ++l) {
    const int cp = l < nlayers ? S.lay[l].cin_p : S.lay[l - 1].cout_p;
    S.off_act[l] = take((size_t)(cp / 8) * plane_rows * 16);
  }
  S.off_grad[0] = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_grad[1] = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_dpre = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_partial = take(partial_max);
  S.off_colsum = take(colsum_max);
  S.ok = true;
  return S;
}

int check_stack_call(int32_t device, const StackLayout& S, void* workspace, int64_t workspace_bytes, int* sms) {
  if (!S.ok) return tfail(C6_ERR_UNSUPPORTED, "the backbone operators support 1..16 layers of 3 x 3, board_size <= 32, at most 128 channels");
  if (!workspace) return tfail(C6_ERR_ARG, "null pointer");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return tfail(C6_ERR_ARG, "workspace must be 256-byte aligned");
  if (workspace_bytes < (int64_t)S.total) {
    char buf[160];
    snprintf(buf, sizeof(buf), "workspace of %lld bytes is smaller than the %zu this shape needs", (long long)workspace_bytes, S.total);
    return tfail(C6_ERR_ARG, buf);
  }
  int ndev = 0, major = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev)
    return tfail(C6_ERR_CUDA, "no such CUDA device (this operator has no CPU path)");
  C6T_CUDA(cudaSetDevice(device));
  C6T_CUDA(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, device));
  C6T_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10) return tfail(C6_ERR_UNSUPPORTED, "the backward operators need an sm_100 GPU (tcgen05 tensor cores)");
  return C6_OK;
}

}  // namespace

extern "C" {

const char* c6_train_last_error(void) { return g_train_error.c_str(); }

int64_t c6_conv_layer_backward_workspace_bytes(int32_t board_size, int32_t kside, int32_t cin, int32_t cout, int64_t B) {
  const BackwardLayout L = make_layout(board_size, kside, cin, cout, B, 148);
  return L.ok ? (int64_t)L.total : 0;
}

int c6_conv_layer_backward(int32_t device, int32_t board_size, int32_t kside, int32_t cin, int32_t cout, int64_t B,
                           const float* x, const float* w, const float* bias, const float* dy, float* dx, float* dw,
                           float* db, void* workspace, int64_t workspace_bytes, void* stream) {
  if (B < 0) return tfail(C6_ERR_ARG, "negative board count");
  if (!w || !dw || !db || !workspace || (B > 0 && (!x || !dy))) return tfail(C6_ERR_ARG, "null pointer");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return tfail(C6_ERR_ARG, "workspace must be 256-byte aligned");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev)
    return tfail(C6_ERR_CUDA, "no such CUDA device (this operator has no CPU path)");
  C6T_CUDA(cudaSetDevice(device));
  int sms = 0, major = 0;
  C6T_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  C6T_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10) return tfail(C6_ERR_UNSUPPORTED, "the backward operators need an sm_100 GPU (tcgen05 tensor cores)");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (B == 0) {
    C6T_CUDA(cudaMemsetAsync(dw, 0, (size_t)cout * cin * kside * kside * sizeof(float), st));
    C6T_CUDA(cudaMemsetAsync(db, 0, (size_t)cout * sizeof(float), st));
    return C6_OK;
  }
  // the workspace layout must not depend on the device: always planned for 148 SMs, launched on what is there
  const BackwardLayout L = make_layout(board_size, kside, cin, cout, B, 148);
  if (!L.ok) return tfail(C6_ERR_UNSUPPORTED, "c6_conv_layer_backward supports k = 3, board_size <= 32, cin and cout <= 128");
  if (workspace_bytes < (int64_t)L.total) {
    char buf[160];
    snprintf(buf, sizeof(buf), "workspace of %lld bytes is smaller than the %zu this shape needs", (long long)workspace_bytes, L.total);
    return tfail(C6_ERR_ARG, buf);
  }
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  float* bias_f = reinterpret_cast<float*>(ws + L.off_bias);
  float* zero_f = reinterpret_cast<float*>(ws + L.off_zero);
  uint4* wf = reinterpret_cast<uint4*>(ws + L.off_wf);
  uint4* wf_pair = reinterpret_cast<uint4*>(ws + L.off_wf_pair);
  uint4* wd = reinterpret_cast<uint4*>(ws + L.off_wd);
  uint4* wd_pair = reinterpret_cast<uint4*>(ws + L.off_wd_pair);
  uint4* xp = reinterpret_cast<uint4*>(ws + L.off_x);
  uint4* dyp = reinterpret_cast<uint4*>(ws + L.off_dy);
  uint4* dpre = reinterpret_cast<uint4*>(ws + L.off_dpre);
  uint4* dxp = reinterpret_cast<uint4*>(ws + L.off_dx);
  float* partial = reinterpret_cast<float*>(ws + L.off_partial);
  float* colsum = reinterpret_cast<float*>(ws + L.off_colsum);
  const int taps = kside * kside;

  // operands
  copy_pad_f32_kernel<<<(L.cout_p + 127) / 128, 128, 0, st>>>(bias, bias_f, cout, L.cout_p);
  C6T_LAUNCHED("copy_pad_f32_kernel");
  {
    const long long rows = (long long)L.fwd.w_rows_per_group;
    pack_conv_weights_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(w, wf, cout, cin, kside, L.cout_p, L.cin_p, 0);
    C6T_LAUNCHED("pack_conv_weights_kernel");
    pack_conv_weights_pair_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(w, wf_pair, cout, cin, kside, L.cout_p, L.cin_p, 0);
    C6T_LAUNCHED("pack_conv_weights_pair_kernel");
    const long long drows = (long long)L.dgrad.w_rows_per_group;
    pack_dgrad_weights_kernel<<<(unsigned)((drows + 255) / 256), 256, 0, st>>>(w, wd, cout, cin, kside, L.cout_p, L.cin_p, 1);
    C6T_LAUNCHED("pack_dgrad_weights_kernel");
    pack_dgrad_weights_kernel<<<(unsigned)((drows + 255) / 256), 256, 0, st>>>(w, wd_pair, cout, cin, kside, L.cout_p, L.cin_p, 2);
    C6T_LAUNCHED("pack_dgrad_weights_kernel");
  }
  {
    const long long tx = B * L.slots * (L.cin_p / 8), ty = B * L.slots * (L.cout_p / 8);
    pack_nchw_planes_kernel<<<(unsigned)((tx + 255) / 256), 256, 0, st>>>(x, xp, L.plane_rows, L.front, L.slots, L.wp, L.n, cin, L.cin_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
    pack_nchw_planes_kernel<<<(unsigned)((ty + 255) / 256), 256, 0, st>>>(dy, dyp, L.plane_rows, L.front, L.slots, L.wp, L.n, cout, L.cout_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
  }
  // dPre = dy * silu'(conv(x, W) + b)
  int rc = launch_conv(L, L.fwd, kEpiDsilu, xp, dpre, dyp, wf, wf_pair, bias_f, status, sms, st);
  if (rc) return rc;
  // db
  colsum_planes_kernel<<<dim3((unsigned)(L.cout_p / 8), kColsumSlices), kColsumThreads, 0, st>>>(dpre, L.plane_rows, L.front,
                                                                                                  L.total_pos, kColsumSlices, colsum);
  C6T_LAUNCHED("colsum_planes_kernel");
  colsum_finish_kernel<<<(cout + 127) / 128, 128, 0, st>>>(colsum, kColsumSlices, cout, db);
  C6T_LAUNCHED("colsum_finish_kernel");
  // dX
  if (dx) {
    rc = launch_conv(L, L.dgrad, kEpiLinear, dpre, dxp, nullptr, wd, wd_pair, zero_f, status, sms, st);
    if (rc) return rc;
    const long long total = B * ((cin + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(dxp, L.plane_rows, L.front, L.slots, L.wp, L.n, cin, B, dx);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  // dW
  rc = launch_wgrad(L, xp, dpre, partial, dw, status, st);
  if (rc) return rc;
  return C6_OK;
}

int64_t c6_backbone_workspace_bytes(int32_t board_size, int32_t nlayers, const int32_t* channels, int64_t B) {
  if (B < 1) return 0;
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, B);
  return S.ok ? (int64_t)S.total : 0;
}

int c6_backbone_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int64_t B,
                        const float* x, const float* const* w, const float* const* bias, float* y, void* workspace,
                        int64_t workspace_bytes, void* stream) {
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!x || !w || !bias || !y || !channels) return tfail(C6_ERR_ARG, "null pointer");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, B);
  int sms = 0;
  int rc = check_stack_call(device, S, workspace, workspace_bytes, &sms);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  {
    StackPackParams pp{};
    long long max_rows = 0;
    for (int l = 0; l < nlayers; ++l) {
      const BackwardLayout& L = S.lay[l];
      if (!w[l]) return tfail(C6_ERR_ARG, "null weight pointer");
      StackPackParams::Layer& q = pp.layer[l];
      q.w = w[l];
      q.bias = bias[l];
      q.wf = reinterpret_cast<uint4*>(ws + S.off_wf[l]);
      q.wf_pair = reinterpret_cast<uint4*>(ws + S.off_wf_pair[l]);
      q.wd = reinterpret_cast<uint4*>(ws + S.off_wd[l]);
      q.wd_pair = reinterpret_cast<uint4*>(ws + S.off_wd_pair[l]);
      q.bias_f = reinterpret_cast<float*>(ws + S.off_bias[l]);
      q.cout = L.cout; q.cin = L.cin; q.cout_p = L.cout_p; q.cin_p = L.cin_p;
      max_rows = std::max(max_rows, std::max((long long)L.fwd.w_rows_per_group, (long long)L.dgrad.w_rows_per_group));
    }
    pack_stack_weights_kernel<<<dim3((unsigned)((max_rows + 255) / 256), (unsigned)nlayers, 5u), 256, 0, st>>>(pp);
    C6T_LAUNCHED("pack_stack_weights_kernel");
  }
  const BackwardLayout& L0 = S.lay[0];
  {
    const long long t = B * L0.slots * (L0.cin_p / 8);
    pack_nchw_planes_kernel<<<(unsigned)((t + 255) / 256), 256, 0, st>>>(
        x, reinterpret_cast<uint4*>(ws + S.off_act[0]), L0.plane_rows, L0.front, L0.slots, L0.wp, L0.n, L0.cin, L0.cin_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
  }
  for (int l = 0; l < nlayers; ++l) {
    const BackwardLayout& L = S.lay[l];
    rc = launch_conv(L, L.fwd, kEpiSilu, reinterpret_cast<const uint4*>(ws + S.off_act[l]),
                     reinterpret_cast<uint4*>(ws + S.off_act[l + 1]), nullptr, reinterpret_cast<const uint4*>(ws + S.off_wf[l]),
                     reinterpret_cast<const uint4*>(ws + S.off_wf_pair[l]), reinterpret_cast<const float*>(ws + S.off_bias[l]),
                     status, sms, st);
    if (rc) return rc;
  }
  {
    const BackwardLayout& L = S.lay[nlayers - 1];
    const long long total = B * ((L.cout + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(ws + S.off_act[nlayers]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cout, B, y);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  return C6_OK;
}

int c6_backbone_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int64_t B,
                         const float* dy, float* dx, float* const* dw, float* const* db, void* workspace,
                         int64_t workspace_bytes, void* stream) {
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!dy || !dw || !db || !channels) return tfail(C6_ERR_ARG, "null pointer");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, B);
  int sms = 0;
  int rc = check_stack_call(device, S, workspace, workspace_bytes, &sms);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  const float* zero_f = reinterpret_cast<const float*>(ws + S.off_zero);
  uint4* dpre = reinterpret_cast<uint4*>(ws + S.off_dpre);
  float* partial = reinterpret_cast<float*>(ws + S.off_partial);
  float* colsum = reinterpret_cast<float*>(ws + S.off_colsum);
  int cur = 0;
  {
    const BackwardLayout& L = S.lay[nlayers - 1];
    const long long t = B * L.slots * (L.cout_p / 8);
    pack_nchw_planes_kernel<<<(unsigned)((t + 255) / 256), 256, 0, st>>>(
        dy, reinterpret_cast<uint4*>(ws + S.off_grad[cur]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cout, L.cout_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
  }
  for (int l = nlayers - 1; l >= 0; --l) {
    const BackwardLayout& L = S.lay[l];
    if (!dw[l] || !db[l]) return tfail(C6_ERR_ARG, "null gradient pointer");
    const uint4* act = reinterpret_cast<const uint4*>(ws + S.off_act[l]);
    // dPre = dY * silu'(conv(act, W) + b)
    rc = launch_conv(L, L.fwd, kEpiDsilu, act, dpre, reinterpret_cast<const uint4*>(ws + S.off_grad[cur]),
                     reinterpret_cast<const uint4*>(ws + S.off_wf[l]), reinterpret_cast<const uint4*>(ws + S.off_wf_pair[l]),
                     reinterpret_cast<const float*>(ws + S.off_bias[l]), status, sms, st);
    if (rc) return rc;
    colsum_planes_kernel<<<dim3((unsigned)(L.cout_p / 8), kColsumSlices), kColsumThreads, 0, st>>>(dpre, L.plane_rows, L.front,
                                                                                                    L.total_pos, kColsumSlices, colsum);
    C6T_LAUNCHED("colsum_planes_kernel");
    colsum_finish_kernel<<<(L.cout + 127) / 128, 128, 0, st>>>(colsum, kColsumSlices, L.cout, db[l]);
    C6T_LAUNCHED("colsum_finish_kernel");
    rc = launch_wgrad(L, act, dpre, partial, dw[l], status, st);
    if (rc) return rc;
    if (l > 0 || dx) {
      rc = launch_conv(L, L.dgrad, kEpiLinear, dpre, reinterpret_cast<uint4*>(ws + S.off_grad[cur ^ 1]), nullptr,
                       reinterpret_cast<const uint4*>(ws + S.off_wd[l]), reinterpret_cast<const uint4*>(ws + S.off_wd_pair[l]),
                       zero_f, status, sms, st);
      if (rc) return rc;
      cur ^= 1;
    }
  }
  if (dx) {
    const BackwardLayout& L = S.lay[0];
    const long long total = B * ((L.cin + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(ws + S.off_grad[cur]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cin, B, dx);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  return C6_OK;
}

}  // extern "C"
