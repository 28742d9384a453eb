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
#include <cmath>
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
constexpr int kHeadBlocks = 592;     // blocks of the heads' backward kernel (4 per SM of a B200), each leaves one row of partial sums (four times as many
                                     // blocks made the kernel 15 % faster and the sum over their rows four times slower: no gain)

// Shape-derived layout of one call: the forward kernels' padded linear board geometry and the carve-up of
// the workspace.
struct BackwardLayout {
  bool ok = false;
  int n = 0, k = 0, cin = 0, cout = 0, cin_p = 0, cout_p = 0;
  int wp = 0, slots = 0, halo_rows = 0, front = 0, tiles = 0, tiles_per_board = 0;
  long long B = 0, total_pos = 0, plane_rows = 0;
  LayerPlan fwd, dgrad;           // pipeline plans of the two conv_tc_kernel launches
  int wg_taps_per_cta = 0, wg_groups = 0, wg_slabs = 0, wg_stages = 0, wg_smem = 0, wg_tile_rows = 128, wg_tiles = 0;
  int wg_bias_tap = -1;           // >= 0: the weight-gradient kernel also produces the bias gradient (see WgradParams)
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
  // the bias gradient rides on the last tap of group 0 when 16 more accumulator columns fit; a tap fewer per CTA is
  // taken for that if it needs no further tap group
  {
    int t2 = L.wg_taps_per_cta;
    while (t2 > 1 && t2 * L.cin_p + 16 > 512) --t2;
    if ((k * k + t2 - 1) / t2 == L.wg_groups) L.wg_taps_per_cta = t2;
  }
  const int taps0 = std::min(L.wg_taps_per_cta, k * k);
  const bool with_bias = taps0 * L.cin_p + 16 <= 512;
  L.wg_bias_tap = with_bias ? taps0 - 1 : -1;
  L.wg_tile_rows = 2 * wgrad_stage_bytes(L.cin_p, L.cout_p, L.halo_rows, 256, with_bias) <= room ? 256 : 128;
  const int stage = wgrad_stage_bytes(L.cin_p, L.cout_p, L.halo_rows, L.wg_tile_rows, with_bias);
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
  L.off_partial = take((size_t)L.wg_slabs * k * k * 128 * L.cin_p * 4 + (size_t)L.wg_slabs * 128 * 4);
  L.off_colsum = take((size_t)(L.cout_p / 8) * kColsumSlices * 8 * 4);
  L.ok = true;
  return L;
}

using ConvKernel = void (*)(ConvTcParams);

int launch_conv(const BackwardLayout& L, const LayerPlan& lp, int epi, const uint4* in, uint4* out, const uint4* aux,
                const uint4* w, const uint4* w_pair, const float* bias, int* status, int sms, cudaStream_t st,
                uint4* out2 = nullptr) {
  ConvTcParams p{};
  p.in = in;
  p.out = out;
  p.aux = aux;
  p.out2 = out2;
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
  static const ConvKernel table[2][5] = {
      {conv_tc_kernel<3, false, false, false, kEpiSilu>, conv_tc_kernel<3, false, false, false, kEpiLinear>,
       conv_tc_kernel<3, false, false, false, kEpiDsilu>, conv_tc_kernel<3, false, false, false, kEpiSiluSave>,
       conv_tc_kernel<3, false, false, false, kEpiLinearMul>},
      {conv_tc_kernel<3, true, false, false, kEpiSilu>, conv_tc_kernel<3, true, false, false, kEpiLinear>,
       conv_tc_kernel<3, true, false, false, kEpiDsilu>, conv_tc_kernel<3, true, false, false, kEpiSiluSave>,
       conv_tc_kernel<3, true, false, false, kEpiLinearMul>}};
  ConvKernel kernel = table[lp.pair ? 1 : 0][epi];
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
// With db and a layout that fuses it (L.wg_bias_tap >= 0) the same launches also produce the bias gradient; the caller
// checks L.wg_bias_tap and runs the column-sum kernels otherwise.
int launch_wgrad(const BackwardLayout& L, const uint4* xp, const uint4* dpre, float* partial, float* dw, int* status,
                 cudaStream_t st, float* db = nullptr) {
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
  p.halo_after = L.halo_rows;
  p.dpre_plane_rows = L.plane_rows;
  p.dpre_front = L.front;
  const bool with_bias = db != nullptr && L.wg_bias_tap >= 0;
  float* bias_partial = partial + (size_t)L.wg_slabs * taps * 128 * L.cin_p;
  p.bias_tap = L.wg_bias_tap;      // the stage layout carries the ones planes whenever the layout says so
  p.bias_partial = bias_partial;
  if (cudaFuncSetAttribute(wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
    return tfail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  wgrad_tc_kernel<<<(unsigned)(p.ngroups * p.nslabs), kWgradThreads, (size_t)L.wg_smem, st>>>(p);
  C6T_LAUNCHED("wgrad_tc_kernel");
  const long long total = (long long)L.cout * L.cin * taps;
  wgrad_reduce_kernel<<<(unsigned)((total + L.cout + 255) / 256), 256, 0, st>>>(partial, dw, p.nslabs, taps, L.cin_p, L.cin, L.cout,
                                                                               with_bias ? bias_partial : nullptr, db);
  C6T_LAUNCHED("wgrad_reduce_kernel");
  return C6_OK;
}


// The first layer as the direct stem (conv_tc_kernel's stem mode on x-expanded input planes, see c6_aux_kernels.cuh):
// geometry of the input images, pipeline plan, and the plan of its weight gradient (wgrad_tc_kernel's stem mode).
struct StemLayout {
  bool ok = false;
  int k = 0, kh = 0, hx = 0, wi = 0, slots = 0, halo_b = 0, halo_a = 0, front = 0, cout = 0, cout_p = 0;
  int tiles_per_board = 0, tiles = 0;
  long long group_pos = 0, xe_plane_rows = 0, dsd_plane_rows = 0;
  LayerPlan plan;
  int nkxb = 0, nkyb = 0, wg_ntaps = 0, wg_taps_per_cta = 0, wg_groups = 0, wg_slabs = 0, wg_stages = 0, wg_smem = 0,
      wg_tile_rows = 256, wg_tiles = 0, wg_halo_a = 0;
};

StemLayout make_stem_layout(int n, int k0, int cout, long long B) {
  StemLayout S;
  if (k0 < 3 || (k0 & 1) == 0 || k0 > 31 || n < 1 || n > 32 || cout < 1 || B < 1) return S;
  S.k = k0; S.kh = k0 / 2; S.cout = cout;
  S.cout_p = round_up(cout, 32);
  if (S.cout_p > 64) return S;
  S.hx = (k0 + 15) / 16;
  S.wi = round_up(n + S.kh, 8);
  S.slots = S.wi * (n + S.kh);
  S.halo_b = round_up(S.kh * S.wi + S.kh, 8);
  S.halo_a = round_up(S.kh * S.wi + 16 * S.hx - 1 - S.kh + 8, 8);
  S.front = S.halo_b;
  S.plan.k = k0; S.plan.cin = 3; S.plan.cout = cout; S.plan.cin_p = 48; S.plan.cout_p = S.cout_p;
  if (!plan_tc_layer(true, S.plan, k0 * S.hx, 3, 128 + S.halo_b + S.halo_a, 1, 1)) return S;
  const int used = (n - 1) * S.wi + n, tpb = (used + 127) / 128;
  S.tiles_per_board = tpb * 128 < S.slots ? tpb : 0;
  long long tiles = S.tiles_per_board ? B * tpb : (B * S.slots + 127) / 128;
  if (S.plan.pair) tiles += tiles & 1;
  if (tiles > 0x7fffffffLL / 128) return S;
  S.tiles = (int)tiles;
  S.group_pos = S.tiles_per_board ? round_up_ll((long long)((tiles + tpb - 1) / tpb) * S.slots, 128) : tiles * 128;
  // weight gradient: taps = (input plane, 8 filter columns, 16 filter rows)
  S.nkxb = (k0 + 7) / 8;
  S.nkyb = (k0 + 15) / 16;
  S.wg_ntaps = 3 * S.nkxb * S.nkyb;
  S.wg_taps_per_cta = std::min(std::min(kWgradMaxTaps, 512 / S.cout_p), S.wg_ntaps);
  S.wg_groups = (S.wg_ntaps + S.wg_taps_per_cta - 1) / S.wg_taps_per_cta;
  S.wg_slabs = std::max(1, 148 / S.wg_groups);
  S.wg_halo_a = round_up((16 * S.nkyb - 1 - S.kh) * S.wi + (8 * S.nkxb - 1 - S.kh) + 8, 8);
  const int room = kSmemLimit - 128 - kWgradSmemHeader;
  // K tiles of 128 positions aligned to the board images (the rows behind an image's last cell are padding: the
  // gradient is zero there), or, for geometries whose images are no longer than their tiles, 256 positions running
  // linearly over everything
  S.wg_tile_rows = S.tiles_per_board ? 128 : (2 * wgrad_stem_stage_bytes(S.cout_p, S.halo_b, S.wg_halo_a, 256) <= room ? 256 : 128);
  const int stage = wgrad_stem_stage_bytes(S.cout_p, S.halo_b, S.wg_halo_a, S.wg_tile_rows);
  S.wg_stages = std::min(kWgradMaxStages, room / stage);
  if (S.wg_stages < 2) return S;
  S.wg_smem = 128 + kWgradSmemHeader + S.wg_stages * stage;
  S.wg_tiles = S.tiles_per_board ? (int)(B * S.tiles_per_board) : (int)((B * S.slots + S.wg_tile_rows - 1) / S.wg_tile_rows);
  S.dsd_plane_rows = round_up_ll(B * S.slots + S.wg_tile_rows, 128);
  S.xe_plane_rows = (long long)S.front + std::max(S.group_pos + S.halo_a + 128 + 16, S.dsd_plane_rows + S.wg_halo_a + 16);
  S.ok = true;
  return S;
}

// The direct stem's forward of a training step: out = the first activation planes, out2 = silu' of the same positions,
// both in the layers' geometry G (cells only).
int launch_stem_conv(const StemLayout& S, const BackwardLayout& G, const uint4* xe, uint4* out, uint4* out2, const uint4* w,
                     const uint4* w_pair, const float* bias, int* status, int n, long long B, int sms, cudaStream_t st) {
  const LayerPlan& lp = S.plan;
  ConvTcParams p{};
  p.in = xe;
  p.in_plane_rows = S.xe_plane_rows;
  p.out = out;
  p.out2 = out2;
  p.plane_rows = G.plane_rows;
  p.w = w;
  p.w_pair = w_pair;
  p.bias = bias;
  p.status = status;
  p.front = S.front;
  p.halo_rows = S.halo_b;
  p.halo_after = S.halo_a;
  p.cin = 48;                       // three pipeline steps, one input plane each
  p.n = lp.cout_p;
  p.kside = lp.k;
  p.ntaps = lp.k * S.hx;
  p.planes_step = 1;
  p.stem = 1;
  p.stem_hx = S.hx;
  p.a_lbo_rows = 8;
  p.wp = S.wi;
  p.slots = S.slots;
  p.bsize = n;
  p.nboards = (int)B;
  p.tiles_per_group = S.tiles;
  p.tiles_per_board = S.tiles_per_board;
  p.group_pos = (int)S.group_pos;
  p.out_front = G.front;
  p.out_wp = G.wp;
  p.out_slots = G.slots;
  p.out_group_pos = (int)G.total_pos;
  p.ctas_per_group = std::max(1, std::min(sms, S.tiles));
  if (lp.pair) p.ctas_per_group = std::max(2, p.ctas_per_group & ~1);
  p.resident = lp.resident;
  p.nstages = lp.nstages;
  p.nissue = lp.nissue;
  p.spi = lp.spi;
  p.qps = 1;
  p.acc_stride = lp.acc_stride;
  p.nacc = lp.nacc;
  p.tmem_cols = lp.tmem_cols;
  ConvKernel kernel = lp.pair ? conv_tc_kernel<0, true, false, false, kEpiSiluSave> : conv_tc_kernel<0, false, false, false, kEpiSiluSave>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
    return tfail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  launch_chain(kernel, (unsigned)p.ctas_per_group, 1u, kConvThreads, (size_t)lp.smem, st, lp.pair != 0, true, p);
  C6T_LAUNCHED("conv_tc_kernel (direct stem)");
  return C6_OK;
}

// dW of the stem from the x-expanded input planes and the gradient planes in the input geometry.
int launch_stem_wgrad(const StemLayout& S, const uint4* xe, const uint4* dsd, float* partial, float* dw, int* status,
                      cudaStream_t st) {
  WgradParams p{};
  p.x = xe;
  p.dpre = dsd;
  p.partial = partial;
  p.status = status;
  p.plane_rows = S.xe_plane_rows;
  p.front = S.front;
  p.halo_rows = S.halo_b;
  p.halo_after = S.wg_halo_a;
  p.dpre_plane_rows = S.dsd_plane_rows;
  p.dpre_front = 0;
  p.cin = 0;
  p.cout = S.cout_p;
  p.kside = S.k;
  p.wp = S.wi;
  p.tile_rows = S.wg_tile_rows;
  p.ntiles = S.wg_tiles;
  p.ntaps = S.wg_ntaps;
  p.taps_per_cta = S.wg_taps_per_cta;
  p.ngroups = S.wg_groups;
  p.nslabs = S.wg_slabs;
  p.nstages = S.wg_stages;
  p.stem_k = S.k;
  p.stem_wi = S.wi;
  p.stem_nkxb = S.nkxb;
  p.stem_nkyb = S.nkyb;
  p.tiles_per_board = S.tiles_per_board;
  p.board_rows = S.slots;
  p.bias_tap = -1;
  if (cudaFuncSetAttribute(wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
    return tfail(C6_ERR_CUDA, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed");
  wgrad_tc_kernel<<<(unsigned)(p.ngroups * p.nslabs), kWgradThreads, (size_t)S.wg_smem, st>>>(p);
  C6T_LAUNCHED("wgrad_tc_kernel (stem)");
  const long long total = (long long)S.cout * 3 * S.k * S.k;
  wgrad_reduce_stem_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(partial, dw, p.nslabs, p.ntaps, S.cout_p, S.cout, S.k,
                                                                           S.nkxb, S.nkyb);
  C6T_LAUNCHED("wgrad_reduce_stem_kernel");
  return C6_OK;
}

// A stack of layers differentiated as a whole: an optional first-layer stem (stem_kside x stem_kside on 3 input planes,
// run as the direct stem) followed by 3 x 3 layers.  Every layer's input activation and the derivative silu' of its
// output are kept as channel-chunk planes by the forward call (the stem's input as its x-expanded planes); gradients
// travel between layers in the same layout, as dL/d(convolution output) of the layer about to be processed.
struct StackLayout {
  bool ok = false;
  int L = 0, first = 0, cmax_p = 0;       // layers in all; index of the first 3 x 3 layer (1 with a stem, else 0)
  StemLayout stem;
  BackwardLayout lay[C6_MAX_LAYERS];      // 3 x 3 layers l >= first: pipeline plans; the board geometry is the same for all
  size_t off_bias[C6_MAX_LAYERS] = {}, off_wf[C6_MAX_LAYERS] = {}, off_wf_pair[C6_MAX_LAYERS] = {}, off_wd[C6_MAX_LAYERS] = {},
         off_wd_pair[C6_MAX_LAYERS] = {}, off_act[C6_MAX_LAYERS + 1] = {}, off_der[C6_MAX_LAYERS] = {};
  size_t off_zero = 0, off_grad[2] = {}, off_dpre = 0, off_partial = 0, off_colsum = 0, off_xe = 0, off_dsd = 0, off_heads = 0, total = 0;
};

StackLayout make_stack_layout(int n, int nlayers, const int32_t* channels, int stem_kside, long long B) {
  StackLayout S;
  if (nlayers < 1 || nlayers > C6_MAX_LAYERS || !channels || stem_kside < 0) return S;
  S.L = nlayers;
  S.first = stem_kside > 0 ? 1 : 0;
  if (S.first) {
    if (nlayers < 2 || channels[0] != 3) return S;     // a stem reads the 3 input planes and feeds at least one 3 x 3 layer
    S.stem = make_stem_layout(n, stem_kside, channels[1], B);
    if (!S.stem.ok) return S;
  }
  size_t partial_max = S.first ? (size_t)S.stem.wg_slabs * S.stem.wg_ntaps * 128 * S.stem.cout_p * 4 : 0, colsum_max = 0;
  for (int l = S.first; l < nlayers; ++l) {
    S.lay[l] = make_layout(n, 3, channels[l], channels[l + 1], B, 148);
    if (!S.lay[l].ok) return S;
    S.cmax_p = std::max(S.cmax_p, std::max(S.lay[l].cin_p, S.lay[l].cout_p));
    partial_max = std::max(partial_max, (size_t)S.lay[l].wg_slabs * 9 * 128 * S.lay[l].cin_p * 4 + (size_t)S.lay[l].wg_slabs * 128 * 4);
    colsum_max = std::max(colsum_max, (size_t)(S.lay[l].cout_p / 8) * kColsumSlices * 8 * 4);
  }
  colsum_max = std::max(colsum_max, (size_t)(S.lay[S.first].cin_p / 8) * kColsumSlices * 8 * 4);
  const long long plane_rows = S.lay[S.first].plane_rows;
  auto take = [&](size_t bytes) { size_t o = S.total; S.total += (bytes + 255) & ~(size_t)255; return o; };
  take(256);                                                // status word
  S.off_zero = take((size_t)S.cmax_p * 4);
  if (S.first) {
    S.off_bias[0] = take((size_t)S.stem.cout_p * 4);
    S.off_wf[0] = take(S.stem.plan.w_rows_per_group * 16);
    S.off_wf_pair[0] = take(S.stem.plan.w_rows_per_group * 16);
    S.off_xe = take((size_t)3 * S.stem.xe_plane_rows * 16);
    S.off_dsd = take((size_t)(S.stem.cout_p / 8) * S.stem.dsd_plane_rows * 16);
  }
  for (int l = S.first; l < nlayers; ++l) {
    const BackwardLayout& L = S.lay[l];
    S.off_bias[l] = take((size_t)L.cout_p * 4);
    S.off_wf[l] = take(L.fwd.w_rows_per_group * 16);
    S.off_wf_pair[l] = take(L.fwd.w_rows_per_group * 16);
    S.off_wd[l] = take(L.dgrad.w_rows_per_group * 16);
    S.off_wd_pair[l] = take(L.dgrad.w_rows_per_group * 16);
  }
  for (int l = S.first; l <= nlayers; ++l) {
    const int cp = l < nlayers ? S.lay[l].cin_p : S.lay[l - 1].cout_p;
    S.off_act[l] = take((size_t)(cp / 8) * plane_rows * 16);
  }
  for (int l = 0; l < nlayers; ++l) {      // silu' of every layer's output, kept by the forward for the backward
    const int cp = l < S.first ? S.stem.cout_p : S.lay[l].cout_p;
    S.off_der[l] = take((size_t)(cp / 8) * plane_rows * 16);
  }
  S.off_grad[0] = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_grad[1] = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_dpre = take((size_t)(S.cmax_p / 8) * plane_rows * 16);
  S.off_partial = take(partial_max);
  S.off_colsum = take(colsum_max);
  S.off_heads = take((size_t)kHeadBlocks * ((S.lay[nlayers - 1].cout_p / 8) * 16 + 2) * 4);
  S.ok = true;
  return S;
}

int check_stack_call(int32_t device, const StackLayout& S, void* workspace, int64_t workspace_bytes, int* sms) {
  if (!S.ok)
    return tfail(C6_ERR_UNSUPPORTED, "the backbone operators support 1..16 layers of 3 x 3 with at most 128 channels, board_size <= 32, "
                                     "optionally behind an odd k x k stem (k <= 31) from 3 planes to at most 64 channels");
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
  // db: with the weight gradient when its accumulators have room for the bias columns, else a pass of its own
  if (L.wg_bias_tap < 0) {
    colsum_planes_kernel<<<dim3((unsigned)(L.cout_p / 8), kColsumSlices), kColsumThreads, 0, st>>>(dpre, L.plane_rows, L.front,
                                                                                                    L.total_pos, kColsumSlices, colsum);
    C6T_LAUNCHED("colsum_planes_kernel");
    colsum_finish_kernel<<<(cout + 127) / 128, 128, 0, st>>>(colsum, kColsumSlices, cout, db);
    C6T_LAUNCHED("colsum_finish_kernel");
  }
  // dX
  if (dx) {
    rc = launch_conv(L, L.dgrad, kEpiLinear, dpre, dxp, nullptr, wd, wd_pair, zero_f, status, sms, st);
    if (rc) return rc;
    const long long total = B * ((cin + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(dxp, L.plane_rows, L.front, L.slots, L.wp, L.n, cin, B, dx);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  // dW
  rc = launch_wgrad(L, xp, dpre, partial, dw, status, st, db);
  if (rc) return rc;
  return C6_OK;
}

int64_t c6_backbone_workspace_bytes(int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                                    int64_t B) {
  if (B < 1) return 0;
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, stem_kside, B);
  return S.ok ? (int64_t)S.total : 0;
}

static int backbone_forward_impl(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                                 int64_t B, const InputSrc& in, const float* const* w, const float* const* bias, float* y,
                                 void* workspace, int64_t workspace_bytes, void* stream) {
  const float* x = static_cast<const float*>(in.x);
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!w || !bias || !channels) return tfail(C6_ERR_ARG, "null pointer");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, stem_kside, B);
  int sms = 0;
  int rc = check_stack_call(device, S, workspace, workspace_bytes, &sms);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  {
    StackPackParams pp{};
    long long max_rows = 0;
    for (int l = S.first; l < nlayers; ++l) {
      const BackwardLayout& L = S.lay[l];
      if (!w[l]) return tfail(C6_ERR_ARG, "null weight pointer");
      StackPackParams::Layer& q = pp.layer[l - S.first];
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
    pack_stack_weights_kernel<<<dim3((unsigned)((max_rows + 255) / 256), (unsigned)(nlayers - S.first), 5u), 256, 0, st>>>(pp);
    C6T_LAUNCHED("pack_stack_weights_kernel");
  }
  const BackwardLayout& L0 = S.lay[S.first];
  if (S.first) {
    // the stem: bias, filter rows for the direct stem (whole and split for CTA pairs), x-expanded input planes, convolution
    const StemLayout& T = S.stem;
    if (!w[0]) return tfail(C6_ERR_ARG, "null weight pointer");
    copy_pad_f32_kernel<<<(T.cout_p + 127) / 128, 128, 0, st>>>(bias[0], reinterpret_cast<float*>(ws + S.off_bias[0]), T.cout, T.cout_p);
    C6T_LAUNCHED("copy_pad_f32_kernel");
    const long long rows = (long long)T.plan.w_rows_per_group;
    pack_stem_direct_weights_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
        w[0], reinterpret_cast<uint4*>(ws + S.off_wf[0]), T.cout, T.k, T.cout_p, T.hx, 1, 0);
    C6T_LAUNCHED("pack_stem_direct_weights_kernel");
    pack_stem_direct_weights_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
        w[0], reinterpret_cast<uint4*>(ws + S.off_wf_pair[0]), T.cout, T.k, T.cout_p, T.hx, 2, 0);
    C6T_LAUNCHED("pack_stem_direct_weights_kernel");
    pack_stem_direct_input_kernel<<<dim3((unsigned)B, 1u), kPackDirectThreads, 0, st>>>(
        in, nullptr, reinterpret_cast<uint4*>(ws + S.off_xe), T.xe_plane_rows, T.front, (int)T.group_pos, T.wi, T.slots, board_size,
        (int)B, B, 0, 0, status);
    C6T_LAUNCHED("pack_stem_direct_input_kernel");
    rc = launch_stem_conv(T, L0, reinterpret_cast<const uint4*>(ws + S.off_xe), reinterpret_cast<uint4*>(ws + S.off_act[1]),
                          reinterpret_cast<uint4*>(ws + S.off_der[0]), reinterpret_cast<const uint4*>(ws + S.off_wf[0]),
                          reinterpret_cast<const uint4*>(ws + S.off_wf_pair[0]), reinterpret_cast<const float*>(ws + S.off_bias[0]),
                          status, board_size, B, sms, st);
    if (rc) return rc;
  } else {
    if (!x) return tfail(C6_ERR_ARG, "null pointer");
    const long long t = B * L0.slots * (L0.cin_p / 8);
    pack_nchw_planes_kernel<<<(unsigned)((t + 255) / 256), 256, 0, st>>>(
        x, reinterpret_cast<uint4*>(ws + S.off_act[0]), L0.plane_rows, L0.front, L0.slots, L0.wp, L0.n, L0.cin, L0.cin_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
  }
  for (int l = S.first; l < nlayers; ++l) {
    const BackwardLayout& L = S.lay[l];
    rc = launch_conv(L, L.fwd, kEpiSiluSave, reinterpret_cast<const uint4*>(ws + S.off_act[l]),
                     reinterpret_cast<uint4*>(ws + S.off_act[l + 1]), nullptr, reinterpret_cast<const uint4*>(ws + S.off_wf[l]),
                     reinterpret_cast<const uint4*>(ws + S.off_wf_pair[l]), reinterpret_cast<const float*>(ws + S.off_bias[l]),
                     status, sms, st, reinterpret_cast<uint4*>(ws + S.off_der[l]));
    if (rc) return rc;
  }
  if (y) {
    const BackwardLayout& L = S.lay[nlayers - 1];
    const long long total = B * ((L.cout + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(ws + S.off_act[nlayers]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cout, B, y);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  return C6_OK;
}

int c6_backbone_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                        int64_t B, const float* x, const float* const* w, const float* const* bias, float* y,
                        void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x) return tfail(C6_ERR_ARG, "null pointer");
  InputSrc in{};
  in.x = x;
  return backbone_forward_impl(device, board_size, nlayers, channels, stem_kside, B, in, w, bias, y, workspace, workspace_bytes, stream);
}

int c6_backbone_forward_boards(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                               int64_t B, const int8_t* boards, const int8_t* current_player, const int8_t* stones_left,
                               int64_t num_envs, const int64_t* index, const float* const* w, const float* const* bias, float* y,
                               void* workspace, int64_t workspace_bytes, void* stream) {
  if (!boards || !current_player || !stones_left) return tfail(C6_ERR_ARG, "null pointer");
  if (stem_kside <= 0) return tfail(C6_ERR_ARG, "board input feeds the network's first layer: stem_kside must be given");
  if (num_envs < 1 || (!index && B > num_envs)) return tfail(C6_ERR_ARG, "more boards than environments and no index");
  InputSrc in{};
  in.boards = boards;
  in.player = current_player;
  in.stones_left = stones_left;
  in.index = reinterpret_cast<const long long*>(index);
  in.num_envs = num_envs;
  return backbone_forward_impl(device, board_size, nlayers, channels, stem_kside, B, in, w, bias, y, workspace, workspace_bytes, stream);
}

int c6_backbone_heads_forward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                              int64_t B, const float* wp, const float* bp, const float* wv, const float* bv, float* logits,
                              float* value, void* workspace, int64_t workspace_bytes, void* stream) {
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!wp || !bp || !wv || !bv || !logits || !value || !channels) return tfail(C6_ERR_ARG, "null pointer");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, stem_kside, B);
  int sms = 0;
  int rc = check_stack_call(device, S, workspace, workspace_bytes, &sms);
  if (rc) return rc;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  const BackwardLayout& L = S.lay[nlayers - 1];
  heads_forward_kernel<<<(unsigned)B, kHeadThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(ws + S.off_act[nlayers]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cout, L.cout_p / 8, wp, bp,
      wv, bv, logits, value);
  C6T_LAUNCHED("heads_forward_kernel");
  return C6_OK;
}

int c6_backbone_heads_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                               int64_t B, const float* wp, const float* wv, const float* dlogits, const float* dvalue,
                               const float* value, float* dwp, float* dbp, float* dwv, float* dbv, void* workspace,
                               int64_t workspace_bytes, void* stream) {
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!wp || !wv || !dlogits || !dvalue || !value || !dwp || !dbp || !dwv || !dbv || !channels) return tfail(C6_ERR_ARG, "null pointer");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, stem_kside, B);
  int sms = 0;
  int rc = check_stack_call(device, S, workspace, workspace_bytes, &sms);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  const BackwardLayout& L = S.lay[nlayers - 1];
  const int nq = L.cout_p / 8;
  const int nblocks = (int)std::min<long long>(B, kHeadBlocks);
  float* partial = reinterpret_cast<float*>(ws + S.off_heads);
  heads_backward_kernel<<<(unsigned)nblocks, kHeadThreads, 0, st>>>(
      reinterpret_cast<const uint4*>(ws + S.off_act[nlayers]), reinterpret_cast<const uint4*>(ws + S.off_der[nlayers - 1]),
      reinterpret_cast<uint4*>(ws + S.off_grad[0]), L.plane_rows, L.front,
      L.slots, L.wp, L.n, L.cout, nq, B, wp, wv, dlogits, dvalue, value, partial);
  C6T_LAUNCHED("heads_backward_kernel");
  heads_backward_finish_kernel<<<(2 * L.cout + 2 + 127) / 128, 128, 0, st>>>(partial, nblocks, nq, L.cout, dwp, dbp, dwv, dbv);
  C6T_LAUNCHED("heads_backward_finish_kernel");
  return C6_OK;
}

int c6_backbone_backward(int32_t device, int32_t board_size, int32_t nlayers, const int32_t* channels, int32_t stem_kside,
                         int64_t B, const float* dy, float* dx, float* const* dw, float* const* db, void* workspace,
                         int64_t workspace_bytes, void* stream) {
  if (B < 1) return tfail(C6_ERR_ARG, "board count must be positive");
  if (!dw || !db || !channels) return tfail(C6_ERR_ARG, "null pointer");
  if (stem_kside > 0 && dx) return tfail(C6_ERR_ARG, "with a stem the stack starts at the network input, which has no gradient: dx must be null");
  const StackLayout S = make_stack_layout(board_size, nlayers, channels, stem_kside, B);
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
  // P[cur] holds dPre_l = dL/d(convolution output of layer l) on entry to layer l's step
  int cur = 0;
  if (dy) {   // null: c6_backbone_heads_backward has left dPre of the last layer in the workspace
    const BackwardLayout& L = S.lay[nlayers - 1];
    const long long t = B * L.slots * (L.cout_p / 8);
    pack_nchw_planes_kernel<<<(unsigned)((t + 255) / 256), 256, 0, st>>>(dy, dpre, L.plane_rows, L.front, L.slots, L.wp, L.n, L.cout,
                                                                         L.cout_p, B);
    C6T_LAUNCHED("pack_nchw_planes_kernel");
    const long long rows = (long long)(L.cout_p / 8) * L.plane_rows;
    mul_planes_kernel<<<(unsigned)std::min<long long>((rows + 255) / 256, 4096), 256, 0, st>>>(
        dpre, reinterpret_cast<const uint4*>(ws + S.off_der[nlayers - 1]), reinterpret_cast<uint4*>(ws + S.off_grad[cur]), rows);
    C6T_LAUNCHED("mul_planes_kernel");
  }
  for (int l = nlayers - 1; l >= S.first; --l) {
    const BackwardLayout& L = S.lay[l];
    if (!dw[l] || !db[l]) return tfail(C6_ERR_ARG, "null gradient pointer");
    const uint4* act = reinterpret_cast<const uint4*>(ws + S.off_act[l]);
    const uint4* dpre_l = reinterpret_cast<const uint4*>(ws + S.off_grad[cur]);
    if (L.wg_bias_tap < 0) {     // no room for the bias columns in the weight-gradient kernel's accumulators: a pass of its own
      colsum_planes_kernel<<<dim3((unsigned)(L.cout_p / 8), kColsumSlices), kColsumThreads, 0, st>>>(dpre_l, L.plane_rows, L.front,
                                                                                                      L.total_pos, kColsumSlices, colsum);
      C6T_LAUNCHED("colsum_planes_kernel");
      colsum_finish_kernel<<<(L.cout + 127) / 128, 128, 0, st>>>(colsum, kColsumSlices, L.cout, db[l]);
      C6T_LAUNCHED("colsum_finish_kernel");
    }
    rc = launch_wgrad(L, act, dpre_l, partial, dw[l], status, st, db[l]);
    if (rc) return rc;
    if (l > 0) {
      // the layer below exists: its dPre = (data gradient of this layer) * (its saved silu'), in one pass
      rc = launch_conv(L, L.dgrad, kEpiLinearMul, dpre_l, reinterpret_cast<uint4*>(ws + S.off_grad[cur ^ 1]),
                       reinterpret_cast<const uint4*>(ws + S.off_der[l - 1]), reinterpret_cast<const uint4*>(ws + S.off_wd[l]),
                       reinterpret_cast<const uint4*>(ws + S.off_wd_pair[l]), zero_f, status, sms, st);
      if (rc) return rc;
      cur ^= 1;
    } else if (dx) {
      rc = launch_conv(L, L.dgrad, kEpiLinear, dpre_l, reinterpret_cast<uint4*>(ws + S.off_grad[cur ^ 1]), nullptr,
                       reinterpret_cast<const uint4*>(ws + S.off_wd[l]), reinterpret_cast<const uint4*>(ws + S.off_wd_pair[l]),
                       zero_f, status, sms, st);
      if (rc) return rc;
      cur ^= 1;
    }
  }
  if (S.first) {
    // the stem: db_0 = column sums of dPre_0, dW_0 from the x-expanded input planes and dPre_0 moved into the input geometry
    const StemLayout& T = S.stem;
    const BackwardLayout& G = S.lay[1];
    if (!dw[0] || !db[0]) return tfail(C6_ERR_ARG, "null gradient pointer");
    const uint4* xe = reinterpret_cast<const uint4*>(ws + S.off_xe);
    const uint4* dpre0 = reinterpret_cast<const uint4*>(ws + S.off_grad[cur]);
    uint4* dsd = reinterpret_cast<uint4*>(ws + S.off_dsd);
    colsum_planes_kernel<<<dim3((unsigned)(T.cout_p / 8), kColsumSlices), kColsumThreads, 0, st>>>(dpre0, G.plane_rows, G.front,
                                                                                                    G.total_pos, kColsumSlices, colsum);
    C6T_LAUNCHED("colsum_planes_kernel");
    colsum_finish_kernel<<<(T.cout + 127) / 128, 128, 0, st>>>(colsum, kColsumSlices, T.cout, db[0]);
    C6T_LAUNCHED("colsum_finish_kernel");
    const long long total = B * (T.cout_p / 8) * board_size * board_size;
    repack_planes_geometry_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(dpre0, G.plane_rows, G.front, G.slots, G.wp, dsd,
                                                                                   T.dsd_plane_rows, T.slots, T.wi, board_size,
                                                                                   T.cout_p / 8, B);
    C6T_LAUNCHED("repack_planes_geometry_kernel");
    rc = launch_stem_wgrad(T, xe, dsd, partial, dw[0], status, st);
    if (rc) return rc;
  } else if (dx) {
    const BackwardLayout& L = S.lay[0];
    const long long total = B * ((L.cin + 7) / 8) * L.n * L.n;
    unpack_planes_nchw_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(ws + S.off_grad[cur]), L.plane_rows, L.front, L.slots, L.wp, L.n, L.cin, B, dx);
    C6T_LAUNCHED("unpack_planes_nchw_kernel");
  }
  return C6_OK;
}

int c6_ppo_loss(int32_t device, int64_t B, int32_t A, const float* logits, const uint8_t* legal, const int64_t* actions,
                const float* old_logprob, const float* advantages, const float* returns, const float* values,
                float temperature, float clip_coef, float value_coef, float entropy_coef, float* stats, float* dlogits,
                float* dvalues, void* workspace, int64_t workspace_bytes, void* stream) {
  if (B < 1 || A < 1) return tfail(C6_ERR_ARG, "board and action counts must be positive");
  if (!logits || !legal || !actions || !old_logprob || !advantages || !returns || !values || !stats || !dlogits || !dvalues || !workspace)
    return tfail(C6_ERR_ARG, "null pointer");
  if (workspace_bytes < (int64_t)(B * 5 * sizeof(float))) return tfail(C6_ERR_ARG, "workspace smaller than 20 bytes per board");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev)
    return tfail(C6_ERR_CUDA, "no such CUDA device (this operator has no CPU path)");
  C6T_CUDA(cudaSetDevice(device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* rows = reinterpret_cast<float*>(workspace);
  const float inv_t = 1.f / std::max(temperature, 1e-4f);      // connect6/train.py:1049-1051
  ppo_loss_kernel<<<(unsigned)((B + kPpoWarps - 1) / kPpoWarps), 32 * kPpoWarps, 0, st>>>(
      logits, legal, reinterpret_cast<const long long*>(actions), old_logprob, advantages, returns, values, B, A, inv_t, clip_coef,
      value_coef, entropy_coef, rows, dlogits, dvalues);
  C6T_LAUNCHED("ppo_loss_kernel");
  ppo_loss_reduce_kernel<<<1, 256, 0, st>>>(rows, B, value_coef, entropy_coef, stats);
  C6T_LAUNCHED("ppo_loss_reduce_kernel");
  return C6_OK;
}

int c6_clip_adamw_step(int32_t device, int32_t ntensors, const int64_t* sizes, float* const* params, float* const* grads,
                       float* const* exp_avg, float* const* exp_avg_sq, float lr, float beta1, float beta2, float eps,
                       float weight_decay, float max_grad_norm, int64_t step, float* step_device, float* grad_norm,
                       void* workspace, int64_t workspace_bytes, void* stream) {
  if (ntensors < 1 || ntensors > kOptMaxTensors) return tfail(C6_ERR_ARG, "between 1 and 48 parameter tensors per call");
  if (!sizes || !params || !grads || !exp_avg || !exp_avg_sq || !grad_norm || !workspace) return tfail(C6_ERR_ARG, "null pointer");
  if (!step_device && step < 1) return tfail(C6_ERR_ARG, "step counts from 1");
  constexpr int kBlocks = 148;
  if (workspace_bytes < (int64_t)(kBlocks * sizeof(float))) return tfail(C6_ERR_ARG, "workspace smaller than 592 bytes");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev)
    return tfail(C6_ERR_CUDA, "no such CUDA device (this operator has no CPU path)");
  C6T_CUDA(cudaSetDevice(device));
  OptTensors T{};
  T.n = ntensors;
  long long off = 0;
  for (int i = 0; i < ntensors; ++i) {
    if (sizes[i] < 0 || (sizes[i] > 0 && (!params[i] || !grads[i] || !exp_avg[i] || !exp_avg_sq[i]))) return tfail(C6_ERR_ARG, "null tensor pointer");
    T.p[i] = params[i]; T.g[i] = grads[i]; T.m[i] = exp_avg[i]; T.v[i] = exp_avg_sq[i];
    T.offset[i] = off;
    off += sizes[i];
  }
  T.offset[ntensors] = off;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* partial = reinterpret_cast<float*>(workspace);
  grad_sumsq_kernel<<<kBlocks, kOptThreads, 0, st>>>(T, partial, step_device);
  C6T_LAUNCHED("grad_sumsq_kernel");
  const double tt = (double)std::max<int64_t>(step, 1);
  const double b1t = 1.0 - std::pow((double)beta1, tt), b2t = 1.0 - std::pow((double)beta2, tt);
  const int blocks = (int)std::min<long long>((off + kOptThreads - 1) / kOptThreads, 4 * kBlocks);
  clip_adamw_kernel<<<std::max(blocks, 1), kOptThreads, 0, st>>>(T, partial, kBlocks, lr, beta1, beta2, eps, weight_decay, max_grad_norm,
                                                              (float)b1t, (float)std::sqrt(b2t), step_device, grad_norm);
  C6T_LAUNCHED("clip_adamw_kernel");
  return C6_OK;
}

}  // extern "C"
