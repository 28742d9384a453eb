// fp32 mode: the backbone on CUDA cores with fp32 operands and accumulation, NCHW activations.
// This is the engine's reference-exact arithmetic mode (tolerance 1e-3 against the reference's
// fp32 forward); it is selected explicitly with C6_PREC_FP32 and is never a fallback for the
// tensor-core mode.  Follows connect6/model.py:104-110.
#pragma once

#include "c6_common.cuh"

namespace c6 {

constexpr int kFp32Threads = 128;
constexpr int kFp32CoT = 8;       // output channels per CTA
constexpr int kFp32MaxCells = 8;  // cells per thread -> boards up to 32 x 32

// One CTA: one board, kFp32CoT output channels, all cells.  Input channels are staged through
// shared memory `cit` at a time together with the matching weight slice.
__global__ void __launch_bounds__(kFp32Threads) conv_fp32_kernel(
    const float* __restrict__ in, const float* __restrict__ w, const float* __restrict__ bias,
    float* __restrict__ out, int cin, int cout, int kside, int n, int nb, int cit) {
  extern __shared__ __align__(16) float smem_f[];
  const int pad = kside >> 1, np = n + 2 * pad, taps = kside * kside, cells = n * n;
  float* s_in = smem_f;                                            // [cit][np*np]
  float* s_w = smem_f + (((size_t)cit * np * np + 3) & ~(size_t)3);  // [cit][taps][kFp32CoT], 16-byte aligned

  const int board = blockIdx.x;
  const int g = board / nb;
  const int co0 = blockIdx.y * kFp32CoT;
  const float* wg = w + (size_t)g * cout * cin * taps;
  const float* inb = in + (size_t)board * cin * cells;

  int cell_r[kFp32MaxCells], cell_c[kFp32MaxCells];
  float acc[kFp32MaxCells][kFp32CoT];
#pragma unroll
  for (int j = 0; j < kFp32MaxCells; ++j) {
    const int cell = threadIdx.x + j * kFp32Threads;
    cell_r[j] = cell < cells ? cell / n : -1;
    cell_c[j] = cell < cells ? cell % n : 0;
#pragma unroll
    for (int o = 0; o < kFp32CoT; ++o) acc[j][o] = 0.f;
  }
  const int ncell_iter = (cells + kFp32Threads - 1) / kFp32Threads;

  for (int c0 = 0; c0 < cin; c0 += cit) {
    const int cn = min(cit, cin - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < cn * np * np; i += kFp32Threads) {
      const int ci = i / (np * np), rem = i - ci * np * np;
      const int r = rem / np - pad, c = rem % np - pad;
      s_in[i] = (r >= 0 && r < n && c >= 0 && c < n) ? inb[(size_t)(c0 + ci) * cells + r * n + c] : 0.f;
    }
    for (int i = threadIdx.x; i < cn * taps * kFp32CoT; i += kFp32Threads) {
      const int o = i % kFp32CoT, rem = i / kFp32CoT;
      const int tap = rem % taps, ci = rem / taps;
      const int co = co0 + o;
      s_w[i] = co < cout ? wg[((size_t)co * cin + c0 + ci) * taps + tap] : 0.f;
    }
    __syncthreads();
    for (int ci = 0; ci < cn; ++ci) {
      const float* sin_c = s_in + (size_t)ci * np * np;
      const float* sw_c = s_w + (size_t)ci * taps * kFp32CoT;
      for (int ky = 0; ky < kside; ++ky) {
        for (int kx = 0; kx < kside; ++kx) {
          const float4 w0 = *reinterpret_cast<const float4*>(sw_c + (ky * kside + kx) * kFp32CoT);
          const float4 w1 = *reinterpret_cast<const float4*>(sw_c + (ky * kside + kx) * kFp32CoT + 4);
#pragma unroll
          for (int j = 0; j < kFp32MaxCells; ++j) {
            if (j < ncell_iter && cell_r[j] >= 0) {
              const float xv = sin_c[(cell_r[j] + ky) * np + cell_c[j] + kx];
              acc[j][0] = fmaf(xv, w0.x, acc[j][0]);
              acc[j][1] = fmaf(xv, w0.y, acc[j][1]);
              acc[j][2] = fmaf(xv, w0.z, acc[j][2]);
              acc[j][3] = fmaf(xv, w0.w, acc[j][3]);
              acc[j][4] = fmaf(xv, w1.x, acc[j][4]);
              acc[j][5] = fmaf(xv, w1.y, acc[j][5]);
              acc[j][6] = fmaf(xv, w1.z, acc[j][6]);
              acc[j][7] = fmaf(xv, w1.w, acc[j][7]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kFp32MaxCells; ++j) {
    if (cell_r[j] < 0) continue;
    const int cell = cell_r[j] * n + cell_c[j];
#pragma unroll
    for (int o = 0; o < kFp32CoT; ++o) {
      const int co = co0 + o;
      if (co < cout) {
        const float x = acc[j][o] + (bias ? bias[(size_t)g * cout + co] : 0.f);
        out[((size_t)board * cout + co) * cells + cell] = silu_exact(x);
      }
    }
  }
}

// 1x1 policy and value maps from the last activation (connect6/model.py:108-109), biases added
// later by the finishing kernel.  One CTA per board.
__global__ void __launch_bounds__(kFp32Threads) head_fp32_kernel(
    const float* __restrict__ f, const float* __restrict__ wp, const float* __restrict__ wv,
    float* __restrict__ logit_raw, float* __restrict__ vmap, int c, int n, int nb) {
  const int board = blockIdx.x, g = board / nb, cells = n * n;
  const float* fb = f + (size_t)board * c * cells;
  for (int cell = threadIdx.x; cell < cells; cell += kFp32Threads) {
    float pol = 0.f, val = 0.f;
    for (int ch = 0; ch < c; ++ch) {
      const float v = fb[(size_t)ch * cells + cell];
      pol = fmaf(v, wp[(size_t)g * c + ch], pol);
      val = fmaf(v, wv[(size_t)g * c + ch], val);
    }
    logit_raw[(size_t)board * cells + cell] = pol;
    vmap[(size_t)board * cells + cell] = val;
  }
}

}  // namespace c6
