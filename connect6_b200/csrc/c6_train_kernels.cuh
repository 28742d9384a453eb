// Memory-bound helpers of the training-side operators: NCHW fp32 tensors <-> the forward kernels'
// channel-chunk planes, the flipped / transposed filter of the input-gradient convolution, and the bias
// gradient (column sums of the gradient planes).
#pragma once

#include "c6_common.cuh"

namespace c6 {

// x [B, C, n, n] fp32 -> bf16 planes [C_p/8][plane_rows] of 16-byte rows (8 channels of one position), position
// (b, r, c) at row front + b*slots + r*wp + c.  EVERY slot of every board image is written: cells get their
// values, pad slots and channels beyond C get zeros, so the planes need no clearing between calls.
// Grid: ceil(B*slots*(C_p/8) / 256); one thread per (board, plane, slot).
__global__ void pack_nchw_planes_kernel(const float* __restrict__ x, uint4* __restrict__ planes, long long plane_rows,
                                        int front, int slots, int wp, int n, int C, int C_p, long long B) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int nq = C_p / 8;
  if (idx >= B * slots * nq) return;
  const int slot = (int)(idx % slots);
  const int q = (int)((idx / slots) % nq);
  const long long b = idx / ((long long)slots * nq);
  const int r = slot / wp, c = slot - r * wp;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int ch = q * 8 + e;
    v[e] = (r < n && c < n && ch < C) ? x[((b * C + ch) * n + r) * n + c] : 0.f;
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  planes[(size_t)q * plane_rows + front + b * slots + slot] = o;
}

// bf16 planes -> fp32 [B, C, n, n] (cells only).  One thread per (board, plane, cell): one 16-byte row in,
// eight floats out, each store coalesced across the threads of consecutive cells.
__global__ void unpack_planes_nchw_kernel(const uint4* __restrict__ planes, long long plane_rows, int front, int slots,
                                          int wp, int n, int C, long long B, float* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = n * n, nq = (C + 7) / 8;
  if (idx >= B * nq * cells) return;
  const int cell = (int)(idx % cells);
  const int q = (int)((idx / cells) % nq);
  const long long b = idx / ((long long)cells * nq);
  const int r = cell / n, c = cell - r * n;
  const uint4 v = planes[(size_t)q * plane_rows + front + b * slots + r * wp + c];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float* o = out + ((b * C + q * 8) * cells + cell);
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (q * 8 + e < C) o[(size_t)e * cells] = __uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
}

// Filter of the input-gradient convolution in the k x k kernel's weight layout: dX = conv(dPre, W') with
// W'[ci][co][ky][kx] = W[co][ci][k-1-ky][k-1-kx] (W is the layer's [Cout, Cin, k, k] filter), i.e. a layer with
// Cout input channels and Cin output channels.  Rows [q][tap][j][ci] of 8 bf16 (element e: input channel
// (2q+j)*8+e of the gradient = an output channel of the layer); halves = 2 splits the rows for CTA pairs as
// [half][q][tap][j][ci % (cin_p/2)].
__device__ __forceinline__ void pack_dgrad_weights_row(long long idx, const float* __restrict__ w, uint4* __restrict__ out,
                                                       int cout, int cin, int kside, int cout_p, int cin_p, int halves) {
  const int taps = kside * kside, nh = cin_p / halves;
  const long long total = (long long)(cout_p / 16) * taps * 2 * cin_p;
  if (idx >= total) return;
  const int col = (int)(idx % nh);
  long long r = idx / nh;
  const int j = (int)(r % 2);
  r /= 2;
  const int tap = (int)(r % taps);
  r /= taps;
  const int q = (int)(r % (cout_p / 16));
  const int half = (int)(r / (cout_p / 16));
  const int ci = half * nh + col;              // output channel of this convolution = input channel of the layer
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int co = (2 * q + j) * 8 + e;        // its input channel = output channel of the layer
    v[e] = (co < cout && ci < cin) ? w[((size_t)co * cin + ci) * taps + (taps - 1 - tap)] : 0.f;
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]);
  o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]);
  o.w = pack_bf16x2(v[6], v[7]);
  out[idx] = o;
}
__global__ void pack_dgrad_weights_kernel(const float* __restrict__ w, uint4* __restrict__ out, int cout, int cin,
                                          int kside, int cout_p, int cin_p, int halves) {
  pack_dgrad_weights_row((long long)blockIdx.x * blockDim.x + threadIdx.x, w, out, cout, cin, kside, cout_p, cin_p, halves);
}

// Gradient planes from the layers' padded board geometry (pitch wp, `slots` per image, first row `front`) into the
// direct stem's input geometry (pitch dst_wi, dst_slots per image, first row 0): cells only -- the destination's
// padding is zero from the start and never written.  One thread per (board, 8-channel plane, cell).
__global__ void repack_planes_geometry_kernel(const uint4* __restrict__ src, long long src_plane_rows, int src_front,
                                              int src_slots, int src_wp, uint4* __restrict__ dst, long long dst_plane_rows,
                                              int dst_slots, int dst_wi, int n, int nq, long long B) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = n * n;
  if (idx >= B * nq * cells) return;
  const int cell = (int)(idx % cells);
  const int q = (int)((idx / cells) % nq);
  const long long b = idx / ((long long)cells * nq);
  const int r = cell / n, c = cell - r * n;
  dst[(size_t)q * dst_plane_rows + b * dst_slots + r * dst_wi + c] =
      src[(size_t)q * src_plane_rows + src_front + b * src_slots + r * src_wp + c];
}

// The two 1 x 1 heads (connect6/model.py:70-75,108-110) on feature planes.  One block per board:
//   logits[b][cell] = sum_ch wp[ch] f[b][ch][cell] + bp,   value[b] = tanh(mean_cell(sum_ch wv[ch] f[b][ch][cell]) + bv).
constexpr int kHeadThreads = 128;
__global__ void __launch_bounds__(kHeadThreads) heads_forward_kernel(const uint4* __restrict__ planes, long long plane_rows, int front,
                                                                     int slots, int wp_pitch, int n, int C, int nq,
                                                                     const float* __restrict__ wp, const float* __restrict__ bp,
                                                                     const float* __restrict__ wv, const float* __restrict__ bv,
                                                                     float* __restrict__ logits, float* __restrict__ value) {
  __shared__ float s_wp[128], s_wv[128], s_red[kHeadThreads / 32];
  for (int i = threadIdx.x; i < nq * 8; i += kHeadThreads) {
    s_wp[i] = i < C ? wp[i] : 0.f;
    s_wv[i] = i < C ? wv[i] : 0.f;
  }
  __syncthreads();
  const long long b = blockIdx.x;
  const int cells = n * n;
  const float pb = bp[0];
  float vsum = 0.f;
  for (int cell = threadIdx.x; cell < cells; cell += kHeadThreads) {
    const int r = cell / n, c = cell - r * n;
    const uint4* row = planes + front + b * slots + r * wp_pitch + c;
    float pol = pb;
    for (int q = 0; q < nq; ++q) {
      const uint4 v = row[(size_t)q * plane_rows];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float f = __uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
        pol = fmaf(f, s_wp[q * 8 + e], pol);
        vsum = fmaf(f, s_wv[q * 8 + e], vsum);
      }
    }
    logits[b * cells + cell] = pol;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) vsum += __shfl_xor_sync(0xffffffffu, vsum, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = vsum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < kHeadThreads / 32; ++i) s += s_red[i];
    value[b] = tanhf(s / (float)cells + bv[0]);
  }
}

// Backward of the heads.  Given dL/dlogits [B][cells], dL/dvalue [B] and the forward's value [B]:
//   du_b = dvalue_b (1 - value_b^2)                (gradient at the pre-tanh mean)
//   dfeat[b][ch][cell] = dlogits[b][cell] wp[ch] + du_b wv[ch] / cells;  grad = dfeat * der (the last layer's saved
//   silu') = the gradient at the last convolution's output                        -> 16-bit gradient planes (cells only)
//   dwp[ch] = sum_{b,cell} dlogits f,   dwv[ch] = sum_b du_b / cells sum_cell f,   dbp = sum dlogits,   dbv = sum_b du_b
// Block i walks boards i, i + gridDim.x, ... once per 8-channel plane and leaves its partial sums in
// partial[i][nq*16 + 2] (per plane: 8 dwp, 8 dwv; then dbp, dbv); heads_backward_finish_kernel adds the blocks in order.
__global__ void __launch_bounds__(kHeadThreads) heads_backward_kernel(const uint4* __restrict__ planes, const uint4* __restrict__ der,
                                                                      uint4* __restrict__ grad,
                                                                      long long plane_rows, int front, int slots, int wp_pitch, int n,
                                                                      int C, int nq, long long B, const float* __restrict__ wp,
                                                                      const float* __restrict__ wv, const float* __restrict__ dlogits,
                                                                      const float* __restrict__ dvalue, const float* __restrict__ value,
                                                                      float* __restrict__ partial) {
  __shared__ float s_red[kHeadThreads / 32][18];
  const int cells = n * n, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_cells = 1.f / (float)cells;
  float* my_partial = partial + (size_t)blockIdx.x * (nq * 16 + 2);
  for (int q = 0; q < nq; ++q) {
    float wpq[8], wvq[8], acc[18];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      wpq[e] = q * 8 + e < C ? wp[q * 8 + e] : 0.f;
      wvq[e] = q * 8 + e < C ? wv[q * 8 + e] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 18; ++e) acc[e] = 0.f;
    for (long long b = blockIdx.x; b < B; b += gridDim.x) {
      const float v = value[b];
      const float du = dvalue[b] * (1.f - v * v);
      const float dus = du * inv_cells;
      if (threadIdx.x == 0) acc[17] += du;
      for (int cell = threadIdx.x; cell < cells; cell += kHeadThreads) {
        const int r = cell / n, c = cell - r * n;
        const size_t row = (size_t)q * plane_rows + front + b * slots + r * wp_pitch + c;
        const float dl = dlogits[b * cells + cell];
        acc[16] += dl;
        const uint4 fv = planes[row], dv = der[row];
        const uint32_t w[4] = {fv.x, fv.y, fv.z, fv.w}, wd[4] = {dv.x, dv.y, dv.z, dv.w};
        float g[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float f = __uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
          const float d = __uint_as_float((e & 1) ? (wd[e >> 1] & 0xffff0000u) : (wd[e >> 1] << 16));
          acc[e] = fmaf(dl, f, acc[e]);
          acc[8 + e] = fmaf(dus, f, acc[8 + e]);
          g[e] = fmaf(dl, wpq[e], dus * wvq[e]) * d;    // times the last layer's saved silu': dL/d(its convolution output)
        }
        uint4 o;
        o.x = pack_bf16x2(g[0], g[1]);
        o.y = pack_bf16x2(g[2], g[3]);
        o.z = pack_bf16x2(g[4], g[5]);
        o.w = pack_bf16x2(g[6], g[7]);
        grad[row] = o;
      }
    }
#pragma unroll
    for (int e = 0; e < 18; ++e) {
      float s = acc[e];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) s_red[warp][e] = s;
    }
    __syncthreads();
    if (threadIdx.x < 18) {
      float s = 0.f;
      for (int i = 0; i < kHeadThreads / 32; ++i) s += s_red[i][threadIdx.x];
      if (threadIdx.x < 16) my_partial[q * 16 + threadIdx.x] = s;
      else if (q == 0) my_partial[nq * 16 + (threadIdx.x - 16)] = s;
    }
    __syncthreads();
  }
}
__global__ void heads_backward_finish_kernel(const float* __restrict__ partial, int nblocks, int nq, int C, float* __restrict__ dwp,
                                             float* __restrict__ dbp, float* __restrict__ dwv, float* __restrict__ dbv) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;    // 0..2C+1
  if (i >= 2 * C + 2) return;
  const int stride = nq * 16 + 2;
  int col;
  float* dst;
  if (i < C) { col = (i >> 3) * 16 + (i & 7); dst = dwp + i; }
  else if (i < 2 * C) { const int ch = i - C; col = (ch >> 3) * 16 + 8 + (ch & 7); dst = dwv + ch; }
  else if (i == 2 * C) { col = nq * 16; dst = dbp; }
  else { col = nq * 16 + 1; dst = dbv; }
  // four interleaved running sums in a fixed association, so that four loads are in flight
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int b = 0;
  for (; b + 4 <= nblocks; b += 4) {
    a0 += partial[(size_t)b * stride + col];
    a1 += partial[(size_t)(b + 1) * stride + col];
    a2 += partial[(size_t)(b + 2) * stride + col];
    a3 += partial[(size_t)(b + 3) * stride + col];
  }
  for (; b < nblocks; ++b) a0 += partial[(size_t)b * stride + col];
  *dst = (a0 + a1) + (a2 + a3);
}

// PPO minibatch loss and its gradient at the network outputs (connect6/train.py:1047-1086):
//   z = mask(logits) / T,  logp = z - logsumexp(z),  H = -sum p logp,  ratio = exp(logp[a] - old_logprob),
//   policy = max(-adv ratio, -adv clamp(ratio, 1 - c, 1 + c)),  value = 0.5 (v - ret)^2,
//   loss = mean(policy) + value_coef mean(value) - entropy_coef mean(H).
// One warp per board.  rows[b] = {policy, value, H, (ratio - 1) - logratio, |ratio - 1| > c}; dlogits[b][j] = dloss/dlogits
// (zero at illegal actions: masked_fill passes no gradient), dvalues[b] = dloss/dv.  A board without a legal action has
// the uniform distribution the reference's fill value gives it, and no gradient.
constexpr int kPpoWarps = 4;
__global__ void __launch_bounds__(32 * kPpoWarps) ppo_loss_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ legal,
                                                                  const long long* __restrict__ actions,
                                                                  const float* __restrict__ old_logprob,
                                                                  const float* __restrict__ advantages,
                                                                  const float* __restrict__ returns, const float* __restrict__ values,
                                                                  long long B, int A, float inv_t, float clip, float value_coef,
                                                                  float entropy_coef, float* __restrict__ rows,
                                                                  float* __restrict__ dlogits, float* __restrict__ dvalues) {
  const long long b = (long long)blockIdx.x * kPpoWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const float* lg = logits + b * A;
  const uint8_t* lm = legal + b * A;
  float m = -INFINITY;
  int nlegal = 0;
  for (int j = lane; j < A; j += 32)
    if (lm[j]) { m = fmaxf(m, lg[j] * inv_t); ++nlegal; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    nlegal += __shfl_xor_sync(0xffffffffu, nlegal, o);
  }
  const bool none = nlegal == 0;
  float s = 0.f, t = 0.f;
  if (!none)
    for (int j = lane; j < A; j += 32)
      if (lm[j]) {
        const float z = lg[j] * inv_t, e = expf(z - m);
        s += e;
        t = fmaf(e, z, t);
      }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  const float lse = none ? 0.f : m + logf(s);
  const float H = none ? logf((float)A) : lse - t / s;
  const int a = (int)actions[b];
  const float logp_a = none ? -logf((float)A) : ((a >= 0 && a < A && lm[a]) ? lg[a] * inv_t - lse : -INFINITY);
  const float logratio = logp_a - old_logprob[b];
  const float ratio = expf(logratio);
  const float adv = advantages[b];
  const float pg1 = -adv * ratio, pg2 = -adv * fminf(fmaxf(ratio, 1.f - clip), 1.f + clip);
  const bool inside = ratio >= 1.f - clip && ratio <= 1.f + clip;
  const float inv_b = 1.f / (float)B;
  const float g = (inside || pg1 > pg2) ? -adv * ratio * inv_b : 0.f;      // dloss / dlogp[a]
  const float ce = entropy_coef * inv_b;
  const float v = values[b], ret = returns[b];
  if (lane == 0) {
    float* r = rows + b * 5;
    r[0] = fmaxf(pg1, pg2);
    r[1] = 0.5f * (v - ret) * (v - ret);
    r[2] = H;
    r[3] = (ratio - 1.f) - logratio;
    r[4] = fabsf(ratio - 1.f) > clip ? 1.f : 0.f;
    dvalues[b] = value_coef * (v - ret) * inv_b;
  }
  float* dl = dlogits + b * A;
  for (int j = lane; j < A; j += 32) {
    float d = 0.f;
    if (!none && lm[j]) {
      const float logp = lg[j] * inv_t - lse, p = expf(logp);
      d = (g * ((j == a ? 1.f : 0.f) - p) + ce * p * (logp + H)) * inv_t;
    }
    dl[j] = d;
  }
}
// stats = {loss, mean policy, mean value, mean H, approx_kl, clipfrac}: column sums of rows in a fixed order
__global__ void __launch_bounds__(256) ppo_loss_reduce_kernel(const float* __restrict__ rows, long long B, float value_coef,
                                                              float entropy_coef, float* __restrict__ stats) {
  __shared__ float s_part[5][256];
  float acc[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long b = threadIdx.x; b < B; b += 256)
#pragma unroll
    for (int c = 0; c < 5; ++c) acc[c] += rows[b * 5 + c];
#pragma unroll
  for (int c = 0; c < 5; ++c) s_part[c][threadIdx.x] = acc[c];
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w)
#pragma unroll
      for (int c = 0; c < 5; ++c) s_part[c][threadIdx.x] += s_part[c][threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float inv_b = 1.f / (float)B;
    const float pol = s_part[0][0] * inv_b, val = s_part[1][0] * inv_b, ent = s_part[2][0] * inv_b;
    stats[0] = pol + value_coef * val - entropy_coef * ent;
    stats[1] = pol;
    stats[2] = val;
    stats[3] = ent;
    stats[4] = s_part[3][0] * inv_b;
    stats[5] = s_part[4][0] * inv_b;
  }
}

// out = a * b element by element over `rows` 16-byte rows of 8 bf16 (gradient planes times saved silu' planes).
__global__ void mul_planes_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out, long long rows) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = a[i], y = b[i];
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      o[k] = pack_bf16x2(__uint_as_float(xs[k] << 16) * __uint_as_float(ys[k] << 16),
                         __uint_as_float(xs[k] & 0xffff0000u) * __uint_as_float(ys[k] & 0xffff0000u));
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Gradient clipping by global norm + AdamW for a whole parameter list in two launches (connect6/train.py:1121-1145:
// nn.utils.clip_grad_norm_(model.parameters(), max_grad_norm) then torch.optim.AdamW.step()).
//   total = sqrt(sum over all tensors of g^2);  coef = min(1, max_norm / (total + 1e-6));  g <- g * coef  (written back)
//   p <- p (1 - lr wd);  m <- b1 m + (1 - b1) g;  v <- b2 v + (1 - b2) g^2;
//   p <- p - (lr / (1 - b1^t)) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)
// The tensors are addressed as one flat index space (offset[i] = first flat index of tensor i).  Kernel 1 leaves one
// partial sum of squares per block; every block of kernel 2 adds them up in block order (the same value everywhere,
// the same on every run).  A non-finite norm (overflowed or NaN gradients) leaves parameters and moments untouched;
// the norm is reported either way.  With step_device the 1-based update count is kept on the device (kernel 1 adds one,
// kernel 2 derives the bias corrections from it), so that a captured graph can be replayed.
constexpr int kOptMaxTensors = 48;
constexpr int kOptThreads = 256;
struct OptTensors {
  float* p[kOptMaxTensors];
  float* g[kOptMaxTensors];
  float* m[kOptMaxTensors];
  float* v[kOptMaxTensors];
  long long offset[kOptMaxTensors + 1];
  int n;
};
__device__ __forceinline__ int opt_find(const OptTensors& T, long long i) {
  int t = 0;
  while (t + 1 < T.n && i >= T.offset[t + 1]) ++t;
  return t;
}
__global__ void __launch_bounds__(kOptThreads) grad_sumsq_kernel(const OptTensors T, float* __restrict__ partial,
                                                                 float* __restrict__ step_device) {
  __shared__ float s_red[kOptThreads / 32];
  if (step_device != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *step_device += 1.f;   // the update kernel reads the new count
  const long long total = T.offset[T.n];
  const long long per_block = (total + gridDim.x - 1) / gridDim.x;
  const long long lo = per_block * blockIdx.x, hi = min(total, lo + per_block);
  float acc = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += kOptThreads) {
    const int t = opt_find(T, i);
    const float g = T.g[t][i - T.offset[t]];
    acc = fmaf(g, g, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < kOptThreads / 32; ++w) s += s_red[w];
    partial[blockIdx.x] = s;
  }
}
__global__ void __launch_bounds__(kOptThreads) clip_adamw_kernel(const OptTensors T, const float* __restrict__ partial, int npartial,
                                                                 float lr, float beta1, float beta2, float eps, float weight_decay,
                                                                 float max_norm, float bias1, float bias2_sqrt,
                                                                 const float* __restrict__ step_device,
                                                                 float* __restrict__ grad_norm) {
  if (step_device != nullptr) {        // the update count lives on the device (CUDA-graph replays): bias corrections from it
    const float t = *step_device;
    bias1 = 1.f - powf(beta1, t);
    bias2_sqrt = sqrtf(1.f - powf(beta2, t));
  }
  float sumsq = 0.f;
  for (int b = 0; b < npartial; ++b) sumsq += partial[b];
  const float norm = sqrtf(sumsq);
  if (blockIdx.x == 0 && threadIdx.x == 0) *grad_norm = norm;
  if (!(norm <= 3.0e38f)) return;                      // inf or NaN: no step
  const float coef = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  const float step_size = lr / bias1;
  const long long total = T.offset[T.n];
  for (long long i = (long long)blockIdx.x * kOptThreads + threadIdx.x; i < total; i += (long long)gridDim.x * kOptThreads) {
    const int t = opt_find(T, i);
    const long long k = i - T.offset[t];
    const float g = T.g[t][k] * coef;
    float p = T.p[t][k] * (1.f - lr * weight_decay);
    const float m = beta1 * T.m[t][k] + (1.f - beta1) * g;
    const float v = beta2 * T.v[t][k] + (1.f - beta2) * g * g;
    p -= step_size * (m / (sqrtf(v) / bias2_sqrt + eps));
    T.g[t][k] = g;
    T.m[t][k] = m;
    T.v[t][k] = v;
    T.p[t][k] = p;
  }
}

// Every operand a stack of 3 x 3 layers needs from its parameters, in ONE launch: grid (row blocks, layer, what) with
// what = 0 forward filter, 1 the same for CTA pairs, 2 flipped/transposed filter of the data gradient, 3 the same for
// CTA pairs, 4 bias padded to the kernels' channel granule.
struct StackPackParams {
  struct Layer {
    const float* w;
    const float* bias;     // nullable: zeros
    uint4 *wf, *wf_pair, *wd, *wd_pair;
    float* bias_f;
    int cout, cin, cout_p, cin_p;
  } layer[C6_MAX_LAYERS];
};
__global__ void pack_stack_weights_kernel(const StackPackParams p) {
  const StackPackParams::Layer& L = p.layer[blockIdx.y];
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  switch (blockIdx.z) {
    case 0: pack_conv_weights_row(idx, L.w, L.wf, L.cout, L.cin, 3, L.cout_p, L.cin_p, 0); break;
    case 1: pack_conv_weights_pair_row(idx, L.w, L.wf_pair, L.cout, L.cin, 3, L.cout_p, L.cin_p, 0); break;
    case 2: pack_dgrad_weights_row(idx, L.w, L.wd, L.cout, L.cin, 3, L.cout_p, L.cin_p, 1); break;
    case 3: pack_dgrad_weights_row(idx, L.w, L.wd_pair, L.cout, L.cin, 3, L.cout_p, L.cin_p, 2); break;
    default:
      if (idx < L.cout_p) L.bias_f[idx] = (L.bias != nullptr && idx < L.cout) ? L.bias[idx] : 0.f;
  }
}

// Bias gradient, first pass: block (q, s) sums the rows [s*chunk, (s+1)*chunk) of plane q for its 8 channels
// (fp32) into partial[q][s][8].  Pad slots are zero, so every row may be summed.
constexpr int kColsumThreads = 256;
__global__ void __launch_bounds__(kColsumThreads) colsum_planes_kernel(const uint4* __restrict__ planes, long long plane_rows,
                                                                       long long row0, long long nrows, int nslices,
                                                                       float* __restrict__ partial) {
  const int q = blockIdx.x, s = blockIdx.y;
  const long long chunk = (nrows + nslices - 1) / nslices;
  const long long lo = row0 + s * chunk, hi = min(row0 + nrows, lo + chunk);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long r = lo + threadIdx.x; r < hi; r += kColsumThreads) {
    const uint4 v = planes[(size_t)q * plane_rows + r];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc[2 * k] += __uint_as_float(w[k] << 16);
      acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
    }
  }
  __shared__ float red[kColsumThreads / 32][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float v = acc[e];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5][e] = v;
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    float v = 0.f;
    for (int wv = 0; wv < kColsumThreads / 32; ++wv) v += red[wv][threadIdx.x];
    partial[((size_t)q * nslices + s) * 8 + threadIdx.x] = v;
  }
}

// second pass: db[ch] = sum over slices, in slice order
__global__ void colsum_finish_kernel(const float* __restrict__ partial, int nslices, int C, float* __restrict__ db) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= C) return;
  float v = 0.f;
  for (int s = 0; s < nslices; ++s) v += partial[((size_t)(ch >> 3) * nslices + s) * 8 + (ch & 7)];
  db[ch] = v;
}

}  // namespace c6
