// Memory-bound helper kernels around the convolution stack: input packing (with the per-board
// D4 view), weight repacking, the fused policy/value finishing kernel (mask, log-softmax,
// categorical draw, board mean + tanh) and the small standalone operators of the path.
#pragma once

#include "c6_common.cuh"
#include "c6_tc.cuh"

namespace c6 {

// ------------------------------------------------------------------------------------------------
// K order of the stem GEMM.  Chunks of 8: [planes 0 and 1: k = ci*cells + cell; then two slots that
// carry the third plane's "level"; zero padded to kc_short chunks][plane 2: cell, zero padded].
// The third plane of a real position is constant over the board (connect6/vector_env.py:212-216).
// Every board's third plane is split into a level c (its first cell) and a residual x2 - c: the
// level rides in the two extra K slots against the row sums of the plane-2 Toeplitz block (split
// into a bf16 high and low part), the residual in the plane-2 chunks.  When every residual of a pass
// is zero -- always, for real positions -- the GEMM stops after the first kc_short chunks.
// ------------------------------------------------------------------------------------------------
// kind: 0 = zero padding, 1 = input element (ci, cell), 2 = level slot (cell = 0: high part, 1: low part)
__host__ __device__ __forceinline__ int stem_k_decode(int chunk, int e, int kc_short, int cells, int& ci, int& cell) {
  if (chunk < kc_short) {
    const int k = chunk * 8 + e;
    if (k < 2 * cells) {
      ci = k >= cells ? 1 : 0;
      cell = k - ci * cells;
      return 1;
    }
    ci = 2;
    cell = k - 2 * cells;
    return k < 2 * cells + 2 ? 2 : 0;
  }
  cell = (chunk - kc_short) * 8 + e;
  ci = 2;
  return cell < cells ? 1 : 0;
}

// ------------------------------------------------------------------------------------------------
// Input packing for the tensor-core stem: x [boards,3,n,n] (fp32 or bf16, NCHW) -> 16-byte rows of
// 8 bf16 laid out [board tile of 128][K chunk][128 boards], so that all K chunks of one pipeline
// stage of one board tile are contiguous and travel in ONE bulk copy.  A board with orientation
// `phase` is presented as view.flat[j] = x.flat[d4_inverse(j)] (connect6/train.py:222-230).
// Stores `epoch` into *p2_epoch when some board's third plane is not constant, and one byte of
// occupancy bits per (board, chunk of planes 0/1).
// Grid: (ceil(kc*nb/256), G); one thread per (board, chunk).
// ------------------------------------------------------------------------------------------------
__global__ void pack_stem_input_kernel(const InputSrc in,
                                       const uint8_t* __restrict__ orient, uint4* __restrict__ xk,
                                       long long mrows, int mrows_per_group, int kc, int kc_short, int n,
                                       int nb,                 // boards of this pass per group
                                       long long group_stride, // boards between groups in x
                                       long long board0,       // first board of this pass in a group
                                       unsigned int epoch, unsigned int* __restrict__ p2_epoch,
                                       uint8_t* __restrict__ occ,     // [kc_short][mrows] bit j of a byte: element 8c+j != 0
                                       int f16,                       // operand type of the engine: 0 bf16, 1 fp16
                                       int* __restrict__ status) {
  grid_dep_launch();
  const int g = blockIdx.y;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)kc * nb) return;
  const int t = (int)(idx % nb);
  const int c = (int)(idx / nb);
  const int cells = n * n;
  const long long src_board = (long long)g * group_stride + board0 + t;
  const int phase = orient ? (orient[src_board] & 7) : 0;
  if (c == 0 && in.boards != nullptr && input_env(in, src_board) < 0) atomicOr(status, kStatBadIndex);
  // level of the third plane: needed by the chunk that holds the level slots and by the plane-2 chunks
  const bool wants_level = c >= kc_short || (c + 1) * 8 > 2 * cells;
  const float level = wants_level ? input_value(in, src_board, 2, 0, cells) : 0.f;
  // all eight loads are issued before any value is used (the kernel is bound by memory latency)
  float v[8];
  int kinds[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int ci, cell;
    const int kind = stem_k_decode(c, j, kc_short, cells, ci, cell);
    float val = 0.f;
    if (kind == 1) {
      if (phase) cell = d4_inverse(cell, n, phase);
      val = input_value(in, src_board, ci, cell, cells);
    }
    v[j] = val;
    kinds[j] = kind == 1 && ci == 2 ? 3 : kind;   // 3: element of the third plane
  }
  if (c < kc_short) {
    // occupancy bits of the first two planes, in the view frame: the finishing kernel derives the
    // legal-move mask from these 2 x cells bits instead of re-reading the planes
    unsigned bits = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) bits |= (kinds[j] == 1 && v[j] != 0.f) ? (1u << j) : 0u;
    occ[(size_t)c * mrows + (size_t)g * mrows_per_group + t] = (uint8_t)bits;
  }
  bool varies = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (kinds[j] == 3) {
      v[j] -= level;
      varies |= v[j] != 0.f;
    } else if (kinds[j] == 2) {
      v[j] = level;
    }
  }
  if (varies) atomicExch(p2_epoch, epoch);
  uint4 o;
  o.x = pack_h2(v[0], v[1], f16);
  o.y = pack_h2(v[2], v[3], f16);
  o.z = pack_h2(v[4], v[5], f16);
  o.w = pack_h2(v[6], v[7], f16);
  const size_t brow = (size_t)g * mrows_per_group + t;   // board row over all groups
  xk[((brow >> 7) * kc + c) * 128 + (brow & 127)] = o;
}

// ------------------------------------------------------------------------------------------------
// Direct stem (few boards per weight set): input planes "x-expanded" for the implicit GEMM of
// conv_tc_kernel's stem mode.  Board images are zero padded to slots/wi rows of pitch wi (cells at rows
// and columns 0..n-1; the pad columns and rows of one image are the left/top padding of the next) and
// laid end to end; row R of plane ci holds the 8 consecutive linear positions R .. R+7 of that sequence,
// so the last rows of an image (and the 8 rows in front of a group's first image) already carry the first
// cells of the image behind them.  A group's threads write rows [base - 8, base + nb*slots - 8); the 8 rows
// behind a group's last image are all padding and stay zero.
// Grid: (nb, G), one block per board image: the block first stages the board's three planes (in view orientation) in
// shared memory with coalesced loads, then its threads build the image's 3 * slots rows from there.  Block t writes the
// rows [t*slots - 8, (t+1)*slots - 8) of each plane: what lies in front of its image in those rows is the tail padding
// of the image before (zero).
// ------------------------------------------------------------------------------------------------
constexpr int kPackDirectThreads = 256;
constexpr int kPackDirectMaxCells = 32 * 32;
__global__ void __launch_bounds__(kPackDirectThreads) pack_stem_direct_input_kernel(
    const InputSrc in, const uint8_t* __restrict__ orient, uint4* __restrict__ xe, long long plane_rows, int front, int group_pos,
    int wi, int slots, int n, int nb, long long group_stride, long long board0, int f16, int* __restrict__ status) {
  __shared__ float s_x[3 * kPackDirectMaxCells];
  grid_dep_launch();
  const int g = blockIdx.y, t = blockIdx.x;
  const int cells = n * n;
  const long long src_board = (long long)g * group_stride + board0 + t;
  const int phase = orient ? (orient[src_board] & 7) : 0;
  if (threadIdx.x == 0 && in.boards != nullptr && input_env(in, src_board) < 0) atomicOr(status, kStatBadIndex);
  for (int i = threadIdx.x; i < 3 * cells; i += kPackDirectThreads) {
    const int ci = i / cells, cell = i - ci * cells;
    s_x[i] = input_value(in, src_board, ci, phase ? d4_inverse(cell, n, phase) : cell, cells);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 3 * slots; i += kPackDirectThreads) {
    const int ci = i / slots, p = i - ci * slots - 8;       // row relative to this image's first position
    int q = p < 0 ? 0 : p;
    int r = q / wi, c = q - r * wi;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float val = 0.f;
      if (p + e >= 0) {
        if (r < n && c < n) val = s_x[ci * cells + r * n + c];
        if (++c == wi) { c = 0; ++r; }
      }
      v[e] = val;
    }
    uint4 o;
    o.x = pack_h2(v[0], v[1], f16);
    o.y = pack_h2(v[2], v[3], f16);
    o.z = pack_h2(v[4], v[5], f16);
    o.w = pack_h2(v[6], v[7], f16);
    xe[(size_t)ci * plane_rows + front + (long long)g * group_pos + (long long)t * slots + p] = o;
  }
}

// Filter of the first layer for the direct stem: rows [ci][ky][hb][j][co] of 8 elements, element e of the row
// being filter column kx = 16 hb + 8 j + e (zero for kx >= k0 and for co >= cout).  halves = 2 lays the
// rows out for CTA pairs: [half][ci][ky][hb][j][co % (cout_p/2)].
__global__ void pack_stem_direct_weights_kernel(const float* __restrict__ w, uint4* __restrict__ out, int cout, int kside,
                                                int cout_p, int hx, int halves, int f16) {
  const int nh = cout_p / halves;
  const long long total = 3LL * kside * hx * 2 * cout_p;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int col = (int)(idx % nh);
  long long r = idx / nh;
  const int j = (int)(r % 2);
  r /= 2;
  const int hb = (int)(r % hx);
  r /= hx;
  const int ky = (int)(r % kside);
  r /= kside;
  const int ci = (int)(r % 3);
  const int half = (int)(r / 3);
  const int co = half * nh + col;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int kx = 16 * hb + 8 * j + e;
    v[e] = (co < cout && kx < kside) ? w[(((size_t)co * 3 + ci) * kside + ky) * kside + kx] : 0.f;
  }
  uint4 o;
  o.x = pack_h2(v[0], v[1], f16);
  o.y = pack_h2(v[2], v[3], f16);
  o.z = pack_h2(v[4], v[5], f16);
  o.w = pack_h2(v[6], v[7], f16);
  out[idx] = o;
}

// fp32 mode: x -> fp32 NCHW copy in view orientation, boards of all groups laid out [g][t].
__global__ void view_input_f32_kernel(const InputSrc in,
                                      const uint8_t* __restrict__ orient, float* __restrict__ out,
                                      int n, int nb, long long group_stride, long long board0) {
  const int g = blockIdx.y;
  const int cells = n * n, ktot = 3 * cells;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)nb * ktot) return;
  const int t = (int)(idx / ktot);
  const int k = (int)(idx - (long long)t * ktot);
  const long long src_board = (long long)g * group_stride + board0 + t;
  const int phase = orient ? (orient[src_board] & 7) : 0;
  const int ci = k / cells;
  int cell = k - ci * cells;
  if (phase) cell = d4_inverse(cell, n, phase);
  out[((size_t)g * nb + t) * ktot + k] = input_value(in, src_board, ci, cell, cells);
}

// ------------------------------------------------------------------------------------------------
// Weight repacking (reference layout: [Cout,Cin,K,K] fp32, connect6/model.py:56-63).
// ------------------------------------------------------------------------------------------------

// k x k layer -> rows [q][tap][j][co] of 8 bf16: element e of the row is input channel
// (2q+j)*8+e.  Channels beyond the real counts are zero.
__device__ __forceinline__ void pack_conv_weights_row(long long idx, const float* __restrict__ w, uint4* __restrict__ out,
                                                      int cout, int cin, int kside, int cout_p, int cin_p, int f16) {
  const int taps = kside * kside;
  const long long total = (long long)(cin_p / 16) * taps * 2 * cout_p;
  if (idx >= total) return;
  const int co = (int)(idx % cout_p);
  long long r = idx / cout_p;
  const int j = (int)(r % 2);
  r /= 2;
  const int tap = (int)(r % taps);
  const int q = (int)(r / taps);
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int ci = (2 * q + j) * 8 + e;
    v[e] = (co < cout && ci < cin) ? w[((size_t)co * cin + ci) * taps + tap] : 0.f;
  }
  uint4 o;
  o.x = pack_h2(v[0], v[1], f16);
  o.y = pack_h2(v[2], v[3], f16);
  o.z = pack_h2(v[4], v[5], f16);
  o.w = pack_h2(v[6], v[7], f16);
  out[idx] = o;
}
__global__ void pack_conv_weights_kernel(const float* __restrict__ w, uint4* __restrict__ out,
                                         int cout, int cin, int kside, int cout_p, int cin_p, int f16) {
  pack_conv_weights_row((long long)blockIdx.x * blockDim.x + threadIdx.x, w, out, cout, cin, kside, cout_p, cin_p, f16);
}

// Same rows for the CTA-pair kernel: [half][q][tap][j][co % (cout_p/2)], half = co / (cout_p/2).
__device__ __forceinline__ void pack_conv_weights_pair_row(long long idx, const float* __restrict__ w, uint4* __restrict__ out,
                                                           int cout, int cin, int kside, int cout_p, int cin_p, int f16) {
  const int taps = kside * kside, nh = cout_p / 2;
  const long long total = (long long)(cin_p / 16) * taps * 2 * cout_p;
  if (idx >= total) return;
  const int col = (int)(idx % nh);
  long long r = idx / nh;
  const int j = (int)(r % 2);
  r /= 2;
  const int tap = (int)(r % taps);
  r /= taps;
  const int q = (int)(r % (cin_p / 16));
  const int half = (int)(r / (cin_p / 16));
  const int co = half * nh + col;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int ci = (2 * q + j) * 8 + e;
    v[e] = (co < cout && ci < cin) ? w[((size_t)co * cin + ci) * taps + tap] : 0.f;
  }
  uint4 o;
  o.x = pack_h2(v[0], v[1], f16);
  o.y = pack_h2(v[2], v[3], f16);
  o.z = pack_h2(v[4], v[5], f16);
  o.w = pack_h2(v[6], v[7], f16);
  out[idx] = o;
}
__global__ void pack_conv_weights_pair_kernel(const float* __restrict__ w, uint4* __restrict__ out,
                                              int cout, int cin, int kside, int cout_p, int cin_p, int f16) {
  pack_conv_weights_pair_row((long long)blockIdx.x * blockDim.x + threadIdx.x, w, out, cout, cin, kside, cout_p, cin_p, f16);
}

// Stem -> Toeplitz rows (row o = cell_out*c1 + co, element e of chunk c: see stem_k_decode) laid out
// [output tile of nt][half][K chunk][nt/halves rows]: the K chunks of one pipeline stage of one
// (tile, half) are contiguous.  halves = 2 when CTA pairs split the tile's rows, else 1.
__device__ __forceinline__ float stem_toeplitz_value(const float* __restrict__ w, int cout, int kside, int n, int co,
                                                     int cell_out, int ci, int cell_in) {
  const int pad = kside >> 1;
  const int ro = cell_out / n, cc = cell_out - ro * n;
  const int ri = cell_in / n, cin_c = cell_in - ri * n;
  const int ky = ri - ro + pad, kx = cin_c - cc + pad;
  if (co >= cout || ky < 0 || ky >= kside || kx < 0 || kx >= kside) return 0.f;
  return w[(((size_t)co * 3 + ci) * kside + ky) * kside + kx];
}

__global__ void pack_stem_toeplitz_kernel(const float* __restrict__ w, uint4* __restrict__ out,
                                          int cout, int kside, int n, int c1, int kc, int kc_short, int ntot, int nt,
                                          int halves, int f16) {
  const long long total = (long long)kc * ntot;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int o = (int)(idx % ntot);
  const int c = (int)(idx / ntot);
  const int cells = n * n;
  const int cell_out = o / c1, co = o - cell_out * c1;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int ci, cell_in;
    const int kind = cell_out < cells ? stem_k_decode(c, e, kc_short, cells, ci, cell_in) : 0;
    float val = 0.f;
    if (kind == 1) {
      val = stem_toeplitz_value(w, cout, kside, n, co, cell_out, ci, cell_in);
    } else if (kind == 2) {
      // what a third plane of constant value 1 adds to this output: the sum of its plane-2 weights as
      // the tensor cores see them (rounded to the operand type), carried as a high part in that type
      // and the remainder
      float sum = 0.f;
      for (int ck = 0; ck < cells; ++ck)
        sum += round_h(stem_toeplitz_value(w, cout, kside, n, co, cell_out, 2, ck), f16);
      const float hi = round_h(sum, f16);
      val = cell_in == 0 ? hi : sum - hi;
    }
    v[e] = val;
  }
  uint4 q;
  q.x = pack_h2(v[0], v[1], f16);
  q.y = pack_h2(v[2], v[3], f16);
  q.z = pack_h2(v[4], v[5], f16);
  q.w = pack_h2(v[6], v[7], f16);
  const int tile = o / nt, ol = o - tile * nt, nloc = nt / halves;
  const int h = ol / nloc, rr = ol - h * nloc;
  out[(((size_t)tile * halves + h) * kc + c) * nloc + rr] = q;
}

// dst[i] = i < n_src ? src[i] : 0 for i < n_dst (bias / head vectors padded with zeros)
__global__ void copy_pad_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int n_src,
                                    int n_dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_dst) dst[i] = (src != nullptr && i < n_src) ? src[i] : 0.f;
}

// ------------------------------------------------------------------------------------------------
// Finishing kernel: one CTA of 128 threads per board.
//   raw policy map + bias -> (optional D4 inverse map) -> mask -> logits out
//   masked logits / max(T,1e-4) -> log-softmax -> one inverse-CDF draw -> action, log-prob
//   value map -> board mean + bias -> tanh
// Follows connect6/model.py:108-110,123-125 and connect6/train.py:195-203.
// ------------------------------------------------------------------------------------------------
struct FinishParams {
  // sources (engine path): raw maps in a pitched layout; (standalone path): logits_in + legal_in
  const float* logit_raw;
  const float* vmap;
  long long group_stride;  // elements between groups in the raw maps
  int board_stride;        // elements between boards
  int pitch;               // elements between board rows
  const float* pol_bias;   // [G] or null
  const float* val_bias;   // [G] or null
  const float* logits_in;  // standalone: [B,A] logits
  const uint8_t* legal_in; // standalone: [B,A] legality
  InputSrc in;             // engine path: network input, for occupancy (plane0|plane1) when occ is null
  const uint8_t* occ;      // nullable [chunk][occ_stride]: occupancy bits written by the input pack kernel (view frame)
  long long occ_stride;    // board rows per chunk
  int mrows_per_group;     // board rows reserved per group
  const uint8_t* orient;
  long long x_group_stride; // boards between groups in x / outputs
  long long board0;         // first board of this pass inside a group
  int n;                    // board side (engine path); standalone: A = n_actions
  int n_magic;              // 65536 / n + 1: a / n == (a * n_magic) >> 16 for a < n * n, n <= 32
  int n_actions;
  int nb;                   // boards per group in this pass
  int flags;
  int do_sample;
  float temperature;
  unsigned long long seed, offset;
  long long board_index0;
  float* logits_out;        // [.., A] or null
  float* value_out;         // or null
  long long* action_out;    // or null
  float* logprob_out;       // or null
};

constexpr int kFinishWarps = 4;                    // boards per block: one warp each
constexpr int kFinishThreads = 32 * kFinishWarps;
constexpr int kFinishMaxActions = 1024;
constexpr int kFinishSmallJ = 12;                  // actions per lane of the small instantiation: up to 384 actions

// blocks for nb boards per group
__host__ __device__ inline unsigned finish_blocks(long long nb) {
  return (unsigned)((nb + kFinishWarps - 1) / kFinishWarps);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One warp per board; lane l owns the J consecutive actions J*l .. J*l + J-1 and keeps them in
// registers (J * 32 >= n_actions), so the running sum of the inverse-CDF draw is J additions per
// lane plus one shuffle scan over the lane totals: no shared memory, no block-wide barrier.
// The kernel is bound by memory latency, so resident warps are what counts: the small instantiation is held to
// 96 registers (5 blocks = 20 warps per SM instead of 4 = 16; no spills).
template <int J>
__global__ void __launch_bounds__(kFinishThreads, J <= kFinishSmallJ ? 5 : 1) finish_kernel(const FinishParams p) {
  grid_dep_launch();
  grid_dep_wait();   // raw logits and value maps come from the last conv kernel
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y;
  const long long t = (long long)blockIdx.x * kFinishWarps + warp;   // board inside the group
  if (t >= p.nb) return;                                           // whole warps leave together
  const int A = p.n_actions;
  const long long ob = (long long)g * p.x_group_stride + p.board0 + t;  // board index in x / outputs
  const bool engine = p.logit_raw != nullptr;
  const int n = p.n;
  const int phase = (engine && p.orient) ? (p.orient[ob] & 7) : 0;
  const bool canon = phase != 0 && (p.flags & 2 /*C6_FLAG_INVERSE_MAP*/);
  const long long raw0 = (long long)g * p.group_stride + t * p.board_stride;
  const float bp = (engine && p.pol_bias) ? p.pol_bias[g] : 0.f;
  const float inv_t = 1.0f / fmaxf(p.temperature, 1e-4f);
  const int a0 = lane * J;

  // raw logit of output index a (canonical frame when `canon`, else the view frame)
  auto raw_logit = [&](int a) {
    if (!engine) return p.logits_in[ob * A + a];
    const int view_cell = canon ? d4_forward(a, n, phase) : a;
    const int vr = (view_cell * p.n_magic) >> 16, vc = view_cell - vr * n;
    return p.logit_raw[raw0 + vr * p.pitch + vc] + bp;
  };

  // All loads are issued before any value is used: the kernel is bound by memory latency.
  float raw[J], vm[J];
  unsigned occupied = 0;   // bit j: action a0 + j is not legal
  if (engine && p.occ && phase == 0) {
    // Common case (no per-board orientation): the lane's actions are consecutive cells of one or two
    // board rows, so the row/column pair is stepped instead of divided out, and the occupancy bits
    // of its J cells sit in at most ceil((J + 7) / 8) + 1 consecutive bytes per plane.
    int r = (a0 * p.n_magic) >> 16, c = a0 - r * n;
    const uint8_t* ob_occ = p.occ + (size_t)g * p.mrows_per_group + t;
    constexpr int kBytes = (J + 14) / 8;
    unsigned long long w0 = 0, w1 = 0;
    const int k1 = A + a0;
#pragma unroll
    for (int b = 0; b < kBytes; ++b) {
      if (((a0 >> 3) + b) * 8 < 2 * A) w0 |= (unsigned long long)ob_occ[(size_t)((a0 >> 3) + b) * p.occ_stride] << (8 * b);
      if (((k1 >> 3) + b) * 8 < 2 * A) w1 |= (unsigned long long)ob_occ[(size_t)((k1 >> 3) + b) * p.occ_stride] << (8 * b);
    }
    const long long base = raw0 + (long long)r * p.pitch + c;
    int step = 0;   // offset of the current cell from `base` in the pitched maps
#pragma unroll
    for (int j = 0; j < J; ++j) {
      raw[j] = vm[j] = 0.f;
      if (a0 + j < A) {
        raw[j] = p.logit_raw[base + step] + bp;
        if (p.vmap) vm[j] = p.vmap[base + step];
      }
      ++step;
      if (++c == n) { c = 0; step += p.pitch - n; }
    }
    const unsigned occ_bits = (unsigned)((w0 >> (a0 & 7)) | (w1 >> (k1 & 7)));
    occupied = occ_bits & (J < 32 ? ((1u << (J & 31)) - 1u) : 0xffffffffu);
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (a0 + j >= A) occupied |= 1u << j;
  } else {
    float o0[J], o1[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int a = a0 + j;
      raw[j] = vm[j] = o0[j] = o1[j] = 0.f;
      if (a < A) {
        raw[j] = raw_logit(a);
        if (engine) {
          if (p.occ) {
            const int view_cell = canon ? d4_forward(a, n, phase) : a;
            const int k1 = A + view_cell;
            const uint8_t* ob_occ = p.occ + (size_t)g * p.mrows_per_group + t;
            o0[j] = (float)((ob_occ[(size_t)(view_cell >> 3) * p.occ_stride] >> (view_cell & 7)) & 1);
            o1[j] = (float)((ob_occ[(size_t)(k1 >> 3) * p.occ_stride] >> (k1 & 7)) & 1);
          } else {
            const int orig_cell = (phase != 0 && !canon) ? d4_inverse(a, n, phase) : a;
            o0[j] = input_value(p.in, ob, 0, orig_cell, A);
            o1[j] = input_value(p.in, ob, 1, orig_cell, A);
          }
          if (p.vmap) {
            const int r = (a * p.n_magic) >> 16, c = a - r * n;
            vm[j] = p.vmap[raw0 + r * p.pitch + c];
          }
        } else {
          o0[j] = p.legal_in[ob * A + a] != 0 ? 0.f : 1.f;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (a0 + j >= A || o0[j] != 0.f || o1[j] != 0.f) occupied |= 1u << j;
  }
  float vsum = 0.f, lmax = -INFINITY;
  int nlegal = 0;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int a = a0 + j;
    const bool legal = !((occupied >> j) & 1u);
    if (a < A) {
      vsum += vm[j];
      if (p.logits_out) p.logits_out[ob * A + a] = ((p.flags & 1) && !legal) ? kFp32Min : raw[j];
    }
    raw[j] = legal ? raw[j] * inv_t : -INFINITY;   // z = mask(logits) / max(T, 1e-4)
    lmax = fmaxf(lmax, raw[j]);
    nlegal += legal ? 1 : 0;
  }
  if (engine && p.value_out) {
    const float tot = warp_sum(vsum);
    if (lane == 0) p.value_out[ob] = tanhf(tot / (float)A + (p.val_bias ? p.val_bias[g] : 0.f));
  }
  if (!p.do_sample) return;

  // With no legal cell every z equals the fill: uniform over all A actions.
  const bool none_legal = __reduce_add_sync(0xffffffffu, nlegal) == 0;
  const float zmax = none_legal ? 0.f : warp_max(lmax);
  // e = exp(z - max), then this lane's running sums; the lanes' totals are scanned with shuffles
  float local = 0.f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const float e = a0 + j < A ? (none_legal ? 1.f : expf(raw[j] - zmax)) : 0.f;   // exp(-inf) = 0 for occupied cells
    vm[j] = e;              // vm is free now: it keeps e
    local += e;
    raw[j] = local;         // inclusive running sum inside the lane
  }
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const float before = incl - local;
  const float total = __shfl_sync(0xffffffffu, incl, 31);
  const float u = board_uniform(p.seed, p.offset, (unsigned long long)(p.board_index0 + ob));
  const float target = u * total;
  // first action with mass whose running sum exceeds the target; if rounding left the target at or
  // above the total, the last action with mass
  int cand = 0x7fffffff, last = -1;
#pragma unroll
  for (int j = J - 1; j >= 0; --j) {
    if (vm[j] > 0.f) {
      if (before + raw[j] > target) cand = a0 + j;
      if (last < 0) last = a0 + j;
    }
  }
  int pick = __reduce_min_sync(0xffffffffu, cand);
  if (pick == 0x7fffffff) pick = __reduce_max_sync(0xffffffffu, last);
  if (lane == 0) {
    if (p.action_out) p.action_out[ob] = pick;
    // log-prob = z[a] - logsumexp(z) with logsumexp = max + log(sum exp(z - max)), as torch
    // computes it.  With no legal cell z is the fill everywhere: log(A) is absorbed by the fill
    // and the result is 0, which is what the reference's Categorical returns for that row.
    const float fill_z = fmaxf(kFp32Min * inv_t, -3.4028234663852886e38f);
    const float zpick = none_legal ? fill_z : raw_logit(pick) * inv_t;
    const float lse = (none_legal ? fill_z : zmax) + logf(total);
    if (p.logprob_out) p.logprob_out[ob] = zpick - lse;
  }
}

// Picks the instantiation whose lanes hold all the actions.
inline void (*finish_kernel_for(int n_actions))(FinishParams) {
  return n_actions <= 32 * kFinishSmallJ ? finish_kernel<kFinishSmallJ> : finish_kernel<kFinishMaxActions / 32>;
}

// ------------------------------------------------------------------------------------------------
// Standalone operators
// ------------------------------------------------------------------------------------------------
__global__ void mask_logits_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ legal,
                                   long long count, float fill, float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = legal[i] ? logits[i] : fill;
}

__global__ void transform_actions_kernel(const long long* __restrict__ actions, long long B, int n,
                                         const uint8_t* __restrict__ phase, int phase_all, int inverse,
                                         long long* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int ph = phase ? (phase[i] & 7) : (phase_all & 7);
  const int a = (int)actions[i];
  out[i] = inverse ? d4_inverse(a, n, ph) : d4_forward(a, n, ph);
}

__global__ void transform_boards_kernel(const int8_t* __restrict__ boards, long long B, int n,
                                        const uint8_t* __restrict__ phase, int phase_all,
                                        int8_t* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = n * n;
  if (i >= B * cells) return;
  const long long b = i / cells;
  const int j = (int)(i - b * cells);
  const int ph = phase ? (phase[b] & 7) : (phase_all & 7);
  out[i] = boards[b * cells + d4_inverse(j, n, ph)];
}

__global__ void network_input_kernel(const int8_t* __restrict__ boards, const int8_t* __restrict__ player,
                                     const int8_t* __restrict__ stones_left, long long B, int n,
                                     float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = n * n;
  if (i >= B * cells) return;
  const long long b = i / cells;
  const int j = (int)(i - b * cells);
  const int v = boards[i], me = player[b];
  float* o = out + b * 3 * cells + j;
  o[0] = v == me ? 1.f : 0.f;
  o[cells] = v == -me ? 1.f : 0.f;
  o[2 * cells] = stones_left[b] == 1 ? 1.f : 0.f;
}

// Self-test of the bounded-wait path: the kernels' own wait helper (tc::mbar_wait) on an mbarrier
// that nobody arrives on, with a short limit.  The wait runs out, and the kernel does what every
// role of the tensor-core kernels does then: records its status bit, raises the CTA's abort flag
// (which a second waiter observes and leaves on) and returns normally.
__global__ void expire_wait_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_barrier_init();
  }
  __syncthreads();
  const uint32_t b = tc::smem_u32(&bar);
  if (threadIdx.x == 0) {
    // first waiter: runs into the time limit
    if (!tc::mbar_wait(b, 0, &abort_flag, 0, limit_cycles)) {
      atomicOr(status, kStatWaitFull);
      abort_flag = 1;
    }
  } else if (threadIdx.x == 32) {
    // second waiter, with the kernels' full limit: must leave because the first raised the abort flag
    if (!tc::mbar_wait(b, 0, &abort_flag, 20) && abort_flag) atomicOr(status, kStatWaitEmpty);
  }
}

// Debug aid: activation planes -> fp32 NCHW [G*nb, c, n, n]
__global__ void unpack_activation_kernel(const uint4* __restrict__ planes, long long plane_rows, int front,
                                         int group_pos, int slots, int wp, int n, int c_real, int nb,
                                         float* __restrict__ out, int f16) {
  const int g = blockIdx.y;
  const int cells = n * n;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)nb * c_real * cells) return;
  const int cell = (int)(idx % cells);
  long long r = idx / cells;
  const int ch = (int)(r % c_real);
  const int t = (int)(r / c_real);
  const int rr = cell / n, cc = cell - rr * n;
  const long long row = (long long)front + (long long)g * group_pos + (long long)t * slots + rr * wp + cc;
  const void* e = planes + (size_t)(ch >> 3) * plane_rows + row;
  out[((size_t)g * nb + t) * c_real * cells + (size_t)ch * cells + cell] =
      f16 ? __half2float(reinterpret_cast<const __half*>(e)[ch & 7])
          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e)[ch & 7]);
}

}  // namespace c6
