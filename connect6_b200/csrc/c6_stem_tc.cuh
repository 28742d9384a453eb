// First backbone layer (the wide k0 x k0 stem, connect6/model.py:22,56-63) as ONE dense GEMM
// on tcgen05 tensor cores.
//
// For an n x n board and a k0 x k0 filter with k0 >= n the filter footprint covers most of the
// board from every output cell, so the layer is restated as a Toeplitz product
//     out[b, cell_out*C1 + co] = sum_k  X[b, k] * T[cell_out*C1 + co, k],   k = ci*n*n + cell_in
// with T[.., k] = w[co, ci, r_in - r_out + p, c_in - c_out + p] when that index lies inside the
// filter and 0 otherwise (p = k0/2).  X is simply the flattened NCHW input, so no im2col exists
// at run time; T is expanded once per weight update.  The product needs 3*n*n MACs per output
// (1083 for n = 19) instead of the 3*k0*k0 = 1587 of the zero-padded definition.
//
// Operands are K-major no-swizzle core-matrix rows (16 bytes = 8 bf16 along K) as in the 3x3
// kernel, stored tile-major in HBM so that one pipeline stage of one tile is one contiguous block:
//   X [board tile of 128][K/8][128 boards],   T [output tile][half][K/8][rows of that half].
// Tile: 128 boards x NT outputs (NT = C1 * cells-per-tile <= 256), K walked 32 at a time
// through a ring of bulk-copy stages.  The epilogue adds bias, applies SiLU and scatters each
// 32-channel group to the padded activation planes the next layer reads.
#pragma once

#include "c6_common.cuh"
#include "c6_tc.cuh"

namespace c6 {

struct StemTcParams {
  const uint4* xk;    // [board tile][kc][128] input rows
  const uint4* wt;    // [G][output tile][half][kc][nt/halves] Toeplitz rows
  const float* bias;  // [G][c1]
  uint4* out;         // activation planes [c1/8][plane_rows]
  int* status;
  long long* wait_cycles;  // nullable [8]: slots 1,2,4,5 as in the k x k kernel (MMA warp of CTA 0)
  long long plane_rows;
  long long mrows;     // rows per X plane (= G * mrows_per_group)
  int mrows_per_group; // multiple of 128 (256 in pair mode)
  int front;
  int group_pos;       // positions reserved per group in the activation planes
  int kc;              // K chunks (multiple of kcs)
  int kc_short;        // chunks of input planes 0 and 1 and the third plane's level (multiple of kcs)
  // The remaining chunks hold the third plane's residual (plane minus its level).  When
  // *p2_epoch != epoch every residual of this pass is zero -- the plane is constant on every board --
  // and the GEMM walks only kc_short chunks; otherwise all kc.
  const unsigned int* p2_epoch;
  unsigned int epoch;
  int kcs;             // K chunks per pipeline stage: 4 or 8
  int ntot;            // rows per T plane (= ntiles * nt)
  int nt;              // outputs per tile (multiple of 32, <= 256)
  int ntiles;
  int mtiles;          // per group (even in pair mode)
  int groups;
  int c1;              // padded stem output channels
  int bsize, wp, slots, nboards;
  int nstages;
  int acc_stride, tmem_cols;
};

constexpr int kStemEpiParts = 4;   // epilogue warps per TMEM lane quadrant: they take the 16-column units round robin
constexpr int kStemPatchBytes = 4 * kStemEpiParts * 4096;  // one 4 KB transposition patch per epilogue warp, behind the stages
constexpr int kStemThreads = 32 * (2 + 4 * kStemEpiParts);  // producer warp, MMA warp, sixteen epilogue warps
constexpr int kStemSmemHeader = 2048;
constexpr int kStemMaxStages = 12;

// PAIR = true: clusters of two CTAs share one 256-board x NT-output tile through cta_group::2 MMAs.
// CTA r stages the X rows of boards [128 r, 128 r + 128) and rows [r NT/2, (r+1) NT/2) of the
// Toeplitz tile, so every byte of T is fetched once per 256 boards instead of once per 128: the
// kernel is fed from L2 and this cuts its traffic by a third.
// F16 = true: fp16 operands and activations instead of bf16 (see the k x k kernel).
template <bool PAIR, bool F16>
__global__ void __launch_bounds__(kStemThreads, 1) stem_tc_kernel(const StemTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  // barrier slots: [0,12) full, [12,24) empty, 25-26 acc full, 27-28 acc empty, 29 drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 516);
  volatile int* never_flag = reinterpret_cast<volatile int*>(smem + 520);
  float* s_bias = reinterpret_cast<float*>(smem + 640);  // 0.5 * bias of all groups when that fits
  uint8_t* s_stage = smem + kStemSmemHeader;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dep_launch();
  const uint32_t crank = PAIR ? tc::cluster_ctarank() : 0u;
  const bool leader = crank == 0;
  const int nloc = PAIR ? p.nt / 2 : p.nt;           // Toeplitz rows this CTA stages
  const uint32_t a_plane = 128u * 16u;
  const uint32_t b_plane = (uint32_t)nloc * 16u;
  const uint32_t a_bytes = (uint32_t)p.kcs * a_plane, b_bytes = (uint32_t)p.kcs * b_plane;
  const uint32_t stage_bytes = a_bytes + b_bytes;    // multiples of 128 by construction
  // pipeline steps per tile, known only once the pack kernel in front of this one has finished
  auto steps_per_tile = [&](bool& short_k) {
    grid_dep_wait();
    short_k = __ldcg(p.p2_epoch) != p.epoch;
    return (short_k ? p.kc_short : p.kc) / p.kcs;
  };

  // work items: (group, board tile, output tile), output tile fastest; in pair mode a pair owns a
  // range of (group, board-tile PAIR, output tile) items and CTA r takes board tile 2*mp + r
  const int mt_items = PAIR ? p.mtiles / 2 : p.mtiles;
  const long long items = (long long)p.groups * mt_items * p.ntiles;
  const long long workers = PAIR ? gridDim.x / 2 : gridDim.x;
  const long long me = PAIR ? blockIdx.x / 2 : blockIdx.x;
  const long long i_begin = items * me / workers;
  const long long i_end = items * (me + 1) / workers;

  const uint32_t bar0 = tc::smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (12 + s); };
  auto bar_tfull = [&](int a) { return bar0 + 8u * (25 + a); };
  auto bar_tempty = [&](int a) { return bar0 + 8u * (27 + a); };
  const uint32_t bar_drain = bar0 + 8u * 29;

  if (threadIdx.x == 0) {
    const uint32_t both = (PAIR && leader) ? 2u : 1u;   // leader: the peer's relay arrives too
    for (int s = 0; s < kStemMaxStages; ++s) {
      tc::mbar_init(bar_full(s), both);
      tc::mbar_init(bar_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(bar_tfull(a), 1);
      tc::mbar_init(bar_tempty(a), 4 * kStemEpiParts * both);
    }
    tc::mbar_init(bar_drain, 1);
    *abort_flag = 0;
    *never_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tc::tmem_alloc2(tc::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
      tc::tmem_relinquish2();
    } else {
      tc::tmem_alloc(tc::smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
      tc::tmem_relinquish();
    }
  }
  if (warp >= 2) {
    for (int i = threadIdx.x - 64; i < p.groups * p.c1 && i < 320; i += kStemThreads - 64) s_bias[i] = 0.5f * p.bias[i];  // h = x/2
  }
  tc::fence_before_sync();
  if (PAIR) tc::cluster_sync(); else __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool bias_in_smem = p.groups * p.c1 <= 320;

  auto decode = [&](long long item, int& g, int& mt, int& nt_i) {
    nt_i = (int)(item % p.ntiles);
    const long long gm = item / p.ntiles;
    const int mp = (int)(gm % mt_items);
    g = (int)(gm / mt_items);
    mt = PAIR ? 2 * mp + (int)crank : mp;
  };

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    // Lane 0 waits for the stage and arms its barrier; lanes 0 and 1 then issue the stage's two bulk
    // copies (the operands are stored tile-major so that a stage is one contiguous block each).
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    bool short_k;
    const int ksteps = steps_per_tile(short_k);   // waits: the input rows come from the pack kernel in front of this one
    for (long long item = i_begin; item < i_end && ok; ++item) {
      int g, mt, nt_i;
      decode(item, g, mt, nt_i);
      // tile-major operands: [board tile][K chunk][128] and [group][output tile][half][K chunk][nloc]
      const uint4* xa = p.xk + ((size_t)g * p.mtiles + mt) * p.kc * 128;
      const uint4* wb = p.wt + (size_t)g * p.kc * p.ntot + (((size_t)nt_i * (PAIR ? 2 : 1) + crank) * p.kc) * nloc;
      for (int ks = 0; ks < ksteps; ++ks) {
        int got = 1;
        if (lane == 0) {
          got = tc::mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, 40) ? 1 : 0;
          if (got) tc::mbar_expect_tx(bar_full(s), stage_bytes);
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          if (lane == 0) atomicOr(p.status, kStatWaitEmpty);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint32_t dst = tc::smem_u32(s_stage + (size_t)s * stage_bytes);
        if (lane == 0) {
          tc::bulk_g2s(dst, xa + (size_t)ks * p.kcs * 128, a_bytes, bar_full(s));
        } else if (lane == 1) {
          tc::bulk_g2s(dst + a_bytes, wb + (size_t)ks * p.kcs * nloc, b_bytes, bar_full(s));
        }
        if (++s == p.nstages) { s = 0; ph ^= 1u; }
      }
    }
    if (!ok && lane == 0) {
      for (int st = 0; st < p.nstages; ++st) {
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {
          if (tc::mbar_try_wait(bar_full(st), 0) || tc::mbar_try_wait(bar_full(st), 1)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 && leader) {
    // ------------------------------ MMA issuer ------------------------------
    // Warp-uniform loop, one elected lane issues (see the k x k kernel for the reasoning).
    const uint32_t idesc = tc::make_idesc_16(PAIR ? 256 : 128, p.nt, F16);
    const uint32_t desc_hi = (uint32_t)(tc::make_desc(0, 0, 128u) >> 32);
    const uint32_t a_lbo_field = (a_plane >> 4) << 16, b_lbo_field = (b_plane >> 4) << 16;
    const uint32_t stage0_lo = tc::smem_u32(s_stage) >> 4;
    const uint32_t stage_rows = stage_bytes >> 4;
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    int tcount = 0;
    const bool timing = p.wait_cycles != nullptr && blockIdx.x == 0;
    long long wait_full = 0, wait_acc = 0, issue_clk = 0;
    bool short_k;
    const int ksteps = steps_per_tile(short_k);
    const long long loop_t0 = clock64();
    for (long long item = i_begin; item < i_end && ok; ++item, ++tcount) {
      const int acc = tcount & 1;
      const long long w0 = timing ? clock64() : 0;
      const bool got_acc = tc::mbar_wait(bar_tempty(acc), ((tcount >> 1) & 1u) ^ 1u, abort_flag);
      if (timing) wait_acc += clock64() - w0;
      if (!got_acc) {
        if (lane == 0) atomicOr(p.status, kStatWaitTmemEmpty);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_stride);
      for (int ks = 0; ks < ksteps; ++ks) {
        const long long w1 = timing ? clock64() : 0;
        const bool got = tc::mbar_wait(bar_full(s), ph, abort_flag);
        if (timing) wait_full += clock64() - w1;
        if (!got) {
          if (lane == 0) atomicOr(p.status, kStatWaitFull);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc::fence_after_sync();
        const long long w2 = timing ? clock64() : 0;
        const uint32_t a_lo = (stage0_lo + (uint32_t)s * stage_rows) | a_lbo_field;
        const uint32_t b_lo = (stage0_lo + (uint32_t)s * stage_rows + (a_bytes >> 4)) | b_lbo_field;
        if (tc::elect_one()) {
          for (int j = 0; j < p.kcs / 2; ++j) {
            const uint64_t ad = ((uint64_t)desc_hi << 32) | (a_lo + 2u * j * (a_plane >> 4));
            const uint64_t bd = ((uint64_t)desc_hi << 32) | (b_lo + 2u * j * (b_plane >> 4));
            if (PAIR) tc::mma_bf16_pair(d_tmem, ad, bd, idesc, (ks | j) != 0 ? 1u : 0u);
            else tc::mma_bf16(d_tmem, ad, bd, idesc, (ks | j) != 0 ? 1u : 0u);
          }
          if (PAIR) {
            tc::mma_commit_pair_both(bar_empty(s));
            if (ks == ksteps - 1) tc::mma_commit_pair_both(bar_tfull(acc));
          } else {
            tc::mma_commit(bar_empty(s));
            if (ks == ksteps - 1) tc::mma_commit(bar_tfull(acc));
          }
        }
        __syncwarp();
        if (timing) issue_clk += clock64() - w2;
        if (++s == p.nstages) { s = 0; ph ^= 1u; }
      }
    }
    if (timing && lane == 0) {
      p.wait_cycles[1] += wait_full;
      p.wait_cycles[2] += wait_acc;
      p.wait_cycles[4] += issue_clk;
      p.wait_cycles[5] += clock64() - loop_t0;
    }
    if (lane == 0) {
      if (PAIR) tc::mma_commit_pair_local(bar_drain); else tc::mma_commit(bar_drain);
      if (!tc::mbar_wait(bar_drain, 0, never_flag)) {
        atomicOr(p.status, kStatWaitDrain);
        *abort_flag = 1;
      }
    }
    __syncwarp();
  } else if (PAIR && warp == 1) {
    // ------------------------------ peer relay ------------------------------
    // Forwards every completed "stage full" phase of this CTA to the leader's barrier.
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    bool short_k;
    const int ksteps = steps_per_tile(short_k);
    for (long long item = i_begin; item < i_end && ok; ++item) {
      for (int ks = 0; ks < ksteps; ++ks) {
        if (!tc::mbar_wait_warp(bar_full(s), ph, abort_flag, 0)) {
          if (lane == 0) atomicOr(p.status, kStatWaitFull);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar_full(s), 0));
        if (++s == p.nstages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp >= 2) {
    // ------------------------------ epilogue ------------------------------
    // Sixteen warps: the four warps ("parts") of a TMEM lane quadrant share its 32 boards.  A board's
    // tile output is nt/8 pieces of 16 bytes = 8 channels of one cell, ordered plane-major
    // (piece = chunk plane * cells-per-tile + cell); a part owns a contiguous quarter of them, so its
    // pieces of one chunk plane are consecutive cells = consecutive rows of that plane.  Scattering them
    // straight from the TMEM layout (lane = board: 32 addresses 6.4 KB apart per store instruction)
    // made the stores -- 11.8 M separate 16-byte requests per launch -- the kernel's bottleneck
    // (measured: 0.229 ms with them, 0.124 ms without).  Instead every warp parks its pieces in a
    // private, XOR-swizzled 4 KB patch of shared memory and writes them out with lanes running along
    // the consecutive cells: up to 128 contiguous bytes per (board, plane), full sectors.
    // h = 0.5*acc + 0.5*bias, y = h + h*tanh(h).
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    bool short_k;
    steps_per_tile(short_k);
    const int cells = p.bsize * p.bsize;
    const int cpt = p.nt / p.c1;                    // cells per tile
    const int npieces = p.nt >> 3;                  // pieces per board per tile
    const int per_part = (npieces + kStemEpiParts - 1) / kStemEpiParts;   // <= 8
    const int piece0 = part * per_part;
    const int my_pieces = max(0, min(per_part, npieces - piece0));
    uint4* patch = reinterpret_cast<uint4*>(s_stage + (size_t)p.nstages * stage_bytes) + (size_t)(warp - 2) * 256;
    // cells per tile is a power of two (256 / c1 rounded down to one): piece -> (chunk plane, cell)
    // is a shift and a mask
    const int lcpt = 31 - __clz(cpt);
    const int wi = lane & 7;                                   // piece this lane writes out
    const int wpc = piece0 + (wi < my_pieces ? wi : 0);
    const int wq = wpc >> lcpt, wcl = wpc & (cpt - 1);
    bool ok = true;
    int tcount = 0;
    float amax = 0.f;   // fp16 mode: largest |activation| this thread stored
    for (long long item = i_begin; item < i_end && ok; ++item, ++tcount) {
      const int acc = tcount & 1;
      int g, mt, nt_i;
      decode(item, g, mt, nt_i);
      if (!tc::mbar_wait(bar_tfull(acc), (tcount >> 1) & 1u, abort_flag, 40)) {
        if (lane == 0) atomicOr(p.status, kStatWaitTmemFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)(acc * p.acc_stride) + ((uint32_t)(quad * 32) << 16);
      const float* gbias = p.bias + (size_t)g * p.c1;
      const float* sbias = s_bias + g * p.c1;
      // fetch this part's pieces (8 accumulator columns each), four per wait; the accumulator goes
      // back to the MMA warp as soon as the last fetch has landed
#pragma unroll
      for (int i0 = 0; i0 < 8; i0 += 4) {
        if (i0 < per_part) {
          uint32_t v[4][8];
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (i0 + b < my_pieces) tc::tmem_ld8(taddr + (uint32_t)(((piece0 + i0 + b) & (cpt - 1)) * p.c1 + ((piece0 + i0 + b) >> lcpt) * 8), v[b]);
          tc::tmem_wait_ld();
          if (i0 + 4 >= per_part) {
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if (PAIR) tc::mbar_arrive_cluster(tc::mapa(bar_tempty(acc), 0)); else tc::mbar_arrive(bar_tempty(acc));
            }
          }
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            if (i0 + b >= my_pieces) continue;
            float hb[8];
            const int ch = ((piece0 + i0 + b) >> lcpt) * 8;
            if (bias_in_smem) {
              const float4 b0 = *reinterpret_cast<const float4*>(sbias + ch);
              const float4 b1 = *reinterpret_cast<const float4*>(sbias + ch + 4);
              hb[0] = b0.x; hb[1] = b0.y; hb[2] = b0.z; hb[3] = b0.w;
              hb[4] = b1.x; hb[5] = b1.y; hb[6] = b1.z; hb[7] = b1.w;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) hb[j] = 0.5f * gbias[ch + j];
            }
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = silu_from_half(fmaf(__uint_as_float(v[b][j]), 0.5f, hb[j]));
            if (F16) {
#pragma unroll
              for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j]));
            }
            uint4 o;
            o.x = pack_h2<F16>(y[0], y[1]);
            o.y = pack_h2<F16>(y[2], y[3]);
            o.z = pack_h2<F16>(y[4], y[5]);
            o.w = pack_h2<F16>(y[6], y[7]);
            patch[lane * 8 + ((i0 + b) ^ (lane & 7))] = o;   // [board][piece], swizzled against bank conflicts
          }
        }
      }
      __syncwarp();
      // write out: 8 rounds of 4 boards x 8 pieces; lanes 8k..8k+7 hold consecutive pieces of one board
      const int cell = nt_i * cpt + wcl;
      const int r = cell / p.bsize, c = cell - r * p.bsize;
      const int board0 = mt * 128 + quad * 32 + (lane >> 3);       // this lane's board in round 0
      uint4* dst = p.out + (size_t)wq * p.plane_rows + (long long)p.front + (long long)g * p.group_pos +
                   (long long)board0 * p.slots + r * p.wp + c;
      const bool lane_ok = wi < my_pieces && cell < cells;
#pragma unroll 4
      for (int rd = 0; rd < 8; ++rd) {
        const int bl = rd * 4 + (lane >> 3);
        if (lane_ok && board0 + rd * 4 < p.nboards) dst[(size_t)rd * 4 * p.slots] = patch[bl * 8 + (wi ^ (bl & 7))];
      }
      __syncwarp();   // the patch is reused by the next tile
    }
    if (F16 && !(amax <= 65504.f)) atomicOr(p.status, kStatF16Range);
  }

  tc::fence_before_sync();
  if (PAIR) tc::cluster_sync(); else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::fence_after_sync();
    if (PAIR) tc::tmem_dealloc2(tmem_base, (uint32_t)p.tmem_cols); else tc::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace c6
