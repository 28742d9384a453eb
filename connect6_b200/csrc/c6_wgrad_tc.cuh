// Weight gradient of one k x k "same" convolution layer on tcgen05 tensor cores (the backward of
// connect6/model.py:104-106 as PyTorch's autograd computes it inside the PPO update,
// connect6/train.py:1047-1119):
//     dW[co, ci, tap] = sum over positions p of  dPre[p, co] * x[p + shift(tap), ci]
// with dPre = dL/d(conv output) and shift(tap) = dy * Wp + dx in the padded linear board layout of the
// forward kernels (pad slots of both operands are zero, so the sum may run over every slot).
//
// GEMM view: M = Cout (one 128-row block), N = Cin, K = positions.  Both operands are read straight from
// the forward layout -- channel-chunk planes whose 16-byte rows hold 8 channels of one position -- as
// MN-major no-swizzle operands: 8 consecutive positions of 8 channels are 128 contiguous bytes (a core
// matrix), the next 8 positions follow 128 bytes later (leading byte offset), the next 8 channels one
// plane later (stride byte offset).  A filter tap is again a pure change of the B descriptor's start
// address, and each tap accumulates into its own TMEM columns.
//
// Work split: a CTA owns a group of taps (as many as fit 512 TMEM columns: floor(512 / Cin), at most
// k*k) and a contiguous slab of K tiles of `tile_rows` positions (256 when two such stages fit shared
// memory, else 128: a stage costs one bulk copy per channel-chunk plane whatever its length, so longer tiles
// mean fewer copies and barrier rounds; tiles run linearly over all slots, padding included); it writes its
// fp32 partial sums
// [slab][tap][128][Cin] to global memory and a second kernel adds the slabs up in a fixed order
// (no atomics: results are reproducible).
// CTA = 256 threads: warp 0 stages operands with bulk copies, warps 1, 6 and 7 issue the MMAs (each every third tap
// of the CTA; warp 1 owns TMEM), warps 2-5 drain the accumulators at the end.  Every wait is bounded.
#pragma once

#include "c6_common.cuh"
#include "c6_tc.cuh"

namespace c6 {

struct WgradParams {
  const uint4* x;       // layer input planes  [cin/8][plane_rows]
  const uint4* dpre;    // gradient planes     [cout/8][plane_rows]
  float* partial;       // [nslabs][ntaps][128][cin] fp32
  int* status;
  long long plane_rows;
  int front;            // plane row of position 0
  int halo_rows;        // rows staged before and after the 128 tile rows of x (multiple of 8, >= kside/2 * (wp + 1))
  int cin, cout;        // padded to multiples of 32; cout <= 128, cin <= 128
  int kside, wp;
  int tile_rows;        // positions per K tile: 128 or 256
  int ntiles;           // K tiles: tile t covers positions [t * tile_rows, (t + 1) * tile_rows)
  int ntaps;            // kside * kside
  int taps_per_cta;     // taps of one tap group
  int ngroups, nslabs;  // grid = ngroups * nslabs; CTA b: group b % ngroups, slab b / ngroups
  int nstages;
  int halo_after;       // rows staged behind the tile rows of x (= halo_rows for a k x k layer)
  long long dpre_plane_rows;   // plane pitch and first row of the gradient planes (= plane_rows, front for a k x k layer)
  int dpre_front;
  // First-layer ("stem") mode, stem_k > 0: the filter is stem_k x stem_k on 3 input planes, too wide for one tap per
  // accumulator.  x = the 3 x-expanded input planes of the direct stem (row R of plane ci holds the 8 consecutive linear
  // positions R..R+7 of the zero-padded input images of pitch stem_wi), dpre = the layer's gradient planes in that same
  // input geometry.  Roles swap: the M operand is the INPUT -- 8 filter columns (the 8 elements of a row) x 16 filter
  // rows (stride byte offset = stem_wi rows) = 128 filter positions per MMA -- and the N operand the gradient's
  // `cout` channels.  A "tap" is (input plane, block of 8 filter columns, block of 16 filter rows): ntaps = 3 *
  // stem_nkxb * stem_nkyb, its accumulator 128 x cout.  partial is [nslabs][ntaps][128][cout].
  int stem_k, stem_wi, stem_nkxb, stem_nkyb;
  // tiles_per_board > 0: K tiles are aligned to board images of `board_rows` positions, tile t covers the positions
  // [(t / tiles_per_board) * board_rows + (t % tiles_per_board) * tile_rows, ... + tile_rows): the all-padding tail of an
  // image is never multiplied.  0: tiles run linearly over all positions.
  int tiles_per_board, board_rows;
  // bias_tap >= 0 (k x k mode only): the bias gradient db[co] = sum over positions of dPre[p][co] rides along as 16 more
  // accumulator columns of tap `bias_tap` of tap group 0 (its last tap, so that the columns lie behind every other
  // accumulator): two more "input planes" behind the staged ones hold 1.0 in every element, so the tap's MMA with
  // N = cin + 16 adds up dPre itself.  The CTAs of group 0 write column cin of that accumulator to
  // bias_partial[slab][128]; the reduction kernel adds the slabs.  -1: no bias gradient here.
  int bias_tap;
  float* bias_partial;
};

constexpr int kWgradIssuers = 3;     // MMA-issuing warps: issuer i takes the taps t of the CTA with t % kWgradIssuers == i
constexpr int kWgradThreads = 32 * (6 + kWgradIssuers - 1);   // warp 0 producer, warp 1 and warps 6.. MMA issuers, warps 2-5 epilogue
constexpr int kWgradSmemHeader = 1024;
constexpr int kWgradMaxStages = 8;
constexpr int kWgradMaxTaps = 9;     // taps one CTA may own (a 3 x 3 filter)

// Instruction descriptor: D = fp32, A = B = bf16, both MN-major (bits 15 and 16 set).
__host__ __device__ __forceinline__ uint32_t make_idesc_bf16_mn(int m, int n) {
  return tc::make_idesc_bf16(m, n) | (1u << 15) | (1u << 16);
}

// with_bias: two more planes (the ones that sum dPre into the bias gradient) behind the input planes
__host__ __device__ inline int wgrad_stage_bytes(int cin, int cout, int halo_rows, int tile_rows, bool with_bias = false) {
  return (cout / 8) * tile_rows * 16 + (cin / 8 + (with_bias ? 2 : 0)) * (tile_rows + 2 * halo_rows) * 16;
}
__host__ __device__ inline int wgrad_stem_stage_bytes(int cout, int halo_before, int halo_after, int tile_rows) {
  return (cout / 8) * tile_rows * 16 + 3 * (tile_rows + halo_before + halo_after) * 16;
}

__global__ void __launch_bounds__(kWgradThreads, 1) wgrad_tc_kernel(const WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);   // [0,8) full, [8,16) empty, 16 accumulators ready
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 260);
  uint8_t* s_stage = smem + kWgradSmemHeader;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = blockIdx.x % p.ngroups, slab = blockIdx.x / p.ngroups;
  const int tap0 = group * p.taps_per_cta;
  const int ntap = min(p.taps_per_cta, p.ntaps - tap0);
  const int t_begin = (int)(((long long)p.ntiles * slab) / p.nslabs);
  const int t_end = (int)(((long long)p.ntiles * (slab + 1)) / p.nslabs);
  const bool stem = p.stem_k > 0;
  const int xrows = p.tile_rows + p.halo_rows + p.halo_after;
  const int xplanes = stem ? 3 : p.cin / 8;
  const uint32_t a_plane = (uint32_t)p.tile_rows * 16u;
  const uint32_t b_plane = (uint32_t)xrows * 16u;
  const bool with_bias = !stem && p.bias_tap >= 0;
  const uint32_t a_bytes = (uint32_t)(p.cout / 8) * a_plane;
  const uint32_t b_bytes = (uint32_t)xplanes * b_plane;
  const uint32_t tx_bytes = a_bytes + b_bytes;         // what the bulk copies of one stage deliver
  const uint32_t stage_bytes = tx_bytes + (with_bias ? 2u * b_plane : 0u);     // multiples of 128
  const uint32_t bar0 = tc::smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (8 + s); };
  const uint32_t bar_done = bar0 + 8u * 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWgradMaxStages; ++s) {
      tc::mbar_init(bar_full(s), 1);
      tc::mbar_init(bar_empty(s), kWgradIssuers);      // one commit per issuer
    }
    tc::mbar_init(bar_done, kWgradIssuers);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(tmem_slot), 512u);
    tc::tmem_relinquish();
  }
  if (with_bias) {
    // the two planes of ones behind the input planes of every stage: written once, no copy ever lands on them
    const uint32_t ones = 0x3F803F80u;   // bf16 1.0 twice
    for (int s = 0; s < p.nstages; ++s) {
      uint4* dst = reinterpret_cast<uint4*>(s_stage + (size_t)s * stage_bytes + tx_bytes);
      for (int i = threadIdx.x; i < 2 * xrows; i += kWgradThreads) dst[i] = make_uint4(ones, ones, ones, ones);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    // lane i < cout/8 copies gradient plane i (the tile's rows), the next cin/8 lanes one input plane
    // each (the tile's rows plus the halo on both sides)
    const int na = p.cout / 8, nb = xplanes;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = t_begin; tile < t_end && ok; ++tile) {
      int got = 1;
      if (lane == 0) {
        got = tc::mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, 40) ? 1 : 0;
        if (got) tc::mbar_expect_tx(bar_full(s), tx_bytes);
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        if (lane == 0) atomicOr(p.status, kStatWaitEmpty);
        *abort_flag = 1;
        ok = false;
        break;
      }
      const long long pos0 = p.tiles_per_board > 0
                                 ? (long long)(tile / p.tiles_per_board) * p.board_rows + (long long)(tile % p.tiles_per_board) * p.tile_rows
                                 : (long long)tile * p.tile_rows;
      const long long row0 = (long long)p.front + pos0;
      const long long drow0 = (long long)p.dpre_front + pos0;
      const uint32_t dst = tc::smem_u32(s_stage + (size_t)s * stage_bytes);
      if (lane < na) {
        tc::bulk_g2s(dst + (uint32_t)lane * a_plane, p.dpre + (size_t)lane * p.dpre_plane_rows + drow0, a_plane, bar_full(s));
      } else if (lane < na + nb) {
        const int q = lane - na;
        tc::bulk_g2s(dst + a_bytes + (uint32_t)q * b_plane, p.x + (size_t)q * p.plane_rows + row0 - p.halo_rows, b_plane,
                     bar_full(s));
      }
      if (++s == p.nstages) { s = 0; ph ^= 1u; }
    }
    if (!ok && lane == 0) {
      for (int st = 0; st < p.nstages; ++st) {   // let copies in flight land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {
          if (tc::mbar_try_wait(bar_full(st), 0) || tc::mbar_try_wait(bar_full(st), 1)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp >= 6) {
    // ------------------------------ MMA issuers ------------------------------
    // several warps, each issues the MMAs of its share of the CTA's taps: one thread's issue rate does not feed the pipe
    const int which = warp == 1 ? 0 : warp - 5;
    const int ncols = stem ? p.cout : p.cin;        // accumulator columns of one tap
    const uint32_t idesc = make_idesc_bf16_mn(128, ncols);
    const uint32_t idesc_bias = make_idesc_bf16_mn(128, ncols + 16);      // the tap that also sums dPre itself
    const int bias_t = (with_bias && group == 0) ? p.bias_tap : -1;
    const int kh = (stem ? p.stem_k : p.kside) >> 1;
    // MN-major no-swizzle descriptors: leading byte offset = 128 B (next 8 positions), stride byte offset =
    // the plane pitch of the staged operand (next 8 channels); in stem mode the input operand's "next 8 rows of M"
    // are the next filter row: stem_wi positions further
    const uint32_t a_hi = (uint32_t)(tc::make_desc(0, 128u, a_plane) >> 32);
    const uint32_t b_hi = (uint32_t)(tc::make_desc(0, 128u, stem ? (uint32_t)p.stem_wi * 16u : b_plane) >> 32);
    const uint32_t lbo_field = (128u >> 4) << 16;
    uint32_t tshift[kWgradMaxTaps];      // row of the staged input planes where tap t's operand starts
#pragma unroll
    for (int t = 0; t < kWgradMaxTaps; ++t) {
      const int tap = min(tap0 + t, p.ntaps - 1);
      if (stem) {
        const int per_plane = p.stem_nkxb * p.stem_nkyb;
        const int ci = tap / per_plane, rem = tap - ci * per_plane;
        const int kxb = rem / p.stem_nkyb, kyb = rem - kxb * p.stem_nkyb;
        tshift[t] = (uint32_t)(ci * xrows + p.halo_rows + (kyb * 16 - kh) * p.stem_wi + kxb * 8 - kh);
      } else {
        tshift[t] = (uint32_t)(p.halo_rows + (tap / p.kside - kh) * p.wp + (tap % p.kside - kh));
      }
    }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = t_begin; tile < t_end && ok; ++tile) {
      if (!tc::mbar_wait(bar_full(s), ph, abort_flag)) {
        if (lane == 0) atomicOr(p.status, kStatWaitFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t a_lo0 = (tc::smem_u32(s_stage + (size_t)s * stage_bytes) >> 4) | lbo_field;
      const uint32_t b_lo0 = a_lo0 + (a_bytes >> 4);
      if (tc::elect_one()) {
        for (int ks = 0; ks < p.tile_rows / 16; ++ks) {            // 16 positions per MMA
          const uint32_t a_lo = a_lo0 + (uint32_t)ks * 16u;
          const uint32_t b_lo = b_lo0 + (uint32_t)ks * 16u;
          const uint32_t acc = (tile != t_begin || ks != 0) ? 1u : 0u;
          // unrolled over the CTA's taps: the issue loop must stay well below the ~50 clocks an MMA takes,
          // so the per-tap row shifts live in registers (no division, no table in memory)
#pragma unroll
          for (int t = 0; t < kWgradMaxTaps; ++t)
            if (t < ntap && t % kWgradIssuers == which) {
              const uint64_t grad_desc = ((uint64_t)a_hi << 32) | a_lo, in_desc = ((uint64_t)b_hi << 32) | (b_lo + tshift[t]);
              tc::mma_bf16(tmem_base + (uint32_t)(t * ncols), stem ? in_desc : grad_desc, stem ? grad_desc : in_desc,
                           t == bias_t ? idesc_bias : idesc, acc);
            }
        }
        tc::mma_commit(bar_empty(s));
        if (tile == t_end - 1) tc::mma_commit(bar_done);
      }
      __syncwarp();
      if (++s == p.nstages) { s = 0; ph ^= 1u; }
    }
    if (t_begin >= t_end && lane == 0) tc::mbar_arrive(bar_done);   // an empty slab still releases the epilogue (one arrival per issuer)
  } else if (warp >= 2 && warp <= 5) {
    // ------------------------------ epilogue ------------------------------
    // warp w may read TMEM lanes 32*(w%4)..+31: output channels (stem mode: filter positions); each lane writes its
    // rows of the partial sums
    const int quad = warp & 3;
    const int co = quad * 32 + lane;
    const int ncols = stem ? p.cout : p.cin;
    if (!tc::mbar_wait(bar_done, 0, abort_flag, 100)) {
      if (lane == 0) atomicOr(p.status, kStatWaitTmemFull);
      *abort_flag = 1;
    } else {
      tc::fence_after_sync();
      const bool empty = t_begin >= t_end;
      for (int t = 0; t < ntap; ++t) {
        float* dst = p.partial + (((size_t)slab * p.ntaps + tap0 + t) * 128 + co) * ncols;
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          uint32_t v[16];
          tc::tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(t * ncols + c0), v);
          tc::tmem_wait_ld();
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            float4 o;
            o.x = empty ? 0.f : __uint_as_float(v[j4 * 4 + 0]);
            o.y = empty ? 0.f : __uint_as_float(v[j4 * 4 + 1]);
            o.z = empty ? 0.f : __uint_as_float(v[j4 * 4 + 2]);
            o.w = empty ? 0.f : __uint_as_float(v[j4 * 4 + 3]);
            reinterpret_cast<float4*>(dst + c0)[j4] = o;
          }
        }
      }
      if (with_bias && group == 0) {
        uint32_t v[16];
        tc::tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(p.bias_tap * ncols + ncols), v);
        tc::tmem_wait_ld();
        p.bias_partial[(size_t)slab * 128 + co] = empty ? 0.f : __uint_as_float(v[0]);
      }
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512u);
  }
}

// sum of p[s * stride] over the slabs in a fixed order: four interleaved running sums (slab s goes to sum s % 4) so that
// four loads are in flight, added up as (s0 + s1) + (s2 + s3) -- the same association on every run
__device__ __forceinline__ float sum_slabs(const float* __restrict__ p, size_t stride, int nslabs) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int s = 0;
  for (; s + 4 <= nslabs; s += 4) {
    a0 += p[(size_t)s * stride];
    a1 += p[(size_t)(s + 1) * stride];
    a2 += p[(size_t)(s + 2) * stride];
    a3 += p[(size_t)(s + 3) * stride];
  }
  if (s < nslabs) a0 += p[(size_t)s * stride];
  if (s + 1 < nslabs) a1 += p[(size_t)(s + 1) * stride];
  if (s + 2 < nslabs) a2 += p[(size_t)(s + 2) * stride];
  return (a0 + a1) + (a2 + a3);
}

// dW[co][ci][tap] (the reference's [Cout,Cin,K,K] fp32 layout) = sum over slabs of the partial sums, in a fixed order.
// With bias_partial: the threads behind the last weight add up db[co] = sum over slabs of bias_partial[slab][co].
__global__ void wgrad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nslabs, int ntaps,
                                    int cin_p, int cin, int cout, const float* __restrict__ bias_partial,
                                    float* __restrict__ db) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nw = (long long)cout * cin * ntaps;
  if (idx >= nw) {
    if (bias_partial != nullptr && idx - nw < cout) db[idx - nw] = sum_slabs(bias_partial + (idx - nw), 128, nslabs);
    return;
  }
  const int tap = (int)(idx % ntaps);
  const int ci = (int)((idx / ntaps) % cin);
  const int co = (int)(idx / ((long long)ntaps * cin));
  dw[idx] = sum_slabs(partial + ((size_t)tap * 128 + co) * cin_p + ci, (size_t)ntaps * 128 * cin_p, nslabs);
}

// Stem mode: dW[co][ci][ky][kx] from partial[slab][tap = (ci, kx / 8, ky / 16)][m = (ky % 16) * 8 + kx % 8][co].
__global__ void wgrad_reduce_stem_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nslabs, int ntaps,
                                         int cout_p, int cout, int kside, int nkxb, int nkyb) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)cout * 3 * kside * kside) return;
  const int kx = (int)(idx % kside);
  const int ky = (int)((idx / kside) % kside);
  const int ci = (int)((idx / ((long long)kside * kside)) % 3);
  const int co = (int)(idx / (3LL * kside * kside));
  const int tap = (ci * nkxb + (kx >> 3)) * nkyb + (ky >> 4);
  const int m = (ky & 15) * 8 + (kx & 7);
  dw[idx] = sum_slabs(partial + ((size_t)tap * 128 + m) * cout_p + co, (size_t)ntaps * 128 * cout_p, nslabs);
}

}  // namespace c6
