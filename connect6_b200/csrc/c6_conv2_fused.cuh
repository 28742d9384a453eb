// Two consecutive narrow 3 x 3 "same" convolution + bias + SiLU layers in ONE kernel, the intermediate
// activation never leaving the SM (backbone layers 1 and 2 of the default network, 32 -> 32 -> 64 channels:
// connect6/model.py:52-67,104-106).  Run separately, those two layers are bound by HBM (420 + 630 MB per 8192
// boards at 75-80 % of the copy rate); fused, the 32-channel intermediate (26 KB per board image) stays in shared
// memory and 420 MB of that traffic disappears.
//
// Why no halo exchange is needed: tiles are aligned to board images (see c6_conv_tc.cuh), and a board image
// carries its own zero padding -- the rows in front of its first cell and behind its last are pad slots of the
// neighbouring images.  So the second layer's input for ALL tiles of a board is the first layer's output for the
// tiles of that board plus zeros: a CTA that owns whole boards owns everything it needs.
//
// Work unit: a CTA pair (cta_group::2 MMAs, M = 256) takes two boards at a time, CTA r the board 2j + r.  Per board
// and CTA:  bulk-copy the input image (Cin/8 planes x (T*128 + 2*halo) rows)  ->  layer-1 MMAs of its T tiles
// (9 taps x Cin/16 groups each) into T accumulators  ->  epilogue 1: bias + SiLU, one 16-bit rounding, rows written
// into the "mid" image in shared memory (same plane layout, pad slots zero)  ->  layer-2 MMAs of the T tiles
// straight from the mid image (a tap is again a start-address shift)  ->  epilogue 2: bias + SiLU, global stores.
// Two MMA issuers (warps 1 and 2 of the leader CTA) each run this chain on their own boards with their own input
// ring, mid image and accumulators, so that one chain's epilogue latency hides behind the other's MMAs; four
// epilogue teams of four warps, two per issuer, share the six tile epilogues of a board so that every accumulator
// always meets the same team.  The writes of epilogue 1 are generic-proxy stores that the tensor core reads through
// the async proxy: each writer fences (fence.proxy.async) before it arrives on the "mid full" barrier.
// Every wait is bounded: when one runs out the CTA records a status bit, stops, frees TMEM and returns.
#pragma once

#include "c6_common.cuh"
#include "c6_conv_tc.cuh"
#include "c6_tc.cuh"

namespace c6 {

struct Conv2FusedParams {
  const uint4* in;        // input planes  [cin/8][plane_rows]
  uint4* out;             // output planes [c2/8][plane_rows]
  const uint4* w1_pair;   // layer-1 weights, pair layout [2 halves][cin/16][9][2][c1/2] rows
  const uint4* w2_pair;   // layer-2 weights, pair layout [2 halves][c1/16][9][2][c2/2] rows
  int* status;
  long long plane_rows;
  int front, halo_rows;   // plane row of position 0; rows staged in front of / behind a board's tiles (multiple of 8)
  int cin, c1, c2;        // channel counts padded to multiples of 32 (cin, c1 <= 32 KB budget below; c2 <= 64)
  int wp, slots, bsize, nboards;
  int tiles_per_board;    // T: 128-position tiles that cover the cells of one board image
  int board_pairs;        // ceil(nboards / 2)
  alignas(16) float c_hb1[64];   // 0.5 * bias of layer 1 (constant bank: the epilogue must not read shared memory)
  float c_hb2[64];               // 0.5 * bias of layer 2
};

constexpr int kFusedIssuers = 2;
constexpr int kFusedMaxTiles = 3;          // tiles per board image (19 x 19: 3)
constexpr int kFusedSmemHeader = 1024;
constexpr int kFusedThreads = kConvThreads;   // same warp layout as the k x k kernel: 0 producer, 1-4 issuer slots, 5-20 epilogue

__host__ __device__ inline int fused_image_rows(int tiles_per_board, int halo_rows) { return tiles_per_board * 128 + 2 * halo_rows; }
// shared memory: header | layer-1 weights | layer-2 weights | per issuer: 2 input stages + 1 mid image
__host__ __device__ inline int fused_smem_bytes(int cin, int c1, int c2, int tiles_per_board, int halo_rows) {
  const int rows = fused_image_rows(tiles_per_board, halo_rows);
  const int w1 = (cin / 16) * 9 * 2 * (c1 / 2) * 16, w2 = (c1 / 16) * 9 * 2 * (c2 / 2) * 16;
  const int in_img = (cin / 8) * rows * 16, mid_img = (c1 / 8) * rows * 16;
  return 128 + kFusedSmemHeader + ((w1 + 127) & ~127) + ((w2 + 127) & ~127) + kFusedIssuers * (2 * in_img + mid_img);
}

template <bool F16>
__global__ void __launch_bounds__(kFusedThreads, 1) conv2_fused_kernel(const Conv2FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 768);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 772);
  volatile int* never_flag = reinterpret_cast<volatile int*>(smem + 776);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dep_launch();
  const uint32_t crank = tc::cluster_ctarank();
  const bool leader = crank == 0;
  const int T = p.tiles_per_board;
  const int rows = fused_image_rows(T, p.halo_rows);
  const uint32_t plane_bytes = (uint32_t)rows * 16u;
  const uint32_t in_img = (uint32_t)(p.cin / 8) * plane_bytes, mid_img = (uint32_t)(p.c1 / 8) * plane_bytes;
  const int n1 = p.c1 / 2, n2 = p.c2 / 2;                           // weight rows this CTA holds per block
  const uint32_t w1q = 9u * 2u * n1 * 16u, w2q = 9u * 2u * n2 * 16u;  // bytes of one 16-channel group
  const uint32_t w1_bytes = w1q * (p.cin / 16), w2_bytes = w2q * (p.c1 / 16);
  uint8_t* s_w1 = smem + kFusedSmemHeader;
  uint8_t* s_w2 = s_w1 + ((w1_bytes + 127u) & ~127u);
  uint8_t* s_work = s_w2 + ((w2_bytes + 127u) & ~127u);
  const uint32_t issuer_bytes = 2u * in_img + mid_img;
  auto s_in = [&](int i, int s) { return s_work + (size_t)i * issuer_bytes + (size_t)s * in_img; };
  auto s_mid = [&](int i) { return s_work + (size_t)i * issuer_bytes + 2u * in_img; };

  // barrier slots, per issuer i (16 slots each): 0-1 in_full, 2-3 in_empty, 4-6 l1_full, 7-9 l1_empty, 10 mid_full,
  // 11 mid_empty, 12-13 l2_full, 14-15 l2_empty; then 32 weights, 33-34 drain
  const uint32_t bar0 = tc::smem_u32(bars);
  auto bar = [&](int i, int k) { return bar0 + 8u * (16 * i + k); };
  const uint32_t bar_w = bar0 + 8u * 32;
  auto bar_drain = [&](int i) { return bar0 + 8u * (33 + i); };

  // this pair's contiguous range of board pairs; issuer i takes the pairs jb + i, jb + i + 2, ...
  const int npairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const int jb = (int)(((long long)p.board_pairs * pair) / npairs), je = (int)(((long long)p.board_pairs * (pair + 1)) / npairs);
  auto nboards_of = [&](int i) { return je - jb > i ? (je - jb - i + kFusedIssuers - 1) / kFusedIssuers : 0; };

  if (threadIdx.x == 0) {
    const uint32_t both = leader ? 2u : 1u;
    for (int i = 0; i < kFusedIssuers; ++i) {
      for (int s = 0; s < 2; ++s) {
        tc::mbar_init(bar(i, s), both);          // in_full: own copies (+ the peer's relay at the leader)
        tc::mbar_init(bar(i, 2 + s), 1);         // in_empty: one commit
      }
      for (int t = 0; t < 3; ++t) {
        tc::mbar_init(bar(i, 4 + t), 1);         // l1_full: one commit
        tc::mbar_init(bar(i, 7 + t), 4 * both);  // l1_empty: the four warps of the draining team, in both CTAs
      }
      tc::mbar_init(bar(i, 10), (uint32_t)(4 * T) * both);   // mid_full: every epilogue-1 warp of both CTAs
      tc::mbar_init(bar(i, 11), 1);              // mid_empty: one commit
      for (int s = 0; s < 2; ++s) {
        tc::mbar_init(bar(i, 12 + s), 1);        // l2_full
        tc::mbar_init(bar(i, 14 + s), 4 * both); // l2_empty
      }
      tc::mbar_init(bar_drain(i), 1);
    }
    tc::mbar_init(bar_w, both);
    *abort_flag = 0;
    *never_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc2(tc::smem_u32(tmem_slot), 512u);
    tc::tmem_relinquish2();
  }
  // The rows of the mid images in front of the first tile and behind the last are never written by the epilogue:
  // they are the zero padding above the first and below the last board row.  (Pad slots inside the tiles are
  // written as zeros by epilogue 1 every time.)
  for (int i = 0; i < kFusedIssuers; ++i) {
    uint4* mid = reinterpret_cast<uint4*>(s_mid(i));
    const int nplanes = p.c1 / 8;
    for (int k = threadIdx.x; k < nplanes * 2 * p.halo_rows; k += kFusedThreads) {
      const int q = k / (2 * p.halo_rows), r = k % (2 * p.halo_rows);
      mid[q * rows + (r < p.halo_rows ? r : rows - 2 * p.halo_rows + r)] = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc::fence_before_sync();
  tc::cluster_sync();
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns of issuer i: layer-1 accumulator t at 256 i + 32 t... (stride c1 rounded to 32), layer-2 ring at 256 i + 128
  auto l1_acc = [&](int i, int t) { return tmem_base + (uint32_t)(256 * i + 32 * t); };
  auto l2_acc = [&](int i, int s) { return tmem_base + (uint32_t)(256 * i + 128 + 64 * s); };

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    bool ok = true;
    if (lane == 0) {
      tc::mbar_expect_tx(bar_w, w1_bytes + w2_bytes);
      tc::bulk_g2s(tc::smem_u32(s_w1), reinterpret_cast<const uint8_t*>(p.w1_pair) + (size_t)crank * w1_bytes, w1_bytes, bar_w);
      tc::bulk_g2s(tc::smem_u32(s_w2), reinterpret_cast<const uint8_t*>(p.w2_pair) + (size_t)crank * w2_bytes, w2_bytes, bar_w);
    }
    grid_dep_wait();   // the weights do not depend on the previous kernel, the activations do
    const int nplanes = p.cin / 8;
    const int nmax = nboards_of(0);
    for (int n = 0; n < nmax && ok; ++n) {
      for (int i = 0; i < kFusedIssuers && ok; ++i) {
        if (n >= nboards_of(i)) break;
        const int j = jb + i + n * kFusedIssuers;
        const long long board = 2LL * j + crank;
        const int s = n & 1;
        const uint32_t ph = (uint32_t)(n >> 1) & 1u;
        int got = 1;
        if (lane == 0) {
          got = tc::mbar_wait(bar(i, 2 + s), ph ^ 1u, abort_flag, kIdleBackoffNs) ? 1 : 0;
          if (got) tc::mbar_expect_tx(bar(i, s), in_img);
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          if (lane == 0) atomicOr(p.status, kStatWaitEmpty);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (lane < nplanes) {
          const uint4* src = p.in + (size_t)lane * p.plane_rows + p.front + board * p.slots - p.halo_rows;
          tc::bulk_g2s(tc::smem_u32(s_in(i, s)) + (uint32_t)lane * plane_bytes, src, plane_bytes, bar(i, s));
        }
      }
    }
    if (!ok && lane == 0) {
      for (int i = 0; i < kFusedIssuers; ++i)
        for (int s = 0; s < 2; ++s) {
          const long long t0 = clock64();
          while (clock64() - t0 < 200000) {
            if (tc::mbar_try_wait(bar(i, s), 0) || tc::mbar_try_wait(bar(i, s), 1)) break;
          }
        }
    }
    __syncwarp();
  } else if (warp >= 1 && warp <= kFusedIssuers && leader) {
    // ------------------------------ MMA issuers ------------------------------
    const int i = warp - 1;
    const uint32_t idesc1 = tc::make_idesc_16(256, p.c1, F16), idesc2 = tc::make_idesc_16(256, p.c2, F16);
    const uint32_t desc_hi = (uint32_t)(tc::make_desc(0, 0, 128u) >> 32);
    const uint32_t a_lbo = (plane_bytes >> 4) << 16;
    const uint32_t b1_lbo = ((uint32_t)(n1 * 16) >> 4) << 16, b2_lbo = ((uint32_t)(n2 * 16) >> 4) << 16;
    const uint32_t w1_lo = (tc::smem_u32(s_w1) >> 4) | b1_lbo, w2_lo = (tc::smem_u32(s_w2) >> 4) | b2_lbo;
    bool ok = true;
    if (!tc::mbar_wait_warp(bar_w, 0, abort_flag, 32)) {
      if (lane == 0) atomicOr(p.status, kStatWaitWeights);
      *abort_flag = 1;
      ok = false;
    }
    int l2_use[2] = {0, 0};
    const int nmine = nboards_of(i);
    for (int n = 0; n < nmine && ok; ++n) {
      const int s = n & 1;
      const uint32_t np = (uint32_t)n & 1u;
      if (!tc::mbar_wait(bar(i, s), (uint32_t)(n >> 1) & 1u, abort_flag)) {
        if (lane == 0) atomicOr(p.status, kStatWaitFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      // ---- layer 1: T tiles from the staged input image ----
      const uint32_t in_lo = (tc::smem_u32(s_in(i, s)) >> 4) | a_lbo;
      for (int t = 0; t < T && ok; ++t) {
        if (!tc::mbar_wait(bar(i, 7 + t), np ^ 1u, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatWaitTmemEmpty);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc::fence_after_sync();
        if (tc::elect_one()) {
          const uint32_t d = l1_acc(i, t);
          for (int q = 0; q < p.cin / 16; ++q) {
            const uint32_t a_lo = in_lo + (uint32_t)q * 2u * (uint32_t)rows + (uint32_t)(t * 128 + p.halo_rows);
            const uint32_t b_lo = w1_lo + (uint32_t)q * (w1q >> 4);
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
              const int dy = tap / 3 - 1, dx = tap % 3 - 1;
              tc::mma_bf16_pair(d, ((uint64_t)desc_hi << 32) | (a_lo + (uint32_t)(dy * p.wp + dx)),
                                ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * 2u * (uint32_t)n1), idesc1, (q | tap) != 0 ? 1u : 0u);
            }
          }
          tc::mma_commit_pair_both(bar(i, 4 + t));               // accumulator t ready (both CTAs)
          if (t == T - 1) tc::mma_commit_pair_both(bar(i, 2 + s));   // input stage reusable
        }
        __syncwarp();
      }
      if (!ok) break;
      // ---- layer 2: T tiles from the mid image that epilogue 1 has written ----
      if (!tc::mbar_wait(bar(i, 10), np, abort_flag)) {
        if (lane == 0) atomicOr(p.status, kStatWaitFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t mid_lo = (tc::smem_u32(s_mid(i)) >> 4) | a_lbo;
      for (int t = 0; t < T && ok; ++t) {
        const int slot = t & 1;
        if (!tc::mbar_wait(bar(i, 14 + slot), ((uint32_t)l2_use[slot] & 1u) ^ 1u, abort_flag)) {
          if (lane == 0) atomicOr(p.status, kStatWaitTmemEmpty);
          *abort_flag = 1;
          ok = false;
          break;
        }
        ++l2_use[slot];
        tc::fence_after_sync();
        if (tc::elect_one()) {
          const uint32_t d = l2_acc(i, slot);
          for (int q = 0; q < p.c1 / 16; ++q) {
            const uint32_t a_lo = mid_lo + (uint32_t)q * 2u * (uint32_t)rows + (uint32_t)(t * 128 + p.halo_rows);
            const uint32_t b_lo = w2_lo + (uint32_t)q * (w2q >> 4);
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
              const int dy = tap / 3 - 1, dx = tap % 3 - 1;
              tc::mma_bf16_pair(d, ((uint64_t)desc_hi << 32) | (a_lo + (uint32_t)(dy * p.wp + dx)),
                                ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * 2u * (uint32_t)n2), idesc2, (q | tap) != 0 ? 1u : 0u);
            }
          }
          tc::mma_commit_pair_both(bar(i, 12 + slot));
          if (t == T - 1) tc::mma_commit_pair_both(bar(i, 11));   // mid image reusable
        }
        __syncwarp();
      }
    }
    if (lane == 0) {   // every MMA issued must have retired before TMEM is freed
      tc::mma_commit_pair_local(bar_drain(i));
      if (!tc::mbar_wait(bar_drain(i), 0, never_flag)) {
        atomicOr(p.status, kStatWaitDrain);
        *abort_flag = 1;
      }
    }
    __syncwarp();
  } else if (warp >= 1 && warp <= kFusedIssuers && !leader) {
    // ------------------------------ peer relays ------------------------------
    // forward "weights landed" and every "input stage landed" of this CTA to the leader's barriers
    const int i = warp - 1;
    bool ok = true;
    if (i == 0) {
      if (tc::mbar_wait_warp(bar_w, 0, abort_flag, 32)) {
        if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar_w, 0));
      } else {
        if (lane == 0) atomicOr(p.status, kStatWaitWeights);
        *abort_flag = 1;
        ok = false;
      }
    }
    const int nmine = nboards_of(i);
    for (int n = 0; n < nmine && ok; ++n) {
      const int s = n & 1;
      if (!tc::mbar_wait_warp(bar(i, s), (uint32_t)(n >> 1) & 1u, abort_flag, 0)) {
        if (lane == 0) atomicOr(p.status, kStatWaitFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar(i, s), 0));
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 16) {
    // ------------------------------ epilogue ------------------------------
    // teams 0,1 serve issuer 0, teams 2,3 issuer 1.  Jobs of a board in issue order: L1 tile 0..T-1, then L2 tile
    // 0..T-1; job k of the 2T belongs to team k % 2 of the issuer, so layer-2 ring slot t % 2 and layer-1
    // accumulator t always meet the same team (T = 3: team 0 takes L1.0, L1.2, L2.1; team 1 takes L1.1, L2.0, L2.2).
    const int quad = warp & 3;
    const int team = (warp - kEpiWarp0) >> 2;
    const int i = team >> 1, sub = team & 1;
    grid_dep_wait();
    const int row = quad * 32 + lane;
    const int nmine = nboards_of(i);
    int l2_use[2] = {0, 0};
    float amax = 0.f;
    bool ok = true;
    uint4* mid = reinterpret_cast<uint4*>(s_mid(i));
    for (int n = 0; n < nmine && ok; ++n) {
      const uint32_t np = (uint32_t)n & 1u;
      const int j = jb + i + n * kFusedIssuers;
      const long long board = 2LL * j + crank;
      const bool board_ok = board < p.nboards;
      bool mid_free = false;
      for (int k = sub; k < 2 * T && ok; k += 2) {
        const bool first = k < T;
        const int t = first ? k : k - T;
        const int slot_pos = t * 128 + row;                     // slot inside the board image
        const int r = slot_pos / p.wp, c = slot_pos - r * p.wp;
        const bool valid = board_ok && r < p.bsize && c < p.bsize;
        if (first) {
          // ---- epilogue 1: accumulator t of layer 1 -> mid image ----
          if (!mid_free) {
            // the previous board's layer-2 MMAs must have finished reading the mid image
            if (!tc::mbar_wait(bar(i, 11), np ^ 1u, abort_flag, kIdleBackoffNs)) {
              if (lane == 0) atomicOr(p.status, kStatWaitEmpty);
              *abort_flag = 1;
              ok = false;
              break;
            }
            mid_free = true;
          }
          if (!tc::mbar_wait(bar(i, 4 + t), np, abort_flag, kIdleBackoffNs)) {
            if (lane == 0) atomicOr(p.status, kStatWaitTmemFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc::fence_after_sync();
          const uint32_t taddr = l1_acc(i, t) + ((uint32_t)(quad * 32) << 16);
          const int nunits = p.c1 >> 4;
          for (int u = 0; u < nunits; ++u) {
            uint32_t v[16];
            tc::tmem_ld16(taddr + (uint32_t)(u * 16), v);
            tc::tmem_wait_ld();
            if (u == nunits - 1) {
              tc::fence_before_sync();
              __syncwarp();
              if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar(i, 7 + t), 0));   // accumulator t drained
            }
            float y[16];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 hb = reinterpret_cast<const float4*>(p.c_hb1)[u * 4 + j4];
              y[j4 * 4 + 0] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 0]), 0.5f, hb.x));
              y[j4 * 4 + 1] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 1]), 0.5f, hb.y));
              y[j4 * 4 + 2] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 2]), 0.5f, hb.z));
              y[j4 * 4 + 3] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 3]), 0.5f, hb.w));
            }
            if (F16) {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) amax = fmaxf(amax, fabsf(y[jj]));
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              uint4 o;
              o.x = valid ? pack_h2<F16>(y[8 * kk + 0], y[8 * kk + 1]) : 0u;
              o.y = valid ? pack_h2<F16>(y[8 * kk + 2], y[8 * kk + 3]) : 0u;
              o.z = valid ? pack_h2<F16>(y[8 * kk + 4], y[8 * kk + 5]) : 0u;
              o.w = valid ? pack_h2<F16>(y[8 * kk + 6], y[8 * kk + 7]) : 0u;
              mid[(size_t)(u * 2 + kk) * rows + p.halo_rows + slot_pos] = o;
            }
          }
          // generic-proxy stores -> async-proxy reads of the tensor core
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar(i, 10), 0));
        } else {
          // ---- epilogue 2: layer-2 ring slot t % 2 -> global ----
          const int slot = t & 1;
          if (!tc::mbar_wait(bar(i, 12 + slot), (uint32_t)l2_use[slot] & 1u, abort_flag, kIdleBackoffNs)) {
            if (lane == 0) atomicOr(p.status, kStatWaitTmemFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ++l2_use[slot];
          tc::fence_after_sync();
          const uint32_t taddr = l2_acc(i, slot) + ((uint32_t)(quad * 32) << 16);
          uint4* out_row = p.out + p.front + board * p.slots + slot_pos;
          const int nunits = p.c2 >> 4;
          for (int u = 0; u < nunits; ++u) {
            uint32_t v[16];
            tc::tmem_ld16(taddr + (uint32_t)(u * 16), v);
            tc::tmem_wait_ld();
            if (u == nunits - 1) {
              tc::fence_before_sync();
              __syncwarp();
              if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar(i, 14 + slot), 0));
            }
            float y[16];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 hb = reinterpret_cast<const float4*>(p.c_hb2)[u * 4 + j4];
              y[j4 * 4 + 0] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 0]), 0.5f, hb.x));
              y[j4 * 4 + 1] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 1]), 0.5f, hb.y));
              y[j4 * 4 + 2] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 2]), 0.5f, hb.z));
              y[j4 * 4 + 3] = silu_from_half(fmaf(__uint_as_float(v[j4 * 4 + 3]), 0.5f, hb.w));
            }
            if (F16) {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) amax = fmaxf(amax, fabsf(y[jj]));
            }
            if (board_ok) {
#pragma unroll
              for (int kk = 0; kk < 2; ++kk) {
                uint4 o;
                o.x = valid ? pack_h2<F16>(y[8 * kk + 0], y[8 * kk + 1]) : 0u;
                o.y = valid ? pack_h2<F16>(y[8 * kk + 2], y[8 * kk + 3]) : 0u;
                o.z = valid ? pack_h2<F16>(y[8 * kk + 4], y[8 * kk + 5]) : 0u;
                o.w = valid ? pack_h2<F16>(y[8 * kk + 6], y[8 * kk + 7]) : 0u;
                out_row[(size_t)(u * 2 + kk) * p.plane_rows] = o;
              }
            }
          }
        }
      }
    }
    if (F16 && !(amax <= 65504.f)) atomicOr(p.status, kStatF16Range);
  }

  tc::fence_before_sync();
  tc::cluster_sync();   // the peer's shared memory outlives the leader's MMAs
  if (warp == 1) {
    __syncwarp();
    tc::fence_after_sync();
    tc::tmem_dealloc2(tmem_base, 512u);
  }
}

}  // namespace c6
