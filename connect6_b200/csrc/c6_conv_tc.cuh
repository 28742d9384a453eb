// k x k "same" convolution + bias + SiLU as an implicit GEMM on tcgen05 tensor cores
// (backbone layers after the stem: connect6/model.py:52-67,104-106), optionally fused with
// the two 1x1 heads (connect6/model.py:70-75,108-109).
//
// Data layout in HBM.  Activations are bf16 "channel-chunk planes": plane q holds channels
// 8q..8q+7 of every board position as one 16-byte row, positions running linearly through a
// zero-padded board image: cell (r,c) of board b is row  front + b*S + r*Wp + c  with
// Wp = n + pad, S = Wp*Wp.  Column n..Wp-1 of every image row and image rows n..Wp-1 are
// zero, so they serve as the right/left and bottom/top zero padding of neighbouring cells and
// boards at once.  With this layout the input of filter tap (dy,dx) for 128 consecutive output
// positions is the same plane shifted by dy*Wp+dx rows: ONE staged copy of 128+2*halo rows per
// channel chunk feeds all k*k taps, and a tap is selected by moving the start address of the
// MMA's shared-memory descriptor.
//
// GEMM view per tile: M = 128 positions (TMEM lanes), N = Cout, K = k*k*Cin walked as
// (16-channel group q) x (tap).  Weights are pre-packed [q][tap][2][Cout] rows of 8 bf16 and stay
// resident in shared memory when they fit; otherwise the blocks of a step travel with its
// activation stage.  A pipeline step stages 32 input channels (two q: 4 planes of 128+2*halo rows).
//
// CTA = 704 threads: warp 0 issues bulk copies; warps 1-4 (one per SM sub-partition) issue the
// MMAs of tiles t = i mod 4, each into its own accumulator -- a lone issuer that shares its
// scheduler with busy epilogue warps only reaches half the tensor pipe's rate (measured), four keep
// it saturated and hide each other's per-step barrier work; warps 5-20 drain the accumulators
// (bias + SiLU in fp32, one bf16 rounding, 16-byte coalesced stores) as four teams of four warps;
// warp 21 is a second producer.  The epilogue of one tile is a chain of long latencies (a TMEM
// fetch takes ~450 clocks, the tanh unit 8 clocks per warp instruction): with two teams it, not
// the tensor pipe, bounded every layer of up to 64 output channels (measured with the MMAs and
// copies switched off: no change), with four teams -- four epilogue warps per scheduler -- the
// layers run at their MMA or HBM floor.
// A ring of 2, 4 or 8 TMEM accumulators lets the teams overlap the MMAs of later tiles.  Every wait
// is bounded: when one runs out the CTA records a status bit, stops, frees TMEM and returns.
//
// Direct stem mode (generic instantiation KS = 0 with p.stem set): the first backbone layer
// (3 input planes, one wide k0 x k0 filter, connect6/model.py:22,56-63) as an implicit GEMM straight from
// the filter, for passes with few boards per weight set -- the Toeplitz stem GEMM reads 27 MB of expanded
// weights per model whatever the batch, this mode reads the model's own k0*k0*3*Cout filter.  K runs
// along the filter's x axis: input plane ci is stored "x-expanded", row p holding the 8 consecutive
// linear positions p .. p+7 of the zero-padded board image (pitch Wi), so one 128 x N x 16 MMA with
// A chunk pitch (LBO) = 8 rows covers 16 consecutive kx of one (ci, ky): a "tap" is (ky, 16-wide kx
// block), its shift (ky - k0/2) * Wi + 16 * block - k0/2, and the filter is zero beyond kx = k0 - 1.
// A pipeline step is one input plane; output positions are walked in the INPUT geometry and stored to the
// output planes' own (narrower) geometry, cells only.
#pragma once

#include "c6_common.cuh"
#include "c6_tc.cuh"

namespace c6 {

struct ConvTcParams {
  const uint4* in;       // input planes  [cin/8][plane_rows] of 16-byte rows
  uint4* out;            // output planes [n/8][plane_rows]; unused when head != 0
  const uint4* aux;      // kEpiDsilu, kEpiLinearMul: planes of the same shape as `out`
  uint4* out2;           // kEpiSiluSave: second output, planes of the same shape as `out`
  const uint4* w;        // packed weights, per group [cin/16][taps][2][n] rows
  const uint4* w_pair;   // pair mode: per group [2 halves][cin/16][taps][2][n/2] rows
  const float* bias;     // [G][n]
  const float* head_wp;  // [G][n] policy 1x1 weights (head only)
  const float* head_wv;  // [G][n] value 1x1 weights (head only)
  float* logit_raw;      // [G * group_pos] (head only)
  float* vmap;           // same shape (head only)
  int* status;
  long long* wait_cycles;  // nullable [8]: CTA 0's clocks {producer waits empty, MMA waits full, MMA waits acc empty, epilogue waits acc full, MMA issue blocks, MMA loop total, epilogue first TMEM fetch, epilogue arithmetic}
  long long plane_rows;
  int front;             // plane row of position 0
  int halo_rows;         // rows staged before and after the 128 tile rows (multiple of 8)
  int cin, n;            // channel counts, padded to multiples of 32
  int kside;             // filter side k
  int wp, slots;         // padded row pitch Wp and slots per board S
  int bsize;             // board side n
  int nboards;           // boards per group in this pass
  int tiles_per_group;
  int tiles_per_board;   // > 0: tile t covers positions (t / tpb) * slots + (t % tpb) * 128 ... + 127 of its group
                         // (the all-padding tail of every board image is never computed); 0: tile t covers 128 t ...
  int group_pos;         // positions reserved per group in the planes
  int ctas_per_group;
  int resident;
  int nstages;           // = nissue * spi
  int nissue;            // MMA issuer warps in use (1, 2 or 4; divides nacc)
  int spi;               // pipeline stages owned by each issuer (its private ring)
  int qps;               // 16-channel groups per pipeline step: 1 or 2
  int acc_stride;        // TMEM columns between accumulator buffers
  int nacc;              // accumulator buffers in the ring: 2, 4 or 8 (twice the issuers when possible)
  int tmem_cols;
  int head;
  // ---- generalisations used by the direct stem mode (plain layers: the values in brackets) ----
  long long in_plane_rows; // rows per input plane [= plane_rows]
  int ntaps;             // MMAs per 16-channel group [kside * kside]
  int halo_after;        // rows staged behind the 128 tile rows [= halo_rows]
  int planes_step;       // activation planes per pipeline step [2 * qps]
  int stem;              // 1: direct stem mode
  int stem_hx;           // stem: 16-wide kx blocks per filter row
  int a_lbo_rows;        // stem: rows between the two K chunks of an A operand (8) [0: the stage's plane pitch]
  int out_front, out_wp, out_slots, out_group_pos;   // stem: geometry of the output planes (wp, slots, front, group_pos describe the input)
  // Single-model engines pass the epilogue vectors by value: kernel parameters live in the
  // constant bank, whose cache is separate from shared memory -- the MMAs already use the whole
  // shared-memory bandwidth, so epilogue reads from shared memory would queue behind them.
  int use_const;         // 1: read the three arrays below instead of the shared-memory copies
  alignas(16) float c_hbias[256];    // 0.5 * bias
  float c_wp[256];       // policy head weights
  float c_wv[256];       // value head weights
};

constexpr int kEpiSilu = 0, kEpiLinear = 1, kEpiDsilu = 2, kEpiSiluSave = 3, kEpiLinearMul = 4;
constexpr int kEpiTeams = 4;                   // epilogue teams of four warps (as many as the accumulator ring allows are used)
constexpr int kEpiWarp0 = 5;                   // first epilogue warp
constexpr int kProducer2Warp = kEpiWarp0 + 4 * kEpiTeams;
constexpr int kConvThreads = 32 * (kProducer2Warp + 1);  // producer, four MMA warps, 4*kEpiTeams epilogue warps, second producer
constexpr int kEpiBatch = 1;                   // 16-column units fetched from TMEM per wait (80 registers per thread at 704 threads)
constexpr int kConvSmemHeader = 5888;  // barriers, TMEM slot, abort flag, bias and head vectors, head partials
constexpr int kMaxStages = 16;
constexpr int kMaxAcc = 8;
constexpr uint32_t kIdleBackoffNs = 40;   // sleep between polls of the roles that wait long (saves issue slots and power)

__host__ __device__ inline int conv_stage_rows(int halo_rows) { return 128 + 2 * halo_rows; }

// KS = filter side known at compile time (1, 3, 5) so that the tap loop unrolls and the per-tap
// descriptor offsets live in registers; KS = 0 is the generic run-time loop.
// PAIR = true: the kernel runs as clusters of two CTAs that drive one cta_group::2 MMA (M = 256 =
// two tiles).  CTA r of the pair stages the activations of tile 2j + r and keeps rows
// [r*N/2, (r+1)*N/2) of every weight block; the leader (r = 0) issues the MMAs, which read both
// CTAs' shared memory at the same offsets.  Halving the B operand per CTA cuts the shared-memory
// operand traffic that bounds a 128 x N MMA for N < 128 and frees shared memory for more stages.
// F16 = true: operands and stored activations are fp16 instead of bf16 (same MMA rate, 11-bit instead
// of 8-bit significands, range +-65504: stores saturate and the CTA reports kStatF16Range).
// TIMED = true compiles the in-kernel clock counters in (p.wait_cycles); the plain instantiation
// carries none of them: even untaken, they cost the epilogue 2-3 % on the narrow layers.
// EPI selects what the epilogue makes of z = accumulator + bias:
//   kEpiSilu    y = silu(z)                      the forward layer
//   kEpiLinear  y = z                            a plain convolution (the input gradient of a layer: its
//                                                output gradient convolved with the flipped, transposed filter)
//   kEpiDsilu   y = aux * silu'(z)               the layer's forward recomputed and turned straight into the
//                                                gradient at the convolution output: aux holds dL/d(layer output)
//                                                in the output's own plane layout
//   kEpiSiluSave  y = silu(z), out2 = silu'(z)   the forward layer of a training step: the derivative is kept (same
//                                                layout as y) so that the backward needs no recomputation
//   kEpiLinearMul y = z * aux                    the input gradient of a layer times the saved silu' of the layer below:
//                                                the gradient at that layer's convolution output in one pass
template <int KS, bool PAIR, bool F16, bool TIMED, int EPI = 0>
__global__ void __launch_bounds__(kConvThreads, 1) conv_tc_kernel(const ConvTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte aligned view of dynamic shared memory
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  // barrier slots: [0,16) full, [16,32) empty, 32 weights, 33-40 acc full, 41-48 acc empty, 49-52 drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 516);
  volatile int* never_flag = reinterpret_cast<volatile int*>(smem + 520);  // stays 0
  float* s_bias = reinterpret_cast<float*>(smem + 640);
  float* s_wp = s_bias + 256;
  float* s_wv = s_wp + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dep_launch();   // the next kernel's CTAs may move in as ours exit; its own wait orders the data
  unsigned long long gt_start = 0;
  if (TIMED && p.wait_cycles) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt_start));
  const uint32_t crank = PAIR ? tc::cluster_ctarank() : 0u;
  const bool leader = crank == 0;
  const int nloc = PAIR ? p.n / 2 : p.n;   // weight rows this CTA holds
  const int taps = p.ntaps;
  const int nq = p.cin >> 4;
  const int rows = 128 + p.halo_rows + p.halo_after;
  const uint32_t a_bytes = (uint32_t)p.planes_step * rows * 16u;  // channel-chunk planes of one step (2 * qps)
  const uint32_t wq_bytes = (uint32_t)taps * 2u * nloc * 16u;   // this CTA's weights of one q (16 input channels)
  const int nsteps = nq / p.qps;                                 // pipeline steps per tile
  const uint32_t w_bytes = wq_bytes * nq;
  const uint32_t stage_bytes = (a_bytes + (p.resident ? 0u : (uint32_t)p.qps * wq_bytes) + 127u) & ~127u;
  const uint32_t w_region = p.resident ? ((w_bytes + 127u) & ~127u) : 0u;
  uint8_t* s_w = smem + kConvSmemHeader;
  uint8_t* s_stage = s_w + w_region;

  const int group = blockIdx.x / p.ctas_per_group;
  const int cta_in_group = blockIdx.x - group * p.ctas_per_group;
  // Contiguous, balanced tile range inside the group.  Local tile number tl = 0 .. ntl-1 maps to
  // tile t_first + tl * t_stride; in pair mode the pair owns a range of tile PAIRS and this CTA takes
  // the even or odd member of each.
  int t_first, ntl;
  constexpr int t_stride = PAIR ? 2 : 1;
  if (PAIR) {
    const int npairs = p.ctas_per_group >> 1, pair = cta_in_group >> 1, ptiles = p.tiles_per_group >> 1;
    const int pb = (int)(((long long)ptiles * pair) / npairs), pe = (int)(((long long)ptiles * (pair + 1)) / npairs);
    t_first = 2 * pb + (int)crank;
    ntl = pe - pb;
  } else {
    t_first = (int)(((long long)p.tiles_per_group * cta_in_group) / p.ctas_per_group);
    ntl = (int)(((long long)p.tiles_per_group * (cta_in_group + 1)) / p.ctas_per_group) - t_first;
  }

  const uint32_t bar0 = tc::smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (16 + s); };
  const uint32_t bar_w = bar0 + 8u * 32;
  auto bar_tfull = [&](int a) { return bar0 + 8u * (33 + a); };
  auto bar_tempty = [&](int a) { return bar0 + 8u * (41 + a); };
  auto bar_drain = [&](int i) { return bar0 + 8u * (49 + i); };   // one per issuer

  if (threadIdx.x == 0) {
    // pair mode, leader: "full" and "weights" also need the peer's relay arrival, "accumulator
    // drained" the four warps of the draining team in BOTH CTAs
    const uint32_t both = (PAIR && leader) ? 2u : 1u;
    for (int s = 0; s < kMaxStages; ++s) {
      tc::mbar_init(bar_full(s), both);
      tc::mbar_init(bar_empty(s), 1);
    }
    tc::mbar_init(bar_w, both);
    for (int a = 0; a < kMaxAcc; ++a) {
      tc::mbar_init(bar_tfull(a), 1);
      tc::mbar_init(bar_tempty(a), 4 * both);
    }
    for (int i = 0; i < 4; ++i) tc::mbar_init(bar_drain(i), 1);
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
  if (warp >= kEpiWarp0 && warp < kProducer2Warp) {
    for (int i = threadIdx.x - 32 * kEpiWarp0; i < p.n; i += 128 * kEpiTeams) {
      s_bias[i] = 0.5f * p.bias[(size_t)group * p.n + i];  // the epilogue works on h = x/2
      if (p.head) {
        s_wp[i] = p.head_wp[(size_t)group * p.n + i];
        s_wv[i] = p.head_wv[(size_t)group * p.n + i];
      }
    }
  }
  tc::fence_before_sync();
  if (PAIR) tc::cluster_sync(); else __syncthreads();   // barriers of both CTAs exist before anyone arrives
  tc::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const uint4* w_group = PAIR ? p.w_pair + ((size_t)group * 2 + crank) * (w_bytes / 16) : p.w + (size_t)group * (w_bytes / 16);
  const long long group_row0 = (long long)p.front + (long long)group * p.group_pos;
  // first position (inside the group) of a tile
  auto tile_pos = [&](int tile) {
    return p.tiles_per_board ? (tile / p.tiles_per_board) * p.slots + (tile % p.tiles_per_board) * 128 : tile * 128;
  };

  if (warp == 0 || warp == kProducer2Warp) {
    // ------------------------------ producers ------------------------------
    // The warp walks the loop together: lane 0 waits for the stage and arms its barrier, then lanes
    // 0 .. 2*qps-1 each issue the bulk copy of one channel-chunk plane (issuing a copy costs a few
    // hundred clocks per thread, so the planes of a stage are issued in parallel).
    // Two producer warps split the issuers' rings between them (ring i belongs to producer i % 2):
    // one warp alone cannot issue copies fast enough for four consumers.
    const int prod = warp == 0 ? 0 : 1;
    const int nprod = p.nissue >= 2 ? 2 : 1;
    bool ok = prod < nprod;
    if (p.resident && lane == 0 && prod == 0) {
      tc::mbar_expect_tx(bar_w, w_bytes);
      for (uint32_t off = 0; off < w_bytes; off += 32768u) {
        const uint32_t len = (w_bytes - off) < 32768u ? (w_bytes - off) : 32768u;
        tc::bulk_g2s(tc::smem_u32(s_w + off), reinterpret_cast<const uint8_t*>(w_group) + off, len, bar_w);
      }
    }
    grid_dep_wait();   // weights do not depend on the previous kernel, the activations do
    long long waited = 0;
    const bool timing = TIMED && p.wait_cycles != nullptr && blockIdx.x == 0 && prod == 0;
    // Every issuer owns a private ring of `spi` stages, so each stage barrier has exactly one
    // producer and one consumer that sees all of its phases.  Tiles are fed in waves of `nissue`
    // (tile tb + i belongs to issuer i), step by step across the wave, so that all issuers advance
    // together; every ring has received the same number of steps, hence one (position, parity) pair.
    int sl = 0;
    uint32_t ph = 0;
    const int nplanes = p.planes_step;
    for (int tb = 0; tb < ntl && ok; tb += p.nissue) {
      for (int step = 0; step < nsteps && ok; ++step) {
        for (int iss = prod; iss < p.nissue; iss += nprod) {
          if (tb + iss >= ntl) break;
          const int tile = t_first + (tb + iss) * t_stride;
          const long long row0 = group_row0 + tile_pos(tile) - p.halo_rows;
          const int s = iss * p.spi + sl;
          const long long w0 = timing ? clock64() : 0;
          int got = 1;
          if (lane == 0) {
            got = tc::mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, kIdleBackoffNs) ? 1 : 0;
            if (got) tc::mbar_expect_tx(bar_full(s), a_bytes + (p.resident ? 0u : (uint32_t)p.qps * wq_bytes));
          }
          got = __shfl_sync(0xffffffffu, got, 0);
          if (timing) waited += clock64() - w0;
          if (!got) {
            if (lane == 0) atomicOr(p.status, kStatWaitEmpty);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t dst = tc::smem_u32(s_stage + (size_t)s * stage_bytes);
          if (lane < nplanes) {
            const uint4* src = p.in + (size_t)(nplanes * step + lane) * p.in_plane_rows + row0;
            tc::bulk_g2s(dst + (uint32_t)lane * rows * 16u, src, rows * 16u, bar_full(s));
          } else if (lane == nplanes && !p.resident) {
            tc::bulk_g2s(dst + a_bytes, reinterpret_cast<const uint8_t*>(w_group) + (size_t)(p.qps * step) * wq_bytes,
                         (uint32_t)p.qps * wq_bytes, bar_full(s));
          }
        }
        if (++sl == p.spi) { sl = 0; ph ^= 1u; }
      }
    }
    if (timing && lane == 0) p.wait_cycles[0] += waited;
    if (!ok && lane == 0) {
      // let copies already in flight land before the CTA's shared memory is released
      for (int st = 0; st < p.nstages; ++st) {
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {
          if (tc::mbar_try_wait(bar_full(st), 0) || tc::mbar_try_wait(bar_full(st), 1)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp >= 1 && warp <= 4 && warp - 1 < p.nissue && leader) {
    // ------------------------------ MMA issuers ------------------------------
    // Issuer i walks local tiles i, i + nissue, ... in lock step (warp-uniform control flow
    // keeps descriptors and barrier addresses in uniform registers); one elected lane issues the
    // MMAs and commits.  It consumes its private stage ring [i*spi, (i+1)*spi).
    const int issuer = warp - 1;
    const uint32_t idesc = tc::make_idesc_16(PAIR ? 256 : 128, p.n, F16);
    const int kh = p.kside >> 1;
    const uint32_t desc_hi = (uint32_t)(tc::make_desc(0, 0, 128u) >> 32);   // SBO = 128 B, version 1
    const uint32_t a_lbo_field = (uint32_t)(p.a_lbo_rows ? p.a_lbo_rows : rows) << 16;   // LBO (16-byte units) = plane pitch of a stage
    const uint32_t b_lbo_field = ((uint32_t)(nloc * 16) >> 4) << 16;          // LBO = this CTA's Cout rows
    const uint32_t b_step = 2u * (uint32_t)nloc;                               // rows between taps
    const uint32_t w_lo = (tc::smem_u32(s_w) >> 4) | b_lbo_field;
    const uint32_t wq_rows = wq_bytes >> 4;
    const uint32_t stage0_lo = (tc::smem_u32(s_stage) >> 4) | a_lbo_field;
    const uint32_t stage_rows = stage_bytes >> 4;
    const bool timing = TIMED && p.wait_cycles != nullptr && blockIdx.x == 0 && issuer == 0;
    bool ok = true;
    if (p.resident && !tc::mbar_wait_warp(bar_w, 0, abort_flag, 32)) {
      if (lane == 0) atomicOr(p.status, kStatWaitWeights);
      *abort_flag = 1;
      ok = false;
    }
    int sl = 0;             // position in the private ring and parity of its current round
    uint32_t ph = 0;
    long long wait_full = 0, wait_acc = 0, issue_clk = 0;
    const long long loop_t0 = clock64();
    if (TIMED && p.wait_cycles && lane == 0 && issuer == 0 && blockIdx.x < 512) {
      unsigned long long g;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(g));
      p.wait_cycles[8 + 4 * blockIdx.x + 2] = (long long)g;   // MMA loop begins (weights resident)
    }
    for (int tcount = issuer; tcount < ntl && ok; tcount += p.nissue) {
      const int acc = tcount % p.nacc;
      const uint32_t acc_ph = (uint32_t)(tcount / p.nacc) & 1u;
      const long long w0 = timing ? clock64() : 0;
      const bool got_acc = tc::mbar_wait(bar_tempty(acc), acc_ph ^ 1u, abort_flag);
      if (timing) wait_acc += clock64() - w0;
      if (!got_acc) {
        if (lane == 0) atomicOr(p.status, kStatWaitTmemEmpty);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_stride);
      for (int step = 0; step < nsteps; ++step) {
        const int s = issuer * p.spi + sl;
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
        // Descriptors of one stage differ only in the start-address field (16-byte units, low word),
        // so a tap costs two integer adds: the issue loop must stay far below the ~50 clocks an MMA
        // of this shape takes, or the tensor pipe starves.
        const uint32_t a_lo0 = stage0_lo + (uint32_t)s * stage_rows;
        const uint32_t b_lo0 = p.resident ? w_lo + (uint32_t)(p.qps * step) * wq_rows
                                          : a_lo0 - a_lbo_field + (a_bytes >> 4) + b_lbo_field;
        const long long w2 = timing ? clock64() : 0;
        if (tc::elect_one()) {
          for (int qq = 0; qq < p.qps; ++qq) {
            const uint32_t a_lo = a_lo0 + (uint32_t)qq * 2u * (uint32_t)rows;
            const uint32_t b_lo = b_lo0 + (uint32_t)qq * wq_rows;
            if (KS > 0) {
#pragma unroll
              for (int tap = 0; tap < KS * KS; ++tap) {
                const int dy = tap / (KS > 0 ? KS : 1) - KS / 2, dx = tap % (KS > 0 ? KS : 1) - KS / 2;
                const uint32_t shift = (uint32_t)(p.halo_rows + dy * p.wp + dx);
                if (PAIR)
                  tc::mma_bf16_pair(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + shift),
                                    ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc,
                                    (step | qq | tap) != 0 ? 1u : 0u);
                else
                  tc::mma_bf16(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + shift),
                               ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc,
                               (step | qq | tap) != 0 ? 1u : 0u);
              }
            } else if (p.stem) {
              // direct stem: tap = (filter row ky, 16-wide kx block hb)
              int tap = 0;
              for (int ky = 0; ky < p.kside; ++ky)
                for (int hb = 0; hb < p.stem_hx; ++hb, ++tap) {
                  const uint32_t shift = (uint32_t)(p.halo_rows + (ky - kh) * p.wp + hb * 16 - kh);
                  if (PAIR)
                    tc::mma_bf16_pair(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + shift),
                                      ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc, (step | tap) != 0 ? 1u : 0u);
                  else
                    tc::mma_bf16(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + shift),
                                 ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc, (step | tap) != 0 ? 1u : 0u);
                }
            } else {
              int tap = 0;
              for (int dy = -kh; dy <= kh; ++dy)
                for (int dx = -kh; dx <= kh; ++dx, ++tap)
                  if (PAIR)
                    tc::mma_bf16_pair(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + (uint32_t)(p.halo_rows + dy * p.wp + dx)),
                                      ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc,
                                      (step | qq | tap) != 0 ? 1u : 0u);
                  else
                    tc::mma_bf16(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + (uint32_t)(p.halo_rows + dy * p.wp + dx)),
                                 ((uint64_t)desc_hi << 32) | (b_lo + (uint32_t)tap * b_step), idesc,
                                 (step | qq | tap) != 0 ? 1u : 0u);
            }
          }
          // stage reusable / accumulator ready once these MMAs have completed (in both CTAs of a pair)
          if (PAIR) {
            tc::mma_commit_pair_both(bar_empty(s));
            if (step == nsteps - 1) tc::mma_commit_pair_both(bar_tfull(acc));
          } else {
            tc::mma_commit(bar_empty(s));
            if (step == nsteps - 1) tc::mma_commit(bar_tfull(acc));
          }
        }
        __syncwarp();
        if (timing) issue_clk += clock64() - w2;
        if (++sl == p.spi) { sl = 0; ph ^= 1u; }
      }
    }
    if (timing && lane == 0) {
      p.wait_cycles[1] += wait_full;
      p.wait_cycles[2] += wait_acc;
      p.wait_cycles[4] += issue_clk;
      p.wait_cycles[5] += clock64() - loop_t0;
    }
    if (TIMED && p.wait_cycles && lane == 0 && issuer == 0 && blockIdx.x < 512) {
      unsigned long long g;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(g));
      p.wait_cycles[8 + 4 * blockIdx.x + 3] = (long long)g;   // MMA loop ends (all MMAs issued)
    }
    // every MMA issued must have retired before TMEM is freed
    if (lane == 0) {
      if (PAIR) tc::mma_commit_pair_local(bar_drain(issuer)); else tc::mma_commit(bar_drain(issuer));
      if (!tc::mbar_wait(bar_drain(issuer), 0, never_flag)) {
        atomicOr(p.status, kStatWaitDrain);
        *abort_flag = 1;
      }
    }
    __syncwarp();
  } else if (PAIR && !leader && warp >= 1 && warp <= 4 && warp - 1 < p.nissue) {
    // ------------------------------ peer relays ------------------------------
    // The leader's issuer i must know when the PEER's copy of a stage has landed: this warp follows
    // ring i of its own CTA and forwards every completed phase to the leader's barrier.
    const int issuer = warp - 1;
    bool ok = true;
    if (issuer == 0 && p.resident) {
      if (tc::mbar_wait_warp(bar_w, 0, abort_flag, 32)) {
        if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar_w, 0));
      } else {
        if (lane == 0) atomicOr(p.status, kStatWaitWeights);
        *abort_flag = 1;
        ok = false;
      }
    }
    int sl = 0;
    uint32_t ph = 0;
    for (int tcount = issuer; tcount < ntl && ok; tcount += p.nissue) {
      for (int step = 0; step < nsteps; ++step) {
        const int s = issuer * p.spi + sl;
        if (!tc::mbar_wait_warp(bar_full(s), ph, abort_flag, 0)) {
          if (lane == 0) atomicOr(p.status, kStatWaitFull);
          *abort_flag = 1;
          ok = false;
          break;
        }
        if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(bar_full(s), 0));
        if (++sl == p.spi) { sl = 0; ph ^= 1u; }
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4 * (p.nacc < kEpiTeams ? p.nacc : kEpiTeams)) {
    // ------------------------------ epilogue ------------------------------
    // Teams of four warps take tiles round robin (team = tile mod nteams; nteams divides the
    // accumulator ring, so an accumulator's barriers always see the same team).  A warp may read TMEM
    // lanes 32*(w%4)..+31 only, so inside a team each warp owns one lane quadrant = 32 positions
    // and all their channels; the accumulator ring (2 or 4 buffers) lets the MMA warp run ahead
    // while both teams are busy.  Per element: h = 0.5*acc + 0.5*bias (one FMA),
    // y = h + h*tanh(h) (one MUFU, one FMA).  On the head layer the thread already holds every
    // channel of its position, so both 1x1 heads reduce inside the thread.
    const bool timing = TIMED && p.wait_cycles != nullptr && blockIdx.x == 0;
    const int quad = warp & 3;
    const int team = (warp - kEpiWarp0) >> 2;
    grid_dep_wait();   // redundant with the producers' wait (no accumulator fills before it); every role that touches global memory orders itself
    const int nteams = p.nacc < kEpiTeams ? p.nacc : kEpiTeams;
    const int row = quad * 32 + lane;
    const int nunits = p.n >> 4;
    bool ok = true;
    unsigned int wait_tfull = 0, ep_ld = 0, ep_math = 0;   // 32-bit clocks: registers are scarce here
    float amax = 0.f;                                      // fp16 mode: largest |activation| this thread stored
    for (int tcount = team; tcount < ntl && ok; tcount += nteams) {
      const int tile = t_first + tcount * t_stride;
      const int acc = tcount % p.nacc;
      const uint32_t acc_ph = (uint32_t)(tcount / p.nacc) & 1u;
      const unsigned int w0 = timing ? (unsigned int)clock() : 0u;
      const bool got = tc::mbar_wait(bar_tfull(acc), acc_ph, abort_flag, kIdleBackoffNs);
      if (timing) wait_tfull += (unsigned int)clock() - w0;
      if (!got) {
        if (lane == 0) atomicOr(p.status, kStatWaitTmemFull);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc::fence_after_sync();
      const unsigned int e0 = timing ? (unsigned int)clock() : 0u;
      unsigned int e1 = e0;
      const int pos = tile_pos(tile) + row;            // position inside the group
      const int board = pos / p.slots, slot = pos - board * p.slots;
      const int r = slot / p.wp, c = slot - r * p.wp;
      const bool valid = board < p.nboards && r < p.bsize && c < p.bsize;
      const uint32_t taddr = tmem_base + (uint32_t)(acc * p.acc_stride) + ((uint32_t)(quad * 32) << 16);
      // plain layers write every position of the tile (zeros into the pad slots); the direct stem walks
      // the input geometry and writes cells only, into the output planes' own geometry
      const bool store = (KS == 0 && p.stem) ? valid : true;
      uint4* out_row = (KS == 0 && p.stem)
                           ? p.out + (long long)p.out_front + (long long)group * p.out_group_pos + (long long)board * p.out_slots + r * p.out_wp + c
                           : p.out + group_row0 + pos;
      float pol = 0.f, val = 0.f;
      // Up to three 16-channel units are fetched from TMEM with one wait so that their latencies
      // overlap; after the last fetch the accumulator goes back to the MMA warp before the
      // arithmetic starts.
      for (int u0 = 0; u0 < nunits; u0 += kEpiBatch) {
        uint32_t v[kEpiBatch][16];
#pragma unroll
        for (int b = 0; b < kEpiBatch; ++b)
          if (u0 + b < nunits) tc::tmem_ld16(taddr + (uint32_t)((u0 + b) * 16), v[b]);
        tc::tmem_wait_ld();
        if (timing && u0 == 0) e1 = (unsigned int)clock();
        if (u0 + kEpiBatch >= nunits) {
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) tc::mbar_arrive_cluster(tc::mapa(bar_tempty(acc), 0)); else tc::mbar_arrive(bar_tempty(acc));
          }
        }
#pragma unroll
        for (int b = 0; b < kEpiBatch; ++b) {
          const int u = u0 + b;
          if (u < nunits) {
            float y[16];
            if (EPI == kEpiSiluSave) {
              // y = silu(z) as in the forward, and silu'(z) = s + z s (1 - s), s = sigmoid(z) = 0.5 + 0.5 tanh(z / 2), from
              // the same tanh; the derivative is stored at once (8 channels at a time: registers are scarce)
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                float d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float h = fmaf(__uint_as_float(v[b][8 * k + j]), 0.5f, s_bias[u * 16 + 8 * k + j]);
                  const float t = tanh_approx(h);
                  y[8 * k + j] = fmaf(h, t, h);
                  const float sg = fmaf(0.5f, t, 0.5f);
                  d[j] = fmaf((h + h) * sg, 1.0f - sg, sg);
                }
                uint4 o2;
                o2.x = valid ? pack_h2<F16>(d[0], d[1]) : 0u;
                o2.y = valid ? pack_h2<F16>(d[2], d[3]) : 0u;
                o2.z = valid ? pack_h2<F16>(d[4], d[5]) : 0u;
                o2.w = valid ? pack_h2<F16>(d[6], d[7]) : 0u;
                if (store) (p.out2 + (out_row - p.out))[(size_t)(u * 2 + k) * p.plane_rows] = o2;
              }
            } else if (EPI != kEpiSilu) {
              // h = z / 2 as in the forward; the backward operators always read the bias from shared memory
              uint4 g[2];
              if (EPI == kEpiDsilu || EPI == kEpiLinearMul) {
                const uint4* aux_row = p.aux + (out_row - p.out);
                g[0] = valid ? aux_row[(size_t)(u * 2) * p.plane_rows] : make_uint4(0, 0, 0, 0);
                g[1] = valid ? aux_row[(size_t)(u * 2 + 1) * p.plane_rows] : make_uint4(0, 0, 0, 0);
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float h = fmaf(__uint_as_float(v[b][j]), 0.5f, s_bias[u * 16 + j]);
                if (EPI == kEpiLinear) {
                  y[j] = h + h;
                } else if (EPI == kEpiLinearMul) {
                  const uint32_t w = reinterpret_cast<const uint32_t*>(g)[j >> 1];
                  y[j] = (h + h) * __uint_as_float((j & 1) ? (w & 0xffff0000u) : (w << 16));
                } else {
                  // silu'(z) = s + z s (1 - s) with s = sigmoid(z) = 0.5 + 0.5 tanh(z / 2)
                  const float sg = fmaf(0.5f, tanh_approx(h), 0.5f);
                  const float d = fmaf((h + h) * sg, 1.0f - sg, sg);
                  const uint32_t w = reinterpret_cast<const uint32_t*>(g)[j >> 1];
                  const float gy = __uint_as_float((j & 1) ? (w & 0xffff0000u) : (w << 16));   // bf16 -> fp32
                  y[j] = gy * d;
                }
              }
            } else if (p.use_const) {
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 hb = reinterpret_cast<const float4*>(p.c_hbias)[u * 4 + j4];
                y[j4 * 4 + 0] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 0]), 0.5f, hb.x));
                y[j4 * 4 + 1] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 1]), 0.5f, hb.y));
                y[j4 * 4 + 2] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 2]), 0.5f, hb.z));
                y[j4 * 4 + 3] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 3]), 0.5f, hb.w));
              }
            } else {
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 hb = *reinterpret_cast<const float4*>(s_bias + u * 16 + j4 * 4);  // 0.5 * bias
                y[j4 * 4 + 0] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 0]), 0.5f, hb.x));
                y[j4 * 4 + 1] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 1]), 0.5f, hb.y));
                y[j4 * 4 + 2] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 2]), 0.5f, hb.z));
                y[j4 * 4 + 3] = silu_from_half(fmaf(__uint_as_float(v[b][j4 * 4 + 3]), 0.5f, hb.w));
              }
            }
            if (p.head) {
              if (p.use_const) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  pol = fmaf(y[j], p.c_wp[u * 16 + j], pol);
                  val = fmaf(y[j], p.c_wv[u * 16 + j], val);
                }
              } else {
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                  const float4 wp4 = *reinterpret_cast<const float4*>(s_wp + u * 16 + j4 * 4);
                  const float4 wv4 = *reinterpret_cast<const float4*>(s_wv + u * 16 + j4 * 4);
                  pol = fmaf(y[j4 * 4 + 0], wp4.x, pol);
                  pol = fmaf(y[j4 * 4 + 1], wp4.y, pol);
                  pol = fmaf(y[j4 * 4 + 2], wp4.z, pol);
                  pol = fmaf(y[j4 * 4 + 3], wp4.w, pol);
                  val = fmaf(y[j4 * 4 + 0], wv4.x, val);
                  val = fmaf(y[j4 * 4 + 1], wv4.y, val);
                  val = fmaf(y[j4 * 4 + 2], wv4.z, val);
                  val = fmaf(y[j4 * 4 + 3], wv4.w, val);
                }
              }
            } else {
              if (F16) {
#pragma unroll
                for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(y[j]));
              }
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                uint4 o;
                o.x = valid ? pack_h2<F16>(y[8 * k + 0], y[8 * k + 1]) : 0u;
                o.y = valid ? pack_h2<F16>(y[8 * k + 2], y[8 * k + 3]) : 0u;
                o.z = valid ? pack_h2<F16>(y[8 * k + 4], y[8 * k + 5]) : 0u;
                o.w = valid ? pack_h2<F16>(y[8 * k + 6], y[8 * k + 7]) : 0u;
                if (store) out_row[(size_t)(u * 2 + k) * p.plane_rows] = o;
              }
            }
          }
        }
      }
      if (p.head) {
        const long long o = (long long)group * p.group_pos + pos;
        p.logit_raw[o] = valid ? pol : 0.f;
        p.vmap[o] = valid ? val : 0.f;
      }
      if (timing) {
        ep_ld += e1 - e0;            // first TMEM fetch: issue to data
        ep_math += (unsigned int)clock() - e1;   // release + arithmetic + stores (+ later fetches)
      }
    }
    if (F16 && !(amax <= 65504.f)) atomicOr(p.status, kStatF16Range);
    if (timing && threadIdx.x == 32 * kEpiWarp0) {
      p.wait_cycles[3] += wait_tfull;
      p.wait_cycles[6] += ep_ld;     // first TMEM fetch of each tile: issue to data
      p.wait_cycles[7] += ep_math;   // arithmetic + stores (+ later fetches)
    }
  }

  tc::fence_before_sync();
  if (PAIR) tc::cluster_sync(); else __syncthreads();   // the peer's shared memory outlives the leader's MMAs
  if (TIMED && p.wait_cycles && threadIdx.x == 0 && blockIdx.x < 512) {
    unsigned long long gt_end;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt_end));
    p.wait_cycles[8 + 4 * blockIdx.x] = (long long)gt_start;       // ns timestamps of this CTA
    p.wait_cycles[8 + 4 * blockIdx.x + 1] = (long long)gt_end;
  }
  if (warp == 1) {
    __syncwarp();
    tc::fence_after_sync();
    if (PAIR) tc::tmem_dealloc2(tmem_base, (uint32_t)p.tmem_cols); else tc::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace c6
