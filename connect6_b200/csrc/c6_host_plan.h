// Host-side helpers shared by the translation units of the library: the pipeline plan of one
// tensor-core layer (what fits the 227 KB of shared memory and the 512 TMEM columns) and the launch
// wrapper for 2-CTA clusters / programmatic dependent launch.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>

#include "c6_conv_tc.cuh"

namespace c6 {

constexpr int kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory per CTA on sm_100
constexpr int kVersion = 10100;
#ifdef C6_TIMED_BUILD
constexpr bool kTimedBuild = true;    // the clock-counter instantiations of the k x k kernel are compiled in
#else
constexpr bool kTimedBuild = false;
#endif


inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline long long round_up_ll(long long v, long long m) { return (v + m - 1) / m * m; }
inline int pow2_ceil(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

struct LayerPlan {
  int k = 0, cin = 0, cout = 0, cin_p = 0, cout_p = 0;
  // tensor-core plan (layers >= 1)
  int resident = 0, nstages = 0, smem = 0, acc_stride = 0, tmem_cols = 0, nacc = 2, nissue = 1, spi = 2, qps = 2;
  int pair = 0;                 // run as 2-CTA clusters (cta_group::2)
  size_t w_rows_per_group = 0;  // 16-byte rows of packed weights per group
};


// Launch with optional 2-CTA clusters and optional programmatic dependent launch (the kernel then
// orders itself behind its predecessor with grid_dep_wait(), so its prologue -- barrier setup, TMEM
// allocation, resident weights -- overlaps the predecessor's tail).
template <typename Params>
inline void launch_chain(void (*kernel)(Params), unsigned grid_x, unsigned grid_y, unsigned threads, size_t smem,
                  cudaStream_t st, bool cluster2, bool dependent, const Params& p) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid_x, grid_y);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (cluster2) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = 2;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  if (dependent) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = (unsigned)n;
  cudaLaunchKernelEx(&cfg, kernel, p);
}


// Pipeline shape of one tensor-core layer: `taps` MMAs per 16-channel group, `nq` groups, `rows` staged
// rows per activation plane, `planes_per_q` planes per group (2; the direct stem: 1), steps of up to
// `max_qps` groups.  Prefers resident weights and wide steps; every MMA issuer (up to one per two
// accumulators, at most 4) needs a private ring of at least 2 stages.  False when nothing fits.
inline bool plan_tc_layer(bool pair_mode, LayerPlan& p, int taps, int nq, int rows, int planes_per_q, int max_qps) {
  const int budget = kSmemLimit - 128 - kConvSmemHeader;
  const long long wq = (long long)taps * 2 * p.cout_p * 16;
  const long long wb = wq * nq;
  p.w_rows_per_group = (size_t)(wb / 16);
  p.acc_stride = pow2_ceil(p.cout_p);
  p.nacc = std::min(kMaxAcc, 512 / p.acc_stride);  // 512 TMEM columns in total: 8, 4 or 2 accumulators
  p.tmem_cols = p.nacc * p.acc_stride;
  p.pair = 0;
  const int want = std::max(1, std::min(p.nacc / 2, 4));   // two accumulators per issuer
  // First choice: CTA pairs with resident weights (each CTA keeps half of the rows).
  if (pair_mode) {
    for (int qps = max_qps; qps >= 1; --qps) {
      const long long stage = round_up_ll((long long)planes_per_q * qps * rows * 16, 128);
      const long long fixed = round_up_ll(wb / 2, 128);
      if (fixed + 2LL * want * stage > budget) continue;
      const int ns = (int)std::min<long long>(kMaxStages, (budget - fixed) / stage);
      p.pair = 1;
      p.resident = 1;
      p.qps = qps;
      p.nissue = want;
      p.spi = std::min(4, ns / want);
      p.nstages = p.nissue * p.spi;
      p.smem = 128 + kConvSmemHeader + (int)fixed + p.nstages * (int)stage;
      return true;
    }
  }
  for (int resident = 1; resident >= 0; --resident) {
    for (int qps = max_qps; qps >= 1; --qps) {
      const long long a_bytes = (long long)planes_per_q * qps * rows * 16;
      const long long stage = round_up_ll(a_bytes + (resident ? 0 : qps * wq), 128);
      const long long fixed = resident ? round_up_ll(wb, 128) : 0;
      if (fixed + 2 * stage > budget) continue;
      const int ns = (int)std::min<long long>(kMaxStages, (budget - fixed) / stage);
      if (qps == 2 && ns < 2 * want && resident) {
        // smaller steps may buy enough stages for all issuers: try qps = 1 first
        const long long stage1 = round_up_ll((long long)planes_per_q * rows * 16, 128);
        if ((budget - fixed) / stage1 >= 2 * want) continue;
      }
      int nissue = want;
      while (nissue > 1 && ns < 2 * nissue) nissue >>= 1;
      p.resident = resident;
      p.qps = qps;
      p.nissue = nissue;
      p.spi = std::min(3, ns / nissue);
      p.nstages = p.nissue * p.spi;
      p.smem = 128 + kConvSmemHeader + (int)fixed + p.nstages * (int)stage;
      return true;
    }
  }
  return false;
}


}  // namespace c6
