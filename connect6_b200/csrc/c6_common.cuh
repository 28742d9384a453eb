// Shared device helpers: D4 index maps, Philox4x32-10, SiLU, bf16 packing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace c6 {

constexpr float kFp32Min = -3.4028234663852886e38f;  // torch.finfo(torch.float32).min

// device status bits (engine status word)
constexpr int kStatWaitFull = 1;      // consumer wait on a "stage full" barrier ran out
constexpr int kStatWaitEmpty = 2;     // producer wait on a "stage empty" barrier ran out
constexpr int kStatWaitTmemFull = 4;  // epilogue wait on accumulator-ready ran out
constexpr int kStatWaitTmemEmpty = 8; // MMA wait on accumulator-drained ran out
constexpr int kStatWaitWeights = 16;  // wait on resident-weights barrier ran out
constexpr int kStatWaitDrain = 32;    // final drain wait ran out
constexpr int kStatBadIndex = 64;     // a gather index pointed outside [0, num_envs): that board was read as empty
constexpr int kStatF16Range = 128;    // fp16 mode: an activation exceeded the fp16 range and was clamped to +-65504

// ---- D4 maps (connect6/train.py:216-277) ------------------------------------------
// phase p in 0..7 -> k = p % 4 quarter turns (counter-clockwise), mirror columns if p >= 4.

// canonical cell index -> index of the same cell inside view `phase`
__host__ __device__ __forceinline__ int d4_forward(int a, int n, int phase) {
  int r = a / n, c = a - r * n;
  const int k = phase & 3;
  int r2 = r, c2 = c;
  if (k == 1) { r2 = n - 1 - c; c2 = r; }
  else if (k == 2) { r2 = n - 1 - r; c2 = n - 1 - c; }
  else if (k == 3) { r2 = c; c2 = n - 1 - r; }
  if (phase & 4) c2 = n - 1 - c2;
  return r2 * n + c2;
}

// view cell index -> canonical cell index (undo the mirror first, then the rotation)
__host__ __device__ __forceinline__ int d4_inverse(int a, int n, int phase) {
  int r = a / n, c = a - r * n;
  const int k = phase & 3;
  if (phase & 4) c = n - 1 - c;
  int r2 = r, c2 = c;
  if (k == 1) { r2 = c; c2 = n - 1 - r; }
  else if (k == 2) { r2 = n - 1 - r; c2 = n - 1 - c; }
  else if (k == 3) { r2 = n - 1 - c; c2 = r; }
  return r2 * n + c2;
}

// ---- Philox4x32-10 ------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// The single uniform in [0,1) drawn for one board of one self-play step.
__device__ __forceinline__ float board_uniform(uint64_t seed, uint64_t offset, uint64_t board) {
  const uint4 ctr = make_uint4((uint32_t)board, (uint32_t)(board >> 32), (uint32_t)offset,
                               (uint32_t)(offset >> 32));
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const uint4 r = philox4x32_10(ctr, key);
  return (float)(r.x >> 8) * (1.0f / 16777216.0f);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may start while its predecessor in the stream still runs; grid_dep_wait() blocks until
// the predecessor has completed and its writes are visible (a no-op for an ordinary launch).
// grid_dep_launch() lets the successor's CTAs take over SMs as this grid's CTAs exit.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- activations ----------------------------------------------------------------------
// SiLU through the hardware tanh: x*sigmoid(x) = h + h*tanh(h) with h = x/2.  One MUFU and two
// FMAs per element when the caller folds the bias into h.  tanh.approx.f32 is accurate to about
// 2^-11 relative, well below the bf16 rounding applied to the result.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float silu_from_half(float h) { return fmaf(h, tanh_approx(h), h); }
__device__ __forceinline__ float silu_exact(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// fp16 pair, round to nearest even; values beyond the fp16 range become +-65504 instead of infinity
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// The 16-bit operand type of a tensor-core engine: bf16 (8-bit significand, fp32's exponent range) or
// fp16 (11-bit significand, range +-65504).
template <bool F16>
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  return F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi, int f16) {
  return f16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}
// value -> 16-bit operand type -> float (what the tensor cores will see)
__device__ __forceinline__ float round_h(float v, int f16) {
  return f16 ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float load_x(const void* x, int x_bf16, int64_t idx) {
  return x_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[idx])
                : reinterpret_cast<const float*>(x)[idx];
}

// Where the network input comes from: float planes [B,3,n,n] (the reference's model(x) argument), or
// the environment's raw state -- int8 boards (+1/-1/0), current player, stones left, optionally
// gathered through an index vector -- from which the three planes are derived on the fly
// (connect6/vector_env.py:196-218, gathers of connect6/train.py:793).
struct InputSrc {
  const void* x;             // planes, or null in board mode
  int x_bf16;
  const int8_t* boards;      // [envs, n, n]
  const int8_t* player;      // [envs]
  const int8_t* stones_left; // [envs]
  const long long* index;    // nullable [B]: board b of the batch is environment index[b]
  long long num_envs;        // environments behind `boards`: an index outside [0, num_envs) reads as an empty board
};

// environment of batch board b, or -1 when its index entry lies outside the state tensors
__device__ __forceinline__ long long input_env(const InputSrc& in, long long b) {
  const long long e = in.index ? in.index[b] : b;
  return (e >= 0 && e < in.num_envs) ? e : -1;
}

__device__ __forceinline__ float input_value(const InputSrc& in, long long b, int ci, int cell, int cells) {
  if (in.boards == nullptr) return load_x(in.x, in.x_bf16, (b * 3 + ci) * cells + cell);
  const long long e = input_env(in, b);
  if (e < 0) return 0.f;   // never dereferenced: the pack kernel records kStatBadIndex for it
  if (ci == 2) return in.stones_left[e] == 1 ? 1.f : 0.f;
  const int v = in.boards[e * cells + cell], me = in.player[e];
  return (ci == 0 ? v == me : v == -me) ? 1.f : 0.f;
}

}  // namespace c6
