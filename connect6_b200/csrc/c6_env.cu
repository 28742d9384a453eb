// Vectorised Connect6 environment step, reset and finished-game bookkeeping (C ABI of c6_env.h).
//
// Integer work, a few dozen bytes per environment: every kernel is bound by launch latency and by
// scattered 32-byte sector reads, not by arithmetic.  One thread owns one environment in the step
// kernel (its 4 x (2*win-2) probe cells live in that environment's own 361-byte board); the
// bookkeeping uses one launch to count finished environments per block and one to rank them
// (stable, ascending environment index, like torch.nonzero), record, reset and renumber them.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/c6_env.h"
#include "c6_common.cuh"

namespace c6 {
namespace {

constexpr int kEnvThreads = 256;
constexpr int kStepThreads = 64;  // small blocks: 8192 environments still spread over 128 SMs

struct EnvView {
  int8_t* boards;
  int8_t* player;
  int8_t* stones;
  int16_t* empty;
  int16_t* moves;
  long long E;
  int n;
  int win;
};

// number of consecutive stones of `who` starting one cell away from (r, c) in direction (dr, dc),
// at most win - 1 (connect6/vector_env.py:166-193: cumulative product over the near-to-far matches)
__device__ __forceinline__ int run_length(const int8_t* __restrict__ b, int n, int win, int r, int c, int dr, int dc,
                                          int who) {
  int k = 0;
  for (int s = 1; s < win; ++s) {
    const int rr = r + dr * s, cc = c + dc * s;
    if (rr < 0 || rr >= n || cc < 0 || cc >= n || b[rr * n + cc] != who) break;
    ++k;
  }
  return k;
}

__global__ void __launch_bounds__(kStepThreads)
env_step_kernel(EnvView s, const long long* __restrict__ actions, int phase, float* __restrict__ reward,
                uint8_t* __restrict__ done, int8_t* __restrict__ winner, int8_t* __restrict__ tsign,
                int16_t* __restrict__ lengths, int* __restrict__ faults) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= s.E) return;
  const int n = s.n, cells = n * n;
  const long long raw = actions[e];
  if (raw < 0 || raw >= cells) {
    if (faults) atomicAdd(faults + C6_ENV_FAULT_ACTION, 1);
    reward[e] = 0.f; done[e] = 0; winner[e] = 0; tsign[e] = 0; lengths[e] = s.moves[e];
    return;
  }
  const int a = phase ? d4_inverse((int)raw, n, phase) : (int)raw;
  const int r = a / n, c = a - r * n;
  int8_t* b = s.boards + e * cells;
  const int actor = s.player[e];
  if (faults && b[a] != 0) atomicAdd(faults + C6_ENV_FAULT_OCCUPIED, 1);
  b[a] = (int8_t)actor;
  const int16_t empty = (int16_t)(s.empty[e] - 1);
  const int16_t moves = (int16_t)(s.moves[e] + 1);
  s.empty[e] = empty;
  s.moves[e] = moves;

  bool won = false;
  const int dirs[4][2] = {{1, 0}, {0, 1}, {1, 1}, {1, -1}};
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    const int total = 1 + run_length(b, n, s.win, r, c, dirs[d][0], dirs[d][1], actor) +
                      run_length(b, n, s.win, r, c, -dirs[d][0], -dirs[d][1], actor);
    won |= total >= s.win;
  }
  const bool over = won || empty == 0;
  int sign = 0;
  if (!over) {
    const int remaining = (int8_t)(s.stones[e] - 1);
    if (remaining > 0) {
      s.stones[e] = (int8_t)remaining;
      sign = 1;
    } else {
      s.player[e] = (int8_t)(-actor);
      s.stones[e] = 2;
      sign = -1;
    }
  }
  reward[e] = won ? 1.f : 0.f;
  done[e] = over ? 1 : 0;
  winner[e] = won ? (int8_t)actor : (int8_t)0;
  tsign[e] = (int8_t)sign;
  lengths[e] = moves;
}

__device__ __forceinline__ void reset_scalars(const EnvView& s, long long e) {
  s.player[e] = 1;
  s.stones[e] = 1;
  s.empty[e] = (int16_t)(s.n * s.n);
  s.moves[e] = 0;
}

// one thread per (selected environment, cell)
__global__ void __launch_bounds__(kEnvThreads)
env_reset_kernel(EnvView s, const long long* __restrict__ indices, long long count) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cells = s.n * s.n;
  if (i >= count * cells) return;
  const long long k = i / cells;
  const int cell = (int)(i - k * cells);
  const long long e = indices ? indices[k] : k;
  if (e < 0 || e >= s.E) return;
  s.boards[e * cells + cell] = 0;
  if (cell == 0) reset_scalars(s, e);
}

__global__ void __launch_bounds__(kEnvThreads)
env_legal_mask_kernel(const int8_t* __restrict__ boards, long long total, uint8_t* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = boards[i] == 0 ? 1 : 0;
}

// ---- finished-game bookkeeping ------------------------------------------------------------------
// scratch: [0] episode id base of this call, [1 ...] finished environments per block
struct CollectScratch {
  long long* base_id;
  int* counts;
};

__device__ __forceinline__ CollectScratch scratch_of(void* ws) {
  return CollectScratch{reinterpret_cast<long long*>(ws), reinterpret_cast<int*>(reinterpret_cast<long long*>(ws) + 1)};
}

__global__ void __launch_bounds__(kEnvThreads)
env_done_count_kernel(const uint8_t* __restrict__ done, long long E, const long long* __restrict__ next_episode_id,
                      long long* __restrict__ stats, void* ws) {
  const CollectScratch sc = scratch_of(ws);
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int n = __syncthreads_count(e < E && done[e] != 0);
  if (threadIdx.x == 0) sc.counts[blockIdx.x] = n;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) *sc.base_id = *next_episode_id;
    if (threadIdx.x < C6_STAT_COUNT) stats[threadIdx.x] = 0;
  }
}

struct CollectorView {
  int* episode_ids;
  int* segment_lengths;
  const uint8_t* hist_mask;
  int8_t* hist_colors;
  int8_t* results;
  int16_t* terminal_moves;
  long long capacity;
  long long* next_episode_id;
};

__global__ void __launch_bounds__(kEnvThreads)
env_done_apply_kernel(EnvView s, CollectorView col, const uint8_t* __restrict__ done, const int8_t* __restrict__ winner,
                      const int16_t* __restrict__ lengths, long long* __restrict__ done_idx,
                      long long* __restrict__ stats, int* __restrict__ faults, void* ws) {
  const CollectScratch sc = scratch_of(ws);
  __shared__ long long s_before, s_total;
  __shared__ unsigned long long s_stats[C6_STAT_DONE_COUNT];
  __shared__ int s_warp[kEnvThreads / 32];
  __shared__ int s_list[kEnvThreads];
  __shared__ int s_nlist;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s_before = 0; s_total = 0; s_nlist = 0; }
  if (tid < C6_STAT_DONE_COUNT) s_stats[tid] = 0;
  __syncthreads();
  // finished environments in the blocks before this one, and in all blocks
  long long before = 0, total = 0;
  for (int b = tid; b < (int)gridDim.x; b += kEnvThreads) {
    const int n = sc.counts[b];
    total += n;
    if (b < (int)blockIdx.x) before += n;
  }
  for (int o = 16; o; o >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, o);
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  if (lane == 0 && total) {
    atomicAdd(reinterpret_cast<unsigned long long*>(&s_total), (unsigned long long)total);
    atomicAdd(reinterpret_cast<unsigned long long*>(&s_before), (unsigned long long)before);
  }
  // rank of this thread's environment among the finished ones of the block
  const long long e = (long long)blockIdx.x * kEnvThreads + tid;
  const bool fin = e < s.E && done[e] != 0;
  const unsigned ballot = __ballot_sync(0xffffffffu, fin);
  if (lane == 0) s_warp[warp] = __popc(ballot);
  __syncthreads();
  int rank = __popc(ballot & ((1u << lane) - 1u));
  for (int w = 0; w < warp; ++w) rank += s_warp[w];
  const long long base = *sc.base_id;
  if (fin) {
    const long long r = s_before + rank;
    done_idx[r] = e;
    const int id = col.episode_ids[e];
    const int w = winner[e];
    const int len = lengths[e];
    if (id >= 0 && id < col.capacity) {
      col.results[id] = (int8_t)w;
      col.terminal_moves[id] = (int16_t)len;
    } else if (faults) {
      atomicAdd(faults + C6_ENV_FAULT_EPISODE, 1);
    }
    const bool hist = col.hist_mask && col.hist_mask[e] != 0;
    const int colour = hist ? col.hist_colors[e] : 0;
    atomicAdd(&s_stats[C6_STAT_SEGMENT_LENGTHS], (unsigned long long)(long long)col.segment_lengths[e]);
    atomicAdd(&s_stats[w == 1 ? C6_STAT_BLACK_WINS : (w == -1 ? C6_STAT_WHITE_WINS : C6_STAT_DRAWS)], 1ull);
    atomicAdd(&s_stats[C6_STAT_GAME_LENGTHS], (unsigned long long)(long long)len);
    if (hist) {
      atomicAdd(&s_stats[C6_STAT_HIST_GAMES], 1ull);
      if (w == colour) atomicAdd(&s_stats[C6_STAT_HIST_WINS], 1ull);
      if (w == -colour) atomicAdd(&s_stats[C6_STAT_HIST_LOSSES], 1ull);
      if (w == 0) atomicAdd(&s_stats[C6_STAT_HIST_DRAWS], 1ull);
      col.hist_colors[e] = (int8_t)(-colour);
    }
    col.segment_lengths[e] = 0;
    col.episode_ids[e] = (int)(base + r);
    reset_scalars(s, e);
    s_list[atomicAdd(&s_nlist, 1)] = tid;
  }
  __syncthreads();
  // the whole block clears the boards of its finished environments
  const int cells = s.n * s.n;
  for (int k = 0; k < s_nlist; ++k) {
    int8_t* b = s.boards + ((long long)blockIdx.x * kEnvThreads + s_list[k]) * cells;
    for (int c = tid; c < cells; c += kEnvThreads) b[c] = 0;
  }
  if (tid < C6_STAT_DONE_COUNT && s_stats[tid])
    atomicAdd(reinterpret_cast<unsigned long long*>(stats) + tid, s_stats[tid]);
  if (blockIdx.x == 0 && tid == 0) {
    stats[C6_STAT_DONE_COUNT] = s_total;
    *col.next_episode_id = base + s_total;
  }
}

bool env_ok(const C6EnvState* env) {
  return env && env->num_envs >= 0 && env->board_size >= 1 && env->board_size <= 127 && env->win_length >= 1 &&
         env->win_length <= env->board_size &&
         (env->num_envs == 0 ||
          (env->boards && env->current_player && env->stones_left && env->empty_count && env->move_count));
}

EnvView view_of(const C6EnvState* env) {
  return EnvView{env->boards, env->current_player, env->stones_left, env->empty_count, env->move_count,
                 (long long)env->num_envs, env->board_size, env->win_length};
}

unsigned blocks_for(long long items) { return (unsigned)((items + kEnvThreads - 1) / kEnvThreads); }

int launched() { return cudaGetLastError() == cudaSuccess ? C6_OK : C6_ERR_CUDA; }

}  // namespace
}  // namespace c6

using namespace c6;

extern "C" {

int c6_env_step(const C6EnvState* env, const int64_t* actions, int32_t view_phase, float* reward, uint8_t* done,
                int8_t* winner, int8_t* transition_sign, int16_t* game_lengths, int32_t* faults, void* stream) {
  if (!env_ok(env) || view_phase < 0 || view_phase > 7) return C6_ERR_ARG;
  if (env->num_envs == 0) return C6_OK;
  if (!actions || !reward || !done || !winner || !transition_sign || !game_lengths) return C6_ERR_ARG;
  env_step_kernel<<<(unsigned)((env->num_envs + kStepThreads - 1) / kStepThreads), kStepThreads, 0,
                    reinterpret_cast<cudaStream_t>(stream)>>>(
      view_of(env), reinterpret_cast<const long long*>(actions), view_phase, reward, done, winner, transition_sign,
      game_lengths, faults);
  return launched();
}

int c6_env_reset(const C6EnvState* env, const int64_t* indices, int64_t count, void* stream) {
  if (!env_ok(env) || (indices && count < 0)) return C6_ERR_ARG;
  const long long k = indices ? count : env->num_envs;
  if (k == 0) return C6_OK;
  const long long cells = (long long)env->board_size * env->board_size;
  env_reset_kernel<<<blocks_for(k * cells), kEnvThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      view_of(env), reinterpret_cast<const long long*>(indices), k);
  return launched();
}

int c6_env_legal_mask(const C6EnvState* env, uint8_t* out, void* stream) {
  if (!env_ok(env)) return C6_ERR_ARG;
  if (env->num_envs == 0) return C6_OK;
  if (!out) return C6_ERR_ARG;
  const long long total = env->num_envs * env->board_size * env->board_size;
  env_legal_mask_kernel<<<blocks_for(total), kEnvThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(env->boards,
                                                                                                      total, out);
  return launched();
}

int64_t c6_env_collect_workspace_bytes(int64_t num_envs) {
  if (num_envs < 0) return 0;
  return 8 + 4 * (int64_t)((num_envs + kEnvThreads - 1) / kEnvThreads) + 8;
}

int c6_env_collect_done(const C6EnvState* env, const C6CollectorState* col, const uint8_t* done, const int8_t* winner,
                        const int16_t* game_lengths, int64_t* done_idx, int64_t* stats, int32_t* faults,
                        void* workspace, void* stream) {
  if (!env_ok(env) || !col || !stats || !workspace) return C6_ERR_ARG;
  if (!col->next_episode_id || col->episode_capacity < 0) return C6_ERR_ARG;
  if (col->historical_mask && !col->historical_current_colors) return C6_ERR_ARG;
  if (env->num_envs > 0 && (!done || !winner || !game_lengths || !done_idx || !col->current_episode_ids ||
                            !col->current_segment_lengths || !col->episode_results || !col->episode_terminal_moves))
    return C6_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 7) != 0) return C6_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = env->num_envs ? blocks_for(env->num_envs) : 1u;
  env_done_count_kernel<<<blocks, kEnvThreads, 0, st>>>(done, env->num_envs, reinterpret_cast<long long*>(col->next_episode_id),
                                                        reinterpret_cast<long long*>(stats), workspace);
  if (cudaGetLastError() != cudaSuccess) return C6_ERR_CUDA;
  const CollectorView cv{col->current_episode_ids, col->current_segment_lengths, col->historical_mask,
                         col->historical_current_colors, col->episode_results, col->episode_terminal_moves,
                         (long long)col->episode_capacity, reinterpret_cast<long long*>(col->next_episode_id)};
  env_done_apply_kernel<<<blocks, kEnvThreads, 0, st>>>(view_of(env), cv, done, winner, game_lengths,
                                                        reinterpret_cast<long long*>(done_idx),
                                                        reinterpret_cast<long long*>(stats), faults, workspace);
  return launched();
}

}  // extern "C"
