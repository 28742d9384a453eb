/*
 * c6_env.h -- C ABI of the vectorised Connect6 environment step on the GPU.
 *
 * The reference project (mgxmateusz/connect6) steps its environments with some thirty small
 * PyTorch kernels and three host synchronisations per self-play step
 * (connect6/vector_env.py:106-193, connect6/train.py:866-941).  The entry points below do the same
 * integer work in one or two launches each, in place, on the reference's own state tensors.
 * Same conventions as c6_engine.h: extern "C", plain DEVICE pointers and sizes, int status
 * (0 = C6_OK), work enqueued on the stream handed in (a cudaStream_t passed as void*), no
 * synchronisation, no allocation.  Results are bit-identical to the reference's.
 */
#ifndef C6_ENV_H_
#define C6_ENV_H_

#include <stdint.h>

#include "c6_engine.h" /* status codes */

#ifdef __cplusplus
extern "C" {
#endif

/* The state tensors of VectorConnect6 (connect6/vector_env.py:34-53), owned by the caller. */
typedef struct C6EnvState {
  int8_t* boards;          /* [num_envs, n, n]: +1 black, -1 white, 0 empty */
  int8_t* current_player;  /* [num_envs]: +1 / -1                           */
  int8_t* stones_left;     /* [num_envs]: stones left in the current turn   */
  int16_t* empty_count;    /* [num_envs]                                    */
  int16_t* move_count;     /* [num_envs]                                    */
  int64_t num_envs;
  int32_t board_size;      /* n, 1..127                                     */
  int32_t win_length;      /* stones in a row that win (6), 1..n            */
} C6EnvState;

/* Per-environment bookkeeping of the rollout collector (connect6/train.py:702-721), owned by
 * the caller. */
typedef struct C6CollectorState {
  int32_t* current_episode_ids;       /* [num_envs]                                           */
  int32_t* current_segment_lengths;   /* [num_envs]                                           */
  const uint8_t* historical_mask;     /* nullable [num_envs] bool: table plays an old model   */
  int8_t* historical_current_colors;  /* nullable [num_envs]: colour the current model holds  */
  int8_t* episode_results;            /* [episode_capacity]: winner per finished episode      */
  int16_t* episode_terminal_moves;    /* [episode_capacity]: length per finished episode      */
  int64_t episode_capacity;
  int64_t* next_episode_id;           /* device scalar, read and advanced by the call         */
} C6CollectorState;

/* slots of the fault counters written by c6_env_step and c6_env_collect_done */
enum {
  C6_ENV_FAULT_OCCUPIED = 0,  /* stones placed on an occupied cell (debug_checks, vector_env.py:121-127) */
  C6_ENV_FAULT_ACTION = 1,    /* actions outside [0, n*n): that environment was left untouched          */
  C6_ENV_FAULT_EPISODE = 2,   /* episode ids outside [0, episode_capacity): that record was skipped     */
  C6_ENV_FAULT_COUNT = 4
};

/* slots of the statistics vector of c6_env_collect_done: the reference's batch_stats
 * (connect6/train.py:888-900) followed by the number of finished environments */
enum {
  C6_STAT_SEGMENT_LENGTHS = 0, C6_STAT_BLACK_WINS = 1, C6_STAT_WHITE_WINS = 2, C6_STAT_DRAWS = 3,
  C6_STAT_GAME_LENGTHS = 4, C6_STAT_HIST_GAMES = 5, C6_STAT_HIST_WINS = 6, C6_STAT_HIST_LOSSES = 7,
  C6_STAT_HIST_DRAWS = 8, C6_STAT_DONE_COUNT = 9, C6_STAT_COUNT = 10
};

/* Replaces: VectorConnect6.step + _check_win_local (connect6/vector_env.py:106-193), and, when
 * view_phase != 0, the _inverse_transform_actions call in front of it (connect6/train.py:255-277,
 * 846-853): actions are then cell indices inside D4 view `view_phase` (0..7) and are mapped back
 * to board coordinates first.  actions int64 [num_envs].  Outputs, all [num_envs]: reward fp32,
 * done bool (one byte), winner int8, transition_sign int8, game_lengths int16.  faults: nullable
 * int32 [C6_ENV_FAULT_COUNT], counters that the call only ever increments. */
int c6_env_step(const C6EnvState* env, const int64_t* actions, int32_t view_phase, float* reward,
                uint8_t* done, int8_t* winner, int8_t* transition_sign, int16_t* game_lengths,
                int32_t* faults, void* stream);

/* Replaces: VectorConnect6.reset (connect6/vector_env.py:77-92).  indices nullable int64 [count]:
 * null resets every environment (count ignored); entries outside [0, num_envs) are skipped. */
int c6_env_reset(const C6EnvState* env, const int64_t* indices, int64_t count, void* stream);

/* Replaces: VectorConnect6.legal_mask (connect6/vector_env.py:94-95): out bool [num_envs, n*n]. */
int c6_env_legal_mask(const C6EnvState* env, uint8_t* out, void* stream);

/* Bytes of scratch c6_env_collect_done needs for num_envs environments (no initialisation
 * needed; contents are overwritten by every call). */
int64_t c6_env_collect_workspace_bytes(int64_t num_envs);

/* Replaces: the finished-game bookkeeping of the rollout collector (connect6/train.py:866-941):
 * done_idx = nonzero(done) in ascending order; winners and game lengths recorded per episode id;
 * the nine sums of batch_stats; reset of the finished environments and of their segment lengths;
 * new episode ids next_episode_id + rank in done_idx; colour swap of finished historical tables.
 * done / winner / game_lengths are c6_env_step's outputs.  done_idx int64 [num_envs] (first
 * stats[C6_STAT_DONE_COUNT] entries written); stats int64 [C6_STAT_COUNT] overwritten; nothing is
 * copied to the host: the caller reads stats when it chooses to.  faults as for c6_env_step. */
int c6_env_collect_done(const C6EnvState* env, const C6CollectorState* col, const uint8_t* done,
                        const int8_t* winner, const int16_t* game_lengths, int64_t* done_idx,
                        int64_t* stats, int32_t* faults, void* workspace, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* C6_ENV_H_ */
