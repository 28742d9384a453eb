/*
 * c6_debug.h -- development and test aids of the engine library, kept apart from the product ABI
 * of c6_engine.h.  None of them has a counterpart in the reference project.  Same conventions:
 * extern "C", int status, device pointers unless a parameter is documented as host memory.
 */
#ifndef C6_DEBUG_H_
#define C6_DEBUG_H_

#include <stdint.h>

#include "c6_engine.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Test aid with no reference function of its own: runs the backbone up to and including
 * `layer` and writes that layer's activation, SiLU applied (the `features` tensor inside the
 * loop at connect6/model.py:104-106), as fp32 [G*T, channels[layer], n, n].  T is limited to
 * one internal pass. */
int c6_debug_layer_output(C6Engine* eng, const void* x, int x_dtype, int64_t T,
                          const uint8_t* orient, int layer, float* out_nchw, void* stream);

/* Diagnostic with no reference counterpart, available when the library was built with -DC6_TIMED_BUILD
 * (C6_ERR_UNSUPPORTED otherwise; the default build carries no clock counters in its kernels): while
 * profiling level 2 is enabled, CTA 0 of every k x k
 * tensor-core conv launch adds SM clocks to eight device counters: {producer waiting for an empty
 * stage, MMA warp waiting for a full stage, MMA warp waiting for a drained accumulator, epilogue
 * waiting for a ready accumulator, MMA warp inside its issue blocks, MMA warp loop total, 0, 0}.
 * Copies them to the HOST array out8 (synchronous) and optionally clears them. */
int c6_debug_wait_cycles(C6Engine* eng, int64_t* out8, int reset);

/* Diagnostic: four global-timer stamps (ns) per CTA {kernel entry, kernel exit, MMA loop begin,
 * MMA loop end} for the first n_ctas (<= 512) CTAs of the most recent k x k conv launch made
 * while profiling was enabled; HOST array of 4*n_ctas. */
int c6_debug_cta_times(C6Engine* eng, int64_t* out, int n_ctas);

/* Self-test of the failure path, no reference counterpart: enqueues a one-CTA kernel that waits, with
 * a limit of about half a millisecond, on a barrier nobody arrives on, through the same wait helper the
 * tensor-core kernels use.  The wait runs out, the waiter sets its status bit and the CTA's abort flag, a
 * second waiter sees the flag and leaves too, and the kernel returns normally -- the path a real kernel
 * takes if its pipeline stalls.
 * Nothing faults or hangs; c6_status then reports C6_ERR_DEVICE until c6_clear_status. */
int c6_debug_expire_wait(C6Engine* eng, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* C6_DEBUG_H_ */
