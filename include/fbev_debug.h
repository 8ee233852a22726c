/*
 * fbev_debug.h - experiment and test helpers of libfbev.so.  Not part of the operator's interface: a binding
 * that only replaces the reference operator needs fbev.h alone.
 */
#ifndef FBEV_DEBUG_H_
#define FBEV_DEBUG_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Launch tuning for experiments and tests, per host thread (a launch reads what its own thread set; other
 * threads are not affected): cells per tile in x and y, 16-byte chunks per
 * lane, warps per block, and a selector (last argument); 0 = choose automatically.  Selector values:
 *   2  forward compiled for two resident blocks per SM (128 registers) instead of three
 *   3  forward (two chunks per lane) compiled for five resident blocks of four warps (96 registers) instead of six
 *   1  feature gradient by direct reductions      6  feature gradient with the per-tile sort
 *   5  record-based depth-gradient kernel also for the parametric modes without entry lists
 *   7  gradients through the global sort whatever the problem size      8  the same with a 4096-entry list
 *   9  global sort with tile_x = gather blocks per SM and tile_y = entries per gather run
 *   10 global sort with tile_x = scatter blocks per SM and tile_y = threads per scatter block
 *   12 global sort, the parametric depth gradient never on the entry lists      13 always on them
 *   16 global sort with tile_x = 16-byte chunks per lane of the gather kernel (1, 2 or 4)
 *   14 forward / list kernels always on the tile counter      15 always in the static unit order (one sample)
 * Any non-zero selector other than 7, 8, 9, 10, 12, 13, 16 also turns the global sort off. */
void fbev_set_tuning(int tile_x, int tile_y, int chunks_per_lane, int warps, int min_blocks);

/* Experiment switches of the forward kernel, per host thread like the tuning above; a bit mask, 0 = off.
 *   FBEV_EXP_PREFETCH  every block first asks the L2 for its share of the feature and depth tensors
 *                      (prefetch.global.L2), so that a cold L2 is filled by wide requests instead of by the
 *                      dependent misses of the first gathers
 *   FBEV_EXP_GROUP_CULL the camera cull is evaluated for the box of the warp's own group of cells instead of
 *                      the whole tile: fewer candidates per sweep near the edges of a camera's field of view
 *   FBEV_EXP_DRAW      static unit order for a warp's first unit only; the remaining units are handed out one at
 *                      a time through the scheduler word (needs FbevProblem.workspace)
 *   FBEV_EXP_SHARED_GATHER_CEILING  TIMING ONLY, THE RESULT IS WRONG: the channel phase takes its texel chunks from
 *                      the block's shared memory (whatever is there) instead of from global memory.  It shows what a
 *                      scheme that stages feature rows in shared memory could gain at most, were the staging free */
enum { FBEV_EXP_PREFETCH = 1, FBEV_EXP_GROUP_CULL = 2, FBEV_EXP_DRAW = 4, FBEV_EXP_SHARED_GATHER_CEILING = 8 };
void fbev_set_experiment(int bits);

/* Reads `bytes` of device memory `repeats` times with 16-byte loads (a bandwidth
 * probe for roofline denominators: L2-resident when bytes fits the L2).  sink:
 * device, >= 4 bytes. */
int fbev_probe_read(const void* buf, size_t bytes, int repeats, void* sink, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FBEV_DEBUG_H_ */
