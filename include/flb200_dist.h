/* flb200_dist.h — C ABI of the gradient-synchronisation backend (libflb200_dist.so).
 *
 * One process per GPU.  The functions mirror the free functions a Flashlight
 * distributed backend defines (flashlight/fl/distributed/DistributedApi.h:33-136 and
 * flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp:114-290) and the Reducer
 * interface (flashlight/fl/distributed/reducers/Reducer.h:21-41), over plain pointers:
 *
 *   fl::distributedInit(FILE_SYSTEM, rank, size, {kFilePath,…})  -> flb200_dist_init_file
 *   fl::isDistributedInit / getWorldRank / getWorldSize          -> flb200_dist_is_initialized / _world_rank / _world_size
 *   fl::allReduce(Tensor&, async) [+ "*= scale"]                 -> flb200_dist_all_reduce
 *   fl::allReduceMultiple(vector<Tensor*>, async, contiguous)    -> flb200_dist_all_reduce_multiple
 *   fl::syncDistributed()                                        -> flb200_dist_sync
 *   fl::barrier()                                                -> flb200_dist_barrier
 *   Reducer::add / Reducer::finalize                             -> flb200_reducer_add / flb200_reducer_finalize
 *
 * Every function returns a flb200_status (flb200.h) and never throws; the text of the last
 * failure on the calling thread is flb200_dist_last_error().  Reductions are in place and
 * run on the backend's own reduction stream; `stream` arguments are the cudaStream_t on which
 * the caller produced the buffers and will consume the results.  The scale of the reference's
 * "allReduce then multiply" is fused into the collective (a pre-multiplied sum), so a scaled
 * reduction is still one kernel.
 */
#ifndef FLB200_DIST_H
#define FLB200_DIST_H

#include <stdint.h>

#include "flb200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Element types: the three of flb200.h plus the other types the reference's NCCL backend
 * accepts (DistributedBackend.cpp:66-85). */
enum { FLB200_DIST_F64 = 16, FLB200_DIST_I32 = 17, FLB200_DIST_I64 = 18 };

/* Largest set flb200_dist_all_reduce_multiple(contiguous=1) coalesces: the reference's
 * DistributedConstants::kCoalesceCacheSize (flashlight/fl/common/Defines.h:97). */
#define FLB200_DIST_COALESCE_BYTES ((int64_t)20 << 20)

/* File-system rendezvous (NcclContext::initWithFileSystem, DistributedBackend.cpp:443-487):
 * rank 0 publishes the communicator id in `path`, the others wait for it up to `timeout_s`
 * seconds (FLB200_TIMEOUT afterwards: a rank that never came), then all join.  `device` is the
 * CUDA device of this process.  A second call warns and returns FLB200_OK like the reference. */
int flb200_dist_init_file(const char* path, int world_rank, int world_size, int device,
                          double timeout_s);
int flb200_dist_is_initialized(void);
int flb200_dist_world_rank(void); /* 0 before initialisation, like fl::getWorldRank */
int flb200_dist_world_size(void); /* 1 before initialisation */
/* Waits for outstanding work, destroys the communicator and streams. */
int flb200_dist_shutdown(void);

/* data[i] <- scale * sum over ranks of data[i].  async=0: ordered after the work already on
 * `stream`, and `stream` waits for the result.  async=1: the result is ready only after
 * flb200_dist_sync.  Integer types require scale == 1.  FLB200_INVALID_ARG with
 * "distributed environment not initialized" before initialisation. */
int flb200_dist_all_reduce(void* data, int64_t count, int dtype, double scale, int async,
                           void* stream);

/* The same for n buffers.  contiguous=0: one grouped launch, mixed types allowed.
 * contiguous=1: the buffers are packed into the backend's coalescing buffer, reduced once and
 * unpacked; all types must be equal ("…of different types") and the packed size must not exceed
 * FLB200_DIST_COALESCE_BYTES ("Total coalesce buffer size is larger…"), as in the reference. */
int flb200_dist_all_reduce_multiple(void* const* data, const int64_t* counts, const int* dtypes,
                                    int n, double scale, int async, int contiguous, void* stream);

/* Makes `stream` wait for everything the backend has queued (fl::syncDistributed) and reports a
 * communicator error seen since the last call as FLB200_LAUNCH_FAILURE. */
int flb200_dist_sync(void* stream);
/* Blocks the HOST until the queued reductions have finished or `timeout_s` passed; after a
 * time-out the communicator is aborted (a peer that died must not hang this rank for ever) and
 * FLB200_TIMEOUT is returned; the backend is uninitialised afterwards. */
int flb200_dist_wait(double timeout_s);
int flb200_dist_barrier(void);
const char* flb200_dist_last_error(void);

/* ---- bucketed gradient reducer --------------------------------------------------------------
 * The gradients of n parameters (counts[i] elements of `dtype` each, in the order the backward
 * pass produces them LAST to FIRST is best) live inside one caller-provided arena, grouped into
 * buckets of about bucket_bytes.  flb200_reducer_slot(i) is where gradient i lives: a backward
 * pass that writes there needs no copy.  add(i) marks gradient i ready; a bucket is reduced (on
 * the reduction stream, overlapping the rest of the backward pass) as soon as it and every
 * bucket before it are complete, so every rank launches the same collectives in the same order
 * whatever order its gradients arrive in.  finalize() zero-fills gradients that never came,
 * reduces what is left and makes `stream` wait. */
typedef struct flb200_reducer flb200_reducer;
int64_t flb200_reducer_arena_bytes(const int64_t* counts, int n, int dtype, int64_t bucket_bytes);
int flb200_reducer_create(const int64_t* counts, int n, int dtype, double scale,
                          int64_t bucket_bytes, void* arena, int64_t arena_bytes,
                          flb200_reducer** out);
void* flb200_reducer_slot(const flb200_reducer* r, int index);
int flb200_reducer_num_buckets(const flb200_reducer* r);
int flb200_reducer_bucket_of(const flb200_reducer* r, int index);
/* Number of collectives this reducer has launched so far (for tests of the firing order). */
int flb200_reducer_launched(const flb200_reducer* r);
/* grad == NULL or == slot: the gradient was written in place; else it is copied in on `stream`.
 * Adding an index twice, or out of range, is FLB200_INVALID_ARG. */
int flb200_reducer_add(flb200_reducer* r, int index, const void* grad, void* stream);
int flb200_reducer_finalize(flb200_reducer* r, void* stream);
int flb200_reducer_destroy(flb200_reducer* r);

#ifdef __cplusplus
}
#endif
#endif /* FLB200_DIST_H */
