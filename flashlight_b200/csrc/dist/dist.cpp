// libflb200_dist.so: gradient synchronisation for one process per GPU over NCCL.
//
// Replaces the NCCL backend of the reference
// (flashlight/fl/distributed/backend/cuda/DistributedBackend.cpp) behind a C ABI.  What differs
// by design: the scale is fused into the collective (pre-multiplied sum) instead of a second
// element-wise pass; the bucketed reducer keeps gradients inside flat buckets so nothing is packed
// or unpacked, and fires buckets in index order so that all ranks agree on the collective order;
// every host-side wait has a deadline, after which the communicator is aborted.
#include "flb200_dist.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;

int fail(int status, const std::string& msg) {
  g_error = msg;
  return status;
}

#define CUDA_TRY(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e_ = (expr);                                                                \
    if (e_ != cudaSuccess)                                                                  \
      return fail(FLB200_LAUNCH_FAILURE, std::string(#expr ": ") + cudaGetErrorString(e_)); \
  } while (0)

// Mirrors detail::ncclCheck (DistributedBackend.cpp:292-304): invalid argument / usage are the
// caller's fault, the rest are run-time failures.
int nccl_status(ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return FLB200_OK;
  const int st = (r == ncclInvalidArgument || r == ncclInvalidUsage) ? FLB200_INVALID_ARG
                                                                     : FLB200_LAUNCH_FAILURE;
  return fail(st, std::string(what) + ": " + ncclGetErrorString(r));
}
ncclResult_t settle(ncclResult_t r);
#define NCCL_TRY(expr)                                  \
  do {                                                  \
    int s_ = nccl_status(settle(expr), #expr);          \
    if (s_ != FLB200_OK) return s_;                     \
  } while (0)

struct Context {
  bool init = false;
  int rank = 0, size = 1, device = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t reduce = nullptr;  // collectives run here
  cudaStream_t worker = nullptr;  // pack / unpack copies of the contiguous mode
  cudaEvent_t ready = nullptr;    // caller stream -> backend
  cudaEvent_t done = nullptr;     // backend -> caller stream
  void* coalesce = nullptr;
  bool pending = false;           // work queued since the last sync
};
Context g_ctx;
std::mutex g_mu;

// The communicator is created non-blocking (so that joining it can time out), which lets any
// later call answer "in progress": wait, with a limit, until the call has really been queued.
ncclResult_t settle(ncclResult_t r) {
  if (r != ncclInProgress || !g_ctx.comm) return r;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(60);
  ncclResult_t state = ncclInProgress;
  while (state == ncclInProgress) {
    if (ncclCommGetAsyncError(g_ctx.comm, &state) != ncclSuccess) return ncclSystemError;
    if (state == ncclInProgress) {
      if (std::chrono::steady_clock::now() >= deadline) return ncclSystemError;
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  return state;
}

bool type_info(int dtype, ncclDataType_t* t, size_t* size, bool* is_float) {
  switch (dtype) {
    case FLB200_F32: *t = ncclFloat32; *size = 4; *is_float = true; return true;
    case FLB200_F16: *t = ncclFloat16; *size = 2; *is_float = true; return true;
    case FLB200_BF16: *t = ncclBfloat16; *size = 2; *is_float = true; return true;
    case FLB200_DIST_F64: *t = ncclFloat64; *size = 8; *is_float = true; return true;
    case FLB200_DIST_I32: *t = ncclInt32; *size = 4; *is_float = false; return true;
    case FLB200_DIST_I64: *t = ncclInt64; *size = 8; *is_float = false; return true;
  }
  return false;
}

// A reduction operator "scale * sum" for one call; plain sum when scale == 1.
struct ScaledSum {
  ncclRedOp_t op = ncclSum;
  bool custom = false;
  int make(double scale, int dtype) {
    if (scale == 1.0) return FLB200_OK;
    union { float f; double d; __half h; __nv_bfloat16 b; } v;
    ncclDataType_t t; size_t sz; bool fl;
    type_info(dtype, &t, &sz, &fl);
    if (!fl) return fail(FLB200_INVALID_ARG, "integer reductions cannot be scaled");
    switch (dtype) {
      case FLB200_F32: v.f = static_cast<float>(scale); break;
      case FLB200_F16: v.h = __float2half(static_cast<float>(scale)); break;
      case FLB200_BF16: v.b = __float2bfloat16(static_cast<float>(scale)); break;
      default: v.d = scale; break;
    }
    NCCL_TRY(ncclRedOpCreatePreMulSum(&op, &v, t, ncclScalarHostImmediate, g_ctx.comm));
    custom = true;
    return FLB200_OK;
  }
  ~ScaledSum() {
    if (custom) ncclRedOpDestroy(op, g_ctx.comm);
  }
};

int require_init() {
  if (!g_ctx.init) return fail(FLB200_INVALID_ARG, "distributed environment not initialized");
  return FLB200_OK;
}

// `from` -> `to`: work queued on `to` afterwards runs after what `from` holds now.
int chain(cudaStream_t from, cudaStream_t to, cudaEvent_t ev) {
  CUDA_TRY(cudaEventRecord(ev, from));
  CUDA_TRY(cudaStreamWaitEvent(to, ev, 0));
  return FLB200_OK;
}

int write_id_file(const std::string& path, const ncclUniqueId& id) {
  const std::string tmp = path + ".tmp." + std::to_string(getpid());
  FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) return fail(FLB200_INVALID_ARG, "cannot create rendezvous file " + tmp);
  const size_t n = std::fwrite(&id, 1, sizeof(id), f);
  std::fclose(f);
  if (n != sizeof(id) || std::rename(tmp.c_str(), path.c_str()) != 0) {
    std::remove(tmp.c_str());
    return fail(FLB200_INVALID_ARG, "cannot publish rendezvous file " + path);
  }
  return FLB200_OK;
}

int read_id_file(const std::string& path, double timeout_s, ncclUniqueId* id) {
  const auto deadline = std::chrono::steady_clock::now() +
      std::chrono::duration_cast<std::chrono::steady_clock::duration>(
          std::chrono::duration<double>(timeout_s));
  for (;;) {
    struct stat st;
    if (stat(path.c_str(), &st) == 0 && static_cast<size_t>(st.st_size) == sizeof(*id)) {
      FILE* f = std::fopen(path.c_str(), "rb");
      if (f) {
        const size_t n = std::fread(id, 1, sizeof(*id), f);
        std::fclose(f);
        if (n == sizeof(*id)) return FLB200_OK;
      }
    }
    if (std::chrono::steady_clock::now() >= deadline)
      return fail(FLB200_TIMEOUT, "rank 0 did not publish " + path + " within the time limit");
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

void release_resources() {
  if (g_ctx.coalesce) cudaFree(g_ctx.coalesce);
  if (g_ctx.ready) cudaEventDestroy(g_ctx.ready);
  if (g_ctx.done) cudaEventDestroy(g_ctx.done);
  if (g_ctx.reduce) cudaStreamDestroy(g_ctx.reduce);
  if (g_ctx.worker) cudaStreamDestroy(g_ctx.worker);
  g_ctx = Context();
}

int all_reduce_locked(void* data, int64_t count, int dtype, double scale, int async,
                      cudaStream_t stream) {
  ncclDataType_t t; size_t sz; bool fl;
  if (!type_info(dtype, &t, &sz, &fl)) return fail(FLB200_INVALID_ARG, "unsupported element type");
  if (count < 0 || (count > 0 && !data)) return fail(FLB200_INVALID_ARG, "null buffer");
  if (count == 0) return FLB200_OK;
  ScaledSum op;
  if (int s = op.make(scale, dtype)) return s;
  if (int s = chain(stream, g_ctx.reduce, g_ctx.ready)) return s;
  NCCL_TRY(ncclAllReduce(data, data, static_cast<size_t>(count), t, op.op, g_ctx.comm,
                         g_ctx.reduce));
  g_ctx.pending = true;
  if (!async) return chain(g_ctx.reduce, stream, g_ctx.done);
  return FLB200_OK;
}

}  // namespace

extern "C" {

const char* flb200_dist_last_error(void) { return g_error.c_str(); }
int flb200_dist_is_initialized(void) { return g_ctx.init ? 1 : 0; }
int flb200_dist_world_rank(void) { return g_ctx.init ? g_ctx.rank : 0; }
int flb200_dist_world_size(void) { return g_ctx.init ? g_ctx.size : 1; }

int flb200_dist_init_file(const char* path, int world_rank, int world_size, int device,
                          double timeout_s) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_ctx.init) {
    std::fprintf(stderr, "warning: flb200_dist_init_file() called more than once\n");
    return FLB200_OK;
  }
  if (!path || !*path) return fail(FLB200_INVALID_ARG, "invalid FilePath for file-system rendezvous");
  if (world_size < 1 || world_rank < 0 || world_rank >= world_size)
    return fail(FLB200_INVALID_ARG, "world rank outside [0, world size)");
  if (device < 0) return fail(FLB200_INVALID_ARG, "invalid device");
  if (!(timeout_s > 0)) return fail(FLB200_INVALID_ARG, "the rendezvous needs a positive time limit");

  ncclUniqueId id;
  if (world_rank == 0) {
    if (int s = nccl_status(ncclGetUniqueId(&id), "ncclGetUniqueId")) return s;
    if (int s = write_id_file(path, id)) return s;
  } else {
    // Before any CUDA or NCCL call: a rank 0 that never comes costs this rank nothing but time.
    if (int s = read_id_file(path, timeout_s, &id)) return s;
  }
  CUDA_TRY(cudaSetDevice(device));
  ncclComm_t comm = nullptr;
  // Non-blocking initialisation so that a peer that never joins ends in a time-out, not a hang.
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  ncclResult_t r = ncclCommInitRankConfig(&comm, world_size, id, world_rank, &cfg);
  const auto deadline = std::chrono::steady_clock::now() +
      std::chrono::duration_cast<std::chrono::steady_clock::duration>(
          std::chrono::duration<double>(timeout_s));
  while (r == ncclInProgress || r == ncclSuccess) {
    ncclResult_t state = ncclSuccess;
    r = ncclCommGetAsyncError(comm, &state);
    if (r != ncclSuccess) break;
    r = state;
    if (state == ncclSuccess) break;
    if (state == ncclInProgress && std::chrono::steady_clock::now() >= deadline) {
      ncclCommAbort(comm);
      if (world_rank == 0) std::remove(path);
      return fail(FLB200_TIMEOUT, "not every rank joined the communicator within the time limit");
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  if (world_rank == 0) std::remove(path);  // the reference clears its key after the join too
  if (r != ncclSuccess) {
    if (comm) ncclCommAbort(comm);
    return nccl_status(r, "ncclCommInitRank");
  }
  g_ctx.comm = comm;
  g_ctx.rank = world_rank;
  g_ctx.size = world_size;
  g_ctx.device = device;
  CUDA_TRY(cudaStreamCreateWithFlags(&g_ctx.reduce, cudaStreamNonBlocking));
  CUDA_TRY(cudaStreamCreateWithFlags(&g_ctx.worker, cudaStreamNonBlocking));
  CUDA_TRY(cudaEventCreateWithFlags(&g_ctx.ready, cudaEventDisableTiming));
  CUDA_TRY(cudaEventCreateWithFlags(&g_ctx.done, cudaEventDisableTiming));
  g_ctx.init = true;
  return FLB200_OK;
}

int flb200_dist_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_ctx.init) return FLB200_OK;
  cudaStreamSynchronize(g_ctx.worker);
  cudaStreamSynchronize(g_ctx.reduce);
  ncclResult_t r = ncclCommFinalize(g_ctx.comm);
  if (r == ncclSuccess || r == ncclInProgress) {
    ncclResult_t state = ncclInProgress;
    for (int i = 0; i < 20000 && state == ncclInProgress; ++i) {  // at most about 20 s
      if (ncclCommGetAsyncError(g_ctx.comm, &state) != ncclSuccess) break;
      if (state == ncclInProgress) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    if (state == ncclSuccess) ncclCommDestroy(g_ctx.comm); else ncclCommAbort(g_ctx.comm);
  } else {
    ncclCommAbort(g_ctx.comm);
  }
  release_resources();
  return FLB200_OK;
}

int flb200_dist_all_reduce(void* data, int64_t count, int dtype, double scale, int async,
                           void* stream) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (int s = require_init()) return s;
  return all_reduce_locked(data, count, dtype, scale, async, static_cast<cudaStream_t>(stream));
}

int flb200_dist_all_reduce_multiple(void* const* data, const int64_t* counts, const int* dtypes,
                                    int n, double scale, int async, int contiguous, void* stream_) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (n < 0) return fail(FLB200_INVALID_ARG, "negative buffer count");
  if (n == 0) return FLB200_OK;  // the reference's fast path comes before every check too
  if (!data || !counts || !dtypes) return fail(FLB200_INVALID_ARG, "null argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::vector<size_t> bytes(n);
  size_t total = 0;
  int64_t total_count = 0;
  for (int i = 0; i < n; ++i) {
    ncclDataType_t t; size_t sz; bool fl;
    if (!type_info(dtypes[i], &t, &sz, &fl))
      return fail(FLB200_INVALID_ARG, "unsupported element type");
    if (counts[i] < 0 || (counts[i] > 0 && !data[i])) return fail(FLB200_INVALID_ARG, "null buffer");
    if (contiguous && dtypes[i] != dtypes[0])
      return fail(FLB200_INVALID_ARG,
                  "Cannot perform contiguous set allReduce on a set of tensors of different types");
    bytes[i] = static_cast<size_t>(counts[i]) * sz;
    total += bytes[i];
    total_count += counts[i];
  }
  if (contiguous && total > static_cast<size_t>(FLB200_DIST_COALESCE_BYTES))
    return fail(FLB200_INVALID_ARG,
                "Total coalesce buffer size is larger than existing buffer size");
  if (int s = require_init()) return s;
  if (!contiguous) {
    // One grouped launch (DistributedBackend.cpp:138-146).
    std::vector<ScaledSum> ops(n);
    for (int i = 0; i < n; ++i)
      if (int s = ops[i].make(scale, dtypes[i])) return s;
    if (int s = chain(stream, g_ctx.reduce, g_ctx.ready)) return s;
    NCCL_TRY(ncclGroupStart());
    for (int i = 0; i < n; ++i) {
      if (counts[i] == 0) continue;
      ncclDataType_t t; size_t sz; bool fl;
      type_info(dtypes[i], &t, &sz, &fl);
      ncclResult_t r = ncclAllReduce(data[i], data[i], static_cast<size_t>(counts[i]), t,
                                     ops[i].op, g_ctx.comm, g_ctx.reduce);
      if (r != ncclSuccess && r != ncclInProgress) {
        ncclGroupEnd();
        return nccl_status(r, "ncclAllReduce");
      }
    }
    NCCL_TRY(ncclGroupEnd());
    g_ctx.pending = true;
    if (!async) return chain(g_ctx.reduce, stream, g_ctx.done);
    return FLB200_OK;
  }
  if (total == 0) return FLB200_OK;
  if (!g_ctx.coalesce) CUDA_TRY(cudaMalloc(&g_ctx.coalesce, FLB200_DIST_COALESCE_BYTES));
  ncclDataType_t t; size_t sz; bool fl;
  type_info(dtypes[0], &t, &sz, &fl);
  ScaledSum op;
  if (int s = op.make(scale, dtypes[0])) return s;
  // pack on the worker stream, after the producers and after earlier users of the buffer
  if (int s = chain(stream, g_ctx.worker, g_ctx.ready)) return s;
  if (int s = chain(g_ctx.reduce, g_ctx.worker, g_ctx.ready)) return s;
  char* cur = static_cast<char*>(g_ctx.coalesce);
  for (int i = 0; i < n; ++i) {
    if (bytes[i])
      CUDA_TRY(cudaMemcpyAsync(cur, data[i], bytes[i], cudaMemcpyDeviceToDevice, g_ctx.worker));
    cur += bytes[i];
  }
  if (int s = chain(g_ctx.worker, g_ctx.reduce, g_ctx.ready)) return s;
  NCCL_TRY(ncclAllReduce(g_ctx.coalesce, g_ctx.coalesce, static_cast<size_t>(total_count), t, op.op,
                         g_ctx.comm, g_ctx.reduce));
  if (int s = chain(g_ctx.reduce, g_ctx.worker, g_ctx.ready)) return s;
  cur = static_cast<char*>(g_ctx.coalesce);
  for (int i = 0; i < n; ++i) {
    if (bytes[i])
      CUDA_TRY(cudaMemcpyAsync(data[i], cur, bytes[i], cudaMemcpyDeviceToDevice, g_ctx.worker));
    cur += bytes[i];
  }
  g_ctx.pending = true;
  if (!async) return chain(g_ctx.worker, stream, g_ctx.done);
  return FLB200_OK;
}

int flb200_dist_sync(void* stream_) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_ctx.init) return FLB200_OK;  // nothing can be queued
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int s = chain(g_ctx.worker, stream, g_ctx.done)) return s;
  if (int s = chain(g_ctx.reduce, stream, g_ctx.done)) return s;
  ncclResult_t state = ncclSuccess;
  NCCL_TRY(ncclCommGetAsyncError(g_ctx.comm, &state));
  if (state != ncclSuccess && state != ncclInProgress)
    return fail(FLB200_LAUNCH_FAILURE,
                std::string("communicator error: ") + ncclGetErrorString(state));
  return FLB200_OK;
}

int flb200_dist_wait(double timeout_s) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_ctx.init) return FLB200_OK;
  if (!(timeout_s > 0)) return fail(FLB200_INVALID_ARG, "the wait needs a positive time limit");
  if (int s = chain(g_ctx.worker, g_ctx.reduce, g_ctx.ready)) return s;
  CUDA_TRY(cudaEventRecord(g_ctx.done, g_ctx.reduce));
  const auto deadline = std::chrono::steady_clock::now() +
      std::chrono::duration_cast<std::chrono::steady_clock::duration>(
          std::chrono::duration<double>(timeout_s));
  for (;;) {
    cudaError_t q = cudaEventQuery(g_ctx.done);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady)
      return fail(FLB200_LAUNCH_FAILURE, std::string("cudaEventQuery: ") + cudaGetErrorString(q));
    ncclResult_t state = ncclSuccess;
    ncclCommGetAsyncError(g_ctx.comm, &state);
    const bool broken = state != ncclSuccess && state != ncclInProgress;
    if (broken || std::chrono::steady_clock::now() >= deadline) {
      ncclCommAbort(g_ctx.comm);
      release_resources();
      return broken ? fail(FLB200_LAUNCH_FAILURE, std::string("communicator error: ") +
                                                      ncclGetErrorString(state))
                    : fail(FLB200_TIMEOUT,
                           "a reduction did not finish within the time limit; communicator aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  g_ctx.pending = false;
  return FLB200_OK;
}

int flb200_dist_barrier(void) {
  // fl::barrier (DistributedApi.cpp:49-56): reduce one element and wait for it on the host.
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (int s = require_init()) return s;
    if (!g_ctx.coalesce) CUDA_TRY(cudaMalloc(&g_ctx.coalesce, FLB200_DIST_COALESCE_BYTES));
    if (int s = chain(g_ctx.worker, g_ctx.reduce, g_ctx.ready)) return s;
    CUDA_TRY(cudaMemsetAsync(g_ctx.coalesce, 0, sizeof(int), g_ctx.reduce));
    NCCL_TRY(ncclAllReduce(g_ctx.coalesce, g_ctx.coalesce, 1, ncclInt32, ncclSum, g_ctx.comm,
                           g_ctx.reduce));
    CUDA_TRY(cudaStreamSynchronize(g_ctx.reduce));
  }
  return FLB200_OK;
}

// ----------------------------------------------------------------------------- bucketed reducer
struct flb200_reducer {
  int n = 0, dtype = FLB200_F32;
  double scale = 1.0;
  size_t elem = 4;
  char* arena = nullptr;
  std::vector<int64_t> counts, offset;  // element counts and byte offsets into the arena
  std::vector<int> bucket_of;
  std::vector<int64_t> bucket_begin, bucket_count;  // byte offset / element count per bucket
  std::vector<int> bucket_missing;                  // gradients not yet added, per bucket
  std::vector<int> bucket_size;
  std::vector<char> added;
  std::vector<cudaEvent_t> events;
  int next_bucket = 0, launched = 0;
};

namespace {

constexpr int64_t kSlotAlign = 256;  // every gradient starts on a 256-byte boundary

int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Greedy grouping in index order: a bucket closes once it holds at least bucket_bytes.
bool plan(const int64_t* counts, int n, int dtype, int64_t bucket_bytes, flb200_reducer* r) {
  ncclDataType_t t; size_t sz; bool fl;
  if (!counts || n < 0 || bucket_bytes <= 0 || !type_info(dtype, &t, &sz, &fl)) return false;
  r->n = n; r->dtype = dtype; r->elem = sz;
  r->counts.assign(counts, counts + n);
  r->offset.resize(n); r->bucket_of.resize(n);
  int64_t cur = 0, begin = 0;
  int members = 0;
  for (int i = 0; i < n; ++i) {
    if (counts[i] < 0) return false;
    r->offset[i] = cur;
    r->bucket_of[i] = static_cast<int>(r->bucket_begin.size());
    cur += round_up(counts[i] * static_cast<int64_t>(sz), kSlotAlign);
    ++members;
    if (cur - begin >= bucket_bytes || i == n - 1) {
      r->bucket_begin.push_back(begin);
      r->bucket_count.push_back((cur - begin) / static_cast<int64_t>(sz));
      r->bucket_size.push_back(members);
      begin = cur;
      members = 0;
    }
  }
  return true;
}

int fire_ready(flb200_reducer* r, cudaStream_t stream) {
  const int nb = static_cast<int>(r->bucket_begin.size());
  while (r->next_bucket < nb && r->bucket_missing[r->next_bucket] == 0) {
    const int b = r->next_bucket;
    CUDA_TRY(cudaEventRecord(r->events[b], stream));
    CUDA_TRY(cudaStreamWaitEvent(g_ctx.reduce, r->events[b], 0));
    ncclDataType_t t; size_t sz; bool fl;
    type_info(r->dtype, &t, &sz, &fl);
    ScaledSum op;
    if (int s = op.make(r->scale, r->dtype)) return s;
    void* p = r->arena + r->bucket_begin[b];
    if (r->bucket_count[b] > 0)
      NCCL_TRY(ncclAllReduce(p, p, static_cast<size_t>(r->bucket_count[b]), t, op.op, g_ctx.comm,
                             g_ctx.reduce));
    g_ctx.pending = true;
    ++r->launched;
    ++r->next_bucket;
  }
  return FLB200_OK;
}

void reset(flb200_reducer* r) {
  r->bucket_missing = r->bucket_size;
  std::fill(r->added.begin(), r->added.end(), 0);
  r->next_bucket = 0;
}

}  // namespace

int64_t flb200_reducer_arena_bytes(const int64_t* counts, int n, int dtype, int64_t bucket_bytes) {
  flb200_reducer r;
  if (!plan(counts, n, dtype, bucket_bytes, &r)) {
    fail(FLB200_INVALID_ARG, "invalid reducer description");
    return -1;
  }
  return n == 0 ? 0 : r.bucket_begin.back() + r.bucket_count.back() * static_cast<int64_t>(r.elem);
}

int flb200_reducer_create(const int64_t* counts, int n, int dtype, double scale,
                          int64_t bucket_bytes, void* arena, int64_t arena_bytes,
                          flb200_reducer** out) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!out) return fail(FLB200_INVALID_ARG, "null argument");
  if (int s = require_init()) return s;
  auto* r = new flb200_reducer();
  if (!plan(counts, n, dtype, bucket_bytes, r)) {
    delete r;
    return fail(FLB200_INVALID_ARG, "invalid reducer description");
  }
  const int64_t need =
      n == 0 ? 0 : r->bucket_begin.back() + r->bucket_count.back() * static_cast<int64_t>(r->elem);
  ncclDataType_t t; size_t sz; bool fl;
  type_info(dtype, &t, &sz, &fl);
  if (!fl && scale != 1.0) {
    delete r;
    return fail(FLB200_INVALID_ARG, "integer reductions cannot be scaled");
  }
  if (need > 0 && (!arena || arena_bytes < need ||
                   reinterpret_cast<uintptr_t>(arena) % static_cast<uintptr_t>(kSlotAlign))) {
    delete r;
    return fail(arena && arena_bytes < need ? FLB200_WORKSPACE_TOO_SMALL : FLB200_INVALID_ARG,
                "the arena is missing, too small or not 256-byte aligned");
  }
  r->scale = scale;
  r->arena = static_cast<char*>(arena);
  r->added.assign(n, 0);
  r->events.resize(r->bucket_begin.size());
  for (auto& e : r->events) {
    cudaError_t ce = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    if (ce != cudaSuccess) {
      delete r;
      return fail(FLB200_LAUNCH_FAILURE, cudaGetErrorString(ce));
    }
  }
  reset(r);
  *out = r;
  return FLB200_OK;
}

void* flb200_reducer_slot(const flb200_reducer* r, int i) {
  if (!r || i < 0 || i >= r->n) return nullptr;
  return r->arena + r->offset[i];
}
int flb200_reducer_num_buckets(const flb200_reducer* r) {
  return r ? static_cast<int>(r->bucket_begin.size()) : 0;
}
int flb200_reducer_bucket_of(const flb200_reducer* r, int i) {
  return (!r || i < 0 || i >= r->n) ? -1 : r->bucket_of[i];
}
int flb200_reducer_launched(const flb200_reducer* r) { return r ? r->launched : 0; }

int flb200_reducer_add(flb200_reducer* r, int i, const void* grad, void* stream_) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!r) return fail(FLB200_INVALID_ARG, "null reducer");
  if (int s = require_init()) return s;
  if (i < 0 || i >= r->n) return fail(FLB200_INVALID_ARG, "gradient index out of range");
  if (r->added[i]) return fail(FLB200_INVALID_ARG, "gradient added twice before finalize");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  void* slot = r->arena + r->offset[i];
  if (grad && grad != slot && r->counts[i] > 0)
    CUDA_TRY(cudaMemcpyAsync(slot, grad, static_cast<size_t>(r->counts[i]) * r->elem,
                             cudaMemcpyDeviceToDevice, stream));
  r->added[i] = 1;
  --r->bucket_missing[r->bucket_of[i]];
  return fire_ready(r, stream);
}

int flb200_reducer_finalize(flb200_reducer* r, void* stream_) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!r) return fail(FLB200_INVALID_ARG, "null reducer");
  if (int s = require_init()) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // A parameter that took no part in this step contributes zeros, so that the collectives of
  // all ranks keep the same sizes and order.
  for (int i = 0; i < r->n; ++i) {
    if (r->added[i]) continue;
    if (r->counts[i] > 0)
      CUDA_TRY(cudaMemsetAsync(r->arena + r->offset[i], 0,
                               static_cast<size_t>(r->counts[i]) * r->elem, stream));
    r->added[i] = 1;
    --r->bucket_missing[r->bucket_of[i]];
  }
  if (int s = fire_ready(r, stream)) return s;
  if (int s = chain(g_ctx.reduce, stream, g_ctx.done)) return s;
  reset(r);
  ncclResult_t state = ncclSuccess;
  NCCL_TRY(ncclCommGetAsyncError(g_ctx.comm, &state));
  if (state != ncclSuccess && state != ncclInProgress)
    return fail(FLB200_LAUNCH_FAILURE,
                std::string("communicator error: ") + ncclGetErrorString(state));
  return FLB200_OK;
}

int flb200_reducer_destroy(flb200_reducer* r) {
  if (!r) return FLB200_OK;
  for (auto e : r->events)
    if (e) cudaEventDestroy(e);
  delete r;
  return FLB200_OK;
}

}  // extern "C"
