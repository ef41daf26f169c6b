// Data-parallel gradient exchange behind the C ABI: THGPUComm.
//
// The reference has no multi-GPU code; the contract here is mini-batch data parallelism over the GPUs of one
// box: every rank holds a replica, computes gradWeight / gradBias of its rows into one flat gradient buffer, the
// buffer is summed over the ranks bucket by bucket while the backward pass is still running, and each bucket's
// parameter update runs right behind its all-reduce:
//
//   compute stream   ... backward of the classifier | backward of conv5 | ... | conv1 |      next step ...
//   comm stream                    all-reduce(fc) -> SGD(fc)   all-reduce(conv5) -> SGD(conv5) ...
//
// THGPUComm_allReduceAsync(bucket) records an event on the compute stream (everything that produced the bucket
// is queued before it), makes the communicator's own stream wait for it, and queues the all-reduce and the
// update of that slice there; THGPUComm_wait makes the compute stream wait for all of it (no host
// synchronisation anywhere).  A host watchdog thread gives every queued bucket a deadline; a bucket that has not
// completed by then (a rank that never joined, a hung link) gets the communicator aborted and the next call
// returns the error instead of blocking for ever.
//
// The host logic (bucket table, launch order, the check that every rank describes the same layout, the
// watchdog) is separate from the transport: a THGPUCommBackend is a table of callbacks.  The NCCL backend
// (second half of this file; libnccl.so.2 is loaded at run time, not linked) is the product; tests drive the host
// logic on machines without a GPU through a fake backend whose callbacks they control.
#include "thc_internal.h"

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <dlfcn.h>
#include <nccl.h>

struct THGPUComm {
  int world = 1, rank = 0;
  THGPUCommBackend be{};
  // gradient layout
  float *grad = nullptr;
  long n = 0;
  std::vector<long> begin, count;
  bool update = false;
  // per-round state, guarded by mu
  std::mutex mu;
  std::condition_variable cv;
  std::vector<char> launched, finished;
  std::vector<std::chrono::steady_clock::time_point> deadline;
  double timeout_s = 30.0;
  std::string error;          // non-empty: the communicator is dead
  bool stop = false;
  std::thread watchdog;
};

namespace thc {
namespace {

using Clock = std::chrono::steady_clock;

void comm_fail(THGPUComm *c, const std::string &msg) {   // caller holds c->mu
  if (c->error.empty()) c->error = msg;
}

// Polls the queued buckets every few milliseconds: marks those that completed, aborts the communicator when one
// has passed its deadline or the transport reports an error.
void watchdog_loop(THGPUComm *c) {
  std::unique_lock<std::mutex> lock(c->mu);
  while (!c->stop) {
    c->cv.wait_for(lock, std::chrono::milliseconds(5));
    if (c->stop || !c->error.empty()) continue;
    const auto now = Clock::now();
    for (size_t b = 0; b < c->launched.size(); b++) {
      if (!c->launched[b] || c->finished[b]) continue;
      lock.unlock();
      const int d = c->be.done ? c->be.done(c->be.ctx, (int)b) : 1;
      lock.lock();
      if (c->stop) break;
      if (d > 0) {
        c->finished[b] = 1;
        if (c->launched[b] == 2) c->launched[b] = 0;   // a bucket of the previous step: nothing left to watch
        continue;
      }
      if (d < 0 || now > c->deadline[b]) {
        char msg[256];
        snprintf(msg, sizeof(msg), d < 0 ? "the transport reported an error on gradient bucket %zu; communicator aborted"
                                         : "all-reduce of gradient bucket %zu did not complete within %.3g s; communicator aborted",
                 b, c->timeout_s);
        comm_fail(c, msg);
        lock.unlock();
        if (c->be.abort) c->be.abort(c->be.ctx);
        lock.lock();
        break;
      }
    }
  }
}

void check_alive(THGPUComm *c) {
  std::lock_guard<std::mutex> lock(c->mu);
  THC_CHECK(c->error.empty(), "%s", c->error.c_str());
}

}  // namespace
}  // namespace thc

using namespace thc;

THC_API THGPUComm *THGPUComm_newWithBackend(int world, int rank, const THGPUCommBackend *backend) {
  THC_BEGIN
  THC_ARG(world >= 1 && rank >= 0 && rank < world, 1, "rank must lie in [0, world)");
  THC_ARG(backend && backend->all_reduce && backend->join, 3, "a backend needs at least all_reduce and join");
  THGPUComm *c = new THGPUComm();
  c->world = world; c->rank = rank; c->be = *backend;
  c->watchdog = std::thread(watchdog_loop, c);
  return c;
  THC_END(nullptr)
}

THC_API void THGPUComm_free(THGPUComm *c) {
  if (!c) return;
  {
    std::lock_guard<std::mutex> lock(c->mu);
    c->stop = true;
  }
  c->cv.notify_all();
  if (c->watchdog.joinable()) c->watchdog.join();
  if (c->be.destroy) c->be.destroy(c->be.ctx);
  delete c;
}

THC_API const char *THGPUComm_error(THGPUComm *c) {
  std::lock_guard<std::mutex> lock(c->mu);
  return c->error.empty() ? nullptr : c->error.c_str();
}

THC_API int THGPUComm_setTimeout(THGPUComm *c, double seconds) {
  THC_BEGIN
  THC_ARG(seconds > 0, 2, "timeout must be positive");
  std::lock_guard<std::mutex> lock(c->mu);
  c->timeout_s = seconds;
  return 0;
  THC_END(1)
}

// bounds: 2 * nbuckets longs, bucket b = elements [bounds[2b], bounds[2b+1]) of flat_grad, in the order in which
// the backward pass completes them.  Every rank must pass the same numbers: checked over the transport before
// any gradient traffic is queued.
THC_API int THGPUComm_setBuckets(THGPUComm *c, THGPUTensor *flat_grad, const long *bounds, int nbuckets) {
  THC_BEGIN
  check_alive(c);
  THC_ARG(flat_grad && is_contiguous(flat_grad) && nelem(flat_grad) > 0, 2, "flat contiguous gradient buffer expected");
  THC_ARG(nbuckets >= 1 && nbuckets <= 1024 && bounds, 4, "between 1 and 1024 buckets expected");
  const long n = nelem(flat_grad);
  std::vector<long> sig;
  sig.push_back(n); sig.push_back(nbuckets);
  std::vector<char> covered((size_t)nbuckets, 0);
  for (int b = 0; b < nbuckets; b++) {
    const long lo = bounds[2 * b], hi = bounds[2 * b + 1];
    THC_ARG(lo >= 0 && hi > lo && hi <= n, 3, "bucket outside the gradient buffer");
    for (int a = 0; a < b; a++)
      THC_ARG(hi <= bounds[2 * a] || lo >= bounds[2 * a + 1], 3, "buckets overlap");
    sig.push_back(lo); sig.push_back(hi);
  }
  if (c->world > 1 && c->be.agree) {
    const int same = c->be.agree(c->be.ctx, sig.data(), (int)sig.size());
    THC_CHECK(same >= 0, "the transport failed while comparing the gradient layout across ranks");
    THC_CHECK(same == 1, "gradient layout differs between ranks (element count or bucket bounds): nothing was queued");
  }
  std::lock_guard<std::mutex> lock(c->mu);
  c->grad = data_ptr(flat_grad); c->n = n;
  c->begin.assign((size_t)nbuckets, 0); c->count.assign((size_t)nbuckets, 0);
  for (int b = 0; b < nbuckets; b++) { c->begin[b] = bounds[2 * b]; c->count[b] = bounds[2 * b + 1] - bounds[2 * b]; }
  c->launched.assign((size_t)nbuckets, 0); c->finished.assign((size_t)nbuckets, 0);
  c->deadline.assign((size_t)nbuckets, Clock::now());
  return 0;
  THC_END(1)
}

// After each bucket's all-reduce the backend updates that slice of the parameters: v = momentum * v + g;
// w -= lr * v (v NULL / momentum 0: w -= lr * g).  The buffers have the gradient buffer's layout.
THC_API int THGPUComm_setUpdate(THGPUComm *c, THGPUTensor *flat_w, THGPUTensor *flat_v, float lr, float momentum) {
  THC_BEGIN
  check_alive(c);
  THC_CHECK(c->n > 0, "set the gradient buckets first");
  THC_CHECK(c->be.set_update, "this backend has no parameter update");
  THC_ARG(flat_w && is_contiguous(flat_w) && nelem(flat_w) == c->n, 2, "weights must have the gradient buffer's size");
  float *v = nullptr;
  if (momentum != 0.f) {
    THC_ARG(flat_v && is_contiguous(flat_v) && nelem(flat_v) == c->n, 3, "velocity buffer of the gradient buffer's size expected");
    v = data_ptr(flat_v);
  }
  THC_CHECK(c->be.set_update(c->be.ctx, data_ptr(flat_w), v, lr, momentum) == 0, "the backend refused the update");
  c->update = true;
  return 0;
  THC_END(1)
}

THC_API int THGPUComm_allReduceAsync(THGPUComm *c, int bucket) {
  THC_BEGIN
  {
    std::lock_guard<std::mutex> lock(c->mu);
    THC_CHECK(c->error.empty(), "%s", c->error.c_str());
    THC_CHECK(c->n > 0, "set the gradient buckets first");
    THC_ARG(bucket >= 0 && bucket < (int)c->launched.size(), 2, "no such bucket");
    THC_CHECK(c->launched[bucket] != 1, "gradient bucket %d was already queued in this step", bucket);
  }
  const int rc = c->be.all_reduce(c->be.ctx, bucket, c->grad + c->begin[bucket], c->begin[bucket], c->count[bucket]);
  std::lock_guard<std::mutex> lock(c->mu);
  if (rc != 0) {
    comm_fail(c, "the transport failed to queue the all-reduce of gradient bucket " + std::to_string(bucket));
    THC_CHECK(false, "%s", c->error.c_str());
  }
  c->launched[bucket] = 1; c->finished[bucket] = 0;
  c->deadline[bucket] = Clock::now() + std::chrono::microseconds((long long)(c->timeout_s * 1e6));
  return 0;
  THC_END(1)
}

// Orders everything the caller queues next on the compute stream behind the all-reduces (and updates) of this
// step, and opens the next step.  Every bucket must have been queued: a forgotten bucket would leave its
// gradients unsummed on this rank and the other ranks waiting.
THC_API int THGPUComm_wait(THGPUComm *c) {
  THC_BEGIN
  {
    std::lock_guard<std::mutex> lock(c->mu);
    THC_CHECK(c->error.empty(), "%s", c->error.c_str());
    for (size_t b = 0; b < c->launched.size(); b++)
      THC_CHECK(c->launched[b] == 1, "gradient bucket %zu was never queued in this step", b);
  }
  const int rc = c->be.join(c->be.ctx);
  std::lock_guard<std::mutex> lock(c->mu);
  if (rc != 0) {
    comm_fail(c, "the transport failed while joining the streams");
    THC_CHECK(false, "%s", c->error.c_str());
  }
  // the watchdog keeps the deadlines of what is still in flight; a bucket may be queued again right away, the
  // stream order puts it behind its previous round
  for (size_t b = 0; b < c->launched.size(); b++)
    if (c->finished[b]) c->launched[b] = 0;
    else c->launched[b] = 2;          // in flight from the last round: still watched, may be queued again
  return 0;
  THC_END(1)
}

// ---- NCCL backend ------------------------------------------------------------------------------------------
namespace thc {
namespace {

struct Nccl {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;   // optional
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
// libnccl.so.2 is looked up when the first communicator is made: a process that never makes one (one GPU, or a
// host that brings its own exchange) does not need NCCL installed.
Nccl &nccl() {
  static Nccl n;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (n.handle) return n;
  // The copy the process already has, if any (a host framework that bundles its own NCCL): one process must not
  // end up with two.  Otherwise the system's, without exporting its symbols.  A host that loads a NEWER NCCL under
  // the same soname AFTER this call gets this one from the loader: such a host loads its own first.
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
  THC_CHECK(h, "libnccl.so.2 could not be loaded (%s): multi-GPU exchange is unavailable", dlerror());
#define THC_NCCL_SYM(field, name)                                              \
  n.field = reinterpret_cast<decltype(n.field)>(dlsym(h, name));               \
  THC_CHECK(n.field, "libnccl.so.2 has no symbol %s", name)
  THC_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
  THC_NCCL_SYM(CommInitRank, "ncclCommInitRank");
  n.CommInitRankConfig = reinterpret_cast<decltype(n.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
  THC_NCCL_SYM(AllReduce, "ncclAllReduce");
  THC_NCCL_SYM(CommDestroy, "ncclCommDestroy");
  THC_NCCL_SYM(CommAbort, "ncclCommAbort");
  THC_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  THC_NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef THC_NCCL_SYM
  n.handle = h;
  return n;
}
#define THC_NCCL(expr)                                                                                   \
  do { ncclResult_t r__ = (expr); if (r__ != ncclSuccess && r__ != ncclInProgress)                       \
    ::thc::fail("NCCL error at %s:%d: %s", __FILE__, __LINE__, nccl().GetErrorString(r__)); } while (0)

struct NcclBackend {
  int device = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  std::vector<cudaEvent_t> ready, done;
  std::vector<char> queued;
  long *agree_dev = nullptr;
  // parameter update behind each bucket
  float *w = nullptr, *v = nullptr;
  float lr = 0.f, momentum = 0.f;
  std::atomic<bool> aborted{false};
  void ensure_events(int bucket) {
    while ((int)ready.size() <= bucket) {
      cudaEvent_t a, b;
      THC_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
      THC_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
      ready.push_back(a); done.push_back(b); queued.push_back(0);
    }
  }
};

// C callbacks never let an exception out: they return a status.
#define THC_CB_BEGIN try {
#define THC_CB_END(fail_value) } catch (const std::exception &e__) { ::thc::record_error(e__.what()); return fail_value; }

int nccl_all_reduce(void *ctx, int bucket, float *data, long begin, long count) {
  THC_CB_BEGIN
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  b->ensure_events(bucket);
  // everything that wrote this slice is already queued on the compute stream
  THC_CUDA(cudaEventRecord(b->ready[bucket], stream()));
  THC_CUDA(cudaStreamWaitEvent(b->comm_stream, b->ready[bucket], 0));
  THC_NCCL(nccl().AllReduce(data, data, (size_t)count, ncclFloat, ncclSum, b->comm, b->comm_stream));
  if (b->w) sgd_update_async(b->w + begin, data, b->v ? b->v + begin : nullptr, count, b->lr, b->momentum, b->comm_stream);
  THC_CUDA(cudaEventRecord(b->done[bucket], b->comm_stream));
  b->queued[bucket] = 1;
  return 0;
  THC_CB_END(1)
}
int nccl_set_update(void *ctx, float *w, float *v, float lr, float momentum) {
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  b->w = w; b->v = v; b->lr = lr; b->momentum = momentum;
  return 0;
}
int nccl_done(void *ctx, int bucket) {   // called from the watchdog thread
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  if (b->aborted.load()) return -1;
  if (bucket >= (int)b->done.size()) return 0;
  cudaSetDevice(b->device);
  ncclResult_t async = ncclSuccess;
  if (nccl().CommGetAsyncError(b->comm, &async) == ncclSuccess && async != ncclSuccess && async != ncclInProgress) return -1;
  const cudaError_t e = cudaEventQuery(b->done[bucket]);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  cudaGetLastError();
  return -1;
}
int nccl_join(void *ctx) {
  THC_CB_BEGIN
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  for (size_t k = 0; k < b->done.size(); k++)
    if (b->queued[k]) { THC_CUDA(cudaStreamWaitEvent(stream(), b->done[k], 0)); b->queued[k] = 0; }
  return 0;
  THC_CB_END(1)
}
// Every rank passes its numbers; max and min over the ranks agree exactly when all ranks passed the same.
int nccl_agree(void *ctx, const long *values, int n) {
  THC_CB_BEGIN
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  THC_CHECK(n <= 4096, "layout signature too long");
  if (!b->agree_dev) THC_CUDA(cudaMalloc((void **)&b->agree_dev, sizeof(long) * 3 * 4096));
  long *in = b->agree_dev, *mx = in + 4096, *mn = mx + 4096;
  THC_CUDA(cudaMemcpyAsync(in, values, sizeof(long) * n, cudaMemcpyHostToDevice, b->comm_stream));
  THC_NCCL(nccl().AllReduce(in, mx, (size_t)n, ncclInt64, ncclMax, b->comm, b->comm_stream));
  THC_NCCL(nccl().AllReduce(in, mn, (size_t)n, ncclInt64, ncclMin, b->comm, b->comm_stream));
  std::vector<long> host(2 * (size_t)n);
  THC_CUDA(cudaMemcpyAsync(host.data(), mx, sizeof(long) * n, cudaMemcpyDeviceToHost, b->comm_stream));
  THC_CUDA(cudaMemcpyAsync(host.data() + n, mn, sizeof(long) * n, cudaMemcpyDeviceToHost, b->comm_stream));
  THC_CUDA(cudaStreamSynchronize(b->comm_stream));
  for (int i = 0; i < n; i++)
    if (host[i] != host[n + i]) return 0;
  return 1;
  THC_CB_END(-1)
}
int nccl_abort(void *ctx) {
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  if (!b->aborted.exchange(true) && b->comm) nccl().CommAbort(b->comm);
  return 0;
}
void nccl_destroy(void *ctx) {
  NcclBackend *b = static_cast<NcclBackend *>(ctx);
  cudaSetDevice(b->device);
  if (b->comm_stream) cudaStreamSynchronize(b->comm_stream);
  if (b->comm && !b->aborted.load()) nccl().CommDestroy(b->comm);
  for (cudaEvent_t e : b->ready) cudaEventDestroy(e);
  for (cudaEvent_t e : b->done) cudaEventDestroy(e);
  if (b->agree_dev) cudaFree(b->agree_dev);
  if (b->comm_stream) cudaStreamDestroy(b->comm_stream);
  delete b;
}

}  // namespace
}  // namespace thc

THC_API int THGPUComm_getUniqueId(void *id_out) {
  THC_BEGIN
  static_assert(sizeof(ncclUniqueId) == 128, "the C ABI states 128 bytes");
  THC_NCCL(nccl().GetUniqueId(static_cast<ncclUniqueId *>(id_out)));
  return 0;
  THC_END(1)
}

// One communicator per rank (= per process and GPU).  `unique_id`: the 128 bytes rank 0 got from
// THGPUComm_getUniqueId, handed to the other ranks by whatever the host has (a file, MPI, torch.distributed).
// `max_ctas` > 0 caps the thread blocks (= SMs) a collective of this communicator may occupy.  The gradient
// exchange of a step needs a fraction of NVLink's bandwidth, and every SM a collective holds is one the
// persistent matrix-multiply launches of the backward pass running beside it cannot use; 0 leaves NCCL's default.
THC_API THGPUComm *THGPUComm_newWithOptions(int world, int rank, const void *unique_id, int max_ctas) {
  THC_BEGIN
  THC_ARG(world >= 1 && rank >= 0 && rank < world, 2, "rank must lie in [0, world)");
  THC_ARG(unique_id, 3, "unique id expected");
  Context &c = ctx();
  NcclBackend *b = new NcclBackend();
  b->device = c.device;
  struct Guard { NcclBackend *b; ~Guard() { if (b) nccl_destroy(b); } } guard{b};
  int lo, hi;
  THC_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  THC_CUDA(cudaStreamCreateWithPriority(&b->comm_stream, cudaStreamNonBlocking, hi));
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  if (max_ctas > 0 && nccl().CommInitRankConfig) {
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.maxCTAs = max_ctas;
    cfg.minCTAs = 1;
    THC_NCCL(nccl().CommInitRankConfig(&b->comm, world, id, rank, &cfg));
  } else {
    THC_NCCL(nccl().CommInitRank(&b->comm, world, id, rank));
  }
  THGPUCommBackend be;
  be.all_reduce = nccl_all_reduce; be.set_update = nccl_set_update; be.done = nccl_done; be.join = nccl_join;
  be.agree = nccl_agree; be.abort = nccl_abort; be.destroy = nccl_destroy; be.ctx = b;
  THGPUComm *comm = THGPUComm_newWithBackend(world, rank, &be);
  THC_CHECK(comm, "could not create the communicator");
  guard.b = nullptr;
  return comm;
  THC_END(nullptr)
}
THC_API THGPUComm *THGPUComm_new(int world, int rank, const void *unique_id) {
  return THGPUComm_newWithOptions(world, rank, unique_id, 0);
}
