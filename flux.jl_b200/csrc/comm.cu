// DistributedUtils collectives over NCCL (NVLink 5 / NVSwitch): communicator bootstrap, mean all-reduce of
// gradient buffers, broadcast of parameters / optimiser state, reduce-to-root.
//
// libnccl is opened at run time (the copy already loaded into the process is preferred), so the library
// itself loads on machines without NCCL; the fb_comm_* calls then fail with FB_ERR_NCCL.
#include <dlfcn.h>

#include "common.cuh"

namespace {

struct NcclUniqueId { char internal[FB_UNIQUE_ID_BYTES]; };
typedef void* NcclComm;
constexpr int NCCL_FLOAT32 = 7, NCCL_SUM = 0, NCCL_AVG = 4;

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*CommAbort)(NcclComm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*Reduce)(const void*, void*, size_t, int, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*CommGetAsyncError)(NcclComm, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (int pass = 0; pass < 2 && !api.handle; ++pass)
    for (const char* nm : names) {
      api.handle = dlopen(nm, RTLD_NOW | RTLD_LOCAL | (pass == 0 ? RTLD_NOLOAD : 0));
      if (api.handle) break;
    }
  if (!api.handle) return api;
#define FB_SYM(field, name) *(void**)(&api.field) = dlsym(api.handle, name)
  FB_SYM(GetUniqueId, "ncclGetUniqueId");
  FB_SYM(CommInitRank, "ncclCommInitRank");
  FB_SYM(CommDestroy, "ncclCommDestroy");
  FB_SYM(CommAbort, "ncclCommAbort");
  FB_SYM(AllReduce, "ncclAllReduce");
  FB_SYM(Broadcast, "ncclBroadcast");
  FB_SYM(Reduce, "ncclReduce");
  FB_SYM(ReduceScatter, "ncclReduceScatter");
  FB_SYM(AllGather, "ncclAllGather");
  FB_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  FB_SYM(GetErrorString, "ncclGetErrorString");
#undef FB_SYM
  api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.Broadcast && api.Reduce &&
           api.GetErrorString;
  return api;
}

int32_t nccl_fail(const char* what, int rc) {
  NcclApi& n = nccl();
  return fb_fail(FB_ERR_NCCL, "%s failed: %s", what, n.GetErrorString ? n.GetErrorString(rc) : "unknown NCCL error");
}

}  // namespace

struct fb_comm {
  NcclComm comm;
  int rank, nranks, device;
};

#define FB_NCCL_READY()                                                                                   \
  NcclApi& n = nccl();                                                                                    \
  if (!n.ok) return fb_fail(FB_ERR_NCCL, "%s: libnccl.so.2 could not be loaded (%s)", __func__, dlerror() ? "dlopen failed" : "missing symbols")

FB_API int32_t fb_comm_get_unique_id(void* id_host) {
  FB_REQUIRE(id_host, FB_ERR_INVALID_ARG, "fb_comm_get_unique_id: NULL pointer");
  FB_NCCL_READY();
  NcclUniqueId id;
  const int rc = n.GetUniqueId(&id);
  if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
  memcpy(id_host, id.internal, FB_UNIQUE_ID_BYTES);
  return FB_OK;
}

FB_API int32_t fb_comm_init_rank(fb_ctx* ctx, const void* id_host, int32_t nranks, int32_t rank, fb_comm** out) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(id_host && out, FB_ERR_INVALID_ARG, "fb_comm_init_rank: NULL pointer");
  FB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, FB_ERR_INVALID_ARG, "fb_comm_init_rank: rank %d of %d", rank, nranks);
  FB_NCCL_READY();
  FB_CUDA(cudaSetDevice(ctx->device));
  NcclUniqueId id;
  memcpy(id.internal, id_host, FB_UNIQUE_ID_BYTES);
  NcclComm c = nullptr;
  const int rc = n.CommInitRank(&c, nranks, id, rank);
  if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
  fb_comm* fc = new fb_comm();
  fc->comm = c; fc->rank = rank; fc->nranks = nranks; fc->device = ctx->device;
  *out = fc;
  return FB_OK;
}

FB_API int32_t fb_comm_destroy(fb_comm* comm) {
  if (!comm) return FB_OK;
  NcclApi& n = nccl();
  if (n.ok && comm->comm) n.CommDestroy(comm->comm);
  delete comm;
  return FB_OK;
}

FB_API int32_t fb_comm_rank(const fb_comm* comm) { return comm ? comm->rank : -1; }
FB_API int32_t fb_comm_size(const fb_comm* comm) { return comm ? comm->nranks : -1; }

FB_API int32_t fb_allreduce(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t op) {
  FB_REQUIRE(comm, FB_ERR_INVALID_ARG, "fb_allreduce: comm is NULL");
  FB_REQUIRE(count >= 0 && (op == FB_OP_SUM || op == FB_OP_AVG), FB_ERR_INVALID_ARG, "fb_allreduce: bad count or op");
  if (count == 0) return FB_OK;
  FB_REQUIRE(send && recv, FB_ERR_INVALID_ARG, "fb_allreduce: NULL pointer");
  FB_NCCL_READY();
  const int rc = n.AllReduce(send, recv, (size_t)count, NCCL_FLOAT32, op == FB_OP_AVG ? NCCL_AVG : NCCL_SUM, comm->comm,
                             (cudaStream_t)stream);
  if (rc != 0) return nccl_fail("ncclAllReduce", rc);
  return FB_OK;
}

FB_API int32_t fb_reduce_scatter(fb_comm* comm, void* stream, const float* send, float* recv, int64_t recv_count, int32_t op) {
  FB_REQUIRE(comm, FB_ERR_INVALID_ARG, "fb_reduce_scatter: comm is NULL");
  FB_REQUIRE(recv_count >= 0, FB_ERR_INVALID_ARG, "fb_reduce_scatter: negative count");
  FB_REQUIRE(op == FB_OP_SUM || op == FB_OP_AVG, FB_ERR_INVALID_ARG, "fb_reduce_scatter: op must be FB_OP_SUM or FB_OP_AVG");
  if (recv_count == 0) return FB_OK;
  FB_REQUIRE(send && recv, FB_ERR_INVALID_ARG, "fb_reduce_scatter: NULL pointer");
  NcclApi& n = nccl();
  if (!n.ok || !n.ReduceScatter) return fb_fail(FB_ERR_NCCL, "fb_reduce_scatter: NCCL is not available");
  const int rc = n.ReduceScatter(send, recv, (size_t)recv_count, NCCL_FLOAT32, op == FB_OP_AVG ? NCCL_AVG : NCCL_SUM,
                                 comm->comm, (cudaStream_t)stream);
  if (rc != 0) return nccl_fail("ncclReduceScatter", rc);
  return FB_OK;
}

FB_API int32_t fb_allgather(fb_comm* comm, void* stream, const float* send, float* recv, int64_t send_count) {
  FB_REQUIRE(comm, FB_ERR_INVALID_ARG, "fb_allgather: comm is NULL");
  FB_REQUIRE(send_count >= 0, FB_ERR_INVALID_ARG, "fb_allgather: negative count");
  if (send_count == 0) return FB_OK;
  FB_REQUIRE(send && recv, FB_ERR_INVALID_ARG, "fb_allgather: NULL pointer");
  NcclApi& n = nccl();
  if (!n.ok || !n.AllGather) return fb_fail(FB_ERR_NCCL, "fb_allgather: NCCL is not available");
  const int rc = n.AllGather(send, recv, (size_t)send_count, NCCL_FLOAT32, comm->comm, (cudaStream_t)stream);
  if (rc != 0) return nccl_fail("ncclAllGather", rc);
  return FB_OK;
}

FB_API int32_t fb_bcast(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t root) {
  FB_REQUIRE(comm, FB_ERR_INVALID_ARG, "fb_bcast: comm is NULL");
  FB_REQUIRE(count >= 0 && root >= 0 && root < comm->nranks, FB_ERR_INVALID_ARG, "fb_bcast: bad count or root");
  if (count == 0) return FB_OK;
  FB_REQUIRE(send && recv, FB_ERR_INVALID_ARG, "fb_bcast: NULL pointer");
  FB_NCCL_READY();
  const int rc = n.Broadcast(send, recv, (size_t)count, NCCL_FLOAT32, root, comm->comm, (cudaStream_t)stream);
  if (rc != 0) return nccl_fail("ncclBroadcast", rc);
  return FB_OK;
}

FB_API int32_t fb_reduce(fb_comm* comm, void* stream, const float* send, float* recv, int64_t count, int32_t op,
                         int32_t root) {
  FB_REQUIRE(comm, FB_ERR_INVALID_ARG, "fb_reduce: comm is NULL");
  FB_REQUIRE(count >= 0 && (op == FB_OP_SUM || op == FB_OP_AVG) && root >= 0 && root < comm->nranks, FB_ERR_INVALID_ARG,
             "fb_reduce: bad count, op or root");
  if (count == 0) return FB_OK;
  FB_REQUIRE(send && recv, FB_ERR_INVALID_ARG, "fb_reduce: NULL pointer");
  FB_NCCL_READY();
  const int rc = n.Reduce(send, recv, (size_t)count, NCCL_FLOAT32, op == FB_OP_AVG ? NCCL_AVG : NCCL_SUM, root, comm->comm,
                          (cudaStream_t)stream);
  if (rc != 0) return nccl_fail("ncclReduce", rc);
  return FB_OK;
}

FB_API int32_t fb_comm_async_error(fb_comm* comm, int32_t* out_host) {
  FB_REQUIRE(comm && out_host, FB_ERR_INVALID_ARG, "fb_comm_async_error: NULL pointer");
  FB_NCCL_READY();
  *out_host = 0;
  if (!n.CommGetAsyncError) return FB_OK;
  int err = 0;
  const int rc = n.CommGetAsyncError(comm->comm, &err);
  if (rc != 0) return nccl_fail("ncclCommGetAsyncError", rc);
  *out_host = err;
  return FB_OK;
}

// ------------------------------------------------------------------------------------------- gradient buckets ---
// The native form of the bucketed, overlapped gradient averaging: a flat gradient buffer cut into buckets; every
// gradient leaf is a slice of it.  The reverse sweep marks a leaf ready when its gradient has been written (stream
// order); when the last leaf of a bucket is ready the bucket's mean all-reduce starts on the communication stream
// while the compute stream goes on.  fb_bucket_wait makes the compute stream wait for every bucket.
struct fb_bucket_set {
  fb_comm* comm;
  float* flat;
  int64_t total;
  int nbuckets;
  int64_t* start;        // [nbuckets + 1]
  int* leaves_in;        // leaves registered per bucket
  int* pending;          // leaves not yet ready in this step
  int* launched;
  cudaEvent_t* ready_ev; // compute stream -> communication stream
  cudaEvent_t* done_ev;  // communication stream -> compute stream
  int nleaves, cap_leaves;
  int* leaf_bucket;
  unsigned char* leaf_ready;
  cudaStream_t comm_stream;
  int own_stream;
};

static int32_t bucket_launch(fb_bucket_set* b, int bi, cudaStream_t compute) {
  b->launched[bi] = 1;
  if (b->comm == nullptr || b->comm->nranks == 1) return FB_OK;   // one worker: the mean is the gradient itself
  FB_CUDA(cudaEventRecord(b->ready_ev[bi], compute));
  FB_CUDA(cudaStreamWaitEvent(b->comm_stream, b->ready_ev[bi], 0));
  float* p = b->flat + b->start[bi];
  const int32_t st = fb_allreduce(b->comm, (void*)b->comm_stream, p, p, b->start[bi + 1] - b->start[bi], FB_OP_AVG);
  if (st != FB_OK) return st;
  FB_CUDA(cudaEventRecord(b->done_ev[bi], b->comm_stream));
  return FB_OK;
}

FB_API int32_t fb_bucket_create(fb_ctx* ctx, fb_comm* comm, float* flat, int64_t total, int32_t nbuckets,
                                const int64_t* bucket_ends_host, void* comm_stream, fb_bucket_set** out) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out != nullptr, FB_ERR_INVALID_ARG, "fb_bucket_create: out is NULL");
  *out = nullptr;
  FB_REQUIRE(flat != nullptr && total >= 1 && nbuckets >= 1 && bucket_ends_host != nullptr, FB_ERR_INVALID_ARG,
             "fb_bucket_create: bad arguments");
  int64_t prev = 0;
  for (int i = 0; i < nbuckets; ++i) {
    FB_REQUIRE(bucket_ends_host[i] > prev && bucket_ends_host[i] <= total, FB_ERR_INVALID_ARG,
               "fb_bucket_create: bucket ends must increase and stay inside the buffer");
    prev = bucket_ends_host[i];
  }
  FB_REQUIRE(prev == total, FB_ERR_INVALID_ARG, "fb_bucket_create: the last bucket must end at %lld", (long long)total);
  FB_CUDA(cudaSetDevice(ctx->device));
  fb_bucket_set* b = new fb_bucket_set();
  b->comm = comm; b->flat = flat; b->total = total; b->nbuckets = nbuckets;
  b->start = new int64_t[nbuckets + 1];
  b->start[0] = 0;
  for (int i = 0; i < nbuckets; ++i) b->start[i + 1] = bucket_ends_host[i];
  b->leaves_in = new int[nbuckets]();
  b->pending = new int[nbuckets]();
  b->launched = new int[nbuckets]();
  b->ready_ev = new cudaEvent_t[nbuckets];
  b->done_ev = new cudaEvent_t[nbuckets];
  for (int i = 0; i < nbuckets; ++i) {
    cudaEventCreateWithFlags(&b->ready_ev[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&b->done_ev[i], cudaEventDisableTiming);
  }
  b->nleaves = 0; b->cap_leaves = 64;
  b->leaf_bucket = new int[b->cap_leaves];
  b->leaf_ready = new unsigned char[b->cap_leaves];
  b->comm_stream = (cudaStream_t)comm_stream;
  b->own_stream = 0;
  if (b->comm_stream == nullptr) {
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (cudaStreamCreateWithPriority(&b->comm_stream, cudaStreamNonBlocking, hi) != cudaSuccess) {
      cudaGetLastError();
      fb_bucket_destroy(b);
      return fb_fail(FB_ERR_CUDA, "fb_bucket_create: could not create the communication stream");
    }
    b->own_stream = 1;
  }
  *out = b;
  return FB_OK;
}

FB_API int32_t fb_bucket_destroy(fb_bucket_set* b) {
  if (b == nullptr) return FB_OK;
  if (b->own_stream && b->comm_stream) {
    cudaStreamSynchronize(b->comm_stream);
    cudaStreamDestroy(b->comm_stream);
  }
  for (int i = 0; i < b->nbuckets; ++i) {
    cudaEventDestroy(b->ready_ev[i]);
    cudaEventDestroy(b->done_ev[i]);
  }
  delete[] b->start; delete[] b->leaves_in; delete[] b->pending; delete[] b->launched;
  delete[] b->ready_ev; delete[] b->done_ev; delete[] b->leaf_bucket; delete[] b->leaf_ready;
  delete b;
  return FB_OK;
}

FB_API int32_t fb_bucket_register(fb_bucket_set* b, int64_t offset, int64_t count, int32_t* leaf_id) {
  FB_REQUIRE(b != nullptr && leaf_id != nullptr, FB_ERR_INVALID_ARG, "fb_bucket_register: NULL pointer");
  FB_REQUIRE(offset >= 0 && count >= 1 && offset + count <= b->total, FB_ERR_INVALID_ARG,
             "fb_bucket_register: slice [%lld, %lld) is outside the buffer", (long long)offset, (long long)(offset + count));
  int bi = 0;
  while (bi < b->nbuckets && offset >= b->start[bi + 1]) ++bi;
  FB_REQUIRE(offset + count <= b->start[bi + 1], FB_ERR_INVALID_ARG, "fb_bucket_register: a leaf must lie inside one bucket");
  if (b->nleaves == b->cap_leaves) {
    const int cap = 2 * b->cap_leaves;
    int* lb = new int[cap];
    unsigned char* lr = new unsigned char[cap];
    memcpy(lb, b->leaf_bucket, sizeof(int) * b->nleaves);
    memcpy(lr, b->leaf_ready, b->nleaves);
    delete[] b->leaf_bucket; delete[] b->leaf_ready;
    b->leaf_bucket = lb; b->leaf_ready = lr; b->cap_leaves = cap;
  }
  b->leaf_bucket[b->nleaves] = bi;
  b->leaf_ready[b->nleaves] = 0;
  b->leaves_in[bi] += 1;
  b->pending[bi] += 1;
  *leaf_id = b->nleaves++;
  return FB_OK;
}

FB_API int32_t fb_bucket_begin_step(fb_bucket_set* b) {
  FB_REQUIRE(b != nullptr, FB_ERR_INVALID_ARG, "fb_bucket_begin_step: NULL pointer");
  for (int i = 0; i < b->nbuckets; ++i) {
    b->pending[i] = b->leaves_in[i];
    b->launched[i] = 0;
  }
  memset(b->leaf_ready, 0, (size_t)b->nleaves);
  return FB_OK;
}

FB_API int32_t fb_bucket_mark_ready(fb_bucket_set* b, int32_t leaf_id, void* compute_stream) {
  FB_REQUIRE(b != nullptr && leaf_id >= 0 && leaf_id < b->nleaves, FB_ERR_INVALID_ARG, "fb_bucket_mark_ready: bad leaf id %d", leaf_id);
  if (b->leaf_ready[leaf_id]) return FB_OK;
  b->leaf_ready[leaf_id] = 1;
  const int bi = b->leaf_bucket[leaf_id];
  if (--b->pending[bi] == 0 && !b->launched[bi]) return bucket_launch(b, bi, (cudaStream_t)compute_stream);
  return FB_OK;
}

FB_API int32_t fb_bucket_wait(fb_bucket_set* b, void* compute_stream) {
  FB_REQUIRE(b != nullptr, FB_ERR_INVALID_ARG, "fb_bucket_wait: NULL pointer");
  for (int i = 0; i < b->nbuckets; ++i)
    if (!b->launched[i]) {
      const int32_t st = bucket_launch(b, i, (cudaStream_t)compute_stream);
      if (st != FB_OK) return st;
    }
  if (b->comm != nullptr && b->comm->nranks > 1)
    for (int i = 0; i < b->nbuckets; ++i) FB_CUDA(cudaStreamWaitEvent((cudaStream_t)compute_stream, b->done_ev[i], 0));
  return FB_OK;
}
