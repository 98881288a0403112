// The one collective of the training variant: the mean of a flat gradient bucket over the ranks.
//
// gorgonia has no distributed path (its data-parallel precedent applies the gradients of several
// VMs serially through one solver: example_concurrent_training_test.go:80-115). Here every rank
// holds a replica; after the last backward kernel the bucket is summed over the ranks and divided
// by their number before Solver.Step (solvers.go:13-15). The forward path never comes here.
//
// The transport sits behind a function pointer, so that the host program chooses it and the error
// paths can be exercised among CPU ranks: b200_comm_create wraps any all-reduce (a Go program's own,
// a test's), b200_comm_create_nccl binds NCCL, found at run time by its soname, on the engine's
// stream (rings or trees over NVLink / NVSwitch are NCCL's choice).
#include <dlfcn.h>

#include "engine.h"

struct b200_comm {
  b200_allreduce_fn fn = nullptr;
  void *ctx = nullptr;
  int rank = 0, world = 1;
  // NCCL binding (b200_comm_create_nccl)
  void *dl = nullptr;
  void *nccl_comm = nullptr;
  int (*nccl_allreduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
  int (*nccl_destroy)(void *) = nullptr;
  const char *(*nccl_errstr)(int) = nullptr;
  std::string last_error;
};

namespace b200 {

static void *open_nccl(std::string *why) {
  for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
    if (void *h = dlopen(name, RTLD_NOW | RTLD_GLOBAL)) return h;
  }
  *why = dlerror() ? dlerror() : "libnccl.so.2 not found";
  return nullptr;
}

static int nccl_transport(void *ctx, void *buf, int64_t count, int dtype, uintptr_t stream) {
  b200_comm *c = (b200_comm *)ctx;
  const int nccl_type = dtype == B200_F32 ? 7 : 8;  // ncclFloat32 / ncclFloat64
  return c->nccl_allreduce(buf, buf, (size_t)count, nccl_type, 0 /* ncclSum */, c->nccl_comm, (cudaStream_t)stream);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_comm_create(b200_allreduce_fn fn, void *ctx, int rank, int world, b200_comm **out) {
  if (!out) return B200_ERR_INVALID;
  *out = nullptr;
  if (!fn || world < 1 || rank < 0 || rank >= world) return B200_ERR_INVALID;
  b200_comm *c = new b200_comm();
  c->fn = fn;
  c->ctx = ctx;
  c->rank = rank;
  c->world = world;
  *out = c;
  return B200_OK;
}

int b200_comm_destroy(b200_comm *c) {
  if (!c) return B200_OK;
  if (c->nccl_comm && c->nccl_destroy) c->nccl_destroy(c->nccl_comm);
  if (c->dl) dlclose(c->dl);
  delete c;
  return B200_OK;
}

int b200_comm_world(const b200_comm *c) { return c ? c->world : 0; }
int b200_comm_rank(const b200_comm *c) { return c ? c->rank : -1; }
const char *b200_comm_last_error(const b200_comm *c) { return c ? c->last_error.c_str() : ""; }

int b200_nccl_unique_id(void *id128) {
  if (!id128) return B200_ERR_INVALID;
  std::string why;
  void *dl = open_nccl(&why);
  if (!dl) return B200_ERR_UNSUPPORTED;
  auto get = (int (*)(void *))dlsym(dl, "ncclGetUniqueId");
  const int rc = get ? get(id128) : -1;
  dlclose(dl);
  return rc == 0 ? B200_OK : B200_ERR_CUDA;
}

int b200_comm_create_nccl(b200_engine *e, const void *id128, int rank, int world, b200_comm **out) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, out != nullptr && id128 != nullptr, "b200_comm_create_nccl: null pointer");
  *out = nullptr;
  B200_REQUIRE(e, world >= 1 && rank >= 0 && rank < world, "b200_comm_create_nccl: rank %d of %d", rank, world);
  std::string why;
  void *dl = open_nccl(&why);
  if (!dl) return set_error(e, B200_ERR_UNSUPPORTED, "NCCL is not available: %s", why.c_str());
  struct Id { char bytes[128]; } id;
  memcpy(id.bytes, id128, 128);
  auto init = (int (*)(void **, int, Id, int))dlsym(dl, "ncclCommInitRank");
  b200_comm *c = new b200_comm();
  c->dl = dl;
  c->nccl_allreduce = (decltype(c->nccl_allreduce))dlsym(dl, "ncclAllReduce");
  c->nccl_destroy = (decltype(c->nccl_destroy))dlsym(dl, "ncclCommDestroy");
  c->nccl_errstr = (decltype(c->nccl_errstr))dlsym(dl, "ncclGetErrorString");
  if (!init || !c->nccl_allreduce || !c->nccl_destroy) {
    b200_comm_destroy(c);
    return set_error(e, B200_ERR_UNSUPPORTED, "the NCCL library lacks ncclCommInitRank / ncclAllReduce / ncclCommDestroy");
  }
  DeviceGuard g(e);
  const int rc = init(&c->nccl_comm, world, id, rank);
  if (rc != 0) {
    const char *txt = c->nccl_errstr ? c->nccl_errstr(rc) : "";
    c->nccl_comm = nullptr;
    b200_comm_destroy(c);
    return set_error(e, B200_ERR_CUDA, "ncclCommInitRank failed (%d): %s", rc, txt);
  }
  c->fn = nccl_transport;
  c->ctx = c;
  c->rank = rank;
  c->world = world;
  *out = c;
  return B200_OK;
}

int b200_allreduce_mean(b200_engine *e, b200_comm *c, void *dptr, int64_t n, int dtype) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, c != nullptr && c->fn != nullptr, "b200_allreduce_mean: no communicator");
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_allreduce_mean: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_allreduce_mean: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, dptr != nullptr, "b200_allreduce_mean: null pointer");
  B200_NOT_WHILE_CAPTURING(e, "b200_allreduce_mean");
  if (c->world == 1) return B200_OK;
  DeviceGuard g(e);
  int rc = flush_pending(e);  // the bucket must be complete on the engine's stream
  if (rc != B200_OK) return rc;
  const int trc = c->fn(c->ctx, dptr, n, dtype, (uintptr_t)e->stream);
  if (trc != 0) {
    const char *txt = (c->nccl_comm && c->nccl_errstr) ? c->nccl_errstr(trc) : "";
    return set_error(e, B200_ERR_CUDA, "the all-reduce failed on rank %d of %d (transport code %d) %s; the bucket is "
                     "not a mean", c->rank, c->world, trc, txt);
  }
  // sum / world on the engine's stream, after the collective
  return b200_binary(e, B200_OP_DIV, dtype, B200_VS, dptr, dptr, nullptr, (double)c->world, 0, n);
}

int b200_comm_allreduce_mean_host(b200_comm *c, void *buf, int64_t n, int dtype) {
  if (!c || !c->fn) return B200_ERR_INVALID;
  if ((dtype != B200_F32 && dtype != B200_F64) || n < 0) {
    c->last_error = "b200_comm_allreduce_mean_host: bad dtype or count";
    return B200_ERR_INVALID;
  }
  if (n == 0 || c->world == 1) return B200_OK;
  if (!buf) {
    c->last_error = "b200_comm_allreduce_mean_host: null pointer";
    return B200_ERR_INVALID;
  }
  const int trc = c->fn(c->ctx, buf, n, dtype, 0);
  if (trc != 0) {
    char msg[160];
    snprintf(msg, sizeof msg, "the all-reduce failed on rank %d of %d (transport code %d); the bucket is not a mean",
             c->rank, c->world, trc);
    c->last_error = msg;
    return B200_ERR_CUDA;
  }
  if (dtype == B200_F32) {
    float *p = (float *)buf;
    const float w = (float)c->world;
    for (int64_t i = 0; i < n; ++i) p[i] = p[i] / w;
  } else {
    double *p = (double *)buf;
    const double w = (double)c->world;
    for (int64_t i = 0; i < n; ++i) p[i] = p[i] / w;
  }
  return B200_OK;
}

}  // extern "C"
