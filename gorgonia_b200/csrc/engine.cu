// Engine lifecycle, arena, copies, error reporting.
//
// Replaces, behind the C ABI: Engine.Init/doInit/Close/DoWork/Signal/Sync
// (gorgonia cuda/external.go:88-276), Engine.Get/Put/ResetAllocator (cuda/arena.go:13-36),
// Engine.Memcpy/Alloc/Free (cuda/engine.go:72-138) and the host<->device moves of
// ExternMetadata.Transfer (cuda.go:168-207) and deviceTransport.exec (vm_tape_cuda.go:220-243).
//
// Differences by design: one cudaMalloc'd (or, on request, managed) slab per engine with a
// best-fit allocator on the host; one non-blocking stream per engine instead of the default
// stream; no worker thread and no call batching, since a call through this ABI is one plain
// function call rather than a queue of cgo crossings.
#include "engine.h"

#include <cstring>

namespace b200 {

thread_local std::string g_create_error;

int set_error(b200_engine *e, int code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (e)
    e->last_error = buf;
  else
    g_create_error = buf;
  return code;
}

bool is_constant(b200_engine *e, const void *ptr) { return e->constants.count(ptr) != 0; }

CachedSplit *find_cached(b200_engine *e, const void *ptr, int kind, long long d0, long long d1, long long d2,
                         long long ld_in) {
  auto it = e->constants.find(ptr);
  if (it == e->constants.end()) return nullptr;
  for (auto &c : it->second.derived)
    if (c.kind == kind && c.d0 == d0 && c.d1 == d1 && c.d2 == d2 && c.ld_in == ld_in) {
      pin_cached(e, c);  // whoever asks is about to launch a kernel that reads it
      return &c;
    }
  return nullptr;
}

void add_cached(b200_engine *e, const void *ptr, const CachedSplit &c) {
  e->constants[ptr].derived.push_back(c);
  pin_cached(e, c);
}

void arena_release(b200_engine *e, int64_t off) {
  if (!e->bfc.is_live(off)) return;
  if (e->capturing) {
    // the recording's kernels keep this address: reusable inside the recording, the tape's afterwards
    const int64_t sz = e->bfc.live_size(off);
    auto range = e->capture_free.equal_range(sz);
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == off) return;  // handed back twice
    e->capture_free.insert({sz, off});
    return;
  }
  if (e->pins.count(off)) {
    e->zombies.insert(off);  // a recorded tape still reads it
    return;
  }
  // a plain arena free: whoever gets the block next runs later on the same stream
  e->bfc.free(off);
}

void pin_cached(b200_engine *e, const CachedSplit &c) {
  if (!e->capturing) return;
  for (const void *p : {(const void *)c.hi, (const void *)c.lo}) {
    const int64_t off = (const char *)p - (const char *)e->slab;
    if (p && off >= 0 && off < e->slab_bytes) e->capture_pins.push_back(off);
  }
}

void drop_constant(b200_engine *e, const void *ptr) {
  auto it = e->constants.find(ptr);
  if (it == e->constants.end()) return;
  for (auto &c : it->second.derived) {
    int64_t off = (char *)c.hi - (char *)e->slab;
    if (off >= 0 && off < e->slab_bytes) arena_release(e, off);
    off = (char *)c.lo - (char *)e->slab;
    if (off >= 0 && off < e->slab_bytes) arena_release(e, off);
  }
  e->constants.erase(it);
}

int sync_stream_checked(b200_engine *e) {
  if (e->flags_dirty) {
    // kernels with bounded waits report a wait that ran out through d_flags[2]
    // d_flags[3]: a gather met an index outside its range; a replayed tape cannot say so itself
    B200_CHECK_CUDA(e, cudaMemcpyAsync(e->h_flags + 2, e->d_flags + 2, 2 * sizeof(int), cudaMemcpyDeviceToHost,
                                       e->stream));
    B200_CHECK_CUDA(e, cudaStreamSynchronize(e->stream));
    e->flags_dirty = false;
    const bool gather = e->gather_dirty;
    e->gather_dirty = false;
    if (e->h_flags[2] != 0) {
      e->h_flags[2] = 0;
      cudaMemsetAsync(e->d_flags + 2, 0, sizeof(int), e->stream);
      // a kernel that gave up may have left tiles half delivered: re-arm the arrival counters
      cudaMemsetAsync(e->sk_counters, 0, b200_engine::kSkCounters * sizeof(int), e->stream);
      return set_error(e, B200_ERR_TIMEOUT, "a device-side wait ran out of time; results of the last "
                       "kernels are incomplete");
    }
    if (gather && e->h_flags[3] != 0) {
      cudaMemsetAsync(e->d_flags + 3, 0, sizeof(int), e->stream);
      return set_error(e, B200_ERR_INVALID, "a replayed tape holds a gather whose index lies outside its "
                       "range; those rows were not written");
    }
    return B200_OK;
  }
  B200_CHECK_CUDA(e, cudaStreamSynchronize(e->stream));
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_set_constant(b200_engine *e, const void *ptr, int is_const) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, ptr != nullptr, "b200_set_constant: null pointer");
  if (is_const)
    e->constants[ptr];  // creates the entry
  else
    drop_constant(e, ptr);
  return B200_OK;
}

int b200_engine_create(int device, size_t arena_bytes, unsigned flags, b200_engine **out) {
  if (!out) return set_error(nullptr, B200_ERR_INVALID, "b200_engine_create: out is null");
  *out = nullptr;
  int ndev = 0;
  cudaError_t err = cudaGetDeviceCount(&ndev);
  if (err != cudaSuccess)
    return set_error(nullptr, B200_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(err));
  if (device < 0 || device >= ndev)
    return set_error(nullptr, B200_ERR_INVALID, "device %d out of range (%d devices)", device, ndev);
  cudaDeviceProp prop;
  err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess)
    return set_error(nullptr, B200_ERR_CUDA, "cudaGetDeviceProperties failed: %s", cudaGetErrorString(err));
  if (prop.major != 10)
    return set_error(nullptr, B200_ERR_UNSUPPORTED,
                     "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major,
                     prop.minor);

  b200_engine *e = new b200_engine();
  e->device = device;
  e->flags = flags;
  e->sm_count = prop.multiProcessorCount;
  e->smem_optin = prop.sharedMemPerBlockOptin;
  int prev = -1;
  cudaGetDevice(&prev);
  auto fail = [&](const char *what, cudaError_t ce) {
    set_error(nullptr, B200_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(ce));
    if (e->slab) cudaFree(e->slab);
    if (e->d_flags) cudaFree(e->d_flags);
    if (e->sk_counters) cudaFree(e->sk_counters);
    if (e->h_flags) cudaFreeHost(e->h_flags);
    if (e->upload_done) cudaEventDestroy(e->upload_done);
    if (e->compute_mark) cudaEventDestroy(e->compute_mark);
    if (e->copy_stream) cudaStreamDestroy(e->copy_stream);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
    if (prev >= 0) cudaSetDevice(prev);
    return B200_ERR_CUDA;
  };
  if ((err = cudaSetDevice(device)) != cudaSuccess) return fail("cudaSetDevice", err);
  if ((err = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail("cudaStreamCreateWithFlags", err);
  if ((err = cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail("cudaStreamCreateWithFlags", err);
  if ((err = cudaEventCreateWithFlags(&e->upload_done, cudaEventDisableTiming)) != cudaSuccess ||
      (err = cudaEventCreateWithFlags(&e->compute_mark, cudaEventDisableTiming)) != cudaSuccess)
    return fail("cudaEventCreateWithFlags", err);
  if (arena_bytes == 0) arena_bytes = (size_t)256 << 20;
  arena_bytes = (arena_bytes + 255) / 256 * 256;
  if (flags & B200_ENGINE_MANAGED) {
    if ((err = cudaMallocManaged(&e->slab, arena_bytes, cudaMemAttachGlobal)) != cudaSuccess)
      return fail("cudaMallocManaged", err);
    // keep the pages in HBM: kernels stream from device memory, host reads fault pages over
    cudaMemAdvise(e->slab, arena_bytes, cudaMemAdviseSetPreferredLocation, device);
    cudaMemPrefetchAsync(e->slab, arena_bytes, device, e->stream);
    cudaGetLastError();
  } else {
    if ((err = cudaMalloc(&e->slab, arena_bytes)) != cudaSuccess) {
      int rc = fail("cudaMalloc(arena)", err);
      (void)rc;
      return B200_ERR_OOM;
    }
  }
  e->slab_bytes = (int64_t)arena_bytes;
  e->bfc.reserve(e->slab_bytes, 256);
  if ((err = cudaMalloc((void **)&e->d_flags, 16 * sizeof(int))) != cudaSuccess)
    return fail("cudaMalloc(flags)", err);
  if ((err = cudaMemset(e->d_flags, 0, 16 * sizeof(int))) != cudaSuccess) return fail("cudaMemset", err);
  if ((err = cudaMalloc((void **)&e->sk_counters, b200_engine::kSkCounters * sizeof(int))) != cudaSuccess)
    return fail("cudaMalloc(counters)", err);
  if ((err = cudaMemset(e->sk_counters, 0, b200_engine::kSkCounters * sizeof(int))) != cudaSuccess)
    return fail("cudaMemset", err);
  if ((err = cudaHostAlloc((void **)&e->h_flags, 16 * sizeof(int), cudaHostAllocDefault)) != cudaSuccess)
    return fail("cudaHostAlloc", err);
  memset(e->h_flags, 0, 16 * sizeof(int));
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  *out = e;
  return B200_OK;
}

int b200_engine_destroy(b200_engine *e) {
  if (!e) return B200_OK;
  {
    std::lock_guard<std::recursive_mutex> lk(e->mu);
    DeviceGuard g(e);
    e->pending.clear();
    cudaStreamSynchronize(e->stream);
    if (e->gemm_state && e->gemm_state_free) e->gemm_state_free(e->gemm_state);
    if (e->slab) cudaFree(e->slab);
    if (e->d_flags) cudaFree(e->d_flags);
    if (e->sk_counters) cudaFree(e->sk_counters);
    if (e->reduce_scratch) cudaFree(e->reduce_scratch);
    if (e->h_flags) cudaFreeHost(e->h_flags);
    cudaStreamSynchronize(e->copy_stream);
    cudaEventDestroy(e->upload_done);
    cudaEventDestroy(e->compute_mark);
    cudaStreamDestroy(e->copy_stream);
    cudaStreamDestroy(e->stream);
  }
  delete e;
  return B200_OK;
}

int b200_engine_device(const b200_engine *e) { return e ? e->device : -1; }
uintptr_t b200_engine_stream(const b200_engine *e) { return e ? (uintptr_t)e->stream : 0; }
uint64_t b200_launch_count(const b200_engine *e) { return e ? e->launches : 0; }

const char *b200_last_error(const b200_engine *e) {
  return e ? e->last_error.c_str() : g_create_error.c_str();
}

int b200_flush(b200_engine *e) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  DeviceGuard g(e);
  return flush_pending(e);
}

int b200_sync(b200_engine *e) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_NOT_WHILE_CAPTURING(e, "b200_sync");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  return sync_stream_checked(e);
}

/* ---- tapes: a recorded sequence of engine calls replayed with one call ---- */

struct b200_tape {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t launches = 0;  // kernels recorded, so that replays keep the launch counter honest
  // Arena blocks the recorded kernels use although nobody else holds them any more: scratch the
  // library took and handed back while recording, and buffers the caller released while recording.
  // They stay allocated until the tape is destroyed (gorgonia frees a register at its last use,
  // vm_tape.go:639-653; a replay is a use).
  std::vector<int64_t> held;
  std::vector<int64_t> pinned;  // derived forms of constants the tape reads (see b200_engine::pins)
  uint64_t arena_epoch = 0;
  bool has_gather = false;
};

// Ends the special treatment of blocks released during a recording that produced no tape.
static void abandon_capture_blocks(b200_engine *e) {
  for (auto &kv : e->capture_free) e->bfc.free(kv.second);
  e->capture_free.clear();
  e->capture_pins.clear();
}

int b200_tape_begin(b200_engine *e) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (e->capturing) return set_error(e, B200_ERR_STATE, "b200_tape_begin: a tape is already being recorded");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  B200_CHECK_CUDA(e, cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
  e->capturing = true;
  e->capture_free.clear();
  e->capture_pins.clear();
  e->capture_has_gather = false;
  e->capture_launch_base = e->launches;
  return B200_OK;
}

int b200_tape_end(b200_engine *e, b200_tape **out) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (!e->capturing) return set_error(e, B200_ERR_STATE, "b200_tape_end: no tape is being recorded");
  B200_REQUIRE(e, out != nullptr, "b200_tape_end: out is null");
  *out = nullptr;
  DeviceGuard g(e);
  int rc = flush_pending(e);  // queued pointwise calls belong to the tape
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
  e->capturing = false;
  if (rc != B200_OK) {
    if (graph) cudaGraphDestroy(graph);
    abandon_capture_blocks(e);
    return rc;
  }
  if (ce != cudaSuccess) {
    cudaGetLastError();
    abandon_capture_blocks(e);
    return set_error(e, B200_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(ce));
  }
  b200_tape *t = new b200_tape();
  t->graph = graph;
  t->launches = e->launches - e->capture_launch_base;
  e->launches = e->capture_launch_base;  // nothing ran yet
  ce = cudaGraphInstantiate(&t->exec, graph, 0);
  if (ce != cudaSuccess) {
    cudaGetLastError();
    cudaGraphDestroy(graph);
    delete t;
    abandon_capture_blocks(e);
    return set_error(e, B200_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(ce));
  }
  t->arena_epoch = e->arena_epoch;
  t->has_gather = e->capture_has_gather;
  for (auto &kv : e->capture_free) t->held.push_back(kv.second);
  e->capture_free.clear();
  t->pinned.swap(e->capture_pins);
  for (int64_t off : t->pinned) e->pins[off]++;
  *out = t;
  return B200_OK;
}

int b200_tape_launch(b200_engine *e, b200_tape *t) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, t && t->exec, "b200_tape_launch: null tape");
  if (e->capturing) return set_error(e, B200_ERR_STATE, "b200_tape_launch: a tape is being recorded");
  if (t->arena_epoch != e->arena_epoch)
    return set_error(e, B200_ERR_STATE, "b200_tape_launch: the arena was reset after this tape was recorded; "
                     "its buffers may belong to someone else now");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  B200_CHECK_CUDA(e, cudaGraphLaunch(t->exec, e->stream));
  e->launches += t->launches;
  e->flags_dirty = true;
  if (t->has_gather) e->gather_dirty = true;
  return B200_OK;
}

int b200_tape_destroy(b200_engine *e, b200_tape *t) {
  if (!t) return B200_OK;
  if (e) {
    std::lock_guard<std::recursive_mutex> lk(e->mu);
    DeviceGuard g(e);
    cudaStreamSynchronize(e->stream);
    if (t->exec) cudaGraphExecDestroy(t->exec);
    if (t->graph) cudaGraphDestroy(t->graph);
    if (t->arena_epoch == e->arena_epoch) {
      for (int64_t off : t->held) arena_release(e, off);
      for (int64_t off : t->pinned) {
        auto it = e->pins.find(off);
        if (it == e->pins.end()) continue;
        if (--it->second > 0) continue;
        e->pins.erase(it);
        if (e->zombies.erase(off)) arena_release(e, off);
      }
    }
  }
  delete t;
  return B200_OK;
}

/* ---- events ---- */

int b200_event_create(b200_engine *e, void **event) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, event != nullptr, "b200_event_create: null pointer");
  DeviceGuard g(e);
  cudaEvent_t ev;
  B200_CHECK_CUDA(e, cudaEventCreate(&ev));
  *event = (void *)ev;
  return B200_OK;
}
int b200_event_record(b200_engine *e, void *event) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, event != nullptr, "b200_event_record: null event");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  B200_CHECK_CUDA(e, cudaEventRecord((cudaEvent_t)event, e->stream));
  return B200_OK;
}
int b200_event_elapsed_ms(b200_engine *e, void *start, void *stop, float *ms) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, start && stop && ms, "b200_event_elapsed_ms: null pointer");
  DeviceGuard g(e);
  B200_CHECK_CUDA(e, cudaEventSynchronize((cudaEvent_t)stop));
  B200_CHECK_CUDA(e, cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return B200_OK;
}
int b200_event_destroy(b200_engine *e, void *event) {
  if (!e) return B200_ERR_INVALID;
  if (!event) return B200_OK;
  DeviceGuard g(e);
  B200_CHECK_CUDA(e, cudaEventDestroy((cudaEvent_t)event));
  return B200_OK;
}

/* ---- arena ---- */

int b200_get(b200_engine *e, int64_t bytes, void **dptr) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dptr != nullptr, "b200_get: dptr is null");
  *dptr = nullptr;
  B200_REQUIRE(e, bytes > 0, "b200_get: cannot allocate %lld bytes", (long long)bytes);
  int64_t off = 0;
  if (e->capturing && !e->capture_free.empty()) {
    // blocks released earlier in this recording: their last recorded user runs before this one
    const int64_t need = (bytes + e->bfc.align() - 1) / e->bfc.align() * e->bfc.align();
    auto it = e->capture_free.lower_bound(need);
    if (it != e->capture_free.end() && it->first <= need + need / 4) {
      *dptr = (char *)e->slab + it->second;
      e->capture_free.erase(it);
      return B200_OK;
    }
  }
  int rc = e->bfc.alloc(bytes, &off);
  if (rc == -2) {
    // Queued writes to buffers that were already handed back keep nothing alive, but a flush
    // lets a caller that frees and retries succeed; report the shortage as the reference does.
    return set_error(e, B200_ERR_OOM, "out of memory: requested %lld bytes, %lld of %lld in use",
                     (long long)bytes, (long long)e->bfc.used(), (long long)e->bfc.capacity());
  }
  if (rc != 0) return set_error(e, B200_ERR_INVALID, "b200_get: bad size %lld", (long long)bytes);
  *dptr = (char *)e->slab + off;
  return B200_OK;
}

int b200_put(b200_engine *e, void *dptr, int64_t /*bytes*/) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (!dptr) return B200_OK;
  int64_t off = (char *)dptr - (char *)e->slab;
  if (off < 0 || off >= e->slab_bytes) return B200_OK;  // not ours: no-op, as in the reference
  if (e->bfc.is_live(off)) note_put(e, dptr);
  drop_constant(e, dptr);  // a released buffer is no longer a constant; what was derived from it goes too
  arena_release(e, off);
  return B200_OK;
}

int b200_reset(b200_engine *e) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (e->capturing)
    return set_error(e, B200_ERR_STATE, "b200_reset: a tape is being recorded");
  DeviceGuard g(e);
  // queued work may still read or write arena blocks: run it before the blocks are recycled
  int rc = flush_pending(e);
  e->constants.clear();  // derived blocks live in the arena that is being reset
  // tapes recorded before this point keep addresses that are about to be handed out again:
  // they must not be replayed, and they give nothing back when they are destroyed
  e->arena_epoch++;
  e->pins.clear();
  e->zombies.clear();
  e->bfc.reset();
  return rc;
}

int b200_arena_stats(b200_engine *e, int64_t *used, int64_t *free_bytes, int64_t *largest_free,
                     int64_t *n_free_blocks) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (used) *used = e->bfc.used();
  if (free_bytes) *free_bytes = e->bfc.capacity() - e->bfc.used();
  if (largest_free) *largest_free = e->bfc.largest_free();
  if (n_free_blocks) *n_free_blocks = e->bfc.free_blocks();
  return B200_OK;
}

/* ---- allocator without a device ---- */

struct b200_bfc {
  b200::Bfc impl;
};

b200_bfc *b200_bfc_create(int64_t bytes, int64_t align) {
  if (bytes <= 0 || align <= 0) return nullptr;
  b200_bfc *a = new b200_bfc();
  a->impl.reserve(bytes, align);
  return a;
}
void b200_bfc_destroy(b200_bfc *a) { delete a; }
int b200_bfc_alloc(b200_bfc *a, int64_t bytes, int64_t *offset) {
  if (!a || !offset) return B200_ERR_INVALID;
  int rc = a->impl.alloc(bytes, offset);
  return rc == 0 ? B200_OK : (rc == -2 ? B200_ERR_OOM : B200_ERR_INVALID);
}
int b200_bfc_free(b200_bfc *a, int64_t offset) {
  if (!a) return B200_ERR_INVALID;
  a->impl.free(offset);
  return B200_OK;
}
void b200_bfc_reset(b200_bfc *a) {
  if (a) a->impl.reset();
}
int64_t b200_bfc_free_blocks(const b200_bfc *a) { return a ? a->impl.free_blocks() : -1; }
int64_t b200_bfc_used(const b200_bfc *a) { return a ? a->impl.used() : -1; }
int64_t b200_bfc_largest_free(const b200_bfc *a) { return a ? a->impl.largest_free() : -1; }

/* ---- copies ---- */

static int copy_common(b200_engine *e, void *dst, const void *src, int64_t bytes, cudaMemcpyKind kind,
                       bool wait, const char *who) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, bytes >= 0, "%s: negative size", who);
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(e, dst && src, "%s: null pointer", who);
  if (wait) B200_NOT_WHILE_CAPTURING(e, who);
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  B200_CHECK_CUDA(e, cudaMemcpyAsync(dst, src, (size_t)bytes, kind, e->stream));
  if (wait) return sync_stream_checked(e);  // the bytes just read may come from a kernel whose wait ran out
  return B200_OK;
}

int b200_memcpy_h2d(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  // pageable sources are staged by the runtime before the call returns; waiting keeps the
  // contract simple: the host buffer may be reused as soon as this returns
  return copy_common(e, dst, src, bytes, cudaMemcpyHostToDevice, true, "b200_memcpy_h2d");
}
int b200_memcpy_d2h(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  return copy_common(e, dst, src, bytes, cudaMemcpyDeviceToHost, true, "b200_memcpy_d2h");
}
int b200_memcpy_d2d(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  return copy_common(e, dst, src, bytes, cudaMemcpyDeviceToDevice, false, "b200_memcpy_d2d");
}
int b200_memcpy_h2d_async(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  return copy_common(e, dst, src, bytes, cudaMemcpyHostToDevice, false, "b200_memcpy_h2d_async");
}
int b200_memcpy_d2h_async(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  return copy_common(e, dst, src, bytes, cudaMemcpyDeviceToHost, false, "b200_memcpy_d2h_async");
}
int b200_memset(b200_engine *e, void *dst, int value, int64_t bytes) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, bytes >= 0, "b200_memset: negative size");
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(e, dst != nullptr, "b200_memset: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  B200_CHECK_CUDA(e, cudaMemsetAsync(dst, value, (size_t)bytes, e->stream));
  return B200_OK;
}

/* ---- uploads that overlap compute ---- */

int b200_upload_async(b200_engine *e, void *dst, const void *src, int64_t bytes) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, bytes >= 0, "b200_upload_async: negative size");
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(e, dst && src, "b200_upload_async: null pointer");
  B200_NOT_WHILE_CAPTURING(e, "b200_upload_async");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  // the copy may not overtake compute work queued so far: that work may still read `dst`
  B200_CHECK_CUDA(e, cudaEventRecord(e->compute_mark, e->stream));
  B200_CHECK_CUDA(e, cudaStreamWaitEvent(e->copy_stream, e->compute_mark, 0));
  B200_CHECK_CUDA(e, cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, e->copy_stream));
  B200_CHECK_CUDA(e, cudaEventRecord(e->upload_done, e->copy_stream));
  return B200_OK;
}

int b200_upload_wait(b200_engine *e) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_NOT_WHILE_CAPTURING(e, "b200_upload_wait");
  DeviceGuard g(e);
  B200_CHECK_CUDA(e, cudaStreamWaitEvent(e->stream, e->upload_done, 0));
  return B200_OK;
}

int b200_host_alloc(int64_t bytes, void **hptr) {
  if (!hptr || bytes <= 0) return B200_ERR_INVALID;
  cudaError_t err = cudaHostAlloc(hptr, (size_t)bytes, cudaHostAllocDefault);
  if (err != cudaSuccess) {
    set_error(nullptr, B200_ERR_CUDA, "cudaHostAlloc failed: %s", cudaGetErrorString(err));
    return B200_ERR_CUDA;
  }
  return B200_OK;
}
int b200_host_free(void *hptr) {
  if (!hptr) return B200_OK;
  return cudaFreeHost(hptr) == cudaSuccess ? B200_OK : B200_ERR_CUDA;
}

}  // extern "C"
