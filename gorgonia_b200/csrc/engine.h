// Internal definition of the engine handle shared by the .cu files of the library.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/gorgonia_b200.h"
#include "bfc.h"

namespace b200 {
// A derived form of a constant buffer (weights) kept for reuse: the TF32 head/tail split of a
// matrix (kind 0) or of convolution filters permuted to (tap, channel) order (kind 1).
struct CachedSplit {
  int kind;
  long long d0, d1, d2, ld_in;  // the shape it was made for
  void *hi, *lo;                // arena blocks
  long long ld_out;
};
struct ConstantEntry {
  std::vector<CachedSplit> derived;
};
}  // namespace b200

struct b200_engine {
  int device = 0;
  unsigned flags = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;      // uploads that overlap compute (b200_upload_*)
  cudaEvent_t upload_done = nullptr;       // last upload queued on copy_stream
  cudaEvent_t compute_mark = nullptr;      // point of the compute stream an upload must not pass
  int sm_count = 148;
  size_t smem_optin = 0;

  // arena
  void *slab = nullptr;
  int64_t slab_bytes = 0;
  b200::Bfc bfc;

  // buffers the caller declared constant (b200_set_constant), with what was derived from them
  std::map<const void *, b200::ConstantEntry> constants;

  // deferred pointwise queue
  std::vector<b200_pw_call> pending;
  std::vector<void *> dead;  // (pointer, queue length) pairs: buffers returned to the arena while writes to them were queued

  // small device scratch owned by the engine: flag words for has_nan/has_inf and the
  // error word bounded waits report through
  int *d_flags = nullptr;   // 16 ints
  int *h_flags = nullptr;   // pinned mirror
  bool flags_dirty = false; // a kernel that may raise d_flags[2] (bounded wait ran out) was launched

  void *reduce_scratch = nullptr;  // partials + ticket of the whole-tensor reduction (reduce.cu)
  // Arrival counters of the tensor-core kernels that share tiles' k ranges between CTAs (one per
  // tile). Zero between launches: the CTA that completes a tile puts its counter back to zero.
  int *sk_counters = nullptr;
  static constexpr int kSkCounters = 1 << 16;

  // lazily created resources of other translation units (gemm.cu etc.)
  void *gemm_state = nullptr;
  void (*gemm_state_free)(void *) = nullptr;

  bool capturing = false;   // between b200_tape_begin and b200_tape_end
  bool capture_has_gather = false;  // the recording holds a gather, whose index check replays with it
  bool gather_dirty = false;        // such a tape was replayed since the last synchronising call
  // A recorded tape keeps the addresses its kernels were launched with, so arena blocks handed
  // back while recording stay allocated: they may serve later requests of the same recording
  // (stream order), and at b200_tape_end they become the tape's until b200_tape_destroy.
  std::multimap<int64_t, int64_t> capture_free;  // size -> offset
  std::vector<int64_t> capture_pins;             // blocks derived from constants that the recording reads
  std::map<int64_t, int> pins;                   // offset -> live tapes reading it
  std::set<int64_t> zombies;                     // released while pinned: freed with the last tape
  uint64_t arena_epoch = 0;                      // bumped by b200_reset; older tapes own nothing
  uint64_t launches = 0;
  uint64_t capture_launch_base = 0;
  std::string last_error;
  std::recursive_mutex mu;
};

namespace b200 {

extern thread_local std::string g_create_error;

int set_error(b200_engine *e, int code, const char *fmt, ...);

#define B200_CHECK_CUDA(e, call)                                                       \
  do {                                                                                 \
    cudaError_t err__ = (call);                                                        \
    if (err__ != cudaSuccess) {                                                        \
      cudaGetLastError(); /* do not let it resurface at the next launch check */       \
      return b200::set_error((e), B200_ERR_CUDA, "%s failed: %s (%s:%d)", #call,       \
                             cudaGetErrorString(err__), __FILE__, __LINE__);           \
    }                                                                                  \
  } while (0)

#define B200_REQUIRE(e, cond, ...)                                       \
  do {                                                                   \
    if (!(cond)) return b200::set_error((e), B200_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// Makes the engine's device current for the calling thread.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(const b200_engine *e) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != e->device) ok = cudaSetDevice(e->device) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Launch-error check used after every <<<>>>.
#define B200_CHECK_LAUNCH(e, name)                                                     \
  do {                                                                                 \
    cudaError_t err__ = cudaGetLastError();                                            \
    if (err__ != cudaSuccess)                                                          \
      return b200::set_error((e), B200_ERR_CUDA, "launch of %s failed: %s", (name),    \
                             cudaGetErrorString(err__));                               \
    (e)->launches++;                                                                   \
  } while (0)

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case B200_F32: return 4;
    case B200_F64: return 8;
    case B200_BF16: return 2;
    default: return 0;
  }
}

// Entry points that must wait for the device cannot run while a tape is being recorded.
#define B200_NOT_WHILE_CAPTURING(e, who)                                                          \
  do {                                                                                            \
    if ((e)->capturing)                                                                           \
      return b200::set_error((e), B200_ERR_STATE, "%s waits for the device and cannot be recorded " \
                             "into a tape", (who));                                               \
  } while (0)

// constants (engine.cu)
CachedSplit *find_cached(b200_engine *e, const void *ptr, int kind, long long d0, long long d1, long long d2,
                         long long ld_in);
bool is_constant(b200_engine *e, const void *ptr);
void add_cached(b200_engine *e, const void *ptr, const CachedSplit &c);
void drop_constant(b200_engine *e, const void *ptr);
// Hands an arena block back, honouring a recording in progress and tapes that still read it.
void arena_release(b200_engine *e, int64_t off);
// Called with a derived form that a launch is about to read: a recording keeps it alive.
void pin_cached(b200_engine *e, const CachedSplit &c);

// Waits for the engine's stream; B200_ERR_TIMEOUT if a kernel launched since the last check gave
// up a bounded wait. Every entry point that synchronises goes through it.
int sync_stream_checked(b200_engine *e);

// implemented in pointwise.cu
int flush_pending(b200_engine *e);
int plan_pending(b200_engine *e, int *n_kernels);
void note_put(b200_engine *e, void *ptr);

}  // namespace b200
