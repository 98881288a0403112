// Whole-tensor predicates: Engine.HasNaN / Engine.HasInf (gorgonia cuda/engine.go:144-191).
//
// The reference kernels (cuda modules/src/misc.cu:13-55) bump a counter without atomics and
// are handed a host address; here each warp votes and one lane per warp that saw a hit sets a
// flag word in the engine's device scratch, which the host reads back after the kernel.
#include "engine.h"
#include "ptx.cuh"

namespace b200 {

template <typename T, bool INF>
__global__ void __launch_bounds__(256) has_special_kernel(const T *__restrict__ x, long long n, int *flag) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool hit = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const T v = x[i];
    hit |= INF ? (isinf(v) != 0) : (v != v);
  }
  if (__any_sync(0xffffffffu, hit) && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

template <bool INF>
static int has_special(b200_engine *e, int dtype, const void *x, int64_t n, int *result, const char *who) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, result != nullptr, "%s: result is null", who);
  *result = 0;
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "%s: dtype %d not supported", who, dtype);
  B200_REQUIRE(e, n >= 0, "%s: negative element count", who);
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, x != nullptr, "%s: null pointer", who);
  B200_NOT_WHILE_CAPTURING(e, who);
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  int *flag = e->d_flags + (INF ? 1 : 0);
  B200_CHECK_CUDA(e, cudaMemsetAsync(flag, 0, sizeof(int), e->stream));
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)std::max<long long>(1, std::min<long long>(want, (long long)e->sm_count * 8));
  if (dtype == B200_F32)
    has_special_kernel<float, INF><<<blocks, threads, 0, e->stream>>>((const float *)x, n, flag);
  else
    has_special_kernel<double, INF><<<blocks, threads, 0, e->stream>>>((const double *)x, n, flag);
  B200_CHECK_LAUNCH(e, "has_special_kernel");
  B200_CHECK_CUDA(e, cudaMemcpyAsync(e->h_flags, flag, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
  rc = sync_stream_checked(e);
  if (rc != B200_OK) return rc;
  *result = e->h_flags[0] != 0;
  return B200_OK;
}

// One warp; lane 0 waits on a barrier that expects one arrival and gets none. The wait is the
// library's ordinary bounded wait with a short limit: it gives up, raises the error word the way
// the tensor-core kernels do, and the kernel returns normally.
__global__ void selftest_wait_kernel(unsigned long long limit_ns, int *err_flag) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
    if (!ptx::mbar_wait(&bar, 0, limit_ns)) atomicExch(err_flag, 1);
    ptx::mbar_inval(&bar);
  }
}

}  // namespace b200

extern "C" {
int b200_has_nan(b200_engine *e, int dtype, const void *x, int64_t n, int *result) {
  return b200::has_special<false>(e, dtype, x, n, result, "b200_has_nan");
}
int b200_has_inf(b200_engine *e, int dtype, const void *x, int64_t n, int *result) {
  return b200::has_special<true>(e, dtype, x, n, result, "b200_has_inf");
}

int b200_selftest_wait(b200_engine *e, int64_t limit_us) {
  using namespace b200;
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, limit_us >= 1 && limit_us <= 10000, "b200_selftest_wait: limit of 1 .. 10000 microseconds");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  selftest_wait_kernel<<<1, 32, 0, e->stream>>>((unsigned long long)limit_us * 1000ull, e->d_flags + 2);
  B200_CHECK_LAUNCH(e, "selftest_wait_kernel");
  e->flags_dirty = true;
  return B200_OK;
}
}
