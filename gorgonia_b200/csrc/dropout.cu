// Dropout without cuDNN: dropoutOp.do / dropoutDiffOp (gorgonia op_dropout.go:106-128,205-240), which
// the reference's CUDA build replaces with cuDNN's dropout (ops/nn/dropout_cuda.go:76-149).
//
// Forward, for keep = 1 - probability:  y[i] = r[i] < keep ? x[i] / keep : 0, with keep rounded to the
// tensor's type first, as the reference does. r[i] is either read from a device array the caller
// passes (gorgonia injects its generator the same way, which is what its own test relies on:
// op_dropout_test.go:14-68) or drawn on the fly from Philox-4x32-10 keyed by `seed`, counter =
// element index: no state, no mask tensor, the same numbers on every replay of a recorded tape.
// Backward, as the reference writes it:  dx[i] = (probability != 0 && y[i] != 0) ? dy[i] / probability : 0.
// It tells kept elements from dropped ones by the forward output, not by a mask, and it divides by
// the drop probability, not by the keep probability; both are reproduced.
#include "engine.h"

namespace b200 {

// Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11).
__host__ __device__ inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t (&out)[4]) {
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Uniform draw for element i: float32 takes word i % 4 of block i / 4 (24 bits), float64 takes the
// word pair (2 (i % 2), 2 (i % 2) + 1) of block i / 2 (53 bits). Both lie in [0, 1).
template <typename T>
__device__ __forceinline__ T philox_uniform(unsigned long long seed, unsigned long long i);
template <>
__device__ __forceinline__ float philox_uniform<float>(unsigned long long seed, unsigned long long i) {
  uint32_t r[4];
  const unsigned long long blk = i >> 2;
  philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
  return (float)(r[i & 3] >> 8) * 5.9604644775390625e-08f;  // 2^-24
}
template <>
__device__ __forceinline__ double philox_uniform<double>(unsigned long long seed, unsigned long long i) {
  uint32_t r[4];
  const unsigned long long blk = i >> 1;
  philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
  const uint32_t a = r[2 * (i & 1)], b = r[2 * (i & 1) + 1];
  return ((double)(a >> 5) * 67108864.0 + (double)(b >> 6)) * 1.1102230246251565e-16;  // 2^-53
}

template <typename T>
__global__ void __launch_bounds__(256) dropout_fwd_kernel(const T *__restrict__ x, T *__restrict__ y, long long n,
                                                          T keep, const T *__restrict__ rnd, unsigned long long seed,
                                                          unsigned long long offset) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const T r = rnd ? rnd[i] : philox_uniform<T>(seed, offset + (unsigned long long)i);
    y[i] = r < keep ? x[i] / keep : T(0);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dropout_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ out,
                                                          T *__restrict__ dx, long long n, T prob) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = (prob != T(0) && out[i] != T(0)) ? dy[i] / prob : T(0);
}

static int grid_of(const b200_engine *e, long long n) {
  const long long want = (n + 255) / 256;
  return (int)std::max<long long>(1, std::min<long long>(want, (long long)e->sm_count * 16));
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_dropout_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t n, double probability,
                     const void *uniforms, uint64_t seed, uint64_t offset) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_dropout_fwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_dropout_fwd: negative element count");
  B200_REQUIRE(e, probability >= 0.0 && probability <= 1.0, "b200_dropout_fwd: probability %g outside [0, 1]",
               probability);
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, x && y, "b200_dropout_fwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (probability == 0.0) {  // the reference hands the input through (op_dropout.go:81-83)
    if (x != y)
      B200_CHECK_CUDA(e, cudaMemcpyAsync(y, x, (size_t)n * dtype_size(dtype), cudaMemcpyDeviceToDevice, e->stream));
    return B200_OK;
  }
  if (dtype == B200_F32)
    dropout_fwd_kernel<float><<<grid_of(e, n), 256, 0, e->stream>>>((const float *)x, (float *)y, n,
                                                                   (float)(1.0 - probability),
                                                                   (const float *)uniforms, seed, offset);
  else
    dropout_fwd_kernel<double><<<grid_of(e, n), 256, 0, e->stream>>>((const double *)x, (double *)y, n,
                                                                    1.0 - probability, (const double *)uniforms, seed,
                                                                    offset);
  B200_CHECK_LAUNCH(e, "dropout_fwd_kernel");
  return B200_OK;
}

int b200_dropout_bwd(b200_engine *e, int dtype, const void *dy, const void *out, void *dx, int64_t n,
                     double probability) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_dropout_bwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_dropout_bwd: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, dy && out && dx, "b200_dropout_bwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32)
    dropout_bwd_kernel<float><<<grid_of(e, n), 256, 0, e->stream>>>((const float *)dy, (const float *)out, (float *)dx,
                                                                   n, (float)probability);
  else
    dropout_bwd_kernel<double><<<grid_of(e, n), 256, 0, e->stream>>>((const double *)dy, (const double *)out,
                                                                    (double *)dx, n, probability);
  B200_CHECK_LAUNCH(e, "dropout_bwd_kernel");
  return B200_OK;
}

}  // extern "C"
