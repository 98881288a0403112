// BLAS-2 kernels (matrix-vector, outer product) and the general CUDA-core matrix multiply.
//
// Engine.MatVecMul and Engine.Outer of gorgonia (cuda/linalg.go:47-107, 232-285) call cuBLAS
// Sgemv / Sger; both are bound by HBM, not by arithmetic, so they are written here as streaming
// kernels: 128-bit loads, one warp per matrix row with a shuffle reduction (A x), column strips
// with a deterministic two-pass reduction through arena scratch (A^T x), 128-bit stores (x y^T).
//
// gemm_simt is the matrix multiply for everything the tensor-core path (gemm_tc.cu) does not
// take: float64, shapes whose leading dimensions break TMA's 16-byte rule, and problems too
// small to fill a 128-row tile. Row-major operands with leading dimensions, either operand
// transposed, batched with strides, the same fused epilogue as the tensor-core kernel.
#include <algorithm>

#include "engine.h"
#include "epilogue.cuh"

namespace b200 {

__device__ __forceinline__ float fma_(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double fma_(double a, double b, double c) { return fma(a, b, c); }

// ---- y = A x : one warp per row ---------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) gemv_n_kernel(const T *__restrict__ A, long long lda, const T *__restrict__ x,
                                                     T *__restrict__ y, long long M, long long N) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < M; r += nwarps) {
    const T *a = A + r * lda;
    T acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = T(0);
    if (VEC) {
      const long long nv = N / V;
      long long c = lane;
      // four 16-byte loads of the matrix row in flight per lane before any of them is used: the
      // row is streamed once from HBM, and bytes in flight are what a streaming kernel lives on
      for (; c + 96 < nv; c += 128) {
        uint4 ra[4], rx[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) ra[u] = __ldcs(reinterpret_cast<const uint4 *>(a + (c + 32 * u) * V));
#pragma unroll
        for (int u = 0; u < 4; ++u) rx[u] = __ldg(reinterpret_cast<const uint4 *>(x + (c + 32 * u) * V));
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          T av[V], xv[V];
          memcpy(av, &ra[u], 16);
          memcpy(xv, &rx[u], 16);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = fma_(av[j], xv[j], acc[j]);
        }
      }
      for (; c < nv; c += 32) {
        const uint4 ra = *reinterpret_cast<const uint4 *>(a + c * V);
        const uint4 rx = __ldg(reinterpret_cast<const uint4 *>(x + c * V));
        T av[V], xv[V];
        memcpy(av, &ra, 16);
        memcpy(xv, &rx, 16);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = fma_(av[j], xv[j], acc[j]);
      }
      for (long long c = nv * V + lane; c < N; c += 32) acc[0] = fma_(a[c], x[c], acc[0]);
    } else {
      for (long long c = lane; c < N; c += 32) acc[0] = fma_(a[c], x[c], acc[0]);
    }
    T s = acc[0];
#pragma unroll
    for (int j = 1; j < V; ++j) s += acc[j];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) y[r] = s;
  }
}

// ---- y = A x for long rows: x staged in shared memory -------------------------------------------------
// The warp-per-row kernel reads as many bytes of x (from L1/L2) as of A. Here the eight warps of a block take
// eight consecutive rows and share each 32 KB piece of x through shared memory, so x passes through the load
// pipe once per block instead of once per warp. Every row's sums are formed in the same order as in
// gemv_n_kernel: the results are the same bits.
template <typename T>
__global__ void __launch_bounds__(256) gemv_n_smemx_kernel(const T *__restrict__ A, long long lda,
                                                           const T *__restrict__ x, T *__restrict__ y, long long M,
                                                           long long N) {
  constexpr int V = 16 / sizeof(T);
  constexpr int CH = 2048;  // 16-byte pieces of x per chunk
  __shared__ uint4 xs[CH];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long nv = N / V;
  const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
  for (long long row0 = (long long)blockIdx.x * 8; row0 < M; row0 += (long long)gridDim.x * 8) {
    const long long r = row0 + w;
    const bool live = r < M;
    const T *a = A + (live ? r : 0) * lda;
    T acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = T(0);
    for (long long c0 = 0; c0 < nv; c0 += CH) {
      const int len = (int)(nv - c0 < CH ? nv - c0 : CH);
      __syncthreads();  // the previous piece of x has been used by every warp
      for (int i = threadIdx.x; i < len; i += 256) xs[i] = __ldg(x4 + c0 + i);
      __syncthreads();
      if (live) {
        const uint4 *a4 = reinterpret_cast<const uint4 *>(a) + c0;
        int c = lane;
        // the 128-piece steps of gemv_n_kernel continue across chunks (CH is a multiple of 128)
        for (; c + 96 < len && c0 + c + 96 < nv; c += 128) {
          uint4 ra[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) ra[u] = __ldcs(a4 + c + 32 * u);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            T av[V], xv[V];
            memcpy(av, &ra[u], 16);
            memcpy(xv, &xs[c + 32 * u], 16);
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] = fma_(av[j], xv[j], acc[j]);
          }
        }
        for (; c < len; c += 32) {
          const uint4 ra = a4[c];
          T av[V], xv[V];
          memcpy(av, &ra, 16);
          memcpy(xv, &xs[c], 16);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = fma_(av[j], xv[j], acc[j]);
        }
      }
    }
    if (live) {
      for (long long c = nv * V + lane; c < N; c += 32) acc[0] = fma_(a[c], x[c], acc[0]);
      T s = acc[0];
#pragma unroll
      for (int j = 1; j < V; ++j) s += acc[j];
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) y[r] = s;
    }
  }
}

// ---- y = A^T x : column strips, partial sums per row chunk, then a fold ---------------------------
template <typename T>
__global__ void __launch_bounds__(256) gemv_t_partial_kernel(const T *__restrict__ A, long long lda,
                                                             const T *__restrict__ x, T *__restrict__ part,
                                                             long long M, long long N, long long rows_per_chunk) {
  const long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * rows_per_chunk;
  const long long r1 = r0 + rows_per_chunk < M ? r0 + rows_per_chunk : M;
  if (col >= N) return;
  T p0 = 0, p1 = 0, p2 = 0, p3 = 0;
  long long r = r0;
  for (; r + 3 < r1; r += 4) {
    p0 = fma_(A[r * lda + col], x[r], p0);
    p1 = fma_(A[(r + 1) * lda + col], x[r + 1], p1);
    p2 = fma_(A[(r + 2) * lda + col], x[r + 2], p2);
    p3 = fma_(A[(r + 3) * lda + col], x[r + 3], p3);
  }
  for (; r < r1; ++r) p0 = fma_(A[r * lda + col], x[r], p0);
  part[(long long)blockIdx.y * N + col] = (p0 + p1) + (p2 + p3);
}
// The same with four (float32) or two (float64) adjacent columns per thread, read 16 bytes at a time:
// four times the bytes in flight per thread. part has the layout of the scalar kernel.
template <typename T>
__global__ void __launch_bounds__(256) gemv_t_partial_vec_kernel(const T *__restrict__ A, long long lda,
                                                                 const T *__restrict__ x, T *__restrict__ part,
                                                                 long long M, long long N, long long rows_per_chunk) {
  constexpr int V = 16 / sizeof(T);
  const long long cv = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // column group
  const long long r0 = (long long)blockIdx.y * rows_per_chunk;
  const long long r1 = r0 + rows_per_chunk < M ? r0 + rows_per_chunk : M;
  if (cv * V >= N) return;
  T p[4][V];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int j = 0; j < V; ++j) p[u][j] = T(0);
  const T *ac = A + cv * V;
  long long r = r0;
  for (; r + 3 < r1; r += 4) {
    uint4 ra[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) ra[u] = __ldcs(reinterpret_cast<const uint4 *>(ac + (r + u) * lda));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      T av[V];
      memcpy(av, &ra[u], 16);
      const T xr = x[r + u];
#pragma unroll
      for (int j = 0; j < V; ++j) p[u][j] = fma_(av[j], xr, p[u][j]);
    }
  }
  for (; r < r1; ++r) {
    const uint4 ra = *reinterpret_cast<const uint4 *>(ac + r * lda);
    T av[V];
    memcpy(av, &ra, 16);
    const T xr = x[r];
#pragma unroll
    for (int j = 0; j < V; ++j) p[0][j] = fma_(av[j], xr, p[0][j]);
  }
  T o[V];
#pragma unroll
  for (int j = 0; j < V; ++j) o[j] = (p[0][j] + p[1][j]) + (p[2][j] + p[3][j]);  // as the scalar kernel sums
  uint4 ro;
  memcpy(&ro, o, 16);
  *reinterpret_cast<uint4 *>(part + (long long)blockIdx.y * N + cv * V) = ro;
}
template <typename T>
__global__ void __launch_bounds__(256) fold_rows_kernel(const T *__restrict__ part, T *__restrict__ y, long long N,
                                                        int chunks) {
  const long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= N) return;
  T s = 0;
  for (int c = 0; c < chunks; ++c) s += part[(long long)c * N + col];
  y[col] = s;
}

// ---- A = x y^T ------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) ger_kernel(const T *__restrict__ x, const T *__restrict__ y, T *__restrict__ A,
                                                  long long M, long long N) {
  constexpr int V = 16 / sizeof(T);
  if (VEC) {
    // A block takes groups of four consecutive rows (group blockIdx.x, blockIdx.x + gridDim.x, ...; the
    // host launches many more blocks than are resident at once, so groups are handed out as blocks
    // retire); its threads keep up to eight 16-byte pieces of y in registers across the rows (a strip
    // of 2048 pieces), so a row costs a thread one scalar load of x and eight multiplies and stores,
    // and nothing is divided.
    const long long nv = N / V;
    for (long long c0 = 0; c0 < nv; c0 += 8 * 256) {
      T yv[8][V];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const long long c = c0 + threadIdx.x + 256 * u;
        uint4 ry = make_uint4(0, 0, 0, 0);
        if (c < nv) ry = __ldg(reinterpret_cast<const uint4 *>(y + c * V));
        memcpy(yv[u], &ry, 16);
      }
      for (long long i4 = (long long)blockIdx.x * 4; i4 < M; i4 += (long long)gridDim.x * 4)
      for (long long i = i4; i < i4 + 4 && i < M; ++i) {
        const T xi = x[i];
        T *row = A + i * N;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const long long c = c0 + threadIdx.x + 256 * u;
          if (c < nv) {
            T o[V];
#pragma unroll
            for (int j = 0; j < V; ++j) o[j] = xi * yv[u][j];
            uint4 ro;
            memcpy(&ro, o, 16);
            *reinterpret_cast<uint4 *>(row + c * V) = ro;
          }
        }
      }
    }
  } else {
    const long long total = M * N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride)
      A[t] = x[t / N] * y[t % N];
  }
}

// ---- general matrix multiply on CUDA cores -----------------------------------------------------
// 64x64 tile of C per CTA, 16-deep k slices through shared memory, 4x4 accumulators per thread.
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(int transA, int transB, long long M, long long N,
                                                        long long K, const T *__restrict__ A, long long lda,
                                                        const T *__restrict__ B, long long ldb, T *__restrict__ C,
                                                        long long ldc, long long strideA, long long strideB,
                                                        long long strideC, Epilogue ep) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ T As[BK][BM + 1];
  __shared__ T Bs[BK][BN + 1];
  A += (long long)blockIdx.z * strideA;
  B += (long long)blockIdx.z * strideB;
  C += (long long)blockIdx.z * strideC;
  const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T(0);
  for (long long k0 = 0; k0 < K; k0 += BK) {
    // A tile: BM x BK. Consecutive threads walk the contiguous direction of the operand.
    for (int t = threadIdx.x; t < BM * BK; t += 256) {
      int mi, ki;
      if (!transA) {
        ki = t % BK;
        mi = t / BK;
      } else {
        mi = t % BM;
        ki = t / BM;
      }
      const long long m = m0 + mi, k = k0 + ki;
      T v = T(0);
      if (m < M && k < K) v = transA ? A[k * lda + m] : A[m * lda + k];
      As[ki][mi] = v;
    }
    for (int t = threadIdx.x; t < BN * BK; t += 256) {
      int ni, ki;
      if (!transB) {
        ni = t % BN;
        ki = t / BN;
      } else {
        ki = t % BK;
        ni = t / BK;
      }
      const long long n = n0 + ni, k = k0 + ki;
      T v = T(0);
      if (n < N && k < K) v = transB ? B[n * ldb + k] : B[k * ldb + n];
      Bs[ki][ni] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma_(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long n = n0 + tx * 4 + j;
      if (n < N) {
        const T o = apply_epilogue<T>(acc[i][j], ep, m, n);
        C[m * ldc + n] = ep.accumulate ? epi_add<T>(C[m * ldc + n], o) : o;  // Incr mode: C += result
      }
    }
  }
}

// ---- products with very few output columns (a classifier's last layer: 256 x 100 by 100 x 10) -----
// A 64 x 64 tile would be mostly padding and the whole product would sit on a handful of SMs. Here a
// warp owns one row of C: lane l takes k = l, l + 32, ... for all N <= 16 columns, the 32 partial
// sums per column are folded by shuffles in a fixed order, and lane n stores column n.
template <typename T>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(int transB, long long M, int N, long long K,
                                                          const T *__restrict__ A, long long lda,
                                                          const T *__restrict__ B, long long ldb, T *__restrict__ C,
                                                          long long ldc, long long strideA, long long strideB,
                                                          long long strideC, Epilogue ep) {
  constexpr int NMAX = 16;
  A += (long long)blockIdx.y * strideA;
  B += (long long)blockIdx.y * strideB;
  C += (long long)blockIdx.y * strideC;
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long m = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); m < M; m += warps) {
    T acc[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) acc[n] = T(0);
    const T *arow = A + m * lda;
    for (long long k = lane; k < K; k += 32) {
      const T a = arow[k];
#pragma unroll
      for (int n = 0; n < NMAX; ++n)
        if (n < N) acc[n] = fma_(a, transB ? B[(long long)n * ldb + k] : B[k * ldb + n], acc[n]);
    }
    T mine = T(0);
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      T v = acc[n];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == n) mine = v;
    }
    if (lane < N) {
      const T o = apply_epilogue<T>(mine, ep, m, lane);
      C[m * ldc + lane] = ep.accumulate ? epi_add<T>(C[m * ldc + lane], o) : o;
    }
  }
}

int gemm_simt(b200_engine *e, int dtype, int transA, int transB, long long M, long long N, long long K,
              const void *A, long long lda, const void *B, long long ldb, void *C, long long ldc, long long batch,
              long long strideA, long long strideB, long long strideC, const Epilogue &ep) {
  if (!transA && N <= 16 && K >= 1 && batch <= 65535) {  // whatever M is: one summation order per shape class
    const unsigned blocks = (unsigned)std::max<long long>(1, std::min<long long>((M + 7) / 8, (long long)e->sm_count * 8));
    dim3 sgrid(blocks, (unsigned)batch);
    if (dtype == B200_F32)
      gemm_skinny_kernel<float><<<sgrid, 256, 0, e->stream>>>(transB, M, (int)N, K, (const float *)A, lda,
                                                             (const float *)B, ldb, (float *)C, ldc, strideA, strideB,
                                                             strideC, ep);
    else
      gemm_skinny_kernel<double><<<sgrid, 256, 0, e->stream>>>(transB, M, (int)N, K, (const double *)A, lda,
                                                              (const double *)B, ldb, (double *)C, ldc, strideA,
                                                              strideB, strideC, ep);
    B200_CHECK_LAUNCH(e, "gemm_skinny_kernel");
    return B200_OK;
  }
  dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64), (unsigned)batch);
  if (dtype == B200_F32)
    gemm_simt_kernel<float><<<grid, 256, 0, e->stream>>>(transA, transB, M, N, K, (const float *)A, lda,
                                                        (const float *)B, ldb, (float *)C, ldc, strideA, strideB,
                                                        strideC, ep);
  else
    gemm_simt_kernel<double><<<grid, 256, 0, e->stream>>>(transA, transB, M, N, K, (const double *)A, lda,
                                                         (const double *)B, ldb, (double *)C, ldc, strideA, strideB,
                                                         strideC, ep);
  B200_CHECK_LAUNCH(e, "gemm_simt_kernel");
  return B200_OK;
}

template <typename T>
static int gemv_typed(b200_engine *e, int transA, long long M, long long N, const T *A, long long lda, const T *x,
                      T *y) {
  const long long cap = (long long)e->sm_count * 8;
  if (!transA) {
    const bool vec = lda % (16 / sizeof(T)) == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)x % 16 == 0;
    // One row per warp and many more blocks than fit the GPU at once: blocks are then handed out as
    // earlier ones retire. A grid that is resident all at once with a fixed share of rows per warp
    // measured 15 % slower at 16384 x 16384 (800 to 1184 blocks: 4.8 TB/s; 1400 and more: 5.6), the
    // share of the SMs that got an extra block setting the time.
    const int blocks = (int)std::max<long long>(1, std::min<long long>((M + 7) / 8, cap * 8));
    // few long rows (every block resident from the start): the variant that shares x through shared memory
    // measured 5.6 against 4.8 TB/s at 8192 x 32768; with more blocks than fit, the plain kernel is ahead
    // (5.6 against 5.5 at 16384 x 16384, 5.3 against 5.2 at 40000 x 6000). The two give the same bits.
    if (vec && N >= 4096 && (M + 7) / 8 <= cap)
      gemv_n_smemx_kernel<T><<<blocks, 256, 0, e->stream>>>(A, lda, x, y, M, N);
    else if (vec)
      gemv_n_kernel<T, true><<<blocks, 256, 0, e->stream>>>(A, lda, x, y, M, N);
    else
      gemv_n_kernel<T, false><<<blocks, 256, 0, e->stream>>>(A, lda, x, y, M, N);
    B200_CHECK_LAUNCH(e, "gemv_n_kernel");
    return B200_OK;
  }
  // y (length N) = A^T x (x length M): split the rows so that the grid fills the machine
  constexpr int V = 16 / (int)sizeof(T);
  const bool tvec = N % V == 0 && lda % V == 0 && (uintptr_t)A % 16 == 0 && N >= 256 * V;
  const long long col_blocks = tvec ? (N / V + 255) / 256 : (N + 255) / 256;
  long long chunks = std::max<long long>(1, std::min<long long>((cap + col_blocks - 1) / col_blocks, (M + 63) / 64));
  chunks = std::min<long long>(chunks, 65535);
  const long long rows_per_chunk = (M + chunks - 1) / chunks;
  chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
  void *part = nullptr;
  int rc = b200_get(e, (int64_t)(chunks * N * sizeof(T)), &part);
  if (rc != B200_OK) return rc;
  dim3 grid((unsigned)col_blocks, (unsigned)chunks);
  if (tvec)
    gemv_t_partial_vec_kernel<T><<<grid, 256, 0, e->stream>>>(A, lda, x, (T *)part, M, N, rows_per_chunk);
  else
    gemv_t_partial_kernel<T><<<grid, 256, 0, e->stream>>>(A, lda, x, (T *)part, M, N, rows_per_chunk);
  cudaError_t le = cudaGetLastError();
  if (le == cudaSuccess) {
    e->launches++;
    fold_rows_kernel<T><<<(unsigned)((N + 255) / 256), 256, 0, e->stream>>>((const T *)part, y, N, (int)chunks);
    le = cudaGetLastError();
    if (le == cudaSuccess) e->launches++;
  }
  // stream order makes handing the block back safe: whoever gets it next runs after the fold
  b200_put(e, part, 0);
  if (le != cudaSuccess) return set_error(e, B200_ERR_CUDA, "gemv launch failed: %s", cudaGetErrorString(le));
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_gemv(b200_engine *e, int dtype, int transA, int64_t M, int64_t N, const void *A, int64_t lda, const void *x,
              void *y) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_gemv: dtype %d not supported", dtype);
  B200_REQUIRE(e, M >= 0 && N >= 0, "b200_gemv: negative extent");
  B200_REQUIRE(e, lda >= N, "b200_gemv: lda %lld < N %lld", (long long)lda, (long long)N);
  const int64_t ylen = transA ? N : M, xlen = transA ? M : N;
  if (ylen == 0) return B200_OK;
  B200_REQUIRE(e, y != nullptr, "b200_gemv: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (xlen == 0) {  // empty sum
    B200_CHECK_CUDA(e, cudaMemsetAsync(y, 0, (size_t)ylen * dtype_size(dtype), e->stream));
    return B200_OK;
  }
  B200_REQUIRE(e, A && x, "b200_gemv: null pointer");
  if (dtype == B200_F32) return gemv_typed<float>(e, transA, M, N, (const float *)A, lda, (const float *)x, (float *)y);
  return gemv_typed<double>(e, transA, M, N, (const double *)A, lda, (const double *)x, (double *)y);
}

int b200_ger(b200_engine *e, int dtype, int64_t M, int64_t N, const void *x, const void *y, void *A) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_ger: dtype %d not supported", dtype);
  B200_REQUIRE(e, M >= 0 && N >= 0, "b200_ger: negative extent");
  if (M == 0 || N == 0) return B200_OK;
  B200_REQUIRE(e, x && y && A, "b200_ger: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const size_t es = dtype_size(dtype);
  const bool vec = N % (16 / es) == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)y % 16 == 0;
  const long long work = vec ? M * (N / (16 / (long long)es)) : M * N;
  int blocks = (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, (long long)e->sm_count * 16));
  if (vec) blocks = (int)std::max<long long>(1, std::min<long long>((M + 3) / 4, (long long)e->sm_count * 64));  // groups of four rows
  if (dtype == B200_F32) {
    if (vec)
      ger_kernel<float, true><<<blocks, 256, 0, e->stream>>>((const float *)x, (const float *)y, (float *)A, M, N);
    else
      ger_kernel<float, false><<<blocks, 256, 0, e->stream>>>((const float *)x, (const float *)y, (float *)A, M, N);
  } else {
    if (vec)
      ger_kernel<double, true><<<blocks, 256, 0, e->stream>>>((const double *)x, (const double *)y, (double *)A, M, N);
    else
      ger_kernel<double, false><<<blocks, 256, 0, e->stream>>>((const double *)x, (const double *)y, (double *)A, M,
                                                              N);
  }
  B200_CHECK_LAUNCH(e, "ger_kernel");
  return B200_OK;
}

}  // extern "C"
