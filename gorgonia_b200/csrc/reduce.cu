// Softmax, axis reductions and argmax.
//
// Give gorgonia's softmaxOp (op_softmax.go:99-128 -> tensor.SoftMax / LogSoftMax), sumOp /
// maxOp (op_reduction.go:70-99 -> tensor.Sum / tensor.Max) a device implementation; in the
// reference they are CPU-only ops and force a device->host->device round trip. A tensor is
// viewed as (outer, len, inner) around the reduced axis.
//
// Kernels
//   rows (inner == 1, len <= 2048): one warp per row, the row held in registers, max and sum by
//     warp shuffles, 128-bit loads when the row length allows. 10-class outputs (MLP, LeNet)
//     pack several rows per warp-sized group of lanes instead of wasting 22 lanes out of 32.
//   columns (inner > 1) and long rows: one thread per (outer, inner) column walking the axis
//     with stride `inner` (coalesced across threads), or one CTA per row with a shared-memory
//     tree for long rows.
// Sums are pairwise (lane partials, then a butterfly), so their error grows with log(len).
#include <algorithm>
#include <cfloat>
#include <mutex>

#include "engine.h"

namespace b200 {

template <typename T>
__device__ __forceinline__ T neg_inf();
template <>
__device__ __forceinline__ float neg_inf<float>() {
  return -INFINITY;
}
template <>
__device__ __forceinline__ double neg_inf<double>() {
  return -(double)INFINITY;
}

template <typename T>
__device__ __forceinline__ T group_max(T v, int width) {
  for (int o = width / 2; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o, width));
  return v;
}
template <typename T>
__device__ __forceinline__ T group_sum(T v, int width) {
  for (int o = width / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o, width);
  return v;
}

// mode: 0 softmax, 1 log-softmax, 2 sum, 3 max. A row of `len` contiguous elements is handled by
// a group of G lanes (G = 32, or a smaller power of two for short rows); PER = elements per lane.
template <typename T, int PER, int MODE>
__global__ void __launch_bounds__(256) row_kernel(const T *__restrict__ x, T *__restrict__ y, long long rows,
                                                  int len, int G) {
  const int lane_in_group = threadIdx.x % G;
  const int group_in_warp = (threadIdx.x & 31) / G;
  const int groups_per_warp = 32 / G;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  // all lanes of a warp run the same number of iterations (the shuffles below need every lane);
  // a group whose row falls past the end computes on padding and stores nothing
  for (long long r0 = warp * groups_per_warp; r0 < rows; r0 += nwarps * groups_per_warp) {
    const long long r = r0 + group_in_warp;
    const bool live = r < rows;
    const T *xr = x + (live ? r : 0) * len;
    T v[PER];
    T mx = neg_inf<T>();
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = lane_in_group + k * G;
      v[k] = (live && i < len) ? xr[i] : neg_inf<T>();
      mx = fmax(mx, v[k]);
    }
    mx = group_max(mx, G);
    if (MODE == 3) {
      if (live && lane_in_group == 0) y[r] = mx;
      continue;
    }
    T s = T(0);
    if (MODE == 2) {
#pragma unroll
      for (int k = 0; k < PER; ++k) s += (live && lane_in_group + k * G < len) ? v[k] : T(0);
      s = group_sum(s, G);
      if (live && lane_in_group == 0) y[r] = s;
      continue;
    }
    T ex[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      ex[k] = (live && lane_in_group + k * G < len) ? exp(v[k] - mx) : T(0);
      s += ex[k];
    }
    s = group_sum(s, G);
    if (!live) continue;
    T *yr = y + r * len;
    if (MODE == 0) {
      const T inv = T(1) / s;
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int i = lane_in_group + k * G;
        if (i < len) yr[i] = ex[k] * inv;
      }
    } else {
      const T ls = log(s);
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int i = lane_in_group + k * G;
        if (i < len) yr[i] = (v[k] - mx) - ls;
      }
    }
  }
}

// One thread per (outer, inner) column; consecutive threads take consecutive `inner`, so each
// step along the axis is a coalesced access. Sums use 4 interleaved partials.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) col_kernel(const T *__restrict__ x, T *__restrict__ y, long long outer,
                                                  long long len, long long inner) {
  const long long total = outer * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride) {
    const long long o = c / inner, in = c % inner;
    const T *xp = x + o * len * inner + in;
    T mx = neg_inf<T>();
    if (MODE != 2)
      for (long long k = 0; k < len; ++k) mx = fmax(mx, xp[k * inner]);
    if (MODE == 3) {
      y[c] = mx;
      continue;
    }
    T p0 = 0, p1 = 0, p2 = 0, p3 = 0;
    long long k = 0;
    if (MODE == 2) {
      for (; k + 3 < len; k += 4) {
        p0 += xp[k * inner];
        p1 += xp[(k + 1) * inner];
        p2 += xp[(k + 2) * inner];
        p3 += xp[(k + 3) * inner];
      }
      for (; k < len; ++k) p0 += xp[k * inner];
      y[c] = (p0 + p1) + (p2 + p3);
      continue;
    }
    for (; k + 3 < len; k += 4) {
      p0 += exp(xp[k * inner] - mx);
      p1 += exp(xp[(k + 1) * inner] - mx);
      p2 += exp(xp[(k + 2) * inner] - mx);
      p3 += exp(xp[(k + 3) * inner] - mx);
    }
    for (; k < len; ++k) p0 += exp(xp[k * inner] - mx);
    const T s = (p0 + p1) + (p2 + p3);
    T *yp = y + o * len * inner + in;
    if (MODE == 0) {
      const T inv = T(1) / s;
      for (long long q = 0; q < len; ++q) yp[q * inner] = exp(xp[q * inner] - mx) * inv;
    } else {
      const T ls = log(s);
      for (long long q = 0; q < len; ++q) yp[q * inner] = (xp[q * inner] - mx) - ls;
    }
  }
}

// Long rows (inner == 1, len > 2048): one CTA per row, shared-memory tree.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) long_row_kernel(const T *__restrict__ x, T *__restrict__ y, long long rows,
                                                       long long len) {
  __shared__ T red[256 / 32];
  __shared__ T bcast;
  auto block_reduce = [&](T v, bool is_max) -> T {
    v = is_max ? group_max(v, 32) : group_sum(v, 32);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
      T w = threadIdx.x < 256 / 32 ? red[threadIdx.x] : (is_max ? neg_inf<T>() : T(0));
      w = is_max ? group_max(w, 32) : group_sum(w, 32);
      if (threadIdx.x == 0) bcast = w;
    }
    __syncthreads();
    const T r = bcast;
    __syncthreads();
    return r;
  };
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T *xr = x + r * len;
    T mx = neg_inf<T>();
    if (MODE != 2) {
      for (long long i = threadIdx.x; i < len; i += blockDim.x) mx = fmax(mx, xr[i]);
      mx = block_reduce(mx, true);
    }
    if (MODE == 3) {
      if (threadIdx.x == 0) y[r] = mx;
      continue;
    }
    T s = 0;
    for (long long i = threadIdx.x; i < len; i += blockDim.x) s += MODE == 2 ? xr[i] : exp(xr[i] - mx);
    s = block_reduce(s, false);
    if (MODE == 2) {
      if (threadIdx.x == 0) y[r] = s;
      continue;
    }
    T *yr = y + r * len;
    const T inv = T(1) / s, ls = log(s);
    for (long long i = threadIdx.x; i < len; i += blockDim.x)
      yr[i] = MODE == 0 ? exp(xr[i] - mx) * inv : (xr[i] - mx) - ls;
  }
}

// First maximum along the axis, as an int64 index (strict '>' keeps the earliest).
template <typename T>
__global__ void __launch_bounds__(256) argmax_kernel(const T *__restrict__ x, long long *__restrict__ y,
                                                     long long outer, long long len, long long inner) {
  const long long total = outer * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride) {
    const long long o = c / inner, in = c % inner;
    const T *xp = x + o * len * inner + in;
    T m = xp[0];
    long long arg = 0;
    for (long long k = 1; k < len; ++k) {
      const T v = xp[k * inner];
      if (v > m) {
        m = v;
        arg = k;
      }
    }
    y[c] = arg;
  }
}

// Whole-tensor sum / max into one element. Every CTA reduces a grid-stride share and leaves its
// partial in scratch memory; the CTA that takes the last ticket folds the partials in index
// order (so the result does not depend on which CTA finished last) and re-arms the ticket.
// scratch layout: [0, REDUCE_ALL_MAX_BLOCKS) partials of type T, then the ticket word.
constexpr int REDUCE_ALL_MAX_BLOCKS = 1024;
constexpr size_t REDUCE_ALL_TICKET_OFFSET = REDUCE_ALL_MAX_BLOCKS * sizeof(double);
constexpr size_t REDUCE_ALL_SCRATCH_BYTES = REDUCE_ALL_TICKET_OFFSET + 256;

template <typename T, bool IS_MAX>
__global__ void __launch_bounds__(256) reduce_all_kernel(const T *__restrict__ x, long long n,
                                                         unsigned char *__restrict__ scratch, T *__restrict__ y) {
  T *partials = reinterpret_cast<T *>(scratch);
  unsigned int *ticket = reinterpret_cast<unsigned int *>(scratch + REDUCE_ALL_TICKET_OFFSET);
  __shared__ T red[256 / 32];
  __shared__ bool is_last;
  auto block_reduce = [&](T v) -> T {
    v = IS_MAX ? group_max(v, 32) : group_sum(v, 32);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    T w = IS_MAX ? neg_inf<T>() : T(0);
    if (threadIdx.x < 32) {
      if (threadIdx.x < 256 / 32) w = red[threadIdx.x];
      w = IS_MAX ? group_max(w, 32) : group_sum(w, 32);
    }
    __syncthreads();
    return w;  // valid in thread 0
  };
  const long long stride = (long long)gridDim.x * blockDim.x;
  T p0 = IS_MAX ? neg_inf<T>() : T(0), p1 = p0, p2 = p0, p3 = p0;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const T a = x[i], b = x[i + stride], c = x[i + 2 * stride], d = x[i + 3 * stride];
    if (IS_MAX) {
      p0 = fmax(p0, a); p1 = fmax(p1, b); p2 = fmax(p2, c); p3 = fmax(p3, d);
    } else {
      p0 += a; p1 += b; p2 += c; p3 += d;
    }
  }
  for (; i < n; i += stride) p0 = IS_MAX ? fmax(p0, x[i]) : p0 + x[i];
  T v = IS_MAX ? fmax(fmax(p0, p1), fmax(p2, p3)) : (p0 + p1) + (p2 + p3);
  v = block_reduce(v);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = v;
    __threadfence();
    is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // fold the partials: thread t takes partials t, t+256, ... in order, then the block tree
  T w = IS_MAX ? neg_inf<T>() : T(0);
  for (int b = threadIdx.x; b < (int)gridDim.x; b += blockDim.x) {
    const T q = *reinterpret_cast<volatile T *>(&partials[b]);
    w = IS_MAX ? fmax(w, q) : w + q;
  }
  w = block_reduce(w);
  if (threadIdx.x == 0) {
    y[0] = w;
    *ticket = 0;  // ready for the next call
  }
}

template <typename T>
static int launch_reduce_all(b200_engine *e, int kind, const T *x, long long n, unsigned char *scratch, T *y) {
  long long want = (n + 1023) / 1024;
  want = std::min<long long>(want, (long long)e->sm_count * 4);
  want = std::min<long long>(want, REDUCE_ALL_MAX_BLOCKS);
  const int blocks = (int)std::max<long long>(1, want);
  if (kind == 0)
    reduce_all_kernel<T, false><<<blocks, 256, 0, e->stream>>>(x, n, scratch, y);
  else
    reduce_all_kernel<T, true><<<blocks, 256, 0, e->stream>>>(x, n, scratch, y);
  B200_CHECK_LAUNCH(e, "reduce_all_kernel");
  return B200_OK;
}

// ---- whole-tensor reduction that allocates nothing ---------------------------------------------
// Scratch for b200_reduce_all_static: a fixed array that lives in the library image, one copy on
// every GPU that loads the library, held until the process exits. Layout as above, for at most
// REDUCE_STATIC_MAX_BLOCKS partials. In HOST code the name of this array is only a handle for
// cudaGetSymbolAddress; it is never a device address and is never passed to a kernel.
constexpr int REDUCE_STATIC_MAX_BLOCKS = 256;
constexpr size_t REDUCE_STATIC_TICKET_OFFSET = REDUCE_ALL_TICKET_OFFSET;  // the kernel's fixed layout
static __device__ __align__(256) unsigned char g_reduce_static_scratch[REDUCE_ALL_SCRATCH_BYTES];

// Device address of the array on each device, looked up once per device with that device current.
static unsigned char *g_reduce_static_ptr[64];
static std::mutex g_reduce_static_mu;

static int reduce_static_scratch(b200_engine *e, unsigned char **out) {
  const int dev = e->device;
  if (dev < 0 || dev >= 64) return set_error(e, B200_ERR_UNSUPPORTED, "b200_reduce_all_static: device %d", dev);
  std::lock_guard<std::mutex> lk(g_reduce_static_mu);
  if (!g_reduce_static_ptr[dev]) {
    void *ptr = nullptr;
    B200_CHECK_CUDA(e, cudaGetSymbolAddress(&ptr, g_reduce_static_scratch));
    g_reduce_static_ptr[dev] = (unsigned char *)ptr;
  }
  *out = g_reduce_static_ptr[dev];
  return B200_OK;
}

template <typename T, int MODE>
static int launch_mode(b200_engine *e, const T *x, T *y, long long outer, long long len, long long inner) {
  const int threads = 256;
  const long long cap = (long long)e->sm_count * 8;
  if (inner == 1 && len <= 2048) {
    int G = 32;
    while (G > 1 && G / 2 >= len) G /= 2;  // smallest power of two >= len, at most 32
    const int per = (int)((len + G - 1) / G);
    const long long groups_per_block = threads / G;
    const int blocks = (int)std::max<long long>(1, std::min((outer + groups_per_block - 1) / groups_per_block, cap));
#define B200_ROW(P)                                                                           \
  row_kernel<T, P, MODE><<<blocks, threads, 0, e->stream>>>(x, y, outer, (int)len, G)
    if (per <= 1) B200_ROW(1);
    else if (per <= 2) B200_ROW(2);
    else if (per <= 4) B200_ROW(4);
    else if (per <= 8) B200_ROW(8);
    else if (per <= 16) B200_ROW(16);
    else if (per <= 32) B200_ROW(32);
    else B200_ROW(64);
#undef B200_ROW
    B200_CHECK_LAUNCH(e, "row_kernel");
  } else if (inner == 1) {
    const int blocks = (int)std::max<long long>(1, std::min(outer, cap));
    long_row_kernel<T, MODE><<<blocks, threads, 0, e->stream>>>(x, y, outer, len);
    B200_CHECK_LAUNCH(e, "long_row_kernel");
  } else {
    const long long total = outer * inner;
    const int blocks = (int)std::max<long long>(1, std::min((total + threads - 1) / threads, cap));
    col_kernel<T, MODE><<<blocks, threads, 0, e->stream>>>(x, y, outer, len, inner);
    B200_CHECK_LAUNCH(e, "col_kernel");
  }
  return B200_OK;
}

// ---- softmax / log-softmax derivative --------------------------------------------------------
// softmaxDiffOp (op_softmax.go:262-274) hands (y, grad) to tensor.SoftMaxB / LogSoftMaxB:
//   softmax:      dx_i = y_i * (g_i - sum_j g_j y_j)
//   log-softmax:  dx_i = g_i - exp(y_i) * sum_j g_j
// on a tensor viewed as (outer, len, inner). The row sum is taken in double (rows are short and
// the subtraction that follows cancels). inner == 1: one warp per row, shuffle reduction;
// inner > 1: one thread per (outer, inner) pair walking len with coalesced strided accesses.
template <typename T, bool LOG>
__global__ void __launch_bounds__(256) softmax_bwd_rows_kernel(const T *__restrict__ y, const T *__restrict__ g,
                                                               T *__restrict__ dx, long long rows, long long len) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp0; r < rows; r += nwarps) {
    const T *yp = y + r * len, *gp = g + r * len;
    double s = 0.0;
    for (long long k = lane; k < len; k += 32) s += LOG ? (double)gp[k] : (double)gp[k] * (double)yp[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    for (long long k = lane; k < len; k += 32) {
      const double yy = yp[k], gg = gp[k];
      dx[r * len + k] = (T)(LOG ? gg - exp(yy) * s : yy * (gg - s));
    }
  }
}
template <typename T, bool LOG>
__global__ void __launch_bounds__(256) softmax_bwd_strided_kernel(const T *__restrict__ y, const T *__restrict__ g,
                                                                  T *__restrict__ dx, long long outer, long long len,
                                                                  long long inner) {
  const long long total = outer * inner;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long o = t / inner, in = t - o * inner;
    const long long base = o * len * inner + in;
    double s = 0.0;
    for (long long k = 0; k < len; ++k)
      s += LOG ? (double)g[base + k * inner] : (double)g[base + k * inner] * (double)y[base + k * inner];
    for (long long k = 0; k < len; ++k) {
      const double yy = y[base + k * inner], gg = g[base + k * inner];
      dx[base + k * inner] = (T)(LOG ? gg - exp(yy) * s : yy * (gg - s));
    }
  }
}

// Rows of at most 16 elements (the 10-class heads of the configs): a warp takes 32 rows at a time,
// loads their 32 * len values of y and grad with consecutive lanes on consecutive addresses, lets
// each lane work through one row out of shared memory, and stores the 32 * len results the same
// coalesced way. A warp-per-row walk would leave 22 of 32 lanes idle on a 10-element row.
template <typename T, bool LOG>
__global__ void __launch_bounds__(128) softmax_bwd_short_kernel(const T *__restrict__ y, const T *__restrict__ g,
                                                                T *__restrict__ dx, long long rows, int len) {
  __shared__ __align__(16) T sy[4][32 * 16], sg[4][32 * 16];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long groups = (rows + 31) / 32;
  // whole groups move 16 bytes per lane and instruction, with every load of a group in flight before
  // the first one is used (a group of 32 rows is 32 * len elements, a whole number of 16-byte pieces
  // when len is even for float32 / any len for pairs of float64 rows)
  constexpr int PER = 16 / (int)sizeof(T);        // elements in 16 bytes
  constexpr int MAXV = (32 * 16 / PER + 31) / 32;  // 16-byte pieces per lane and array, at most
  const bool vec_ok = ((32 * len) % PER) == 0 && (((uintptr_t)y | (uintptr_t)g | (uintptr_t)dx) & 15) == 0 &&
                      ((32LL * len * sizeof(T)) & 15) == 0;
  for (long long grp = warp0; grp < groups; grp += nwarps) {
    const long long r0 = grp * 32;
    const int nrows = (int)min((long long)32, rows - r0);
    const int n = nrows * len;
    const long long base = r0 * len;
    const bool vec = vec_ok && nrows == 32;
    if (vec) {
      const int nv = n / PER;
      const uint4 *yv = reinterpret_cast<const uint4 *>(y + base), *gv = reinterpret_cast<const uint4 *>(g + base);
      uint4 ry[MAXV], rg[MAXV];
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int i = lane + v * 32;
        if (i < nv) {
          ry[v] = __ldg(yv + i);
          rg[v] = __ldg(gv + i);
        }
      }
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int i = lane + v * 32;
        if (i < nv) {
          reinterpret_cast<uint4 *>(sy[w])[i] = ry[v];
          reinterpret_cast<uint4 *>(sg[w])[i] = rg[v];
        }
      }
    } else {
      for (int i = lane; i < n; i += 32) {
        sy[w][i] = y[base + i];
        sg[w][i] = g[base + i];
      }
    }
    __syncwarp();
    if (lane < nrows) {
      T *yp = &sy[w][lane * len], *gp = &sg[w][lane * len];
      double s = 0.0;
      for (int k = 0; k < len; ++k) s += LOG ? (double)gp[k] : (double)gp[k] * (double)yp[k];
      for (int k = 0; k < len; ++k) {
        const double yy = yp[k], gg = gp[k];
        gp[k] = (T)(LOG ? gg - exp(yy) * s : yy * (gg - s));
      }
    }
    __syncwarp();
    if (vec) {
      const int nv = n / PER;
      uint4 *dv = reinterpret_cast<uint4 *>(dx + base);
      for (int i = lane; i < nv; i += 32) dv[i] = reinterpret_cast<const uint4 *>(sg[w])[i];
    } else {
      for (int i = lane; i < n; i += 32) dx[base + i] = sg[w][i];
    }
    __syncwarp();
  }
}

template <typename T, bool LOG>
static int launch_softmax_bwd(b200_engine *e, const T *y, const T *g, T *dx, long long outer, long long len,
                              long long inner) {
  if (inner == 1 && len <= 16) {
    const long long groups = (outer + 31) / 32;
    // more blocks than are resident at once: groups of rows are then handed out as blocks retire
    const long long blocks = std::max<long long>(1, std::min<long long>((groups + 3) / 4, (long long)e->sm_count * 64));
    softmax_bwd_short_kernel<T, LOG><<<(int)blocks, 128, 0, e->stream>>>(y, g, dx, outer, (int)len);
  } else if (inner == 1) {
    const long long blocks = std::max<long long>(1, std::min<long long>((outer + 7) / 8, (long long)e->sm_count * 16));
    softmax_bwd_rows_kernel<T, LOG><<<(int)blocks, 256, 0, e->stream>>>(y, g, dx, outer, len);
  } else {
    const long long total = outer * inner;
    const long long blocks = std::max<long long>(1, std::min<long long>((total + 255) / 256, (long long)e->sm_count * 16));
    softmax_bwd_strided_kernel<T, LOG><<<(int)blocks, 256, 0, e->stream>>>(y, g, dx, outer, len, inner);
  }
  B200_CHECK_LAUNCH(e, "softmax_bwd_kernel");
  return B200_OK;
}

static int axis_op(b200_engine *e, int dtype, int mode, const void *x, void *y, int64_t outer, int64_t len,
                   int64_t inner, const char *who) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "%s: dtype %d not supported", who, dtype);
  B200_REQUIRE(e, outer >= 0 && len >= 0 && inner >= 0, "%s: negative extent", who);
  if (outer == 0 || inner == 0) return B200_OK;
  B200_REQUIRE(e, len > 0, "%s: cannot reduce an axis of length 0", who);
  B200_REQUIRE(e, x && y, "%s: null pointer", who);
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
#define B200_MODE(T, M) return launch_mode<T, M>(e, (const T *)x, (T *)y, outer, len, inner)
  if (dtype == B200_F32) {
    switch (mode) {
      case 0: B200_MODE(float, 0);
      case 1: B200_MODE(float, 1);
      case 2: B200_MODE(float, 2);
      default: B200_MODE(float, 3);
    }
  }
  switch (mode) {
    case 0: B200_MODE(double, 0);
    case 1: B200_MODE(double, 1);
    case 2: B200_MODE(double, 2);
    default: B200_MODE(double, 3);
  }
#undef B200_MODE
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_softmax(b200_engine *e, int dtype, const void *x, void *y, int64_t outer, int64_t len, int64_t inner,
                 int is_log) {
  return axis_op(e, dtype, is_log ? 1 : 0, x, y, outer, len, inner, "b200_softmax");
}

int b200_softmax_bwd(b200_engine *e, int dtype, const void *y, const void *grad, void *dx, int64_t outer, int64_t len,
                     int64_t inner, int is_log) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_softmax_bwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, outer >= 0 && len >= 0 && inner >= 0, "b200_softmax_bwd: negative extent");
  if (outer == 0 || inner == 0) return B200_OK;
  B200_REQUIRE(e, len > 0, "b200_softmax_bwd: an axis of length 0");
  B200_REQUIRE(e, y && grad && dx, "b200_softmax_bwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32) {
    if (is_log) return launch_softmax_bwd<float, true>(e, (const float *)y, (const float *)grad, (float *)dx, outer, len, inner);
    return launch_softmax_bwd<float, false>(e, (const float *)y, (const float *)grad, (float *)dx, outer, len, inner);
  }
  if (is_log) return launch_softmax_bwd<double, true>(e, (const double *)y, (const double *)grad, (double *)dx, outer, len, inner);
  return launch_softmax_bwd<double, false>(e, (const double *)y, (const double *)grad, (double *)dx, outer, len, inner);
}

int b200_reduce(b200_engine *e, int dtype, int kind, const void *x, void *y, int64_t outer, int64_t len,
                int64_t inner) {
  if (e && kind != 0 && kind != 1) {
    std::lock_guard<std::recursive_mutex> lk(e->mu);
    return set_error(e, B200_ERR_INVALID, "b200_reduce: kind %d (0 = sum, 1 = max)", kind);
  }
  return axis_op(e, dtype, kind == 0 ? 2 : 3, x, y, outer, len, inner, "b200_reduce");
}

int b200_reduce_all(b200_engine *e, int dtype, int kind, const void *x, int64_t n, void *y) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_reduce_all: dtype %d not supported", dtype);
  B200_REQUIRE(e, kind == 0 || kind == 1, "b200_reduce_all: kind %d (0 = sum, 1 = max)", kind);
  B200_REQUIRE(e, n > 0, "b200_reduce_all: needs at least one element");
  B200_REQUIRE(e, x && y, "b200_reduce_all: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (!e->reduce_scratch) {
    // once per engine; the ticket word must start at zero and every launch leaves it at zero
    B200_CHECK_CUDA(e, cudaMalloc(&e->reduce_scratch, REDUCE_ALL_SCRATCH_BYTES));
    B200_CHECK_CUDA(e, cudaMemsetAsync(e->reduce_scratch, 0, REDUCE_ALL_SCRATCH_BYTES, e->stream));
  }
  unsigned char *scratch = (unsigned char *)e->reduce_scratch;
  if (dtype == B200_F32) return launch_reduce_all<float>(e, kind, (const float *)x, n, scratch, (float *)y);
  return launch_reduce_all<double>(e, kind, (const double *)x, n, scratch, (double *)y);
}

int b200_reduce_all_static(b200_engine *e, int dtype, int kind, const void *x, int64_t n, void *y) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_reduce_all_static: dtype %d not supported", dtype);
  B200_REQUIRE(e, kind == 0 || kind == 1, "b200_reduce_all_static: kind %d (0 = sum, 1 = max)", kind);
  B200_REQUIRE(e, n > 0, "b200_reduce_all_static: needs at least one element");
  if (n > B200_REDUCE_ALL_STATIC_MAX_N)
    return set_error(e, B200_ERR_UNSUPPORTED,
                     "b200_reduce_all_static: %lld elements exceed the limit of %lld that its fixed scratch is "
                     "sized for; use b200_reduce_all",
                     (long long)n, (long long)B200_REDUCE_ALL_STATIC_MAX_N);
  B200_REQUIRE(e, x && y, "b200_reduce_all_static: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  unsigned char *scratch = nullptr;
  rc = reduce_static_scratch(e, &scratch);  // first call on this device: looks the address up
  if (rc != B200_OK) return rc;
  // the array keeps whatever the previous call (or an aborted one) left: the ticket must be zero
  B200_CHECK_CUDA(e, cudaMemsetAsync(scratch + REDUCE_STATIC_TICKET_OFFSET, 0, sizeof(unsigned int), e->stream));
  long long want = (n + 1023) / 1024;
  want = std::min<long long>(want, REDUCE_STATIC_MAX_BLOCKS);
  const int blocks = (int)std::max<long long>(1, want);
  if (dtype == B200_F32) {
    if (kind == 0)
      reduce_all_kernel<float, false><<<blocks, 256, 0, e->stream>>>((const float *)x, n, scratch, (float *)y);
    else
      reduce_all_kernel<float, true><<<blocks, 256, 0, e->stream>>>((const float *)x, n, scratch, (float *)y);
  } else {
    if (kind == 0)
      reduce_all_kernel<double, false><<<blocks, 256, 0, e->stream>>>((const double *)x, n, scratch, (double *)y);
    else
      reduce_all_kernel<double, true><<<blocks, 256, 0, e->stream>>>((const double *)x, n, scratch, (double *)y);
  }
  B200_CHECK_LAUNCH(e, "reduce_all_kernel");
  return B200_OK;
}

int b200_argmax(b200_engine *e, int dtype, const void *x, int64_t *y, int64_t outer, int64_t len, int64_t inner) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_argmax: dtype %d not supported", dtype);
  B200_REQUIRE(e, outer >= 0 && len >= 0 && inner >= 0, "b200_argmax: negative extent");
  if (outer == 0 || inner == 0) return B200_OK;
  B200_REQUIRE(e, len > 0, "b200_argmax: cannot reduce an axis of length 0");
  B200_REQUIRE(e, x && y, "b200_argmax: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const long long total = outer * inner;
  const int blocks = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, (long long)e->sm_count * 8));
  if (dtype == B200_F32)
    argmax_kernel<float><<<blocks, 256, 0, e->stream>>>((const float *)x, (long long *)y, outer, len, inner);
  else
    argmax_kernel<double><<<blocks, 256, 0, e->stream>>>((const double *)x, (long long *)y, outer, len, inner);
  B200_CHECK_LAUNCH(e, "argmax_kernel");
  return B200_OK;
}

}  // extern "C"
