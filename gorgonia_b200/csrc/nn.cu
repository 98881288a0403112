// Max-pooling, im2col, N-d transpose and row gather.
//
// In gorgonia these are CPU ops (maxPoolOp.do, op_nn.go:828-907; im2colOp.do, op_nn.go:317-444;
// transposeOp.Do, op_tensor.go:937-952; byIndicesOp.Do, op_by_indices.go:90-97): the tape bounces
// every one of them through host memory. Here they are device kernels, so a whole forward tape
// stays resident. All of them are pure data movement, bound by HBM; the kernels are laid out so
// that consecutive threads write consecutive addresses.
#include <algorithm>
#include <cfloat>

#include <atomic>

#include "engine.h"
#include "ptx.cuh"

namespace b200 {

// ---- max-pool --------------------------------------------------------------------------------
// One thread per output element. The window is clipped to the image; the accumulator starts at
// -FLT_MAX and only a strictly larger value replaces it, so the first maximum in row-major window
// order wins and an all-NaN window yields -FLT_MAX, as in the reference loop (op_nn.go:877-900).
// (oh0, ow0) is the offset of the window origin: gorgonia uses the north/west pads, or, with
// explicit 4-way padding, the south/east pads (op_nn.go:870-875).
template <typename T>
__device__ __forceinline__ T lowest();
template <>
__device__ __forceinline__ float lowest<float>() { return -FLT_MAX; }
template <>
__device__ __forceinline__ double lowest<double>() { return -DBL_MAX; }

template <typename T>
__global__ void __launch_bounds__(256) maxpool_kernel(const T *__restrict__ x, T *__restrict__ y,
                                                      long long *__restrict__ mask, long long planes, int H, int W,
                                                      int Ho, int Wo, int kh, int kw, int sH, int sW, int oh0,
                                                      int ow0) {
  const long long total = planes * Ho * Wo;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int pw = (int)(t % Wo);
    const int ph = (int)((t / Wo) % Ho);
    const long long plane = t / ((long long)Wo * Ho);
    const T *in = x + plane * H * W;
    int hs = ph * sH - oh0, ws = pw * sW - ow0;
    const int he = min(hs + kh, H), we = min(ws + kw, W);
    hs = max(hs, 0);
    ws = max(ws, 0);
    T best = lowest<T>();
    long long arg = -1;
    for (int hi = hs; hi < he; ++hi)
      for (int wi = ws; wi < we; ++wi) {
        const T v = in[hi * W + wi];
        if (v > best) {
          best = v;
          arg = (long long)hi * W + wi;
        }
      }
    y[t] = best;
    if (mask) mask[t] = arg;
  }
}

// Max-pool whose result goes to a tensor-core convolution: written channels-innermost (NHWC) as a
// TF32 head and the TF32 rounding of the remainder, the form those kernels read, and optionally in
// NCHW as well. A block takes 32 channels x 32 pooled positions of one image: it pools along the
// positions (contiguous reads per channel), turns the tile in shared memory and writes along the
// channels (contiguous 128-byte rows per position). Same comparison order as maxpool_kernel.
__device__ __forceinline__ float pool_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}
template <bool K2>  // K2: a 2 x 2 window, whose four loads are issued together
__global__ void __launch_bounds__(256) maxpool_split_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                            float *__restrict__ hi, float *__restrict__ lo,
                                                            long long B, int C, int H, int W, int Ho, int Wo, int kh,
                                                            int kw, int sH, int sW, int oh0, int ow0) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int HWo = Ho * Wo;
  const int ptiles = (HWo + 31) / 32, ctiles = (C + 31) / 32;
  const long long per_image = (long long)ptiles * ctiles, total = B * per_image;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b = t / per_image;
    const int rem = (int)(t - b * per_image);
    const int ct = rem / ptiles, pt = rem - ct * ptiles;
    const int c0 = ct * 32, p0 = pt * 32;
    const int pp = p0 + tx;
    const int ph = pp / Wo, pw = pp - ph * Wo;
    int hs = ph * sH - oh0, ws = pw * sW - ow0;
    if (K2) {
      // window rows hs, hs + 1 and columns ws, ws + 1, each inside the image or not; loads go to clamped
      // addresses and the ones outside are dropped afterwards, so that all sixteen are in flight at once
      const bool r0 = hs >= 0 && hs < H, r1 = hs + 1 >= 0 && hs + 1 < H;
      const bool q0 = ws >= 0 && ws < W, q1 = ws + 1 >= 0 && ws + 1 < W;
      const int h0c = min(max(hs, 0), H - 1), h1c = min(max(hs + 1, 0), H - 1);
      const int w0c = min(max(ws, 0), W - 1), w1c = min(max(ws + 1, 0), W - 1);
      float v[4][4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = min(c0 + ty + 8 * jj, C - 1);
        const float *in = x + (b * C + c) * (long long)H * W;
        const bool live = pp < HWo;
        v[jj][0] = live ? __ldg(in + h0c * W + w0c) : 0.f;
        v[jj][1] = live ? __ldg(in + h0c * W + w1c) : 0.f;
        v[jj][2] = live ? __ldg(in + h1c * W + w0c) : 0.f;
        v[jj][3] = live ? __ldg(in + h1c * W + w1c) : 0.f;
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = ty + 8 * jj, c = c0 + j;
        float best = -FLT_MAX;   // row-major window order, strict '>': the reference's comparison
        if (r0 && q0 && v[jj][0] > best) best = v[jj][0];
        if (r0 && q1 && v[jj][1] > best) best = v[jj][1];
        if (r1 && q0 && v[jj][2] > best) best = v[jj][2];
        if (r1 && q1 && v[jj][3] > best) best = v[jj][3];
        if (y && c < C && pp < HWo) y[(b * C + c) * (long long)HWo + pp] = best;
        tile[j][tx] = best;
      }
    } else {
      const int he = min(hs + kh, H), we = min(ws + kw, W);
      hs = max(hs, 0);
      ws = max(ws, 0);
#pragma unroll
      for (int j = ty; j < 32; j += 8) {
        const int c = c0 + j;
        float best = -FLT_MAX;
        if (c < C && pp < HWo) {
          const float *in = x + (b * C + c) * (long long)H * W;
          for (int hh = hs; hh < he; ++hh)
            for (int ww = ws; ww < we; ++ww) {
              const float v = __ldg(in + hh * W + ww);
              if (v > best) best = v;
            }
          if (y) y[(b * C + c) * (long long)HWo + pp] = best;
        }
        tile[j][tx] = best;
      }
    }
    __syncthreads();
    const long long ob = b * (long long)HWo * C;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
      const int q = p0 + j, c = c0 + tx;
      if (q < HWo && c < C) {
        const float v = tile[tx][j];
        const float h = pool_tf32(v);
        const long long o = ob + (long long)q * C + c;
        hi[o] = h;
        lo[o] = pool_tf32(__fsub_rn(v, h));
      }
    }
    __syncthreads();
  }
}

// The pooling every config here uses: 2x2 window, stride 2, no padding, W a multiple of 4, no mask.
// One thread makes two neighbouring outputs from two 16-byte loads (one per input row) and writes
// them with one 8-byte store. Same comparison order as the general kernel: row-major inside the
// window, strict '>', starting from -FLT_MAX.
__global__ void __launch_bounds__(256) maxpool2x2_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                         long long planes, int H, int W, int Ho, int Wo) {
  const int pairs = Wo >> 1;  // Wo = W/2 is even because W % 4 == 0
  const long long total = planes * Ho * pairs;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int j = (int)(t % pairs);
    const int ph = (int)((t / pairs) % Ho);
    const long long plane = t / ((long long)pairs * Ho);
    const float *in = x + (plane * H + 2 * ph) * (long long)W + 4 * j;
    const float4 a = *reinterpret_cast<const float4 *>(in);
    const float4 b = *reinterpret_cast<const float4 *>(in + W);
    float m0 = -FLT_MAX, m1 = -FLT_MAX;
    if (a.x > m0) m0 = a.x;
    if (a.y > m0) m0 = a.y;
    if (b.x > m0) m0 = b.x;
    if (b.y > m0) m0 = b.y;
    if (a.z > m1) m1 = a.z;
    if (a.w > m1) m1 = a.w;
    if (b.z > m1) m1 = b.z;
    if (b.w > m1) m1 = b.w;
    *reinterpret_cast<float2 *>(y + (plane * Ho + ph) * (long long)Wo + 2 * j) = make_float2(m0, m1);
  }
}

// The same for any even W and any H: one output per thread from two 8-byte loads. A trailing
// odd input row (H odd) is simply never read, as the output size formula drops it.
__global__ void __launch_bounds__(256) maxpool2x2_even_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                              long long planes, int H, int W, int Ho, int Wo) {
  const long long total = planes * Ho * Wo;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int pw = (int)(t % Wo);
    const int ph = (int)((t / Wo) % Ho);
    const long long plane = t / ((long long)Wo * Ho);
    const float *in = x + (plane * H + 2 * ph) * (long long)W + 2 * pw;
    const float2 a = *reinterpret_cast<const float2 *>(in);
    const float2 b = *reinterpret_cast<const float2 *>(in + W);
    float m0 = -FLT_MAX;
    if (a.x > m0) m0 = a.x;
    if (a.y > m0) m0 = a.y;
    if (b.x > m0) m0 = b.x;
    if (b.y > m0) m0 = b.y;
    y[t] = m0;
  }
}

// Any other 2x2 pooling without a mask (odd planes, stride 1, gorgonia's explicit padding): one
// output per thread, the four window positions unrolled with their bounds checks, index arithmetic
// in 32 bits (the caller checks that the element counts fit). Same comparison order as the general
// kernel: row-major inside the clipped window, strict '>', starting from -FLT_MAX.
__global__ void __launch_bounds__(256) maxpool2x2_any_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                             uint32_t planes, int H, int W, int Ho, int Wo, int sH,
                                                             int sW, int oh0, int ow0) {
  const uint32_t per = (uint32_t)Ho * Wo, total = planes * per, hw = (uint32_t)H * W;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const uint32_t plane = t / per, r = t - plane * per;
    const int ph = (int)(r / (uint32_t)Wo), pw = (int)(r - (uint32_t)ph * Wo);
    const int h0 = ph * sH - oh0, w0 = pw * sW - ow0;
    const float *in = x + (size_t)plane * hw;
    float best = -FLT_MAX;
#pragma unroll
    for (int dh = 0; dh < 2; ++dh)
#pragma unroll
      for (int dw = 0; dw < 2; ++dw) {
        const int hi = h0 + dh, wi = w0 + dw;
        if ((unsigned)hi < (unsigned)H && (unsigned)wi < (unsigned)W) {
          const float v = __ldg(in + hi * W + wi);
          if (v > best) best = v;
        }
      }
    y[t] = best;
  }
}

// ---- im2col ------------------------------------------------------------------------------------
// col[(b, oh, ow), (c, r, s)] = x[b, c, oh*sH - padH + r*dH, ow*sW - padW + s*dW], 0 outside.
// One thread per column element; consecutive threads write consecutive (c, r, s), which makes
// the big side (the col buffer) perfectly coalesced while reads of x hit L1/L2.
// SPLIT: write the TF32 head and tail of each value instead (feeds the 3xTF32 matrix multiply
// without a second pass over the col buffer); the row pitch `ld` may exceed C*kh*kw (padding = 0).
__device__ __forceinline__ float to_tf32_rna(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) im2col_kernel(const T *__restrict__ x, T *__restrict__ col,
                                                     T *__restrict__ col_lo, long long B, int C, int H, int W,
                                                     int Ho, int Wo, int kh, int kw, int padH, int padW, int sH,
                                                     int sW, int dH, int dW, int ld) {
  const int crs = C * kh * kw;
  const long long total = B * Ho * Wo * (long long)ld;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int q = (int)(t % ld);
    const long long row = t / ld;
    T v = T(0);
    if (q < crs) {
      const int s = q % kw;
      const int r = (q / kw) % kh;
      const int c = q / (kw * kh);
      const int ow = (int)(row % Wo);
      const int oh = (int)((row / Wo) % Ho);
      const long long b = row / ((long long)Wo * Ho);
      const int ih = oh * sH - padH + r * dH;
      const int iw = ow * sW - padW + s * dW;
      if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = x[((b * C + c) * H + ih) * (long long)W + iw];
    }
    if (SPLIT) {
      const float h = to_tf32_rna((float)v);
      col[t] = (T)h;
      col_lo[t] = (T)to_tf32_rna(__fsub_rn((float)v, h));
    } else {
      col[t] = v;
    }
  }
}

// ---- transpose ---------------------------------------------------------------------------------
struct TransposeDesc {
  int ndim;
  long long out_shape[8];
  long long in_stride_of_out_dim[8];  // stride, in the input, of the input axis that output axis d reads
};

// General N-d permutation: one thread per output element (writes coalesced).
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ x, T *__restrict__ y, long long n,
                                                        TransposeDesc d) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long rem = i, src = 0;
#pragma unroll 1
    for (int k = d.ndim - 1; k >= 0; --k) {
      const long long c = rem % d.out_shape[k];
      rem /= d.out_shape[k];
      src += c * d.in_stride_of_out_dim[k];
    }
    y[i] = x[src];
  }
}

// Batched 2-D transpose through a padded shared-memory tile: y[b][c][r] = x[b][r][c]. Both the
// reads and the writes are coalesced. Covers (0,3,1,2)/(0,2,3,1)-style permutations of 4-D
// tensors, which collapse to this form.
template <typename T>
__global__ void __launch_bounds__(256) transpose2d_kernel(const T *__restrict__ x, T *__restrict__ y, long long R,
                                                          long long Cc) {
  __shared__ T tile[32][33];
  const long long b = blockIdx.z;
  const T *xb = x + b * R * Cc;
  T *yb = y + b * R * Cc;
  const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    const long long r = r0 + j, c = c0 + tx;
    if (r < R && c < Cc) tile[j][tx] = xb[r * Cc + c];
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const long long c = c0 + j, r = r0 + tx;
    if (r < R && c < Cc) yb[c * R + r] = tile[tx][j];
  }
}

// ---- gather of rows ------------------------------------------------------------------------------
// y[i, :] = x[idx[i], :]; rows are copied in 16-byte words when the row size and the bases allow.
// An index outside [0, n_rows) raises the flag and leaves the row untouched.
// With outer > 1 the same gather is applied to every leading slice: y[o, i, :] = x[o, idx[i], :].
template <typename W>
__global__ void __launch_bounds__(256) gather_rows_kernel(const W *__restrict__ x, const long long *__restrict__ idx,
                                                          W *__restrict__ y, long long outer, long long n_idx,
                                                          long long row_words, long long n_rows, int *bad) {
  const long long total = outer * n_idx * row_words;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const long long w = t % row_words;
    const long long i = (t / row_words) % n_idx;
    const long long o = t / (row_words * n_idx);
    const long long src = idx[i];
    if (src < 0 || src >= n_rows) {
      if (w == 0) atomicExch(bad, 1);
      continue;
    }
    y[t] = x[(o * n_rows + src) * row_words + w];
  }
}

// Gradient of the max-pool with respect to its input (maxPoolDiffOp.f32s, op_nn.go:1067-1093): the
// reference zeroes the gradient and adds every pooled position's gradient to the input position its
// mask entry names, walking the pooled plane in (ph, pw) order. Here one thread owns one INPUT
// element, visits the windows that can contain it in the same (ph, pw) order and adds those whose
// mask entry names it: the same additions in the same order, so the result is bit-identical also
// where windows overlap, and no atomics are needed.
template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const T *__restrict__ dy, const long long *__restrict__ mask,
                                                          T *__restrict__ dx, long long planes, int H, int W, int Ho,
                                                          int Wo, int kh, int kw, int sH, int sW, int oh0, int ow0) {
  const long long total = planes * H * W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int w = (int)(t % W);
    const int h = (int)((t / W) % H);
    const long long plane = t / ((long long)W * H);
    const long long me = (long long)h * W + w;
    // windows (ph, pw) with ph*sH - oh0 <= h < ph*sH - oh0 + kh
    int ph_lo = h + oh0 - kh + 1;
    ph_lo = ph_lo <= 0 ? 0 : (ph_lo + sH - 1) / sH;
    const int ph_hi = min((h + oh0) / sH, Ho - 1);
    int pw_lo = w + ow0 - kw + 1;
    pw_lo = pw_lo <= 0 ? 0 : (pw_lo + sW - 1) / sW;
    const int pw_hi = min((w + ow0) / sW, Wo - 1);
    const long long *mk = mask + plane * Ho * Wo;
    const T *g = dy + plane * Ho * Wo;
    T acc = T(0);
    for (int ph = ph_lo; ph <= ph_hi; ++ph)
      for (int pw = pw_lo; pw <= pw_hi; ++pw)
        if (mk[ph * Wo + pw] == me) acc = acc + g[ph * Wo + pw];
    dx[t] = acc;
  }
}

// col (B, Ho, Wo, C*kh*kw) accumulated back into the image (col2imOp.f32s, op_nn.go:603-637). The
// reference walks col in memory order, so the additions that land on one pixel happen in ascending
// (output row, output column) order. One thread owns one pixel and makes the same additions in the
// same order: ascending output row means descending kernel row, likewise for columns.
template <typename T>
__global__ void __launch_bounds__(256) col2im_kernel(const T *__restrict__ col, T *__restrict__ im, long long B, int C,
                                                     int H, int W, int Ho, int Wo, int kh, int kw, int padH, int padW,
                                                     int sH, int sW, int dH, int dW) {
  const long long total = B * C * H * W;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int crs = C * kh * kw;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int iw = (int)(t % W);
    const int ih = (int)((t / W) % H);
    const int c = (int)((t / ((long long)W * H)) % C);
    const long long b = t / ((long long)W * H * C);
    const T *colb = col + b * (long long)Ho * Wo * crs + (long long)c * kh * kw;
    T acc = T(0);
    for (int r = kh - 1; r >= 0; --r) {
      const int num_h = ih + padH - r * dH;
      if (num_h < 0 || num_h % sH != 0) continue;
      const int oh = num_h / sH;
      if (oh >= Ho) continue;
      for (int sx = kw - 1; sx >= 0; --sx) {
        const int num_w = iw + padW - sx * dW;
        if (num_w < 0 || num_w % sW != 0) continue;
        const int ow = num_w / sW;
        if (ow >= Wo) continue;
        acc = acc + colb[((long long)oh * Wo + ow) * crs + r * kw + sx];
      }
    }
    im[t] = acc;
  }
}

// The gradient of the pooling every config here uses (2x2 window, stride 2, no padding, W a multiple
// of 4): windows do not overlap, so an input element receives at most one term, 0 + dy (the
// reference adds into a zeroed array, which turns a -0.0 gradient into +0.0; so does this). One
// thread handles two neighbouring windows: 8 bytes of gradient and 16 of mask in, two float4 rows
// out. Rows and columns past the last whole window (odd H) are written as zeros.
__global__ void __launch_bounds__(256) maxpool2x2_bwd_kernel(const float *__restrict__ dy,
                                                             const long long *__restrict__ mask,
                                                             float *__restrict__ dx, long long planes, int H, int W,
                                                             int Ho, int Wo) {
  const int pairs = Wo >> 1;  // Wo = W/2 is even because W % 4 == 0
  const int rows = (H + 1) >> 1;  // one extra, window-less row when H is odd
  const long long total = planes * rows * pairs;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int j = (int)(t % pairs);
    const int ph = (int)((t / pairs) % rows);
    const long long plane = t / ((long long)pairs * rows);
    float *out = dx + (plane * H + 2 * ph) * (long long)W + 4 * j;
    if (ph >= Ho) {  // the last row of an odd-height plane belongs to no window
      *reinterpret_cast<float4 *>(out) = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    const long long o = (plane * Ho + ph) * (long long)Wo + 2 * j;
    const float2 g = *reinterpret_cast<const float2 *>(dy + o);
    const longlong2 m = *reinterpret_cast<const longlong2 *>(mask + o);
    const long long base = (long long)(2 * ph) * W + 4 * j;  // index of out[0] inside the plane
    const float g0 = 0.f + g.x, g1 = 0.f + g.y;
    float4 r0, r1;
    r0.x = m.x == base ? g0 : 0.f;
    r0.y = m.x == base + 1 ? g0 : 0.f;
    r0.z = m.y == base + 2 ? g1 : 0.f;
    r0.w = m.y == base + 3 ? g1 : 0.f;
    r1.x = m.x == base + W ? g0 : 0.f;
    r1.y = m.x == base + W + 1 ? g0 : 0.f;
    r1.z = m.y == base + W + 2 ? g1 : 0.f;
    r1.w = m.y == base + W + 3 ? g1 : 0.f;
    *reinterpret_cast<float4 *>(out) = r0;
    *reinterpret_cast<float4 *>(out + W) = r1;
  }
}

// col2im for stride-1, undilated rows with the col rows staged in shared memory: a block walks one
// image from top to bottom and keeps the kh col rows that can touch the current image row in a
// ring (slot = output row mod kh), so every col row is read from memory exactly once, with
// consecutive threads on consecutive addresses. The ring's pitch is padded by one word so that
// neighbouring pixels hit different banks. Every pixel adds its taps in the reference's order
// (ascending output row and column = descending kernel row and column).
template <typename T, bool UNIT_W>  // UNIT_W: stride 1 and no dilation along W as well (no divisions)
__global__ void __launch_bounds__(256) col2im_rows_kernel(const T *__restrict__ col, T *__restrict__ im, long long B,
                                                          int C, int H, int W, int Ho, int Wo, int kh, int kw,
                                                          int padH, int padW, int sW, int dW) {
  extern __shared__ __align__(16) unsigned char c2i_smem[];
  T *ring = reinterpret_cast<T *>(c2i_smem);
  const int crs = C * kh * kw, khw = kh * kw;
  const int pitch = crs + 1;
  const long long row_elems = (long long)Wo * crs;
  auto load_row = [&](long long b, int oh) {
    const T *src = col + (b * Ho + oh) * row_elems;
    T *dst = ring + (long long)(oh % kh) * Wo * pitch;
    int ow = 0, q = threadIdx.x;  // element i = ow * crs + q of the row, i = threadIdx.x, + 256, ...
    for (long long i = threadIdx.x; i < row_elems; i += blockDim.x, q += blockDim.x) {
      while (q >= crs) {
        q -= crs;
        ++ow;
      }
      dst[ow * pitch + q] = src[i];
    }
  };
  for (long long b = blockIdx.x; b < B; b += gridDim.x) {
    for (int oh = 0; oh < padH && oh < Ho; ++oh) load_row(b, oh);  // rows above the first new one
    for (int ih = 0; ih < H; ++ih) {
      if (ih + padH < Ho) load_row(b, ih + padH);
      __syncthreads();
      T *out = im + (b * C * H + ih) * (long long)W;
      for (int i = threadIdx.x; i < C * W; i += blockDim.x) {
        const int c = i / W, iw = i - c * W;
        T acc = T(0);
        for (int r = kh - 1; r >= 0; --r) {
          const int oh = ih + padH - r;
          if (oh < 0 || oh >= Ho) continue;
          const T *slot = ring + (long long)(oh % kh) * Wo * pitch + c * khw + r * kw;
          for (int sx = kw - 1; sx >= 0; --sx) {
            int ow;
            if (UNIT_W) {
              ow = iw + padW - sx;
              if (ow < 0) continue;
            } else {
              const int num_w = iw + padW - sx * dW;
              if (num_w < 0 || num_w % sW != 0) continue;
              ow = num_w / sW;
            }
            if (ow >= Wo) continue;
            acc = acc + slot[ow * pitch + sx];
          }
        }
        out[(long long)c * H * W + iw] = acc;
      }
      __syncthreads();
    }
  }
}

// The float32 ring kernel with the memory side pipelined: C*kh*kw a multiple of 4, so a col row is
// a whole number of float4 that never straddle two output columns. A thread holds up to 8 float4
// of the NEXT col row in registers; their loads are issued before the current image row is
// computed and land while it runs, instead of one dependent load per loop trip. Where a thread's
// float4 land in a ring row, and which (channel, column) outputs it computes, is the same for every
// row of every image: both are worked out once, so no element pays an index division. The ring
// holds kh + 1 rows: the row being stashed is then never one the row being computed reads, and one
// barrier per image row is enough.
template <bool UNIT_W>
__global__ void __launch_bounds__(256) col2im_rows4_kernel(const float *__restrict__ col, float *__restrict__ im,
                                                           long long B, int C, int H, int W, int Ho, int Wo, int kh,
                                                           int kw, int padH, int padW, int sW, int dW) {
  extern __shared__ __align__(16) unsigned char c2i4_smem[];
  float *ring = reinterpret_cast<float *>(c2i4_smem);
  const int crs = C * kh * kw, khw = kh * kw;
  const int pitch = crs + 1;
  const int row_vec = (Wo * crs) >> 2;  // float4 per col row, at most 8 * 256
  const int slots = kh + 1, slot_floats = Wo * pitch;
  float4 pre[8];
  int stash_at[8];  // offset of float4 v of a col row inside a ring row, or -1
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    const int i = threadIdx.x + v * 256;
    const int e0 = i << 2, ow = e0 / crs;
    stash_at[v] = i < row_vec ? ow * pitch + (e0 - ow * crs) : -1;
  }
  constexpr int NOUT = 4;  // outputs per thread and image row kept in registers; more take the slow loop
  int out_c[NOUT], out_w[NOUT];
#pragma unroll
  for (int k = 0; k < NOUT; ++k) {
    const int i = threadIdx.x + k * 256;
    out_c[k] = i < C * W ? i / W : -1;
    out_w[k] = i - (i / W) * W;
  }
  auto fetch = [&](long long b, int oh) {
    const float4 *src = reinterpret_cast<const float4 *>(col + (b * Ho + oh) * (long long)Wo * crs);
#pragma unroll
    for (int v = 0; v < 8; ++v)
      if (stash_at[v] >= 0) pre[v] = __ldg(src + threadIdx.x + v * 256);
  };
  auto stash = [&](int oh) {
    float *dst = ring + (oh % slots) * slot_floats;
#pragma unroll
    for (int v = 0; v < 8; ++v)
      if (stash_at[v] >= 0) {
        float *d = dst + stash_at[v];
        d[0] = pre[v].x; d[1] = pre[v].y; d[2] = pre[v].z; d[3] = pre[v].w;
      }
  };
  // the sum of one output, taps in the reference's order (bottom-right tap first)
  auto gather = [&](int ih, int c, int iw) {
    float acc = 0.f;
    for (int r = kh - 1; r >= 0; --r) {
      const int oh = ih + padH - r;
      if (oh < 0 || oh >= Ho) continue;
      const float *slot = ring + (oh % slots) * slot_floats + c * khw + r * kw;
      for (int sx = kw - 1; sx >= 0; --sx) {
        int ow;
        if (UNIT_W) {
          ow = iw + padW - sx;
          if (ow < 0) continue;
        } else {
          const int num_w = iw + padW - sx * dW;
          if (num_w < 0 || num_w % sW != 0) continue;
          ow = num_w / sW;
        }
        if (ow >= Wo) continue;
        acc = acc + slot[ow * pitch + sx];
      }
    }
    return acc;
  };
  for (long long b = blockIdx.x; b < B; b += gridDim.x) {
    __syncthreads();  // the previous image's last rows have been read
    for (int oh = 0; oh < padH && oh < Ho; ++oh) {  // rows above the first new one
      fetch(b, oh);
      stash(oh);
    }
    if (padH < Ho) fetch(b, padH);
    for (int ih = 0; ih < H; ++ih) {
      if (ih + padH < Ho) stash(ih + padH);
      __syncthreads();
      if (ih + 1 + padH < Ho) fetch(b, ih + 1 + padH);  // lands while this image row is computed
      float *out = im + (b * C * H + ih) * (long long)W;
#pragma unroll
      for (int k = 0; k < NOUT; ++k)
        if (out_c[k] >= 0) out[(long long)out_c[k] * H * W + out_w[k]] = gather(ih, out_c[k], out_w[k]);
      for (int i = threadIdx.x + NOUT * 256; i < C * W; i += blockDim.x) {
        const int c = i / W, iw = i - c * W;
        out[(long long)c * H * W + iw] = gather(ih, c, iw);
      }
    }
  }
}

// The 3 x 3-class case (stride 1, no dilation, float32, C*kh*kw a multiple of 4) with the memory side
// taken off the threads altogether. A col row (one output row of positions: Wo * crs floats) is one
// bulk asynchronous copy into a ring of R shared-memory rows, queued by one thread up to R - kh rows
// ahead across image boundaries, its landing signalled by an mbarrier; nobody holds col data in
// registers. The rows lie unpadded, so consecutive channels of one position are kh*kw words apart:
// a warp takes 32 consecutive channels of one column (bank-conflict free for odd kh*kw), sums the
// taps in the reference's order (bottom-right first, acc = acc + v from 0), and puts the value into a
// shared-memory copy of the image, which leaves for HBM as one linear pass per image. One barrier
// per image row; every mbarrier wait is bounded.
constexpr int C2I_MAX_RING = 8;
constexpr int C2I_THREADS = 512;

template <int KH, int KW>
__global__ void __launch_bounds__(C2I_THREADS, 2) col2im_bulk_kernel(const float *__restrict__ col, float *__restrict__ im,
                                                          long long B, int C, int H, int W, int Ho, int Wo, int padH,
                                                          int padW, int R, int *err_flag) {
  extern __shared__ __align__(128) unsigned char c2ib_smem[];
  __shared__ __align__(8) uint64_t full[C2I_MAX_RING];
  __shared__ int s_fail;
  constexpr int KHW = KH * KW;
  const int crs = C * KHW;
  const int row_floats = Wo * crs;
  const uint32_t row_bytes = (uint32_t)row_floats * 4u;
  float *ring = reinterpret_cast<float *>(c2ib_smem);
  float *outimg = ring + (size_t)R * row_floats;
  const int plane = H * W, img_floats = C * plane;

  const long long my_images = blockIdx.x < B ? (B - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    for (int s2 = 0; s2 < R; ++s2) ptx::mbar_init(&full[s2], 1);
    ptx::fence_mbar_init();
    s_fail = 0;
  }
  __syncthreads();
  // Every index below advances by one step at a time: nothing in the loops divides.
  long long issued = 0;                      // thread 0 only: rows queued so far,
  long long iss_k = 0;                       // the image (of this block) and row the next one is,
  int iss_oh = 0, iss_slot = 0;              // and the ring slot it goes to
  auto issue_upto = [&](long long freed) {
    while (iss_k < my_images && issued - freed < R) {
      const long long b = blockIdx.x + iss_k * gridDim.x;
      ptx::mbar_arrive_expect_tx(&full[iss_slot], row_bytes);
      ptx::bulk_g2s(ring + (size_t)iss_slot * row_floats, col + (b * Ho + iss_oh) * (long long)row_floats, row_bytes,
                    &full[iss_slot]);
      ++issued;
      if (++iss_oh == Ho) {
        iss_oh = 0;
        ++iss_k;
      }
      if (++iss_slot == R) iss_slot = 0;
    }
  };
  if (threadIdx.x == 0) issue_upto(0);

  // the (channel, column) outputs of this thread in an image row: channel fastest
  constexpr int NOUT = 2;
  int out_c[NOUT], out_w[NOUT];
#pragma unroll
  for (int k = 0; k < NOUT; ++k) {
    const int i = threadIdx.x + k * C2I_THREADS;
    out_w[k] = i / C;
    out_c[k] = i < C * W ? i - out_w[k] * C : -1;
  }
  long long waited = 0;  // rows whose barrier this thread has seen complete,
  int w_slot = 0;        // the slot of the next one
  uint32_t w_phase = 0;  // and the parity its barrier completes with
  int img_slot0 = 0;     // ring slot of the current image's row 0
  long long row0 = 0;    // that row's place in the block's sequence
  bool ok = true;
  for (long long k = 0; k < my_images && ok; ++k) {
    const long long b = blockIdx.x + k * gridDim.x;
    int cur = (img_slot0 + padH) % R;  // slot of row ih + padH (a row past the last one exists only as an index)
    for (int ih = 0; ih < H; ++ih) {
      const int newest = ih + padH < Ho - 1 ? ih + padH : Ho - 1;
      bool landed = true;
      while (waited <= row0 + newest) {
        if (!ptx::mbar_wait(&full[w_slot], w_phase)) {
          landed = false;
          break;
        }
        ++waited;
        if (++w_slot == R) {
          w_slot = 0;
          w_phase ^= 1u;
        }
      }
      auto gather = [&](int c, int iw) {
        float acc = 0.f;
#pragma unroll
        for (int r = KH - 1; r >= 0; --r) {
          const int oh = ih + padH - r;
          if (oh < 0 || oh >= Ho) continue;
          const int slot = cur - r < 0 ? cur - r + R : cur - r;
          const float *rowp = ring + slot * row_floats + c * KHW + r * KW;
#pragma unroll
          for (int sx = KW - 1; sx >= 0; --sx) {
            const int ow = iw + padW - sx;
            if (ow < 0 || ow >= Wo) continue;
            acc = acc + rowp[ow * crs + sx];
          }
        }
        return acc;
      };
      if (landed) {
#pragma unroll
        for (int q = 0; q < NOUT; ++q)
          if (out_c[q] >= 0) outimg[out_c[q] * plane + ih * W + out_w[q]] = gather(out_c[q], out_w[q]);
        for (int i = threadIdx.x + NOUT * C2I_THREADS; i < C * W; i += C2I_THREADS) {
          const int iw = i / C, c = i - iw * C;
          outimg[c * plane + ih * W + iw] = gather(c, iw);
        }
      }
      // this row's reads are over; a wait that ran out in any thread ends the block for all of them
      if (!__syncthreads_and(landed ? 1 : 0)) {
        ok = false;
        break;
      }
      if (threadIdx.x == 0) {
        // rows of this image that no later output row reads; after the last output row, all of them
        int dead = ih + padH - (KH - 1) + 1;
        dead = ih == H - 1 ? Ho : (dead < 0 ? 0 : (dead > Ho ? Ho : dead));
        issue_upto(row0 + dead);
      }
      if (++cur == R) cur = 0;
    }
    if (!ok) break;
    // the image is complete in shared memory (the barrier above): one linear pass to HBM
    float *dst = im + b * (long long)img_floats;
    if ((img_floats & 3) == 0 && ((uintptr_t)dst & 15) == 0) {
      for (int i = threadIdx.x; i < (img_floats >> 2); i += C2I_THREADS)
        reinterpret_cast<float4 *>(dst)[i] = reinterpret_cast<const float4 *>(outimg)[i];
    } else {
      for (int i = threadIdx.x; i < img_floats; i += C2I_THREADS) dst[i] = outimg[i];
    }
    __syncthreads();  // before the next image's first row overwrites the copy
    row0 += Ho;
    img_slot0 = (img_slot0 + Ho) % R;
  }
  if (!ok) s_fail = 1;
  __syncthreads();
  if (threadIdx.x == 0 && s_fail) {
    // A wait ran out. Report it, and give the copies still queued a last bounded chance to land before
    // this block's shared memory goes away.
    atomicExch(err_flag, 1);
    const long long first = issued > R ? issued - R : 0;
    for (long long q = first; q < issued; ++q)
      ptx::mbar_wait(&full[(int)(q % R)], (uint32_t)((q / R) & 1), 100000000ull);
  }
}

// ---- BatchNormOp (op_nn.go:1346-1640) on (B, C, S) -------------------------------------------------
// Three launches. (1) partial sums of x and x^2 per (channel, group of samples) in double; (2) one
// thread per channel folds the groups in a fixed order and makes everything that is per channel:
// saveMean = sum / n rounded to the tensor's type, saveVar = sum (x - saveMean)^2 (from the two sums:
// sum x^2 - 2 m sum x + n m^2, in double), the running statistics, alpha = 1 / sqrt(var + eps) and
// beta = -mean * alpha in the tensor's type as the reference computes them; (3) y = x * alpha + beta,
// a product then a sum, plane by plane so that no element pays an index division. The reference sums
// sequentially in the tensor's type; the double sums here are closer to the exact value.
constexpr int BN_GROUPS = 64;

template <typename T>
__global__ void __launch_bounds__(256) bn_partial_kernel(const T *__restrict__ x, long long B, int C, long long S,
                                                         double *__restrict__ part) {
  const int c = blockIdx.x, grp = blockIdx.y;
  const long long per = (B + BN_GROUPS - 1) / BN_GROUPS;
  const long long b0 = grp * per, b1 = min(B, b0 + per);
  double s1 = 0.0, s2 = 0.0;
  if (sizeof(T) == 4 && S % 4 == 0 && (uintptr_t)x % 16 == 0 && (b1 - b0) * (S >> 2) < (1LL << 31)) {
    // float planes as float4; the threads spread over (sample, float4) pairs so that short planes
    // keep the whole block busy
    const uint32_t S4 = (uint32_t)(S >> 2), total4 = (uint32_t)(b1 > b0 ? (b1 - b0) * S4 : 0);
    for (uint32_t i = threadIdx.x; i < total4; i += blockDim.x) {
      const uint32_t bb = i / S4, d = i - bb * S4;
      const float4 q = __ldg(reinterpret_cast<const float4 *>(x + ((b0 + bb) * C + c) * S) + d);
      const double v0 = q.x, v1 = q.y, v2 = q.z, v3 = q.w;
      s1 += (v0 + v1) + (v2 + v3);
      s2 += (v0 * v0 + v1 * v1) + (v2 * v2 + v3 * v3);
    }
  } else if (S >= 32) {
    for (long long b = b0; b < b1; ++b) {
      const T *p = x + (b * C + c) * S;
      for (long long d = threadIdx.x; d < S; d += blockDim.x) {
        const double v = p[d];
        s1 += v;
        s2 += v * v;
      }
    }
  } else {  // short planes (a matrix has S = 1): threads spread over (sample, position) pairs
    for (long long i = b0 * S + threadIdx.x; i < b1 * S; i += blockDim.x) {
      const long long b = i / S, d = i - b * S;
      const double v = x[(b * C + c) * S + d];
      s1 += v;
      s2 += v * v;
    }
  }
  __shared__ double sh1[8], sh2[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if ((threadIdx.x & 31) == 0) {
    sh1[threadIdx.x >> 5] = s1;
    sh2[threadIdx.x >> 5] = s2;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0.0, b2 = 0.0;
    for (int w = 0; w < 8; ++w) {
      a += sh1[w];
      b2 += sh2[w];
    }
    part[((long long)c * BN_GROUPS + grp) * 2] = a;
    part[((long long)c * BN_GROUPS + grp) * 2 + 1] = b2;
  }
}

template <typename T>
__global__ void bn_finish_kernel(const double *__restrict__ part, int C, long long n, int training, T momentum, T eps,
                                 T *__restrict__ running_mean, T *__restrict__ running_var, T *__restrict__ save_mean,
                                 T *__restrict__ save_var, T *__restrict__ alpha_beta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  T mean, inv;
  if (training) {
    double s1 = 0.0, s2 = 0.0;
    for (int gq = 0; gq < BN_GROUPS; ++gq) {
      s1 += part[((long long)c * BN_GROUPS + gq) * 2];
      s2 += part[((long long)c * BN_GROUPS + gq) * 2 + 1];
    }
    const T m = (T)(s1 / (double)n);
    const double md = (double)m;
    double vd = s2 - 2.0 * md * s1 + (double)n * md * md;
    if (vd < 0.0) vd = 0.0;
    const T v = (T)vd;
    save_mean[c] = m;
    save_var[c] = v;
    running_mean[c] = momentum * m + (T(1) - momentum) * running_mean[c];
    running_var[c] = momentum * (v / (T)(n - 1)) + (T(1) - momentum) * running_var[c];
    mean = m;
    inv = T(1) / sqrt(v / (T)n + eps);
  } else {
    mean = running_mean[c];
    inv = T(1) / sqrt(running_var[c] + eps);
  }
  alpha_beta[2 * c] = inv;
  alpha_beta[2 * c + 1] = -mean * inv;
}

__device__ __forceinline__ float bn_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double bn_mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float bn_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double bn_add(double a, double b) { return __dadd_rn(a, b); }

// GROUP threads (a warp or a whole block) walk one (sample, channel) plane at a time
template <typename T, int GROUP>
__global__ void __launch_bounds__(256) bn_apply_kernel(const T *__restrict__ x, T *__restrict__ y, long long planes,
                                                       int C, long long S, const T *__restrict__ alpha_beta,
                                                       bool vec4) {
  const long long group0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / GROUP;
  const long long ngroups = ((long long)gridDim.x * blockDim.x) / GROUP;
  const int lane = threadIdx.x % GROUP;
  for (long long pl = group0; pl < planes; pl += ngroups) {
    const int c = (int)(pl % C);
    const T a = alpha_beta[2 * c], b = alpha_beta[2 * c + 1];
    const T *xp = x + pl * S;
    T *yp = y + pl * S;
    if (sizeof(T) == 4 && vec4) {  // S % 4 == 0 and both tensors 16-byte aligned: float4 in, float4 out
      const float4 *x4 = reinterpret_cast<const float4 *>(xp);
      float4 *y4 = reinterpret_cast<float4 *>(yp);
      const float fa = (float)a, fb = (float)b;
      for (long long d = lane; d < (S >> 2); d += GROUP) {
        float4 q = __ldg(x4 + d);
        q.x = __fadd_rn(__fmul_rn(q.x, fa), fb);
        q.y = __fadd_rn(__fmul_rn(q.y, fa), fb);
        q.z = __fadd_rn(__fmul_rn(q.z, fa), fb);
        q.w = __fadd_rn(__fmul_rn(q.w, fa), fb);
        y4[d] = q;
      }
    } else {
      for (long long d = lane; d < S; d += GROUP) yp[d] = bn_add(bn_mul(xp[d], a), b);
    }
  }
}

// ---- batchnormDiffOp (op_nn.go:1727-1940): the input gradient of BatchNormOp --------------------
// Same three-launch shape as the forward op: partial sums of dy and x*dy per (channel, sample group)
// in double; one thread per channel folds them into gradMean = sum dy / n, dotp = sum (x - mean) dy,
// k = dotp * invstd^2 / n in the tensor's type; the output pass then evaluates the reference's
// expression, including its order of subtractions, which differs between the matrix and the
// spatial branch, and its choice of variance in inference mode.
template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_partial_kernel(const T *__restrict__ x, const T *__restrict__ dy,
                                                             long long B, int C, long long S,
                                                             double *__restrict__ part) {
  const int c = blockIdx.x, grp = blockIdx.y;
  const long long per = (B + BN_GROUPS - 1) / BN_GROUPS;
  const long long b0 = grp * per, b1 = min(B, b0 + per);
  double s1 = 0.0, s2 = 0.0;
  for (long long i = b0 * S + threadIdx.x; i < b1 * S; i += blockDim.x) {
    const long long b = i / S, d = i - b * S;
    const long long at = (b * C + c) * S + d;
    const double g = dy[at];
    s1 += g;
    s2 += (double)x[at] * g;
  }
  __shared__ double sh1[8], sh2[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if ((threadIdx.x & 31) == 0) {
    sh1[threadIdx.x >> 5] = s1;
    sh2[threadIdx.x >> 5] = s2;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0.0, b2 = 0.0;
    for (int w = 0; w < 8; ++w) {
      a += sh1[w];
      b2 += sh2[w];
    }
    part[((long long)c * BN_GROUPS + grp) * 2] = a;
    part[((long long)c * BN_GROUPS + grp) * 2 + 1] = b2;
  }
}

template <typename T>
__global__ void bn_bwd_finish_kernel(const double *__restrict__ part, int C, long long n, long long S, int training,
                                     T eps, const T *__restrict__ running_var, const T *__restrict__ save_mean,
                                     const T *__restrict__ save_var, T *__restrict__ coef) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s1 = 0.0, s2 = 0.0;
  for (int gq = 0; gq < BN_GROUPS; ++gq) {
    s1 += part[((long long)c * BN_GROUPS + gq) * 2];
    s2 += part[((long long)c * BN_GROUPS + gq) * 2 + 1];
  }
  const T mean = save_mean[c];
  const T sum = (T)s1, dotp = (T)(s2 - (double)mean * s1);
  T invstd = T(1) / sqrt(save_var[c] / (T)n + eps);
  if (!training && S == 1) invstd = T(1) / sqrt(running_var[c] + eps);
  coef[4 * c] = mean;
  coef[4 * c + 1] = (T)(dotp * invstd * invstd) / (T)n;  // k
  coef[4 * c + 2] = sum / (T)n;                          // gradMean
  coef[4 * c + 3] = invstd;
}

__device__ __forceinline__ float bn_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double bn_sub(double a, double b) { return __dsub_rn(a, b); }

template <typename T>
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const T *__restrict__ x, const T *__restrict__ dy,
                                                           T *__restrict__ dx, long long planes, int C, long long S,
                                                           int training, const T *__restrict__ coef) {
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long pl = warp0; pl < planes; pl += nwarps) {
    const int c = (int)(pl % C);
    const T mean = coef[4 * c], k = coef[4 * c + 1], gm = coef[4 * c + 2], inv = coef[4 * c + 3];
    const T *xp = x + pl * S, *gp = dy + pl * S;
    T *op = dx + pl * S;
    for (long long d = lane; d < S; d += 32) {
      if (!training) {
        op[d] = bn_mul(gp[d], inv);
      } else {
        const T t = bn_mul(bn_sub(xp[d], mean), k);
        const T u = S == 1 ? bn_sub(bn_sub(gp[d], t), gm) : bn_sub(bn_sub(gp[d], gm), t);
        op[d] = bn_mul(u, inv);
      }
    }
  }
}

static int grid_for(b200_engine *e, long long work) {
  return (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, (long long)e->sm_count * 16));
}

template <typename T>
static int batchnorm_fwd_t(b200_engine *e, const T *x, T *y, long long B, int C, long long S, int training,
                           double momentum, double eps, T *running_mean, T *running_var, T *save_mean, T *save_var) {
  void *part = nullptr, *ab = nullptr;
  int rc = b200_get(e, (long long)C * BN_GROUPS * 2 * sizeof(double), &part);
  if (rc == B200_OK) rc = b200_get(e, (long long)C * 2 * sizeof(T), &ab);
  if (rc != B200_OK) {
    if (part) b200_put(e, part, 0);
    return rc;
  }
  auto done = [&](int r) {
    b200_put(e, part, 0);
    b200_put(e, ab, 0);
    return r;
  };
  if (training) {
    bn_partial_kernel<T><<<dim3(C, BN_GROUPS), 256, 0, e->stream>>>(x, B, C, S, (double *)part);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_partial_kernel: %s", cudaGetErrorString(le)));
    e->launches++;
  }
  bn_finish_kernel<T><<<(C + 127) / 128, 128, 0, e->stream>>>((const double *)part, C, B * S, training, (T)momentum,
                                                              (T)eps, running_mean, running_var, save_mean, save_var,
                                                              (T *)ab);
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_finish_kernel: %s", cudaGetErrorString(le)));
  e->launches++;
  const long long planes = B * C;
  const bool vec4 = S % 4 == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0;
  if (S >= 2048) {
    const int blocks = (int)std::max<long long>(1, std::min<long long>(planes, (long long)e->sm_count * 16));
    bn_apply_kernel<T, 256><<<blocks, 256, 0, e->stream>>>(x, y, planes, C, S, (const T *)ab, vec4);
  } else {
    const int blocks = (int)std::max<long long>(1, std::min<long long>((planes + 7) / 8, (long long)e->sm_count * 16));
    bn_apply_kernel<T, 32><<<blocks, 256, 0, e->stream>>>(x, y, planes, C, S, (const T *)ab, vec4);
  }
  le = cudaGetLastError();
  if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_apply_kernel: %s", cudaGetErrorString(le)));
  e->launches++;
  return done(B200_OK);
}

template <typename T>
static int batchnorm_bwd_t(b200_engine *e, const T *x, const T *dy, T *dx, long long B, int C, long long S,
                           int training, double eps, const T *running_var, const T *save_mean, const T *save_var) {
  void *part = nullptr, *coef = nullptr;
  int rc = b200_get(e, (long long)C * BN_GROUPS * 2 * sizeof(double), &part);
  if (rc == B200_OK) rc = b200_get(e, (long long)C * 4 * sizeof(T), &coef);
  if (rc != B200_OK) {
    if (part) b200_put(e, part, 0);
    return rc;
  }
  auto done = [&](int r) {
    b200_put(e, part, 0);
    b200_put(e, coef, 0);
    return r;
  };
  bn_bwd_partial_kernel<T><<<dim3(C, BN_GROUPS), 256, 0, e->stream>>>(x, dy, B, C, S, (double *)part);
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_bwd_partial_kernel: %s", cudaGetErrorString(le)));
  e->launches++;
  bn_bwd_finish_kernel<T><<<(C + 127) / 128, 128, 0, e->stream>>>((const double *)part, C, B * S, S, training, (T)eps,
                                                                  running_var, save_mean, save_var, (T *)coef);
  le = cudaGetLastError();
  if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_bwd_finish_kernel: %s", cudaGetErrorString(le)));
  e->launches++;
  const long long planes = B * C;
  const int blocks = (int)std::max<long long>(1, std::min<long long>((planes + 7) / 8, (long long)e->sm_count * 16));
  bn_bwd_apply_kernel<T><<<blocks, 256, 0, e->stream>>>(x, dy, dx, planes, C, S, training, (const T *)coef);
  le = cudaGetLastError();
  if (le != cudaSuccess) return done(set_error(e, B200_ERR_CUDA, "bn_bwd_apply_kernel: %s", cudaGetErrorString(le)));
  e->launches++;
  return done(B200_OK);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_maxpool2d_split_fwd(b200_engine *e, const void *x, void *y, void *y_hi, void *y_lo, int64_t B, int64_t C,
                             int64_t H, int64_t W, int kh, int kw, int pad_north, int pad_south, int pad_west,
                             int pad_east, int explicit_padding, int stride_h, int stride_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, B >= 0 && C >= 0 && H > 0 && W > 0, "b200_maxpool2d_split_fwd: bad input shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0, "b200_maxpool2d_split_fwd: bad kernel or stride");
  B200_REQUIRE(e, pad_north >= 0 && pad_south >= 0 && pad_west >= 0 && pad_east >= 0,
               "b200_maxpool2d_split_fwd: bad pad");
  B200_REQUIRE(e, H < 32768 && W < 32768 && C < (1LL << 30), "b200_maxpool2d_split_fwd: image too large");
  const long long Ho = (H + pad_south + pad_north - (kh - 1) - 1) / stride_h + 1;
  const long long Wo = (W + pad_east + pad_west - (kw - 1) - 1) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_maxpool2d_split_fwd: window larger than the padded image");
  if (B * C == 0) return B200_OK;
  B200_REQUIRE(e, x && y_hi && y_lo, "b200_maxpool2d_split_fwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const long long tiles = B * ((Ho * Wo + 31) / 32) * ((C + 31) / 32);
  const int blocks = (int)std::max<long long>(1, std::min<long long>(tiles, (long long)e->sm_count * 32));
  const int oh0 = explicit_padding ? pad_south : pad_north, ow0 = explicit_padding ? pad_east : pad_west;
  if (kh == 2 && kw == 2)
    maxpool_split_kernel<true><<<blocks, 256, 0, e->stream>>>((const float *)x, (float *)y, (float *)y_hi,
                                                              (float *)y_lo, B, (int)C, (int)H, (int)W, (int)Ho,
                                                              (int)Wo, kh, kw, stride_h, stride_w, oh0, ow0);
  else
    maxpool_split_kernel<false><<<blocks, 256, 0, e->stream>>>((const float *)x, (float *)y, (float *)y_hi,
                                                               (float *)y_lo, B, (int)C, (int)H, (int)W, (int)Ho,
                                                               (int)Wo, kh, kw, stride_h, stride_w, oh0, ow0);
  B200_CHECK_LAUNCH(e, "maxpool_split_kernel");
  return B200_OK;
}

int b200_maxpool2d_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t *mask, int64_t B, int64_t C,
                       int64_t H, int64_t W, int kh, int kw, int pad_north, int pad_south, int pad_west,
                       int pad_east, int explicit_padding, int stride_h, int stride_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_maxpool2d_fwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C >= 0 && H > 0 && W > 0, "b200_maxpool2d_fwd: bad input shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0, "b200_maxpool2d_fwd: bad kernel or stride");
  B200_REQUIRE(e, pad_north >= 0 && pad_south >= 0 && pad_west >= 0 && pad_east >= 0, "b200_maxpool2d_fwd: bad pad");
  B200_REQUIRE(e, H < (1LL << 30) && W < (1LL << 30), "b200_maxpool2d_fwd: image too large");
  const long long Ho = (H + pad_south + pad_north - (kh - 1) - 1) / stride_h + 1;
  const long long Wo = (W + pad_east + pad_west - (kw - 1) - 1) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_maxpool2d_fwd: window larger than the padded image");
  if (B * C == 0) return B200_OK;
  B200_REQUIRE(e, x && y, "b200_maxpool2d_fwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const int oh0 = explicit_padding ? pad_south : pad_north;
  const int ow0 = explicit_padding ? pad_east : pad_west;
  const long long total = B * C * Ho * Wo;
  if (dtype == B200_F32 && !mask && kh == 2 && kw == 2 && stride_h == 2 && stride_w == 2 && pad_north == 0 &&
      pad_south == 0 && pad_west == 0 && pad_east == 0 && W % 4 == 0 && (uintptr_t)x % 16 == 0 &&
      (uintptr_t)y % 8 == 0) {
    maxpool2x2_kernel<<<grid_for(e, total / 2), 256, 0, e->stream>>>((const float *)x, (float *)y, B * C, (int)H,
                                                                    (int)W, (int)Ho, (int)Wo);
    B200_CHECK_LAUNCH(e, "maxpool2x2_kernel");
    return B200_OK;
  }
  if (dtype == B200_F32 && !mask && kh == 2 && kw == 2 && stride_h == 2 && stride_w == 2 && pad_north == 0 &&
      pad_south == 0 && pad_west == 0 && pad_east == 0 && W % 2 == 0 && (uintptr_t)x % 8 == 0) {
    maxpool2x2_even_kernel<<<grid_for(e, total), 256, 0, e->stream>>>((const float *)x, (float *)y, B * C, (int)H,
                                                                     (int)W, (int)Ho, (int)Wo);
    B200_CHECK_LAUNCH(e, "maxpool2x2_even_kernel");
    return B200_OK;
  }
  if (dtype == B200_F32 && !mask && kh == 2 && kw == 2 && total < (1LL << 31) && B * C * H * W < (1LL << 32)) {
    maxpool2x2_any_kernel<<<grid_for(e, total), 256, 0, e->stream>>>((const float *)x, (float *)y, (uint32_t)(B * C),
                                                                    (int)H, (int)W, (int)Ho, (int)Wo, stride_h,
                                                                    stride_w, oh0, ow0);
    B200_CHECK_LAUNCH(e, "maxpool2x2_any_kernel");
    return B200_OK;
  }
  if (dtype == B200_F32)
    maxpool_kernel<float><<<grid_for(e, total), 256, 0, e->stream>>>((const float *)x, (float *)y, (long long *)mask,
                                                                    B * C, (int)H, (int)W, (int)Ho, (int)Wo, kh, kw,
                                                                    stride_h, stride_w, oh0, ow0);
  else
    maxpool_kernel<double><<<grid_for(e, total), 256, 0, e->stream>>>((const double *)x, (double *)y,
                                                                     (long long *)mask, B * C, (int)H, (int)W,
                                                                     (int)Ho, (int)Wo, kh, kw, stride_h, stride_w,
                                                                     oh0, ow0);
  B200_CHECK_LAUNCH(e, "maxpool_kernel");
  return B200_OK;
}

int b200_batchnorm_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t B, int64_t C, int64_t S, int training,
                       double momentum, double epsilon, void *running_mean, void *running_var, void *save_mean,
                       void *save_var) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_batchnorm_fwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && S > 0 && C < (1LL << 30), "b200_batchnorm_fwd: bad shape");
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, x && y && running_mean && running_var, "b200_batchnorm_fwd: null pointer");
  B200_REQUIRE(e, !training || (save_mean && save_var), "b200_batchnorm_fwd: training needs save_mean and save_var");
  B200_REQUIRE(e, !training || B * S > 1, "b200_batchnorm_fwd: training needs more than one value per channel");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32)
    return batchnorm_fwd_t<float>(e, (const float *)x, (float *)y, B, (int)C, S, training, momentum, epsilon,
                                  (float *)running_mean, (float *)running_var, (float *)save_mean, (float *)save_var);
  return batchnorm_fwd_t<double>(e, (const double *)x, (double *)y, B, (int)C, S, training, momentum, epsilon,
                                 (double *)running_mean, (double *)running_var, (double *)save_mean,
                                 (double *)save_var);
}

int b200_batchnorm_bwd(b200_engine *e, int dtype, const void *x, const void *dy, void *dx, int64_t B, int64_t C,
                       int64_t S, int training, double epsilon, const void *running_var, const void *save_mean,
                       const void *save_var) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_batchnorm_bwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && S > 0 && C < (1LL << 30), "b200_batchnorm_bwd: bad shape");
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, x && dy && dx && running_var && save_mean && save_var, "b200_batchnorm_bwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  if (dtype == B200_F32)
    return batchnorm_bwd_t<float>(e, (const float *)x, (const float *)dy, (float *)dx, B, (int)C, S, training, epsilon,
                                  (const float *)running_var, (const float *)save_mean, (const float *)save_var);
  return batchnorm_bwd_t<double>(e, (const double *)x, (const double *)dy, (double *)dx, B, (int)C, S, training, epsilon,
                                 (const double *)running_var, (const double *)save_mean, (const double *)save_var);
}

int b200_maxpool2d_bwd(b200_engine *e, int dtype, const void *dy, const int64_t *mask, void *dx, int64_t B, int64_t C,
                       int64_t H, int64_t W, int kh, int kw, int pad_north, int pad_south, int pad_west,
                       int pad_east, int explicit_padding, int stride_h, int stride_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_maxpool2d_bwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C >= 0 && H > 0 && W > 0, "b200_maxpool2d_bwd: bad input shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0, "b200_maxpool2d_bwd: bad kernel or stride");
  B200_REQUIRE(e, pad_north >= 0 && pad_south >= 0 && pad_west >= 0 && pad_east >= 0, "b200_maxpool2d_bwd: bad pad");
  B200_REQUIRE(e, H < (1LL << 30) && W < (1LL << 30), "b200_maxpool2d_bwd: image too large");
  const long long Ho = (H + pad_south + pad_north - (kh - 1) - 1) / stride_h + 1;
  const long long Wo = (W + pad_east + pad_west - (kw - 1) - 1) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_maxpool2d_bwd: window larger than the padded image");
  if (B * C == 0) return B200_OK;
  B200_REQUIRE(e, dy && mask && dx, "b200_maxpool2d_bwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const int oh0 = explicit_padding ? pad_south : pad_north;
  const int ow0 = explicit_padding ? pad_east : pad_west;
  const long long total = B * C * H * W;
  if (dtype == B200_F32 && kh == 2 && kw == 2 && stride_h == 2 && stride_w == 2 && pad_north == 0 && pad_south == 0 &&
      pad_west == 0 && pad_east == 0 && W % 4 == 0 && (uintptr_t)dx % 16 == 0 && (uintptr_t)dy % 8 == 0 &&
      (uintptr_t)mask % 16 == 0) {
    const long long work = B * C * ((H + 1) / 2) * (Wo / 2);
    maxpool2x2_bwd_kernel<<<grid_for(e, work), 256, 0, e->stream>>>((const float *)dy, (const long long *)mask,
                                                                   (float *)dx, B * C, (int)H, (int)W, (int)Ho,
                                                                   (int)Wo);
    B200_CHECK_LAUNCH(e, "maxpool2x2_bwd_kernel");
    return B200_OK;
  }
  if (dtype == B200_F32)
    maxpool_bwd_kernel<float><<<grid_for(e, total), 256, 0, e->stream>>>(
        (const float *)dy, (const long long *)mask, (float *)dx, B * C, (int)H, (int)W, (int)Ho, (int)Wo, kh, kw,
        stride_h, stride_w, oh0, ow0);
  else
    maxpool_bwd_kernel<double><<<grid_for(e, total), 256, 0, e->stream>>>(
        (const double *)dy, (const long long *)mask, (double *)dx, B * C, (int)H, (int)W, (int)Ho, (int)Wo, kh, kw,
        stride_h, stride_w, oh0, ow0);
  B200_CHECK_LAUNCH(e, "maxpool_bwd_kernel");
  return B200_OK;
}

int b200_col2im(b200_engine *e, int dtype, const void *col, void *im, int64_t B, int64_t C, int64_t H, int64_t W,
                int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_col2im: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && H > 0 && W > 0, "b200_col2im: bad image shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 &&
                      pad_w >= 0,
               "b200_col2im: bad kernel, stride, dilation or pad");
  B200_REQUIRE(e, C * (long long)kh * kw < (1LL << 30) && H < (1LL << 30) && W < (1LL << 30), "b200_col2im: too large");
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_col2im: kernel larger than the padded image");
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, col && im, "b200_col2im: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const long long total = B * C * H * W;
  // staged variant (stride 1 and no dilation along H, fewer pad rows than kernel rows): a ring of kh
  // col rows of Wo * (crs + 1) elements must fit in 96 KB of shared memory
  const size_t es = dtype_size(dtype);
  const size_t staged = (size_t)kh * Wo * (C * kh * kw + 1) * es;
  if (staged <= 96 * 1024 && stride_h == 1 && dil_h == 1 && pad_h < kh) {
    static std::atomic<int> attr_dev_mask{0};  // devices on which the attribute is set; engines on other threads share it
    if (!(attr_dev_mask & (1 << (e->device & 31)))) {
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows_kernel<float, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows_kernel<float, false>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows_kernel<double, true>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows_kernel<double, false>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      attr_dev_mask |= 1 << (e->device & 31);
    }
    const int blocks = (int)std::max<long long>(1, std::min<long long>(B, (long long)e->sm_count * 8));
    const bool unit_w = stride_w == 1 && dil_w == 1;
    if (dtype == B200_F32 && kh == 3 && kw == 3 && unit_w && (C * 9) % 4 == 0 && (uintptr_t)col % 16 == 0 && pad_h <= 2) {
      // bulk-copy ring: as many rows as fit beside the image copy, at most 8 (five rows ahead of the three in use)
      const size_t row_b = (size_t)Wo * C * 9 * 4, img_b = (size_t)C * H * W * 4;
      // taken where five ring rows and the image fit in half of an SM's shared memory (two blocks per SM:
      // with one, 1.9 TB/s against 3.1 at LeNet's conv1 shape); larger planes keep the register-staged kernel
      const size_t whole = std::min<size_t>(e->smem_optin, 227 * 1024) - 2048;
      const size_t room = whole / 2 - 1024;
      if (img_b + 5 * row_b <= room) {
        const int R = (int)std::min<size_t>(C2I_MAX_RING, (room - img_b) / row_b);
        const size_t smem = (size_t)R * row_b + img_b;
        static std::atomic<int> attrb_dev_mask{0};
        if (!(attrb_dev_mask & (1 << (e->device & 31)))) {
          B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_bulk_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)whole));
          attrb_dev_mask |= 1 << (e->device & 31);
        }
        const long long per_sm = std::max<long long>(1, (long long)(whole / (smem + 1024)));
        const int bblocks = (int)std::max<long long>(1, std::min<long long>(B, (long long)e->sm_count * per_sm));
        col2im_bulk_kernel<3, 3><<<bblocks, C2I_THREADS, smem, e->stream>>>((const float *)col, (float *)im, B, (int)C, (int)H,
                                                                    (int)W, (int)Ho, (int)Wo, pad_h, pad_w, R,
                                                                    e->d_flags + 2);
        B200_CHECK_LAUNCH(e, "col2im_bulk_kernel");
        e->flags_dirty = true;
        return B200_OK;
      }
    }
    const size_t staged4 = (size_t)(kh + 1) * Wo * (C * kh * kw + 1) * es;  // its ring holds one row more
    if (dtype == B200_F32 && (C * kh * kw) % 4 == 0 && Wo * C * kh * kw <= 8 * 256 * 4 && (uintptr_t)col % 16 == 0 &&
        staged4 <= 96 * 1024) {
      static int attr4_dev_mask = 0;
      if (!(attr4_dev_mask & (1 << (e->device & 31)))) {
        B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                96 * 1024));
        B200_CHECK_CUDA(e, cudaFuncSetAttribute(col2im_rows4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                96 * 1024));
        attr4_dev_mask |= 1 << (e->device & 31);
      }
      if (unit_w)
        col2im_rows4_kernel<true><<<blocks, 256, staged4, e->stream>>>((const float *)col, (float *)im, B, (int)C, (int)H,
                                                                     (int)W, (int)Ho, (int)Wo, kh, kw, pad_h, pad_w,
                                                                     stride_w, dil_w);
      else
        col2im_rows4_kernel<false><<<blocks, 256, staged4, e->stream>>>((const float *)col, (float *)im, B, (int)C,
                                                                      (int)H, (int)W, (int)Ho, (int)Wo, kh, kw, pad_h,
                                                                      pad_w, stride_w, dil_w);
      B200_CHECK_LAUNCH(e, "col2im_rows4_kernel");
      return B200_OK;
    }
#define B200_C2I(T, U)                                                                                          \
  col2im_rows_kernel<T, U><<<blocks, 256, staged, e->stream>>>((const T *)col, (T *)im, B, (int)C, (int)H, (int)W, \
                                                               (int)Ho, (int)Wo, kh, kw, pad_h, pad_w, stride_w, dil_w)
    if (dtype == B200_F32) {
      if (unit_w) B200_C2I(float, true); else B200_C2I(float, false);
    } else {
      if (unit_w) B200_C2I(double, true); else B200_C2I(double, false);
    }
#undef B200_C2I
    B200_CHECK_LAUNCH(e, "col2im_rows_kernel");
    return B200_OK;
  }
  if (dtype == B200_F32)
    col2im_kernel<float><<<grid_for(e, total), 256, 0, e->stream>>>((const float *)col, (float *)im, B, (int)C, (int)H,
                                                                   (int)W, (int)Ho, (int)Wo, kh, kw, pad_h, pad_w,
                                                                   stride_h, stride_w, dil_h, dil_w);
  else
    col2im_kernel<double><<<grid_for(e, total), 256, 0, e->stream>>>((const double *)col, (double *)im, B, (int)C,
                                                                    (int)H, (int)W, (int)Ho, (int)Wo, kh, kw, pad_h,
                                                                    pad_w, stride_h, stride_w, dil_h, dil_w);
  B200_CHECK_LAUNCH(e, "col2im_kernel");
  return B200_OK;
}

int b200_im2col(b200_engine *e, int dtype, const void *x, void *col, int64_t B, int64_t C, int64_t H, int64_t W,
                int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_im2col: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && H > 0 && W > 0, "b200_im2col: bad input shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 &&
                      pad_w >= 0,
               "b200_im2col: bad kernel, stride, dilation or pad");
  B200_REQUIRE(e, C * (long long)kh * kw < (1LL << 30) && H < (1LL << 30) && W < (1LL << 30), "b200_im2col: too large");
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_im2col: kernel larger than the padded image");
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, x && col, "b200_im2col: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  const int crs = (int)(C * kh * kw);
  const long long total = B * Ho * Wo * crs;
  if (dtype == B200_F32)
    im2col_kernel<float, false><<<grid_for(e, total), 256, 0, e->stream>>>(
        (const float *)x, (float *)col, nullptr, B, (int)C, (int)H, (int)W, (int)Ho, (int)Wo, kh, kw, pad_h, pad_w,
        stride_h, stride_w, dil_h, dil_w, crs);
  else
    im2col_kernel<double, false><<<grid_for(e, total), 256, 0, e->stream>>>(
        (const double *)x, (double *)col, nullptr, B, (int)C, (int)H, (int)W, (int)Ho, (int)Wo, kh, kw, pad_h, pad_w,
        stride_h, stride_w, dil_h, dil_w, crs);
  B200_CHECK_LAUNCH(e, "im2col_kernel");
  return B200_OK;
}

int b200_transpose(b200_engine *e, int elem_bytes, const void *x, void *y, int ndim, const int64_t *shape,
                   const int *perm) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, elem_bytes == 4 || elem_bytes == 8 || elem_bytes == 2, "b200_transpose: element size %d", elem_bytes);
  B200_REQUIRE(e, ndim >= 1 && ndim <= 8 && shape && perm, "b200_transpose: bad rank or null shape");
  long long in_stride[8], n = 1;
  bool seen[8] = {false, false, false, false, false, false, false, false};
  for (int d = ndim - 1; d >= 0; --d) {
    B200_REQUIRE(e, shape[d] >= 0, "b200_transpose: negative extent");
    in_stride[d] = n;
    n *= shape[d];
  }
  for (int d = 0; d < ndim; ++d) {
    B200_REQUIRE(e, perm[d] >= 0 && perm[d] < ndim && !seen[perm[d]], "b200_transpose: perm is not a permutation");
    seen[perm[d]] = true;
  }
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, x && y, "b200_transpose: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;

  // Collapse: drop axes of extent 1 and merge output axes that are adjacent in the input too.
  long long oshape[8], ostride[8];
  int m = 0;
  for (int d = 0; d < ndim; ++d) {
    const long long ext = shape[perm[d]], st = in_stride[perm[d]];
    if (ext == 1) continue;
    if (m > 0 && ostride[m - 1] == st * ext) {
      oshape[m - 1] *= ext;
      ostride[m - 1] = st;
    } else {
      oshape[m] = ext;
      ostride[m] = st;
      ++m;
    }
  }
  if (m <= 1) {  // the permutation moves nothing
    B200_CHECK_CUDA(e, cudaMemcpyAsync(y, x, (size_t)n * elem_bytes, cudaMemcpyDeviceToDevice, e->stream));
    return B200_OK;
  }
  // batched 2-D form: output (b, c, r) reading input (b, r, c)
  bool is2d = false;
  long long Bt = 1, R = 0, Cc = 0;
  if (m == 2 && ostride[1] == oshape[0] && ostride[0] == 1) {
    is2d = true;
    Cc = oshape[0];
    R = oshape[1];
  } else if (m == 3 && ostride[0] == oshape[1] * oshape[2] && ostride[2] == oshape[1] && ostride[1] == 1) {
    is2d = true;
    Bt = oshape[0];
    Cc = oshape[1];
    R = oshape[2];
  }
  if (is2d && Bt <= 65535 && (R + 31) / 32 <= 65535) {
    dim3 grid((unsigned)((Cc + 31) / 32), (unsigned)((R + 31) / 32), (unsigned)Bt);
    if (elem_bytes == 4)
      transpose2d_kernel<uint32_t><<<grid, 256, 0, e->stream>>>((const uint32_t *)x, (uint32_t *)y, R, Cc);
    else if (elem_bytes == 8)
      transpose2d_kernel<uint64_t><<<grid, 256, 0, e->stream>>>((const uint64_t *)x, (uint64_t *)y, R, Cc);
    else
      transpose2d_kernel<uint16_t><<<grid, 256, 0, e->stream>>>((const uint16_t *)x, (uint16_t *)y, R, Cc);
    B200_CHECK_LAUNCH(e, "transpose2d_kernel");
    return B200_OK;
  }
  TransposeDesc d;
  d.ndim = m;
  for (int k = 0; k < m; ++k) {
    d.out_shape[k] = oshape[k];
    d.in_stride_of_out_dim[k] = ostride[k];
  }
  if (elem_bytes == 4)
    transpose_kernel<uint32_t><<<grid_for(e, n), 256, 0, e->stream>>>((const uint32_t *)x, (uint32_t *)y, n, d);
  else if (elem_bytes == 8)
    transpose_kernel<uint64_t><<<grid_for(e, n), 256, 0, e->stream>>>((const uint64_t *)x, (uint64_t *)y, n, d);
  else
    transpose_kernel<uint16_t><<<grid_for(e, n), 256, 0, e->stream>>>((const uint16_t *)x, (uint16_t *)y, n, d);
  B200_CHECK_LAUNCH(e, "transpose_kernel");
  return B200_OK;
}

int b200_gather_axis(b200_engine *e, const void *x, const int64_t *idx, void *y, int64_t outer, int64_t n_rows,
                     int64_t n_idx, int64_t row_bytes) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, outer >= 0 && n_idx >= 0 && row_bytes >= 0 && n_rows >= 0, "b200_gather_axis: negative extent");
  if (outer == 0 || n_idx == 0 || row_bytes == 0) return B200_OK;
  B200_REQUIRE(e, x && idx && y, "b200_gather_axis: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  int *bad = e->d_flags + 3;
  B200_CHECK_CUDA(e, cudaMemsetAsync(bad, 0, sizeof(int), e->stream));
  const bool w16 = row_bytes % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0;
  const bool w4 = row_bytes % 4 == 0 && (uintptr_t)x % 4 == 0 && (uintptr_t)y % 4 == 0;
  if (w16) {
    const long long words = row_bytes / 16;
    gather_rows_kernel<uint4><<<grid_for(e, outer * n_idx * words), 256, 0, e->stream>>>(
        (const uint4 *)x, (const long long *)idx, (uint4 *)y, outer, n_idx, words, n_rows, bad);
  } else if (w4) {
    const long long words = row_bytes / 4;
    gather_rows_kernel<uint32_t><<<grid_for(e, outer * n_idx * words), 256, 0, e->stream>>>(
        (const uint32_t *)x, (const long long *)idx, (uint32_t *)y, outer, n_idx, words, n_rows, bad);
  } else {
    gather_rows_kernel<unsigned char><<<grid_for(e, outer * n_idx * row_bytes), 256, 0, e->stream>>>(
        (const unsigned char *)x, (const long long *)idx, (unsigned char *)y, outer, n_idx, row_bytes, n_rows, bad);
  }
  B200_CHECK_LAUNCH(e, "gather_rows_kernel");
  if (e->capturing) {
    // the check replays with the tape: the synchronising call after a replay reports it
    e->capture_has_gather = true;
    return B200_OK;
  }
  B200_CHECK_CUDA(e, cudaMemcpyAsync(e->h_flags + 3, bad, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
  rc = sync_stream_checked(e);
  if (rc != B200_OK) return rc;
  if (e->h_flags[3])
    return set_error(e, B200_ERR_INVALID, "b200_gather_axis: an index lies outside [0, %lld)", (long long)n_rows);
  return B200_OK;
}

int b200_gather_rows(b200_engine *e, const void *x, const int64_t *idx, void *y, int64_t n_idx, int64_t row_bytes,
                     int64_t n_rows) {
  return b200_gather_axis(e, x, idx, y, 1, n_rows, n_idx, row_bytes);
}

}  // extern "C"
