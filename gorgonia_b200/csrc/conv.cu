// 2-D convolution, forward. Gives gorgonia's Conv2d (nn.go:211-305: Im2Col -> Reshape -> MatMul
// with the filters transposed -> Reshape -> Transpose(0,3,1,2)) one device entry point in place of
// five tape instructions, three of which are CPU-only in the reference.
//
// float32 runs as an implicit GEMM on the tensor cores (conv_tc.cu): the im2col matrix is never
// written to memory, the product lands in NCHW order, the filters are used untouched, bias and
// activation fuse into the store. float64 and problems under 64^3 multiply-adds take the
// CUDA-core path below: im2col of a chunk of images into arena scratch, then per image
//   Y_b (K x Ho*Wo) = Wf (K x C*kh*kw) . col_b^T,
// which also lands in NCHW order (column order of col: channel, kernel row, kernel column,
// op_nn.go:418-441).
#include <algorithm>

#include "engine.h"
#include "epilogue.cuh"

namespace b200 {

int conv2d_tc(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
              int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW, int Ho, int Wo,
              const Epilogue &ep);
int conv2d_tma(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
               int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW, int Ho, int Wo,
               const Epilogue &ep, const float *x_hi, const float *x_lo, float *y_hi, float *y_lo);
int conv2d_win(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H, int W, int K,
               int kh, int kw, int padH, int padW, int dH, int dW, int Ho, int Wo, const Epilogue &ep, bool pool2,
               const float *x_hi, const float *x_lo, float *y_hi, float *y_lo);
int conv_nhwc_split_into(b200_engine *e, const float *x, long long B, int C, int HW, float *hi, float *lo);
bool conv_win_eligible(const b200_engine *e, long long B, int C, int H, int W, int K, int kh, int kw, int padH,
                       int padW, int sH, int sW, int dH, int dW, int Ho, int Wo);
bool conv_tma_eligible(long long B, int C, int H, int W, int kh, int kw, int padH, int padW, int sH, int sW, int dH,
                       int dW);
int gemm_simt(b200_engine *e, int dtype, int transA, int transB, long long M, long long N, long long K,
              const void *A, long long lda, const void *B, long long ldb, void *C, long long ldc, long long batch,
              long long strideA, long long strideB, long long strideC, const Epilogue &ep);
// ---- direct convolution for the first layer of a network -------------------------------------
// When C*kh*kw <= 32 and K <= 32 (LeNet conv0: 1x3x3 -> 32; tiny-YOLO conv0: 3x3x3 -> 16) a pixel
// needs at most 32 inputs and the layer is bound by writing its output, not by arithmetic: one
// thread per output pixel keeps its taps in registers, the filters sit in shared memory laid out
// [q][K] so that all threads read the same address (a broadcast), and the K results of a pixel go
// out as K stores that are each contiguous across the warp (NCHW). fp32 FMA in q order.
template <int KP>  // filters padded to a multiple of 4, at most 32
__global__ void __launch_bounds__(256) conv_direct_small_kernel(const float *__restrict__ x,
                                                                const float *__restrict__ w, float *__restrict__ y,
                                                                long long Mtot, int C, int H, int W, int K, int Ho,
                                                                int Wo, int kh, int kw, int padH, int padW, int sH,
                                                                int sW, int dH, int dW, Epilogue ep,
                                                                const float *__restrict__ zero) {
  __shared__ __align__(16) float ws[32 * KP];
  __shared__ int q_off[32];  // offset of tap q relative to the pixel's window origin, inside one image
  __shared__ int q_tap[32];  // r*kw + s of tap q, or 32 for q past the end of the filter
  const int crs = C * kh * kw, hw = Ho * Wo, khw = kh * kw;
  for (int i = threadIdx.x; i < 32 * KP; i += blockDim.x) {
    const int q = i / KP, k = i % KP;
    ws[i] = (q < crs && k < K) ? w[k * crs + q] : 0.f;
  }
  if (threadIdx.x < 32) {
    const int q = threadIdx.x;
    const int c = q / khw, rs = q - c * khw, r = rs / kw, sx = rs - r * kw;
    q_off[q] = q < crs ? (c * H + r * dH) * W + sx * dW : 0;
    q_tap[q] = q < crs ? rs : 32;
  }
  __syncthreads();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x; m < Mtot; m += stride) {
    long long b;
    int pix;
    if (Mtot < (1LL << 31)) {
      const uint32_t mu = (uint32_t)m, bu = mu / (uint32_t)hw;
      b = bu;
      pix = (int)(mu - bu * (uint32_t)hw);
    } else {
      b = m / hw;
      pix = (int)(m - b * hw);
    }
    const int oh = pix / Wo, ow = pix - oh * Wo;
    const int ih0 = oh * sH - padH, iw0 = ow * sW - padW;
    // which taps of this pixel fall inside the image: one bit per (r, s); all of them for a
    // pixel whose whole window is inside, which is every pixel but the border ones
    uint32_t tap_mask = 0xffffffffu;
    if (ih0 < 0 || iw0 < 0 || ih0 + (kh - 1) * dH >= H || iw0 + (kw - 1) * dW >= W) {
      tap_mask = 0;
      for (int r = 0; r < kh; ++r)
        for (int sx = 0; sx < kw; ++sx) {
          const int ih = ih0 + r * dH, iw = iw0 + sx * dW;
          if ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) tap_mask |= 1u << (r * kw + sx);
        }
    }
    const float *xpix = x + b * (long long)C * H * W + (long long)ih0 * W + iw0;
    float v[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      v[q] = 0.f;
      if (q < crs) {  // the same for every thread: no divergence, and no loads for taps that do not exist
        const bool in = ((tap_mask >> q_tap[q]) & 1u) != 0;
        v[q] = __ldg(in ? xpix + q_off[q] : zero);  // a word that always holds 0.0f stands for padding
      }
    }
    float acc[KP];
#pragma unroll
    for (int k = 0; k < KP; ++k) acc[k] = 0.f;
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      if (q < crs) {
#pragma unroll
        for (int k4 = 0; k4 < KP; k4 += 4) {
          const float4 wv = *reinterpret_cast<const float4 *>(&ws[q * KP + k4]);
          acc[k4 + 0] = fmaf(v[q], wv.x, acc[k4 + 0]);
          acc[k4 + 1] = fmaf(v[q], wv.y, acc[k4 + 1]);
          acc[k4 + 2] = fmaf(v[q], wv.z, acc[k4 + 2]);
          acc[k4 + 3] = fmaf(v[q], wv.w, acc[k4 + 3]);
        }
      }
    }
    float *yb = y + (b * K) * (long long)hw + pix;
    if (ep.bias_kind == B200_BIAS_NONE && ep.act == B200_ACT_NONE) {
#pragma unroll
      for (int k = 0; k < KP; ++k)
        if (k < K) yb[(long long)k * hw] = acc[k];
    } else {
#pragma unroll
      for (int k = 0; k < KP; ++k)
        if (k < K) yb[(long long)k * hw] = apply_epilogue<float>(acc[k], ep, k, 0);
    }
  }
}

// Two fp32 fused multiply-adds in one instruction (fma.rn.f32x2 on 64-bit register pairs): the
// first-layer kernels are bound by instruction issue, and this halves their FMA count. Each lane of
// the pair rounds exactly as fmaf does.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma2(unsigned long long &d, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

// The same first-layer case at its usual geometry: 3x3 window, pad 1, stride 1, no dilation, at
// most 3 input channels, image width a multiple of 4. One thread computes FOUR neighbouring
// outputs of a row for 16 filters at a time: the 6 inputs of a window row (one aligned float4 and
// the two halo words) serve 3 taps x 4 outputs, a filter word read from shared memory (a broadcast)
// feeds 4 multiply-adds, and results leave as float4 stores. That is 4 multiply-adds per
// non-arithmetic instruction instead of the general kernel's one, which is what bounds a layer
// whose reduction is only 9 or 27 long. Bias and activation are compile-time variants.
template <int C, int ACT, bool BIAS>
__global__ void __launch_bounds__(256, 2) conv3x3_first_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                            float *__restrict__ y, const float *__restrict__ bias,
                                                            float alpha, long long groups, int H, int W, int K) {
  constexpr int Q = C * 9;
  __shared__ __align__(16) float ws[Q * 32];  // [q][k], zero for k >= K
  __shared__ float bs[32];
  for (int i = threadIdx.x; i < Q * 32; i += blockDim.x) {
    const int q = i >> 5, k = i & 31;
    ws[i] = k < K ? w[k * Q + q] : 0.f;
  }
  if (threadIdx.x < 32) bs[threadIdx.x] = (BIAS && threadIdx.x < K) ? bias[threadIdx.x] : 0.f;
  __syncthreads();
  const int Wg = W >> 2;
  const long long per_image = (long long)H * Wg;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const long long b = g / per_image;
    const int rem = (int)(g - b * per_image);
    const int oh = rem / Wg, og = rem - oh * Wg, ow = og << 2;
    const float *xb = x + b * (long long)C * H * W + ow;
    float *yb = y + (b * K) * (long long)H * W + (long long)oh * W + ow;
    for (int k0 = 0; k0 < K; k0 += 16) {
      unsigned long long accp[4][8];  // filter pairs (k, k+1) packed for fma.rn.f32x2
#pragma unroll
      for (int pz = 0; pz < 4; ++pz)
#pragma unroll
        for (int k = 0; k < 8; ++k) accp[pz][k] = 0ull;
#pragma unroll 1
      for (int c = 0; c < C; ++c) {  // not unrolled: one channel's 18 inputs in registers at a time
#pragma unroll
        for (int r = 0; r < 3; ++r) {
          const int ih = oh - 1 + r;
          float in[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if ((unsigned)ih < (unsigned)H) {
            const float *row = xb + ((long long)c * H + ih) * W;
            const float4 mid = __ldg(reinterpret_cast<const float4 *>(row));
            in[1] = mid.x; in[2] = mid.y; in[3] = mid.z; in[4] = mid.w;
            if (og > 0) in[0] = __ldg(row - 1);
            if (og < Wg - 1) in[5] = __ldg(row + 4);
          }
          unsigned long long in2[6];
#pragma unroll
          for (int i = 0; i < 6; ++i) in2[i] = pack2(in[i], in[i]);
#pragma unroll
          for (int sx = 0; sx < 3; ++sx) {
            const float *wq = &ws[(c * 9 + r * 3 + sx) * 32 + k0];
#pragma unroll
            for (int k4 = 0; k4 < 16; k4 += 4) {
              const float4 wv = *reinterpret_cast<const float4 *>(wq + k4);
              const unsigned long long w01 = pack2(wv.x, wv.y), w23 = pack2(wv.z, wv.w);
#pragma unroll
              for (int pz = 0; pz < 4; ++pz) {
                fma2(accp[pz][k4 / 2], in2[pz + sx], w01);
                fma2(accp[pz][k4 / 2 + 1], in2[pz + sx], w23);
              }
            }
          }
        }
      }
      float acc[4][16];
#pragma unroll
      for (int pz = 0; pz < 4; ++pz)
#pragma unroll
        for (int k = 0; k < 8; ++k) unpack2(accp[pz][k], acc[pz][2 * k], acc[pz][2 * k + 1]);
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        if (k0 + k < K) {
          float o[4];
#pragma unroll
          for (int pz = 0; pz < 4; ++pz) {
            float t = acc[pz][k];
            if (BIAS) t = __fadd_rn(t, bs[k0 + k]);
            o[pz] = apply_act<float>(t, ACT, alpha);
          }
          *reinterpret_cast<float4 *>(yb + (long long)(k0 + k) * H * W) = make_float4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
}

template <int C>
static int launch_conv3x3_first(b200_engine *e, const float *x, const float *w, float *y, long long B, int H, int W,
                                int K, const Epilogue &ep) {
  const long long groups = B * H * (W / 4);
  const int blocks = (int)std::max<long long>(1, std::min<long long>((groups + 255) / 256, (long long)e->sm_count * 16));
  const float *bias = (const float *)ep.bias;
  const float alpha = (float)ep.alpha;
#define B200_FIRST(ACT, BIAS) \
  conv3x3_first_kernel<C, ACT, BIAS><<<blocks, 256, 0, e->stream>>>(x, w, y, bias, alpha, groups, H, W, K)
  const bool hb = ep.bias_kind != B200_BIAS_NONE;
  if (ep.act == B200_ACT_NONE) { if (hb) B200_FIRST(B200_ACT_NONE, true); else B200_FIRST(B200_ACT_NONE, false); }
  else if (ep.act == B200_ACT_RECTIFY) { if (hb) B200_FIRST(B200_ACT_RECTIFY, true); else B200_FIRST(B200_ACT_RECTIFY, false); }
  else { if (hb) B200_FIRST(B200_ACT_LEAKY, true); else B200_FIRST(B200_ACT_LEAKY, false); }
#undef B200_FIRST
  B200_CHECK_LAUNCH(e, "conv3x3_first_kernel");
  return B200_OK;
}

// The first-layer kernel with the 2x2 / stride-2 max-pool that follows it folded in (H even): a
// thread computes a 2 x 4 block of outputs for 8 filters at a time from a 4 x 6 patch of inputs
// per channel and stores the two pooled values of each filter as one float2. The convolution output
// itself (four times the pooled bytes, and the largest tensor of the network) is never written.
template <int C, int ACT, bool BIAS>
__global__ void __launch_bounds__(256, 2) conv3x3_first_pool_kernel(const float *__restrict__ x,
                                                                    const float *__restrict__ w,
                                                                    float *__restrict__ y,
                                                                    const float *__restrict__ bias, float alpha,
                                                                    long long groups, int H, int W, int K,
                                                                    float *__restrict__ y_hi,
                                                                    float *__restrict__ y_lo) {
  constexpr int Q = C * 9;
  __shared__ __align__(16) float ws[Q * 32];  // [q][k], zero for k >= K
  __shared__ float bs[32];
  for (int i = threadIdx.x; i < Q * 32; i += blockDim.x) {
    const int q = i >> 5, k = i & 31;
    ws[i] = k < K ? w[k * Q + q] : 0.f;
  }
  if (threadIdx.x < 32) bs[threadIdx.x] = (BIAS && threadIdx.x < K) ? bias[threadIdx.x] : 0.f;
  __syncthreads();
  const int Wg = W >> 2, Hq = H >> 1, Wq = W >> 1;
  const long long per_image = (long long)Hq * Wg;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const long long b = g / per_image;
    const int rem = (int)(g - b * per_image);
    const int ph = rem / Wg, og = rem - ph * Wg, ow = og << 2, oh = ph << 1;
    const float *xb = x + b * (long long)C * H * W + ow;
    float *yb = y + (b * K) * (long long)Hq * Wq + (long long)ph * Wq + (ow >> 1);
    for (int k0 = 0; k0 < K; k0 += 8) {
      unsigned long long accp[2][4][4];  // filter pairs (k, k+1) packed
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int pz = 0; pz < 4; ++pz)
#pragma unroll
          for (int k = 0; k < 4; ++k) accp[rr][pz][k] = 0ull;
#pragma unroll 1
      for (int c = 0; c < C; ++c) {
        unsigned long long in2[4][6];  // every input duplicated into both lanes of a pair
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int ih = oh - 1 + r;
          float in[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if ((unsigned)ih < (unsigned)H) {
            const float *row = xb + ((long long)c * H + ih) * W;
            const float4 mid = __ldg(reinterpret_cast<const float4 *>(row));
            in[1] = mid.x; in[2] = mid.y; in[3] = mid.z; in[4] = mid.w;
            if (og > 0) in[0] = __ldg(row - 1);
            if (og < Wg - 1) in[5] = __ldg(row + 4);
          }
#pragma unroll
          for (int i = 0; i < 6; ++i) in2[r][i] = pack2(in[i], in[i]);
        }
#pragma unroll
        for (int r = 0; r < 3; ++r) {
#pragma unroll
          for (int sx = 0; sx < 3; ++sx) {
            const float *wq = &ws[(c * 9 + r * 3 + sx) * 32 + k0];
            const float4 w0 = *reinterpret_cast<const float4 *>(wq);
            const float4 w1 = *reinterpret_cast<const float4 *>(wq + 4);
            const unsigned long long wp[4] = {pack2(w0.x, w0.y), pack2(w0.z, w0.w), pack2(w1.x, w1.y),
                                              pack2(w1.z, w1.w)};
#pragma unroll
            for (int rr = 0; rr < 2; ++rr)
#pragma unroll
              for (int pz = 0; pz < 4; ++pz)
#pragma unroll
                for (int k = 0; k < 4; ++k) fma2(accp[rr][pz][k], in2[rr + r][pz + sx], wp[k]);
          }
        }
      }
      float acc[2][4][8];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int pz = 0; pz < 4; ++pz)
#pragma unroll
          for (int k = 0; k < 4; ++k) unpack2(accp[rr][pz][k], acc[rr][pz][2 * k], acc[rr][pz][2 * k + 1]);
      float pooled[2][8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float best = -3.402823466e+38f;
#pragma unroll
          for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              float t = acc[rr][2 * half + j][k];
              if (BIAS) t = __fadd_rn(t, bs[(k0 + k) & 31]);
              best = fmaxf(best, pool_candidate(apply_act<float>(t, ACT, alpha)));
            }
          pooled[half][k] = best;
        }
        if (y && k0 + k < K)
          *reinterpret_cast<float2 *>(yb + (long long)(k0 + k) * Hq * Wq) = make_float2(pooled[0][k], pooled[1][k]);
      }
      if (y_hi) {  // the same values as NHWC TF32 head / tail for the next convolution (K a multiple of 4)
        const long long pos = (b * Hq + ph) * (long long)Wq + (ow >> 1);
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int k4 = 0; k4 < 8; k4 += 4)
            if (k0 + k4 < K) {
              float h[4], l[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                h[j] = epi_tf32(pooled[half][k4 + j]);
                l[j] = epi_tf32(__fsub_rn(pooled[half][k4 + j], h[j]));
              }
              const long long at = (pos + half) * K + k0 + k4;
              *reinterpret_cast<float4 *>(y_hi + at) = make_float4(h[0], h[1], h[2], h[3]);
              *reinterpret_cast<float4 *>(y_lo + at) = make_float4(l[0], l[1], l[2], l[3]);
            }
      }
    }
  }
}

template <int C>
static int launch_conv3x3_first_pool(b200_engine *e, const float *x, const float *w, float *y, long long B, int H,
                                     int W, int K, const Epilogue &ep, float *y_hi = nullptr, float *y_lo = nullptr) {
  const long long groups = B * (H / 2) * (W / 4);
  const int blocks = (int)std::max<long long>(1, std::min<long long>((groups + 255) / 256, (long long)e->sm_count * 16));
  const float *bias = (const float *)ep.bias;
  const float alpha = (float)ep.alpha;
#define B200_FIRSTP(ACT, BIAS) \
  conv3x3_first_pool_kernel<C, ACT, BIAS><<<blocks, 256, 0, e->stream>>>(x, w, y, bias, alpha, groups, H, W, K, y_hi, \
                                                                         y_lo)
  const bool hb = ep.bias_kind != B200_BIAS_NONE;
  if (ep.act == B200_ACT_NONE) { if (hb) B200_FIRSTP(B200_ACT_NONE, true); else B200_FIRSTP(B200_ACT_NONE, false); }
  else if (ep.act == B200_ACT_RECTIFY) { if (hb) B200_FIRSTP(B200_ACT_RECTIFY, true); else B200_FIRSTP(B200_ACT_RECTIFY, false); }
  else { if (hb) B200_FIRSTP(B200_ACT_LEAKY, true); else B200_FIRSTP(B200_ACT_LEAKY, false); }
#undef B200_FIRSTP
  B200_CHECK_LAUNCH(e, "conv3x3_first_pool_kernel");
  return B200_OK;
}

// whether the specialised first-layer kernels take a convolution
static bool conv3x3_first_ok(const void *x, const void *y, long long C, long long W, int kh, int kw, int padH, int padW,
                             int sH, int sW, int dH, int dW) {
  return kh == 3 && kw == 3 && padH == 1 && padW == 1 && sH == 1 && sW == 1 && dH == 1 && dW == 1 && C <= 3 &&
         W % 4 == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0;
}

static int conv_direct_small(b200_engine *e, const float *x, const float *w, float *y, long long B, int C, int H,
                             int W, int K, int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW, int Ho,
                             int Wo, const Epilogue &ep) {
  if (conv3x3_first_ok(x, y, C, W, kh, kw, padH, padW, sH, sW, dH, dW)) {
    if (C == 1) return launch_conv3x3_first<1>(e, x, w, y, B, H, W, K, ep);
    if (C == 2) return launch_conv3x3_first<2>(e, x, w, y, B, H, W, K, ep);
    return launch_conv3x3_first<3>(e, x, w, y, B, H, W, K, ep);
  }
  const long long Mtot = B * Ho * Wo;
  const float *zero = reinterpret_cast<const float *>(e->d_flags + 8);  // zeroed at engine creation, never written
  const int blocks = (int)std::max<long long>(1, std::min<long long>((Mtot + 255) / 256, (long long)e->sm_count * 16));
#define B200_DIRECT(KP)                                                                                        \
  conv_direct_small_kernel<KP><<<blocks, 256, 0, e->stream>>>(x, w, y, Mtot, C, H, W, K, Ho, Wo, kh, kw, padH, padW, \
                                                             sH, sW, dH, dW, ep, zero)
  if (K <= 8) B200_DIRECT(8);
  else if (K <= 16) B200_DIRECT(16);
  else if (K <= 24) B200_DIRECT(24);
  else B200_DIRECT(32);
#undef B200_DIRECT
  B200_CHECK_LAUNCH(e, "conv_direct_small_kernel");
  return B200_OK;
}

// scratch budget for the col data of one chunk (head + tail together)
static const long long kColChunkBytes = 64LL << 20;

// Which kernel a convolution runs on (the B200_CONV_* values of the header).
static int conv_path(const b200_engine *e, int dtype, long long B, long long C, long long H, long long W, long long K,
                     int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                     long long Ho, long long Wo) {
  const long long crs = C * kh * kw, hw = Ho * Wo;
  if (dtype == B200_F32 && crs <= 32 && K <= 32 && C * H * W < (1LL << 31)) return B200_CONV_DIRECT;
  // the tensor-core kernels keep per-image offsets in 32 bits and pack tap offsets in 14 bits
  const bool tc = dtype == B200_F32 && B * K * hw * crs >= 64LL * 64 * 64 && B * hw < (1LL << 40) &&
                  C * H * W < (1LL << 31) && H < 16000 && W < 16000 && (long long)dil_h * kh < 16000 &&
                  (long long)dil_w * kw < 16000;
  if (!tc) return B200_CONV_SIMT;
  if (!(e->flags & B200_ENGINE_CONV_GATHER) &&
      conv_win_eligible(e, B, (int)C, (int)H, (int)W, (int)K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
                        (int)Ho, (int)Wo))
    return B200_CONV_TC_WINDOW;
  if (!(e->flags & B200_ENGINE_CONV_GATHER) &&
      conv_tma_eligible(B, (int)C, (int)H, (int)W, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w))
    return B200_CONV_TC_TMA;
  return B200_CONV_TC_GATHER;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_conv2d_fwd(b200_engine *e, int dtype, const void *x, const void *w, void *y, int64_t B, int64_t C,
                    int64_t H, int64_t W, int64_t K, int kh, int kw, int pad_h, int pad_w, int stride_h,
                    int stride_w, int dil_h, int dil_w, const b200_epilogue *epi) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_conv2d_fwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && H > 0 && W > 0 && K > 0, "b200_conv2d_fwd: bad shape");
  B200_REQUIRE(e, kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 &&
                      pad_w >= 0,
               "b200_conv2d_fwd: bad kernel, stride, dilation or pad");
  B200_REQUIRE(e, C * (long long)kh * kw < (1LL << 30) && H < (1LL << 30) && W < (1LL << 30),
               "b200_conv2d_fwd: too large");
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_conv2d_fwd: kernel larger than the padded image");
  if (epi) {
    B200_REQUIRE(e, epi->bias_kind == B200_BIAS_NONE || epi->bias_kind == B200_BIAS_ROW,
                 "b200_conv2d_fwd: the bias is one value per output channel (B200_BIAS_ROW)");
    B200_REQUIRE(e, epi->act >= 0 && epi->act <= 2, "b200_conv2d_fwd: bad activation");
    B200_REQUIRE(e, epi->bias_kind == 0 || epi->bias != nullptr, "b200_conv2d_fwd: bias is null");
    B200_REQUIRE(e, epi->accumulate == 0, "b200_conv2d_fwd: accumulate is a matrix-product option");
  }
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, x && w && y, "b200_conv2d_fwd: null pointer");
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  Epilogue ep = make_epilogue(epi);

  const long long crs = C * kh * kw, hw = Ho * Wo;
  const size_t es = dtype_size(dtype);
  const long long img_bytes = hw * crs * (long long)es;
  long long chunk = std::max<long long>(1, std::min<long long>(B, kColChunkBytes / std::max<long long>(1, img_bytes)));

  switch (conv_path(e, dtype, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, Ho, Wo)) {
    case B200_CONV_DIRECT:
      return conv_direct_small(e, (const float *)x, (const float *)w, (float *)y, B, (int)C, (int)H, (int)W, (int)K,
                               kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, (int)Ho, (int)Wo, ep);
    case B200_CONV_TC_TMA:
      return conv2d_tma(e, (const float *)x, (const float *)w, (float *)y, B, (int)C, (int)H, (int)W, (int)K, kh, kw,
                        pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, (int)Ho, (int)Wo, ep, nullptr, nullptr, nullptr,
                        nullptr);
    case B200_CONV_TC_WINDOW:
      return conv2d_win(e, (const float *)x, (const float *)w, (float *)y, B, (int)C, (int)H, (int)W, (int)K, kh, kw,
                        pad_h, pad_w, dil_h, dil_w, (int)Ho, (int)Wo, ep, false, nullptr, nullptr, nullptr, nullptr);
    case B200_CONV_TC_GATHER:
      return conv2d_tc(e, (const float *)x, (const float *)w, (float *)y, B, (int)C, (int)H, (int)W, (int)K, kh, kw,
                       pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, (int)Ho, (int)Wo, ep);
    default:
      break;
  }

  // CUDA-core path: plain im2col of a chunk, then Y_b = Wf . col_b^T per image
  void *colbuf = nullptr;
  rc = b200_get(e, chunk * hw * crs * (long long)es, &colbuf);
  if (rc != B200_OK) return rc;
  for (long long b0 = 0; rc == B200_OK && b0 < B; b0 += chunk) {
    const long long nb = std::min(chunk, B - b0);
    rc = b200_im2col(e, dtype, (const char *)x + b0 * C * H * W * es, colbuf, nb, C, H, W, kh, kw, pad_h, pad_w,
                     stride_h, stride_w, dil_h, dil_w);
    if (rc != B200_OK) break;
    rc = gemm_simt(e, dtype, 0, 1, K, hw, crs, w, crs, colbuf, crs, (char *)y + b0 * K * hw * es, hw, nb, 0, hw * crs,
                   K * hw, ep);
  }
  b200_put(e, colbuf, 0);
  return rc;
}

int b200_conv2d_maxpool_fwd(b200_engine *e, int dtype, const void *x, const void *w, void *y, int64_t B, int64_t C,
                            int64_t H, int64_t W, int64_t K, int kh, int kw, int pad_h, int pad_w, int stride_h,
                            int stride_w, int dil_h, int dil_w, const b200_epilogue *epi, int pool_h, int pool_w,
                            int pool_stride_h, int pool_stride_w) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_conv2d_maxpool_fwd: dtype %d not supported", dtype);
  B200_REQUIRE(e, B >= 0 && C > 0 && H > 0 && W > 0 && K > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0,
               "b200_conv2d_maxpool_fwd: bad convolution shape");
  B200_REQUIRE(e, pool_h > 0 && pool_w > 0 && pool_stride_h > 0 && pool_stride_w > 0,
               "b200_conv2d_maxpool_fwd: bad pooling window");
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  B200_REQUIRE(e, Ho >= pool_h && Wo >= pool_w, "b200_conv2d_maxpool_fwd: pooling window larger than the convolution output");
  if (B == 0) return B200_OK;
  B200_REQUIRE(e, x && w && y, "b200_conv2d_maxpool_fwd: null pointer");
  const bool pool2 = pool_h == 2 && pool_w == 2 && pool_stride_h == 2 && pool_stride_w == 2 && Ho % 2 == 0 &&
                     Wo % 2 == 0 && dtype == B200_F32;
  if (pool2) {
    const int path = conv_path(e, dtype, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, Ho, Wo);
    const bool first = path == B200_CONV_DIRECT &&
                       conv3x3_first_ok(x, y, C, W, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w);
    if (first || path == B200_CONV_TC_WINDOW) {
      if (epi) {
        B200_REQUIRE(e, epi->bias_kind == B200_BIAS_NONE || epi->bias_kind == B200_BIAS_ROW,
                     "b200_conv2d_maxpool_fwd: the bias is one value per output channel (B200_BIAS_ROW)");
        B200_REQUIRE(e, epi->act >= 0 && epi->act <= 2, "b200_conv2d_maxpool_fwd: bad activation");
        B200_REQUIRE(e, epi->bias_kind == 0 || epi->bias != nullptr, "b200_conv2d_maxpool_fwd: bias is null");
        B200_REQUIRE(e, epi->accumulate == 0, "b200_conv2d_maxpool_fwd: accumulate is a matrix-product option");
      }
      DeviceGuard g(e);
      int rc = flush_pending(e);
      if (rc != B200_OK) return rc;
      const Epilogue ep = make_epilogue(epi);
      if (path == B200_CONV_TC_WINDOW)
        return conv2d_win(e, (const float *)x, (const float *)w, (float *)y, B, (int)C, (int)H, (int)W, (int)K, kh, kw,
                          pad_h, pad_w, dil_h, dil_w, (int)Ho, (int)Wo, ep, true, nullptr, nullptr, nullptr, nullptr);
      if (C == 1) return launch_conv3x3_first_pool<1>(e, (const float *)x, (const float *)w, (float *)y, B, (int)H, (int)W, (int)K, ep);
      if (C == 2) return launch_conv3x3_first_pool<2>(e, (const float *)x, (const float *)w, (float *)y, B, (int)H, (int)W, (int)K, ep);
      return launch_conv3x3_first_pool<3>(e, (const float *)x, (const float *)w, (float *)y, B, (int)H, (int)W, (int)K, ep);
    }
  }
  // any other shape: the two operations one after the other, the convolution output in arena scratch
  void *tmp = nullptr;
  int rc = b200_get(e, B * K * Ho * Wo * (long long)dtype_size(dtype), &tmp);
  if (rc != B200_OK) return rc;
  rc = b200_conv2d_fwd(e, dtype, x, w, tmp, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, epi);
  if (rc == B200_OK)
    rc = b200_maxpool2d_fwd(e, dtype, tmp, y, nullptr, B, K, Ho, Wo, pool_h, pool_w, 0, 0, 0, 0, 0, pool_stride_h,
                            pool_stride_w);
  b200_put(e, tmp, 0);
  return rc;
}

int b200_conv2d_chain_fwd(b200_engine *e, const void *x, const void *x_hi, const void *x_lo, const void *w, void *y,
                          void *y_hi, void *y_lo, int64_t B, int64_t C, int64_t H, int64_t W, int64_t K, int kh, int kw,
                          int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                          const b200_epilogue *epi, int pool2) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, B >= 0 && C > 0 && H > 0 && W > 0 && K > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 &&
                      dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0,
               "b200_conv2d_chain_fwd: bad convolution shape");
  B200_REQUIRE(e, (x_hi == nullptr) == (x_lo == nullptr) && (y_hi == nullptr) == (y_lo == nullptr),
               "b200_conv2d_chain_fwd: a head needs its tail");
  B200_REQUIRE(e, x || x_hi, "b200_conv2d_chain_fwd: no input");
  B200_REQUIRE(e, y || y_hi, "b200_conv2d_chain_fwd: no output");
  B200_REQUIRE(e, !y_hi || K % 4 == 0, "b200_conv2d_chain_fwd: the split output needs K to be a multiple of 4");
  B200_REQUIRE(e, w, "b200_conv2d_chain_fwd: null filters");
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  B200_REQUIRE(e, Ho > 0 && Wo > 0, "b200_conv2d_chain_fwd: kernel larger than the padded image");
  B200_REQUIRE(e, !pool2 || (Ho >= 2 && Wo >= 2), "b200_conv2d_chain_fwd: nothing to pool");
  if (epi) {
    B200_REQUIRE(e, epi->bias_kind == B200_BIAS_NONE || epi->bias_kind == B200_BIAS_ROW,
                 "b200_conv2d_chain_fwd: the bias is one value per output channel (B200_BIAS_ROW)");
    B200_REQUIRE(e, epi->act >= 0 && epi->act <= 2, "b200_conv2d_chain_fwd: bad activation");
    B200_REQUIRE(e, epi->bias_kind == 0 || epi->bias != nullptr, "b200_conv2d_chain_fwd: bias is null");
    B200_REQUIRE(e, epi->accumulate == 0, "b200_conv2d_chain_fwd: accumulate is a matrix-product option");
  }
  if (B == 0) return B200_OK;
  const int path = conv_path(e, B200_F32, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, Ho, Wo);
  const bool even = Ho % 2 == 0 && Wo % 2 == 0;
  const float *xf = (const float *)x, *wf = (const float *)w;
  float *yf = (float *)y;
  if ((path == B200_CONV_TC_WINDOW && (!pool2 || even)) || (path == B200_CONV_TC_TMA && !pool2) ||
      (path == B200_CONV_DIRECT && pool2 && even && x &&
       conv3x3_first_ok(x, y, C, W, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w))) {
    DeviceGuard g(e);
    int rc = flush_pending(e);
    if (rc != B200_OK) return rc;
    const Epilogue ep = make_epilogue(epi);
    if (path == B200_CONV_TC_WINDOW)
      return conv2d_win(e, xf, wf, yf, B, (int)C, (int)H, (int)W, (int)K, kh, kw, pad_h, pad_w, dil_h, dil_w, (int)Ho,
                        (int)Wo, ep, pool2 != 0, (const float *)x_hi, (const float *)x_lo, (float *)y_hi,
                        (float *)y_lo);
    if (path == B200_CONV_TC_TMA)
      return conv2d_tma(e, xf, wf, yf, B, (int)C, (int)H, (int)W, (int)K, kh, kw, pad_h, pad_w, stride_h, stride_w,
                        dil_h, dil_w, (int)Ho, (int)Wo, ep, (const float *)x_hi, (const float *)x_lo, (float *)y_hi,
                        (float *)y_lo);
    if (C == 1) return launch_conv3x3_first_pool<1>(e, xf, wf, yf, B, (int)H, (int)W, (int)K, ep, (float *)y_hi, (float *)y_lo);
    if (C == 2) return launch_conv3x3_first_pool<2>(e, xf, wf, yf, B, (int)H, (int)W, (int)K, ep, (float *)y_hi, (float *)y_lo);
    return launch_conv3x3_first_pool<3>(e, xf, wf, yf, B, (int)H, (int)W, (int)K, ep, (float *)y_hi, (float *)y_lo);
  }
  // any other shape: the plain calls, then the rewrite pass; both need the tensors in NCHW
  if (!x)
    return set_error(e, B200_ERR_UNSUPPORTED,
                     "b200_conv2d_chain_fwd: this shape runs on a kernel that reads NCHW; pass x as well");
  const long long Hq = pool2 ? (Ho - 2) / 2 + 1 : Ho, Wq = pool2 ? (Wo - 2) / 2 + 1 : Wo;
  void *tmp = nullptr;
  int rc = B200_OK;
  if (!y) {
    rc = b200_get(e, B * K * Hq * Wq * 4, &tmp);
    if (rc != B200_OK) return rc;
    yf = (float *)tmp;
  }
  rc = pool2 ? b200_conv2d_maxpool_fwd(e, B200_F32, x, w, yf, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w,
                                       dil_h, dil_w, epi, 2, 2, 2, 2)
             : b200_conv2d_fwd(e, B200_F32, x, w, yf, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h,
                               dil_w, epi);
  if (rc == B200_OK && y_hi) {
    DeviceGuard g(e);
    rc = conv_nhwc_split_into(e, yf, B, (int)K, (int)(Hq * Wq), (float *)y_hi, (float *)y_lo);
  }
  if (tmp) b200_put(e, tmp, 0);
  return rc;
}

int b200_conv2d_path(b200_engine *e, int dtype, int64_t B, int64_t C, int64_t H, int64_t W, int64_t K, int kh, int kw,
                     int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w) {
  if (!e || B < 0 || C <= 0 || H <= 0 || W <= 0 || K <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0 ||
      dil_h <= 0 || dil_w <= 0 || pad_h < 0 || pad_w < 0)
    return -1;
  const long long Ho = (H + 2 * pad_h - (dil_h * (kh - 1) + 1)) / stride_h + 1;
  const long long Wo = (W + 2 * pad_w - (dil_w * (kw - 1) + 1)) / stride_w + 1;
  if (Ho <= 0 || Wo <= 0) return -1;
  return conv_path(e, dtype, B, C, H, W, K, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, Ho, Wo);
}

}  // extern "C"
