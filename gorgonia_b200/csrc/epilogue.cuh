// The fused tail of a matrix multiply or convolution: bias add and activation applied to the
// accumulator before it is stored, with exactly the arithmetic the unfused graph would do.
//   bias:  t = acc + bias[n] (per output column / conv channel) or bias[m] (per row)
//   act 1: Rectify as gorgonia builds it, t * (t >= 0 ? 1 : 0)            (nn.go:136-163)
//   act 2: LeakyRelu, t*(t>=0) + (t*(t<0))*alpha in that association        (nn.go:83-131)
#pragma once
#include "../../include/gorgonia_b200.h"

namespace b200 {

struct Epilogue {
  int bias_kind = 0;  // B200_BIAS_NONE / _COL / _ROW
  const void *bias = nullptr;
  int act = 0;        // B200_ACT_NONE / _RECTIFY / _LEAKY
  double alpha = 0.0;
  int accumulate = 0; // matrix product only: add the result to what the output holds
};

inline Epilogue make_epilogue(const b200_epilogue *ep) {
  Epilogue r;
  if (ep) {
    r.bias_kind = ep->bias_kind;
    r.bias = ep->bias;
    r.act = ep->act;
    r.alpha = ep->alpha;
    r.accumulate = ep->accumulate;
  }
  return r;
}

template <typename T>
__device__ __forceinline__ T epi_add(T a, T b);
template <>
__device__ __forceinline__ float epi_add<float>(float a, float b) { return __fadd_rn(a, b); }
template <>
__device__ __forceinline__ double epi_add<double>(double a, double b) { return __dadd_rn(a, b); }
template <typename T>
__device__ __forceinline__ T epi_mul(T a, T b);
template <>
__device__ __forceinline__ float epi_mul<float>(float a, float b) { return __fmul_rn(a, b); }
template <>
__device__ __forceinline__ double epi_mul<double>(double a, double b) { return __dmul_rn(a, b); }

template <typename T>
__device__ __forceinline__ T apply_act(T t, int act, T alpha) {
  if (act == B200_ACT_RECTIFY) return epi_mul<T>(t, t >= T(0) ? T(1) : T(0));
  if (act == B200_ACT_LEAKY) {
    const T pos = epi_mul<T>(t, t >= T(0) ? T(1) : T(0));
    const T neg = epi_mul<T>(epi_mul<T>(t, t < T(0) ? T(1) : T(0)), alpha);
    return epi_add<T>(pos, neg);
  }
  return t;
}

template <typename T>
__device__ __forceinline__ T apply_epilogue(T acc, const Epilogue &ep, long long m, long long n) {
  T t = acc;
  if (ep.bias_kind == B200_BIAS_COL)
    t = epi_add<T>(t, reinterpret_cast<const T *>(ep.bias)[n]);
  else if (ep.bias_kind == B200_BIAS_ROW)
    t = epi_add<T>(t, reinterpret_cast<const T *>(ep.bias)[m]);
  return apply_act<T>(t, ep.act, (T)ep.alpha);
}

// Stores the N accumulators one thread holds for N consecutive output channels of ONE position of
// an NCHW tensor: y[n * plane] = act(acc[n] + bias[n]). `bias` points at this column tile's first
// channel (shared or global memory, or null), `valid` is how many of the N channels exist. The
// activation switch sits outside the loops so that each loop body is straight-line code.
template <int N, int ACT, bool BIAS>
__device__ __forceinline__ void store_channels_variant(const float (&acc)[N], float *y, long long plane, int valid,
                                                       const float *bias, float alpha) {
  if (valid >= N) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float t = acc[j];
      if (BIAS) t = __fadd_rn(t, bias[j]);
      *y = apply_act<float>(t, ACT, alpha);
      y += plane;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      if (j < valid) {
        float t = acc[j];
        if (BIAS) t = __fadd_rn(t, bias[j]);
        *y = apply_act<float>(t, ACT, alpha);
      }
      y += plane;
    }
  }
}
template <int N>
__device__ __forceinline__ void store_channels(const float (&acc)[N], float *y, long long plane, int valid,
                                               const float *bias, int act, float alpha) {
  if (bias) {
    if (act == B200_ACT_NONE) store_channels_variant<N, B200_ACT_NONE, true>(acc, y, plane, valid, bias, alpha);
    else if (act == B200_ACT_RECTIFY) store_channels_variant<N, B200_ACT_RECTIFY, true>(acc, y, plane, valid, bias, alpha);
    else store_channels_variant<N, B200_ACT_LEAKY, true>(acc, y, plane, valid, bias, alpha);
  } else {
    if (act == B200_ACT_NONE) store_channels_variant<N, B200_ACT_NONE, false>(acc, y, plane, valid, bias, alpha);
    else if (act == B200_ACT_RECTIFY) store_channels_variant<N, B200_ACT_RECTIFY, false>(acc, y, plane, valid, bias, alpha);
    else store_channels_variant<N, B200_ACT_LEAKY, false>(acc, y, plane, valid, bias, alpha);
  }
}

// ---- the same store with a 2x2 / stride-2 max-pool folded in -----------------------------------
// maxPoolOp.do (op_nn.go:828-907) starts every window at -MaxFloat32 and replaces the running value
// only on a strict '>': a NaN or a -Inf never wins, and a window of nothing else yields -MaxFloat32.
// pool_candidate() maps a value to what it contributes under that rule; the plain maximum of the
// four candidates is then exactly the reference's result.
__device__ __forceinline__ float pool_candidate(float v) { return v > -3.402823466e+38f ? v : -3.402823466e+38f; }

// The four positions of a pooling window sit in lanes l, l^1 (next column) and l^8, l^9 (next
// row) of the warp. Every lane takes part in the exchange; lanes with `writer` set (the window's
// first position, inside the image) store to the pooled plane.
template <int N, int ACT, bool BIAS>
__device__ __forceinline__ void store_channels_pooled_variant(const float (&acc)[N], float *y, long long plane,
                                                              int valid, const float *bias, float alpha,
                                                              bool writer) {
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float t = acc[j];
    if (BIAS) t = __fadd_rn(t, bias[j]);
    float v = pool_candidate(apply_act<float>(t, ACT, alpha));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    if (writer && j < valid) *y = v;
    y += plane;
  }
}
template <int N>
__device__ __forceinline__ void store_channels_pooled(const float (&acc)[N], float *y, long long plane, int valid,
                                                      const float *bias, int act, float alpha, bool writer) {
  if (bias) {
    if (act == B200_ACT_NONE) store_channels_pooled_variant<N, B200_ACT_NONE, true>(acc, y, plane, valid, bias, alpha, writer);
    else if (act == B200_ACT_RECTIFY) store_channels_pooled_variant<N, B200_ACT_RECTIFY, true>(acc, y, plane, valid, bias, alpha, writer);
    else store_channels_pooled_variant<N, B200_ACT_LEAKY, true>(acc, y, plane, valid, bias, alpha, writer);
  } else {
    if (act == B200_ACT_NONE) store_channels_pooled_variant<N, B200_ACT_NONE, false>(acc, y, plane, valid, bias, alpha, writer);
    else if (act == B200_ACT_RECTIFY) store_channels_pooled_variant<N, B200_ACT_RECTIFY, false>(acc, y, plane, valid, bias, alpha, writer);
    else store_channels_pooled_variant<N, B200_ACT_LEAKY, false>(acc, y, plane, valid, bias, alpha, writer);
  }
}

// ---- the same stores, additionally (or only) in the form the NEXT convolution reads -------------
// The tensor-core convolutions read their input channels-innermost (NHWC), split into a TF32 head
// and the TF32 rounding of the remainder. A thread that holds N consecutive channels of one
// position can write exactly that, 16 bytes at a time, and spare the separate rewrite pass.
// nh / nl point at this position's channel n0 in the head / tail tensors; y (NCHW) may be null.
// POOL folds the 2x2 / stride-2 max-pool in as above. `valid` must be a multiple of 4.
__device__ __forceinline__ float epi_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}
// ---- the pooled store, the short way --------------------------------------------------------------
// Bias add, Rectify and LeakyRelu with a slope >= 0 never reverse the order of two numbers, so the
// maximum of the four activated values of a pooling window is the activated maximum of the four raw
// sums. The four lanes of a window therefore first exchange raw sums, halving twice what each lane
// keeps (lane bit 0 picks a half of the channels, lane bit 3 a half of that), and every lane then
// applies bias and activation to N/4 channels only and stores them, in NCHW (y) and / or in the split
// NHWC form (nh, nl). A quarter of the arithmetic and three eighths of the shuffles of the long way.
// The equivalence needs finite numbers (an infinite sum turns into NaN under the reference's
// x*(x>=0) forms and then never wins a window): if any result of the warp is not finite the function
// stores nothing and returns false, and the caller takes the long way, which follows the reference
// step by step. `inside`: this lane's pooling window lies in the image. The result is warp-uniform.
template <int N, int ACT, bool BIAS>
__device__ __forceinline__ bool store_channels_pool4_variant(const float (&acc)[N], float *y, long long plane,
                                                             int valid, const float *bias, float alpha, bool inside,
                                                             float *nh, float *nl) {
  static_assert(N % 16 == 0, "a lane keeps N / 4 channels, stored four at a time");
  const int lane = threadIdx.x & 31;
  const bool b0 = (lane & 1) != 0, b1 = (lane & 8) != 0;
  float h[N / 2];
#pragma unroll
  for (int j = 0; j < N / 2; ++j) {
    const float keep = b0 ? acc[j + N / 2] : acc[j];
    const float send = b0 ? acc[j] : acc[j + N / 2];
    h[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 1));
  }
  float q[N / 4];
#pragma unroll
  for (int j = 0; j < N / 4; ++j) {
    const float keep = b1 ? h[j + N / 4] : h[j];
    const float send = b1 ? h[j] : h[j + N / 4];
    q[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
  const int cb = (b0 ? N / 2 : 0) + (b1 ? N / 4 : 0);  // first channel this lane keeps
  bool bad = false;
#pragma unroll
  for (int j = 0; j < N / 4; ++j) {
    float t = q[j];
    if (BIAS) t = __fadd_rn(t, bias[cb + j]);
    t = apply_act<float>(t, ACT, alpha);
    q[j] = t;
    bad |= !(fabsf(t) <= 3.402823466e+38f);
  }
  if (__any_sync(0xffffffffu, bad)) return false;
  if (inside) {
    if (y) {
#pragma unroll
      for (int j = 0; j < N / 4; ++j)
        if (cb + j < valid) y[(long long)(cb + j) * plane] = q[j];
    }
    if (nh) {
#pragma unroll
      for (int j0 = 0; j0 < N / 4; j0 += 4) {
        if (cb + j0 < valid) {
          float hh[4], ll[4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            hh[jj] = epi_tf32(q[j0 + jj]);
            ll[jj] = epi_tf32(__fsub_rn(q[j0 + jj], hh[jj]));
          }
          *reinterpret_cast<float4 *>(nh + cb + j0) = make_float4(hh[0], hh[1], hh[2], hh[3]);
          *reinterpret_cast<float4 *>(nl + cb + j0) = make_float4(ll[0], ll[1], ll[2], ll[3]);
        }
      }
    }
  }
  return true;
}
template <int N>
__device__ __forceinline__ bool store_channels_pool4(const float (&acc)[N], float *y, long long plane, int valid,
                                                     const float *bias, int act, float alpha, bool inside, float *nh,
                                                     float *nl) {
  if (act == B200_ACT_LEAKY && !(alpha >= 0.f)) return false;  // a negative slope reverses the order of negatives
#define B200_POOL4_CASE(A, BI) return store_channels_pool4_variant<N, A, BI>(acc, y, plane, valid, bias, alpha, inside, nh, nl)
  if (bias) {
    if (act == B200_ACT_NONE) B200_POOL4_CASE(B200_ACT_NONE, true);
    else if (act == B200_ACT_RECTIFY) B200_POOL4_CASE(B200_ACT_RECTIFY, true);
    else B200_POOL4_CASE(B200_ACT_LEAKY, true);
  } else {
    if (act == B200_ACT_NONE) B200_POOL4_CASE(B200_ACT_NONE, false);
    else if (act == B200_ACT_RECTIFY) B200_POOL4_CASE(B200_ACT_RECTIFY, false);
    else B200_POOL4_CASE(B200_ACT_LEAKY, false);
  }
#undef B200_POOL4_CASE
}

template <int N, int ACT, bool BIAS, bool POOL>
__device__ __forceinline__ void store_channels_split_variant(const float (&acc)[N], float *y, long long plane,
                                                             int valid, const float *bias, float alpha, bool writer,
                                                             float *nh, float *nl) {
#pragma unroll
  for (int j0 = 0; j0 < N; j0 += 4) {
    float o[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      float t = acc[j0 + jj];
      if (BIAS) t = __fadd_rn(t, bias[j0 + jj]);
      float v = apply_act<float>(t, ACT, alpha);
      if (POOL) {
        v = pool_candidate(v);
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
      }
      o[jj] = v;
    }
    if (writer && j0 < valid) {
      if (y) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) y[(long long)(j0 + jj) * plane] = o[jj];
      }
      float h[4], l[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        h[jj] = epi_tf32(o[jj]);
        l[jj] = epi_tf32(__fsub_rn(o[jj], h[jj]));
      }
      *reinterpret_cast<float4 *>(nh + j0) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4 *>(nl + j0) = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
}
template <int N, bool POOL>
__device__ __forceinline__ void store_channels_split(const float (&acc)[N], float *y, long long plane, int valid,
                                                     const float *bias, int act, float alpha, bool writer, float *nh,
                                                     float *nl) {
#define B200_SPLIT_CASE(A, BI) store_channels_split_variant<N, A, BI, POOL>(acc, y, plane, valid, bias, alpha, writer, nh, nl)
  if (bias) {
    if (act == B200_ACT_NONE) B200_SPLIT_CASE(B200_ACT_NONE, true);
    else if (act == B200_ACT_RECTIFY) B200_SPLIT_CASE(B200_ACT_RECTIFY, true);
    else B200_SPLIT_CASE(B200_ACT_LEAKY, true);
  } else {
    if (act == B200_ACT_NONE) B200_SPLIT_CASE(B200_ACT_NONE, false);
    else if (act == B200_ACT_RECTIFY) B200_SPLIT_CASE(B200_ACT_RECTIFY, false);
    else B200_SPLIT_CASE(B200_ACT_LEAKY, false);
  }
#undef B200_SPLIT_CASE
}

}  // namespace b200
