// Pointwise kernels, the deferred queue and its run-time fusion pass.
//
// Takes over Engine.Add…Pow / Lt…ElNe (+Scalar) (gorgonia cuda/arith.go:14-701,
// cuda/cmp.go:14-701), elemUnaryOp.CUDADo / elemBinOp.CUDADo (op_math_cuda.go:23-176) and the
// kernels of "cuda modules/src/elembinop.cu" and "elemunaryop.cu". The reference runs one
// thread per element, one launch (and often one device-to-device copy) per op, in place.
//
// Here one kernel evaluates a short program of pointwise instructions per pass over memory:
//   - each thread owns 16-byte chunks (4 floats / 2 doubles), grid-stride, 64-bit indices;
//   - all sources of a chunk are loaded first (independent 128-bit loads in flight), then the
//     program runs on registers, then the outputs are stored with 128-bit stores;
//   - the program is interpreted with warp-uniform branches: the instruction loop is unrolled,
//     instruction k writes register slot k (a compile-time index) and its operands are picked
//     by a switch whose selector is the same for every thread, so nothing diverges and no
//     value leaves the register file;
//   - multiplies and adds are never contracted into FMAs (the reference builds its kernels
//     with -fmad=false and the Go CPU engine does not fuse either).
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include <atomic>

#include "engine.h"
#include "ptx.cuh"

namespace b200 {

// ------------------------------------------------------------------------------------------
// device-side program
// ------------------------------------------------------------------------------------------

enum SrcMode : uint8_t {
  SRC_FULL = 0,     // element i reads src[i]
  SRC_ROWVEC = 1,   // div == 1 and mod % VEC == 0: chunk at i reads the chunk at i % mod
  SRC_GENERAL = 2,  // element i reads src[(i / div) % mod], one element at a time
  SRC_SCALAR = 3,   // every element reads src[0]
  SRC_CHUNK = 4     // div % VEC == 0: all elements of a chunk read the same src[(i / div) % mod]
};

struct PwDev {
  const void *src[B200_PW_MAX_SRC];
  void *out[B200_PW_MAX_OUT];
  long long n;
  long long src_div[B200_PW_MAX_SRC];
  long long src_mod[B200_PW_MAX_SRC];
  double imm[B200_PW_MAX_IMM];
  uint8_t n_instr, n_src, n_out, pad0;
  uint8_t src_mode[B200_PW_MAX_SRC];
  uint8_t op[B200_PW_MAX_INSTR];
  uint8_t ra[B200_PW_MAX_INSTR];  // operand selectors: [0,NS) sources, [16,24) immediates, [32,48) results
  uint8_t rb[B200_PW_MAX_INSTR];
  uint8_t out_ins[B200_PW_MAX_OUT];
  // ---- streaming kernel only: operands addressed in shared memory
  uint8_t n_full;                      // number of SRC_FULL sources (they travel through the ring)
  uint8_t n_file;                      // number of per-thread slots outside the ring
  uint8_t src_slot[B200_PW_MAX_SRC];   // SRC_FULL: index inside a ring stage; otherwise: file slot
  uint8_t ka[B200_PW_MAX_INSTR], xa[B200_PW_MAX_INSTR];  // operand kind (OperandKind) and index
  uint8_t kb[B200_PW_MAX_INSTR], xb[B200_PW_MAX_INSTR];
  uint8_t keep_slot[B200_PW_MAX_INSTR];  // file slot that keeps the result for later, or 0xFF
  uint8_t out_of[B200_PW_MAX_INSTR];     // output index this instruction's result is stored to, or 0xFF
};

enum OperandKind : uint8_t {
  K_ACC = 0,   // the result of the previous instruction, still in registers
  K_IMM = 1,   // immediate xa
  K_RING = 2,  // full-size source: slot xa of the current ring stage
  K_FILE = 3   // file slot xa: a broadcast source or a kept result
};

#define SEL_IMM 16
#define SEL_INS 32

template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
};
template <>
struct Vec<double> {
  static constexpr int N = 2;
};

// ---- scalar op semantics ---------------------------------------------------------------
// f32 thresholds of sigmoid/softplus follow elemunaryop.cu:166-189, f64 ones :83-105.

__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }

// Without the subnormal handling, for arguments and results known to be normal:
__device__ __forceinline__ float rcp_approx_ftz(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}
__device__ __forceinline__ float ex2_approx_ftz(float d) {  // relative error below 2^-22
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}

// 1 / (1 + e^-x) from t = e^-|x| <= 1: 1 / (1 + t) for x >= 0 and t / (1 + t) below, so that the
// reciprocal's argument lies in [1, 2] (the fast reciprocal, 1 ulp) and a result below the normal
// range comes out of the last multiplication as the subnormal it is. expf is within 2 ulp: 4 ulp in all.
__device__ __forceinline__ float sigmoid_(float x) {
  const float t = expf(-fabsf(x));
  const float r = rcp_approx_ftz(__fadd_rn(1.f, t));
  float s = x >= 0.f ? r : __fmul_rn(t, r);  // a NaN takes the second arm and stays a NaN
  if (x < -88.f) s = 0.f;
  if (x > 15.f) s = 1.f;
  return s;
}
__device__ __forceinline__ double sigmoid_(double x) {
  if (x < -709.0) return 0.0;
  if (x > 19.0) return 1.0;
  return 1.0 / (1.0 + exp(-x));
}
__device__ __forceinline__ float softplus_(float x) {
  if (x < -103.f) return 0.f;
  if (x > 14.f) return x;
  return log1pf(expf(x));
}
__device__ __forceinline__ double softplus_(double x) {
  if (x < -708.0) return 0.0;
  if (x > 16.0) return x;
  return log1p(exp(x));
}

// tanh in float32 without a branch: below 0.55 an odd polynomial (x + x z q(z), z = x^2, fitted to
// 7e-8 relative), above it 1 - 2 / (e^{2|x|} + 1), where the errors of the fast exponential and
// reciprocal are scaled by 2 / (e^{2|x|} + 1) <= 0.5 against a result >= 0.5: 3e-7 relative in all.
__device__ __forceinline__ float tanh_(float x) {
  const float ax = fabsf(x);
  const float z = __fmul_rn(x, x);
  float q = -0.006188455503433943f;
  q = __fmaf_rn(q, z, 0.021012423560023308f);
  q = __fmaf_rn(q, z, -0.05383826792240143f);
  q = __fmaf_rn(q, z, 0.1333245486021042f);
  q = __fmaf_rn(q, z, -0.3333331346511841f);
  const float small = __fmaf_rn(ax, __fmul_rn(z, q), ax);
  const float E = ex2_approx_ftz(__fmul_rn(ax, 2.8853900817779268f));  // e^{2|x|} >= 1; +inf from |x| > 44.4
  const float big = __fmaf_rn(-2.f, rcp_approx_ftz(__fadd_rn(E, 1.f)), 1.f);
  return copysignf(ax < 0.55f ? small : big, x);  // a NaN takes the second arm and stays a NaN; -0 stays -0
}
__device__ __forceinline__ double tanh_(double x) { return tanh(x); }

// x^y in float32 for positive normal x: 2^(y log2 x) with log2 x carried as a pair of floats.
//   x = 2^e m, m in [sqrt(1/2), sqrt 2); s = (m - 1) / (m + 1) as sh + sl (the rounding of m + 1 and
//   of the quotient are recovered with fused multiply-adds); log2 m = (2 / ln 2) (s + s^3/3 + ... +
//   s^11/11), the first term as an exact product pair, the rest (below 1 % of it) in plain floats;
//   L = e + log2 m as Lh + Ll; p = y L as ph + pl with the product's rounding error recovered;
//   result = ex2(ph - n + pl) 2^n, n = rint(ph).
// The pair carries log2 x to about 2^-30 relative, so the result is within 8e-8 of the exact power
// before the final ex2.approx (2^-22), for every |y log2 x| < 125. Anything else (x <= 0, subnormal,
// infinite or NaN; a result near the ends of the exponent range; y infinite or NaN) goes to powf.
__device__ __forceinline__ float pow_(float x, float y) {
  const int bits = __float_as_int(x);
  if ((unsigned)(bits - 0x00800000) < 0x7F000000u) {
    const int e = (bits - 0x3F3504F3) >> 23;
    const float m = __int_as_float(bits - (e << 23));
    const float ef = (float)e;
    const float f = __fsub_rn(m, 1.f);                 // exact
    const float d = __fadd_rn(m, 1.f);
    const float dl = __fsub_rn(m, __fsub_rn(d, 1.f));  // m + 1 == d + dl exactly
    const float r = rcp_approx_ftz(d);                 // d in [1.7, 2.42)
    const float sh = __fmul_rn(f, r);
    const float res = __fmaf_rn(-sh, dl, __fmaf_rn(-sh, d, f));
    const float sl = __fmul_rn(res, r);
    const float s2 = __fmul_rn(sh, sh);
    float Q = 1.f / 11.f;
    Q = __fmaf_rn(Q, s2, 1.f / 9.f);
    Q = __fmaf_rn(Q, s2, 1.f / 7.f);
    Q = __fmaf_rn(Q, s2, 1.f / 5.f);
    Q = __fmaf_rn(Q, s2, 1.f / 3.f);
    Q = __fmul_rn(Q, s2);
    constexpr float ch = 2.8853900817779268f;             // 2 / ln 2 rounded to float
    constexpr float cl = (float)(2.8853900817779268 - (double)ch);
    const float th = __fmul_rn(ch, sh);
    float tl = __fmaf_rn(ch, sh, -th);
    tl = __fmaf_rn(ch, sl, tl);
    tl = __fmaf_rn(cl, sh, tl);
    tl = __fmaf_rn(th, Q, tl);
    const float Lh = __fadd_rn(ef, th);
    const float Ll = __fadd_rn(__fadd_rn(__fsub_rn(ef, Lh), th), tl);
    const float ph = __fmul_rn(y, Lh);
    const float pl = __fmaf_rn(y, Ll, __fmaf_rn(y, Lh, -ph));
    if (fabsf(ph) < 125.f) {
      const float n = rintf(ph);
      const float v = ex2_approx_ftz(__fadd_rn(__fsub_rn(ph, n), pl));  // argument within [-0.5, 0.5]
      return __int_as_float(__float_as_int(v) + ((int)n << 23));
    }
  }
  return powf(x, y);
}
__device__ __forceinline__ double pow_(double x, double y) { return pow(x, y); }

#define PW_LOOP(expr)                 \
  _Pragma("unroll") for (int j = 0; j < V; ++j) { \
    const T x = a[j];                 \
    const T y = b[j];                 \
    (void)x; (void)y;                 \
    r[j] = (expr);                    \
  }                                   \
  break;

template <typename T, int V>
__device__ __forceinline__ void pw_apply(int op, const T (&a)[V], const T (&b)[V], T (&r)[V]) {
  const T one = T(1), zero = T(0);
  switch (op) {
    case B200_OP_ADD: PW_LOOP(add_rn(x, y))
    case B200_OP_SUB: PW_LOOP(sub_rn(x, y))
    case B200_OP_MUL: PW_LOOP(mul_rn(x, y))
    case B200_OP_DIV: PW_LOOP(x / y)
    case B200_OP_POW: PW_LOOP(pow_(x, y))
    case B200_OP_MOD: PW_LOOP(fmod(x, y))
    case B200_OP_LT: PW_LOOP(x < y ? one : zero)
    case B200_OP_GT: PW_LOOP(x > y ? one : zero)
    case B200_OP_LTE: PW_LOOP(x <= y ? one : zero)
    case B200_OP_GTE: PW_LOOP(x >= y ? one : zero)
    case B200_OP_EQ: PW_LOOP(x == y ? one : zero)
    case B200_OP_NE: PW_LOOP(x != y ? one : zero)
    case B200_OP_ABS: PW_LOOP(fabs(x))
    case B200_OP_SIGN: PW_LOOP(T((x > zero) - (x < zero)))
    case B200_OP_CEIL: PW_LOOP(ceil(x))
    case B200_OP_FLOOR: PW_LOOP(floor(x))
    case B200_OP_SIN: PW_LOOP(sin(x))
    case B200_OP_COS: PW_LOOP(cos(x))
    case B200_OP_EXP: PW_LOOP(exp(x))
    case B200_OP_LN: PW_LOOP(log(x))
    case B200_OP_LOG2: PW_LOOP(log2(x))
    case B200_OP_NEG: PW_LOOP(-x)
    case B200_OP_SQUARE: PW_LOOP(mul_rn(x, x))
    case B200_OP_SQRT: PW_LOOP(sqrt(x))
    case B200_OP_INV: PW_LOOP(one / x)
    case B200_OP_INVSQRT: PW_LOOP(one / sqrt(x))
    case B200_OP_CUBE: PW_LOOP(mul_rn(mul_rn(x, x), x))
    case B200_OP_TANH: PW_LOOP(tanh_(x))
    case B200_OP_SIGMOID: PW_LOOP(sigmoid_(x))
    case B200_OP_LOG1P: PW_LOOP(log1p(x))
    case B200_OP_EXPM1: PW_LOOP(expm1(x))
    case B200_OP_SOFTPLUS: PW_LOOP(softplus_(x))
    default:
      _Pragma("unroll") for (int j = 0; j < V; ++j) r[j] = zero;
      break;
  }
}

template <typename T, int V>
__device__ __forceinline__ void copyv(T (&d)[V], const T (&s)[V]) {
#pragma unroll
  for (int j = 0; j < V; ++j) d[j] = s[j];
}

// Picks operand `sel` for instruction K: a source, an immediate, or the result of an earlier
// instruction. `sel` is uniform across the grid, so the switches never diverge.
template <typename T, int V, int NS, int NI, int K>
__device__ __forceinline__ void fetch(T (&d)[V], int sel, const T (&S)[NS][V], const T (&R)[NI][V],
                                      const PwDev &p) {
  if (sel >= SEL_INS) {
    const int k = sel - SEL_INS;
    bool hit = false;
#pragma unroll
    for (int q = 0; q < K; ++q)
      if (k == q) {
        copyv(d, R[q]);
        hit = true;
      }
    if (!hit) {
#pragma unroll
      for (int j = 0; j < V; ++j) d[j] = T(0);
    }
  } else if (sel >= SEL_IMM) {
    const T v = (T)p.imm[sel - SEL_IMM];
#pragma unroll
    for (int j = 0; j < V; ++j) d[j] = v;
  } else {
    bool hit = false;
#pragma unroll
    for (int q = 0; q < NS; ++q)
      if (sel == q) {
        copyv(d, S[q]);
        hit = true;
      }
    if (!hit) {
#pragma unroll
      for (int j = 0; j < V; ++j) d[j] = T(0);
    }
  }
}

template <typename T, int V, int NS, int NI, int K>
struct Step {
  static __device__ __forceinline__ void run(const PwDev &p, const T (&S)[NS][V], T (&R)[NI][V]) {
    if (K < p.n_instr) {
      T a[V], b[V];
      fetch<T, V, NS, NI, K>(a, p.ra[K], S, R, p);
      fetch<T, V, NS, NI, K>(b, p.rb[K], S, R, p);
      pw_apply<T, V>(p.op[K], a, b, R[K]);
      Step<T, V, NS, NI, K + 1>::run(p, S, R);
    }
  }
};
template <typename T, int V, int NS, int NI>
struct Step<T, V, NS, NI, NI> {
  static __device__ __forceinline__ void run(const PwDev &, const T (&)[NS][V], T (&)[NI][V]) {}
};

template <typename T, int V>
__device__ __forceinline__ void load_chunk(T *d, const T *p, long long i, int valid) {
  if (V > 1 && valid == V) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p + i);
    memcpy(d, &raw, sizeof(uint4));
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) d[j] = j < valid ? p[i + j] : T(0);
  }
}

template <typename T, int V>
__device__ __forceinline__ void store_chunk(T *p, long long i, const T *s, int valid) {
  if (V > 1 && valid == V) {
    uint4 raw;
    memcpy(&raw, s, sizeof(uint4));
    *reinterpret_cast<uint4 *>(p + i) = raw;
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j)
      if (j < valid) p[i + j] = s[j];
  }
}

// V = elements per chunk (16 bytes' worth, or 1 when some pointer is not 16-byte aligned),
// NS / NI = compile-time capacity for sources and instructions.
template <typename T, int V, int NS, int NI>
__global__ void __launch_bounds__(256) pw_kernel(const __grid_constant__ PwDev p) {
  const long long n = p.n;
  const long long nchunks = (n + V - 1) / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nchunks; c += stride) {
    const long long i = c * V;
    const int valid = (n - i) >= V ? V : (int)(n - i);
    T S[NS][V];
    T R[NI][V];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (s < p.n_src) {
        const T *sp = reinterpret_cast<const T *>(p.src[s]);
        const int mode = p.src_mode[s];
        if (mode == SRC_FULL) {
          load_chunk<T, V>(S[s], sp, i, valid);
        } else if (mode == SRC_ROWVEC) {
          load_chunk<T, V>(S[s], sp, i % p.src_mod[s], V);
        } else if (mode == SRC_SCALAR) {
          const T v = sp[0];
#pragma unroll
          for (int j = 0; j < V; ++j) S[s][j] = v;
        } else if (mode == SRC_CHUNK) {
          const T v = sp[(i / p.src_div[s]) % p.src_mod[s]];
#pragma unroll
          for (int j = 0; j < V; ++j) S[s][j] = v;
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            S[s][j] = j < valid ? sp[((i + j) / p.src_div[s]) % p.src_mod[s]] : T(0);
        }
      }
    }
    Step<T, V, NS, NI, 0>::run(p, S, R);
#pragma unroll
    for (int o = 0; o < B200_PW_MAX_OUT; ++o) {
      if (o < p.n_out) {
        T v[V];
        fetch<T, V, NS, NI, NI>(v, SEL_INS + p.out_ins[o], S, R, p);
        store_chunk<T, V>(reinterpret_cast<T *>(p.out[o]), i, v, valid);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// The streaming kernel for large tensors.
//
// A pointwise kernel is bound by HBM, and two things keep a plain load/compute/store loop off
// that bound: every outstanding 16-byte load pins registers of a thread, so bytes in flight are
// tied to occupancy; and a register-resident interpreter pays for operand selection with long
// chains of predicated moves. This kernel removes both:
//   - full-size sources are staged through shared memory with bulk asynchronous copies (the TMA
//     engine, no tensor map) in a multi-stage ring. ONE thread per CTA queues whole tiles
//     (16 bytes x U x 512 threads per source) several stages ahead, so bytes in flight are set
//     by the ring depth, not by registers;
//   - operands are addressed, not selected: an operand is the previous result (registers), an
//     immediate, a ring slot or a per-thread "file" slot in shared memory (broadcast sources
//     and results needed again later). Fetching one is a uniform branch and a 16-byte shared
//     load, whatever the program length, so the instruction loop is a plain run-time loop.
// One persistent CTA of 512 threads per SM walks the tiles; results go straight from registers
// to global memory with 16-byte stores.
// ------------------------------------------------------------------------------------------
constexpr int PW_STREAM_THREADS = 512;
constexpr int PW_MAX_STAGES = 12;

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// One tile of the streaming kernel. INSIDE = the whole tile lies inside the tensor and is made
// of complete 16-byte chunks, which is every tile but possibly the last one: no bounds logic.
// ring_s / file_s: shared-memory addresses of this stage's ring slots and of the file slots,
// already offset by this thread's lane (tid * 16).
template <typename T, int V, int U, bool INSIDE>
__device__ __forceinline__ void pw_tile(const PwDev &p, uint32_t ring_s, uint32_t file_s, long long c_tile,
                                        int tid) {
  constexpr int W = U * V;
  constexpr uint32_t SLOT_BYTES = PW_STREAM_THREADS * U * 16;
  constexpr uint32_t USTRIDE = PW_STREAM_THREADS * 16;  // bytes between a thread's consecutive chunks
  int valid[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (INSIDE) {
      valid[u] = V;
    } else {
      const long long left = p.n - (c_tile + u * PW_STREAM_THREADS + tid) * V;
      valid[u] = left >= V ? V : (left > 0 ? (int)left : 0);
    }
  }
  // sources that are not full-size: fetch this thread's elements into its file slot
  if (p.n_file) {
    for (int s = 0; s < p.n_src; ++s) {
      const int mode = p.src_mode[s];
      if (mode == SRC_FULL) continue;
      const T *sp = reinterpret_cast<const T *>(p.src[s]);
      const uint32_t slot = file_s + p.src_slot[s] * SLOT_BYTES;
      if (mode == SRC_ROWVEC) {
        // the row offset of the tile start, once; the rest is 32-bit arithmetic
        const uint32_t mod = (uint32_t)p.src_mod[s];
        const uint32_t base = (uint32_t)((c_tile * V) % p.src_mod[s]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t off = (base + (uint32_t)(u * PW_STREAM_THREADS + tid) * V) % mod;
          uint4 raw = make_uint4(0, 0, 0, 0);
          if (valid[u] > 0) raw = *reinterpret_cast<const uint4 *>(sp + off);
          sts128(slot + u * USTRIDE, raw);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = (c_tile + u * PW_STREAM_THREADS + tid) * V;
          T v[V];
          if (mode == SRC_SCALAR) {
            const T x = sp[0];
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = x;
          } else if (mode == SRC_CHUNK) {
            const T x = valid[u] > 0 ? sp[(i / p.src_div[s]) % p.src_mod[s]] : T(0);
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = x;
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j)
              v[j] = j < valid[u] ? sp[((i + j) / p.src_div[s]) % p.src_mod[s]] : T(0);
          }
          uint4 raw;
          memcpy(&raw, v, sizeof raw);
          sts128(slot + u * USTRIDE, raw);
        }
      }
    }
  }
  if (!INSIDE) {
    // the ragged last chunk of the tensor is not part of the bulk copy: its owner patches it in
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (valid[u] > 0 && valid[u] < V) {
        for (int s = 0; s < p.n_src; ++s)
          if (p.src_mode[s] == SRC_FULL) {
            const T *sp = reinterpret_cast<const T *>(p.src[s]);
            T v[V];
#pragma unroll
            for (int j = 0; j < V; ++j)
              v[j] = j < valid[u] ? sp[(c_tile + u * PW_STREAM_THREADS + tid) * V + j] : T(0);
            uint4 raw;
            memcpy(&raw, v, sizeof raw);
            sts128(ring_s + p.src_slot[s] * SLOT_BYTES + u * USTRIDE, raw);
          }
      }
    }
  }

  T acc[W];
#pragma unroll
  for (int j = 0; j < W; ++j) acc[j] = T(0);
  const int n_instr = p.n_instr;
#pragma unroll 1
  for (int q = 0; q < n_instr; ++q) {
    T a[W], b[W];
    auto fetch_op = [&](T(&d)[W], int kind, int idx) {
      if (kind >= K_RING) {
        const uint32_t base = (kind == K_RING ? ring_s : file_s) + (uint32_t)idx * SLOT_BYTES;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint4 raw = lds128(base + u * USTRIDE);
          memcpy(&d[u * V], &raw, sizeof raw);
        }
      } else if (kind == K_ACC) {
#pragma unroll
        for (int j = 0; j < W; ++j) d[j] = acc[j];
      } else {
        const T x = (T)p.imm[idx];
#pragma unroll
        for (int j = 0; j < W; ++j) d[j] = x;
      }
    };
    const int op = p.op[q];
    fetch_op(a, p.ka[q], p.xa[q]);
    if (op < B200_OP_ABS) {
      fetch_op(b, p.kb[q], p.xb[q]);
    } else {
#pragma unroll
      for (int j = 0; j < W; ++j) b[j] = a[j];
    }
    pw_apply<T, W>(op, a, b, acc);
    const int keep = p.keep_slot[q];
    if (keep != 0xFF) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        uint4 raw;
        memcpy(&raw, &acc[u * V], sizeof raw);
        sts128(file_s + (uint32_t)keep * SLOT_BYTES + u * USTRIDE, raw);
      }
    }
    const int o = p.out_of[q];
    if (o != 0xFF) {
      unsigned char *op_ = reinterpret_cast<unsigned char *>(p.out[o]) + (c_tile + tid) * 16;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (INSIDE) {
          uint4 raw;
          memcpy(&raw, &acc[u * V], sizeof raw);
          *reinterpret_cast<uint4 *>(op_ + (size_t)u * USTRIDE) = raw;
        } else {
          store_chunk<T, V>(reinterpret_cast<T *>(p.out[o]), (c_tile + u * PW_STREAM_THREADS + tid) * V,
                            &acc[u * V], valid[u]);
        }
      }
    }
  }
}

// A full tile of a ONE-instruction program whose operands are ring slots or immediates (every
// plain engine call: Add, Mul, Exp, ...). The program was decoded once, before the tile loop; here
// there is nothing left but two shared loads per operand, the op and two stores.
template <typename T, int V, int U>
__device__ __forceinline__ void pw_tile_single(int op, bool a_imm, bool b_imm, bool unary, T imm_a, T imm_b,
                                               uint32_t a_s, uint32_t b_s, unsigned char *out_ptr) {
  constexpr int W = U * V;
  constexpr uint32_t USTRIDE = PW_STREAM_THREADS * 16;
  T a[W], b[W], r[W];
  if (a_imm) {
#pragma unroll
    for (int j = 0; j < W; ++j) a[j] = imm_a;
  } else {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint4 raw = lds128(a_s + u * USTRIDE);
      memcpy(&a[u * V], &raw, sizeof raw);
    }
  }
  if (unary) {
#pragma unroll
    for (int j = 0; j < W; ++j) b[j] = a[j];
  } else if (b_imm) {
#pragma unroll
    for (int j = 0; j < W; ++j) b[j] = imm_b;
  } else {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint4 raw = lds128(b_s + u * USTRIDE);
      memcpy(&b[u * V], &raw, sizeof raw);
    }
  }
  pw_apply<T, W>(op, a, b, r);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    uint4 raw;
    memcpy(&raw, &r[u * V], sizeof raw);
    *reinterpret_cast<uint4 *>(out_ptr + (size_t)u * USTRIDE) = raw;
  }
}

// SINGLE: the program is one instruction over ring slots and immediates (decided on the host), and
// full tiles take the lean path above. A separate instantiation, so that the general kernel's code
// and register allocation are not touched by it (measured: sharing one kernel cost the fused
// chains 5 %).
template <typename T, int V, int U, bool SINGLE>
__global__ void __launch_bounds__(PW_STREAM_THREADS, 2)
    pw_stream_kernel(const __grid_constant__ PwDev p, int stages, int *err_flag) {
  constexpr int TILE_CHUNKS = PW_STREAM_THREADS * U;
  constexpr int SLOT_BYTES = TILE_CHUNKS * 16;
  extern __shared__ __align__(128) unsigned char pw_smem[];
  __shared__ __align__(8) uint64_t full_bar[PW_MAX_STAGES];
  __shared__ int s_fail;

  const int tid = threadIdx.x;
  const long long nchunks_full = p.n / V;  // chunks that lie entirely inside the tensor
  const long long nchunks = (p.n + V - 1) / V;
  const long long ntiles = (nchunks + TILE_CHUNKS - 1) / TILE_CHUNKS;
  const long long my_count = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int nfull = p.n_full;
  const uint32_t stage_bytes = (uint32_t)nfull * SLOT_BYTES;
  const uint32_t smem_s = ptx::smem_addr(pw_smem);
  const uint32_t file_s = smem_s + (uint32_t)stages * stage_bytes + (uint32_t)tid * 16;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::fence_mbar_init();
    s_fail = 0;
  }
  __syncthreads();

  // thread 0: queue the copies of this CTA's k-th tile into ring stage `stage`
  auto issue = [&](long long k, int stage) {
    const long long c_begin = (blockIdx.x + k * (long long)gridDim.x) * TILE_CHUNKS;
    long long nfc = nchunks_full - c_begin;
    nfc = nfc < 0 ? 0 : (nfc > TILE_CHUNKS ? TILE_CHUNKS : nfc);
    const uint32_t bytes = (uint32_t)nfc * 16u;
    ptx::mbar_arrive_expect_tx(&full_bar[stage], bytes * (uint32_t)nfull);
    if (bytes) {
      for (int s = 0; s < p.n_src; ++s)
        if (p.src_mode[s] == SRC_FULL)
          ptx::bulk_g2s(pw_smem + (size_t)stage * stage_bytes + (size_t)p.src_slot[s] * SLOT_BYTES,
                        reinterpret_cast<const unsigned char *>(p.src[s]) + c_begin * 16, bytes,
                        &full_bar[stage]);
    }
  };
  if (tid == 0) {
    const long long pre = my_count < stages ? my_count : stages;
    for (long long k = 0; k < pre; ++k) issue(k, (int)k);
  }

  // decode once what a one-instruction program over ring slots and immediates needs per tile
  const int s_op = p.op[0];
  const bool s_unary = s_op >= B200_OP_ABS;
  const bool s_a_imm = p.ka[0] == K_IMM, s_b_imm = p.kb[0] == K_IMM;
  const T s_imm_a = (SINGLE && s_a_imm) ? (T)p.imm[p.xa[0]] : T(0);
  const T s_imm_b = (SINGLE && !s_unary && s_b_imm) ? (T)p.imm[p.xb[0]] : T(0);
  const uint32_t s_a_off = (uint32_t)p.xa[0] * SLOT_BYTES, s_b_off = (uint32_t)p.xb[0] * SLOT_BYTES;
  unsigned char *const s_out = reinterpret_cast<unsigned char *>(p.out[0]) + (size_t)tid * 16;

  long long k = 0;
  int stage = 0;
  uint32_t parity = 0;
  for (; k < my_count; ++k) {
    const long long c_tile = (blockIdx.x + k * (long long)gridDim.x) * TILE_CHUNKS;
    const uint32_t ring_s = smem_s + (uint32_t)stage * stage_bytes + (uint32_t)tid * 16;
    if (!ptx::mbar_wait(&full_bar[stage], parity)) s_fail = 1;
    if (SINGLE && c_tile + TILE_CHUNKS <= nchunks_full)
      pw_tile_single<T, V, U>(s_op, s_a_imm, s_b_imm, s_unary, s_imm_a, s_imm_b, ring_s + s_a_off, ring_s + s_b_off,
                              s_out + c_tile * 16);
    else if (c_tile + TILE_CHUNKS <= nchunks_full)
      pw_tile<T, V, U, true>(p, ring_s, file_s, c_tile, tid);
    else
      pw_tile<T, V, U, false>(p, ring_s, file_s, c_tile, tid);
    __syncthreads();    // every thread is done reading this ring stage
    if (s_fail) break;  // uniform: s_fail was written before the barrier
    if (tid == 0 && k + stages < my_count) issue(k + stages, stage);
    if (++stage == stages) {
      stage = 0;
      parity ^= 1;
    }
  }
  if (k < my_count) {
    // A wait ran out. Report it, then give copies that are still queued a last bounded chance to
    // land before this CTA's shared memory goes away.
    if (tid == 0) {
      atomicExch(err_flag, 1);
      const long long last = (k + stages < my_count ? k + stages : my_count);
      for (long long q = k; q < last; ++q)
        ptx::mbar_wait(&full_bar[q % stages], (uint32_t)((q / stages) & 1), 100000000ull);
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side: program checking, lowering, launch
// ------------------------------------------------------------------------------------------

static bool is_binary(int op) { return op >= B200_OP_ADD && op < B200_OP_BINARY_END; }
static bool is_unary(int op) { return op >= B200_OP_ABS && op < B200_OP_UNARY_END; }

static int lower_ref(b200_engine *e, const b200_pw_prog *prog, uint8_t ref, int k, uint8_t *sel) {
  const int kind = ref & 0xC0, idx = ref & 0x3F;
  if (kind == 0x00) {
    B200_REQUIRE(e, (uint32_t)idx < prog->n_src, "pointwise: instr %d reads source %d of %u", k, idx,
                 prog->n_src);
    *sel = (uint8_t)idx;
  } else if (kind == 0x40) {
    B200_REQUIRE(e, (uint32_t)idx < prog->n_imm, "pointwise: instr %d reads immediate %d of %u", k, idx,
                 prog->n_imm);
    *sel = (uint8_t)(SEL_IMM + idx);
  } else if (kind == 0x80) {
    B200_REQUIRE(e, idx < k, "pointwise: instr %d reads the result of instr %d", k, idx);
    *sel = (uint8_t)(SEL_INS + idx);
  } else {
    return set_error(e, B200_ERR_INVALID, "pointwise: bad operand reference 0x%02x", ref);
  }
  return B200_OK;
}

// one instruction over ring slots and immediates: every plain engine call (Add, Mul, Exp, ...)
static bool pw_is_single(const PwDev &d) {
  return d.n_instr == 1 && d.n_file == 0 && d.n_out == 1 && d.out_of[0] == 0 &&
         (d.ka[0] == K_RING || d.ka[0] == K_IMM) && (d.op[0] >= B200_OP_ABS || d.kb[0] == K_RING || d.kb[0] == K_IMM);
}

// One full-size source and one instruction (a unary op, a tensor-scalar op): tiles of four chunks per
// thread. With a single 16-byte stream per thread the per-tile work (barrier, ring bookkeeping, op
// dispatch) weighs twice as much per element as it does for two sources, and the ring has room.
template <typename T, int V>
static int launch_stream_wide(b200_engine *e, const PwDev &d, size_t budget, int stages) {
  constexpr int U = 4;
  constexpr int TILE_CHUNKS = PW_STREAM_THREADS * U;
  const long long nchunks = (d.n + V - 1) / V;
  const long long ntiles = (nchunks + TILE_CHUNKS - 1) / TILE_CHUNKS;
  const size_t smem = (size_t)stages * TILE_CHUNKS * 16;
  const int blocks = (int)std::min<long long>(ntiles, 2LL * e->sm_count);
  static std::atomic<int> attr_dev_mask{0};
  auto kern = pw_stream_kernel<T, V, U, true>;
  if (!(attr_dev_mask & (1 << (e->device & 31)))) {
    B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
    attr_dev_mask |= 1 << (e->device & 31);
  }
  kern<<<blocks, PW_STREAM_THREADS, smem, e->stream>>>(d, stages, e->d_flags + 2);
  B200_CHECK_LAUNCH(e, "pw_stream_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

template <typename T, int V, int U>
static int launch_stream_u(b200_engine *e, const PwDev &d, size_t budget, int stages) {
  constexpr int TILE_CHUNKS = PW_STREAM_THREADS * U;
  constexpr int SLOT_BYTES = TILE_CHUNKS * 16;
  const long long nchunks = (d.n + V - 1) / V;
  const long long ntiles = (nchunks + TILE_CHUNKS - 1) / TILE_CHUNKS;
  const size_t smem = ((size_t)stages * d.n_full + d.n_file) * SLOT_BYTES;
  const bool single = pw_is_single(d);
  const int blocks = (int)std::min<long long>(ntiles, 2LL * e->sm_count);  // two resident CTAs per SM
  static std::atomic<int> attr_dev_mask[2];  // per instantiation: devices on which the attribute is set
  if (single) {
    auto kern = pw_stream_kernel<T, V, U, true>;
    if (!(attr_dev_mask[1] & (1 << (e->device & 31)))) {
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
      attr_dev_mask[1] |= 1 << (e->device & 31);
    }
    kern<<<blocks, PW_STREAM_THREADS, smem, e->stream>>>(d, stages, e->d_flags + 2);
  } else {
    auto kern = pw_stream_kernel<T, V, U, false>;
    if (!(attr_dev_mask[0] & (1 << (e->device & 31)))) {
      B200_CHECK_CUDA(e, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
      attr_dev_mask[0] |= 1 << (e->device & 31);
    }
    kern<<<blocks, PW_STREAM_THREADS, smem, e->stream>>>(d, stages, e->d_flags + 2);
  }
  B200_CHECK_LAUNCH(e, "pw_stream_kernel");
  e->flags_dirty = true;
  return B200_OK;
}

// Picks the tile width and ring depth that fit shared memory; -1 if the program does not fit.
template <typename T, int V>
static int launch_stream(b200_engine *e, const PwDev &d) {
  // two CTAs share an SM: each gets just under half of its shared memory
  const size_t budget = std::min<size_t>(e->smem_optin > 4096 ? e->smem_optin - 4096 : 0, 220 * 1024) / 2;
  if (d.n_full == 1 && pw_is_single(d)) {
    const size_t slot = (size_t)PW_STREAM_THREADS * 4 * 16;
    const long long nchunks = (d.n + V - 1) / V;
    // wide tiles only where every CTA still gets several of them
    if (budget / slot >= 3 && nchunks >= 8LL * 2 * e->sm_count * PW_STREAM_THREADS * 4)
      return launch_stream_wide<T, V>(e, d, budget, (int)std::min<size_t>(budget / slot, PW_MAX_STAGES));
  }
  for (int u = 2; u >= 1; --u) {
    const size_t slot = (size_t)PW_STREAM_THREADS * u * 16;
    if (budget < d.n_file * slot) continue;
    int stages = (int)((budget - d.n_file * slot) / ((size_t)d.n_full * slot));
    stages = std::min(stages, PW_MAX_STAGES);
    if (stages >= (u == 2 ? 3 : 2))
      return u == 2 ? launch_stream_u<T, V, 2>(e, d, budget, stages) : launch_stream_u<T, V, 1>(e, d, budget, stages);
  }
  return -1;
}

template <typename T, int V>
static int launch_sized(b200_engine *e, const PwDev &d, int ns, int ni) {
  const long long nchunks = (d.n + V - 1) / V;
  // Large, 16-byte aligned tensors take the streaming kernel. Below ~2 tiles per SM the ring
  // never fills and the plain kernel, with its many small blocks, spreads the work better.
  if constexpr (V > 1) {
    if (d.n_full >= 1 && nchunks >= (long long)e->sm_count * PW_STREAM_THREADS * 2 * 2) {
      const int rc = launch_stream<T, V>(e, d);
      if (rc >= 0) return rc;
    }
  }
  const int threads = 256;
  long long want = (nchunks + threads - 1) / threads;
  long long cap = (long long)e->sm_count * 8;
  int blocks = (int)std::max<long long>(1, std::min(want, cap));
  if (ns <= 2 && ni <= 2)
    pw_kernel<T, V, 2, 2><<<blocks, threads, 0, e->stream>>>(d);
  else if (ns <= 3 && ni <= 4)
    pw_kernel<T, V, 3, 4><<<blocks, threads, 0, e->stream>>>(d);
  else
    pw_kernel<T, V, B200_PW_MAX_SRC, B200_PW_MAX_INSTR><<<blocks, threads, 0, e->stream>>>(d);
  B200_CHECK_LAUNCH(e, "pw_kernel");
  return B200_OK;
}

// Validates a program, lowers it to the device form and launches it (no queueing).
static int run_program(b200_engine *e, int dtype, const b200_pw_prog *prog, void *const *outs,
                       const void *const *srcs, int64_t n) {
  B200_REQUIRE(e, prog && outs && (srcs || prog->n_src == 0), "pointwise: null argument");
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "pointwise: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "pointwise: negative element count");
  B200_REQUIRE(e, prog->n_instr >= 1 && prog->n_instr <= B200_PW_MAX_INSTR, "pointwise: %u instructions",
               prog->n_instr);
  B200_REQUIRE(e, prog->n_src <= B200_PW_MAX_SRC, "pointwise: %u sources", prog->n_src);
  B200_REQUIRE(e, prog->n_imm <= B200_PW_MAX_IMM, "pointwise: %u immediates", prog->n_imm);
  B200_REQUIRE(e, prog->n_out >= 1 && prog->n_out <= B200_PW_MAX_OUT, "pointwise: %u outputs", prog->n_out);
  if (n == 0) return B200_OK;

  const size_t es = dtype_size(dtype);
  const int V = (int)(16 / es);
  PwDev d;
  memset(&d, 0, sizeof d);
  d.n = n;
  d.n_instr = (uint8_t)prog->n_instr;
  d.n_src = (uint8_t)prog->n_src;
  d.n_out = (uint8_t)prog->n_out;
  bool aligned = true;
  for (uint32_t s = 0; s < prog->n_src; ++s) {
    B200_REQUIRE(e, srcs[s] != nullptr, "pointwise: source %u is null", s);
    d.src[s] = srcs[s];
    const int64_t div = prog->src_div[s], mod = prog->src_mod[s];
    if (div == 0) {
      d.src_mode[s] = SRC_FULL;
      d.src_slot[s] = d.n_full++;
      if ((uintptr_t)srcs[s] % 16) aligned = false;
    } else {
      B200_REQUIRE(e, div > 0 && mod > 0, "pointwise: source %u has div %lld mod %lld", s, (long long)div,
                   (long long)mod);
      d.src_div[s] = div;
      d.src_mod[s] = mod;
      if (mod == 1)
        d.src_mode[s] = SRC_SCALAR;
      else if (div == 1 && mod % V == 0 && mod < (1LL << 30) && (uintptr_t)srcs[s] % 16 == 0)
        d.src_mode[s] = SRC_ROWVEC;
      else if (div % V == 0)
        d.src_mode[s] = SRC_CHUNK;
      else
        d.src_mode[s] = SRC_GENERAL;
    }
  }
  for (uint32_t k = 0; k < prog->n_imm; ++k) d.imm[k] = prog->imm[k];
  for (uint32_t k = 0; k < prog->n_instr; ++k) {
    const b200_pw_instr &in = prog->instr[k];
    B200_REQUIRE(e, is_binary(in.op) || is_unary(in.op), "pointwise: unknown op %d in instr %u", in.op, k);
    d.op[k] = in.op;
    int rc = lower_ref(e, prog, in.a, (int)k, &d.ra[k]);
    if (rc) return rc;
    if (is_binary(in.op)) {
      rc = lower_ref(e, prog, in.b, (int)k, &d.rb[k]);
      if (rc) return rc;
    } else {
      d.rb[k] = d.ra[k];
    }
  }
  for (uint32_t o = 0; o < prog->n_out; ++o) {
    B200_REQUIRE(e, outs[o] != nullptr, "pointwise: output %u is null", o);
    B200_REQUIRE(e, prog->out_instr[o] < prog->n_instr, "pointwise: output %u names instr %u", o,
                 prog->out_instr[o]);
    d.out[o] = outs[o];
    d.out_ins[o] = prog->out_instr[o];
    if ((uintptr_t)outs[o] % 16) aligned = false;
  }
  // operand addressing of the streaming kernel
  for (uint32_t s2 = 0; s2 < prog->n_src; ++s2)
    if (d.src_mode[s2] != SRC_FULL) d.src_slot[s2] = d.n_file++;
  {
    auto classify = [&](uint8_t sel, int k, uint8_t *kind, uint8_t *idx) {
      if (sel >= SEL_INS) {
        const int j = sel - SEL_INS;
        if (j == k - 1) {
          *kind = K_ACC;
          *idx = 0;
        } else {
          if (d.keep_slot[j] == 0xFF) d.keep_slot[j] = d.n_file++;
          *kind = K_FILE;
          *idx = d.keep_slot[j];
        }
      } else if (sel >= SEL_IMM) {
        *kind = K_IMM;
        *idx = (uint8_t)(sel - SEL_IMM);
      } else {
        *kind = d.src_mode[sel] == SRC_FULL ? K_RING : K_FILE;
        *idx = d.src_slot[sel];
      }
    };
    memset(d.keep_slot, 0xFF, sizeof d.keep_slot);
    memset(d.out_of, 0xFF, sizeof d.out_of);
    for (uint32_t k = 0; k < prog->n_instr; ++k) {
      classify(d.ra[k], (int)k, &d.ka[k], &d.xa[k]);
      classify(d.rb[k], (int)k, &d.kb[k], &d.xb[k]);
    }
    for (uint32_t o = 0; o < prog->n_out; ++o) {
      // one instruction may feed several outputs only through the plain kernel; the streaming
      // kernel stores each result once, which is all the engine's own planner ever asks for
      if (d.out_of[d.out_ins[o]] != 0xFF) d.n_full = 0;
      d.out_of[d.out_ins[o]] = (uint8_t)o;
    }
  }
  // a ROWVEC source needs the chunk grid itself aligned, which `aligned` guarantees
  if (!aligned)
    for (uint32_t s = 0; s < prog->n_src; ++s)
      if (d.src_mode[s] == SRC_ROWVEC || d.src_mode[s] == SRC_CHUNK) d.src_mode[s] = SRC_GENERAL;

  const int ns = (int)prog->n_src, ni = (int)prog->n_instr;
  if (dtype == B200_F32)
    return aligned ? launch_sized<float, 4>(e, d, ns, ni) : launch_sized<float, 1>(e, d, ns, ni);
  return aligned ? launch_sized<double, 2>(e, d, ns, ni) : launch_sized<double, 1>(e, d, ns, ni);
}

// ------------------------------------------------------------------------------------------
// the fusion pass: turns a list of queued calls into programs
// ------------------------------------------------------------------------------------------

struct Range {
  uint64_t lo, hi;  // [lo, hi)
};
static bool overlaps(const Range &x, const Range &y) { return x.lo < y.hi && y.lo < x.hi; }

struct FusedKernel {
  b200_pw_prog prog;
  const void *srcs[B200_PW_MAX_SRC];
  void *outs[B200_PW_MAX_OUT];
  int dtype;
  int64_t n;
  int first, last;  // calls [first, last)
  int loads, stores;
};

namespace {

struct Builder {
  // value currently held for a full-size buffer: a source slot or an instruction result
  struct Loc {
    uint64_t ptr;
    uint8_t ref;
    int writer;  // index of the call that last wrote it inside this kernel, -1 if only read
  };
  std::vector<Loc> locs;
  struct Bsrc {
    uint64_t ptr;
    int64_t div, mod;
    uint8_t ref;
  };
  std::vector<Bsrc> bsrcs;
  std::vector<Range> read_ranges, write_ranges, bcast_ranges;
  b200_pw_prog prog;
  const void *srcs[B200_PW_MAX_SRC];
  int dtype = 0;
  int64_t n = 0;
  int first = 0;

  void start(const b200_pw_call &c, int idx) {
    locs.clear();
    bsrcs.clear();
    read_ranges.clear();
    write_ranges.clear();
    bcast_ranges.clear();
    memset(&prog, 0, sizeof prog);
    dtype = c.dtype;
    n = c.n;
    first = idx;
  }
  Loc *find(uint64_t ptr) {
    for (auto &l : locs)
      if (l.ptr == ptr) return &l;
    return nullptr;
  }
  int count_outputs() const {
    int k = 0;
    for (auto &l : locs)
      if (l.writer >= 0) ++k;
    return k;
  }
};

// Number of new source slots / immediates / output buffers a call would add, and whether it
// can legally join the kernel under construction.
bool can_join(const Builder &b, const b200_pw_call &c, size_t es, int max_instr) {
  if (c.dtype != b.dtype || c.n != b.n) return false;
  if ((int)b.prog.n_instr + 1 > max_instr) return false;
  const uint64_t bytes = (uint64_t)c.n * es;
  int new_src = 0, new_imm = 0;
  auto full_operand = [&](uint64_t ptr) -> bool {
    for (auto &l : b.locs)
      if (l.ptr == ptr) return true;
    Range r{ptr, ptr + bytes};
    // a buffer that partly overlaps something this kernel writes would see half-updated data
    for (auto &w : b.write_ranges)
      if (overlaps(r, w)) return false;
    ++new_src;
    return true;
  };
  auto small_operand = [&](uint64_t ptr, int64_t div, int64_t mod) -> bool {
    for (auto &s : b.bsrcs)
      if (s.ptr == ptr && s.div == div && s.mod == mod) return true;
    Range r{ptr, ptr + (uint64_t)mod * es};
    for (auto &w : b.write_ranges)
      if (overlaps(r, w)) return false;
    ++new_src;
    return true;
  };
  const bool unary = c.form == 3;
  const bool a_is_tensor = unary || c.form == B200_VV || c.form == B200_VS;
  const bool b_is_tensor = !unary && (c.form == B200_VV || c.form == B200_SV);
  if (a_is_tensor) {
    if (c.bcast == 2) {
      if (!small_operand(c.a, c.bdiv, c.bmod)) return false;
    } else if (!full_operand(c.a))
      return false;
  }
  if (b_is_tensor && !(c.a == c.b && c.bcast == 0)) {
    if (c.bcast == 1) {
      if (!small_operand(c.b, c.bdiv, c.bmod)) return false;
    } else if (!full_operand(c.b))
      return false;
  }
  if (!unary && c.form != B200_VV) {
    if (c.scalar_ptr) {
      if (!small_operand(c.scalar_ptr, 1, 1)) return false;
    } else
      ++new_imm;
  }
  if ((int)b.prog.n_src + new_src > B200_PW_MAX_SRC) return false;
  if ((int)b.prog.n_imm + new_imm > B200_PW_MAX_IMM) return false;
  // destination: must be a buffer already tracked, or disjoint from everything touched so far
  bool known = false;
  for (auto &l : b.locs)
    if (l.ptr == c.dst) known = true;
  Range d{c.dst, c.dst + bytes};
  if (!known) {
    for (auto &r : b.read_ranges)
      if (overlaps(d, r)) return false;
    for (auto &w : b.write_ranges)
      if (overlaps(d, w)) return false;
    // operands of this very call that are new and partly overlap dst
    if (a_is_tensor && c.bcast != 2 && c.a != c.dst && overlaps(d, Range{c.a, c.a + bytes})) return false;
    if (b_is_tensor && c.bcast != 1 && c.b != c.dst && overlaps(d, Range{c.b, c.b + bytes})) return false;
  }
  for (auto &r : b.bcast_ranges)
    if (overlaps(d, r)) return false;
  if (c.bcast == 1 && overlaps(d, Range{c.b, c.b + (uint64_t)c.bmod * es})) return false;
  if (c.bcast == 2 && overlaps(d, Range{c.a, c.a + (uint64_t)c.bmod * es})) return false;
  if (c.scalar_ptr && overlaps(d, Range{c.scalar_ptr, c.scalar_ptr + es})) return false;
  int outs = b.count_outputs();
  bool dst_written = false;
  for (auto &l : b.locs)
    if (l.ptr == c.dst && l.writer >= 0) dst_written = true;
  if (!dst_written && outs + 1 > B200_PW_MAX_OUT) return false;
  return true;
}

void join(Builder &b, const b200_pw_call &c, int idx, size_t es) {
  const uint64_t bytes = (uint64_t)c.n * es;
  auto full_operand = [&](uint64_t ptr) -> uint8_t {
    if (auto *l = b.find(ptr)) return l->ref;
    const int k = (int)b.prog.n_src++;
    b.srcs[k] = (const void *)ptr;
    b.prog.src_div[k] = 0;
    b.prog.src_mod[k] = 0;
    b.locs.push_back({ptr, B200_REF_SRC(k), -1});
    b.read_ranges.push_back({ptr, ptr + bytes});
    return B200_REF_SRC(k);
  };
  auto small_operand = [&](uint64_t ptr, int64_t div, int64_t mod) -> uint8_t {
    for (auto &s : b.bsrcs)
      if (s.ptr == ptr && s.div == div && s.mod == mod) return s.ref;
    const int k = (int)b.prog.n_src++;
    b.srcs[k] = (const void *)ptr;
    b.prog.src_div[k] = div;
    b.prog.src_mod[k] = mod;
    b.bsrcs.push_back({ptr, div, mod, B200_REF_SRC(k)});
    b.bcast_ranges.push_back({ptr, ptr + (uint64_t)mod * es});
    return B200_REF_SRC(k);
  };
  auto scalar_operand = [&]() -> uint8_t {
    if (c.scalar_ptr) return small_operand(c.scalar_ptr, 1, 1);
    const int k = (int)b.prog.n_imm++;
    b.prog.imm[k] = c.scalar;
    return B200_REF_IMM(k);
  };
  const bool unary = c.form == 3;
  uint8_t ra = 0, rb = 0;
  if (unary) {
    ra = c.bcast == 2 ? small_operand(c.a, c.bdiv, c.bmod) : full_operand(c.a);
    rb = ra;
  } else {
    if (c.form == B200_SV)
      ra = scalar_operand();
    else
      ra = c.bcast == 2 ? small_operand(c.a, c.bdiv, c.bmod) : full_operand(c.a);
    if (c.form == B200_VS)
      rb = scalar_operand();
    else
      rb = c.bcast == 1 ? small_operand(c.b, c.bdiv, c.bmod) : full_operand(c.b);
  }
  const int k = (int)b.prog.n_instr++;
  b.prog.instr[k].op = (uint8_t)c.op;
  b.prog.instr[k].a = ra;
  b.prog.instr[k].b = rb;
  if (auto *l = b.find(c.dst)) {
    l->ref = B200_REF_INS(k);
    l->writer = idx;
  } else {
    b.locs.push_back({c.dst, B200_REF_INS(k), idx});
  }
  b.write_ranges.push_back({c.dst, c.dst + bytes});
}

// Closes the kernel: every buffer written becomes an output unless it was released before
// any call outside this kernel could have read it.
void finish(Builder &b, int end, const int *released_at, FusedKernel *fk) {
  fk->dtype = b.dtype;
  fk->n = b.n;
  fk->first = b.first;
  fk->last = end;
  fk->loads = 0;
  for (auto &l : b.locs) (void)l;
  for (uint32_t s = 0; s < b.prog.n_src; ++s)
    if (b.prog.src_div[s] == 0) fk->loads++;
  int nout = 0;
  int last_out_candidate = -1;
  for (size_t i = 0; i < b.locs.size(); ++i) {
    auto &l = b.locs[i];
    if (l.writer < 0) continue;
    last_out_candidate = (int)i;
    const int rel = released_at ? released_at[l.writer] : -1;
    const bool dead = rel >= 0 && rel > l.writer && rel <= end;
    if (dead) continue;
    fk->outs[nout] = (void *)l.ptr;
    b.prog.out_instr[nout] = (uint8_t)(l.ref & 0x3F);
    ++nout;
  }
  if (nout == 0 && last_out_candidate >= 0) {
    // every result was released unread: nothing observable remains, but keep one store so
    // the program stays well-formed (the caller released that memory; writing it is harmless)
    auto &l = b.locs[last_out_candidate];
    fk->outs[0] = (void *)l.ptr;
    b.prog.out_instr[0] = (uint8_t)(l.ref & 0x3F);
    nout = 1;
  }
  b.prog.n_out = (uint32_t)nout;
  fk->stores = nout;
  fk->prog = b.prog;
  for (int s = 0; s < B200_PW_MAX_SRC; ++s) fk->srcs[s] = b.srcs[s];
}

}  // namespace

// The fused kernels never exceed the program capacity of the largest kernel instantiation.
static const int kMaxFusedInstr = B200_PW_MAX_INSTR;

static void plan(const b200_pw_call *calls, int n_calls, const int *released_at,
                 std::vector<FusedKernel> *out) {
  out->clear();
  Builder b;
  int i = 0;
  while (i < n_calls) {
    const size_t es = dtype_size(calls[i].dtype);
    b.start(calls[i], i);
    join(b, calls[i], i, es);
    int j = i + 1;
    while (j < n_calls && can_join(b, calls[j], es, kMaxFusedInstr)) {
      join(b, calls[j], j, es);
      ++j;
    }
    FusedKernel fk;
    memset(&fk, 0, sizeof fk);
    finish(b, j, released_at, &fk);
    out->push_back(fk);
    i = j;
  }
}

static void released_positions(b200_engine *e, std::vector<int> *rel) {
  rel->assign(e->pending.size(), -1);
  // e->dead holds (pointer, queue length at release) pairs flattened as two entries
  for (size_t k = 0; k + 1 < e->dead.size(); k += 2) {
    const uint64_t ptr = (uint64_t)e->dead[k];
    const int pos = (int)(uintptr_t)e->dead[k + 1];
    // the release concerns the last write to ptr queued before `pos`
    for (int c = std::min<int>(pos, (int)e->pending.size()) - 1; c >= 0; --c)
      if (e->pending[c].dst == ptr) {
        (*rel)[c] = pos;
        break;
      }
  }
}

void note_put(b200_engine *e, void *ptr) {
  if (e->pending.empty()) return;
  for (auto &c : e->pending)
    if (c.dst == (uint64_t)ptr) {
      e->dead.push_back(ptr);
      e->dead.push_back((void *)(uintptr_t)e->pending.size());
      return;
    }
}

int plan_pending(b200_engine *e, int *n_kernels) {
  std::vector<int> rel;
  released_positions(e, &rel);
  std::vector<FusedKernel> ks;
  plan(e->pending.data(), (int)e->pending.size(), rel.data(), &ks);
  *n_kernels = (int)ks.size();
  return B200_OK;
}

int flush_pending(b200_engine *e) {
  if (e->pending.empty()) {
    e->dead.clear();
    return B200_OK;
  }
  std::vector<int> rel;
  released_positions(e, &rel);
  std::vector<FusedKernel> ks;
  plan(e->pending.data(), (int)e->pending.size(), rel.data(), &ks);
  e->pending.clear();
  e->dead.clear();
  for (auto &k : ks) {
    int rc = run_program(e, k.dtype, &k.prog, k.outs, k.srcs, k.n);
    if (rc != B200_OK) return rc;
  }
  return B200_OK;
}

static int enqueue(b200_engine *e, const b200_pw_call &c) {
  e->pending.push_back(c);
  if (e->flags & B200_ENGINE_NO_DEFER) return flush_pending(e);
  // keep the queue bounded: a tape that never flushes would otherwise grow without limit
  if (e->pending.size() >= 4096) return flush_pending(e);
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_binary(b200_engine *e, int op, int dtype, int form, void *dst, const void *a, const void *b,
                double scalar, int scalar_on_device, int64_t n) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, is_binary(op), "b200_binary: %d is not a binary op", op);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_binary: dtype %d not supported", dtype);
  B200_REQUIRE(e, form == B200_VV || form == B200_VS || form == B200_SV, "b200_binary: bad form %d", form);
  B200_REQUIRE(e, n >= 0, "b200_binary: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, dst != nullptr, "b200_binary: dst is null");
  b200_pw_call c;
  memset(&c, 0, sizeof c);
  c.op = op;
  c.dtype = dtype;
  c.form = form;
  c.dst = (uint64_t)dst;
  c.n = n;
  c.scalar = scalar;
  if (form == B200_VV) {
    B200_REQUIRE(e, a && b, "b200_binary: null operand");
    c.a = (uint64_t)a;
    c.b = (uint64_t)b;
  } else if (form == B200_VS) {
    B200_REQUIRE(e, a != nullptr, "b200_binary: null operand");
    c.a = (uint64_t)a;
    if (scalar_on_device) {
      B200_REQUIRE(e, b != nullptr, "b200_binary: device scalar is null");
      c.scalar_ptr = (uint64_t)b;
    }
  } else {
    B200_REQUIRE(e, b != nullptr, "b200_binary: null operand");
    c.b = (uint64_t)b;
    if (scalar_on_device) {
      B200_REQUIRE(e, a != nullptr, "b200_binary: device scalar is null");
      c.scalar_ptr = (uint64_t)a;
    }
  }
  DeviceGuard g(e);
  return enqueue(e, c);
}

// ExternalOp.Do in Incr mode (execution.go:113-127): CUDADo into a temporary, then an unsafe add of
// the temporary into op.Incr. Queued as exactly those two calls; the temporary is handed back before
// the queue is flushed, so the fused kernel keeps it in registers and never stores it.
int b200_binary_incr(b200_engine *e, int op, int dtype, int form, void *incr, const void *a, const void *b,
                     double scalar, int scalar_on_device, int64_t n) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_binary_incr: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_binary_incr: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, incr != nullptr, "b200_binary_incr: incr is null");
  void *tmp = nullptr;
  int rc = b200_get(e, n * (int64_t)dtype_size(dtype), &tmp);
  if (rc != B200_OK) return rc;
  rc = b200_binary(e, op, dtype, form, tmp, a, b, scalar, scalar_on_device, n);
  if (rc == B200_OK) rc = b200_binary(e, B200_OP_ADD, dtype, B200_VV, incr, incr, tmp, 0.0, 0, n);
  b200_put(e, tmp, 0);
  return rc;
}

int b200_unary_incr(b200_engine *e, int op, int dtype, void *incr, const void *a, int64_t n) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_unary_incr: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_unary_incr: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, incr != nullptr, "b200_unary_incr: incr is null");
  void *tmp = nullptr;
  int rc = b200_get(e, n * (int64_t)dtype_size(dtype), &tmp);
  if (rc != B200_OK) return rc;
  rc = b200_unary(e, op, dtype, tmp, a, n);
  if (rc == B200_OK) rc = b200_binary(e, B200_OP_ADD, dtype, B200_VV, incr, incr, tmp, 0.0, 0, n);
  b200_put(e, tmp, 0);
  return rc;
}

int b200_unary(b200_engine *e, int op, int dtype, void *dst, const void *a, int64_t n) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, is_unary(op), "b200_unary: %d is not a unary op", op);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_unary: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_unary: negative element count");
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, dst && a, "b200_unary: null pointer");
  b200_pw_call c;
  memset(&c, 0, sizeof c);
  c.op = op;
  c.dtype = dtype;
  c.form = 3;
  c.dst = (uint64_t)dst;
  c.a = (uint64_t)a;
  c.n = n;
  DeviceGuard g(e);
  return enqueue(e, c);
}

int b200_binary_bcast(b200_engine *e, int op, int dtype, void *dst, const void *a, const void *b, int64_t n,
                      int64_t b_div, int64_t b_mod, int bcast_is_a) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  B200_REQUIRE(e, is_binary(op), "b200_binary_bcast: %d is not a binary op", op);
  B200_REQUIRE(e, dtype == B200_F32 || dtype == B200_F64, "b200_binary_bcast: dtype %d not supported", dtype);
  B200_REQUIRE(e, n >= 0, "b200_binary_bcast: negative element count");
  B200_REQUIRE(e, b_div > 0 && b_mod > 0, "b200_binary_bcast: div %lld mod %lld", (long long)b_div,
               (long long)b_mod);
  if (n == 0) return B200_OK;
  B200_REQUIRE(e, dst && a && b, "b200_binary_bcast: null pointer");
  b200_pw_call c;
  memset(&c, 0, sizeof c);
  c.op = op;
  c.dtype = dtype;
  c.form = B200_VV;
  c.dst = (uint64_t)dst;
  c.a = (uint64_t)a;
  c.b = (uint64_t)b;
  c.n = n;
  c.bcast = bcast_is_a ? 2 : 1;
  c.bdiv = b_div;
  c.bmod = b_mod;
  DeviceGuard g(e);
  return enqueue(e, c);
}

int b200_pointwise(b200_engine *e, int dtype, const b200_pw_prog *prog, void *const *outs,
                   const void *const *srcs, int64_t n) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  DeviceGuard g(e);
  int rc = flush_pending(e);
  if (rc != B200_OK) return rc;
  return run_program(e, dtype, prog, outs, srcs, n);
}

int b200_pending(b200_engine *e, int *n_calls, int *n_kernels) {
  if (!e) return B200_ERR_INVALID;
  std::lock_guard<std::recursive_mutex> lk(e->mu);
  if (n_calls) *n_calls = (int)e->pending.size();
  if (n_kernels) {
    *n_kernels = 0;
    if (!e->pending.empty()) return plan_pending(e, n_kernels);
  }
  return B200_OK;
}

int b200_fusion_plan(const b200_pw_call *calls, int n_calls, const int *released_at, int *kernel_of_call,
                     int *n_kernels, int *loads, int *stores) {
  if (!calls || n_calls < 0 || !n_kernels) return B200_ERR_INVALID;
  std::vector<FusedKernel> ks;
  plan(calls, n_calls, released_at, &ks);
  *n_kernels = (int)ks.size();
  for (size_t k = 0; k < ks.size(); ++k) {
    if (kernel_of_call)
      for (int c = ks[k].first; c < ks[k].last; ++c) kernel_of_call[c] = (int)k;
    if (loads) loads[k] = ks[k].loads;
    if (stores) stores[k] = ks[k].stores;
  }
  return B200_OK;
}

}  // extern "C"
