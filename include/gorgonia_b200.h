/*
 * gorgonia_b200.h — C ABI of libgorgonia_b200.so, the sm_100a execution engine that sits
 * behind Gorgonia's tape VM.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int status
 * (B200_OK == 0) and never throws. Device pointers are raw CUDA addresses; they come from
 * b200_get() (the engine's arena) or from any other allocation on the engine's device.
 * The text of the most recent failure on an engine is returned by b200_last_error().
 *
 * Each declaration cites the piece of gorgonia (path:line inside the gorgonia repository)
 * whose job it takes over.
 *
 * Conventions
 *   - tensors are dense, row-major, contiguous unless a leading dimension is given;
 *   - element counts and strides are 64-bit;
 *   - work is enqueued on the engine's stream; host-visible results are valid after
 *     b200_sync() (or the d2h copy entry points, which synchronise themselves);
 *   - the compare ops write 1.0 / 0.0 in the operand dtype, as gorgonia's device kernels do.
 */
#ifndef GORGONIA_B200_H
#define GORGONIA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_engine b200_engine;

/* ---- status codes -------------------------------------------------------------------- */
enum {
  B200_OK = 0,
  B200_ERR_INVALID = 1,     /* bad argument: null pointer, negative size, unknown op/dtype     */
  B200_ERR_OOM = 2,         /* arena exhausted (gorgonia: oomError, cuda/errors.go:5-13)      */
  B200_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed; text in b200_last_error   */
  B200_ERR_UNSUPPORTED = 4, /* valid request that this build has no kernel for              */
  B200_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out (kernel returned early)   */
  B200_ERR_STATE = 6        /* call not legal in the engine's current state                  */
};

/* ---- dtypes ------------------------------------------------------------------------- */
enum { B200_F32 = 0, B200_F64 = 1, B200_BF16 = 2 };

/* ---- pointwise op codes ---------------------------------------------------------------
 * Binary ops mirror ʘBinaryOperatorType (operatorPointwise_binary_const.go:29-47) and the
 * device kernels add/sub/mul/div/pow/gt/gte/lt/lte/eq/ne (cuda modules/src/elembinop.cu).
 * Unary ops mirror ʘUnaryOperatorType (operatorPointwise_unary_const.go:75-103) and
 * cuda modules/src/elemunaryop.cu. */
enum {
  B200_OP_ADD = 0, B200_OP_SUB, B200_OP_MUL, B200_OP_DIV, B200_OP_POW, B200_OP_MOD,
  B200_OP_LT, B200_OP_GT, B200_OP_LTE, B200_OP_GTE, B200_OP_EQ, B200_OP_NE,
  B200_OP_BINARY_END,
  B200_OP_ABS = 32, B200_OP_SIGN, B200_OP_CEIL, B200_OP_FLOOR, B200_OP_SIN, B200_OP_COS,
  B200_OP_EXP, B200_OP_LN, B200_OP_LOG2, B200_OP_NEG, B200_OP_SQUARE, B200_OP_SQRT,
  B200_OP_INV, B200_OP_INVSQRT, B200_OP_CUBE, B200_OP_TANH, B200_OP_SIGMOID, B200_OP_LOG1P,
  B200_OP_EXPM1, B200_OP_SOFTPLUS,
  B200_OP_UNARY_END
};

/* operand forms of a binary op (constructName2 / constructName1, cuda/utils.go:114-139) */
enum { B200_VV = 0, B200_VS = 1, B200_SV = 2 };

/* ---- engine lifecycle  (cuda/external.go:88-220 Init/doInit/Close; cuda/engine.go:38-69) */
enum {
  B200_ENGINE_MANAGED = 1u,  /* arena in CUDA managed memory, preferred location = device:  *
                              * host code may dereference arena pointers, as gorgonia does   *
                              * (cuda/external.go:162, cuda/engine.go:71-72)                 */
  B200_ENGINE_NO_DEFER = 2u  /* launch each pointwise call at once instead of queueing it   */
};
int b200_engine_create(int device, size_t arena_bytes, unsigned flags, b200_engine **out);
int b200_engine_destroy(b200_engine *e);
int b200_engine_device(const b200_engine *e);
/* cudaStream_t of the engine, as an integer (for events recorded by the caller). */
uintptr_t b200_engine_stream(const b200_engine *e);
/* Text of the last failure on `e`; with e == NULL, of the last failed create on this thread. */
const char *b200_last_error(const b200_engine *e);
/* Engine.DoWork (cuda/external.go:223-226): launch whatever the deferred queue holds. */
int b200_flush(b200_engine *e);
/* Engine.Signal + Sync (cuda/external.go:46-50,229-276): flush, then wait for the stream.
 * Asynchronous device errors surface here. */
int b200_sync(b200_engine *e);
/* Number of kernels this engine has launched since creation (tests and bench count with it). */
uint64_t b200_launch_count(const b200_engine *e);

/* CUDA events on the engine's stream, for callers that time device work without linking the
 * CUDA runtime themselves (no counterpart in gorgonia, which has no device timing).
 * b200_event_elapsed_ms waits for `stop` to complete. */
int b200_event_create(b200_engine *e, void **event);
int b200_event_record(b200_engine *e, void *event);
int b200_event_elapsed_ms(b200_engine *e, void *start, void *stop, float *ms);
int b200_event_destroy(b200_engine *e, void *event);

/* ---- arena: Engine.Get / Put / ResetAllocator (cuda/arena.go:13-36) over a best-fit
 * allocator with coalescing (cuda/bfc.go:298-463). Addresses are 256-byte aligned.
 * b200_get(bytes <= 0) is an error; b200_put of an unknown address is a no-op; `bytes`
 * of b200_put is ignored, as in the reference. */
int b200_get(b200_engine *e, int64_t bytes, void **dptr);
int b200_put(b200_engine *e, void *dptr, int64_t bytes);
int b200_reset(b200_engine *e);
/* used / free / largest free block / number of free blocks */
int b200_arena_stats(b200_engine *e, int64_t *used, int64_t *free_bytes, int64_t *largest_free,
                     int64_t *n_free_blocks);

/* The allocator alone, over offsets, with no device behind it (cuda/bfc_test.go:47-120). */
typedef struct b200_bfc b200_bfc;
b200_bfc *b200_bfc_create(int64_t bytes, int64_t align);
void b200_bfc_destroy(b200_bfc *a);
int b200_bfc_alloc(b200_bfc *a, int64_t bytes, int64_t *offset);
int b200_bfc_free(b200_bfc *a, int64_t offset);
void b200_bfc_reset(b200_bfc *a);
int64_t b200_bfc_free_blocks(const b200_bfc *a);
int64_t b200_bfc_used(const b200_bfc *a);
int64_t b200_bfc_largest_free(const b200_bfc *a);

/* ---- copies: Engine.Memcpy (cuda/engine.go:118-138), ExternMetadata.Transfer
 * (cuda.go:168-207), deviceTransport.exec (vm_tape_cuda.go:220-243).
 * h2d/d2h flush the deferred queue first; d2h returns after the data has arrived.
 * The _async forms return at once and expect pinned host memory. */
int b200_memcpy_h2d(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_memcpy_d2h(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_memcpy_d2d(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_memcpy_h2d_async(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_memcpy_d2h_async(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_memset(b200_engine *e, void *dst, int value, int64_t bytes);
/* pinned host staging buffers */
int b200_host_alloc(int64_t bytes, void **hptr);
int b200_host_free(void *hptr);

/* ---- pointwise ------------------------------------------------------------------------
 * b200_binary: Engine.Add/Sub/Mul/Div/Pow/Mod and Lt/Lte/Gt/Gte/ElEq/ElNe with their
 * *Scalar forms (cuda/arith.go:14-701, cuda/cmp.go:14-701), reached from
 * elemBinOp.CUDADo (op_math_cuda.go:89-176).
 *   form VV: dst[i] = a[i] op b[i]
 *   form VS: dst[i] = a[i] op s          (b is ignored unless scalar_on_device)
 *   form SV: dst[i] = s    op b[i]       (a is ignored unless scalar_on_device)
 * dst may alias a or b (the reference's "unsafe" mode) or be a third buffer ("reuse").
 * With scalar_on_device != 0 the scalar is read from a[0] (SV) or b[0] (VS) on the device,
 * as the reference passes it (cuda/arith.go:73-77); otherwise `scalar` is used. */
int b200_binary(b200_engine *e, int op, int dtype, int form, void *dst, const void *a,
                const void *b, double scalar, int scalar_on_device, int64_t n);
/* b200_unary: elemUnaryOp.CUDADo (op_math_cuda.go:23-85). dst may alias a. */
int b200_unary(b200_engine *e, int op, int dtype, void *dst, const void *a, int64_t n);

/* Binary op with one operand broadcast, replacing the reference's materialised repeat
 * (broadcast.go:69-129, op_tensor.go:354-473). Element i of the broadcast operand is
 * b[(i / b_div) % b_mod]: row vector over (R,C): div=1, mod=C; column over (R,C): div=C,
 * mod=R; per-channel over (B,C,H,W): div=H*W, mod=C. bcast_is_a != 0 broadcasts a instead. */
int b200_binary_bcast(b200_engine *e, int op, int dtype, void *dst, const void *a, const void *b,
                      int64_t n, int64_t b_div, int64_t b_mod, int bcast_is_a);

/* A fused chain of pointwise instructions evaluated in one pass over memory. */
#define B200_PW_MAX_INSTR 8
#define B200_PW_MAX_SRC 6
#define B200_PW_MAX_IMM 8
#define B200_PW_MAX_OUT 4
/* operand references */
#define B200_REF_SRC(k) ((uint8_t)(0x00 | (k)))  /* k-th source tensor            */
#define B200_REF_IMM(k) ((uint8_t)(0x40 | (k)))  /* k-th immediate                */
#define B200_REF_INS(k) ((uint8_t)(0x80 | (k)))  /* result of the k-th instruction */
typedef struct {
  uint8_t op; /* B200_OP_* */
  uint8_t a;  /* operand reference */
  uint8_t b;  /* operand reference; ignored by unary ops */
  uint8_t reserved;
} b200_pw_instr;
typedef struct {
  uint32_t n_instr, n_src, n_imm, n_out;
  b200_pw_instr instr[B200_PW_MAX_INSTR];
  double imm[B200_PW_MAX_IMM];
  uint8_t out_instr[B200_PW_MAX_OUT]; /* output k stores the result of instr out_instr[k] */
  /* per source: element i reads src[(i / div) % mod]; div = 0 means a full-size tensor */
  int64_t src_div[B200_PW_MAX_SRC];
  int64_t src_mod[B200_PW_MAX_SRC];
} b200_pw_prog;
int b200_pointwise(b200_engine *e, int dtype, const b200_pw_prog *prog, void *const *outs,
                   const void *const *srcs, int64_t n);

/* ---- run-time fusion of pointwise calls ---------------------------------------------------
 * gorgonia defers device work: cu.BatchedContext queues launches until DoWork, and the
 * compiler emits flushInstr only where a consumer needs a value (compile.go:391-462,
 * vm_tape.go:735-745, cuda/external.go:223-226). This engine keeps that contract and uses it:
 * b200_binary / b200_unary / b200_binary_bcast calls are queued, and at the next flush
 * (b200_flush, b200_sync, any copy, any non-pointwise entry point) runs of calls over the
 * same element count and dtype become ONE kernel each. A value produced and consumed inside
 * a run travels in registers; a buffer handed back with b200_put before the flush, and not
 * read by a later run, is never written.
 *
 * b200_pending reports the queue length and how many kernels a flush would launch now.
 * b200_fusion_plan runs the same grouping pass on a caller-supplied list, without a device:
 * kernel_of_call[i] is the kernel call i lands in; loads/stores count the full-size tensor
 * reads/writes of each kernel (arrays sized n_calls). released_at[i] is the queue position
 * at which call i's dst was released with b200_put, or -1. */
typedef struct {
  int32_t op, dtype, form; /* form: B200_VV / B200_VS / B200_SV, or 3 for a unary op */
  int32_t bcast;           /* 0 none, 1 operand b is broadcast, 2 operand a is broadcast */
  uint64_t dst, a, b;      /* device addresses */
  uint64_t scalar_ptr;     /* non-zero: scalar operand is read from this device address */
  double scalar;
  int64_t n, bdiv, bmod;
} b200_pw_call;
int b200_pending(b200_engine *e, int *n_calls, int *n_kernels);
int b200_fusion_plan(const b200_pw_call *calls, int n_calls, const int *released_at,
                     int *kernel_of_call, int *n_kernels, int *loads, int *stores);

/* Engine.HasNaN / HasInf (cuda/engine.go:144-191; kernels cuda modules/src/misc.cu:13-55).
 * *result is 1 if any element is NaN (resp. ±Inf), else 0. Synchronises. */
int b200_has_nan(b200_engine *e, int dtype, const void *x, int64_t n, int *result);
int b200_has_inf(b200_engine *e, int dtype, const void *x, int64_t n, int *result);

#ifdef __cplusplus
}
#endif
#endif /* GORGONIA_B200_H */
