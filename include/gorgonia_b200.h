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
  B200_ENGINE_NO_DEFER = 2u, /* launch each pointwise call at once instead of queueing it   */
  B200_ENGINE_CONV_GATHER = 4u, /* tensor-core convolutions build their col operand with gather *
                                 * warps even where the TMA unit could (tests, comparisons)    */
  B200_ENGINE_NO_STREAMK = 8u,  /* tensor-core kernels never share a tile's k range between    *
                                 * CTAs: every output element is then summed in one fixed      *
                                 * order whatever the batch size (tests, comparisons)          */
  B200_ENGINE_NO_PAIRS = 16u    /* tensor-core kernels never run as pairs of CTAs on one       *
                                 * 256-row tile (tests, comparisons); results are the same     *
                                 * bits either way                                             */
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
 * Asynchronous device errors surface here, and so does a bounded device-side wait that ran out
 * (B200_ERR_TIMEOUT: the results of the kernels since the last synchronising call are incomplete;
 * the engine stays usable). Every entry point that waits for the stream reports it the same way:
 * b200_memcpy_h2d / _d2h, b200_has_nan / _inf, b200_gather_axis. */
int b200_sync(b200_engine *e);
/* Launches one warp that waits, with the library's bounded wait and a limit of `limit_us`
 * microseconds (1 .. 10000), on a barrier nobody arrives at. The wait gives up, the kernel returns
 * normally, and the next synchronising call returns B200_ERR_TIMEOUT. It exists so that the
 * time-out path can be exercised without a stuck kernel; no counterpart in gorgonia. */
int b200_selftest_wait(b200_engine *e, int64_t limit_us);
/* Number of kernels this engine has launched since creation (tests and bench count with it). */
uint64_t b200_launch_count(const b200_engine *e);

/* ---- tapes -------------------------------------------------------------------------------------
 * The per-instruction launch path of the tape VM (execOp.exec, vm_tape_cuda.go:66-150; RunAll,
 * vm_tape.go:213-347) costs one host call per instruction. A forward tape whose shapes and buffers
 * do not change between runs can instead be recorded once and replayed with ONE call:
 * between b200_tape_begin and b200_tape_end every engine call is recorded (into a CUDA graph on
 * the engine's stream) instead of executed; b200_tape_launch replays it. Buffers the caller still
 * holds when recording ends must stay allocated, at the same addresses, for as long as the tape is
 * used. Everything else the recorded kernels touch belongs to the tape: arena scratch the library
 * took and handed back while recording, buffers the caller released with b200_put while recording,
 * and forms derived from constant buffers stay allocated until b200_tape_destroy, so allocations
 * made between replays can never be given those bytes (gorgonia frees a register at its last use,
 * vm_tape.go:639-653; every replay is a use). b200_reset ends that ownership: tapes recorded before
 * it refuse to launch (B200_ERR_STATE), and it is refused while recording.
 * Entry points that wait for the device (b200_sync, the synchronous copies, b200_has_nan/inf)
 * return B200_ERR_STATE while recording; the _async copies can be recorded. Run the sequence once
 * unrecorded first, so that one-time set-up (kernel attributes, lazily created scratch) is done. */
typedef struct b200_tape b200_tape;
int b200_tape_begin(b200_engine *e);
int b200_tape_end(b200_engine *e, b200_tape **out);
int b200_tape_launch(b200_engine *e, b200_tape *t);
int b200_tape_destroy(b200_engine *e, b200_tape *t);

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
/* Uploads that overlap compute (the H->D half of deviceTransport.exec, vm_tape_cuda.go:227-230,
 * without stalling the tape). b200_upload_async copies pinned host memory to the device on a
 * second stream; it starts only after the compute work queued so far (which may still read
 * `dst`), and compute queued AFTER the call runs concurrently with it. b200_upload_wait makes
 * the compute stream wait for the uploads queued so far; call it before the first kernel that
 * reads `dst`. With two input buffers used in turn, the upload of batch i+1 hides behind the
 * forward pass of batch i. Neither call can be recorded into a tape. */
int b200_upload_async(b200_engine *e, void *dst, const void *src, int64_t bytes);
int b200_upload_wait(b200_engine *e);
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
  uint64_t scalar_ptr;     /* Incr mode of ExternalOp.Do (execution.go:113-127; NewAddOp / NewSubOp / NewHadamardProdOp,
 * op_math_cuda.go:245-308): incr = incr + op(a, b), the result of the op rounded to the tensor's type
 * before the addition, as "CUDADo into a temporary, then an unsafe add" does. One fused kernel when
 * the queue is deferred; the temporary is never written to memory. Same operand forms as b200_binary
 * and b200_unary. */
int b200_binary_incr(b200_engine *e, int op, int dtype, int form, void *incr, const void *a,
                     const void *b, double scalar, int scalar_on_device, int64_t n);
int b200_unary_incr(b200_engine *e, int op, int dtype, void *incr, const void *a, int64_t n);
/* non-zero: scalar operand is read from this device address */
  double scalar;
  int64_t n, bdiv, bmod;
} b200_pw_call;
int b200_pending(b200_engine *e, int *n_calls, int *n_kernels);
int b200_fusion_plan(const b200_pw_call *calls, int n_calls, const int *released_at,
                     int *kernel_of_call, int *n_kernels, int *loads, int *stores);

/* Dropout without cuDNN: dropoutOp.do and dropoutDiffOp (op_dropout.go:106-128,205-240), in place of
 * the cuDNN calls of ops/nn/dropout_cuda.go:76-149.
 * b200_dropout_fwd: y[i] = r[i] < keep ? x[i] / keep : 0 with keep = 1 - probability rounded to the
 *   tensor's type. r comes from `uniforms` (a device array of n values in [0, 1) in the tensor's type;
 *   gorgonia injects its generator the same way) or, with uniforms == NULL, from Philox-4x32-10 keyed
 *   by `seed` with the element index + `offset` as the counter: stateless, the same draw on every
 *   replay. probability == 0 copies x (the reference hands the input through).
 * b200_dropout_bwd: dx[i] = (probability != 0 && out[i] != 0) ? dy[i] / probability : 0, where `out`
 *   is what the forward pass wrote: the reference finds the kept elements by their non-zero output
 *   and divides by the DROP probability; both are reproduced as written. */
int b200_dropout_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t n, double probability,
                     const void *uniforms, uint64_t seed, uint64_t offset);
int b200_dropout_bwd(b200_engine *e, int dtype, const void *dy, const void *out, void *dx, int64_t n,
                     double probability);

/* ---- the training variant's collective ----------------------------------------------------------
 * The mean of a flat gradient bucket over the ranks, taken after the last backward kernel and before
 * Solver.Step (solvers.go:13-15). gorgonia itself has no distributed path (README.md:21; its
 * data-parallel precedent is example_concurrent_training_test.go:80-115); the forward path never
 * calls this. The transport is a function pointer: in-place sum of `count` elements of `dtype` at
 * `buf` over all ranks, enqueued on `stream` (a cudaStream_t as an integer; 0 for host buffers),
 * returning 0 on success.
 * b200_comm_create        wraps any such function (the host program's own, or a test's).
 * b200_comm_create_nccl   binds NCCL (loaded at run time by its soname) for the engine's device; id128
 *                         is the 128-byte ncclUniqueId that rank 0 made with b200_nccl_unique_id and
 *                         handed to the other ranks by whatever rendezvous the host program has.
 * b200_allreduce_mean     device bucket: flushes the engine's queue, runs the transport on the
 *                         engine's stream, then divides by the number of ranks on the same stream.
 *                         A transport failure is B200_ERR_CUDA and leaves the bucket unscaled.
 * b200_comm_allreduce_mean_host  the same on a host buffer, for CPU ranks (tests of the plumbing). */
typedef struct b200_comm b200_comm;
typedef int (*b200_allreduce_fn)(void *ctx, void *buf, int64_t count, int dtype, uintptr_t stream);
int b200_comm_create(b200_allreduce_fn fn, void *ctx, int rank, int world, b200_comm **out);
int b200_comm_create_nccl(b200_engine *e, const void *id128, int rank, int world, b200_comm **out);
int b200_nccl_unique_id(void *id128);
int b200_comm_destroy(b200_comm *c);
int b200_comm_world(const b200_comm *c);
int b200_comm_rank(const b200_comm *c);
const char *b200_comm_last_error(const b200_comm *c);
int b200_allreduce_mean(b200_engine *e, b200_comm *c, void *dptr, int64_t n, int dtype);
int b200_comm_allreduce_mean_host(b200_comm *c, void *buf, int64_t n, int dtype);

/* Engine.HasNaN / HasInf (cuda/engine.go:144-191; kernels cuda modules/src/misc.cu:13-55).
 * *result is 1 if any element is NaN (resp. ±Inf), else 0. Synchronises. */
int b200_has_nan(b200_engine *e, int dtype, const void *x, int64_t n, int *result);
int b200_has_inf(b200_engine *e, int dtype, const void *x, int64_t n, int *result);

/* ---- linear algebra -------------------------------------------------------------------------
 * All matrices are row-major with a leading dimension (elements between consecutive rows).
 *
 * b200_gemm: Engine.MatMul (cuda/linalg.go:110-229; cuBLAS Sgemm/Dgemm in the reference) as
 *   reached from linAlgBinOp.CUDADo (op_math_cuda.go:182-240), and batchedMatMul
 *   (operatorLinAlg.go:435-502) in one launch. C[b] = op(A[b]) op(B[b]), alpha = 1, beta = 0;
 *   op(A) is M x K, op(B) is K x N; transX != 0 means the stored matrix is the transpose
 *   (K x M, resp. N x K). batch >= 1 matrices lie strideX elements apart.
 *   dtype B200_F32: float32 in and out; large aligned problems run on the tensor cores as
 *     3xTF32 (each operand split into a TF32 head and tail, three products, fp32 accumulate),
 *     the rest on CUDA cores in fp32. The splits live in arena scratch for the duration of the
 *     call (about 2 x (|A| + |B|) bytes); when the arena cannot supply them the CUDA-core kernel
 *     computes the product instead, so the call never fails for lack of workspace.
 *   dtype B200_BF16: bfloat16 A and B, float32 C, fp32 accumulate on the tensor cores.
 *   dtype B200_F64: CUDA cores.
 *   `ep` (may be NULL) fuses a bias add and an activation into the store.
 * b200_gemv: Engine.MatVecMul (cuda/linalg.go:47-107): y = A x, or y = A^T x with transA; A is
 *   M x N as stored.
 * b200_ger: Engine.Outer (cuda/linalg.go:232-285): A = x y^T, overwriting A (what tensor.Outer
 *   with a reuse tensor does; the reference's cuBLAS path accumulates instead, for lack of a beta). */
enum { B200_BIAS_NONE = 0, B200_BIAS_COL = 1, B200_BIAS_ROW = 2 };
enum { B200_ACT_NONE = 0, B200_ACT_RECTIFY = 1, B200_ACT_LEAKY = 2 };
typedef struct {
  int32_t bias_kind;  /* B200_BIAS_*: COL = one value per output column (n), ROW = per row (m) */
  int32_t act;        /* B200_ACT_*: Rectify x*(x>=0) (nn.go:136-163), LeakyRelu (nn.go:83-131) */
  const void *bias;   /* device vector in the output dtype */
  double alpha;       /* LeakyRelu slope */
  int32_t accumulate; /* b200_gemm only: C = C + act(A.B + bias), the product rounded to the   *
                       * output type before the addition (Incr mode, execution.go:115-126)     */
  int32_t reserved;   /* must be 0 */
} b200_epilogue;
int b200_gemm(b200_engine *e, int dtype, int transA, int transB, int64_t M, int64_t N, int64_t K,
              const void *A, int64_t lda, const void *B, int64_t ldb, void *C, int64_t ldc,
              int64_t batch, int64_t strideA, int64_t strideB, int64_t strideC,
              const b200_epilogue *ep);
/* Measures what this GPU's tensor cores sustain with kind::tf32 instructions alone: every SM issues
 * `batches` x 16 MMAs of 128 x 256 x 8 on operands resident in shared memory, no loads, no epilogue;
 * best of three timed launches, in TFLOP/s of TF32 work. The float32 (3xTF32) rooflines of the
 * benchmark use it as their denominator. Synchronises. No counterpart in gorgonia. */
int b200_tf32_peak(b200_engine *e, int batches, double *tflops);
/* One link of a CHAIN of float32 matrix products C = act(A.op(B) + bias) (a stack of dense layers:
 * examples/286/main.go:72-99, examples/convnet/main.go:138-159), the counterpart of
 * b200_conv2d_chain_fwd. The tensor-core product reads its operands split into a TF32 head and
 * tail; a link can write its result in that form (C_hi, C_lo, row pitch ld_split = N rounded up to a
 * multiple of 4; C may be NULL) and the next link reads it as its A (A_hi, A_lo with lda = that pitch; A may be
 * NULL), which spares the split pass over every activation. Columns N .. ld_split-1 are zero-filled.
 * Shapes that run on the CUDA-core kernel need A and answer B200_ERR_UNSUPPORTED without it.
 * Results are bit-identical to b200_gemm. */
int b200_gemm_chain(b200_engine *e, int transB, int64_t M, int64_t N, int64_t K, const void *A,
                    const void *A_hi, const void *A_lo, int64_t lda, const void *B, int64_t ldb,
                    void *C, void *C_hi, void *C_lo, int64_t ldc, int64_t ld_split,
                    const b200_epilogue *ep);
int b200_gemv(b200_engine *e, int dtype, int transA, int64_t M, int64_t N, const void *A,
              int64_t lda, const void *x, void *y);
int b200_ger(b200_engine *e, int dtype, int64_t M, int64_t N, const void *x, const void *y, void *A);
/* Which kernel b200_gemm would pick for a problem: 0 = CUDA cores, 1 = tensor cores.
 * Needs no device work; lets tests assert that the tensor-core path is the one exercised. */
int b200_gemm_path(b200_engine *e, int dtype, int transA, int transB, int64_t M, int64_t N, int64_t K,
                   int64_t lda, int64_t ldb, int64_t ldc, const void *A, const void *B, const void *C);

/* Declares a device buffer constant (is_constant != 0) or mutable again (0). gorgonia re-derives
 * nothing from weights, but it re-uploads them on every run (analysis.go:151-176 puts a devTrans
 * in front of every argument node); this engine keeps them resident, and for a buffer declared
 * constant it also keeps what it derives from it — the TF32 head/tail split the tensor-core matrix
 * multiply and convolution need — instead of recomputing it per call. The caller promises not to
 * write the buffer while it is declared constant (a Go shim declares a node's value constant when
 * it is bound with Let and un-declares it when it is rebound; solvers update weights between runs,
 * so a training loop un-declares them). b200_put and b200_reset end the declaration. */
int b200_set_constant(b200_engine *e, const void *ptr, int is_constant);

/* ---- softmax, reductions, argmax ----------------------------------------------------------
 * A tensor is viewed as (outer, len, inner) around the axis that is reduced.
 * b200_softmax: softmaxOp.Do -> tensor.SoftMax / LogSoftMax (op_softmax.go:99-128); y has x's shape.
 * b200_reduce:  reductionDo -> tensor.Sum / tensor.Max along one axis (op_reduction.go:70-99);
 *               kind 0 = sum, 1 = max; y has outer*inner elements.
 * b200_reduce_all: the same ops over every axis at once (sumOp / maxOp with along = all axes);
 *               y is one element on the device.
 * b200_argmax:  index of the first maximum along the axis, as int64 (tensor.Argmax as used by
 *               the examples' accuracy loops, examples/convnet/main.go). */
int b200_softmax(b200_engine *e, int dtype, const void *x, void *y, int64_t outer, int64_t len,
                 int64_t inner, int is_log);
int b200_reduce(b200_engine *e, int dtype, int kind, const void *x, void *y, int64_t outer,
                int64_t len, int64_t inner);
int b200_reduce_all(b200_engine *e, int dtype, int kind, const void *x, int64_t n, void *y);
int b200_argmax(b200_engine *e, int dtype, const void *x, int64_t *y, int64_t outer, int64_t len,
                int64_t inner);

/* b200_reduce_all for callers that must not allocate. It has no counterpart in gorgonia.
 *
 * Who needs it: code that runs where device allocation is off limits once set-up is over, e.g. a
 * serving loop that has handed all free device memory to its own pools, a host thread that must
 * not take the driver's allocation lock on its latency path, or a process whose memory budget is
 * fixed at start-up. b200_reduce_all reserves its scratch (per-CTA partial results and a ticket
 * word) with cudaMalloc on its first call per engine; this entry point keeps the same scratch in
 * a fixed array inside the library image instead, so it calls no cudaMalloc, no cudaFree and no
 * allocating library routine, ever. The cost: that array (8448 bytes) sits on every GPU that
 * loads the library until the process exits.
 *
 * Same arguments and result as b200_reduce_all (kind 0 = sum, 1 = max; y is one element on the
 * device, written on the engine's stream), with these limits:
 *   - at most B200_REDUCE_ALL_STATIC_MAX_N elements; more is refused with B200_ERR_UNSUPPORTED;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress):
 *     make that first call before any stream capture begins;
 *   - all calls on one GPU share the one array, whatever engine they come through. Two calls
 *     whose kernels overlap on the GPU (different engines, i.e. different streams) race on it and
 *     both results are undefined; calls through one engine are ordered by its stream and safe.
 *     The array keeps the last call's contents; each call clears the word that must start at zero. */
#define B200_REDUCE_ALL_STATIC_MAX_N ((int64_t)1 << 32)
int b200_reduce_all_static(b200_engine *e, int dtype, int kind, const void *x, int64_t n, void *y);

/* ---- convolution, pooling, data movement ------------------------------------------------------
 * Tensors are NCHW, dense.
 * b200_conv2d_fwd: Conv2d (nn.go:211-305) as one call: x (B,C,H,W) * w (K,C,kh,kw) -> y (B,K,Ho,Wo),
 *   Ho = (H + 2 pad_h - (dil_h (kh-1) + 1)) / stride_h + 1 (op_nn.go:311-315). The reference builds it
 *   from Im2Col, Reshape, MatMul, Reshape, Transpose; float32 runs on the tensor cores (3xTF32).
 *   `ep` (may be NULL): per-output-channel bias (B200_BIAS_ROW) and activation fused into the store.
 *   Workspace: the tensor-core kernels read an NHWC TF32 head/tail copy of x kept in arena scratch
 *   for the duration of the call (8 bytes per input element) plus the split filters; B200_ERR_OOM
 *   if the arena cannot supply it.
 * b200_im2col: im2colOp.do (op_nn.go:317-444): col (B, Ho, Wo, C*kh*kw), inner order channel, kernel
 *   row, kernel column; taps outside the image are 0.
 * b200_maxpool2d_fwd: maxPoolOp.do (op_nn.go:828-907). Output (H + pad_north + pad_south - kh) /
 *   stride_h + 1 (op_nn.go:810-816). explicit_padding != 0 reproduces gorgonia's 4-value padding,
 *   whose window origin uses the south / east pads (op_nn.go:870-875). mask (may be NULL) receives
 *   the winning index inside the (H,W) plane as int64, -1 for an empty window.
 * b200_transpose: transposeOp.Do -> tensor.Transpose (op_tensor.go:937-952): output axis d is input
 *   axis perm[d]; elem_bytes 2, 4 or 8; rank <= 8.
 * b200_gather_axis: byIndicesOp.Do -> tensor.ByIndices along any axis (op_by_indices.go:90-97), the
 *   tensor viewed as (outer, n_rows, row): y[o,i,:] = x[o,idx[i],:], idx int64 on the device. An
 *   index outside [0, n_rows) is an error (checked on the device, reported by this call). Recorded
 *   into a tape, the call cannot wait for the check: a replay skips such rows, and the next call that
 *   waits for the stream (b200_sync, b200_memcpy_d2h, ...) returns B200_ERR_INVALID.
 *   b200_gather_rows is the axis-0 form (outer = 1). */
int b200_conv2d_fwd(b200_engine *e, int dtype, const void *x, const void *w, void *y, int64_t B,
                    int64_t C, int64_t H, int64_t W, int64_t K, int kh, int kw, int pad_h, int pad_w,
                    int stride_h, int stride_w, int dil_h, int dil_w, const b200_epilogue *ep);
/* Conv2d -> (bias, activation) -> MaxPool2D without padding as ONE call, for a tape in which the
 * convolution output has no other consumer (nn.go:211-305 followed by op_nn.go:828-907; the LeNet and
 * tiny-YOLO graphs of examples/convnet and examples/tiny-yolo-v2-coco are built from exactly this
 * triple). y is (B, K, (Ho - pool_h) / pool_stride_h + 1, (Wo - pool_w) / pool_stride_w + 1). With a
 * 2x2 / stride-2 window and even Ho, Wo the first-layer kernel and the window kernel pool inside
 * their store and never write the convolution output; any other shape runs the two operations one
 * after the other through arena scratch. Results equal b200_conv2d_fwd + b200_maxpool2d_fwd bit
 * for bit. */
int b200_conv2d_maxpool_fwd(b200_engine *e, int dtype, const void *x, const void *w, void *y,
                            int64_t B, int64_t C, int64_t H, int64_t W, int64_t K, int kh, int kw,
                            int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w,
                            const b200_epilogue *ep, int pool_h, int pool_w, int pool_stride_h,
                            int pool_stride_w);
/* One link of a CHAIN of convolutions (float32), for a tape in which a convolution's result is read
 * only by the next convolution (possibly through a 2x2 / stride-2 max-pool: pool2 != 0), as in the
 * convnet and tiny-YOLO graphs. Same arithmetic as b200_conv2d_fwd / b200_conv2d_maxpool_fwd; the
 * tensors between links may additionally, or only, exist in the layout the tensor-core kernels read:
 * channels innermost (B, H, W, C), every value split into its TF32 head and the TF32 rounding of
 * the remainder. A link that writes that form (y_hi, y_lo; K a multiple of 4; y may be NULL) from
 * its epilogue, and a next link that reads it (x_hi, x_lo; x may be NULL), together skip the
 * rewrite pass each tensor-core convolution otherwise starts with. Shapes whose kernel reads NCHW
 * need x and answer B200_ERR_UNSUPPORTED without it; shapes whose kernel cannot write the split
 * form get it from a rewrite pass. Results are bit-identical to the unchained calls. */
int b200_conv2d_chain_fwd(b200_engine *e, const void *x, const void *x_hi, const void *x_lo,
                          const void *w, void *y, void *y_hi, void *y_lo, int64_t B, int64_t C,
                          int64_t H, int64_t W, int64_t K, int kh, int kw, int pad_h, int pad_w,
                          int stride_h, int stride_w, int dil_h, int dil_w, const b200_epilogue *ep,
                          int pool2);
/* Which kernel b200_conv2d_fwd would pick for a problem (no device work; -1 for a bad shape):
 * CUDA cores over an im2col scratch; the direct kernel for a first layer (C*kh*kw <= 32, K <= 32);
 * tensor cores with the col operand gathered by warps; tensor cores with the col operand built
 * by the TMA unit in im2col mode from an NHWC copy (C a multiple of 32, more than one tap);
 * tensor cores reading every tap in place from an input window held in shared memory (stride 1,
 * C = 16, 32 or 64, output planes that 16 x 16 tiles cover well). */
enum { B200_CONV_SIMT = 0, B200_CONV_DIRECT = 1, B200_CONV_TC_GATHER = 2, B200_CONV_TC_TMA = 3,
       B200_CONV_TC_WINDOW = 4 };
int b200_conv2d_path(b200_engine *e, int dtype, int64_t B, int64_t C, int64_t H, int64_t W, int64_t K,
                     int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h,
                     int dil_w);
int b200_im2col(b200_engine *e, int dtype, const void *x, void *col, int64_t B, int64_t C, int64_t H,
                int64_t W, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h,
                int dil_w);
/* ---- backward ops (the training variant of the tapes) ------------------------------------------
 * b200_maxpool2d_bwd: maxPoolDiffOp.do (op_nn.go:1041-1121): dx (B,C,H,W) is zero except where a mask
 *   entry points: dx[plane][mask[i]] += dy[plane][i], summed in (ph, pw) order. `mask` is the int64
 *   mask b200_maxpool2d_fwd wrote for the same geometry (entries of -1 contribute nothing).
 * b200_col2im: col2imOp.do (op_nn.go:446-637), the adjoint of b200_im2col: col (B, Ho, Wo, C*kh*kw)
 *   accumulated into im (B,C,H,W), each pixel's additions in ascending (output row, output column)
 *   order as the reference's walk over col makes them.
 * b200_softmax_bwd: softmaxDiffOp (op_softmax.go:180-285) -> tensor.SoftMaxB / LogSoftMaxB on
 *   (outer, len, inner): dx = y * (g - sum(g * y)), or for log-softmax dx = g - exp(y) * sum(g).
 * Incr-mode matrix product (the "+=" of matMulDiff, operatorLinAlg.go:104-179, which the reference
 * emulates as product-then-add, execution.go:115-126): b200_gemm with b200_epilogue.accumulate = 1. */
/* b200_batchnorm_fwd: BatchNormOp.Do (op_nn.go:1158-1640) on x viewed as (B, C, S), S = product of the
 *   spatial extents (1 for a matrix). The reference has a cuDNN CUDADoer for it only in ops/nn
 *   (ops/nn/batchnorm_cuda.go); this is the cuDNN-free one. training != 0: per-channel saveMean = mean(x),
 *   saveVar = sum (x - mean)^2, running = momentum * new + (1 - momentum) * running with the unbiased
 *   variance saveVar / (n - 1), y = (x - mean) / sqrt(saveVar / n + epsilon). training == 0:
 *   y = (x - running_mean) / sqrt(running_var + epsilon). Output as x * alpha + beta (a product, then
 *   a sum, as the reference rounds it). Scale and bias are separate graph ops (nn.go:430-436), i.e.
 *   b200_binary_bcast calls. All four statistics vectors are device arrays of C elements. */
int b200_batchnorm_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t B, int64_t C,
                       int64_t S, int training, double momentum, double epsilon, void *running_mean,
                       void *running_var, void *save_mean, void *save_var);
/* b200_batchnorm_bwd: batchnormDiffOp (op_nn.go:1727-1940): the gradient with respect to the
 *   BatchNormOp input from x, dy and the statistics the forward call saved. training != 0:
 *   dx = (dy - mean(dy) - (x - mean) * k) / std with k = sum((x - mean) dy) / (n * var_eps);
 *   training == 0: dx = dy / std. The reference's two branches (matrix, spatial) differ in the order of
 *   the subtractions and in which variance the inference case reads; both are reproduced. */
int b200_batchnorm_bwd(b200_engine *e, int dtype, const void *x, const void *dy, void *dx, int64_t B,
                       int64_t C, int64_t S, int training, double epsilon, const void *running_var,
                       const void *save_mean, const void *save_var);
int b200_maxpool2d_bwd(b200_engine *e, int dtype, const void *dy, const int64_t *mask, void *dx,
                       int64_t B, int64_t C, int64_t H, int64_t W, int kh, int kw, int pad_north,
                       int pad_south, int pad_west, int pad_east, int explicit_padding, int stride_h,
                       int stride_w);
int b200_col2im(b200_engine *e, int dtype, const void *col, void *im, int64_t B, int64_t C, int64_t H,
                int64_t W, int kh, int kw, int pad_h, int pad_w, int stride_h, int stride_w, int dil_h,
                int dil_w);
int b200_softmax_bwd(b200_engine *e, int dtype, const void *y, const void *grad, void *dx,
                     int64_t outer, int64_t len, int64_t inner, int is_log);
/* b200_maxpool2d_fwd for float32 whose result feeds a link of b200_conv2d_chain_fwd: the pooled tensor
 * is written as the NHWC TF32 head / tail pair that link reads (y_hi, y_lo: B x Ho x Wo x C each) and,
 * if y is not NULL, in NCHW too. One pass instead of the pool followed by the rewrite. */
int b200_maxpool2d_split_fwd(b200_engine *e, const void *x, void *y, void *y_hi, void *y_lo, int64_t B,
                             int64_t C, int64_t H, int64_t W, int kh, int kw, int pad_north, int pad_south,
                             int pad_west, int pad_east, int explicit_padding, int stride_h, int stride_w);
int b200_maxpool2d_fwd(b200_engine *e, int dtype, const void *x, void *y, int64_t *mask, int64_t B,
                       int64_t C, int64_t H, int64_t W, int kh, int kw, int pad_north, int pad_south,
                       int pad_west, int pad_east, int explicit_padding, int stride_h, int stride_w);
int b200_transpose(b200_engine *e, int elem_bytes, const void *x, void *y, int ndim,
                   const int64_t *shape, const int *perm);
int b200_gather_axis(b200_engine *e, const void *x, const int64_t *idx, void *y, int64_t outer,
                     int64_t n_rows, int64_t n_idx, int64_t row_bytes);
int b200_gather_rows(b200_engine *e, const void *x, const int64_t *idx, void *y, int64_t n_idx,
                     int64_t row_bytes, int64_t n_rows);

#ifdef __cplusplus
}
#endif
#endif /* GORGONIA_B200_H */
