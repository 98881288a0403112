// +build cuda

package cuda

/*
#include "gorgonia_b200.h"
*/
import "C"

import (
	"unsafe"

	"github.com/pkg/errors"
	"gorgonia.org/tensor"
)

// MatMul, MatVecMul, Outer: cuda/linalg.go:47-285. Row-major is the one layout; the transposes that
// linAlgBinOp.CUDADo expresses as lazy T() views (op_math_cuda.go:210-224) arrive here as the views'
// own flags and become the trans arguments of the C entry point, so the eight {row,col} x
// {transA,transB} cases of the reference collapse into one call.

func boolInt(b bool) C.int {
	if b {
		return 1
	}
	return 0
}

// MatMul: prealloc = op(a) . op(b), float32 as 3xTF32 on the tensor cores, float64 on CUDA cores.
func (e *Engine) MatMul(a, b, prealloc tensor.Tensor) error {
	ad, bd, pd, err := e.checkThreeFloat(a, b, prealloc) // cuda/linalg.go:17-44, unchanged
	if err != nil {
		return errors.Wrap(err, "MatMul failed pre check")
	}
	tA, tB := ad.IsTransposed(), bd.IsTransposed() // the views' flags; the data is untouched
	m, k, n := ad.Shape()[0], ad.Shape()[1], bd.Shape()[1]
	lda, ldb := k, n // elements between rows of the STORED matrices
	if tA {
		lda = m
	}
	if tB {
		ldb = k
	}
	rc := C.b200_gemm(e.h, dtypeCode(ad.Dtype()), boolInt(tA), boolInt(tB), C.int64_t(m), C.int64_t(n), C.int64_t(k),
		unsafe.Pointer(ad.Uintptr()), C.int64_t(lda), unsafe.Pointer(bd.Uintptr()), C.int64_t(ldb),
		unsafe.Pointer(pd.Uintptr()), C.int64_t(n), 1, 0, 0, 0, nil)
	return e.err(rc, "MatMul")
}

// MatVecMul: prealloc = a . b or a^T . b.
func (e *Engine) MatVecMul(a, b, prealloc tensor.Tensor) error {
	ad, bd, pd, err := e.checkThreeFloat(a, b, prealloc)
	if err != nil {
		return errors.Wrap(err, "MatVecMul failed pre check")
	}
	tA := ad.IsTransposed()
	m, n := ad.Shape()[0], ad.Shape()[1]
	if tA { // the stored matrix is n x m
		m, n = n, m
	}
	rc := C.b200_gemv(e.h, dtypeCode(ad.Dtype()), boolInt(tA), C.int64_t(m), C.int64_t(n),
		unsafe.Pointer(ad.Uintptr()), C.int64_t(n), unsafe.Pointer(bd.Uintptr()), unsafe.Pointer(pd.Uintptr()))
	return e.err(rc, "MatVecMul")
}

// Outer: prealloc = a b^T, overwriting prealloc (what tensor.Outer with a reuse tensor does; the
// reference's cuBLAS path accumulates for lack of a beta: cuda/linalg.go:276,282).
func (e *Engine) Outer(a, b, prealloc tensor.Tensor) error {
	ad, bd, pd, err := e.checkThreeFloat(a, b, prealloc)
	if err != nil {
		return errors.Wrap(err, "Outer failed pre check")
	}
	rc := C.b200_ger(e.h, dtypeCode(ad.Dtype()), C.int64_t(ad.Size()), C.int64_t(bd.Size()),
		unsafe.Pointer(ad.Uintptr()), unsafe.Pointer(bd.Uintptr()), unsafe.Pointer(pd.Uintptr()))
	return e.err(rc, "Outer")
}

// BatchedMatMul: batchedMatMul (operatorLinAlg.go:435-502) as ONE launch instead of a loop of MatMuls.
func (e *Engine) BatchedMatMul(a, b, prealloc tensor.Tensor, transA, transB bool) error {
	as, bs := a.Shape(), b.Shape()
	d := as.Dims()
	batch := 1
	for _, v := range as[:d-2] {
		batch *= v
	}
	ar, ac, br, bc := as[d-2], as[d-1], bs[d-2], bs[d-1]
	m, k := ar, ac
	if transA {
		m, k = ac, ar
	}
	n := bc
	if transB {
		n = br
	}
	rc := C.b200_gemm(e.h, dtypeCode(a.Dtype()), boolInt(transA), boolInt(transB), C.int64_t(m), C.int64_t(n),
		C.int64_t(k), unsafe.Pointer(a.Uintptr()), C.int64_t(ac), unsafe.Pointer(b.Uintptr()), C.int64_t(bc),
		unsafe.Pointer(prealloc.Uintptr()), C.int64_t(n), C.int64_t(batch), C.int64_t(ar*ac), C.int64_t(br*bc),
		C.int64_t(m*n), nil)
	return e.err(rc, "BatchedMatMul")
}
