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

// The twelve binary methods of cuda/arith.go:14-701 and cuda/cmp.go:14-701 and their *Scalar forms.
// In the reference each is ~55 generated lines that differ in a kernel name; here each is one line
// over two helpers, because the op is an argument of the C entry point. Semantics kept: a reuse
// tensor or unsafe, never safe or incr (cuda/arith.go:34-49); the compare ops write 1.0 / 0.0 in the
// operand dtype (elembinop.cu:51-67). With a reuse tensor the reference copies a into it and then
// works in place; the kernel here is out of place, so that copy disappears.

func (e *Engine) binary(op C.int, name string, a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	if err := binaryCheck(a, b); err != nil { // cuda/utils.go:58-91
		return nil, errors.Wrapf(err, "Basic checks failed for %s", name)
	}
	reuse, safe, toReuse, _, _, err := handleFuncOpts(a.Shape(), a.Dtype(), a.DataOrder(), true, opts...)
	if err != nil {
		return nil, errors.Wrap(err, "Unable to handle funcOpts")
	}
	var dst tensor.Tensor
	switch {
	case toReuse:
		dst = reuse
	case !safe:
		dst = a
	default:
		return nil, errors.New("Impossible state: A reuse tensor must be passed in, or the operation must be unsafe. Incr and safe operations are not supported")
	}
	rc := C.b200_binary(e.h, op, dtypeCode(a.Dtype()), C.B200_VV, unsafe.Pointer(dst.Uintptr()),
		unsafe.Pointer(a.Uintptr()), unsafe.Pointer(b.Uintptr()), 0, 0, C.int64_t(logicalSize(a.Shape())))
	return dst, e.err(rc, name)
}

// b is a device scalar (tensor.Memory), as in the reference (cuda/arith.go:73-77, values.go:150-160).
func (e *Engine) binaryScalar(op C.int, name string, a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	if err := unaryCheck(a); err != nil { // cuda/utils.go:93-105
		return nil, errors.Wrapf(err, "Basic checks failed for %s", name)
	}
	sc, ok := b.(tensor.Memory)
	if !ok {
		return nil, errors.Errorf("b has to be a tensor.Memory. Got %T instead", b)
	}
	reuse, safe, toReuse, _, _, err := handleFuncOpts(a.Shape(), a.Dtype(), a.DataOrder(), true, opts...)
	if err != nil {
		return nil, errors.Wrap(err, "Unable to handle funcOpts")
	}
	var dst tensor.Tensor
	switch {
	case toReuse:
		dst = reuse
	case !safe:
		dst = a
	default:
		return nil, errors.New("Impossible state: A reuse tensor must be passed in, or the operation must be unsafe. Incr and safe operations are not supported")
	}
	form, pa, pb := C.int(C.B200_VS), a.Uintptr(), sc.Uintptr()
	if !leftTensor { // scalar op tensor, written over the tensor's buffer (cuda/arith.go:109-112)
		form, pa, pb = C.B200_SV, pb, pa
	}
	rc := C.b200_binary(e.h, op, dtypeCode(a.Dtype()), form, unsafe.Pointer(dst.Uintptr()), unsafe.Pointer(pa),
		unsafe.Pointer(pb), 0, 1, C.int64_t(logicalSize(a.Shape())))
	return dst, e.err(rc, name)
}

func (e *Engine) Add(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_ADD, "Add", a, b, opts...)
}
func (e *Engine) Sub(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_SUB, "Sub", a, b, opts...)
}
func (e *Engine) Mul(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_MUL, "Mul", a, b, opts...)
}
func (e *Engine) Div(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_DIV, "Div", a, b, opts...)
}
func (e *Engine) Pow(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_POW, "Pow", a, b, opts...)
}
func (e *Engine) Mod(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_MOD, "Mod", a, b, opts...)
}
func (e *Engine) Lt(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_LT, "Lt", a, b, opts...)
}
func (e *Engine) Lte(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_LTE, "Lte", a, b, opts...)
}
func (e *Engine) Gt(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_GT, "Gt", a, b, opts...)
}
func (e *Engine) Gte(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_GTE, "Gte", a, b, opts...)
}
func (e *Engine) ElEq(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_EQ, "ElEq", a, b, opts...)
}
func (e *Engine) ElNe(a, b tensor.Tensor, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binary(C.B200_OP_NE, "ElNe", a, b, opts...)
}

func (e *Engine) AddScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_ADD, "AddScalar", a, b, leftTensor, opts...)
}
func (e *Engine) SubScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_SUB, "SubScalar", a, b, leftTensor, opts...)
}
func (e *Engine) MulScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_MUL, "MulScalar", a, b, leftTensor, opts...)
}
func (e *Engine) DivScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_DIV, "DivScalar", a, b, leftTensor, opts...)
}
func (e *Engine) PowScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_POW, "PowScalar", a, b, leftTensor, opts...)
}
func (e *Engine) ModScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_MOD, "ModScalar", a, b, leftTensor, opts...)
}
func (e *Engine) LtScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_LT, "LtScalar", a, b, leftTensor, opts...)
}
func (e *Engine) LteScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_LTE, "LteScalar", a, b, leftTensor, opts...)
}
func (e *Engine) GtScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_GT, "GtScalar", a, b, leftTensor, opts...)
}
func (e *Engine) GteScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_GTE, "GteScalar", a, b, leftTensor, opts...)
}
func (e *Engine) EqScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_EQ, "EqScalar", a, b, leftTensor, opts...)
}
func (e *Engine) NeScalar(a tensor.Tensor, b interface{}, leftTensor bool, opts ...tensor.FuncOpt) (tensor.Tensor, error) {
	return e.binaryScalar(C.B200_OP_NE, "NeScalar", a, b, leftTensor, opts...)
}

// Unary runs one of the twenty unary ops in place or into prealloc (elemUnaryOp.CUDADo,
// op_math_cuda.go:23-85, whose kernel-name lookup and CPU fallback go away: every op of
// ʘUnaryOperatorType has a device implementation, B200_OP_ABS .. B200_OP_SOFTPLUS in that order).
func (e *Engine) Unary(opType int, a, prealloc tensor.Tensor) error {
	rc := C.b200_unary(e.h, C.int(C.B200_OP_ABS+opType), dtypeCode(a.Dtype()), unsafe.Pointer(prealloc.Uintptr()),
		unsafe.Pointer(a.Uintptr()), C.int64_t(logicalSize(a.Shape())))
	return e.err(rc, "Unary")
}

// Incr is ExternalOp.Do's Incr mode (execution.go:113-127): incr += a op b in one fused kernel.
func (e *Engine) Incr(op C.int, a, b, incr tensor.Tensor) error {
	rc := C.b200_binary_incr(e.h, op, dtypeCode(a.Dtype()), C.B200_VV, unsafe.Pointer(incr.Uintptr()),
		unsafe.Pointer(a.Uintptr()), unsafe.Pointer(b.Uintptr()), 0, 0, C.int64_t(logicalSize(a.Shape())))
	return e.err(rc, "Incr")
}
