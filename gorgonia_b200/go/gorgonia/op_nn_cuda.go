// +build cuda

package gorgonia

/*
#cgo CFLAGS: -I${SRCDIR}/../../../include
#cgo LDFLAGS: -L${SRCDIR}/../.. -lgorgonia_b200
#include "gorgonia_b200.h"
*/
import "C"

import (
	"unsafe"

	"github.com/pkg/errors"
	"gorgonia.org/tensor"
)

// CUDADo methods for the ops that the reference runs on the CPU only (op_nn.go, op_softmax.go,
// op_tensor.go, op_by_indices.go, op_dropout.go). With them the compiler keeps whole forward tapes on
// the device: it places an op on the GPU iff the op is a CUDADoer (analysis.go:52-65). Each method is
// the shape of elemBinOp.CUDADo (op_math_cuda.go:89-176): take the engine of `dev`, call one C entry
// point on the operands' device memory, return prealloc.

func b200Handle(extern External, dev Device) *C.b200_engine {
	e := extern.(CUDAMachine).Engines()[int(dev)]
	return (*C.b200_engine)(e.Handle())
}

func b200Err(h *C.b200_engine, rc C.int, what string) error {
	if rc == C.B200_OK {
		return nil
	}
	return errors.Errorf("%s: %s", what, C.GoString(C.b200_last_error(h)))
}

func b200Dtype(t tensor.Tensor) C.int {
	if t.Dtype() == tensor.Float64 {
		return C.B200_F64
	}
	return C.B200_F32
}

func devPtr(v Value) unsafe.Pointer { return unsafe.Pointer(v.(tensor.Tensor).Uintptr()) }

// im2colOp (op_nn.go:317-444).
func (op im2colOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	im := inputs[0].(tensor.Tensor)
	s := im.Shape()
	h := b200Handle(extern, dev)
	rc := C.b200_im2col(h, b200Dtype(im), devPtr(inputs[0]), devPtr(prealloc), C.int64_t(s[0]), C.int64_t(s[1]),
		C.int64_t(s[2]), C.int64_t(s[3]), C.int(op.h), C.int(op.w), C.int(op.padH), C.int(op.padW),
		C.int(op.strideH), C.int(op.strideW), C.int(op.dilationH), C.int(op.dilationW))
	return prealloc, b200Err(h, rc, "Im2Col")
}

// maxPoolOp (op_nn.go:828-907); the mask lives on the device as int64 for maxPoolDiffOp.
func (op *maxPoolOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in := inputs[0].(tensor.Tensor)
	s := in.Shape()
	h := b200Handle(extern, dev)
	rc := C.b200_maxpool2d_fwd(h, b200Dtype(in), devPtr(inputs[0]), devPtr(prealloc),
		(*C.int64_t)(unsafe.Pointer(op.mask.Uintptr())), C.int64_t(s[0]), C.int64_t(s[1]), C.int64_t(s[2]),
		C.int64_t(s[3]), C.int(op.h), C.int(op.w), C.int(op.padNorth), C.int(op.padSouth), C.int(op.padWest),
		C.int(op.padEast), boolC(op.explicitPadding), C.int(op.strideH), C.int(op.strideW))
	return prealloc, b200Err(h, rc, "MaxPool2D")
}

// maxPoolDiffOp (op_nn.go:958-1121): inputs are (in, pooled, pooledGrad) as in maxPoolDiffOp.Do.
func (op *maxPoolDiffOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in := inputs[0].(tensor.Tensor)
	s := in.Shape()
	h := b200Handle(extern, dev)
	rc := C.b200_maxpool2d_bwd(h, b200Dtype(in), devPtr(inputs[2]), (*C.int64_t)(unsafe.Pointer(op.mask.Uintptr())),
		devPtr(prealloc), C.int64_t(s[0]), C.int64_t(s[1]), C.int64_t(s[2]), C.int64_t(s[3]), C.int(op.h), C.int(op.w),
		C.int(op.padNorth), C.int(op.padSouth), C.int(op.padWest), C.int(op.padEast), boolC(op.explicitPadding),
		C.int(op.strideH), C.int(op.strideW))
	return prealloc, b200Err(h, rc, "MaxPoolDiff")
}

// col2imOp (op_nn.go:446-637).
func (op col2imOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	im := prealloc.(tensor.Tensor)
	s := im.Shape()
	h := b200Handle(extern, dev)
	rc := C.b200_col2im(h, b200Dtype(im), devPtr(inputs[0]), devPtr(prealloc), C.int64_t(s[0]), C.int64_t(s[1]),
		C.int64_t(s[2]), C.int64_t(s[3]), C.int(op.h), C.int(op.w), C.int(op.padH), C.int(op.padW), C.int(op.strideH),
		C.int(op.strideW), C.int(op.dilationH), C.int(op.dilationW))
	return prealloc, b200Err(h, rc, "Col2Im")
}

// softmaxOp (op_softmax.go:99-128) and softmaxDiffOp (op_softmax.go:180-285).
func (op *softmaxOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in := inputs[0].(tensor.Tensor)
	outer, length, inner := splitAxis(in.Shape(), op.axis)
	h := b200Handle(extern, dev)
	rc := C.b200_softmax(h, b200Dtype(in), devPtr(inputs[0]), devPtr(prealloc), C.int64_t(outer), C.int64_t(length),
		C.int64_t(inner), boolC(op.isLog))
	return prealloc, b200Err(h, rc, "SoftMax")
}
func (op *softmaxDiffOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	y := inputs[0].(tensor.Tensor)
	outer, length, inner := splitAxis(y.Shape(), op.axis)
	h := b200Handle(extern, dev)
	rc := C.b200_softmax_bwd(h, b200Dtype(y), devPtr(inputs[0]), devPtr(inputs[1]), devPtr(prealloc), C.int64_t(outer),
		C.int64_t(length), C.int64_t(inner), boolC(op.isLog))
	return prealloc, b200Err(h, rc, "SoftMaxDiff")
}

// byIndicesOp (op_by_indices.go:90-97); the indices are an int64 device vector.
func (op *byIndicesOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in, idx := inputs[0].(tensor.Tensor), inputs[1].(tensor.Tensor)
	outer, rows, inner := splitAxis(in.Shape(), op.axis)
	h := b200Handle(extern, dev)
	rc := C.b200_gather_axis(h, devPtr(inputs[0]), (*C.int64_t)(unsafe.Pointer(idx.Uintptr())), devPtr(prealloc),
		C.int64_t(outer), C.int64_t(rows), C.int64_t(idx.Size()), C.int64_t(inner*int(in.Dtype().Size())))
	return prealloc, b200Err(h, rc, "ByIndices")
}

// transposeOp (op_tensor.go:937-952).
func (op transposeOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in := inputs[0].(tensor.Tensor)
	shape := make([]C.int64_t, in.Dims())
	perm := make([]C.int, in.Dims())
	for i, v := range in.Shape() {
		shape[i] = C.int64_t(v)
		perm[i] = C.int(op.pattern[i])
	}
	h := b200Handle(extern, dev)
	rc := C.b200_transpose(h, C.int(in.Dtype().Size()), devPtr(inputs[0]), devPtr(prealloc), C.int(in.Dims()),
		&shape[0], &perm[0])
	return prealloc, b200Err(h, rc, "Transpose")
}

// dropoutOp (op_dropout.go:106-128): stateless Philox keyed by a seed the op holds; `drawn` counts the
// elements drawn so far, so that successive runs continue one stream.
func (op *dropoutOp) CUDADo(extern External, dev Device, prealloc Value, inputs ...Value) (Value, error) {
	in := inputs[0].(tensor.Tensor)
	if op.probability == 0.0 || !op.isTraining {
		return inputs[0], nil
	}
	n := in.Shape().TotalSize()
	h := b200Handle(extern, dev)
	rc := C.b200_dropout_fwd(h, b200Dtype(in), devPtr(inputs[0]), devPtr(prealloc), C.int64_t(n),
		C.double(op.probability), nil, C.uint64_t(op.seed), C.uint64_t(op.drawn))
	op.drawn += uint64(n)
	return prealloc, b200Err(h, rc, "Dropout")
}

func boolC(b bool) C.int {
	if b {
		return 1
	}
	return 0
}

// splitAxis views a shape as (outer, shape[axis], inner).
func splitAxis(s tensor.Shape, axis int) (outer, length, inner int) {
	outer, inner = 1, 1
	for i, v := range s {
		switch {
		case i < axis:
			outer *= v
		case i > axis:
			inner *= v
		}
	}
	return outer, s[axis], inner
}
