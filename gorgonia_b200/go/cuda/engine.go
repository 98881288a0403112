// +build cuda

// Package cuda: gorgonia's CUDA engine on top of libgorgonia_b200.so.
//
// Replaces engine.go, external.go and arena.go of gorgonia's cuda package. The exported method set is
// unchanged (cuda/engine.go:17-35 lists the interfaces it implements); what is behind it shrinks to one
// handle: no cu.BatchedContext, no module table, no worker goroutine locked to an OS thread
// (cuda/external.go:229-276). A call through the C ABI is an ordinary function call from whatever
// thread runs the tape.
package cuda

/*
#cgo CFLAGS: -I${SRCDIR}/../../../include
#cgo LDFLAGS: -L${SRCDIR}/../.. -lgorgonia_b200
#include <stdlib.h>
#include "gorgonia_b200.h"
*/
import "C"

import (
	"sync"
	"unsafe"

	"github.com/pkg/errors"
	"gorgonia.org/tensor"
)

var (
	_ tensor.Adder       = &Engine{}
	_ tensor.Suber       = &Engine{}
	_ tensor.Muler       = &Engine{}
	_ tensor.Diver       = &Engine{}
	_ tensor.Power       = &Engine{}
	_ tensor.Moder       = &Engine{}
	_ tensor.Lter        = &Engine{}
	_ tensor.Lteer       = &Engine{}
	_ tensor.Gter        = &Engine{}
	_ tensor.Gteer       = &Engine{}
	_ tensor.ElEqer      = &Engine{}
	_ tensor.MatMuler    = &Engine{}
	_ tensor.MatVecMuler = &Engine{}
	_ tensor.OuterProder = &Engine{}
	_ tensor.Engine      = &Engine{}
)

// Memory is a device address handed out by the arena (the role cu.DevicePtr plays in the reference).
type Memory uintptr

func (m Memory) Uintptr() uintptr        { return uintptr(m) }
func (m Memory) MemSize() uintptr        { return 0 }
func (m Memory) Pointer() unsafe.Pointer { return unsafe.Pointer(uintptr(m)) }

// Engine is a CUDA engine (cuda/engine.go:38-69).
type Engine struct {
	tensor.Engine
	sync.Mutex

	h           *C.b200_engine
	device      int
	initialized bool
}

func (e *Engine) err(rc C.int, what string) error {
	switch rc {
	case C.B200_OK:
		return nil
	case C.B200_ERR_OOM:
		return oomError{} // cuda/errors.go:5-13
	default:
		return errors.Errorf("%s: %s", what, C.GoString(C.b200_last_error(e.h)))
	}
}

// Init creates the engine on a device with an arena of `size` bytes (cuda/external.go:88-170): the
// reference asks for 2.5x the bytes the compiler counted plus 256; the caller passes that figure. The
// arena is CUDA managed memory with its preferred location on the device, because gorgonia reads
// device values from Go (values.go:150-160, vm_tape_cuda.go:139-150).
func (e *Engine) Init(device int, size int64) error {
	e.Lock()
	defer e.Unlock()
	if e.initialized {
		return nil
	}
	rc := C.b200_engine_create(C.int(device), C.size_t(size), C.B200_ENGINE_MANAGED, &e.h)
	if rc != C.B200_OK {
		return errors.Errorf("Init: %s", C.GoString(C.b200_last_error(nil)))
	}
	e.device = device
	e.initialized = true
	return nil
}

// Close releases the engine (cuda/external.go:172-220).
func (e *Engine) Close() error {
	e.Lock()
	defer e.Unlock()
	if !e.initialized {
		return nil
	}
	rc := C.b200_engine_destroy(e.h)
	e.h, e.initialized = nil, false
	if rc != C.B200_OK {
		return errors.New("Close: b200_engine_destroy failed")
	}
	return nil
}

// DoWork launches whatever the deferred queue holds (cuda/external.go:223-226).
func (e *Engine) DoWork() error { return e.err(C.b200_flush(e.h), "DoWork") }

// Signal flushes and waits for the device (cuda/external.go:46-50); Sync returns a closed channel,
// because nothing runs asynchronously to the caller any more.
func (e *Engine) Signal() { C.b200_sync(e.h) }
func (e *Engine) Sync() chan struct{} {
	C.b200_sync(e.h)
	ch := make(chan struct{})
	close(ch)
	return ch
}

// Errors reports asynchronous failures, among them a bounded device wait that ran out.
func (e *Engine) Errors() error { return e.err(C.b200_sync(e.h), "Errors") }

/* arena: cuda/arena.go:13-36 */

// Get allocates from the arena.
func (e *Engine) Get(size int64) (tensor.Memory, error) {
	var p unsafe.Pointer
	if err := e.err(C.b200_get(e.h, C.int64_t(size), &p), "Get"); err != nil {
		return nil, err
	}
	return Memory(uintptr(p)), nil
}

// Put hands memory back; the size is ignored, as in the reference.
func (e *Engine) Put(mem tensor.Memory, size int64) {
	C.b200_put(e.h, unsafe.Pointer(mem.Uintptr()), C.int64_t(size))
}

// ResetAllocator frees everything. Tapes recorded before it refuse to launch afterwards.
func (e *Engine) ResetAllocator() { C.b200_reset(e.h) }

/* tensor.Engine plumbing: cuda/engine.go:71-138 */

func (e *Engine) AllocAccessible() bool { return true }
func (e *Engine) Alloc(size int64) (tensor.Memory, error) { return e.Get(size) }
func (e *Engine) AllocFlags() (tensor.MemoryFlag, tensor.DataOrder) {
	// row-major is the one layout of this engine (the reference flags ColMajor although the data it
	// copies in is row-major: cuda/engine.go:81-83)
	return tensor.MakeMemoryFlag(tensor.ManuallyManaged), tensor.DataOrder(0)
}
func (e *Engine) Free(mem tensor.Memory, size int64) error { e.Put(mem, size); return nil }
func (e *Engine) Memset(mem tensor.Memory, val interface{}) error {
	return errors.New("Memset is not implemented: use b200_memset for byte patterns")
}
func (e *Engine) Memclr(mem tensor.Memory) {
	C.b200_memset(e.h, unsafe.Pointer(mem.Uintptr()), 0, C.int64_t(mem.MemSize()))
}
func (e *Engine) Memcpy(dst, src tensor.Memory) error {
	size := dst.MemSize()
	if src.MemSize() < size {
		size = src.MemSize()
	}
	rc := C.b200_memcpy_d2d(e.h, unsafe.Pointer(dst.Uintptr()), unsafe.Pointer(src.Uintptr()), C.int64_t(size))
	return e.err(rc, "Memcpy")
}
func (e *Engine) Accessible(mem tensor.Memory) (tensor.Memory, error) { return mem, nil }
func (e *Engine) WorksWith(order tensor.DataOrder) bool              { return !order.IsColMajor() }
func (e *Engine) NonStdAlloc()                                       {}

// Transfer moves bytes between host and device (ExternMetadata.Transfer, cuda.go:168-207;
// deviceTransport.exec, vm_tape_cuda.go:220-243).
func (e *Engine) Transfer(dst, src unsafe.Pointer, bytes int64, toDevice bool) error {
	if toDevice {
		return e.err(C.b200_memcpy_h2d(e.h, dst, src, C.int64_t(bytes)), "Transfer")
	}
	return e.err(C.b200_memcpy_d2h(e.h, dst, src, C.int64_t(bytes)), "Transfer")
}

// HasNaN / HasInf (cuda/engine.go:144-191).
func (e *Engine) HasNaN(a tensor.Tensor) (bool, error) {
	var r C.int
	rc := C.b200_has_nan(e.h, dtypeCode(a.Dtype()), unsafe.Pointer(a.Uintptr()), C.int64_t(logicalSize(a.Shape())), &r)
	return r != 0, e.err(rc, "HasNaN")
}
func (e *Engine) HasInf(a tensor.Tensor) (bool, error) {
	var r C.int
	rc := C.b200_has_inf(e.h, dtypeCode(a.Dtype()), unsafe.Pointer(a.Uintptr()), C.int64_t(logicalSize(a.Shape())), &r)
	return r != 0, e.err(rc, "HasInf")
}

func dtypeCode(dt tensor.Dtype) C.int {
	switch dt {
	case tensor.Float32:
		return C.B200_F32
	case tensor.Float64:
		return C.B200_F64
	}
	return -1 // refused by the library: B200_ERR_INVALID
}

// Handle exposes the C handle to package gorgonia's CUDADo methods.
func (e *Engine) Handle() unsafe.Pointer { return unsafe.Pointer(e.h) }
