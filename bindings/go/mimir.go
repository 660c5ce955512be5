// Package mimir drives the framework from Go without cgo: the C ABI of libmimir_capi.so
// (mimir_b200/csrc/capi/mimir_capi.h) is loaded with purego, exactly as the reference loads its
// native libraries (backend/cuda/driver_linux.go:105-150).  Every function below is a one-to-one
// mirror of a C entry point; handles are int64, errors are values.
//
// Build: needs github.com/ebitengine/purego in the module cache.  Run with LD_LIBRARY_PATH
// containing the directory of libpython and PYTHONPATH containing the package root and the
// interpreter's site-packages (the shim embeds the interpreter).
package mimir

import (
	"errors"
	"unsafe"

	"github.com/ebitengine/purego"
)

// Handle names a tensor, parameter, module, optimizer, list or mesh inside the framework.
type Handle int64

var (
	capiInit        func(root string) int32
	capiLastError   func() string
	tensorFrom      func(data unsafe.Pointer, dims *int64, rank int32, dtype, device string) int64
	call            func(name string, args *int64, n int32, kwargs string) int64
	tensorDims      func(t int64, out *int64, cap int32) int32
	tensorError     func(t int64, buf *byte, cap int32) int32
	tensorReadF32   func(t int64, out *float32, cap int64) int64
	backward        func(loss int64) int32
	optimizer       func(kind string, module int64, lr float64, kwargs string) int64
	optimizerStep   func(opt int64, zero int32) int32
	release         func(h int64) int32
)

// Open loads the library at path (libmimir_capi.so) and starts the framework; root is the directory
// that contains the mimir_b200 package ("" when it is already importable).
func Open(path, root string) error {
	lib, err := purego.Dlopen(path, purego.RTLD_NOW|purego.RTLD_GLOBAL)
	if err != nil {
		return err
	}
	purego.RegisterLibFunc(&capiInit, lib, "mimir_capi_init")
	purego.RegisterLibFunc(&capiLastError, lib, "mimir_capi_last_error")
	purego.RegisterLibFunc(&tensorFrom, lib, "mimir_tensor_from")
	purego.RegisterLibFunc(&call, lib, "mimir_call")
	purego.RegisterLibFunc(&tensorDims, lib, "mimir_tensor_dims")
	purego.RegisterLibFunc(&tensorError, lib, "mimir_tensor_error")
	purego.RegisterLibFunc(&tensorReadF32, lib, "mimir_tensor_read_f32")
	purego.RegisterLibFunc(&backward, lib, "mimir_backward")
	purego.RegisterLibFunc(&optimizer, lib, "mimir_optimizer")
	purego.RegisterLibFunc(&optimizerStep, lib, "mimir_optimizer_step")
	purego.RegisterLibFunc(&release, lib, "mimir_release")
	if capiInit(root) != 0 {
		return errors.New(capiLastError())
	}
	return nil
}

func lastErr() error { return errors.New(capiLastError()) }

// FromFloat32 copies data into a new tensor of the given shape on device ("cpu", "gpu", "gpu:N").
func FromFloat32(data []float32, device string, dims ...int64) (Handle, error) {
	var p unsafe.Pointer
	if len(data) > 0 {
		p = unsafe.Pointer(&data[0])
	}
	var d *int64
	if len(dims) > 0 {
		d = &dims[0]
	}
	h := tensorFrom(p, d, int32(len(dims)), "f32", device)
	if h == 0 {
		return 0, lastErr()
	}
	return Handle(h), nil
}

// Call runs an entry point by name ("T.matmul", "nn.Linear", "loss.mse", "forward", "parameters", ...)
// with handle arguments and keyword arguments as a JSON object ("" for none).
func Call(name, kwargs string, args ...Handle) (Handle, error) {
	var p *int64
	if len(args) > 0 {
		p = (*int64)(unsafe.Pointer(&args[0]))
	}
	h := call(name, p, int32(len(args)), kwargs)
	if h == 0 {
		return 0, lastErr()
	}
	return Handle(h), nil
}

// Err returns the sticky error a tensor carries, or nil.
func (t Handle) Err() error {
	buf := make([]byte, 512)
	n := tensorError(int64(t), &buf[0], int32(len(buf)))
	if n == 0 {
		return nil
	}
	if n < 0 {
		return lastErr()
	}
	if int(n) > len(buf)-1 {
		n = int32(len(buf) - 1)
	}
	return errors.New(string(buf[:n]))
}

// Shape returns the dimensions of a tensor.
func (t Handle) Shape() ([]int64, error) {
	out := make([]int64, 8)
	r := tensorDims(int64(t), &out[0], 8)
	if r < 0 {
		return nil, lastErr()
	}
	return out[:r], nil
}

// Float32 realizes the tensor and returns its values.
func (t Handle) Float32() ([]float32, error) {
	shape, err := t.Shape()
	if err != nil {
		return nil, err
	}
	n := int64(1)
	for _, s := range shape {
		n *= s
	}
	out := make([]float32, max(n, 1))
	got := tensorReadF32(int64(t), &out[0], n)
	if got < 0 {
		return nil, lastErr()
	}
	return out[:got], nil
}

// Backward computes the loss and accumulates every parameter's gradient.
func (t Handle) Backward() error {
	if backward(int64(t)) != 0 {
		return lastErr()
	}
	return nil
}

// Optimizer makes an optimizer ("SGD", "AdamW", ...) over a module's parameters.
func Optimizer(kind string, module Handle, lr float64, kwargs string) (Handle, error) {
	h := optimizer(kind, int64(module), lr, kwargs)
	if h == 0 {
		return 0, lastErr()
	}
	return Handle(h), nil
}

// Step applies one update and clears the gradients.
func (o Handle) Step() error {
	if optimizerStep(int64(o), 1) != 0 {
		return lastErr()
	}
	return nil
}

// Release drops the framework's reference to the object.
func (h Handle) Release() { release(int64(h)) }
