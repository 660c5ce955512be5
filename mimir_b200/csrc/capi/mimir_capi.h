/* C ABI over the framework's objects: tensors, parameters, modules, optimizers and meshes as
 * opaque handles, every tensor operation reachable by name, errors as values.  Plain C types
 * only (no structs by value, no callbacks), so the same symbols load through dlopen from C, through
 * ctypes from Python and through purego from Go without cgo (bindings/go/mimir.go mirrors this file).
 *
 * A handle is a positive 64-bit integer; 0 is failure and mimir_capi_last_error() says why.  A tensor
 * handle can carry a sticky error instead of a value (mimir_tensor_error): a bad operation does not
 * fail its call, and everything computed from its result carries the error too.
 *
 * Threading: every entry point takes the interpreter lock for the length of the call; calls from
 * several threads are serialised, device work they queue is not. */
#ifndef MIMIR_CAPI_H
#define MIMIR_CAPI_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef int64_t mimir_handle;

/* Starts the embedded interpreter (or attaches to the one already running in this process) and
 * imports the package.  package_root: directory that contains the mimir_b200 package, or NULL when it
 * is already importable.  Returns 0 on success. */
int mimir_capi_init(const char* package_root);
const char* mimir_capi_last_error(void);

/* dtype "f32" or "i64"; device "cpu", "gpu", "gpu:N" or "default".  The data is copied. */
mimir_handle mimir_tensor_from(const void* data, const int64_t* dims, int rank, const char* dtype, const char* device);
/* name: "T.<op>", "nn.<Layer>", "loss.<fn>", "forward", "parameters", "value", "grad", "item", "len";
 * kwargs_json: keyword arguments as a JSON object, or NULL.  For "len" the result is the count. */
mimir_handle mimir_call(const char* name, const mimir_handle* args, int nargs, const char* kwargs_json);
int mimir_tensor_rank(mimir_handle t);
int mimir_tensor_dims(mimir_handle t, int64_t* out, int cap);
/* 0: the tensor carries no error; otherwise the length of the message copied into buf. */
int mimir_tensor_error(mimir_handle t, char* buf, int cap);
/* Realizes the tensor and copies it as float32; returns the element count or -1. */
int64_t mimir_tensor_read_f32(mimir_handle t, float* out, int64_t cap);
int mimir_backward(mimir_handle loss);
mimir_handle mimir_optimizer(const char* kind, mimir_handle module, double lr, const char* kwargs_json);
int mimir_optimizer_step(mimir_handle opt, int zero_grad_after);
mimir_handle mimir_mesh(const int64_t* shape, const char* const* axes, int naxes);
int mimir_release(mimir_handle h);

#ifdef __cplusplus
}
#endif
#endif
