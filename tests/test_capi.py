"""The C ABI over framework objects (csrc/capi/mimir_capi.h): driven once through ctypes inside this
process (the shim attaches to the running interpreter) and once from a C program with no Python
of its own, which is how a Go program reaches it through purego (bindings/go/mimir.go)."""
import ctypes
import os
import subprocess
import sys
import sysconfig

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "mimir_b200", "_native", "libmimir_capi.so")


def _lib():
    from mimir_b200._native import build
    build.build_capi()
    L = ctypes.CDLL(LIB)
    H, I, P, S = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p
    L.mimir_capi_init.argtypes, L.mimir_capi_init.restype = [S], I
    L.mimir_capi_last_error.restype = S
    L.mimir_tensor_from.argtypes, L.mimir_tensor_from.restype = [P, ctypes.POINTER(H), I, S, S], H
    L.mimir_call.argtypes, L.mimir_call.restype = [S, ctypes.POINTER(H), I, S], H
    L.mimir_tensor_dims.argtypes, L.mimir_tensor_dims.restype = [H, ctypes.POINTER(H), I], I
    L.mimir_tensor_error.argtypes, L.mimir_tensor_error.restype = [H, ctypes.c_char_p, I], I
    L.mimir_tensor_read_f32.argtypes, L.mimir_tensor_read_f32.restype = [H, ctypes.POINTER(ctypes.c_float), H], H
    L.mimir_backward.argtypes, L.mimir_backward.restype = [H], I
    L.mimir_optimizer.argtypes, L.mimir_optimizer.restype = [S, H, ctypes.c_double, S], H
    L.mimir_optimizer_step.argtypes, L.mimir_optimizer_step.restype = [H, I], I
    L.mimir_release.argtypes, L.mimir_release.restype = [H], I
    return L


def _tensor(L, values, dims):
    arr = (ctypes.c_float * len(values))(*values)
    d = (ctypes.c_int64 * len(dims))(*dims)
    return L.mimir_tensor_from(arr, d, len(dims), b"f32", b"cpu")


def _hs(*h):
    return (ctypes.c_int64 * len(h))(*h), len(h)


def test_tensors_ops_sticky_errors_and_training_through_the_c_abi():
    L = _lib()
    assert L.mimir_capi_init(ROOT.encode()) == 0, L.mimir_capi_last_error()
    a = _tensor(L, [1, 2, 3, 4, 5, 6], [2, 3])
    b = _tensor(L, [1, 0, 0, 1, 1, 1], [3, 2])
    c = L.mimir_call(b"T.matmul", *_hs(a, b), None)
    assert c > 0, L.mimir_capi_last_error()
    dims = (ctypes.c_int64 * 4)()
    assert L.mimir_tensor_dims(c, dims, 4) == 2 and list(dims[:2]) == [2, 2]
    out = (ctypes.c_float * 4)()
    assert L.mimir_tensor_read_f32(c, out, 4) == 4 and list(out) == [4.0, 5.0, 10.0, 11.0]
    # a shape error is a value: the call succeeds, the tensor carries the error, and so does what follows
    bad = L.mimir_call(b"T.matmul", *_hs(a, a), None)
    assert bad > 0
    buf = ctypes.create_string_buffer(256)
    assert L.mimir_tensor_error(bad, buf, 256) > 0 and b"ErrShape" in buf.value
    worse = L.mimir_call(b"T.relu", *_hs(bad), None)
    assert L.mimir_tensor_error(worse, buf, 256) > 0
    assert L.mimir_tensor_read_f32(worse, out, 4) == -1 and b"ErrShape" in L.mimir_capi_last_error()
    assert L.mimir_tensor_error(c, buf, 256) == 0
    # an unknown entry point and a dead handle fail the call itself
    assert L.mimir_call(b"T.no_such_op", *_hs(a), None) == 0 and b"no_such_op" in L.mimir_capi_last_error()
    assert L.mimir_release(c) == 0 and L.mimir_release(c) == -1
    # a module, a loss, backward and an optimizer step: the loss goes down
    lin = L.mimir_call(b"nn.Linear", None, 0, b'{"fan_in": 3, "fan_out": 1}')
    opt = L.mimir_optimizer(b"SGD", lin, 0.05, None)
    x = _tensor(L, [1, 2, 3, 2, 1, 0, 0, 1, 1, 3, 1, 2], [4, 3])
    y = _tensor(L, [6, 3, 2, 6], [4, 1])
    losses = []
    for _ in range(25):
        pred = L.mimir_call(b"forward", *_hs(lin, x), None)
        loss = L.mimir_call(b"loss.mse", *_hs(pred, y), None)
        assert L.mimir_backward(loss) == 0, L.mimir_capi_last_error()
        one = (ctypes.c_float * 1)()
        assert L.mimir_tensor_read_f32(loss, one, 1) == 1
        losses.append(one[0])
        assert L.mimir_optimizer_step(opt, 1) == 0
        L.mimir_release(pred), L.mimir_release(loss)
    assert losses[-1] < 0.1 * losses[0]
    params = L.mimir_call(b"parameters", *_hs(lin), None)
    assert L.mimir_call(b"len", *_hs(params), None) == 2


C_DRIVER = r"""
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
typedef int64_t H;
int main(int argc, char** argv) {
  void* so = dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL);
  if (!so) { printf("dlopen: %s\n", dlerror()); return 2; }
  int (*init)(const char*) = dlsym(so, "mimir_capi_init");
  const char* (*err)(void) = dlsym(so, "mimir_capi_last_error");
  H (*from)(const void*, const int64_t*, int, const char*, const char*) = dlsym(so, "mimir_tensor_from");
  H (*call)(const char*, const H*, int, const char*) = dlsym(so, "mimir_call");
  int64_t (*read)(H, float*, int64_t) = dlsym(so, "mimir_tensor_read_f32");
  if (init(argv[2])) { printf("init: %s\n", err()); return 3; }
  float a[4] = {1, 2, 3, 4};
  int64_t d[2] = {2, 2};
  H x = from(a, d, 2, "f32", "cpu");
  H hs[2] = {x, x};
  H y = call("T.matmul", hs, 2, 0);
  float out[4];
  if (!y || read(y, out, 4) != 4) { printf("call: %s\n", err()); return 4; }
  printf("%g %g %g %g\n", out[0], out[1], out[2], out[3]);
  return 0;
}
"""


def test_a_c_program_without_python_drives_the_framework(tmp_path):
    _lib()
    src, exe = tmp_path / "driver.c", tmp_path / "driver"
    src.write_text(C_DRIVER)
    cc = subprocess.run(["gcc", str(src), "-o", str(exe), "-ldl"], capture_output=True, text=True)
    if cc.returncode != 0:
        pytest.skip("no C toolchain: " + cc.stderr[-200:])
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + [p for p in sys.path if p]),
               LD_LIBRARY_PATH=sysconfig.get_config_var("LIBDIR") or "")
    out = subprocess.run([str(exe), LIB, ROOT], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.strip().splitlines()[-1] == "7 10 15 22"
