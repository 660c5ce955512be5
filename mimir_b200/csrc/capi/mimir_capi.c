/* See mimir_capi.h.  Every entry point forwards to a function of mimir_b200/capi.py with plain
 * arguments (integers, doubles, strings, tuples of integers) and turns the result back into C. */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <string.h>

#include "mimir_capi.h"

#define API __attribute__((visibility("default")))

static PyObject* g_mod = NULL;
static int g_we_started = 0;
static __thread char g_err[1024];

static void set_err(const char* msg) {
  strncpy(g_err, msg ? msg : "", sizeof(g_err) - 1);
  g_err[sizeof(g_err) - 1] = 0;
}

/* Copies the pending Python exception (if any) or capi.last_error() into the thread's buffer. */
static void take_error(void) {
  if (PyErr_Occurred()) {
    PyObject *t, *v, *tb;
    PyErr_Fetch(&t, &v, &tb);
    PyObject* s = v ? PyObject_Str(v) : NULL;
    set_err(s ? PyUnicode_AsUTF8(s) : "python error");
    Py_XDECREF(s); Py_XDECREF(t); Py_XDECREF(v); Py_XDECREF(tb);
    return;
  }
  if (g_mod) {
    PyObject* r = PyObject_CallMethod(g_mod, "last_error", NULL);
    if (r) { set_err(PyUnicode_AsUTF8(r)); Py_DECREF(r); } else PyErr_Clear();
  }
}

API const char* mimir_capi_last_error(void) { return g_err; }

API int mimir_capi_init(const char* package_root) {
  if (!Py_IsInitialized()) {
    Py_InitializeEx(0);
    g_we_started = 1;
    PyEval_SaveThread(); /* release the lock: every entry point takes it for itself */
  }
  PyGILState_STATE st = PyGILState_Ensure();
  int rc = 0;
  if (!g_mod) {
    if (package_root && package_root[0]) {
      PyObject* path = PySys_GetObject("path"); /* borrowed */
      PyObject* p = PyUnicode_FromString(package_root);
      if (path && p) PyList_Insert(path, 0, p);
      Py_XDECREF(p);
    }
    g_mod = PyImport_ImportModule("mimir_b200.capi");
    if (!g_mod) { take_error(); rc = -1; }
  }
  PyGILState_Release(st);
  return rc;
}

static PyObject* tuple_of_i64(const int64_t* v, int n) {
  PyObject* t = PyTuple_New(n);
  for (int i = 0; t && i < n; ++i) PyTuple_SET_ITEM(t, i, PyLong_FromLongLong(v[i]));
  return t;
}

/* Calls capi.<fn>(*args) and returns the result as int64 (handles, counts, status codes). */
static int64_t call_i64(const char* fn, PyObject* args, int64_t on_error) {
  if (!g_mod) { set_err("mimir_capi_init has not been called"); Py_XDECREF(args); return on_error; }
  PyObject* f = PyObject_GetAttrString(g_mod, fn);
  PyObject* r = f && args ? PyObject_CallObject(f, args) : NULL;
  Py_XDECREF(f); Py_XDECREF(args);
  if (!r) { take_error(); return on_error; }
  int64_t out = PyLong_AsLongLong(r);
  Py_DECREF(r);
  if (out == on_error) take_error();
  return out;
}

API mimir_handle mimir_tensor_from(const void* data, const int64_t* dims, int rank, const char* dtype, const char* device) {
  PyGILState_STATE st = PyGILState_Ensure();
  PyObject* args = Py_BuildValue("(KNss)", (unsigned long long)(uintptr_t)data, tuple_of_i64(dims, rank),
                                 dtype ? dtype : "f32", device ? device : "default");
  mimir_handle h = call_i64("tensor_from_memory", args, 0);
  PyGILState_Release(st);
  return h;
}

API mimir_handle mimir_call(const char* name, const mimir_handle* hs, int n, const char* kwargs_json) {
  PyGILState_STATE st = PyGILState_Ensure();
  PyObject* args = Py_BuildValue("(sNs)", name, tuple_of_i64(hs, n), kwargs_json ? kwargs_json : "");
  mimir_handle h = call_i64("call", args, 0);
  PyGILState_Release(st);
  return h;
}

API int mimir_tensor_dims(mimir_handle t, int64_t* out, int cap) {
  PyGILState_STATE st = PyGILState_Ensure();
  int rank = -1;
  PyObject* r = g_mod ? PyObject_CallMethod(g_mod, "tensor_dims", "L", (long long)t) : NULL;
  if (r && PyList_Check(r)) {
    rank = (int)PyList_Size(r);
    for (int i = 0; i < rank && i < cap && out; ++i) out[i] = PyLong_AsLongLong(PyList_GetItem(r, i));
  } else {
    take_error();
  }
  Py_XDECREF(r);
  PyGILState_Release(st);
  return rank;
}

API int mimir_tensor_rank(mimir_handle t) { return mimir_tensor_dims(t, NULL, 0); }

API int mimir_tensor_error(mimir_handle t, char* buf, int cap) {
  PyGILState_STATE st = PyGILState_Ensure();
  int n = 0;
  PyObject* r = g_mod ? PyObject_CallMethod(g_mod, "tensor_error", "L", (long long)t) : NULL;
  if (r) {
    const char* s = PyUnicode_AsUTF8(r);
    n = s ? (int)strlen(s) : 0;
    if (buf && cap > 0) { strncpy(buf, s ? s : "", cap - 1); buf[cap - 1] = 0; }
    Py_DECREF(r);
  } else {
    take_error();
    n = -1;
  }
  PyGILState_Release(st);
  return n;
}

API int64_t mimir_tensor_read_f32(mimir_handle t, float* out, int64_t cap) {
  PyGILState_STATE st = PyGILState_Ensure();
  PyObject* args = Py_BuildValue("(LKL)", (long long)t, (unsigned long long)(uintptr_t)out, (long long)cap);
  int64_t n = call_i64("tensor_read_f32", args, -1);
  PyGILState_Release(st);
  return n;
}

API int mimir_backward(mimir_handle loss) {
  PyGILState_STATE st = PyGILState_Ensure();
  int rc = (int)call_i64("backward", Py_BuildValue("(L)", (long long)loss), -1);
  PyGILState_Release(st);
  return rc;
}

API mimir_handle mimir_optimizer(const char* kind, mimir_handle module, double lr, const char* kwargs_json) {
  PyGILState_STATE st = PyGILState_Ensure();
  PyObject* args = Py_BuildValue("(sLds)", kind, (long long)module, lr, kwargs_json ? kwargs_json : "");
  mimir_handle h = call_i64("optimizer", args, 0);
  PyGILState_Release(st);
  return h;
}

API int mimir_optimizer_step(mimir_handle opt, int zero_grad_after) {
  PyGILState_STATE st = PyGILState_Ensure();
  int rc = (int)call_i64("optimizer_step", Py_BuildValue("(Li)", (long long)opt, zero_grad_after), -1);
  PyGILState_Release(st);
  return rc;
}

API mimir_handle mimir_mesh(const int64_t* shape, const char* const* axes, int naxes) {
  PyGILState_STATE st = PyGILState_Ensure();
  PyObject* names = PyTuple_New(naxes);
  for (int i = 0; names && i < naxes; ++i) PyTuple_SET_ITEM(names, i, PyUnicode_FromString(axes[i]));
  mimir_handle h = call_i64("mesh", Py_BuildValue("(NN)", tuple_of_i64(shape, naxes), names), 0);
  PyGILState_Release(st);
  return h;
}

API int mimir_release(mimir_handle h) {
  PyGILState_STATE st = PyGILState_Ensure();
  int rc = (int)call_i64("release", Py_BuildValue("(L)", (long long)h), -1);
  PyGILState_Release(st);
  return rc;
}
