// CPython fast-call entry for the bf16 GEMM: one METH_FASTCALL function taking 20 positional numbers, so a GEMM
// launch from Python costs a vectorcall plus integer unboxing instead of a ctypes foreign call with 20 argument
// conversions.  The reference project does the same for its cuBLASLt dispatcher
// (helpers/matmul_dispatcher/src/dispatch_pyext.cpp:37-118, "matmul_fast"), where it removes ~5 us per call
// from the per-expert MoE loops.  Here the kernel library is opened with dlopen at bind() time, so this module
// links against neither CUDA nor the kernel library.
//
//   _ftb_fastcall.bind(path_to_libftb_gemm_tcgen05.so)          -> None
//   _ftb_fastcall.gemm(A, B, D, C, bias, M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, alpha, beta, d_fp32, bn,
//                      max_ctas, stream)                        -> int (the kernel library's return code)
//   _ftb_fastcall.calls()                                       -> number of gemm() calls so far
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <dlfcn.h>
#include <stdint.h>

namespace {

typedef int (*GemmFn)(const void*, const void*, void*, const void*, const float*, int, int, int, int, int, int, int,
                      int, int, float, float, int, int, int, void*);
GemmFn g_gemm = nullptr;
void* g_handle = nullptr;
unsigned long long g_calls = 0;

inline bool as_ptr(PyObject* o, void** out) {
  if (o == Py_None) {
    *out = nullptr;
    return true;
  }
  const unsigned long long v = PyLong_AsUnsignedLongLong(o);
  if (v == static_cast<unsigned long long>(-1) && PyErr_Occurred()) return false;
  *out = reinterpret_cast<void*>(static_cast<uintptr_t>(v));
  return true;
}

inline bool as_int(PyObject* o, int* out) {
  const long v = PyLong_AsLong(o);
  if (v == -1 && PyErr_Occurred()) return false;
  *out = static_cast<int>(v);
  return true;
}

inline bool as_float(PyObject* o, float* out) {
  const double v = PyFloat_AsDouble(o);
  if (v == -1.0 && PyErr_Occurred()) return false;
  *out = static_cast<float>(v);
  return true;
}

PyObject* py_bind(PyObject*, PyObject* arg) {
  const char* path = PyUnicode_AsUTF8(arg);
  if (path == nullptr) return nullptr;
  void* h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) {
    PyErr_Format(PyExc_OSError, "dlopen(%s) failed: %s", path, dlerror());
    return nullptr;
  }
  void* sym = dlsym(h, "ftb_gemm_bf16");
  if (sym == nullptr) {
    PyErr_Format(PyExc_OSError, "%s has no symbol ftb_gemm_bf16", path);
    dlclose(h);
    return nullptr;
  }
  g_handle = h;
  g_gemm = reinterpret_cast<GemmFn>(sym);
  Py_RETURN_NONE;
}

PyObject* py_gemm(PyObject*, PyObject* const* a, Py_ssize_t n) {
  if (n != 20) {
    PyErr_SetString(PyExc_TypeError, "gemm() takes exactly 20 positional arguments");
    return nullptr;
  }
  if (g_gemm == nullptr) {
    PyErr_SetString(PyExc_RuntimeError, "bind() the kernel library first");
    return nullptr;
  }
  void *A, *B, *D, *C, *bias, *stream;
  int M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, d_fp32, bn, max_ctas;
  float alpha, beta;
  if (!as_ptr(a[0], &A) || !as_ptr(a[1], &B) || !as_ptr(a[2], &D) || !as_ptr(a[3], &C) || !as_ptr(a[4], &bias) ||
      !as_int(a[5], &M) || !as_int(a[6], &N) || !as_int(a[7], &K) || !as_int(a[8], &a_mn) || !as_int(a[9], &b_mn) ||
      !as_int(a[10], &lda) || !as_int(a[11], &ldb) || !as_int(a[12], &ldd) || !as_int(a[13], &ldc) ||
      !as_float(a[14], &alpha) || !as_float(a[15], &beta) || !as_int(a[16], &d_fp32) || !as_int(a[17], &bn) ||
      !as_int(a[18], &max_ctas) || !as_ptr(a[19], &stream))
    return nullptr;
  ++g_calls;
  const int rc = g_gemm(A, B, D, C, static_cast<const float*>(bias), M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, alpha,
                        beta, d_fp32, bn, max_ctas, stream);
  return PyLong_FromLong(rc);
}

PyObject* py_calls(PyObject*, PyObject*) { return PyLong_FromUnsignedLongLong(g_calls); }

PyMethodDef kMethods[] = {
    {"bind", py_bind, METH_O, "bind(path): open the GEMM kernel library"},
    {"gemm", reinterpret_cast<PyCFunction>(reinterpret_cast<void (*)(void)>(py_gemm)), METH_FASTCALL,
     "gemm(A, B, D, C, bias, M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, alpha, beta, d_fp32, bn, max_ctas, stream)"},
    {"calls", py_calls, METH_NOARGS, "number of gemm() calls"},
    {nullptr, nullptr, 0, nullptr}};

PyModuleDef kModule = {PyModuleDef_HEAD_INIT, "_ftb_fastcall", "fast-call GEMM entry", -1, kMethods,
                       nullptr, nullptr, nullptr, nullptr};

}  // namespace

PyMODINIT_FUNC PyInit__ftb_fastcall(void) { return PyModule_Create(&kModule); }
