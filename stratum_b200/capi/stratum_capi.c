/* The C interface of stratum_b200: every function forwards to stratum_b200.capi.host inside an embedded (or the
 * already running) interpreter.  See stratum.h. */
#define _GNU_SOURCE
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "stratum.h"

#ifndef STRATUM_PYTHON_EXE
#define STRATUM_PYTHON_EXE ""      /* the interpreter this library was built with (its environment's packages) */
#endif

struct stratum_ctx {
  long handle;                     /* of the engine inside stratum_b200.capi.host */
  char error[2048];
};

static char g_open_error[2048];
static PyObject* g_host = NULL;    /* the module stratum_b200.capi.host */
static int g_started_here = 0;

static void set_error(char* dst, size_t n, const char* msg) {
  snprintf(dst, n, "%s", msg ? msg : "unknown error");
}

/* The pending Python exception as text into dst (and cleared). */
static void take_exception(char* dst, size_t n) {
  PyObject *type = NULL, *value = NULL, *trace = NULL;
  PyErr_Fetch(&type, &value, &trace);
  PyErr_NormalizeException(&type, &value, &trace);
  const char* name = (type && PyType_Check(type)) ? ((PyTypeObject*)type)->tp_name : "error";
  PyObject* text = value ? PyObject_Str(value) : NULL;
  const char* msg = text ? PyUnicode_AsUTF8(text) : NULL;
  snprintf(dst, n, "%s: %s", name, msg ? msg : "(no message)");
  Py_XDECREF(text); Py_XDECREF(type); Py_XDECREF(value); Py_XDECREF(trace);
  PyErr_Clear();
}

/* Bring up the interpreter if this process has none.  Returns 0, or STRATUM_E_INTERPRETER with text in err. */
static int ensure_interpreter(char* err, size_t n) {
  if (Py_IsInitialized()) return 0;
  PyConfig config;
  PyConfig_InitPythonConfig(&config);
  const char* exe = getenv("STRATUM_PYTHON");
  if (!exe || !exe[0]) exe = STRATUM_PYTHON_EXE;
  PyStatus st = PyStatus_Ok();
  if (exe[0]) {                    /* so that the interpreter finds that environment's packages (torch, numpy) */
    st = PyConfig_SetBytesString(&config, &config.program_name, exe);
    if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.executable, exe);
  }
  if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
  PyConfig_Clear(&config);
  if (PyStatus_Exception(st)) {
    snprintf(err, n, "the Python interpreter could not be started: %s", st.err_msg ? st.err_msg : "?");
    return STRATUM_E_INTERPRETER;
  }
  g_started_here = 1;
  PyEval_SaveThread();             /* calls below take the lock themselves */
  return 0;
}

/* With the lock held: the host module, imported once.  NULL with text in err on failure. */
static PyObject* host_module(char* err, size_t n) {
  if (g_host) return g_host;
  /* the folder that holds the package: four levels above this library (<root>/stratum_b200/capi/_build/lib.so) */
  char own[4096] = "";
  const char* root = getenv("STRATUM_PACKAGE_ROOT");
  if (!root || !root[0]) {
    Dl_info info;
    if (dladdr((void*)&stratum_open, &info) && info.dli_fname && realpath(info.dli_fname, own)) {
      for (int up = 0; up < 4; ++up) {
        char* cut = strrchr(own, '/');
        if (!cut) { own[0] = 0; break; }
        *cut = 0;
      }
    }
    root = own;
  }
  if (root[0]) {
    PyObject* path = PySys_GetObject("path");               /* borrowed */
    PyObject* item = PyUnicode_FromString(root);
    if (path && item && !PySequence_Contains(path, item)) PyList_Insert(path, 0, item);
    Py_XDECREF(item);
  }
  g_host = PyImport_ImportModule("stratum_b200.capi.host");
  if (!g_host) take_exception(err, n);
  return g_host;
}

/* Call host.<name>(*args) (args: a new reference to a tuple, consumed).  A new reference, or NULL with text in err. */
static PyObject* call_host(const char* name, PyObject* args, char* err, size_t n) {
  PyObject* result = NULL;
  PyObject* mod = host_module(err, n);
  if (mod && args) {
    PyObject* fn = PyObject_GetAttrString(mod, name);
    if (fn) {
      result = PyObject_CallObject(fn, args);
      Py_DECREF(fn);
    }
    if (!result) take_exception(err, n);
  } else if (mod && !args) {
    take_exception(err, n);
  }
  Py_XDECREF(args);
  return result;
}

/* host.<name>(handle, ...) -> an int written to *out (if out is not null). */
static int call_int(stratum_ctx* ctx, const char* name, PyObject* args, long* out) {
  PyObject* r = call_host(name, args, ctx->error, sizeof ctx->error);
  if (!r) return STRATUM_E_ENGINE;
  if (out) *out = PyLong_AsLong(r);
  Py_DECREF(r);
  if (PyErr_Occurred()) { take_exception(ctx->error, sizeof ctx->error); return STRATUM_E_ENGINE; }
  return STRATUM_OK;
}

int stratum_open(const char* model_dir, const char* dtype, long long max_tokens, int max_seqs, stratum_ctx** out) {
  if (!out) { set_error(g_open_error, sizeof g_open_error, "stratum_open: out is null"); return STRATUM_E_ARGUMENT; }
  *out = NULL;
  if (!model_dir || !dtype || max_tokens < 1 || max_seqs < 0) {
    set_error(g_open_error, sizeof g_open_error, "stratum_open: model_dir and dtype must be given, max_tokens >= 1, max_seqs >= 0");
    return STRATUM_E_ARGUMENT;
  }
  int rc = ensure_interpreter(g_open_error, sizeof g_open_error);
  if (rc != 0) return rc;
  PyGILState_STATE lock = PyGILState_Ensure();
  PyObject* r = call_host("open_model", Py_BuildValue("(ssLi)", model_dir, dtype, max_tokens, max_seqs), g_open_error,
                          sizeof g_open_error);
  if (!r) {
    rc = g_host ? STRATUM_E_ENGINE : STRATUM_E_INTERPRETER;
  } else {
    stratum_ctx* ctx = (stratum_ctx*)calloc(1, sizeof(stratum_ctx));
    if (!ctx) { set_error(g_open_error, sizeof g_open_error, "out of memory"); rc = STRATUM_E_ENGINE; }
    else { ctx->handle = PyLong_AsLong(r); *out = ctx; }
    Py_DECREF(r);
  }
  PyGILState_Release(lock);
  return rc;
}

void stratum_close(stratum_ctx* ctx) {
  if (!ctx) return;
  if (Py_IsInitialized()) {
    PyGILState_STATE lock = PyGILState_Ensure();
    PyObject* r = call_host("close_model", Py_BuildValue("(l)", ctx->handle), ctx->error, sizeof ctx->error);
    Py_XDECREF(r);
    PyGILState_Release(lock);
  }
  free(ctx);
}

#define ENTER(ctx_)                                                                     \
  if (!(ctx_)) return STRATUM_E_ARGUMENT;                                               \
  if (!Py_IsInitialized()) { set_error((ctx_)->error, sizeof (ctx_)->error, "the interpreter is gone"); return STRATUM_E_INTERPRETER; } \
  PyGILState_STATE lock = PyGILState_Ensure();                                          \
  int rc = STRATUM_OK;
#define LEAVE() PyGILState_Release(lock); return rc;

int stratum_vocab(stratum_ctx* ctx, int* vocab) {
  ENTER(ctx)
  long v = 0;
  if (!vocab) { set_error(ctx->error, sizeof ctx->error, "stratum_vocab: vocab is null"); rc = STRATUM_E_ARGUMENT; }
  else if ((rc = call_int(ctx, "vocab", Py_BuildValue("(l)", ctx->handle), &v)) == 0) *vocab = (int)v;
  LEAVE()
}

int stratum_slot_acquire(stratum_ctx* ctx, int* slot) {
  ENTER(ctx)
  long v = 0;
  if (!slot) { set_error(ctx->error, sizeof ctx->error, "stratum_slot_acquire: slot is null"); rc = STRATUM_E_ARGUMENT; }
  else if ((rc = call_int(ctx, "slot_acquire", Py_BuildValue("(l)", ctx->handle), &v)) == 0) *slot = (int)v;
  LEAVE()
}

int stratum_slot_release(stratum_ctx* ctx, int slot) {
  ENTER(ctx)
  rc = call_int(ctx, "slot_release", Py_BuildValue("(li)", ctx->handle, slot), NULL);
  LEAVE()
}

int stratum_slot_length(stratum_ctx* ctx, int slot, int* length) {
  ENTER(ctx)
  long v = 0;
  if (!length) { set_error(ctx->error, sizeof ctx->error, "stratum_slot_length: length is null"); rc = STRATUM_E_ARGUMENT; }
  else if ((rc = call_int(ctx, "slot_length", Py_BuildValue("(li)", ctx->handle, slot), &v)) == 0) *length = (int)v;
  LEAVE()
}

int stratum_step(stratum_ctx* ctx, int n_seq, const int* slots, const int* n_tok, const int* tokens,
                 const int* n_want, const int* want, float* logits) {
  ENTER(ctx)
  if (n_seq < 1 || !slots || !n_tok || !tokens || !n_want) {
    set_error(ctx->error, sizeof ctx->error, "stratum_step: n_seq >= 1 and slots, n_tok, tokens, n_want must be given");
    rc = STRATUM_E_ARGUMENT;
  } else {
    /* arrays travel as addresses; the host reads and writes them in place */
    rc = call_int(ctx, "step", Py_BuildValue("(liKKKKKK)", ctx->handle, n_seq, (unsigned long long)(size_t)slots,
                                             (unsigned long long)(size_t)n_tok, (unsigned long long)(size_t)tokens,
                                             (unsigned long long)(size_t)n_want, (unsigned long long)(size_t)want,
                                             (unsigned long long)(size_t)logits), NULL);
  }
  LEAVE()
}

int stratum_generate(stratum_ctx* ctx, int n_prompts, const int* prompt_len, const int* prompt_tokens, int max_new,
                     const int* stop_ids, int n_stop, float temperature, int top_k, float top_p,
                     unsigned long long seed, int* out_tokens, int* out_count) {
  ENTER(ctx)
  if (n_prompts < 1 || !prompt_len || !prompt_tokens || max_new < 0 || n_stop < 0 || (n_stop > 0 && !stop_ids) ||
      !out_tokens || !out_count) {
    set_error(ctx->error, sizeof ctx->error, "stratum_generate: a count is negative or a needed array is null");
    rc = STRATUM_E_ARGUMENT;
  } else {
    rc = call_int(ctx, "generate", Py_BuildValue("(liKKiKidifKKK)", ctx->handle, n_prompts,
                                                 (unsigned long long)(size_t)prompt_len,
                                                 (unsigned long long)(size_t)prompt_tokens, max_new,
                                                 (unsigned long long)(size_t)stop_ids, n_stop, (double)temperature,
                                                 top_k, top_p, seed, (unsigned long long)(size_t)out_tokens,
                                                 (unsigned long long)(size_t)out_count), NULL);
  }
  LEAVE()
}

const char* stratum_last_error(stratum_ctx* ctx) { return ctx ? ctx->error : g_open_error; }
