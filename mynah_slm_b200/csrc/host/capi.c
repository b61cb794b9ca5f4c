/* The C interface of the engine (include/mynah_slm_b200.h) over an embedded Python interpreter.
 *
 * Every exported function takes the interpreter's lock, calls its counterpart in mynah_slm_b200/engine/capi.py
 * (which returns (code, message, value) and never raises) and copies the message into the caller's buffer.
 * Nothing here computes anything of the model, prints, or exits.
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/mynah_slm_b200.h"
#include "../../include/mynah_slm_b200_host.h"

#ifndef MYNAH_DEFAULT_PYTHON
#define MYNAH_DEFAULT_PYTHON ""
#endif
#ifndef MYNAH_DEFAULT_ROOT
#define MYNAH_DEFAULT_ROOT ""
#endif

struct mynah_engine {
    PyObject* llm;        /* mynah_slm_b200.engine.api.LLM */
};

static PyObject* g_module = NULL;      /* mynah_slm_b200.engine.capi */
static int g_we_started_python = 0;

static void set_err(char* err, size_t errlen, const char* fmt, ...) {
    if (err == NULL || errlen == 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, errlen, fmt, ap);
    va_end(ap);
}

/* The text of the pending Python exception, which is cleared. */
static void take_python_error(char* err, size_t errlen, const char* what) {
    PyObject *type = NULL, *value = NULL, *trace = NULL;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    PyObject* text = value ? PyObject_Str(value) : NULL;
    const char* s = text ? PyUnicode_AsUTF8(text) : NULL;
    set_err(err, errlen, "%s: %s", what, s ? s : "unknown Python error");
    if (s == NULL) PyErr_Clear();
    Py_XDECREF(text);
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(trace);
}

/* Starts the interpreter if the process has none, and imports the package's half of this interface. Returns with
 * the interpreter's lock held (state in *gil) on success. */
static int enter(PyGILState_STATE* gil, char* err, size_t errlen) {
    if (!Py_IsInitialized()) {
        PyConfig config;
        PyConfig_InitPythonConfig(&config);
        config.install_signal_handlers = 0;
        config.parse_argv = 0;
        const char* exe = getenv("MYNAH_PYTHON");
        if (exe == NULL || exe[0] == '\0') exe = MYNAH_DEFAULT_PYTHON;
        PyStatus st = PyStatus_Ok();
        if (exe[0] != '\0') {
            st = PyConfig_SetBytesString(&config, &config.program_name, exe);
            if (!PyStatus_Exception(st)) st = PyConfig_SetBytesString(&config, &config.executable, exe);
        }
        if (!PyStatus_Exception(st)) st = Py_InitializeFromConfig(&config);
        PyConfig_Clear(&config);
        if (PyStatus_Exception(st)) {
            set_err(err, errlen, "the Python interpreter could not be started: %s", st.err_msg ? st.err_msg : "?");
            return MYNAH_ERR_INTERNAL;
        }
        g_we_started_python = 1;
        PyEval_SaveThread();            /* from here on every call takes the lock itself */
    }
    *gil = PyGILState_Ensure();
    if (g_module == NULL) {
        const char* root = getenv("MYNAH_SLM_B200_ROOT");
        if (root == NULL || root[0] == '\0') root = MYNAH_DEFAULT_ROOT;
        if (root[0] != '\0') {
            PyObject* path = PySys_GetObject("path");       /* borrowed */
            PyObject* entry = PyUnicode_FromString(root);
            if (path != NULL && entry != NULL && PySequence_Contains(path, entry) == 0) PyList_Insert(path, 0, entry);
            Py_XDECREF(entry);
        }
        g_module = PyImport_ImportModule("mynah_slm_b200.engine.capi");
        if (g_module == NULL) {
            take_python_error(err, errlen, "the package mynah_slm_b200 could not be imported");
            PyGILState_Release(*gil);
            return MYNAH_ERR_INTERNAL;
        }
    }
    return MYNAH_OK;
}

/* Calls capi.<name>(args...) and unpacks (code, message, value). *value (a new reference, or NULL) is set on success. */
static int call(const char* name, PyObject* args, PyObject** value, char* err, size_t errlen) {
    if (value) *value = NULL;
    if (args == NULL) {
        take_python_error(err, errlen, name);
        return MYNAH_ERR_INTERNAL;
    }
    PyObject* fn = PyObject_GetAttrString(g_module, name);
    PyObject* res = fn ? PyObject_CallObject(fn, args) : NULL;
    Py_XDECREF(fn);
    Py_DECREF(args);
    if (res == NULL || !PyTuple_Check(res) || PyTuple_GET_SIZE(res) != 3) {
        take_python_error(err, errlen, name);
        Py_XDECREF(res);
        return MYNAH_ERR_INTERNAL;
    }
    const int code = (int)PyLong_AsLong(PyTuple_GET_ITEM(res, 0));
    if (code != MYNAH_OK) {
        const char* msg = PyUnicode_AsUTF8(PyTuple_GET_ITEM(res, 1));
        set_err(err, errlen, "%s", msg ? msg : "error");
        if (msg == NULL) PyErr_Clear();
    } else if (value) {
        *value = PyTuple_GET_ITEM(res, 2);
        Py_INCREF(*value);
    }
    Py_DECREF(res);
    return code;
}

static int make_engine(const char* fn, PyObject* args, mynah_engine** out, char* err, size_t errlen) {
    PyObject* llm = NULL;
    const int rc = call(fn, args, &llm, err, errlen);
    if (rc != MYNAH_OK) return rc;
    mynah_engine* e = (mynah_engine*)calloc(1, sizeof *e);
    if (e == NULL) {
        Py_XDECREF(llm);
        set_err(err, errlen, "out of memory");
        return MYNAH_ERR_INTERNAL;
    }
    e->llm = llm;
    *out = e;
    return MYNAH_OK;
}

int mynah_engine_create(const char* model_folder, const char* dtype, int max_tokens, int max_seqs,
                        mynah_engine** out, char* err, size_t errlen) {
    if (out == NULL || model_folder == NULL || dtype == NULL) {
        set_err(err, errlen, "mynah_engine_create: a NULL argument");
        return MYNAH_ERR_ARGUMENT;
    }
    *out = NULL;
    PyGILState_STATE gil;
    int rc = enter(&gil, err, errlen);
    if (rc != MYNAH_OK) return rc;
    rc = make_engine("create", Py_BuildValue("(ssii)", model_folder, dtype, max_tokens, max_seqs), out, err, errlen);
    PyGILState_Release(gil);
    return rc;
}

int mynah_engine_create_random(const char* config_json, uint64_t seed, const char* dtype, int max_tokens, int max_seqs,
                               mynah_engine** out, char* err, size_t errlen) {
    if (out == NULL || config_json == NULL || dtype == NULL) {
        set_err(err, errlen, "mynah_engine_create_random: a NULL argument");
        return MYNAH_ERR_ARGUMENT;
    }
    *out = NULL;
    PyGILState_STATE gil;
    int rc = enter(&gil, err, errlen);
    if (rc != MYNAH_OK) return rc;
    rc = make_engine("create_random", Py_BuildValue("(sKsii)", config_json, (unsigned long long)seed, dtype, max_tokens, max_seqs),
                     out, err, errlen);
    PyGILState_Release(gil);
    return rc;
}

void mynah_engine_free(mynah_engine* e) {
    if (e == NULL) return;
    if (Py_IsInitialized()) {
        PyGILState_STATE gil = PyGILState_Ensure();
        Py_XDECREF(e->llm);
        PyGILState_Release(gil);
    }
    free(e);
}

static int accessor(const mynah_engine* e, const char* what) {
    if (e == NULL || g_module == NULL) return -1;
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject* v = NULL;
    int out = -1;
    if (call("info", Py_BuildValue("(Os)", e->llm, what), &v, NULL, 0) == MYNAH_OK && v != NULL) out = (int)PyLong_AsLong(v);
    Py_XDECREF(v);
    PyGILState_Release(gil);
    return out;
}

int mynah_engine_vocab_size(const mynah_engine* e) { return accessor(e, "vocab_size"); }
int mynah_engine_max_positions(const mynah_engine* e) { return accessor(e, "max_positions"); }
int mynah_engine_hidden_size(const mynah_engine* e) { return accessor(e, "hidden_size"); }
int mynah_engine_n_layers(const mynah_engine* e) { return accessor(e, "n_layers"); }
int mynah_engine_free_tokens(const mynah_engine* e) { return accessor(e, "free_tokens"); }
int mynah_page_size(void) { return MYNAH_PAGE_TOKENS; }

int mynah_engine_eos_ids(const mynah_engine* e, int32_t* ids, int capacity) {
    if (e == NULL || g_module == NULL) return -1;
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject* v = NULL;
    int out = -1;
    if (call("eos_ids", Py_BuildValue("(OKi)", e->llm, (unsigned long long)(uintptr_t)ids, ids ? capacity : 0), &v, NULL, 0) == MYNAH_OK && v)
        out = (int)PyLong_AsLong(v);
    Py_XDECREF(v);
    PyGILState_Release(gil);
    return out;
}

/* A call on an engine that returns a number through *number (may be NULL). */
static int engine_call(const mynah_engine* e, const char* fn, PyObject* (*build)(const mynah_engine*, void*), void* a,
                       long* number, char* err, size_t errlen) {
    if (e == NULL || g_module == NULL) {
        set_err(err, errlen, "%s: no engine", fn);
        return MYNAH_ERR_ARGUMENT;
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject* v = NULL;
    const int rc = call(fn, build(e, a), &v, err, errlen);
    if (rc == MYNAH_OK && number != NULL && v != NULL) *number = PyLong_AsLong(v);
    Py_XDECREF(v);
    PyGILState_Release(gil);
    return rc;
}

static PyObject* build_llm(const mynah_engine* e, void* a) { (void)a; return Py_BuildValue("(O)", e->llm); }
static PyObject* build_llm_int(const mynah_engine* e, void* a) { return Py_BuildValue("(Oi)", e->llm, *(int*)a); }

int mynah_slot_open(mynah_engine* e, int* slot, char* err, size_t errlen) {
    if (slot == NULL) {
        set_err(err, errlen, "mynah_slot_open: slot is NULL");
        return MYNAH_ERR_ARGUMENT;
    }
    long v = -1;
    const int rc = engine_call(e, "slot_open", build_llm, NULL, &v, err, errlen);
    if (rc == MYNAH_OK) *slot = (int)v;
    return rc;
}

int mynah_slot_close(mynah_engine* e, int slot, char* err, size_t errlen) {
    return engine_call(e, "slot_close", build_llm_int, &slot, NULL, err, errlen);
}

int mynah_slot_length(const mynah_engine* e, int slot) {
    long v = -1;
    return engine_call(e, "slot_length", build_llm_int, &slot, &v, NULL, 0) == MYNAH_OK ? (int)v : -1;
}

struct step_args {
    int n;
    const int *slots, *n_new, *n_want, *want;
    const int32_t* tokens;
    float* out;
};

static PyObject* build_step(const mynah_engine* e, void* p) {
    const struct step_args* a = (const struct step_args*)p;
    return Py_BuildValue("(OiKKKKKK)", e->llm, a->n, (unsigned long long)(uintptr_t)a->slots, (unsigned long long)(uintptr_t)a->n_new,
                         (unsigned long long)(uintptr_t)a->tokens, (unsigned long long)(uintptr_t)a->n_want,
                         (unsigned long long)(uintptr_t)a->want, (unsigned long long)(uintptr_t)a->out);
}

int mynah_step(mynah_engine* e, int n, const int* slots, const int* n_new, const int32_t* tokens,
               const int* n_want, const int* want, float* logits_out, char* err, size_t errlen) {
    if (n < 1 || slots == NULL || n_new == NULL || tokens == NULL || n_want == NULL) {
        set_err(err, errlen, "mynah_step: at least one sequence with its slots, token counts, tokens and wanted counts is needed");
        return MYNAH_ERR_ARGUMENT;
    }
    struct step_args a = {n, slots, n_new, n_want, want, tokens, logits_out};
    return engine_call(e, "step", build_step, &a, NULL, err, errlen);
}

void mynah_sampler_defaults(mynah_sampler_params* p) {
    if (p == NULL) return;
    p->temp = 0.6f;
    p->top_k = 20;
    p->top_p = 0.95f;
    p->min_p = 0.0f;
    p->repeat_penalty = 1.0f;
    p->freq_penalty = 0.0f;
    p->presence_penalty = 0.0f;
    p->penalty_window = 64;
    p->seed = 0;
}

static PyObject* params_tuple(const mynah_sampler_params* p) {
    return Py_BuildValue("(dIdddddIK)", (double)p->temp, (unsigned)p->top_k, (double)p->top_p, (double)p->min_p,
                         (double)p->repeat_penalty, (double)p->freq_penalty, (double)p->presence_penalty,
                         (unsigned)p->penalty_window, (unsigned long long)p->seed);
}

int mynah_sample(mynah_engine* e, const float* logits, int n_rows, const mynah_sampler_params* params, uint64_t* rng,
                 int32_t* tokens_out, char* err, size_t errlen) {
    if (e == NULL || g_module == NULL || logits == NULL || params == NULL || tokens_out == NULL || n_rows < 1) {
        set_err(err, errlen, "mynah_sample: an engine, logits, parameters and a place for the tokens are needed");
        return MYNAH_ERR_ARGUMENT;
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject* p = params_tuple(params);
    PyObject* args = p ? Py_BuildValue("(OKiNKK)", e->llm, (unsigned long long)(uintptr_t)logits, n_rows, p,
                                       (unsigned long long)(uintptr_t)rng, (unsigned long long)(uintptr_t)tokens_out) : NULL;
    const int rc = call("sample", args, NULL, err, errlen);
    PyGILState_Release(gil);
    return rc;
}

int mynah_generate(mynah_engine* e, const mynah_request* requests, int n_requests, const mynah_sampler_params* params,
                   const int32_t* stop_ids, int n_stop, int max_batch, mynah_token_cb cb, void* cb_ctx,
                   mynah_result* results, mynah_timing* timing, char* err, size_t errlen) {
    if (e == NULL || g_module == NULL || requests == NULL || results == NULL || params == NULL || n_requests < 1) {
        set_err(err, errlen, "mynah_generate: an engine, requests, parameters and results are needed");
        return MYNAH_ERR_ARGUMENT;
    }
    for (int i = 0; i < n_requests; i++) {
        if (requests[i].tokens == NULL || requests[i].n_tokens < 1 || (requests[i].max_new > 0 && results[i].tokens == NULL)) {
            set_err(err, errlen, "mynah_generate: request %d has no prompt or no room for its tokens", i);
            return MYNAH_ERR_ARGUMENT;
        }
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    int rc = MYNAH_ERR_INTERNAL;
    PyObject *reqs = PyList_New(n_requests), *outs = PyList_New(n_requests), *stop = NULL, *value = NULL;
    if (reqs && outs) {
        for (int i = 0; i < n_requests; i++) {
            PyList_SET_ITEM(reqs, i, Py_BuildValue("(Kii)", (unsigned long long)(uintptr_t)requests[i].tokens, requests[i].n_tokens, requests[i].max_new));
            PyList_SET_ITEM(outs, i, Py_BuildValue("(Ki)", (unsigned long long)(uintptr_t)results[i].tokens,
                                                   requests[i].max_new > 0 ? requests[i].max_new : 0));
        }
        if (n_stop < 0) {
            stop = Py_None;
            Py_INCREF(stop);
        } else {
            stop = PyList_New(n_stop);
            for (int i = 0; stop && i < n_stop; i++) PyList_SET_ITEM(stop, i, PyLong_FromLong(stop_ids ? stop_ids[i] : 0));
        }
        PyObject* p = params_tuple(params);
        PyObject* args = (p && stop) ? Py_BuildValue("(OONOiKKO)", e->llm, reqs, p, stop, max_batch, (unsigned long long)(uintptr_t)cb,
                                                     (unsigned long long)(uintptr_t)cb_ctx, outs) : NULL;
        rc = call("generate", args, &value, err, errlen);
    } else {
        take_python_error(err, errlen, "mynah_generate");
    }
    if (rc == MYNAH_OK && value != NULL) {
        PyObject *summary = PyTuple_GetItem(value, 0), *tm = PyTuple_GetItem(value, 1), *stopped = PyTuple_GetItem(value, 2);
        for (int i = 0; summary && i < n_requests; i++) {
            PyObject* row = PyList_GetItem(summary, i);
            if (row == NULL) break;
            results[i].n_tokens = (int)PyLong_AsLong(PyTuple_GetItem(row, 0));
            results[i].produced = (int)PyLong_AsLong(PyTuple_GetItem(row, 1));
            results[i].finish = (int)PyLong_AsLong(PyTuple_GetItem(row, 2));
        }
        if (timing != NULL && tm != NULL) {
            timing->load_s = PyFloat_AsDouble(PyTuple_GetItem(tm, 0));
            timing->prefill_s = PyFloat_AsDouble(PyTuple_GetItem(tm, 1));
            timing->decode_s = PyFloat_AsDouble(PyTuple_GetItem(tm, 2));
            timing->ttft_s = PyFloat_AsDouble(PyTuple_GetItem(tm, 3));
            timing->n_prompt = (int)PyLong_AsLong(PyTuple_GetItem(tm, 4));
            timing->n_gen = (int)PyLong_AsLong(PyTuple_GetItem(tm, 5));
        }
        if (stopped != NULL && PyObject_IsTrue(stopped)) rc = MYNAH_STOPPED;
        if (PyErr_Occurred()) {
            take_python_error(err, errlen, "mynah_generate");
            rc = MYNAH_ERR_INTERNAL;
        }
    }
    Py_XDECREF(value);
    Py_XDECREF(reqs);
    Py_XDECREF(outs);
    Py_XDECREF(stop);
    PyGILState_Release(gil);
    return rc;
}
