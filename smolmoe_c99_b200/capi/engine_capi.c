/* The C interface (engine.h) over the library's one engine: every function takes the interpreter's lock, hands
 * plain numbers and addresses to smolmoe_c99_b200.engine.capi, and turns what comes back, or the exception,
 * into a status and a message. Nothing of the model is computed here. */
#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "engine.h"

#define API __attribute__((visibility("default")))

struct lm {
    PyObject *handle;   /* the Python side's object */
};

static _Thread_local char g_error[LM_ERROR_BYTES];
static PyObject *g_module;      /* smolmoe_c99_b200.engine.capi */
static int g_started_python;

static void set_error(const char *text) {
    snprintf(g_error, sizeof g_error, "%s", text ? text : "unknown error");
}

/* The pending Python exception as a status and a message. */
static int take_exception(void) {
    PyObject *type = NULL, *value = NULL, *trace = NULL;
    int status = LM_ERR_RUNTIME;
    PyErr_Fetch(&type, &value, &trace);
    PyErr_NormalizeException(&type, &value, &trace);
    if (type && (PyErr_GivenExceptionMatches(type, PyExc_ValueError) || PyErr_GivenExceptionMatches(type, PyExc_KeyError) ||
                 PyErr_GivenExceptionMatches(type, PyExc_OSError)))
        status = LM_ERR_ARGUMENT;
    PyObject *text = value ? PyObject_Str(value) : NULL;
    const char *utf8 = text ? PyUnicode_AsUTF8(text) : NULL;
    set_error(utf8 ? utf8 : "the engine raised an exception without a message");
    Py_XDECREF(text);
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(trace);
    PyErr_Clear();
    return status;
}

/* Starts the interpreter if the process has none, and imports the marshalling module. Returns with the lock held
 * in *gil on success. */
static int enter(const char *package_root, PyGILState_STATE *gil) {
    if (!Py_IsInitialized()) {
        Py_InitializeEx(0);
        if (!Py_IsInitialized()) {
            set_error("the Python interpreter could not be started");
            return LM_ERR_PYTHON;
        }
        g_started_python = 1;
        PyEval_SaveThread();     /* give the lock up: every call takes it again */
    }
    *gil = PyGILState_Ensure();
    if (g_module) return LM_OK;
    char root[4096] = "";
    if (package_root) {
        snprintf(root, sizeof root, "%s", package_root);
    } else {
        /* this library lies in <root>/smolmoe_c99_b200/capi/_build/ */
        Dl_info info;
        if (dladdr((void *)&enter, &info) && info.dli_fname) {
            snprintf(root, sizeof root, "%s", info.dli_fname);
            for (int up = 0; up < 4; ++up) {
                char *slash = strrchr(root, '/');
                if (!slash) break;
                *slash = 0;
            }
        }
    }
    if (root[0]) {
        PyObject *path = PySys_GetObject("path");   /* borrowed */
        PyObject *entry = PyUnicode_FromString(root);
        if (path && entry && !PySequence_Contains(path, entry)) PyList_Insert(path, 0, entry);
        Py_XDECREF(entry);
    }
    g_module = PyImport_ImportModule("smolmoe_c99_b200.engine.capi");
    if (!g_module) {
        int status = take_exception();
        (void)status;
        PyGILState_Release(*gil);
        return LM_ERR_PYTHON;
    }
    return LM_OK;
}

static PyObject *options_dict(const lm_options *o) {
    return Py_BuildValue("{s:s,s:i,s:i,s:i,s:s}", "dtype", o && o->dtype ? o->dtype : "bfloat16", "context", o ? o->context : 0,
                         "batch", o ? o->batch : 0, "step_tokens", o ? o->step_tokens : 0, "kernels",
                         o && o->kernels ? o->kernels : "fast");
}

static lm *open_with(const char *function, const char *path, uint32_t seed, const lm_options *options, char err[LM_ERROR_BYTES]) {
    PyGILState_STATE gil;
    lm *model = NULL;
    if (err) err[0] = 0;
    if (!path) {
        set_error("a path is needed");
        if (err) snprintf(err, LM_ERROR_BYTES, "%s", g_error);
        return NULL;
    }
    if (enter(options ? options->package_root : NULL, &gil) != LM_OK) {
        if (err) snprintf(err, LM_ERROR_BYTES, "%s", g_error);
        return NULL;
    }
    PyObject *opts = options_dict(options);
    PyObject *handle = opts ? PyObject_CallMethod(g_module, function, "sIO", path, (unsigned int)seed, opts) : NULL;
    Py_XDECREF(opts);
    if (!handle) {
        take_exception();
    } else {
        model = (lm *)calloc(1, sizeof *model);
        if (model) model->handle = handle;
        else { Py_DECREF(handle); set_error("out of memory"); }
    }
    PyGILState_Release(gil);
    if (!model && err) snprintf(err, LM_ERROR_BYTES, "%s", g_error);
    return model;
}

API lm *lm_open(const char *folder, const lm_options *options, char err[LM_ERROR_BYTES]) {
    return open_with("open_folder", folder, 0, options, err);
}

API lm *lm_open_random(const char *config_json, uint32_t seed, const lm_options *options, char err[LM_ERROR_BYTES]) {
    return open_with("open_random", config_json, seed, options, err);
}

API void lm_close(lm *model) {
    if (!model) return;
    PyGILState_STATE gil = PyGILState_Ensure();
    PyObject *r = PyObject_CallMethod(g_module, "close", "O", model->handle);
    if (!r) take_exception();
    Py_XDECREF(r);
    Py_DECREF(model->handle);
    PyGILState_Release(gil);
    free(model);
}

/* Calls module.function(handle, ...) with the lock held; returns a new reference or NULL (status set). */
static PyObject *call(lm *model, const char *function, int *status, const char *format, ...) {
    va_list args;
    *status = LM_OK;
    if (!model || !model->handle || !g_module) {
        set_error("the model is not open");
        *status = LM_ERR_ARGUMENT;
        return NULL;
    }
    PyObject *callee = PyObject_GetAttrString(g_module, function);
    va_start(args, format);
    PyObject *rest = callee ? Py_VaBuildValue(format, args) : NULL;
    va_end(args);
    PyObject *result = NULL;
    if (rest) {
        Py_ssize_t n = PyTuple_Check(rest) ? PyTuple_Size(rest) : 1;
        PyObject *all = PyTuple_New(n + 1);
        if (all) {
            Py_INCREF(model->handle);
            PyTuple_SET_ITEM(all, 0, model->handle);
            for (Py_ssize_t i = 0; i < n; ++i) {
                PyObject *item = PyTuple_Check(rest) ? PyTuple_GET_ITEM(rest, i) : rest;
                Py_INCREF(item);
                PyTuple_SET_ITEM(all, i + 1, item);
            }
            result = PyObject_CallObject(callee, all);
            Py_DECREF(all);
        }
    }
    Py_XDECREF(rest);
    Py_XDECREF(callee);
    if (!result) *status = take_exception();
    return result;
}

API void lm_get_info(lm *model, lm_info *out) {
    if (!out) return;
    memset(out, 0, sizeof *out);
    if (!model) return;
    PyGILState_STATE gil = PyGILState_Ensure();
    int status;
    PyObject *r = call(model, "info", &status, "()");
    if (r) {
        int vocab = 0, context = 0, batch = 0, layers = 0, prompt = 0, generated = 0;
        long long weights = 0, cache = 0;
        double prefill = 0, decode = 0;
        if (PyArg_ParseTuple(r, "iiiiLLiidd", &vocab, &context, &batch, &layers, &weights, &cache, &prompt, &generated, &prefill, &decode)) {
            out->vocab_size = vocab; out->context = context; out->batch = batch; out->layers = layers;
            out->weight_bytes = weights; out->cache_bytes = cache; out->prompt_tokens = prompt;
            out->generated_tokens = generated; out->prefill_seconds = prefill; out->decode_seconds = decode;
        } else {
            take_exception();
        }
        Py_DECREF(r);
    }
    PyGILState_Release(gil);
}

API int lm_generate(lm *model, const lm_request *requests, int32_t n, const lm_generation *generation, const lm_sink *sink) {
    if (!requests || n <= 0) {
        set_error("at least one request is needed");
        return LM_ERR_ARGUMENT;
    }
    for (int32_t i = 0; i < n; ++i)
        if (!requests[i].tokens || requests[i].n <= 0) {
            set_error("every request needs at least one prompt token");
            return LM_ERR_ARGUMENT;
        }
    PyGILState_STATE gil = PyGILState_Ensure();
    int status;
    /* addresses travel as integers: the Python side reads the prompts and calls the sink through ctypes */
    PyObject *r = call(model, "generate", &status, "(KiKifif IKi)", (unsigned long long)(uintptr_t)requests, (int)n,
                       (unsigned long long)(uintptr_t)sink, generation ? generation->tokens : 0,
                       generation ? (double)generation->temperature : 0.0, generation ? generation->top_k : 40,
                       generation ? (double)generation->top_p : 0.0, generation ? (unsigned int)generation->seed : 0u,
                       (unsigned long long)(uintptr_t)(generation ? generation->stop_ids : NULL),
                       generation ? generation->n_stop_ids : -1);
    Py_XDECREF(r);
    PyGILState_Release(gil);
    return status;
}

static int call_int(lm *model, const char *function, int32_t argument, int with_argument) {
    PyGILState_STATE gil = PyGILState_Ensure();
    int status;
    PyObject *r = with_argument ? call(model, function, &status, "(i)", (int)argument) : call(model, function, &status, "()");
    int value = status;
    if (r) {
        value = (int)PyLong_AsLong(r);
        if (PyErr_Occurred()) value = take_exception();
        Py_DECREF(r);
    }
    PyGILState_Release(gil);
    return value;
}

API int lm_slot_alloc(lm *model) { return call_int(model, "slot_alloc", 0, 0); }
API int lm_slot_free(lm *model, int32_t slot) { return call_int(model, "slot_free", slot, 1); }
API int lm_slot_length(lm *model, int32_t slot) { return call_int(model, "slot_length", slot, 1); }

API int lm_step(lm *model, const int32_t *slots, const int32_t *counts, int32_t n_sequences, const int32_t *tokens,
                const uint8_t *want, float *logits) {
    if (!slots || !counts || !tokens || n_sequences <= 0) {
        set_error("a step needs sequences, their token counts and their tokens");
        return LM_ERR_ARGUMENT;
    }
    PyGILState_STATE gil = PyGILState_Ensure();
    int status;
    PyObject *r = call(model, "step", &status, "(KKiKKK)", (unsigned long long)(uintptr_t)slots, (unsigned long long)(uintptr_t)counts,
                       (int)n_sequences, (unsigned long long)(uintptr_t)tokens, (unsigned long long)(uintptr_t)want,
                       (unsigned long long)(uintptr_t)logits);
    Py_XDECREF(r);
    PyGILState_Release(gil);
    return status;
}

API const char *lm_last_error(void) { return g_error; }
