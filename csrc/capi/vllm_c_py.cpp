// C interface of the engine (include/vllm.h). The engine itself lives in Python objects; this
// layer embeds the interpreter (or joins the one already running when the library was loaded
// from Python), marshals the POD parameter structs into dicts, and calls the functions of
// vllm_cpp_b200.capi_bridge. No exception crosses the boundary: Python errors become a status
// code plus a thread-local message.
#include <Python.h>

#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "../../include/vllm.h"

namespace {

thread_local std::string g_last_error;
std::once_flag g_py_once;
bool g_we_initialised = false;

void set_error(const std::string& m) { g_last_error = m; }

void ensure_python() {
  std::call_once(g_py_once, [] {
    if (!Py_IsInitialized()) {
      Py_InitializeEx(0);
      g_we_initialised = true;
      // the thread that initialised holds the GIL: release it so that any thread may enter
      PyEval_SaveThread();
    }
  });
}

struct Gil {
  PyGILState_STATE st;
  Gil() { ensure_python(); st = PyGILState_Ensure(); }
  ~Gil() { PyGILState_Release(st); }
};

// Formats the pending Python exception into the thread-local message and clears it.
vllm_status take_py_error(vllm_status fallback) {
  PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  std::string msg = "unknown Python error";
  vllm_status st = fallback;
  if (value) {
    PyObject* s = PyObject_Str(value);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) msg = c;
      Py_DECREF(s);
    }
    if (type && PyErr_GivenExceptionMatches(type, PyExc_ValueError)) st = VLLM_ERR_INVALID_ARGUMENT;
    if (type && (PyErr_GivenExceptionMatches(type, PyExc_FileNotFoundError) ||
                 PyErr_GivenExceptionMatches(type, PyExc_ImportError)))
      st = VLLM_ERR_MODEL_LOAD;
    if (type) {
      PyObject* n = PyObject_GetAttrString(type, "__name__");
      if (n) {
        const char* c = PyUnicode_AsUTF8(n);
        if (c) msg = std::string(c) + ": " + msg;
        Py_DECREF(n);
      }
    }
  }
  PyErr_Clear();
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(tb);
  set_error(msg);
  return st;
}

PyObject* bridge() {   // borrowed-like: cached module (new reference kept forever)
  static PyObject* mod = nullptr;
  if (!mod) mod = PyImport_ImportModule("vllm_cpp_b200.capi_bridge");
  return mod;
}

void dict_set(PyObject* d, const char* k, PyObject* v) {   // steals v
  if (v) {
    PyDict_SetItemString(d, k, v);
    Py_DECREF(v);
  }
}
PyObject* str_or_none(const char* s) {
  if (!s) Py_RETURN_NONE;
  return PyUnicode_FromString(s);
}
PyObject* str_list(const char* const* items, size_t n) {
  PyObject* l = PyList_New(0);
  for (size_t i = 0; i < n; ++i) {
    if (!items || !items[i]) continue;
    PyObject* s = PyUnicode_FromString(items[i]);
    PyList_Append(l, s);
    Py_DECREF(s);
  }
  return l;
}

PyObject* sampling_dict(const vllm_sampling_params* p) {
  PyObject* d = PyDict_New();
  dict_set(d, "temperature", PyFloat_FromDouble(p->temperature));
  dict_set(d, "top_p", PyFloat_FromDouble(p->top_p));
  dict_set(d, "top_k", PyLong_FromLong(p->top_k));
  dict_set(d, "min_p", PyFloat_FromDouble(p->min_p));
  dict_set(d, "max_tokens", PyLong_FromLong(p->max_tokens));
  dict_set(d, "seed", PyLong_FromUnsignedLongLong(p->seed));
  dict_set(d, "has_seed", PyBool_FromLong(p->has_seed));
  dict_set(d, "presence_penalty", PyFloat_FromDouble(p->presence_penalty));
  dict_set(d, "frequency_penalty", PyFloat_FromDouble(p->frequency_penalty));
  dict_set(d, "repetition_penalty", PyFloat_FromDouble(p->repetition_penalty));
  dict_set(d, "min_tokens", PyLong_FromLong(p->min_tokens));
  dict_set(d, "ignore_eos", PyBool_FromLong(p->ignore_eos));
  dict_set(d, "stop", str_list(p->stop, p->n_stop));
  dict_set(d, "structured_json", str_or_none(p->structured_json));
  dict_set(d, "structured_regex", str_or_none(p->structured_regex));
  dict_set(d, "structured_choice", str_list(p->structured_choice, p->n_structured_choice));
  dict_set(d, "structured_grammar", str_or_none(p->structured_grammar));
  dict_set(d, "structured_json_object", PyBool_FromLong(p->structured_json_object));
  return d;
}

const char* static_reason(const std::string& r) {
  if (r == "stop") return "stop";
  if (r == "length") return "length";
  if (r == "abort") return "abort";
  if (r == "tool_calls") return "tool_calls";
  return "error";
}

char* dup_string(const std::string& s) {
  char* p = (char*)std::malloc(s.size() + 1);
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

}  // namespace

struct vllm_engine {
  PyObject* handle = nullptr;   // capi_bridge.EngineHandle
};

struct vllm_request {
  vllm_engine* engine = nullptr;
  std::string rid;
  vllm_token_callback cb = nullptr;
  void* user = nullptr;
  std::thread worker;
  std::mutex mu;
  std::condition_variable cv;
  std::atomic<bool> done{false};
  std::atomic<bool> cancelled{false};
  std::string error;
  bool has_error = false;
};

namespace {

// Drains the stream of `rid`, calling `cb` per delta. Needs the GIL. Fills the totals.
vllm_status drain(vllm_engine* e, const std::string& rid, vllm_token_callback cb, void* user,
                  std::string* text, std::string* reason, int* completion_tokens,
                  const std::atomic<bool>* cancelled) {
  PyObject* gen = PyObject_CallMethod(bridge(), "stream", "Os", e->handle, rid.c_str());
  if (!gen) return take_py_error(VLLM_ERR_RUNTIME);
  PyObject* it = PyObject_GetIter(gen);
  Py_DECREF(gen);
  if (!it) return take_py_error(VLLM_ERR_RUNTIME);
  vllm_status st = VLLM_OK;
  bool stopped = false;
  while (true) {
    PyObject* item;
    item = PyIter_Next(it);   // blocks inside Python (queue.get releases the GIL)
    if (!item) break;
    const char* delta = "";
    int finished = 0, ntok = 0;
    const char* fr = "";
    const char* err = "";
    if (!PyArg_ParseTuple(item, "spsis", &delta, &finished, &fr, &ntok, &err)) {
      Py_DECREF(item);
      st = take_py_error(VLLM_ERR_RUNTIME);
      break;
    }
    if (err && *err) {
      set_error(err);
      st = VLLM_ERR_RUNTIME;
      Py_DECREF(item);
      break;
    }
    if (text) text->append(delta);
    if (completion_tokens) *completion_tokens = ntok;
    if (finished && reason) *reason = fr;
    bool keep = true;
    if (cb && !stopped) {
      // the callback is foreign code: run it without the GIL
      std::string d(delta);
      Py_BEGIN_ALLOW_THREADS
      keep = cb(d.c_str(), finished != 0, user);
      Py_END_ALLOW_THREADS
    }
    Py_DECREF(item);
    if ((!keep || (cancelled && cancelled->load())) && !finished && !stopped) {
      stopped = true;
      PyObject* r = PyObject_CallMethod(bridge(), "abort", "Os", e->handle, rid.c_str());
      if (!r) PyErr_Clear();
      Py_XDECREF(r);
      if (reason) *reason = "abort";
    }
  }
  if (PyErr_Occurred()) st = take_py_error(VLLM_ERR_RUNTIME);
  Py_DECREF(it);
  return st;
}

vllm_status submit_locked(vllm_engine* e, const char* prompt, const vllm_sampling_params* p,
                          std::string* rid, int* prompt_tokens) {
  PyObject* sd = sampling_dict(p);
  PyObject* r = PyObject_CallMethod(bridge(), "submit", "OsO", e->handle, prompt, sd);
  Py_DECREF(sd);
  if (!r) return take_py_error(VLLM_ERR_RUNTIME);
  const char* id = nullptr;
  int np = 0;
  if (!PyArg_ParseTuple(r, "si", &id, &np)) {
    Py_DECREF(r);
    return take_py_error(VLLM_ERR_RUNTIME);
  }
  *rid = id;
  if (prompt_tokens) *prompt_tokens = np;
  Py_DECREF(r);
  return VLLM_OK;
}

}  // namespace

extern "C" {

vllm_model_params vllm_model_params_default(void) {
  vllm_model_params p;
  std::memset(&p, 0, sizeof p);
  p.block_size = 32;
  p.num_blocks = 256;
  p.max_model_len = 0;
  p.max_num_seqs = 8;
  return p;
}

vllm_sampling_params vllm_sampling_params_default(void) {
  vllm_sampling_params p;
  std::memset(&p, 0, sizeof p);
  p.temperature = 1.0f;
  p.top_p = 1.0f;
  p.top_k = 0;
  p.min_p = 0.0f;
  p.max_tokens = 16;
  p.repetition_penalty = 1.0f;
  return p;
}

vllm_status vllm_engine_load(const vllm_model_params* params, vllm_engine** out) {
  return vllm_engine_load_ex(params, nullptr, out);
}

vllm_status vllm_engine_load_ex(const vllm_model_params* params, const vllm_engine_options* options,
                                vllm_engine** out) {
  g_last_error.clear();
  if (!params || !out || !params->model_path || !*params->model_path) {
    set_error("vllm_engine_load: params, out and params->model_path are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  *out = nullptr;
  // options: the caller's struct may be older (smaller) than ours; read only what it has
  int32_t tp = 0, ep = 0;
  const char* device = nullptr;
  if (options) {
    auto has = [&](size_t off, size_t sz) { return options->struct_size >= off + sz; };
    if (has(offsetof(vllm_engine_options, tensor_parallel_size), sizeof(int32_t)))
      tp = options->tensor_parallel_size;
    if (has(offsetof(vllm_engine_options, enable_expert_parallel), sizeof(int32_t)))
      ep = options->enable_expert_parallel;
    if (has(offsetof(vllm_engine_options, device), sizeof(const char*))) device = options->device;
  } else {
    if (const char* v = std::getenv("VLLM_TENSOR_PARALLEL_SIZE")) tp = std::atoi(v);
    if (const char* v = std::getenv("VLLM_ENABLE_EXPERT_PARALLEL")) ep = std::atoi(v);
    device = std::getenv("VLLM_DEVICE");
  }
  Gil gil;
  if (!bridge()) return take_py_error(VLLM_ERR_MODEL_LOAD);
  PyObject* d = PyDict_New();
  dict_set(d, "model_path", PyUnicode_FromString(params->model_path));
  dict_set(d, "tokenizer_config_path", str_or_none(params->tokenizer_config_path));
  dict_set(d, "block_size", PyLong_FromLong(params->block_size > 0 ? params->block_size : 32));
  dict_set(d, "num_blocks", PyLong_FromLong(params->num_blocks > 0 ? params->num_blocks : 256));
  dict_set(d, "max_model_len", PyLong_FromLong(params->max_model_len > 0 ? params->max_model_len : 0));
  dict_set(d, "max_num_seqs", PyLong_FromLong(params->max_num_seqs > 0 ? params->max_num_seqs : 8));
  dict_set(d, "tool_parser", str_or_none(params->tool_parser && *params->tool_parser ? params->tool_parser : nullptr));
  dict_set(d, "reasoning_parser", str_or_none(params->reasoning_parser));
  dict_set(d, "tensor_parallel_size", PyLong_FromLong(tp > 0 ? tp : 1));
  dict_set(d, "enable_expert_parallel", PyBool_FromLong(ep != 0));
  dict_set(d, "device", str_or_none(device));
  PyObject* h = PyObject_CallMethod(bridge(), "load", "O", d);
  Py_DECREF(d);
  if (!h) return take_py_error(VLLM_ERR_MODEL_LOAD);
  vllm_engine* e = new (std::nothrow) vllm_engine();
  if (!e) {
    Py_DECREF(h);
    set_error("out of memory");
    return VLLM_ERR_RUNTIME;
  }
  e->handle = h;
  *out = e;
  return VLLM_OK;
}

void vllm_engine_free(vllm_engine* engine) {
  if (!engine) return;
  {
    Gil gil;
    if (engine->handle) {
      PyObject* r = PyObject_CallMethod(engine->handle, "close", nullptr);
      if (!r) PyErr_Clear();
      Py_XDECREF(r);
      Py_DECREF(engine->handle);
    }
  }
  delete engine;
}

vllm_status vllm_complete_stream(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                                 vllm_token_callback cb, void* user) {
  g_last_error.clear();
  if (!engine || !prompt || !params) {
    set_error("vllm_complete_stream: engine, prompt and params are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  Gil gil;
  std::string rid;
  vllm_status st = submit_locked(engine, prompt, params, &rid, nullptr);
  if (st != VLLM_OK) return st;
  return drain(engine, rid, cb, user, nullptr, nullptr, nullptr, nullptr);
}

vllm_status vllm_complete(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                          vllm_completion* out) {
  g_last_error.clear();
  if (!engine || !prompt || !params || !out) {
    set_error("vllm_complete: engine, prompt, params and out are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  std::memset(out, 0, sizeof *out);
  Gil gil;
  std::string rid, text, reason;
  int np = 0, nc = 0;
  vllm_status st = submit_locked(engine, prompt, params, &rid, &np);
  if (st != VLLM_OK) return st;
  st = drain(engine, rid, nullptr, nullptr, &text, &reason, &nc, nullptr);
  if (st != VLLM_OK) return st;
  out->text = dup_string(text);
  out->finish_reason = static_reason(reason);
  out->prompt_tokens = np;
  out->completion_tokens = nc;
  return VLLM_OK;
}

vllm_status vllm_request_submit(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                                vllm_token_callback cb, void* user, vllm_request** out) {
  g_last_error.clear();
  if (!engine || !prompt || !params || !out) {
    set_error("vllm_request_submit: engine, prompt, params and out are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  *out = nullptr;
  vllm_request* r = new (std::nothrow) vllm_request();
  if (!r) {
    set_error("out of memory");
    return VLLM_ERR_RUNTIME;
  }
  r->engine = engine;
  r->cb = cb;
  r->user = user;
  {
    Gil gil;
    vllm_status st = submit_locked(engine, prompt, params, &r->rid, nullptr);
    if (st != VLLM_OK) {
      delete r;
      return st;
    }
  }
  r->worker = std::thread([r] {
    {
      Gil gil;
      vllm_status st = drain(r->engine, r->rid, r->cb, r->user, nullptr, nullptr, nullptr, &r->cancelled);
      if (st != VLLM_OK) {
        r->error = g_last_error;
        r->has_error = true;
      }
    }
    {
      std::lock_guard<std::mutex> lock(r->mu);
      r->done.store(true);
    }
    r->cv.notify_all();
  });
  *out = r;
  return VLLM_OK;
}

vllm_status vllm_request_cancel(vllm_request* request) {
  if (!request) {
    set_error("vllm_request_cancel: request is NULL");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (request->done.load() || request->cancelled.exchange(true)) return VLLM_OK;
  Gil gil;
  PyObject* r = PyObject_CallMethod(bridge(), "abort", "Os", request->engine->handle, request->rid.c_str());
  if (!r) PyErr_Clear();
  Py_XDECREF(r);
  return VLLM_OK;
}

vllm_status vllm_request_wait(vllm_request* request) {
  if (!request) {
    set_error("vllm_request_wait: request is NULL");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  std::unique_lock<std::mutex> lock(request->mu);
  request->cv.wait(lock, [request] { return request->done.load(); });
  if (request->has_error) {
    set_error(request->error);
    return VLLM_ERR_RUNTIME;
  }
  return VLLM_OK;
}

bool vllm_request_done(const vllm_request* request) { return !request || request->done.load(); }

const char* vllm_request_error(const vllm_request* request) {
  return (request && request->done.load() && request->has_error) ? request->error.c_str() : nullptr;
}

void vllm_request_free(vllm_request* request) {
  if (!request) return;
  if (!request->done.load()) vllm_request_cancel(request);
  if (request->worker.joinable()) request->worker.join();
  delete request;
}

vllm_status vllm_chat(vllm_engine* engine, const char* request_json, char** out_json) {
  g_last_error.clear();
  if (!engine || !request_json || !out_json) {
    set_error("vllm_chat: engine, request_json and out_json are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  *out_json = nullptr;
  Gil gil;
  PyObject* r = PyObject_CallMethod(bridge(), "chat", "Os", engine->handle, request_json);
  if (!r) return take_py_error(VLLM_ERR_RUNTIME);
  const char* s = PyUnicode_AsUTF8(r);
  if (!s) {
    Py_DECREF(r);
    return take_py_error(VLLM_ERR_RUNTIME);
  }
  *out_json = dup_string(s);
  Py_DECREF(r);
  return VLLM_OK;
}

namespace {
struct ChunkSink {
  vllm_token_callback cb;
  void* user;
};
PyObject* chunk_trampoline(PyObject* self, PyObject* args) {
  ChunkSink* sink = (ChunkSink*)PyCapsule_GetPointer(self, "vllm.chunk_sink");
  const char* text = nullptr;
  if (!sink || !PyArg_ParseTuple(args, "s", &text)) return nullptr;
  const bool last = std::strcmp(text, "[DONE]") == 0;
  bool keep = true;
  if (sink->cb) {
    std::string t(last ? "" : text);
    Py_BEGIN_ALLOW_THREADS
    keep = sink->cb(t.c_str(), last, sink->user);
    Py_END_ALLOW_THREADS
  }
  return PyBool_FromLong(keep);
}
PyMethodDef g_chunk_def = {"on_chunk", chunk_trampoline, METH_VARARGS, "forwards one chunk to the C callback"};
}  // namespace

vllm_status vllm_chat_stream(vllm_engine* engine, const char* request_json, vllm_token_callback cb, void* user) {
  g_last_error.clear();
  if (!engine || !request_json) {
    set_error("vllm_chat_stream: engine and request_json are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  Gil gil;
  ChunkSink sink{cb, user};
  PyObject* cap = PyCapsule_New(&sink, "vllm.chunk_sink", nullptr);
  PyObject* fn = PyCFunction_New(&g_chunk_def, cap);
  Py_DECREF(cap);
  PyObject* r = PyObject_CallMethod(bridge(), "chat_stream", "OsO", engine->handle, request_json, fn);
  Py_DECREF(fn);
  if (!r) return take_py_error(VLLM_ERR_RUNTIME);
  Py_DECREF(r);
  return VLLM_OK;
}

void vllm_string_free(char* s) { std::free(s); }

void vllm_completion_free(vllm_completion* c) {
  if (!c) return;
  std::free(c->text);
  c->text = nullptr;
}

const char* vllm_last_error(void) { return g_last_error.c_str(); }
const char* vllm_version(void) { return "0.1.0"; }
int32_t vllm_abi_version(void) { return VLLM_ABI_VERSION; }

}  // extern "C"
