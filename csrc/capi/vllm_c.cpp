// C interface of the engine (include/vllm.h) over the native runtime: scheduler, engine core,
// model runner, dense model, tokenizer and sampler are all C++ (csrc/engine, csrc/runtime), the
// kernels come from the CUDA library or the CPU thread-pool kernels, memory comes from libtorch.
// No interpreter is linked or started.
//
// One engine thread per handle owns the engine: API calls post commands to it and deltas are
// delivered from it ("a thread the library owns"). Architectures the native runtime does not
// cover are served by the Python-hosted build of the same interface (libvllm_b200_py.so, loaded
// on demand from the directory of this library), so one library name serves every model.
//
// Reference: src/capi/vllm_c.cpp:404-855 (engine handle, completion, streaming, requests),
// src/capi/chat_prompt.cpp (chat entry points).
#include <dlfcn.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <future>
#include <map>
#include <mutex>
#include <string>
#include <thread>

#include "../../include/vllm.h"
#include "runtime/native_llm.h"
#include "util/json.h"

using b200::Json;
using b200::SamplingParams;
using b200::rt::NativeLLM;
using b200::rt::RequestDelta;

namespace {

thread_local std::string g_last_error;
void set_error(const std::string& m) { g_last_error = m; }

// ---- the Python-hosted build, loaded only when the native runtime does not cover the model ----
struct PyLib {
  void* h = nullptr;
  decltype(&vllm_engine_load_ex) load_ex = nullptr;
  decltype(&vllm_engine_free) engine_free = nullptr;
  decltype(&vllm_complete) complete = nullptr;
  decltype(&vllm_complete_stream) complete_stream = nullptr;
  decltype(&vllm_request_submit) request_submit = nullptr;
  decltype(&vllm_request_cancel) request_cancel = nullptr;
  decltype(&vllm_request_wait) request_wait = nullptr;
  decltype(&vllm_request_done) request_done = nullptr;
  decltype(&vllm_request_error) request_error = nullptr;
  decltype(&vllm_request_free) request_free = nullptr;
  decltype(&vllm_chat) chat = nullptr;
  decltype(&vllm_chat_stream) chat_stream = nullptr;
  decltype(&vllm_last_error) last_error = nullptr;
};
PyLib* py_lib() {
  static PyLib lib;
  static std::once_flag once;
  std::call_once(once, [] {
    Dl_info info{};
    std::string dir = ".";
    if (dladdr((void*)&set_error, &info) && info.dli_fname) {
      std::string p = info.dli_fname;
      auto s = p.rfind('/');
      if (s != std::string::npos) dir = p.substr(0, s);
    }
    void* h = dlopen((dir + "/libvllm_b200_py.so").c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    lib.h = h;
#define B200_SYM(field, name) lib.field = reinterpret_cast<decltype(lib.field)>(dlsym(h, name))
    B200_SYM(load_ex, "vllm_engine_load_ex");
    B200_SYM(engine_free, "vllm_engine_free");
    B200_SYM(complete, "vllm_complete");
    B200_SYM(complete_stream, "vllm_complete_stream");
    B200_SYM(request_submit, "vllm_request_submit");
    B200_SYM(request_cancel, "vllm_request_cancel");
    B200_SYM(request_wait, "vllm_request_wait");
    B200_SYM(request_done, "vllm_request_done");
    B200_SYM(request_error, "vllm_request_error");
    B200_SYM(request_free, "vllm_request_free");
    B200_SYM(chat, "vllm_chat");
    B200_SYM(chat_stream, "vllm_chat_stream");
    B200_SYM(last_error, "vllm_last_error");
#undef B200_SYM
  });
  return lib.h && lib.load_ex ? &lib : nullptr;
}

// ---- per-request delivery state --------------------------------------------------------------
struct Sink {
  vllm_token_callback cb = nullptr;
  void* user = nullptr;
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::string error;
  std::string text;
  std::string finish_reason;
  int prompt_tokens = 0, completion_tokens = 0;
  std::string rid;
  std::atomic<bool> cancelled{false};
  // chat streaming: deltas are wrapped into chat.completion.chunk objects
  std::function<std::string(const std::string& delta, bool first, bool finished, const std::string& reason)> wrap;
  bool first = true;
};

struct Command {
  enum Kind { kAdd, kAbort, kStop } kind = kAdd;
  std::string prompt;
  SamplingParams params;
  std::shared_ptr<Sink> sink;
  std::string rid;
  std::promise<std::string> reply;     // request id, or an exception
};

}  // namespace

struct vllm_engine {
  vllm_engine* py = nullptr;           // the handle of the Python-hosted build (then nothing else is used)
  std::unique_ptr<NativeLLM> llm;
  std::string model_name;
  std::thread loop;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::unique_ptr<Command>> queue;
  std::map<std::string, std::shared_ptr<Sink>> sinks;   // engine thread only
  std::string dead;                    // non-empty: the engine thread died with this message
  bool stopping = false;

  void run();
  void finish(const std::shared_ptr<Sink>& s, const std::string& err);
};

struct vllm_request {
  vllm_request* py = nullptr;
  vllm_engine* engine = nullptr;
  std::shared_ptr<Sink> sink;
};

namespace {

void deliver(const std::shared_ptr<Sink>& s, const std::string& delta, bool finished, const std::string& reason,
             vllm_engine* e) {
  if (!s->cb || s->cancelled.load()) return;
  std::string payload = delta;
  if (s->wrap) payload = s->wrap(delta, s->first, finished, reason);
  s->first = false;
  if (s->wrap) {
    // chat streaming: every chunk is a JSON object; the stream ends with ("", finished)
    if (!payload.empty() && !s->cb(payload.c_str(), false, s->user)) s->cancelled.store(true);
    if (finished && !s->cancelled.load()) s->cb("", true, s->user);
  } else if (!s->cb(payload.c_str(), finished, s->user)) {
    s->cancelled.store(true);
  }
  if (s->cancelled.load() && !finished) e->llm->abort(s->rid);
}

}  // namespace

void vllm_engine::finish(const std::shared_ptr<Sink>& s, const std::string& err) {
  {
    std::lock_guard<std::mutex> l(s->mu);
    s->done = true;
    if (!err.empty()) s->error = err;
  }
  s->cv.notify_all();
}

void vllm_engine::run() {
  for (;;) {
    std::deque<std::unique_ptr<Command>> cmds;
    {
      std::unique_lock<std::mutex> l(mu);
      cv.wait(l, [&] { return stopping || !queue.empty() || (llm && llm->has_unfinished()); });
      if (stopping) break;
      cmds.swap(queue);
    }
    for (auto& c : cmds) {
      try {
        if (c->kind == Command::kAdd) {
          const std::string rid = llm->add_request(c->prompt, c->params);
          c->sink->rid = rid;
          sinks[rid] = c->sink;
          c->reply.set_value(rid);
        } else if (c->kind == Command::kAbort) {
          auto it = sinks.find(c->rid);
          if (it != sinks.end()) {
            llm->abort(c->rid);
            it->second->finish_reason = "abort";
            auto s = it->second;
            sinks.erase(it);
            finish(s, "");
          }
          c->reply.set_value(c->rid);
        }
      } catch (...) {
        c->reply.set_exception(std::current_exception());
      }
    }
    if (!llm->has_unfinished()) continue;
    std::vector<RequestDelta> deltas;
    try {
      deltas = llm->step();
    } catch (const std::exception& ex) {
      // the engine is dead for every waiter (reference: core_proc.cpp:140-146)
      std::lock_guard<std::mutex> l(mu);
      dead = ex.what();
      for (auto& kv : sinks) finish(kv.second, dead);
      sinks.clear();
      stopping = true;
      break;
    }
    for (auto& d : deltas) {
      auto it = sinks.find(d.request_id);
      if (it == sinks.end()) continue;
      auto s = it->second;
      s->text += d.delta_text;
      s->prompt_tokens = d.prompt_tokens;
      s->completion_tokens = d.completion_tokens;
      if (d.finished) s->finish_reason = d.finish_reason;
      const bool was_cancelled = s->cancelled.load();
      if (!d.delta_text.empty() || d.finished) deliver(s, d.delta_text, d.finished, d.finish_reason, this);
      if (d.finished || (s->cancelled.load() && !was_cancelled)) {
        if (!d.finished) s->finish_reason = "abort";
        sinks.erase(d.request_id);
        finish(s, "");
      }
    }
  }
  // stopping: nobody may wait for ever
  for (auto& kv : sinks) finish(kv.second, dead.empty() ? "engine shut down" : dead);
  sinks.clear();
}

namespace {

const char* static_reason(const std::string& r) {
  if (r == "stop") return "stop";
  if (r == "length") return "length";
  return "abort";
}

// vllm_sampling_params -> SamplingParams; throws std::invalid_argument on a bad field.
SamplingParams to_params(const vllm_sampling_params* p) {
  SamplingParams sp;
  if (!(p->repetition_penalty > 0.f))
    throw std::invalid_argument("repetition_penalty must be > 0 (start from vllm_sampling_params_default())");
  sp.temperature = p->temperature;
  sp.top_p = p->top_p;
  sp.top_k = p->top_k;
  sp.min_p = p->min_p;
  if (p->max_tokens > 0) sp.max_tokens = p->max_tokens;
  else sp.max_tokens = std::nullopt;
  if (p->has_seed) sp.seed = p->seed;
  sp.presence_penalty = p->presence_penalty;
  sp.frequency_penalty = p->frequency_penalty;
  sp.repetition_penalty = p->repetition_penalty;
  sp.min_tokens = p->min_tokens;
  sp.ignore_eos = p->ignore_eos != 0;
  for (int i = 0; i < p->n_stop; ++i)
    if (p->stop && p->stop[i]) sp.stop.emplace_back(p->stop[i]);
  b200::StructuredOutputsParams so;
  if (p->structured_json) so.json = p->structured_json;
  if (p->structured_regex) so.regex = p->structured_regex;
  if (p->structured_choice && p->n_structured_choice > 0) {
    so.choice = std::vector<std::string>();
    for (int i = 0; i < p->n_structured_choice; ++i)
      if (p->structured_choice[i]) so.choice->emplace_back(p->structured_choice[i]);
  }
  if (p->structured_grammar) so.grammar = p->structured_grammar;
  so.json_object = p->structured_json_object != 0;
  if (so.count() > 1) throw std::invalid_argument("at most one structured-output constraint may be set");
  if (so.any()) sp.structured_outputs = so;
  sp.output_kind = b200::OutputKind::kDelta;
  return sp;
}

// Posts an add command and waits for the engine thread's answer. Returns the sink or sets the error.
vllm_status submit(vllm_engine* e, const std::string& prompt, SamplingParams sp, vllm_token_callback cb, void* user,
                   std::shared_ptr<Sink>* out, decltype(Sink::wrap) wrap = nullptr) {
  auto c = std::make_unique<Command>();
  c->kind = Command::kAdd;
  c->prompt = prompt;
  c->params = std::move(sp);
  c->sink = std::make_shared<Sink>();
  c->sink->cb = cb;
  c->sink->user = user;
  c->sink->wrap = std::move(wrap);
  auto sink = c->sink;
  auto fut = c->reply.get_future();
  {
    std::lock_guard<std::mutex> l(e->mu);
    if (e->stopping || !e->dead.empty()) {
      set_error(e->dead.empty() ? "the engine is shutting down" : "the engine is dead: " + e->dead);
      return VLLM_ERR_RUNTIME;
    }
    e->queue.push_back(std::move(c));
  }
  e->cv.notify_all();
  try {
    fut.get();
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  } catch (const std::exception& ex) {
    set_error(ex.what());
    return VLLM_ERR_RUNTIME;
  }
  *out = sink;
  return VLLM_OK;
}

vllm_status wait_sink(const std::shared_ptr<Sink>& s) {
  std::unique_lock<std::mutex> l(s->mu);
  s->cv.wait(l, [&] { return s->done; });
  if (!s->error.empty()) {
    set_error(s->error);
    return VLLM_ERR_RUNTIME;
  }
  return VLLM_OK;
}

char* dup_cstr(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

// ---- chat: OpenAI request JSON -> prompt + sampling parameters -----------------------------------
std::string content_text(const Json& c) {
  if (c.is_string()) return c.as_string();
  std::string out;                       // [{"type": "text", "text": ...}, ...]
  for (auto& part : c.items())
    if (part["type"].as_string() == "text") out += part["text"].as_string();
  return out;
}

// The two formats the native runtime renders itself; anything else (tools, other templates)
// is served by the Python-hosted build, which evaluates the checkpoint's Jinja template.
std::string render_chat(const Json& messages, const std::string& style) {
  std::string p;
  if (style == "llama3") {
    p = "<|begin_of_text|>";
    for (auto& m : messages.items())
      p += "<|start_header_id|>" + m["role"].as_string() + "<|end_header_id|>\n\n" + content_text(m["content"]) +
           "<|eot_id|>";
    p += "<|start_header_id|>assistant<|end_header_id|>\n\n";
  } else {
    for (auto& m : messages.items())
      p += "<|im_start|>" + m["role"].as_string() + "\n" + content_text(m["content"]) + "<|im_end|>\n";
    p += "<|im_start|>assistant\n";
  }
  return p;
}

struct ChatRequest {
  std::string prompt;
  SamplingParams params;
  std::string model;
};

ChatRequest parse_chat(vllm_engine* e, const char* request_json, const std::string& style) {
  Json req;
  std::string err;
  if (!Json::try_parse(request_json, &req, &err) || !req.is_object())
    throw std::invalid_argument("request is not a JSON object: " + err);
  const Json& msgs = req["messages"];
  if (!msgs.is_array() || msgs.size() == 0) throw std::invalid_argument("messages must be a non-empty array");
  if (req["tools"].is_array() && req["tools"].size() > 0)
    throw std::invalid_argument("tool calling is served by the Python-hosted library (libvllm_b200_py.so)");
  ChatRequest out;
  out.model = req["model"].is_string() ? req["model"].as_string() : e->model_name;
  out.prompt = render_chat(msgs, style);
  SamplingParams& sp = out.params;
  sp.temperature = req["temperature"].as_double(1.0);
  sp.top_p = req["top_p"].as_double(1.0);
  sp.top_k = (int)req["top_k"].as_int(0);
  sp.min_p = req["min_p"].as_double(0.0);
  int64_t mt = req["max_completion_tokens"].is_number() ? req["max_completion_tokens"].as_int()
                                                         : req["max_tokens"].as_int(256);
  sp.max_tokens = (int)mt;
  if (req["seed"].is_number()) sp.seed = (uint64_t)req["seed"].as_int();
  sp.presence_penalty = req["presence_penalty"].as_double(0.0);
  sp.frequency_penalty = req["frequency_penalty"].as_double(0.0);
  sp.repetition_penalty = req["repetition_penalty"].as_double(1.0);
  if (req["stop"].is_string()) sp.stop.push_back(req["stop"].as_string());
  for (auto& s : req["stop"].items()) sp.stop.push_back(s.as_string());
  b200::StructuredOutputsParams so;
  if (req["guided_choice"].is_array()) {
    so.choice = std::vector<std::string>();
    for (auto& c : req["guided_choice"].items()) so.choice->push_back(c.as_string());
  }
  if (req["guided_json"].is_object()) so.json = req["guided_json"].dump();
  if (req["guided_json"].is_string()) so.json = req["guided_json"].as_string();
  if (req["guided_regex"].is_string()) so.regex = req["guided_regex"].as_string();
  if (req["guided_grammar"].is_string()) so.grammar = req["guided_grammar"].as_string();
  const Json& rf = req["response_format"];
  if (rf.is_object()) {
    if (rf["type"].as_string() == "json_object") so.json_object = true;
    if (rf["type"].as_string() == "json_schema") so.json = rf["json_schema"]["schema"].dump();
  }
  if (so.any()) sp.structured_outputs = so;
  sp.output_kind = b200::OutputKind::kDelta;
  return out;
}

int64_t unix_time() {
  return std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

std::string chat_style(vllm_engine* e) {
  const b200::tok::Tokenizer* tk = e->llm->tokenizer();
  if (tk && tk->token_to_id("<|start_header_id|>") >= 0) return "llama3";
  return "chatml";
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
  int32_t tp = 0;
  const char* device = nullptr;
  if (options) {
    auto has = [&](size_t off, size_t sz) { return options->struct_size >= off + sz; };
    if (has(offsetof(vllm_engine_options, tensor_parallel_size), sizeof(int32_t))) tp = options->tensor_parallel_size;
    if (has(offsetof(vllm_engine_options, device), sizeof(const char*))) device = options->device;
  } else {
    if (const char* v = std::getenv("VLLM_TENSOR_PARALLEL_SIZE")) tp = std::atoi(v);
    device = std::getenv("VLLM_DEVICE");
  }
  const char* force_py = std::getenv("VLLM_ENGINE");     // "python": always the Python-hosted build
  std::string native_error;
  if (tp <= 1 && !(force_py && std::string(force_py) == "python")) {
    try {
      b200::rt::EngineOptions o;
      o.model_path = params->model_path;
      if (params->tokenizer_config_path) {
        // the reference takes the path of tokenizer_config.json; the tokenizer lives beside it
        std::string t = params->tokenizer_config_path;
        auto s = t.rfind('/');
        o.tokenizer_path = s == std::string::npos ? "." : t.substr(0, s);
      }
      o.device = device ? device : "cuda";
      o.block_size = params->block_size > 0 ? params->block_size : 32;
      o.num_blocks = params->num_blocks > 0 ? params->num_blocks : 256;
      o.max_model_len = params->max_model_len > 0 ? params->max_model_len : 0;
      o.max_num_seqs = params->max_num_seqs > 0 ? params->max_num_seqs : 8;
      auto llm = NativeLLM::load(o);
      auto* e = new vllm_engine();
      e->llm = std::move(llm);
      e->model_name = params->model_path;
      e->loop = std::thread([e] { e->run(); });
      *out = e;
      return VLLM_OK;
    } catch (const std::exception& ex) {
      native_error = ex.what();
      if (native_error.find("not covered by the native runtime") == std::string::npos &&
          native_error.find("native runtime loads") == std::string::npos &&
          native_error.find("native runtime takes") == std::string::npos) {
        set_error(native_error);
        return VLLM_ERR_MODEL_LOAD;
      }
    }
  }
  PyLib* py = py_lib();
  if (!py) {
    set_error((native_error.empty() ? std::string("tensor parallel serving") : native_error) +
              "; the Python-hosted library (libvllm_b200_py.so) that serves it could not be loaded");
    return VLLM_ERR_MODEL_LOAD;
  }
  vllm_engine* inner = nullptr;
  const vllm_status st = py->load_ex(params, options, &inner);
  if (st != VLLM_OK) {
    set_error(py->last_error ? py->last_error() : "engine load failed");
    return st;
  }
  auto* e = new vllm_engine();
  e->py = inner;
  *out = e;
  return VLLM_OK;
}

void vllm_engine_free(vllm_engine* engine) {
  if (!engine) return;
  if (engine->py) {
    py_lib()->engine_free(engine->py);
    delete engine;
    return;
  }
  {
    std::lock_guard<std::mutex> l(engine->mu);
    engine->stopping = true;
  }
  engine->cv.notify_all();
  if (engine->loop.joinable()) engine->loop.join();
  delete engine;
}

#define B200_FORWARD_ERR(st) \
  do { if ((st) != VLLM_OK && py_lib()->last_error) set_error(py_lib()->last_error()); } while (0)

vllm_status vllm_complete(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                          vllm_completion* out) {
  g_last_error.clear();
  if (!engine || !prompt || !params || !out) {
    set_error("vllm_complete: engine, prompt, params and out are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (engine->py) {
    const vllm_status st = py_lib()->complete(engine->py, prompt, params, out);
    B200_FORWARD_ERR(st);
    return st;
  }
  std::memset(out, 0, sizeof *out);
  std::shared_ptr<Sink> s;
  try {
    const vllm_status st = submit(engine, prompt, to_params(params), nullptr, nullptr, &s);
    if (st != VLLM_OK) return st;
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  const vllm_status st = wait_sink(s);
  if (st != VLLM_OK) return st;
  out->text = dup_cstr(s->text);
  out->finish_reason = static_reason(s->finish_reason);
  out->prompt_tokens = s->prompt_tokens;
  out->completion_tokens = s->completion_tokens;
  return out->text ? VLLM_OK : VLLM_ERR_RUNTIME;
}

vllm_status vllm_complete_stream(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                                 vllm_token_callback cb, void* user) {
  g_last_error.clear();
  if (!engine || !prompt || !params || !cb) {
    set_error("vllm_complete_stream: engine, prompt, params and cb are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (engine->py) {
    const vllm_status st = py_lib()->complete_stream(engine->py, prompt, params, cb, user);
    B200_FORWARD_ERR(st);
    return st;
  }
  std::shared_ptr<Sink> s;
  try {
    const vllm_status st = submit(engine, prompt, to_params(params), cb, user, &s);
    if (st != VLLM_OK) return st;
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  return wait_sink(s);
}

vllm_status vllm_request_submit(vllm_engine* engine, const char* prompt, const vllm_sampling_params* params,
                                vllm_token_callback cb, void* user, vllm_request** out) {
  g_last_error.clear();
  if (!engine || !prompt || !params || !out) {
    set_error("vllm_request_submit: engine, prompt, params and out are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  *out = nullptr;
  if (engine->py) {
    vllm_request* inner = nullptr;
    const vllm_status st = py_lib()->request_submit(engine->py, prompt, params, cb, user, &inner);
    B200_FORWARD_ERR(st);
    if (st != VLLM_OK) return st;
    auto* r = new vllm_request();
    r->py = inner;
    *out = r;
    return VLLM_OK;
  }
  std::shared_ptr<Sink> s;
  try {
    const vllm_status st = submit(engine, prompt, to_params(params), cb, user, &s);
    if (st != VLLM_OK) return st;
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  auto* r = new vllm_request();
  r->engine = engine;
  r->sink = s;
  *out = r;
  return VLLM_OK;
}

vllm_status vllm_request_cancel(vllm_request* request) {
  if (!request) {
    set_error("vllm_request_cancel: request is NULL");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (request->py) return py_lib()->request_cancel(request->py);
  {
    std::lock_guard<std::mutex> l(request->sink->mu);
    if (request->sink->done) return VLLM_OK;
  }
  if (request->sink->cancelled.exchange(true)) return VLLM_OK;
  auto c = std::make_unique<Command>();
  c->kind = Command::kAbort;
  c->rid = request->sink->rid;
  auto fut = c->reply.get_future();
  {
    std::lock_guard<std::mutex> l(request->engine->mu);
    if (request->engine->stopping) return VLLM_OK;
    request->engine->queue.push_back(std::move(c));
  }
  request->engine->cv.notify_all();
  try {
    fut.get();
  } catch (...) {
  }
  return VLLM_OK;
}

vllm_status vllm_request_wait(vllm_request* request) {
  if (!request) {
    set_error("vllm_request_wait: request is NULL");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (request->py) return py_lib()->request_wait(request->py);
  return wait_sink(request->sink);
}

bool vllm_request_done(const vllm_request* request) {
  if (!request) return true;
  if (request->py) return py_lib()->request_done(request->py);
  std::lock_guard<std::mutex> l(request->sink->mu);
  return request->sink->done;
}

const char* vllm_request_error(const vllm_request* request) {
  if (!request) return nullptr;
  if (request->py) return py_lib()->request_error(request->py);
  std::lock_guard<std::mutex> l(request->sink->mu);
  return request->sink->error.empty() ? nullptr : request->sink->error.c_str();
}

void vllm_request_free(vllm_request* request) {
  if (!request) return;
  if (request->py) {
    py_lib()->request_free(request->py);
    delete request;
    return;
  }
  if (!vllm_request_done(request)) {
    vllm_request_cancel(request);
    wait_sink(request->sink);
  }
  delete request;
}

vllm_status vllm_chat(vllm_engine* engine, const char* request_json, char** out_json) {
  g_last_error.clear();
  if (!engine || !request_json || !out_json) {
    set_error("vllm_chat: engine, request_json and out_json are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  *out_json = nullptr;
  if (engine->py) {
    const vllm_status st = py_lib()->chat(engine->py, request_json, out_json);
    B200_FORWARD_ERR(st);
    return st;
  }
  std::shared_ptr<Sink> s;
  ChatRequest cr;
  try {
    cr = parse_chat(engine, request_json, chat_style(engine));
    const vllm_status st = submit(engine, cr.prompt, cr.params, nullptr, nullptr, &s);
    if (st != VLLM_OK) return st;
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  const vllm_status st = wait_sink(s);
  if (st != VLLM_OK) return st;
  Json msg = Json::object();
  msg["role"] = "assistant";
  msg["content"] = s->text;
  Json choice = Json::object();
  choice["index"] = 0;
  choice["message"] = msg;
  choice["finish_reason"] = static_reason(s->finish_reason);
  Json usage = Json::object();
  usage["prompt_tokens"] = s->prompt_tokens;
  usage["completion_tokens"] = s->completion_tokens;
  usage["total_tokens"] = s->prompt_tokens + s->completion_tokens;
  Json resp = Json::object();
  resp["id"] = "chatcmpl-" + s->rid;
  resp["object"] = "chat.completion";
  resp["created"] = unix_time();
  resp["model"] = cr.model;
  Json choices = Json::array();
  choices.push_back(choice);
  resp["choices"] = choices;
  resp["usage"] = usage;
  *out_json = dup_cstr(resp.dump());
  return *out_json ? VLLM_OK : VLLM_ERR_RUNTIME;
}

vllm_status vllm_chat_stream(vllm_engine* engine, const char* request_json, vllm_token_callback cb, void* user) {
  g_last_error.clear();
  if (!engine || !request_json || !cb) {
    set_error("vllm_chat_stream: engine, request_json and cb are required");
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  if (engine->py) {
    const vllm_status st = py_lib()->chat_stream(engine->py, request_json, cb, user);
    B200_FORWARD_ERR(st);
    return st;
  }
  std::shared_ptr<Sink> s;
  try {
    ChatRequest cr = parse_chat(engine, request_json, chat_style(engine));
    const int64_t created = unix_time();
    const std::string model = cr.model;
    auto wrap = [created, model](const std::string& delta, bool first, bool finished, const std::string& reason) {
      Json d = Json::object();
      if (first) d["role"] = "assistant";
      d["content"] = delta;
      Json choice = Json::object();
      choice["index"] = 0;
      choice["delta"] = d;
      choice["finish_reason"] = finished ? Json(static_reason(reason)) : Json(nullptr);
      Json chunk = Json::object();
      chunk["id"] = "chatcmpl-stream";
      chunk["object"] = "chat.completion.chunk";
      chunk["created"] = created;
      chunk["model"] = model;
      Json choices = Json::array();
      choices.push_back(choice);
      chunk["choices"] = choices;
      return chunk.dump();
    };
    const vllm_status st = submit(engine, cr.prompt, cr.params, cb, user, &s, wrap);
    if (st != VLLM_OK) return st;
  } catch (const std::invalid_argument& ex) {
    set_error(ex.what());
    return VLLM_ERR_INVALID_ARGUMENT;
  }
  return wait_sink(s);
}

void vllm_string_free(char* s) { std::free(s); }

void vllm_completion_free(vllm_completion* c) {
  if (!c) return;
  std::free(c->text);
  c->text = nullptr;
}

const char* vllm_last_error(void) { return g_last_error.c_str(); }
const char* vllm_version(void) { return "vllm_cpp_b200 0.2 (native runtime)"; }
int32_t vllm_abi_version(void) { return VLLM_ABI_VERSION; }

}  // extern "C"
