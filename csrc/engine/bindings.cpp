// pybind11 surface of the host engine: the Python package drives the C++ scheduler, KV
// manager, engine core and input preparation through these classes, and implements
// ModelRunnerBase in Python (GPU runner) through the trampoline below.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "core/engine_core.h"
#include "core/hashing.h"
#include "core/kv_cache.h"
#include "core/scheduler.h"
#include "worker/input_batch.h"

namespace py = pybind11;
using namespace b200;

void bind_extras(py::module_& m);  // tokenizer, detokenizer, loaders, structured output, ...

namespace {

class PyModelRunner : public ModelRunnerBase {
 public:
  using ModelRunnerBase::ModelRunnerBase;
  void execute_model(const SchedulerOutput& so) override {
    PYBIND11_OVERRIDE_PURE(void, ModelRunnerBase, execute_model, so);
  }
  ModelRunnerOutput sample_tokens(const GrammarOutput* g) override {
    PYBIND11_OVERRIDE_PURE(ModelRunnerOutput, ModelRunnerBase, sample_tokens, g);
  }
  std::function<ModelRunnerOutput()> sample_tokens_async(const GrammarOutput* g) override {
    py::gil_scoped_acquire gil;
    py::function f = py::get_override(static_cast<const ModelRunnerBase*>(this), "sample_tokens_async");
    if (!f) return ModelRunnerBase::sample_tokens_async(g);
    py::object handle = f(g);
    // The handle may be dropped on the engine thread: take the GIL for the decref.
    std::shared_ptr<py::object> holder(new py::object(std::move(handle)), [](py::object* o) {
      py::gil_scoped_acquire g;
      delete o;
    });
    return [holder]() {
      py::gil_scoped_acquire gil2;
      ModelRunnerOutput out = (*holder)().cast<ModelRunnerOutput>();
      return out;
    };
  }
  std::optional<DraftTokenIds> take_draft_token_ids() override {
    PYBIND11_OVERRIDE(std::optional<DraftTokenIds>, ModelRunnerBase, take_draft_token_ids);
  }
  bool supports_async() const override { PYBIND11_OVERRIDE(bool, ModelRunnerBase, supports_async); }
};

// Owns scheduler + executor + core for Python.
struct EngineCoreHolder {
  std::unique_ptr<Executor> executor;
  std::unique_ptr<EngineCore> core;
  std::unique_ptr<InprocClient> client;
  py::object runner_ref;  // keeps the Python runner alive
  py::object so_ref;      // keeps the structured-output manager alive
  py::object kv_ref;      // keeps the KV connector alive
};

}  // namespace

PYBIND11_MODULE(_engine, m) {
  m.doc() = "vllm_cpp_b200 host engine (C++)";

  py::enum_<OutputKind>(m, "OutputKind")
      .value("CUMULATIVE", OutputKind::kCumulative)
      .value("DELTA", OutputKind::kDelta)
      .value("FINAL_ONLY", OutputKind::kFinalOnly);
  py::enum_<RequestStatus>(m, "RequestStatus")
      .value("WAITING", RequestStatus::kWaiting)
      .value("WAITING_FOR_FSM", RequestStatus::kWaitingForFsm)
      .value("WAITING_FOR_REMOTE_KVS", RequestStatus::kWaitingForRemoteKvs)
      .value("RUNNING", RequestStatus::kRunning)
      .value("PREEMPTED", RequestStatus::kPreempted)
      .value("FINISHED_STOPPED", RequestStatus::kFinishedStopped)
      .value("FINISHED_LENGTH_CAPPED", RequestStatus::kFinishedLengthCapped)
      .value("FINISHED_ABORTED", RequestStatus::kFinishedAborted)
      .value("FINISHED_IGNORED", RequestStatus::kFinishedIgnored);
  py::enum_<FinishReason>(m, "FinishReason")
      .value("STOP", FinishReason::kStop)
      .value("LENGTH", FinishReason::kLength)
      .value("ABORT", FinishReason::kAbort);
  m.def("finish_reason_str", [](FinishReason r) { return std::string(finish_reason_str(r)); });

  py::class_<StructuredOutputsParams>(m, "StructuredOutputsParams")
      .def(py::init<>())
      .def_readwrite("json", &StructuredOutputsParams::json)
      .def_readwrite("regex", &StructuredOutputsParams::regex)
      .def_readwrite("choice", &StructuredOutputsParams::choice)
      .def_readwrite("grammar", &StructuredOutputsParams::grammar)
      .def_readwrite("json_object", &StructuredOutputsParams::json_object)
      .def_readwrite("structural_tag", &StructuredOutputsParams::structural_tag)
      .def("any", &StructuredOutputsParams::any)
      .def("count", &StructuredOutputsParams::count);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def(py::init([](py::kwargs kw) {
        SamplingParams p;
        py::object o = py::cast(&p, py::return_value_policy::reference);
        for (auto item : kw) o.attr(item.first) = item.second;
        p.verify();
        return p;
      }))
      .def_readwrite("n", &SamplingParams::n)
      .def_readwrite("presence_penalty", &SamplingParams::presence_penalty)
      .def_readwrite("frequency_penalty", &SamplingParams::frequency_penalty)
      .def_readwrite("repetition_penalty", &SamplingParams::repetition_penalty)
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("min_p", &SamplingParams::min_p)
      .def_readwrite("seed", &SamplingParams::seed)
      .def_readwrite("stop", &SamplingParams::stop)
      .def_readwrite("stop_token_ids", &SamplingParams::stop_token_ids)
      .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("min_tokens", &SamplingParams::min_tokens)
      .def_readwrite("logprobs", &SamplingParams::logprobs)
      .def_readwrite("prompt_logprobs", &SamplingParams::prompt_logprobs)
      .def_readwrite("detokenize", &SamplingParams::detokenize)
      .def_readwrite("skip_special_tokens", &SamplingParams::skip_special_tokens)
      .def_readwrite("spaces_between_special_tokens", &SamplingParams::spaces_between_special_tokens)
      .def_readwrite("include_stop_str_in_output", &SamplingParams::include_stop_str_in_output)
      .def_readwrite("output_kind", &SamplingParams::output_kind)
      .def_readwrite("logit_bias", &SamplingParams::logit_bias)
      .def_readwrite("allowed_token_ids", &SamplingParams::allowed_token_ids)
      .def_readwrite("bad_words_token_ids", &SamplingParams::bad_words_token_ids)
      .def_readwrite("structured_outputs", &SamplingParams::structured_outputs)
      .def("verify", &SamplingParams::verify)
      .def("post_init", &SamplingParams::post_init)
      .def("has_penalties", &SamplingParams::has_penalties)
      .def("is_greedy", [](const SamplingParams& p) { return p.type() == SamplingType::kGreedy; })
      .def("clone", [](const SamplingParams& p) { return p; });

  py::class_<EngineCoreRequest>(m, "EngineCoreRequest")
      .def(py::init<>())
      .def(py::init([](std::string id, std::vector<int32_t> toks, SamplingParams sp,
                       std::optional<int32_t> eos, double arrival, int priority) {
             EngineCoreRequest r;
             r.request_id = std::move(id);
             r.prompt_token_ids = std::move(toks);
             r.sampling_params = std::move(sp);
             r.eos_token_id = eos;
             r.arrival_time = arrival;
             r.priority = priority;
             return r;
           }),
           py::arg("request_id"), py::arg("prompt_token_ids"), py::arg("sampling_params"),
           py::arg("eos_token_id") = std::nullopt, py::arg("arrival_time") = 0.0,
           py::arg("priority") = 0)
      .def_readwrite("request_id", &EngineCoreRequest::request_id)
      .def_readwrite("prompt_token_ids", &EngineCoreRequest::prompt_token_ids)
      .def_readwrite("sampling_params", &EngineCoreRequest::sampling_params)
      .def_readwrite("eos_token_id", &EngineCoreRequest::eos_token_id)
      .def_readwrite("arrival_time", &EngineCoreRequest::arrival_time)
      .def_readwrite("priority", &EngineCoreRequest::priority)
      .def_readwrite("cache_salt", &EngineCoreRequest::cache_salt);

  py::class_<StopReason>(m, "StopReason")
      .def_readonly("is_token", &StopReason::is_token)
      .def_readonly("token", &StopReason::token)
      .def_readonly("text", &StopReason::text);

  py::class_<Request, RequestPtr>(m, "Request")
      .def(py::init<const EngineCoreRequest&>())
      .def_readonly("request_id", &Request::request_id)
      .def_readonly("prompt_token_ids", &Request::prompt_token_ids)
      .def_readonly("output_token_ids", &Request::output_token_ids)
      .def_readonly("all_token_ids", &Request::all_token_ids)
      .def_readwrite("spec_token_ids", &Request::spec_token_ids)
      .def_readwrite("status", &Request::status)
      .def_readwrite("num_computed_tokens", &Request::num_computed_tokens)
      .def_readonly("num_cached_tokens", &Request::num_cached_tokens)
      .def_readonly("num_output_placeholders", &Request::num_output_placeholders)
      .def_readonly("num_preemptions", &Request::num_preemptions)
      .def_readonly("priority", &Request::priority)
      .def_readonly("stop_reason", &Request::stop_reason)
      .def_readonly("block_hashes", &Request::block_hashes)
      .def_property_readonly("num_tokens", &Request::num_tokens)
      .def_property_readonly("num_prompt_tokens", &Request::num_prompt_tokens)
      .def_property_readonly("num_output_tokens", &Request::num_output_tokens)
      .def("append_output_token", &Request::append_output_token)
      .def("finished", &Request::finished);

  py::class_<NewRequestData>(m, "NewRequestData")
      .def_readonly("req_id", &NewRequestData::req_id)
      .def_readonly("prompt_token_ids", &NewRequestData::prompt_token_ids)
      .def_readonly("sampling_params", &NewRequestData::sampling_params)
      .def_readonly("block_ids", &NewRequestData::block_ids)
      .def_readonly("num_computed_tokens", &NewRequestData::num_computed_tokens)
      .def_readonly("num_prompt_tokens", &NewRequestData::num_prompt_tokens);
  py::class_<CachedRequestData>(m, "CachedRequestData")
      .def_readonly("req_ids", &CachedRequestData::req_ids)
      .def_readonly("resumed_from_preemption", &CachedRequestData::resumed_from_preemption)
      .def_readonly("new_token_ids", &CachedRequestData::new_token_ids)
      .def_readonly("new_block_ids", &CachedRequestData::new_block_ids)
      .def_readonly("num_computed_tokens", &CachedRequestData::num_computed_tokens)
      .def_readonly("num_output_tokens", &CachedRequestData::num_output_tokens);
  py::class_<SchedulerOutput>(m, "SchedulerOutput")
      .def(py::init<>())
      .def_readonly("scheduled_new_reqs", &SchedulerOutput::scheduled_new_reqs)
      .def_readonly("scheduled_cached_reqs", &SchedulerOutput::scheduled_cached_reqs)
      .def_property_readonly("num_scheduled_tokens",
                             [](const SchedulerOutput& s) {
                               py::dict d;
                               for (auto& p : s.num_scheduled_tokens) d[py::str(p.first)] = p.second;
                               return d;
                             })
      .def_readonly("total_num_scheduled_tokens", &SchedulerOutput::total_num_scheduled_tokens)
      .def_readonly("scheduled_spec_decode_tokens", &SchedulerOutput::scheduled_spec_decode_tokens)
      .def_readonly("num_common_prefix_blocks", &SchedulerOutput::num_common_prefix_blocks)
      .def_readonly("finished_req_ids", &SchedulerOutput::finished_req_ids)
      .def_readonly("preempted_req_ids", &SchedulerOutput::preempted_req_ids)
      .def_readonly("structured_output_request_ids", &SchedulerOutput::structured_output_request_ids);
  py::class_<GrammarOutput>(m, "GrammarOutput")
      .def(py::init<>())
      .def_readwrite("structured_output_request_ids", &GrammarOutput::structured_output_request_ids)
      .def_readwrite("bitmask", &GrammarOutput::bitmask)
      .def_readwrite("words_per_row", &GrammarOutput::words_per_row);
  py::class_<LogprobsRow>(m, "LogprobsRow")
      .def(py::init<>())
      .def_readwrite("token_ids", &LogprobsRow::token_ids)
      .def_readwrite("logprobs", &LogprobsRow::logprobs)
      .def_readwrite("ranks", &LogprobsRow::ranks);
  py::class_<ModelRunnerOutput>(m, "ModelRunnerOutput")
      .def(py::init<>())
      .def_readwrite("req_ids", &ModelRunnerOutput::req_ids)
      .def_readwrite("sampled_token_ids", &ModelRunnerOutput::sampled_token_ids)
      .def_readwrite("logprobs", &ModelRunnerOutput::logprobs)
      .def_readwrite("num_nans_in_logits", &ModelRunnerOutput::num_nans_in_logits)
      .def_readwrite("finished_sending", &ModelRunnerOutput::finished_sending)
      .def_readwrite("finished_recving", &ModelRunnerOutput::finished_recving)
      .def_readwrite("num_recompute", &ModelRunnerOutput::num_recompute);
  py::class_<DraftTokenIds>(m, "DraftTokenIds")
      .def(py::init<>())
      .def_readwrite("req_ids", &DraftTokenIds::req_ids)
      .def_readwrite("draft_token_ids", &DraftTokenIds::draft_token_ids);
  py::class_<EngineCoreOutput>(m, "EngineCoreOutput")
      .def_readonly("request_id", &EngineCoreOutput::request_id)
      .def_readonly("new_token_ids", &EngineCoreOutput::new_token_ids)
      .def_readonly("new_logprobs", &EngineCoreOutput::new_logprobs)
      .def_readonly("finish_reason", &EngineCoreOutput::finish_reason)
      .def_readonly("stop_reason", &EngineCoreOutput::stop_reason)
      .def_readonly("num_cached_tokens", &EngineCoreOutput::num_cached_tokens)
      .def("finished", &EngineCoreOutput::finished);
  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("num_running_reqs", &SchedulerStats::num_running_reqs)
      .def_readonly("num_waiting_reqs", &SchedulerStats::num_waiting_reqs)
      .def_readonly("kv_cache_usage", &SchedulerStats::kv_cache_usage)
      .def_readonly("prefix_cache_queries", &SchedulerStats::prefix_cache_queries)
      .def_readonly("prefix_cache_hits", &SchedulerStats::prefix_cache_hits)
      .def_readonly("num_preempted", &SchedulerStats::num_preempted)
      .def_readonly("step_scheduled_tokens", &SchedulerStats::step_scheduled_tokens);
  py::class_<EngineCoreOutputs>(m, "EngineCoreOutputs")
      .def_readonly("outputs", &EngineCoreOutputs::outputs)
      .def_readonly("scheduler_stats", &EngineCoreOutputs::scheduler_stats)
      .def_readonly("finished_requests", &EngineCoreOutputs::finished_requests)
      .def_readonly("engine_dead", &EngineCoreOutputs::engine_dead)
      .def_readonly("error", &EngineCoreOutputs::error);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def(py::init([](py::kwargs kw) {
        SchedulerConfig c;
        py::object o = py::cast(&c, py::return_value_policy::reference);
        for (auto item : kw) o.attr(item.first) = item.second;
        return c;
      }))
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("enable_chunked_prefill", &SchedulerConfig::enable_chunked_prefill)
      .def_readwrite("long_prefill_token_threshold", &SchedulerConfig::long_prefill_token_threshold)
      .def_readwrite("policy", &SchedulerConfig::policy)
      .def_readwrite("async_scheduling", &SchedulerConfig::async_scheduling)
      .def_readwrite("num_lookahead_tokens", &SchedulerConfig::num_lookahead_tokens)
      .def_readwrite("enable_prefix_caching", &SchedulerConfig::enable_prefix_caching)
      .def_readwrite("watermark", &SchedulerConfig::watermark)
      .def_readwrite("log_stats", &SchedulerConfig::log_stats);

  py::enum_<KVSpecKind>(m, "KVSpecKind")
      .value("FULL_ATTENTION", KVSpecKind::kFullAttention)
      .value("MLA", KVSpecKind::kMLA)
      .value("SLIDING_WINDOW", KVSpecKind::kSlidingWindow)
      .value("CHUNKED_LOCAL", KVSpecKind::kChunkedLocal)
      .value("MAMBA", KVSpecKind::kMamba);
  py::class_<KVCacheSpec>(m, "KVCacheSpec")
      .def(py::init<>())
      .def(py::init([](py::kwargs kw) {
        KVCacheSpec c;
        py::object o = py::cast(&c, py::return_value_policy::reference);
        for (auto item : kw) o.attr(item.first) = item.second;
        return c;
      }))
      .def_readwrite("kind", &KVCacheSpec::kind)
      .def_readwrite("block_size", &KVCacheSpec::block_size)
      .def_readwrite("num_kv_heads", &KVCacheSpec::num_kv_heads)
      .def_readwrite("head_size", &KVCacheSpec::head_size)
      .def_readwrite("dtype_bytes", &KVCacheSpec::dtype_bytes)
      .def_readwrite("sliding_window", &KVCacheSpec::sliding_window)
      .def_readwrite("attention_chunk_size", &KVCacheSpec::attention_chunk_size)
      .def_readwrite("mamba_state_bytes", &KVCacheSpec::mamba_state_bytes)
      .def("page_size_bytes", &KVCacheSpec::page_size_bytes)
      .def("max_memory_usage_bytes", &KVCacheSpec::max_memory_usage_bytes);
  py::class_<KVCacheGroupSpec>(m, "KVCacheGroupSpec")
      .def(py::init<>())
      .def(py::init([](std::vector<std::string> names, KVCacheSpec spec) {
        return KVCacheGroupSpec{std::move(names), spec};
      }))
      .def_readwrite("layer_names", &KVCacheGroupSpec::layer_names)
      .def_readwrite("spec", &KVCacheGroupSpec::spec);
  py::class_<KVCacheConfig>(m, "KVCacheConfig")
      .def(py::init<>())
      .def(py::init([](int num_blocks, std::vector<KVCacheGroupSpec> groups) {
        return KVCacheConfig{num_blocks, std::move(groups)};
      }))
      .def_readwrite("num_blocks", &KVCacheConfig::num_blocks)
      .def_readwrite("groups", &KVCacheConfig::groups);

  // ---- KV cache internals (exposed for behavioural tests and tools)
  py::class_<KVCacheBlock>(m, "KVCacheBlock")
      .def_readonly("block_id", &KVCacheBlock::block_id)
      .def_readonly("ref_cnt", &KVCacheBlock::ref_cnt)
      .def_readonly("is_null", &KVCacheBlock::is_null)
      .def_property_readonly("block_hash", [](const KVCacheBlock& b) -> py::object {
        if (!b.block_hash) return py::none();
        return py::bytes(*b.block_hash);
      });
  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int, bool>(), py::arg("num_gpu_blocks"), py::arg("enable_caching") = true)
      .def("null_block", &BlockPool::null_block, py::return_value_policy::reference_internal)
      .def("get_new_blocks", &BlockPool::get_new_blocks, py::return_value_policy::reference_internal)
      .def("get_cached_block",
           [](BlockPool& p, py::bytes h, std::vector<int> groups) {
             return p.get_cached_block(std::string(h), groups);
           },
           py::return_value_policy::reference_internal)
      .def("cache_full_blocks", &BlockPool::cache_full_blocks)
      .def("touch", &BlockPool::touch)
      .def("free_blocks", &BlockPool::free_blocks)
      .def("reset_prefix_cache", &BlockPool::reset_prefix_cache)
      .def("get_num_free_blocks", &BlockPool::get_num_free_blocks)
      .def("get_usage", &BlockPool::get_usage)
      .def("block", &BlockPool::block, py::return_value_policy::reference_internal)
      .def("num_gpu_blocks", &BlockPool::num_gpu_blocks);
  py::class_<KVCacheBlocks>(m, "KVCacheBlocks")
      .def("block_ids", &KVCacheBlocks::block_ids)
      .def("empty", &KVCacheBlocks::empty);
  py::class_<KVCacheManager>(m, "KVCacheManager")
      .def(py::init<const KVCacheConfig&, int, bool, bool>(), py::arg("config"),
           py::arg("max_model_len"), py::arg("enable_caching") = true, py::arg("log_stats") = true)
      .def("get_computed_blocks", [](KVCacheManager& k, RequestPtr r) { return k.get_computed_blocks(*r); })
      .def("allocate_slots",
           [](KVCacheManager& k, RequestPtr r, int n, int ncomp, const KVCacheBlocks* cb, int look,
              bool delay) { return k.allocate_slots(*r, n, ncomp, cb, look, delay); },
           py::arg("request"), py::arg("num_new_tokens"), py::arg("num_new_computed_tokens") = 0,
           py::arg("new_computed_blocks") = nullptr, py::arg("num_lookahead_tokens") = 0,
           py::arg("delay_cache_blocks") = false)
      .def("free", [](KVCacheManager& k, RequestPtr r) { k.free(*r); })
      .def("reset_prefix_cache", &KVCacheManager::reset_prefix_cache)
      .def("get_block_ids", &KVCacheManager::get_block_ids)
      .def("get_num_common_prefix_blocks",
           [](KVCacheManager& k, RequestPtr r, int n) { return k.get_num_common_prefix_blocks(*r, n); })
      .def("usage", &KVCacheManager::usage)
      .def("num_free_blocks", [](KVCacheManager& k) { return k.pool().get_num_free_blocks(); })
      .def("pool", [](KVCacheManager& k) { return &k.pool(); }, py::return_value_policy::reference_internal)
      .def("take_prefix_cache_stats", [](KVCacheManager& k) {
        auto s = k.take_prefix_cache_stats();
        return py::make_tuple(s.requests, s.queries, s.hits);
      });

  m.def("sha256_hex", [](py::bytes b) { std::string s = b; return sha256_hex(s.data(), s.size()); });
  m.def("none_hash", []() { return py::bytes(none_hash()); });
  m.def("reset_none_hash_for_test", &reset_none_hash_for_test);
  m.def("hash_block_tokens", [](py::bytes parent, std::vector<int32_t> toks,
                                std::optional<std::vector<std::string>> extra) {
    std::string p = parent;
    return py::bytes(hash_block_tokens(p, toks.data(), toks.size(), extra ? &*extra : nullptr));
  }, py::arg("parent"), py::arg("tokens"), py::arg("extra_keys") = std::nullopt);

  // ---- scheduler
  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init([](const SchedulerConfig& c, const KVCacheConfig& k, py::object connector) {
        // keep_alive below ties the connector's lifetime to the scheduler's
        KVConnectorHook* hook = connector.is_none() ? nullptr : connector.cast<KVConnectorHook*>();
        return c.async_scheduling ? static_cast<Scheduler*>(new AsyncScheduler(c, k, nullptr, hook))
                                  : new Scheduler(c, k, nullptr, hook);
      }), py::arg("scheduler_config"), py::arg("kv_cache_config"), py::arg("kv_connector") = py::none(),
          py::keep_alive<1, 4>())
      .def("add_request", [](Scheduler& s, const EngineCoreRequest& r) {
        EngineCoreRequest rr = r;
        rr.sampling_params.post_init();
        auto req = std::make_shared<Request>(rr);
        s.add_request(req);
        return req;
      })
      .def("schedule", &Scheduler::schedule)
      .def("update_from_output", &Scheduler::update_from_output)
      .def("finish_requests", &Scheduler::finish_requests)
      .def("update_draft_token_ids", &Scheduler::update_draft_token_ids)
      .def("get_request", &Scheduler::get_request)
      .def("num_running", &Scheduler::num_running)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_delayed_free", &Scheduler::num_delayed_free)
      .def("has_unfinished_requests", &Scheduler::has_unfinished_requests)
      .def("has_requests", &Scheduler::has_requests)
      .def("reset_prefix_cache", &Scheduler::reset_prefix_cache)
      .def("make_stats", &Scheduler::make_stats)
      .def("kv_usage", [](Scheduler& s) { return s.kv_cache_manager().usage(); })
      .def("num_free_blocks", [](Scheduler& s) { return s.kv_cache_manager().pool().get_num_free_blocks(); })
      .def("running_ids", [](Scheduler& s) {
        std::vector<std::string> ids;
        for (auto& r : s.running()) ids.push_back(r->request_id);
        return ids;
      });

  // ---- runner + engine core
  py::class_<ModelRunnerBase, PyModelRunner>(m, "ModelRunnerBase")
      .def(py::init<>())
      .def("supports_async", &ModelRunnerBase::supports_async);

  py::class_<EngineCoreHolder>(m, "EngineCore")
      .def(py::init([](const SchedulerConfig& c, const KVCacheConfig& k, py::object runner,
                       int max_concurrent_batches, py::object structured, py::object connector) {
             auto h = std::make_unique<EngineCoreHolder>();
             h->runner_ref = runner;
             h->so_ref = structured;
             h->kv_ref = connector;
             KVConnectorHook* kv_hook = connector.is_none() ? nullptr : connector.cast<KVConnectorHook*>();
             StructuredOutputHook* so_hook =
                 structured.is_none() ? nullptr : structured.cast<StructuredOutputHook*>();
             ModelRunnerBase* rb = runner.cast<ModelRunnerBase*>();
             h->executor = std::make_unique<Executor>(rb, max_concurrent_batches);
             std::unique_ptr<Scheduler> s;
             if (c.async_scheduling) s = std::make_unique<AsyncScheduler>(c, k, so_hook, kv_hook);
             else s = std::make_unique<Scheduler>(c, k, so_hook, kv_hook);
             h->core = std::make_unique<EngineCore>(std::move(s), h->executor.get());
             return h;
           }),
           py::arg("scheduler_config"), py::arg("kv_cache_config"), py::arg("runner"),
           py::arg("max_concurrent_batches") = 1, py::arg("structured_output_manager") = py::none(),
           py::arg("kv_connector") = py::none())
      .def("add_request", [](EngineCoreHolder& h, const EngineCoreRequest& r) { h.core->add_request(r); })
      .def("abort_requests", [](EngineCoreHolder& h, std::vector<std::string> ids) { h.core->abort_requests(ids); })
      .def("step", [](EngineCoreHolder& h) { return h.core->step(); })
      .def("step_with_batch_queue", [](EngineCoreHolder& h) { return h.core->step_with_batch_queue(); })
      .def("has_work", [](EngineCoreHolder& h) { return h.core->has_work(); })
      .def("has_unfinished", [](EngineCoreHolder& h) { return h.core->has_unfinished(); })
      .def("scheduler", [](EngineCoreHolder& h) { return &h.core->scheduler(); },
           py::return_value_policy::reference_internal)
      .def("reset_prefix_cache", [](EngineCoreHolder& h) { return h.core->reset_prefix_cache(); })
      .def_property_readonly("num_steps", [](EngineCoreHolder& h) { return h.core->num_steps; })
      .def_property_readonly("num_executed_steps", [](EngineCoreHolder& h) { return h.core->num_executed_steps; })
      .def_property_readonly("last_schedule_ms", [](EngineCoreHolder& h) { return h.core->last_schedule_ms; })
      .def_property_readonly("last_execute_ms", [](EngineCoreHolder& h) { return h.core->last_execute_ms; })
      .def_property_readonly("last_update_ms", [](EngineCoreHolder& h) { return h.core->last_update_ms; })
      // background busy loop (AsyncLLM path)
      .def("start_busy_loop", [](EngineCoreHolder& h, bool use_batch_queue) {
        if (!h.client) h.client = std::make_unique<InprocClient>(h.core.get(), use_batch_queue);
      }, py::arg("use_batch_queue") = false)
      .def("add_request_async", [](EngineCoreHolder& h, const EngineCoreRequest& r) {
        if (!h.client) throw std::runtime_error("busy loop not started");
        h.client->add_request_async(r);
      })
      .def("abort_requests_async", [](EngineCoreHolder& h, std::vector<std::string> ids) {
        if (h.client) h.client->abort_requests_async(ids);
      })
      .def("get_output", [](EngineCoreHolder& h, double timeout) -> std::optional<EngineCoreOutputs> {
        if (!h.client) throw std::runtime_error("busy loop not started");
        py::gil_scoped_release rel;
        if (timeout < 0) return h.client->get_output();
        return h.client->get_output_for(timeout);
      }, py::arg("timeout") = -1.0)
      .def("engine_dead", [](EngineCoreHolder& h) { return h.client && h.client->engine_dead(); })
      .def("inject_executor_failure", [](EngineCoreHolder& h) {
        if (!h.client) throw std::runtime_error("busy loop not started");
        CoreInput in;
        in.type = CoreRequestType::kExecutorFailed;
        h.client->proc().input().put(in);
      })
      .def("shutdown", [](EngineCoreHolder& h, bool abort) {
        if (h.client) {
          py::gil_scoped_release rel;
          h.client->shutdown(abort);
        }
      }, py::arg("abort") = true);
  py::register_exception<EngineDeadError>(m, "EngineDeadError");

  // ---- worker-side input preparation
  py::class_<StepLayout>(m, "StepLayout")
      .def_static("make", &StepLayout::make, py::arg("max_tokens"), py::arg("max_reqs"),
                  py::arg("max_blocks"), py::arg("num_groups"), py::arg("max_spec") = 0)
      .def_readonly("max_logits", &StepLayout::max_logits)
      .def_readonly("max_tokens", &StepLayout::max_tokens)
      .def_readonly("max_reqs", &StepLayout::max_reqs)
      .def_readonly("max_blocks", &StepLayout::max_blocks)
      .def_readonly("num_groups", &StepLayout::num_groups)
      .def_readonly("max_tiles", &StepLayout::max_tiles)
      .def_readonly("total_bytes", &StepLayout::total_bytes)
      .def("offsets", [](const StepLayout& l) {
        py::dict d;
        d["input_ids"] = l.input_ids; d["positions"] = l.positions; d["slot_mapping"] = l.slot_mapping;
        d["query_start"] = l.query_start; d["seq_lens"] = l.seq_lens; d["block_table"] = l.block_table;
        d["logits_indices"] = l.logits_indices; d["tile_req"] = l.tile_req; d["tile_q0"] = l.tile_q0;
        d["prefill_q_start"] = l.prefill_q_start; d["state_slots"] = l.state_slots;
        d["temperature"] = l.temperature; d["top_p"] = l.top_p; d["min_p"] = l.min_p;
        d["top_k"] = l.top_k; d["seeds"] = l.seeds; d["steps"] = l.steps; d["rep_pen"] = l.rep_pen;
        d["freq_pen"] = l.freq_pen; d["pres_pen"] = l.pres_pen; d["splice_dst"] = l.splice_dst;
        d["splice_src"] = l.splice_src; d["sample_rows"] = l.sample_rows;
        return d;
      });
  py::class_<StepInfo>(m, "StepInfo")
      .def_readonly("num_reqs", &StepInfo::num_reqs)
      .def_readonly("num_tokens", &StepInfo::num_tokens)
      .def_readonly("num_decodes", &StepInfo::num_decodes)
      .def_readonly("num_decode_tokens", &StepInfo::num_decode_tokens)
      .def_readonly("num_prefills", &StepInfo::num_prefills)
      .def_readonly("num_prefill_tokens", &StepInfo::num_prefill_tokens)
      .def_readonly("num_tiles", &StepInfo::num_tiles)
      .def_readonly("max_query_len", &StepInfo::max_query_len)
      .def_readonly("max_seq_len", &StepInfo::max_seq_len)
      .def_readonly("num_logits", &StepInfo::num_logits)
      .def_readonly("num_splice", &StepInfo::num_splice)
      .def_readonly("all_greedy", &StepInfo::all_greedy)
      .def_readonly("any_penalties", &StepInfo::any_penalties)
      .def_readonly("any_top_k_top_p", &StepInfo::any_top_k_top_p)
      .def_readonly("any_min_p", &StepInfo::any_min_p)
      .def_readonly("any_logprobs", &StepInfo::any_logprobs)
      .def_readonly("any_logit_edits", &StepInfo::any_logit_edits)
      .def_readonly("req_ids", &StepInfo::req_ids)
      .def_readonly("num_scheduled", &StepInfo::num_scheduled)
      .def_readonly("produces_token", &StepInfo::produces_token)
      .def_readonly("num_draft", &StepInfo::num_draft)
      .def_readonly("logits_row0", &StepInfo::logits_row0)
      .def_readonly("max_logprobs", &StepInfo::max_logprobs);
  py::class_<InputBatch>(m, "InputBatch")
      .def(py::init<int, int, int, std::vector<int>>())
      .def("update_states", &InputBatch::update_states)
      .def("prepare", [](InputBatch& b, const SchedulerOutput& so, const StepLayout& l,
                         uintptr_t buf, bool async_mode) {
        return b.prepare(so, l, reinterpret_cast<uint8_t*>(buf), async_mode);
      }, py::arg("scheduler_output"), py::arg("layout"), py::arg("buffer_ptr"),
           py::arg("async_mode") = false)
      .def("propose_ngram", &InputBatch::propose_ngram)
      .def("num_tokens", [](const InputBatch& b, const std::string& id) {
        const CachedRequestState* s = b.get(id);
        return s ? (int)s->token_ids.size() : -1;
      })
      .def("plain_greedy", &InputBatch::plain_greedy)
      .def("append_sampled", &InputBatch::append_sampled)
      .def("num_requests", &InputBatch::num_requests)
      .def("token_ids", [](InputBatch& b, const std::string& id) {
        auto* s = b.get(id);
        return s ? s->token_ids : std::vector<int32_t>{};
      })
      .def("penalty_entries", [](InputBatch& b, const StepInfo& info) {
        std::vector<int32_t> r, t, c;
        b.build_penalty_entries(info, r, t, c);
        return py::make_tuple(r, t, c);
      })
      .def("logit_edits", [](InputBatch& b, const StepInfo& info, std::map<std::string, int32_t> eos) {
        std::vector<int32_t> br, btk, nr, nt;
        std::vector<float> bv;
        b.build_logit_edits(info, br, btk, bv, nr, nt, eos);
        return py::make_tuple(br, btk, bv, nr, nt);
      });

  bind_extras(m);
}
