#include "runtime/native_llm.h"

#include <chrono>
#include <filesystem>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "util/json.h"

namespace fs = std::filesystem;

namespace b200::rt {

namespace {
std::string slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}
double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

std::unique_ptr<NativeLLM> NativeLLM::load(const EngineOptions& opt) {
  if (!fs::is_directory(opt.model_path))
    throw std::runtime_error("model path is not a directory: " + opt.model_path +
                             " (the native runtime loads safetensors model directories)");
  std::unique_ptr<NativeLLM> e(new NativeLLM());
  const Json hf = Json::parse(slurp((fs::path(opt.model_path) / "config.json").string()));
  e->cfg_ = DenseConfig::from_hf(hf);
  Device dev = Device::parse(opt.device);
  if (dev.cuda && !cuda_available()) throw std::runtime_error("device " + opt.device + " requested but no GPU is visible");
  const std::string tok_dir = opt.tokenizer_path.empty() ? opt.model_path : opt.tokenizer_path;
  if (fs::exists(fs::path(tok_dir) / "tokenizer.json") || fs::is_regular_file(tok_dir))
    e->tokenizer_ = tok::Tokenizer::from_dir(tok_dir);
  e->max_model_len_ = opt.max_model_len > 0 ? opt.max_model_len : e->cfg_.max_position;
  auto model = std::make_unique<DenseModel>(e->cfg_, dev, e->max_model_len_);
  model->load_weights(opt.model_path);
  const int budget = opt.max_num_batched_tokens > 0 ? opt.max_num_batched_tokens : 2048;
  const int blocks_per_seq = (e->max_model_len_ + opt.block_size - 1) / opt.block_size;
  int64_t num_blocks = opt.num_blocks;
  if (num_blocks <= 0) {
    const int64_t cap = (int64_t)opt.max_num_seqs * blocks_per_seq + 16;
    if (dev.cuda) {
      size_t free_b = 0, total_b = 0;
      free_and_total_memory(dev, &free_b, &total_b);
      const DenseConfig& c = e->cfg_;
      const double act = (double)budget * (4.0 * c.hidden + 3.0 * c.inter) * 2 * 2;
      const double usable = (double)free_b - (1.0 - opt.gpu_memory_utilization) * (double)total_b - act - (double)(2ull << 30);
      num_blocks = (int64_t)(usable / (double)model->kv_bytes_per_block(opt.block_size));
      num_blocks = std::max<int64_t>(16, std::min(num_blocks, cap));
    } else {
      num_blocks = std::max<int64_t>(16, std::min<int64_t>(cap, 4096));
    }
  }
  e->runner_ = std::make_unique<NativeRunner>(std::move(model), opt.block_size, (int)num_blocks, opt.max_num_seqs,
                                              budget, e->max_model_len_);
  SchedulerConfig sc;
  sc.max_num_batched_tokens = budget;
  sc.max_num_seqs = opt.max_num_seqs;
  sc.max_model_len = e->max_model_len_;
  sc.enable_prefix_caching = opt.enable_prefix_caching;
  sc.async_scheduling = false;
  if (e->tokenizer_) {
    const tok::Tokenizer& tk = *e->tokenizer_;
    std::vector<std::string> tb((size_t)tk.vocab_size());
    for (int i = 0; i < tk.vocab_size(); ++i) tb[i] = tk.is_special(i) ? std::string() : tk.token_bytes(i);
    std::vector<int> eos;
    if (e->cfg_.eos_token_id >= 0) eos.push_back(e->cfg_.eos_token_id);
    if (tk.eos_id() >= 0 && tk.eos_id() != e->cfg_.eos_token_id) eos.push_back(tk.eos_id());
    e->structured_ = std::make_unique<so::StructuredOutputManager>(std::move(tb), e->cfg_.vocab_size, eos);
  }
  e->executor_ = std::make_unique<Executor>(e->runner_.get(), 1);
  auto sched = std::make_unique<Scheduler>(sc, e->runner_->kv_cache_config(), e->structured_.get(), nullptr);
  e->core_ = std::make_unique<EngineCore>(std::move(sched), e->executor_.get());
  return e;
}

NativeLLM::~NativeLLM() = default;

std::string NativeLLM::add_request(const std::string& prompt, SamplingParams params, const std::string& request_id) {
  if (!tokenizer_) throw std::invalid_argument("text prompts need a tokenizer beside the model");
  std::vector<int> ids = tokenizer_->encode(prompt);
  return add_request_ids(std::vector<int32_t>(ids.begin(), ids.end()), std::move(params), request_id);
}

std::string NativeLLM::add_request_ids(std::vector<int32_t> ids, SamplingParams params, const std::string& request_id) {
  if (ids.empty()) throw std::invalid_argument("the prompt is empty");
  if ((int)ids.size() >= max_model_len_)
    throw std::invalid_argument("prompt (" + std::to_string(ids.size()) + " tokens) is longer than max_model_len (" +
                                std::to_string(max_model_len_) + ")");
  params.verify();
  if (params.structured_outputs && params.structured_outputs->any()) {
    if (!structured_) throw std::invalid_argument("structured outputs need a tokenizer");
    structured_->compile(*params.structured_outputs);     // throws on a bad constraint
  }
  const std::string rid = request_id.empty() ? "req-" + std::to_string(counter_++) : request_id;
  EngineCoreRequest req;
  req.request_id = rid;
  req.prompt_token_ids = ids;
  req.sampling_params = params;
  if (cfg_.eos_token_id >= 0) req.eos_token_id = cfg_.eos_token_id;
  req.arrival_time = now_s();
  runner_->set_eos(rid, cfg_.eos_token_id);
  Live lv;
  lv.prompt_ids = ids;
  if (tokenizer_ && params.detokenize)
    lv.detok = std::make_unique<tok::IncrementalDetokenizer>(tokenizer_.get(), std::vector<int>(ids.begin(), ids.end()),
                                                             params.skip_special_tokens, params.stop,
                                                             params.include_stop_str_in_output, params.min_tokens);
  core_->add_request(req);
  live_[rid] = std::move(lv);
  return rid;
}

void NativeLLM::abort(const std::string& request_id) {
  core_->abort_requests({request_id});
  live_.erase(request_id);
  runner_->forget(request_id);
}

bool NativeLLM::has_unfinished() const { return core_->has_work(); }

std::vector<RequestDelta> NativeLLM::step() {
  auto [outs, executed] = core_->step();
  (void)executed;
  std::vector<RequestDelta> res;
  for (auto& o : outs.outputs) {
    auto it = live_.find(o.request_id);
    if (it == live_.end()) continue;
    Live& lv = it->second;
    RequestDelta d;
    d.request_id = o.request_id;
    d.new_token_ids = o.new_token_ids;
    d.prompt_tokens = (int)lv.prompt_ids.size();
    lv.completion_tokens += (int)o.new_token_ids.size();
    bool finished = o.finish_reason.has_value();
    std::string reason = finished ? finish_reason_str(*o.finish_reason) : "";
    if (lv.detok && !o.new_token_ids.empty()) {
      // the last token of a request that stopped on EOS / a stop token is not text
      const bool stop_terminated = finished && reason == "stop" && (!o.stop_reason || o.stop_reason->is_token);
      std::string stop_str;
      const bool hit = lv.detok->update(std::vector<int>(o.new_token_ids.begin(), o.new_token_ids.end()),
                                        stop_terminated, &stop_str);
      if (hit && !finished) {
        core_->abort_requests({o.request_id});      // a stop string ends the request here
        finished = true;
        reason = "stop";
      }
      d.delta_text = lv.detok->get_next_output_text(finished, /*delta=*/true);
    }
    d.finished = finished;
    d.finish_reason = reason;
    d.completion_tokens = lv.completion_tokens;
    res.push_back(std::move(d));
    if (finished) {
      runner_->forget(o.request_id);
      live_.erase(it);
    }
  }
  return res;
}

}  // namespace b200::rt
