// Host-side sanitizer driver: the scheduler, KV-cache manager (prefix caching, preemption),
// input batch, tokenizer-free engine core loop, offload policies and the LMCache codec run
// against a fake model runner, in one process without Python, so that the whole host engine
// can be built with -fsanitize=address,undefined (or thread) and exercised on this machine.
// The CUDA side cannot run under compute-sanitizer here, the host side can under these.
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "core/engine_core.h"
#include "core/scheduler.h"
#include "offload/lmcache.h"
#include "offload/offload.h"
#include "parallel/eplb.h"
#include "worker/input_batch.h"

using namespace b200;

// Returns pseudo-random tokens for every request that finishes its known tokens this step and
// keeps a real InputBatch in step with the scheduler (block tables, token lists).
class FakeRunner : public ModelRunnerBase {
 public:
  FakeRunner(int max_reqs, int max_len, int max_tokens, int block_size)
      : batch_(max_reqs, max_len, max_tokens, {block_size}),
        layout_(StepLayout::make(max_tokens, max_reqs, (max_len + block_size - 1) / block_size + 1, 1, 2)),
        buf_(layout_.total_bytes) {}
  void execute_model(const SchedulerOutput& so) override {
    batch_.update_states(so);
    has_ = so.total_num_scheduled_tokens > 0;
    if (has_) info_ = batch_.prepare(so, layout_, buf_.data(), false);
  }
  ModelRunnerOutput sample_tokens(const GrammarOutput*) override {
    ModelRunnerOutput out;
    if (!has_) return out;
    out.req_ids = info_.req_ids;
    for (size_t r = 0; r < info_.req_ids.size(); ++r) {
      std::vector<int32_t> toks;
      if (info_.produces_token[r]) {
        const int n = 1 + (info_.num_draft[r] ? (int)(rng_() % (info_.num_draft[r] + 1)) : 0);
        for (int i = 0; i < n; ++i) toks.push_back((int32_t)(rng_() % 1000));
        batch_.append_sampled(info_.req_ids[r], toks);
        // a runner with recurrent state: every rejection has the kept tokens of the step run again
        if (recompute_ && info_.num_draft[r] && n <= info_.num_draft[r]) out.num_recompute[info_.req_ids[r]] = n;
        drafts_.req_ids.push_back(info_.req_ids[r]);
        drafts_.draft_token_ids.push_back(batch_.propose_ngram(info_.req_ids[r], 1, 3, 2));
      }
      out.sampled_token_ids.push_back(toks);
    }
    return out;
  }
  std::optional<DraftTokenIds> take_draft_token_ids() override {
    if (drafts_.req_ids.empty()) return std::nullopt;
    DraftTokenIds d = std::move(drafts_);
    drafts_ = {};
    return d;
  }

 private:
  InputBatch batch_;
  StepLayout layout_;
  std::vector<uint8_t> buf_;
  StepInfo info_;
  bool has_ = false;
  DraftTokenIds drafts_;
  std::mt19937 rng_{7};

 public:
  bool recompute_ = false;
};

static int run_engine(bool priority, int num_blocks) {
  const int block = 16, max_len = 256, max_reqs = 6, budget = 96;
  SchedulerConfig sc;
  sc.max_num_batched_tokens = budget;
  sc.max_num_seqs = max_reqs;
  sc.max_model_len = max_len;
  sc.policy = priority ? "priority" : "fcfs";
  sc.num_lookahead_tokens = 2;
  KVCacheConfig kv;
  kv.num_blocks = num_blocks;
  KVCacheSpec spec;
  spec.block_size = block;
  kv.groups.push_back(KVCacheGroupSpec{{"layer0"}, spec});
  FakeRunner runner(max_reqs, max_len, budget, block);
  runner.recompute_ = priority;        // one of the two runs rolls state back on rejected drafts
  Executor exec(&runner, 1);
  EngineCore core(std::make_unique<Scheduler>(sc, kv), &exec);
  std::mt19937 rng(3);
  int finished = 0, submitted = 0;
  std::vector<int32_t> shared(40);
  for (auto& t : shared) t = (int32_t)(rng() % 1000);
  for (int step = 0; step < 400; ++step) {
    if (submitted < 40 && step % 3 == 0) {
      EngineCoreRequest r;
      r.request_id = "r" + std::to_string(submitted);
      r.prompt_token_ids = shared;                      // common prefix: prefix-cache hits
      const int extra = (int)(rng() % 60);
      for (int i = 0; i < extra; ++i) r.prompt_token_ids.push_back((int32_t)(rng() % 1000));
      r.sampling_params.max_tokens = 1 + (int)(rng() % 30);
      r.sampling_params.temperature = 0.0;
      r.sampling_params.ignore_eos = true;
      r.priority = (int)(rng() % 3);
      core.add_request(r);
      ++submitted;
    }
    if (step % 37 == 5 && submitted > 2) core.abort_requests({"r" + std::to_string(submitted - 2)});
    auto res = core.step();
    for (auto& o : res.first.outputs)
      if (o.finished()) ++finished;
    if (submitted == 40 && !core.has_work()) break;
  }
  if (core.has_unfinished()) {
    std::fprintf(stderr, "engine did not drain\n");
    return 1;
  }
  std::printf("engine(%s, %d blocks): %d finished of %d\n", priority ? "priority" : "fcfs", num_blocks, finished,
              submitted);
  return finished > 0 ? 0 : 1;
}

static int run_offload_and_lmcache() {
  using namespace b200::offload;
  for (const char* pol : {"lru", "arc"}) {
    auto p = CachePolicy::make(pol, 8);
    for (int i = 0; i < 64; ++i) {
      Key k(32, (char)('a' + i % 13));
      p->insert(k);
      p->touch(k);
      if (p->size() > 8) {
        auto v = p->victim([](const Key&) { return true; });
        if (v) p->erase(*v);
      }
    }
  }
  namespace lm = b200::lmcache;
  lm::TokenHasher h(4);
  std::vector<uint32_t> toks(37);
  for (size_t i = 0; i < toks.size(); ++i) toks[i] = (uint32_t)(i * 2654435761u);
  auto hashes = h.chunk_hashes(toks);
  if (hashes.size() != 9) return 1;
  std::string big(5000, 'x');
  if (lm::blake3(big.data(), big.size()).size() != 32) return 1;
  lm::ClientMeta m;
  m.key = lm::CacheKey{"m", 1, 0, lm::TokenHasher::fold(hashes[0]), lm::Dtype::kBFloat16, {}}.to_string();
  m.shape = {2, 3, 4, 5};
  auto back = lm::ClientMeta::deserialize(m.serialize());
  if (back.key != m.key || back.shape != m.shape) return 1;
  std::vector<std::string> k(2, std::string(3 * 4 * 2, 'k')), v(2, std::string(3 * 4 * 2, 'v'));
  auto packed = lm::pack_kv2ltd(2, 3, 4, 2, k, v);
  std::vector<std::string> k2, v2;
  lm::unpack_kv2ltd(2, 3, 4, 2, packed, &k2, &v2);
  return (k2 == k && v2 == v) ? 0 : 1;
}

static int run_eplb() {
  std::mt19937 rng(11);
  const int cfgs[][6] = {{3, 64, 72, 8, 1, 8}, {2, 12, 16, 4, 2, 8}, {1, 8, 8, 1, 1, 2}, {4, 60, 64, 3, 1, 4},
                         {2, 128, 160, 8, 2, 8}};
  for (auto& c : cfgs) {
    const int L = c[0], E = c[1], P = c[2];
    std::vector<double> loads((size_t)L * E);
    for (double& v : loads) v = (double)(rng() % 1000);
    EplbPlacement p = eplb_rebalance(loads, L, E, P, c[3], c[4], c[5]);
    for (int l = 0; l < L; ++l) {
      std::vector<int> seen(E, 0);
      for (int s = 0; s < P; ++s) {
        const int e = p.phy2log[(size_t)l * P + s];
        if (e < 0 || e >= E) return 1;
        seen[e]++;
      }
      for (int e = 0; e < E; ++e)
        if (seen[e] != p.logcnt[(size_t)l * E + e] || seen[e] < 1) return 1;
    }
  }
  try {
    eplb_rebalance(std::vector<double>(8, 1.0), 1, 8, 9, 1, 1, 2);
    return 1;
  } catch (const std::invalid_argument&) {
  }
  return 0;
}

int main() {
  int rc = 0;
  rc |= run_eplb();
  rc |= run_engine(false, 64);
  rc |= run_engine(true, 24);      // few blocks: preemption and recompute
  rc |= run_offload_and_lmcache();
  std::printf(rc == 0 ? "sanitize driver ok\n" : "sanitize driver FAILED\n");
  return rc;
}
