#include "runtime/native_runner.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <numeric>
#include <stdexcept>

#include "kernels/api.h"

namespace b200::rt {

namespace {
constexpr float kSamplingEps = 1e-5f;

void check(int rc, const char* what) {
  if (rc < 0) throw std::runtime_error(std::string(what) + ": kernel launcher returned " + std::to_string(rc));
}

uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
}  // namespace

NativeRunner::NativeRunner(std::unique_ptr<DenseModel> model, int block_size, int num_blocks, int max_num_seqs,
                           int max_num_batched_tokens, int max_model_len)
    : model_(std::move(model)), dev_(model_->device()), block_size_(block_size), num_blocks_(num_blocks),
      max_num_seqs_(max_num_seqs), max_tokens_(std::max(max_num_batched_tokens, max_num_seqs)),
      max_model_len_(max_model_len), max_blocks_((max_model_len + block_size - 1) / block_size + 1),
      layout_(StepLayout::make(max_tokens_, max_num_seqs, max_blocks_, 1, 0)),
      batch_(max_num_seqs, max_model_len, max_tokens_, std::vector<int>{block_size}) {
  set_device(dev_);
  if (dev_.cuda && b200_init_device() != 0) throw std::runtime_error("kernel library: device set-up failed");
  model_->alloc_kv_cache(num_blocks, block_size);
  model_->reserve(max_tokens_, max_num_seqs);
  host_buf_ = alloc_pinned(layout_.total_bytes);
  if (dev_.cuda) {
    dev_buf_ = alloc(layout_.total_bytes, dev_, true);
    dev_base_ = dev_buf_.as<uint8_t>();
    sampled_dev_ = alloc((size_t)layout_.max_logits * sizeof(int64_t), dev_, true);
    scratch_dev_ = alloc((size_t)layout_.max_logits * 64 * 8 + 1024, dev_);
    probs_dev_ = alloc((size_t)max_num_seqs * model_->config().vocab_size * sizeof(float), dev_);
    status_host_ = alloc_pinned(sizeof(int));
  } else {
    dev_base_ = host_buf_.as<uint8_t>();        // the step buffer is read in place
  }
  sampled_host_ = alloc_pinned((size_t)layout_.max_logits * sizeof(int64_t));
}

KVCacheConfig NativeRunner::kv_cache_config() const {
  KVCacheConfig k;
  k.num_blocks = num_blocks_;
  KVCacheGroupSpec g;
  const DenseConfig& c = model_->config();
  for (int l = 0; l < c.layers; ++l) g.layer_names.push_back("layers." + std::to_string(l));
  g.spec.kind = KVSpecKind::kFullAttention;
  g.spec.block_size = block_size_;
  g.spec.num_kv_heads = c.kv_heads;
  g.spec.head_size = c.head_dim;
  g.spec.dtype_bytes = 2;
  k.groups.push_back(std::move(g));
  return k;
}

void NativeRunner::execute_model(const SchedulerOutput& so) {
  batch_.update_states(so);
  for (auto& id : so.finished_req_ids) eos_.erase(id);
  if (so.total_num_scheduled_tokens == 0) {
    info_.reset();
    return;
  }
  set_device(dev_);
  info_ = batch_.prepare(so, layout_, host_buf_.as<uint8_t>(), /*async_mode=*/false);
  const StepInfo& info = *info_;
  if (dev_.cuda) {
    copy(dev_buf_.data(), dev_, host_buf_.data(), Device{}, layout_.total_bytes);
    h2d_bytes += (int64_t)layout_.total_bytes;
  }
  StepInputs in;
  in.num_tokens = info.num_tokens; in.num_reqs = info.num_reqs; in.num_decodes = info.num_decodes;
  in.num_prefills = info.num_prefills; in.num_prefill_tokens = info.num_prefill_tokens;
  in.num_tiles = info.num_tiles; in.num_logits = info.num_logits;
  in.input_ids = dev<int64_t>(layout_.input_ids);
  in.positions = dev<int64_t>(layout_.positions);
  in.slot_mapping = dev<int64_t>(layout_.slot_mapping);
  in.query_start = dev<int32_t>(layout_.query_start);
  in.seq_lens = dev<int32_t>(layout_.seq_lens);
  in.block_table = dev<int32_t>(layout_.block_table);
  in.max_blocks = max_blocks_;
  in.logits_indices = dev<int32_t>(layout_.logits_indices);
  in.tile_req = dev<int32_t>(layout_.tile_req);
  in.tile_q0 = dev<int32_t>(layout_.tile_q0);
  in.prefill_q_start = dev<int32_t>(layout_.prefill_q_start);
  logits_ = model_->forward(in);
}

// Sampler on host logits (CPU device): grammar bitmask -> logit bias / banned tokens -> penalties
// -> greedy snapshot -> temperature -> min_p -> top-k / top-p -> softmax -> seeded
// exponential-race draw; rows with temperature below eps keep the greedy id.
void NativeRunner::sample_host(const float* logits_in, const GrammarOutput* grammar, std::vector<int64_t>& ids) {
  const StepInfo& info = *info_;
  const int n = info.num_logits, V = model_->config().vocab_size;
  const int32_t* row_req = host<int32_t>(layout_.sample_rows);
  const float* temperature = host<float>(layout_.temperature);
  const float* top_p = host<float>(layout_.top_p);
  const float* min_p = host<float>(layout_.min_p);
  const int32_t* top_k = host<int32_t>(layout_.top_k);
  const uint64_t* seeds = host<uint64_t>(layout_.seeds);
  const uint64_t* steps = host<uint64_t>(layout_.steps);
  const float* rep = host<float>(layout_.rep_pen);
  const float* freq = host<float>(layout_.freq_pen);
  const float* pres = host<float>(layout_.pres_pen);
  std::vector<float> L((size_t)n * V);
  std::memcpy(L.data(), logits_in, L.size() * sizeof(float));
  const float ninf = -std::numeric_limits<float>::infinity();
  if (grammar && !grammar->structured_output_request_ids.empty()) {
    std::map<std::string, int> row_of;
    for (size_t r = 0; r < info.req_ids.size(); ++r)
      if (info.produces_token[r]) row_of[info.req_ids[r]] = info.logits_row0[r];
    for (size_t mi = 0; mi < grammar->structured_output_request_ids.size(); ++mi) {
      auto it = row_of.find(grammar->structured_output_request_ids[mi]);
      if (it == row_of.end()) continue;
      const int32_t* mask = grammar->bitmask.data() + mi * grammar->words_per_row;
      float* row = L.data() + (size_t)it->second * V;
      for (int t = 0; t < V; ++t)
        if (!((mask[t >> 5] >> (t & 31)) & 1)) row[t] = ninf;
    }
  }
  if (info.any_logit_edits) {
    std::vector<int32_t> br, bt, nr, nt;
    std::vector<float> bv;
    batch_.build_logit_edits(info, br, bt, bv, nr, nt, eos_);
    for (size_t i = 0; i < br.size(); ++i)
      if (bt[i] >= 0 && bt[i] < V) L[(size_t)br[i] * V + bt[i]] += bv[i];
    for (size_t i = 0; i < nr.size(); ++i)
      if (nt[i] >= 0 && nt[i] < V) L[(size_t)nr[i] * V + nt[i]] = ninf;
  }
  if (info.any_penalties) {
    std::vector<int32_t> pr, pt, pc;
    batch_.build_penalty_entries(info, pr, pt, pc);
    for (size_t i = 0; i < pr.size(); ++i) {
      if (pt[i] < 0 || pt[i] >= V) continue;
      const int b = row_req[pr[i]];
      float& x = L[(size_t)pr[i] * V + pt[i]];
      x = x > 0 ? x / rep[b] : x * rep[b];
      x = x - freq[b] * (float)pc[i] - (pc[i] > 0 ? pres[b] : 0.f);
    }
  }
  ids.assign(n, 0);
  std::vector<int> order(V);
  std::vector<float> probs(V);
  for (int r = 0; r < n; ++r) {
    float* row = L.data() + (size_t)r * V;
    int best = 0;
    for (int t = 1; t < V; ++t)
      if (row[t] > row[best]) best = t;
    ids[r] = best;
    const int b = row_req[r];
    const float temp = temperature[b];
    if (info.all_greedy || temp < kSamplingEps) continue;
    for (int t = 0; t < V; ++t) row[t] /= temp;
    auto softmax = [&]() {
      float mx = ninf;
      for (int t = 0; t < V; ++t) mx = std::max(mx, row[t]);
      double sum = 0;
      for (int t = 0; t < V; ++t) {
        probs[t] = row[t] == ninf ? 0.f : std::exp(row[t] - mx);
        sum += probs[t];
      }
      for (int t = 0; t < V; ++t) probs[t] = (float)(probs[t] / sum);
    };
    if (min_p[b] > 0) {
      softmax();
      float pm = 0;
      for (int t = 0; t < V; ++t) pm = std::max(pm, probs[t]);
      for (int t = 0; t < V; ++t)
        if (probs[t] < min_p[b] * pm) row[t] = ninf;
    }
    const int k = top_k[b];
    if (k > 0 && k < V) {
      std::vector<float> tmp(row, row + V);
      std::nth_element(tmp.begin(), tmp.begin() + (k - 1), tmp.end(), std::greater<float>());
      const float kth = tmp[k - 1];
      for (int t = 0; t < V; ++t)
        if (row[t] < kth) row[t] = ninf;
    }
    if (top_p[b] < 1.0f) {
      softmax();
      std::iota(order.begin(), order.end(), 0);
      std::stable_sort(order.begin(), order.end(), [&](int a, int c) { return probs[a] > probs[c]; });
      double total = 0;
      for (int t = 0; t < V; ++t) total += probs[t];
      double cs = 0;
      int cut = V - 1;
      for (int i = 0; i < V; ++i) {
        cs += probs[order[i]];
        if (cs >= (double)top_p[b] * total) { cut = i; break; }
      }
      const float thr = row[order[cut]];
      for (int t = 0; t < V; ++t)
        if (row[t] < thr) row[t] = ninf;
    }
    softmax();
    float best_key = -1.f;
    int best_i = 0;
    for (int t = 0; t < V; ++t) {
      if (probs[t] <= 0) continue;
      const uint64_t z = splitmix64(seeds[b] ^ splitmix64(steps[b] * 0x100000001B3ull + (uint64_t)t));
      const double u = ((double)(z >> 11) + 0.5) / 9007199254740992.0;
      const float e = (float)(-std::log(u));
      const float key = probs[t] / e;
      if (key > best_key) { best_key = key; best_i = t; }
    }
    ids[r] = best_i;
  }
}

// The same pipeline on the device, every stage a kernel of the library (sample.cu).
void NativeRunner::sample_device(float* logits, const GrammarOutput* grammar, std::vector<int64_t>& ids) {
  const StepInfo& info = *info_;
  const int n = info.num_logits, V = model_->config().vocab_size, R = info.num_reqs;
  cudaStream_t s = (cudaStream_t)current_stream(dev_);
  // per-row sampling scalars: the packed buffer holds them per batch row; a row compaction is
  // needed only when some request of the batch does not sample this step
  bool compact = n != R;
  for (int r = 0; r < R && !compact; ++r) compact = !info.produces_token[r];
  std::vector<Buffer> keep;
  auto upload_i32 = [&](const std::vector<int32_t>& v) {
    Buffer b = alloc(v.size() * 4 + 4, dev_);
    copy(b.data(), dev_, v.data(), Device{}, v.size() * 4);
    keep.push_back(b);
    return b.data();
  };
  auto upload_f32 = [&](const std::vector<float>& v) {
    Buffer b = alloc(v.size() * 4 + 4, dev_);
    copy(b.data(), dev_, v.data(), Device{}, v.size() * 4);
    keep.push_back(b);
    return b.data();
  };
  const int32_t* row_req = host<int32_t>(layout_.sample_rows);
  auto per_row = [&](size_t off, size_t elem) -> const void* {
    if (!compact) return dev<uint8_t>(off);
    std::vector<uint8_t> tmp((size_t)n * elem);
    for (int r = 0; r < n; ++r)
      std::memcpy(tmp.data() + (size_t)r * elem, host<uint8_t>(off) + (size_t)row_req[r] * elem, elem);
    Buffer b = alloc(tmp.size() + 8, dev_);
    copy(b.data(), dev_, tmp.data(), Device{}, tmp.size());
    synchronize(dev_);                 // tmp goes out of scope
    keep.push_back(b);
    return b.data();
  };
  if (grammar && !grammar->structured_output_request_ids.empty()) {
    std::map<std::string, int> row_of;
    for (size_t r = 0; r < info.req_ids.size(); ++r)
      if (info.produces_token[r]) row_of[info.req_ids[r]] = info.logits_row0[r];
    std::vector<int32_t> rows;
    for (auto& id : grammar->structured_output_request_ids) {
      auto it = row_of.find(id);
      rows.push_back(it == row_of.end() ? -1 : it->second);
    }
    check(b200_apply_bitmask(logits, V, V, upload_i32(grammar->bitmask), (int)rows.size(), upload_i32(rows), s),
          "apply_bitmask");
  }
  if (info.any_logit_edits) {
    std::vector<int32_t> br, bt, nr, nt;
    std::vector<float> bv;
    batch_.build_logit_edits(info, br, bt, bv, nr, nt, eos_);
    if (!br.empty())
      check(b200_sparse_edit(logits, V, V, upload_i32(br), upload_i32(bt), upload_f32(bv), (int)br.size(), 0, s),
            "logit_bias");
    if (!nr.empty())
      check(b200_sparse_edit(logits, V, V, upload_i32(nr), upload_i32(nt), nullptr, (int)nr.size(), 1, s),
            "token_mask");
  }
  if (info.any_penalties) {
    std::vector<int32_t> pr, pt, pc;
    batch_.build_penalty_entries(info, pr, pt, pc);
    if (!pr.empty())
      check(b200_apply_penalties(logits, V, V, upload_i32(pr), upload_i32(pt), upload_i32(pc), (int)pr.size(),
                                 per_row(layout_.rep_pen, 4), per_row(layout_.freq_pen, 4),
                                 per_row(layout_.pres_pen, 4), s), "penalties");
  }
  int64_t* out = sampled_dev_.as<int64_t>();
  float* sf = scratch_dev_.as<float>();
  int* si = reinterpret_cast<int*>(scratch_dev_.as<uint8_t>() + (size_t)n * 64 * 4);
  check(b200_argmax(logits, V, n, V, out, sf, si, s), "argmax");
  if (!info.all_greedy) {
    const void* temp = per_row(layout_.temperature, 4);
    Buffer greedy = alloc((size_t)n * 8, dev_);
    keep.push_back(greedy);
    copy(greedy.data(), dev_, out, dev_, (size_t)n * 8);
    check(b200_apply_temperature(logits, V, n, V, temp, s), "temperature");
    if (info.any_min_p) check(b200_apply_min_p(logits, V, n, V, per_row(layout_.min_p, 4), s), "min_p");
    if (info.any_top_k_top_p)
      check(b200_apply_top_k_top_p(logits, V, n, V, per_row(layout_.top_k, 4), per_row(layout_.top_p, 4), s),
            "top_k_top_p");
    float* probs = probs_dev_.as<float>();
    check(b200_softmax(logits, V, probs, V, n, V, 0, s), "softmax");
    Buffer rnd = alloc((size_t)n * 8, dev_);
    keep.push_back(rnd);
    check(b200_random_sample(probs, V, n, V, per_row(layout_.seeds, 8), per_row(layout_.steps, 8), rnd.data(), s),
          "random_sample");
    check(b200_merge_greedy_random(greedy.data(), rnd.data(), temp, out, n, s), "merge");
  }
  copy(sampled_host_.data(), Device{}, out, dev_, (size_t)n * 8);
  // the kernels' status word rides on the same copy
  copy(status_host_.data(), Device{}, b200_status_ptr(), dev_, sizeof(int));
  synchronize(dev_);
  d2h_bytes += (int64_t)n * 8 + 4;
  check_kernel_status();
  ids.assign(sampled_host_.as<int64_t>(), sampled_host_.as<int64_t>() + n);
}

void NativeRunner::check_kernel_status() {
  const int v = *status_host_.as<int>();
  if (v != 0)
    throw EngineDeadError("GPU kernel status " + std::to_string(v) +
                          ": a bounded wait inside a kernel ran out; the step's output was discarded");
}

ModelRunnerOutput NativeRunner::sample_tokens(const GrammarOutput* grammar) {
  ModelRunnerOutput out;
  if (!info_) return out;
  const StepInfo& info = *info_;
  out.req_ids = info.req_ids;
  std::vector<int64_t> ids;
  if (info.num_logits > 0) {
    set_device(dev_);
    if (dev_.cuda) sample_device(logits_, grammar, ids);
    else sample_host(logits_, grammar, ids);
  }
  int row = 0;
  for (size_t r = 0; r < info.req_ids.size(); ++r) {
    if (info.produces_token[r]) {
      std::vector<int32_t> t{(int32_t)ids[row]};
      batch_.append_sampled(info.req_ids[r], t);
      out.sampled_token_ids.push_back(std::move(t));
      row += 1 + info.num_draft[r];
    } else {
      out.sampled_token_ids.emplace_back();
    }
  }
  return out;
}

}  // namespace b200::rt
