#include "worker/input_batch.h"

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace b200 {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

StepLayout StepLayout::make(int max_tokens, int max_reqs, int max_blocks, int num_groups,
                            int max_spec) {
  StepLayout l;
  l.max_logits = max_reqs * (1 + (max_spec > 0 ? max_spec : 0));
  l.max_tokens = max_tokens;
  l.max_reqs = max_reqs;
  l.max_blocks = max_blocks;
  l.num_groups = num_groups;
  l.max_tiles = (max_tokens + 127) / 128 + max_reqs;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  l.input_ids = take(8ull * max_tokens);
  l.positions = take(8ull * max_tokens);
  l.slot_mapping = take(8ull * max_tokens * num_groups);
  l.query_start = take(4ull * (max_reqs + 1));
  l.seq_lens = take(4ull * max_reqs);
  l.block_table = take(4ull * num_groups * max_reqs * max_blocks);
  l.logits_indices = take(4ull * l.max_logits);
  l.tile_req = take(4ull * l.max_tiles);
  l.tile_q0 = take(4ull * l.max_tiles);
  l.prefill_q_start = take(4ull * (max_reqs + 1));
  l.state_slots = take(4ull * max_reqs);
  l.temperature = take(4ull * max_reqs);
  l.top_p = take(4ull * max_reqs);
  l.min_p = take(4ull * max_reqs);
  l.top_k = take(4ull * max_reqs);
  l.seeds = take(8ull * max_reqs);
  l.steps = take(8ull * max_reqs);
  l.rep_pen = take(4ull * max_reqs);
  l.freq_pen = take(4ull * max_reqs);
  l.pres_pen = take(4ull * max_reqs);
  l.splice_dst = take(4ull * max_reqs);
  l.splice_src = take(4ull * max_reqs);
  l.sample_rows = take(4ull * l.max_logits);
  l.total_bytes = off;
  return l;
}

InputBatch::InputBatch(int max_num_reqs, int max_model_len, int max_num_tokens,
                       const std::vector<int>& block_sizes)
    : max_num_reqs_(max_num_reqs), max_model_len_(max_model_len),
      max_num_tokens_(max_num_tokens), block_sizes_(block_sizes) {
  for (int i = max_num_reqs - 1; i >= 0; --i) free_state_slots_.push_back(i);
}

int InputBatch::alloc_state_slot() {
  if (free_state_slots_.empty()) throw std::runtime_error("no free recurrent-state slot");
  int s = free_state_slots_.back();
  free_state_slots_.pop_back();
  return s;
}

const CachedRequestState* InputBatch::get(const std::string& id) const {
  auto it = reqs_.find(id);
  return it == reqs_.end() ? nullptr : &it->second;
}

std::vector<int32_t> InputBatch::propose_ngram(const std::string& id, int min_n, int max_n,
                                                int k) const {
  std::vector<int32_t> out;
  auto it = reqs_.find(id);
  if (it == reqs_.end() || k <= 0) return out;
  const std::vector<int32_t>& t = it->second.token_ids;
  const int n_tok = (int)t.size();
  for (int n = std::min(max_n, n_tok - 1); n >= std::max(1, min_n); --n) {
    const int32_t* tail = t.data() + n_tok - n;
    for (int start = n_tok - n - 1; start >= 0; --start) {
      if (!std::equal(tail, tail + n, t.data() + start)) continue;
      const int f0 = start + n, f1 = std::min(n_tok, f0 + k);
      if (f1 > f0) {
        out.assign(t.begin() + f0, t.begin() + f1);
        return out;
      }
    }
  }
  return out;
}

bool InputBatch::plain_greedy(const std::string& id) const {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) return false;
  const SamplingParams& sp = it->second.sampling_params;
  const int n_out = (int)it->second.token_ids.size() - it->second.num_prompt_tokens;
  return sp.temperature < kSamplingEps && !sp.has_penalties() && sp.logit_bias.empty() &&
         sp.allowed_token_ids.empty() && sp.bad_words_token_ids.empty() && !sp.logprobs &&
         n_out >= sp.min_tokens;
}

void InputBatch::update_states(const SchedulerOutput& so) {
  auto drop = [&](const std::string& id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return;
    if (it->second.state_slot >= 0) free_state_slots_.push_back(it->second.state_slot);
    reqs_.erase(it);
    last_rows_.erase(id);
  };
  for (auto& id : so.finished_req_ids) drop(id);
  for (auto& id : so.preempted_req_ids) drop(id);
  for (auto& n : so.scheduled_new_reqs) {
    drop(n.req_id);  // a resumed request replaces whatever was left
    CachedRequestState s;
    s.req_id = n.req_id;
    s.token_ids = n.prompt_token_ids;
    s.num_prompt_tokens = n.num_prompt_tokens;
    s.num_computed_tokens = n.num_computed_tokens;
    s.block_ids = n.block_ids;
    s.sampling_params = n.sampling_params;
    s.state_slot = alloc_state_slot();
    s.sample_step = (uint64_t)std::max(0, (int)n.prompt_token_ids.size() - n.num_prompt_tokens);
    reqs_.emplace(n.req_id, std::move(s));
  }
  auto& c = so.scheduled_cached_reqs;
  for (size_t i = 0; i < c.size(); ++i) {
    auto it = reqs_.find(c.req_ids[i]);
    if (it == reqs_.end()) throw std::runtime_error("cached request unknown to the worker: " + c.req_ids[i]);
    CachedRequestState& s = it->second;
    s.num_computed_tokens = c.num_computed_tokens[i];
    auto& nt = c.new_token_ids[i];
    if (!nt.empty()) {
      size_t lo = (size_t)s.num_computed_tokens;
      if (s.token_ids.size() < lo + nt.size()) s.token_ids.resize(lo + nt.size());
      std::copy(nt.begin(), nt.end(), s.token_ids.begin() + lo);
    }
    auto& nb = c.new_block_ids[i];
    if (s.block_ids.size() < nb.size()) s.block_ids.resize(nb.size());
    for (size_t g = 0; g < nb.size(); ++g)
      s.block_ids[g].insert(s.block_ids[g].end(), nb[g].begin(), nb[g].end());
  }
}

void InputBatch::append_sampled(const std::string& req_id, const std::vector<int32_t>& toks) {
  auto it = reqs_.find(req_id);
  if (it == reqs_.end()) return;
  auto& s = it->second;
  s.token_ids.insert(s.token_ids.end(), toks.begin(), toks.end());
}

StepInfo InputBatch::prepare(const SchedulerOutput& so, const StepLayout& L, uint8_t* buf,
                             bool async_mode) {
  StepInfo info;
  struct Item { CachedRequestState* s; int n; const std::vector<int32_t>* spec; };
  std::vector<Item> items;
  items.reserve(so.num_scheduled_tokens.size());
  for (auto& p : so.num_scheduled_tokens) {
    auto it = reqs_.find(p.first);
    if (it == reqs_.end()) throw std::runtime_error("scheduled request unknown to the worker: " + p.first);
    auto sp = so.scheduled_spec_decode_tokens.find(p.first);
    items.push_back({&it->second, p.second,
                     sp == so.scheduled_spec_decode_tokens.end() || sp->second.empty() ? nullptr : &sp->second});
  }
  // decode-first, stable
  std::stable_partition(items.begin(), items.end(), [](const Item& a) { return a.n == 1; });
  if ((int)items.size() > L.max_reqs) throw std::runtime_error("batch exceeds max_num_reqs");

  auto* input_ids = reinterpret_cast<int64_t*>(buf + L.input_ids);
  auto* positions = reinterpret_cast<int64_t*>(buf + L.positions);
  auto* slot_map = reinterpret_cast<int64_t*>(buf + L.slot_mapping);
  auto* qs = reinterpret_cast<int32_t*>(buf + L.query_start);
  auto* seq_lens = reinterpret_cast<int32_t*>(buf + L.seq_lens);
  auto* bt = reinterpret_cast<int32_t*>(buf + L.block_table);
  auto* logits_idx = reinterpret_cast<int32_t*>(buf + L.logits_indices);
  auto* tile_req = reinterpret_cast<int32_t*>(buf + L.tile_req);
  auto* tile_q0 = reinterpret_cast<int32_t*>(buf + L.tile_q0);
  auto* pqs = reinterpret_cast<int32_t*>(buf + L.prefill_q_start);
  auto* slots = reinterpret_cast<int32_t*>(buf + L.state_slots);
  auto* temp = reinterpret_cast<float*>(buf + L.temperature);
  auto* top_p = reinterpret_cast<float*>(buf + L.top_p);
  auto* min_p = reinterpret_cast<float*>(buf + L.min_p);
  auto* top_k = reinterpret_cast<int32_t*>(buf + L.top_k);
  auto* seeds = reinterpret_cast<uint64_t*>(buf + L.seeds);
  auto* steps = reinterpret_cast<uint64_t*>(buf + L.steps);
  auto* rep = reinterpret_cast<float*>(buf + L.rep_pen);
  auto* freq = reinterpret_cast<float*>(buf + L.freq_pen);
  auto* pres = reinterpret_cast<float*>(buf + L.pres_pen);
  auto* sp_dst = reinterpret_cast<int32_t*>(buf + L.splice_dst);
  auto* sp_src = reinterpret_cast<int32_t*>(buf + L.splice_src);
  auto* sample_rows = reinterpret_cast<int32_t*>(buf + L.sample_rows);

  const int G = L.num_groups;
  int tok = 0;
  qs[0] = 0;
  pqs[0] = 0;
  std::unordered_map<std::string, int> new_rows;
  for (size_t r = 0; r < items.size(); ++r) {
    CachedRequestState& s = *items[r].s;
    const int n = items[r].n;
    const int lo = s.num_computed_tokens;
    if (tok + n > L.max_tokens) throw std::runtime_error("batch exceeds max_num_batched_tokens");
    const bool is_decode = (n == 1);
    if (is_decode) { info.num_decodes++; info.num_decode_tokens += n; }
    else { info.num_prefills++; info.num_prefill_tokens += n; }
    for (int i = 0; i < n; ++i) {
      const int p = lo + i;
      int64_t id = 0;
      if (p < (int)s.token_ids.size()) {
        id = s.token_ids[p];
      } else if (items[r].spec && p - (int)s.token_ids.size() < (int)items[r].spec->size()) {
        id = (*items[r].spec)[p - (int)s.token_ids.size()];   // a draft token to verify
      } else if (async_mode) {
        auto lr = last_rows_.find(s.req_id);
        if (lr == last_rows_.end()) throw std::runtime_error("no in-flight token for " + s.req_id);
        sp_dst[info.num_splice] = tok + i;
        sp_src[info.num_splice] = lr->second;
        info.num_splice++;
      } else {
        throw std::runtime_error("token position beyond known tokens for " + s.req_id);
      }
      input_ids[tok + i] = id;
      positions[tok + i] = p;
      for (int g = 0; g < G; ++g) {
        int64_t slot = -1;
        if (g < (int)s.block_ids.size() && g < (int)block_sizes_.size() && block_sizes_[g] > 0) {
          const int bs = block_sizes_[g];
          const size_t bi = (size_t)(p / bs);
          if (bi < s.block_ids[g].size()) slot = (int64_t)s.block_ids[g][bi] * bs + (p % bs);
        }
        slot_map[(size_t)g * L.max_tokens + tok + i] = slot;
      }
    }
    tok += n;
    qs[r + 1] = tok;
    seq_lens[r] = lo + n;
    info.max_query_len = std::max(info.max_query_len, n);
    info.max_seq_len = std::max(info.max_seq_len, lo + n);
    for (int g = 0; g < G; ++g) {
      int32_t* row = bt + ((size_t)g * L.max_reqs + r) * L.max_blocks;
      size_t nb = g < (int)s.block_ids.size() ? s.block_ids[g].size() : 0;
      size_t ncopy = std::min(nb, (size_t)L.max_blocks);
      if (ncopy) std::memcpy(row, s.block_ids[g].data(), ncopy * sizeof(int32_t));
      if (ncopy < (size_t)L.max_blocks) row[ncopy] = 0;
    }
    if (!is_decode) {
      int pi = info.num_prefills - 1;
      for (int q0 = 0; q0 < n; q0 += 128) {
        tile_req[info.num_tiles] = pi;
        tile_q0[info.num_tiles] = q0;
        info.num_tiles++;
      }
      pqs[pi + 1] = pqs[pi] + n;
    }
    slots[r] = s.state_slot;
    const SamplingParams& sp = s.sampling_params;
    temp[r] = (float)sp.temperature;
    top_p[r] = (float)sp.top_p;
    min_p[r] = (float)sp.min_p;
    top_k[r] = sp.top_k;
    seeds[r] = sp.seed ? *sp.seed : (0x5DEECE66Dull ^ std::hash<std::string>{}(s.req_id));
    steps[r] = s.sample_step;
    rep[r] = (float)sp.repetition_penalty;
    freq[r] = (float)sp.frequency_penalty;
    pres[r] = (float)sp.presence_penalty;
    const bool produces = lo + n >= (int)s.token_ids.size();
    info.produces_token.push_back(produces ? 1 : 0);
    // drafts verified this step: the scheduled positions beyond the known tokens
    // (positions beyond the known tokens without a draft are in-flight tokens of async scheduling)
    const int k = (produces && items[r].spec)
                      ? std::min((int)items[r].spec->size(), std::max(0, lo + n - (int)s.token_ids.size()))
                      : 0;
    info.num_draft.push_back(k);
    info.logits_row0.push_back(produces ? info.num_logits : -1);
    if (produces) {
      if (info.num_logits + k + 1 > L.max_logits) throw std::runtime_error("batch exceeds the logits rows of the layout");
      for (int i = 0; i <= k; ++i) {   // one row per draft position plus the bonus position
        sample_rows[info.num_logits] = (int32_t)r;
        logits_idx[info.num_logits++] = tok - 1 - k + i;
      }
      s.sample_step += 1;
      if (sp.temperature >= kSamplingEps) {
        info.all_greedy = false;
        if (sp.top_k > 0 || sp.top_p < 1.0) info.any_top_k_top_p = true;
        if (sp.min_p > 0.0) info.any_min_p = true;
      }
      if (sp.has_penalties()) info.any_penalties = true;
      if (sp.logprobs) info.any_logprobs = true;
      const int n_out_now = (int)s.token_ids.size() - s.num_prompt_tokens;
      if (!sp.logit_bias.empty() || !sp.allowed_token_ids.empty() || !sp.bad_words_token_ids.empty() ||
          n_out_now < sp.min_tokens)
        info.any_logit_edits = true;
    }
    info.max_logprobs.push_back(sp.logprobs ? *sp.logprobs : -1);
    info.req_ids.push_back(s.req_id);
    info.num_scheduled.push_back(n);
    s.batch_row = (int)r;
    new_rows[s.req_id] = (int)r;
  }
  info.num_reqs = (int)items.size();
  info.num_tokens = tok;
  last_rows_.swap(new_rows);
  return info;
}

void InputBatch::build_penalty_entries(const StepInfo& info, std::vector<int32_t>& rows,
                                       std::vector<int32_t>& toks,
                                       std::vector<int32_t>& out_cnt) const {
  rows.clear(); toks.clear(); out_cnt.clear();
  for (size_t r = 0; r < info.req_ids.size(); ++r) {
    if (!info.produces_token[r]) continue;
    const int row = info.logits_row0[r];
    auto it = reqs_.find(info.req_ids[r]);
    if (it == reqs_.end()) continue;
    const CachedRequestState& s = it->second;
    if (!s.sampling_params.has_penalties()) continue;
    std::map<int32_t, int32_t> cnt;  // token -> output count (0 = prompt only)
    for (int i = 0; i < (int)s.token_ids.size(); ++i) {
      auto& c = cnt[s.token_ids[i]];
      if (i >= s.num_prompt_tokens) ++c;
    }
    for (auto& kv : cnt) {
      rows.push_back(row);
      toks.push_back(kv.first);
      out_cnt.push_back(kv.second);
    }
  }
}

void InputBatch::build_logit_edits(const StepInfo& info, std::vector<int32_t>& bias_rows,
                                   std::vector<int32_t>& bias_toks, std::vector<float>& bias_vals,
                                   std::vector<int32_t>& ban_rows, std::vector<int32_t>& ban_toks,
                                   const std::map<std::string, int32_t>& eos_of) const {
  bias_rows.clear(); bias_toks.clear(); bias_vals.clear(); ban_rows.clear(); ban_toks.clear();
  for (size_t r = 0; r < info.req_ids.size(); ++r) {
    if (!info.produces_token[r]) continue;
    const int row = info.logits_row0[r];
    auto it = reqs_.find(info.req_ids[r]);
    if (it == reqs_.end()) continue;
    const CachedRequestState& s = it->second;
    const SamplingParams& sp = s.sampling_params;
    for (auto& kv : sp.logit_bias) {
      bias_rows.push_back(row);
      bias_toks.push_back(kv.first);
      bias_vals.push_back(kv.second);
    }
    const int n_out = (int)s.token_ids.size() - s.num_prompt_tokens;
    if (n_out < sp.min_tokens) {
      auto e = eos_of.find(s.req_id);
      if (e != eos_of.end() && e->second >= 0) { ban_rows.push_back(row); ban_toks.push_back(e->second); }
      for (int32_t t : sp.stop_token_ids) { ban_rows.push_back(row); ban_toks.push_back(t); }
    }
    // bad words: ban the last token of a sequence whose prefix matches the current tail
    for (auto& bw : sp.bad_words_token_ids) {
      if (bw.empty()) continue;
      size_t k = bw.size() - 1;
      if (k > s.token_ids.size()) continue;
      if (std::equal(bw.begin(), bw.begin() + k, s.token_ids.end() - k)) {
        ban_rows.push_back(row);
        ban_toks.push_back(bw.back());
      }
    }
  }
}

}  // namespace b200
