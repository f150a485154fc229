// b200-bench: closed-loop throughput / latency benchmark over the native engine, no interpreter.
// The workload and the report follow the reference's tool (examples/bench/main.cpp,
// bench_core.h): N requests, at most C in flight, fixed input / output lengths, greedy,
// ignore-eos; request / output / total token throughput and TTFT / TPOT / ITL percentiles from
// the host clock around the engine's step() loop.
//
//   b200-bench --model <dir> [--num-prompts N] [--input-len L] [--output-len O] [--concurrency C]
//              [--max-num-batched-tokens B] [--device cuda|cpu] [--block-size S] [--seed S] [--json]
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <string>
#include <vector>

#include "runtime/native_llm.h"

using Clock = std::chrono::steady_clock;

static double pct(std::vector<double> v, double p) {
  if (v.empty()) return 0.0;
  std::sort(v.begin(), v.end());
  const double pos = p / 100.0 * (double)(v.size() - 1);
  const size_t lo = (size_t)pos;
  const size_t hi = std::min(lo + 1, v.size() - 1);
  return v[lo] + (v[hi] - v[lo]) * (pos - (double)lo);
}
static double mean(const std::vector<double>& v) {
  double s = 0;
  for (double x : v) s += x;
  return v.empty() ? 0.0 : s / (double)v.size();
}

int main(int argc, char** argv) {
  std::string model, device = "cuda";
  int num_prompts = 8, input_len = 16, output_len = 16, concurrency = 4, budget = 0, block = 32;
  uint64_t seed = 0;
  bool json = false;
  for (int i = 1; i < argc; ++i) {
    const std::string f = argv[i];
    auto next = [&]() -> const char* {
      if (i + 1 >= argc) { std::fprintf(stderr, "b200-bench: missing value for %s\n", f.c_str()); std::exit(2); }
      return argv[++i];
    };
    if (f == "--model") model = next();
    else if (f == "--num-prompts") num_prompts = std::atoi(next());
    else if (f == "--input-len") input_len = std::atoi(next());
    else if (f == "--output-len") output_len = std::atoi(next());
    else if (f == "--concurrency") concurrency = std::atoi(next());
    else if (f == "--max-num-batched-tokens") budget = std::atoi(next());
    else if (f == "--device") device = next();
    else if (f == "--block-size") block = std::atoi(next());
    else if (f == "--seed") seed = std::strtoull(next(), nullptr, 10);
    else if (f == "--json") json = true;
    else { std::fprintf(stderr, "b200-bench: unknown argument %s\n", f.c_str()); return 2; }
  }
  if (model.empty() || num_prompts <= 0 || input_len <= 0 || output_len <= 0 || concurrency <= 0) {
    std::fprintf(stderr, "usage: b200-bench --model <dir> [--num-prompts N] [--input-len L] [--output-len O]\n"
                         "                  [--concurrency C] [--max-num-batched-tokens B] [--device cuda|cpu]\n");
    return 2;
  }
  try {
    b200::rt::EngineOptions opt;
    opt.model_path = model;
    opt.device = device;
    opt.block_size = block;
    opt.max_model_len = input_len + output_len + block;
    opt.max_num_seqs = concurrency;
    opt.max_num_batched_tokens = budget;
    opt.num_blocks = concurrency * ((opt.max_model_len + block - 1) / block + 1) + 64;
    auto llm = b200::rt::NativeLLM::load(opt);
    const int V = llm->config().vocab_size;
    std::mt19937_64 rng(seed + 1);
    b200::SamplingParams sp;
    sp.temperature = 0.0;
    sp.max_tokens = output_len;
    sp.ignore_eos = true;
    sp.detokenize = false;
    struct Rec { double arrival = 0, first = -1, last = 0, done = 0; int out = 0; std::vector<double> itl; };
    std::map<std::string, Rec> recs;
    const auto t0 = Clock::now();
    auto now = [&] { return std::chrono::duration<double>(Clock::now() - t0).count(); };
    int next = 0, in_flight = 0, done = 0;
    auto admit = [&] {
      while (next < num_prompts && in_flight < concurrency) {
        std::vector<int32_t> ids((size_t)input_len);
        for (auto& t : ids) t = (int32_t)(rng() % (uint64_t)V);
        const std::string rid = llm->add_request_ids(std::move(ids), sp, std::to_string(next));
        recs[rid].arrival = now();
        ++next;
        ++in_flight;
      }
    };
    admit();
    int64_t steps = 0;
    while (done < num_prompts) {
      for (auto& d : llm->step()) {
        Rec& r = recs[d.request_id];
        if (!d.new_token_ids.empty()) {
          const double t = now();
          if (r.first < 0) r.first = t;
          else r.itl.push_back(t - r.last);
          r.last = t;
          r.out += (int)d.new_token_ids.size();
        }
        if (d.finished) {
          r.done = now();
          --in_flight;
          ++done;
        }
      }
      ++steps;
      admit();
    }
    const double dur = now();
    std::vector<double> ttft, tpot, itl;
    int64_t total_out = 0;
    for (auto& kv : recs) {
      const Rec& r = kv.second;
      total_out += r.out;
      ttft.push_back((r.first - r.arrival) * 1e3);
      if (r.out > 1) tpot.push_back((r.done - r.first) / (double)(r.out - 1) * 1e3);
      for (double x : r.itl) itl.push_back(x * 1e3);
    }
    const int64_t total_in = (int64_t)num_prompts * input_len;
    if (json) {
      std::printf("{\"completed\": %d, \"duration_s\": %.4f, \"total_input\": %lld, \"total_output\": %lld, "
                  "\"output_tok_s\": %.2f, \"total_tok_s\": %.2f, \"p50_ttft_ms\": %.2f, \"p50_tpot_ms\": %.3f, "
                  "\"p99_itl_ms\": %.3f, \"engine_steps\": %lld, \"kernel_launches\": %lld}\n",
                  done, dur, (long long)total_in, (long long)total_out, (double)total_out / dur,
                  (double)(total_in + total_out) / dur, pct(ttft, 50), pct(tpot, 50), pct(itl, 99), (long long)steps,
                  (long long)llm->runner().model().launches());
      return 0;
    }
    std::printf("\n============= b200 native engine benchmark =============\n");
    std::printf("%-42s %d\n", "Successful requests:", done);
    std::printf("%-42s %d\n", "Maximum request concurrency:", concurrency);
    std::printf("%-42s %.2f\n", "Benchmark duration (s):", dur);
    std::printf("%-42s %lld\n", "Total input tokens:", (long long)total_in);
    std::printf("%-42s %lld\n", "Total generated tokens:", (long long)total_out);
    std::printf("%-42s %.2f\n", "Request throughput (req/s):", (double)done / dur);
    std::printf("%-42s %.2f\n", "Output token throughput (tok/s):", (double)total_out / dur);
    std::printf("%-42s %.2f\n", "Total token throughput (tok/s):", (double)(total_in + total_out) / dur);
    std::printf("%-42s %.2f\n", "Mean TTFT (ms):", mean(ttft));
    std::printf("%-42s %.2f\n", "Median TTFT (ms):", pct(ttft, 50));
    std::printf("%-42s %.2f\n", "P99 TTFT (ms):", pct(ttft, 99));
    std::printf("%-42s %.2f\n", "Mean TPOT (ms):", mean(tpot));
    std::printf("%-42s %.2f\n", "Median TPOT (ms):", pct(tpot, 50));
    std::printf("%-42s %.2f\n", "P99 TPOT (ms):", pct(tpot, 99));
    std::printf("%-42s %.2f\n", "Median ITL (ms):", pct(itl, 50));
    std::printf("%-42s %.2f\n", "P99 ITL (ms):", pct(itl, 99));
    std::printf("=========================================================\n");
  } catch (const std::exception& ex) {
    std::fprintf(stderr, "b200-bench: %s\n", ex.what());
    return 1;
  }
  return 0;
}
