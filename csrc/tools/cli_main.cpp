// b200-cli: one-shot completion over the native engine (no interpreter).
//   b200-cli --model <dir> --prompt "text" [--max-tokens N] [--temperature T] [--top-p P] [--top-k K]
//            [--seed S] [--device cuda|cpu] [--tokenize]
// With --tokenize it prints the prompt's token ids instead of generating.
// Reference: examples/cli/main.cpp and examples/tokenize/main.cpp.
#include <cstdio>
#include <cstdlib>
#include <string>

#include "runtime/native_llm.h"

int main(int argc, char** argv) {
  std::string model, prompt, device = "cuda";
  int max_tokens = 64;
  double temperature = 0.0, top_p = 1.0;
  int top_k = 0;
  bool tokenize = false, has_seed = false;
  uint64_t seed = 0;
  for (int i = 1; i < argc; ++i) {
    const std::string f = argv[i];
    auto next = [&]() -> const char* {
      if (i + 1 >= argc) { std::fprintf(stderr, "b200-cli: missing value for %s\n", f.c_str()); std::exit(2); }
      return argv[++i];
    };
    if (f == "--model") model = next();
    else if (f == "--prompt") prompt = next();
    else if (f == "--max-tokens") max_tokens = std::atoi(next());
    else if (f == "--temperature") temperature = std::atof(next());
    else if (f == "--top-p") top_p = std::atof(next());
    else if (f == "--top-k") top_k = std::atoi(next());
    else if (f == "--seed") { seed = std::strtoull(next(), nullptr, 10); has_seed = true; }
    else if (f == "--device") device = next();
    else if (f == "--tokenize") tokenize = true;
    else { std::fprintf(stderr, "b200-cli: unknown argument %s\n", f.c_str()); return 2; }
  }
  if (model.empty() || prompt.empty()) {
    std::fprintf(stderr, "usage: b200-cli --model <dir> --prompt \"text\" [--max-tokens N] [--temperature T]\n");
    return 2;
  }
  try {
    b200::rt::EngineOptions opt;
    opt.model_path = model;
    opt.device = device;
    opt.max_num_seqs = 1;
    opt.num_blocks = 0;
    auto llm = b200::rt::NativeLLM::load(opt);
    if (tokenize) {
      if (!llm->tokenizer()) throw std::runtime_error("no tokenizer beside the model");
      for (int t : llm->tokenizer()->encode(prompt)) std::printf("%d ", t);
      std::printf("\n");
      return 0;
    }
    b200::SamplingParams sp;
    sp.temperature = temperature;
    sp.top_p = top_p;
    sp.top_k = top_k;
    sp.max_tokens = max_tokens;
    if (has_seed) sp.seed = seed;
    llm->add_request(prompt, sp);
    while (llm->has_unfinished())
      for (auto& d : llm->step()) {
        std::fputs(d.delta_text.c_str(), stdout);
        std::fflush(stdout);
      }
    std::printf("\n");
  } catch (const std::exception& ex) {
    std::fprintf(stderr, "b200-cli: %s\n", ex.what());
    return 1;
  }
  return 0;
}
