// blok-kimi-exec: the reference executor's command line and output contract
// (src/kimi_exec.cu:532-544 args, :895-904 main) on top of libblok_b200.
//
//   blok-kimi-exec --index <runtime-index.blok> --prompt-tokens <id,id,...> --tokens <n>
//                  [--synthetic-seed <s>] [--layers <n>] [--experts <n>] [--vocab <n>] [--max-ctx <n>]
//                  [--hidden --inter --dense-inter --shared-inter --heads --q-rank --kv-rank <n>]
//                  [--prefill-chunk <n>]   prompt in chunks of n tokens (1..64) instead of token by token
//
// Success: exit 0 and exactly one stdout line {"status":"ok","token_ids":[...]}.
// Failure: a message on stderr and exit 1, which blok/runtime.py:86-94 turns into
// BlokRuntimeError.  Flags come in pairs and an unknown flag is an error, as in the
// reference.  Every tensor of the forward contract is read ONCE from the files the index
// names into the model's resident tensors on the current GPU (the model must fit that
// GPU: the size flags exist for reduced checkpoints and tests).  With --synthetic-seed
// the index is not read and the weights are seeded synthetic tensors of the requested size.
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "blok_b200.h"

[[noreturn]] static void die(const std::string &m) {
  std::cerr << m << "\n";
  std::exit(1);
}

static uint64_t u64(const char *s, const char *what) {
  char *end = nullptr;
  errno = 0;
  auto v = std::strtoull(s, &end, 10);
  if (errno || end == s || *end) die(std::string("bad ") + what);
  return v;
}

int main(int argc, char **argv) {
  std::string index, prompt;
  uint64_t tokens = 0, seed = 0;
  bool synthetic = false;
  blok_model_config cfg;
  blok_model_default_config(&cfg);
  for (int i = 1; i < argc; i += 2) {
    if (i + 1 >= argc) die("usage: blok-kimi-exec --index runtime-index.blok --prompt-tokens ids --tokens n");
    std::string f = argv[i];
    if (f == "--index") index = argv[i + 1];
    else if (f == "--prompt-tokens") prompt = argv[i + 1];
    else if (f == "--tokens") tokens = u64(argv[i + 1], "tokens");
    else if (f == "--synthetic-seed") seed = u64(argv[i + 1], "synthetic-seed"), synthetic = true;
    else if (f == "--layers") cfg.layers = (int)u64(argv[i + 1], "layers");
    else if (f == "--experts") cfg.experts = (int)u64(argv[i + 1], "experts");
    else if (f == "--vocab") cfg.vocab = (int)u64(argv[i + 1], "vocab");
    else if (f == "--max-ctx") cfg.max_ctx = (int)u64(argv[i + 1], "max-ctx");
    else if (f == "--hidden") cfg.hidden = (int)u64(argv[i + 1], "hidden");
    else if (f == "--inter") cfg.inter = (int)u64(argv[i + 1], "inter");
    else if (f == "--dense-inter") cfg.dense_inter = (int)u64(argv[i + 1], "dense-inter");
    else if (f == "--shared-inter") cfg.shared_inter = (int)u64(argv[i + 1], "shared-inter");
    else if (f == "--heads") cfg.heads = (int)u64(argv[i + 1], "heads");
    else if (f == "--q-rank") cfg.q_rank = (int)u64(argv[i + 1], "q-rank");
    else if (f == "--kv-rank") cfg.kv_rank = (int)u64(argv[i + 1], "kv-rank");
    else if (f == "--prefill-chunk") cfg.prefill_chunk = (int)u64(argv[i + 1], "prefill-chunk");
    else die("unknown flag: " + f);
  }
  if ((index.empty() && !synthetic) || prompt.empty() || tokens == 0) die("bad args");
  std::vector<uint32_t> ids;
  {
    std::istringstream in(prompt);
    std::string v;
    while (std::getline(in, v, ',')) {
      auto id = u64(v.c_str(), "prompt token");
      if (id >= (uint64_t)cfg.vocab) die("prompt token outside vocabulary");
      ids.push_back((uint32_t)id);
    }
  }
  if (ids.empty()) die("prompt token list is empty");
  if ((uint64_t)cfg.max_ctx < ids.size() + tokens) cfg.max_ctx = (int)(ids.size() + tokens);
  // --synthetic-seed stands in for the checkpoint: the index is then not read.  Otherwise the index is parsed and
  // checked against the forward contract before any device memory is taken.
  if (!synthetic && blok_index_validate(index.c_str(), &cfg, nullptr, nullptr) != BLOK_OK) die(std::string("index: ") + blok_last_error());
  blok_model_t *model = nullptr;
  if (blok_model_create_synthetic(&cfg, seed, &model) != BLOK_OK) die(std::string("model: ") + blok_last_error());
  // every tensor of the forward contract is read once into the model's resident tensors
  if (!synthetic && blok_model_load_index(model, index.c_str()) != BLOK_OK) die(std::string("index: ") + blok_last_error());
  std::vector<uint32_t> out(tokens);
  int n = 0;
  if (blok_model_generate(model, ids.data(), (int)ids.size(), (int)tokens, out.data(), &n) != BLOK_OK)
    die(std::string("generate: ") + blok_last_error());
  std::cout << "{\"status\":\"ok\",\"token_ids\":[";
  for (int i = 0; i < n; ++i) std::cout << (i ? "," : "") << out[i];
  std::cout << "]}\n";
  blok_model_destroy(model);
  return 0;
}
