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
#include <charconv>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <string_view>
#include <vector>

#include "blok_b200.h"

namespace {

struct Fail {
  std::string message;
};

// Decimal digits only, the whole of `text`; anything else is "bad <what>".
unsigned long long parse_number(std::string_view text, const char *what) {
  unsigned long long value = 0;
  const char *first = text.data(), *last = text.data() + text.size();
  const auto res = std::from_chars(first, last, value, 10);
  if (text.empty() || res.ec != std::errc() || res.ptr != last) throw Fail{std::string("bad ") + what};
  return value;
}

struct Options {
  std::string index, prompt;
  unsigned long long tokens = 0, seed = 0;
  bool synthetic = false;
  blok_model_config cfg;
};

// One row per integer flag that sets a field of the model configuration.
struct ConfigFlag {
  const char *name;
  int blok_model_config::*field;
};
const ConfigFlag kConfigFlags[] = {
    {"layers", &blok_model_config::layers},          {"experts", &blok_model_config::experts},
    {"vocab", &blok_model_config::vocab},            {"max-ctx", &blok_model_config::max_ctx},
    {"hidden", &blok_model_config::hidden},          {"inter", &blok_model_config::inter},
    {"dense-inter", &blok_model_config::dense_inter}, {"shared-inter", &blok_model_config::shared_inter},
    {"heads", &blok_model_config::heads},            {"q-rank", &blok_model_config::q_rank},
    {"kv-rank", &blok_model_config::kv_rank},        {"prefill-chunk", &blok_model_config::prefill_chunk},
};

Options parse_command_line(int argc, char **argv) {
  Options o;
  blok_model_default_config(&o.cfg);
  if ((argc - 1) % 2 != 0) throw Fail{"usage: blok-kimi-exec --index runtime-index.blok --prompt-tokens ids --tokens n"};
  for (int i = 1; i + 1 < argc; i += 2) {
    const std::string_view flag = argv[i], value = argv[i + 1];
    if (flag.substr(0, 2) != "--") throw Fail{"unknown flag: " + std::string(flag)};
    const std::string_view name = flag.substr(2);
    if (name == "index") o.index = value;
    else if (name == "prompt-tokens") o.prompt = value;
    else if (name == "tokens") o.tokens = parse_number(value, "tokens");
    else if (name == "synthetic-seed") o.seed = parse_number(value, "synthetic-seed"), o.synthetic = true;
    else {
      const ConfigFlag *hit = nullptr;
      for (const ConfigFlag &f : kConfigFlags)
        if (name == f.name) hit = &f;
      if (!hit) throw Fail{"unknown flag: " + std::string(flag)};
      o.cfg.*(hit->field) = (int)parse_number(value, hit->name);
    }
  }
  if ((o.index.empty() && !o.synthetic) || o.prompt.empty() || o.tokens == 0) throw Fail{"bad args"};
  return o;
}

std::vector<uint32_t> parse_prompt(const std::string &list, int vocab) {
  std::vector<uint32_t> ids;
  size_t at = 0;
  while (at <= list.size()) {
    size_t comma = list.find(',', at);
    if (comma == std::string::npos) comma = list.size();
    if (comma == at && comma == list.size()) break;  // nothing after a trailing comma
    const unsigned long long id = parse_number(std::string_view(list).substr(at, comma - at), "prompt token");
    if (id >= (unsigned long long)vocab) throw Fail{"prompt token outside vocabulary"};
    ids.push_back((uint32_t)id);
    at = comma + 1;
  }
  if (ids.empty()) throw Fail{"prompt token list is empty"};
  return ids;
}

void require_ok(int rc, const char *stage) {
  if (rc != BLOK_OK) throw Fail{std::string(stage) + ": " + blok_last_error()};
}

int run(int argc, char **argv) {
  Options o = parse_command_line(argc, argv);
  const std::vector<uint32_t> prompt = parse_prompt(o.prompt, o.cfg.vocab);
  if ((unsigned long long)o.cfg.max_ctx < prompt.size() + o.tokens) o.cfg.max_ctx = (int)(prompt.size() + o.tokens);
  // --synthetic-seed stands in for the checkpoint: the index is then not read.  Otherwise the index is parsed and
  // checked against the forward contract before any device memory is taken.
  if (!o.synthetic) require_ok(blok_index_validate(o.index.c_str(), &o.cfg, nullptr, nullptr), "index");
  blok_model_t *model = nullptr;
  require_ok(blok_model_create_synthetic(&o.cfg, o.seed, &model), "model");
  // every tensor of the forward contract is read once into the model's resident tensors
  if (!o.synthetic) require_ok(blok_model_load_index(model, o.index.c_str()), "index");
  std::vector<uint32_t> generated(o.tokens);
  int n = 0;
  require_ok(blok_model_generate(model, prompt.data(), (int)prompt.size(), (int)o.tokens, generated.data(), &n), "generate");
  std::string line = "{\"status\":\"ok\",\"token_ids\":[";
  for (int i = 0; i < n; ++i) {
    if (i) line += ',';
    line += std::to_string(generated[i]);
  }
  line += "]}\n";
  std::fputs(line.c_str(), stdout);
  blok_model_destroy(model);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  try {
    return run(argc, argv);
  } catch (const Fail &f) {
    std::fprintf(stderr, "%s\n", f.message.c_str());
    return 1;
  }
}
