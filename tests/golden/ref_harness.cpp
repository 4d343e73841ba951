// Drives the reference's own model code (src/kernels.cpp, src/model.cpp, src/engine.cpp,
// src/block_manager.cpp of tkran2/bitwise, compiled unmodified beside this file) on a tiny
// model, to anchor the plain implementation of the tests.
//
//   ref_harness MODEL.bw INV_FREQ.f32|- TOKENS.i32 OUT_LOGITS.f32 [GEN_OUT.txt PROMPT_LEN NEW TEMP SEED]
//
// Runs one forward over all tokens with logits wanted at every row (Runner::forward,
// src/model.cpp:267-322) and writes them.  INV_FREQ, when given, overwrites the public
// member Model::inv_freq_ (src/model.h:58) so that a rescaled rotary table can be
// anchored too.  With the optional arguments it also generates NEW tokens from the first
// PROMPT_LEN tokens through the reference's Engine (src/engine.cpp) and writes the tokens
// and the logits fingerprint as text.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "engine.h"
#include "model.h"

using namespace bw;

template <typename T>
static std::vector<T> read_all(const char* path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    std::fprintf(stderr, "cannot open %s\n", path);
    std::exit(2);
  }
  f.seekg(0, std::ios::end);
  const std::size_t n = static_cast<std::size_t>(f.tellg()) / sizeof(T);
  f.seekg(0);
  std::vector<T> v(n);
  f.read(reinterpret_cast<char*>(v.data()), n * sizeof(T));
  return v;
}

int main(int argc, char** argv) {
  if (argc < 5) {
    std::fprintf(stderr, "usage: ref_harness MODEL.bw INV_FREQ|- TOKENS OUT [GEN_OUT PROMPT_LEN NEW TEMP SEED]\n");
    return 2;
  }
  auto model = Model::load(argv[1]);
  if (std::string(argv[2]) != "-") {
    auto inv = read_all<float>(argv[2]);
    if (inv.size() != model->inv_freq_.size()) {
      std::fprintf(stderr, "inv_freq has %zu entries, model wants %zu\n", inv.size(), model->inv_freq_.size());
      return 2;
    }
    model->inv_freq_ = inv;
  }
  const auto tokens = read_all<int32_t>(argv[3]);
  const int n = static_cast<int>(tokens.size());
  const int V = model->config().vocab_size;
  {
    ThreadPool pool(1);
    KVPool kv(model->config(), (n + 15) / 16);
    Runner runner(*model, kv, pool, KernelMode::Invariant);
    std::vector<int32_t> table((n + 15) / 16);
    for (std::size_t i = 0; i < table.size(); ++i) table[i] = static_cast<int32_t>(i);
    std::vector<BatchRow> rows;
    for (int i = 0; i < n; ++i) rows.push_back({tokens[i], i, table.data(), true});
    int nl = 0;
    const float* l = runner.forward(rows, &nl);
    std::ofstream out(argv[4], std::ios::binary);
    out.write(reinterpret_cast<const char*>(l), sizeof(float) * static_cast<std::size_t>(nl) * V);
  }
  if (argc >= 10) {
    const int prompt_len = std::atoi(argv[6]);
    SamplingParams sp;
    sp.max_new_tokens = std::atoi(argv[7]);
    sp.temperature = static_cast<float>(std::atof(argv[8]));
    sp.seed = std::strtoull(argv[9], nullptr, 10);
    sp.ignore_eos = true;
    EngineConfig ec;
    ec.num_blocks = 64;
    ec.threads = 1;
    ec.prefix_caching = false;
    Engine engine(*model, nullptr, ec);
    std::vector<int32_t> prompt(tokens.begin(), tokens.begin() + prompt_len);
    const int64_t id = engine.add_request(prompt, sp);
    int guard = 0;
    while (!engine.idle() && guard++ < 10000) engine.step();
    const RequestResult& r = engine.result(id);
    std::ofstream out(argv[5]);
    out << r.logits_fingerprint << "\n";
    for (int32_t t : r.tokens) out << t << " ";
    out << "\n";
  }
  return 0;
}
