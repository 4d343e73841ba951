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
//
//   ref_harness --sched MODEL.bw TRACE.txt OUT.txt
//
// Runs the reference's Engine (scheduler, block manager, preemption; src/engine.cpp:304-377)
// on a small workload and writes what it decided, step by step.  TRACE.txt: first line
// "num_blocks max_batched_tokens max_num_seqs", then one request a line, "arrival_step
// prompt_len max_new_tokens cancel_step" (cancel_step -1: never).  OUT.txt: for every step
// the events, the counters and Engine::debug_state() (every running and waiting request with
// its length, computed tokens and blocks).  Prefix caching is off and eos is ignored, so the
// schedule does not depend on the tokens the model produces.
//
//   ref_harness --uniform OUT.txt
//
// Writes counter_uniform(seed, position, stream) (src/engine.cpp:35-38) for a fixed list of
// arguments, as hexadecimal bit patterns of the doubles.
#include <cstdio>
#include <cstdlib>
#include <cstring>
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

static int run_sched(const char* model_path, const char* trace_path, const char* out_path) {
  auto model = Model::load(model_path);
  std::ifstream in(trace_path);
  EngineConfig ec;
  in >> ec.num_blocks >> ec.max_batched_tokens >> ec.max_num_seqs;
  ec.threads = 1;
  ec.prefix_caching = false;
  struct Req {
    int arrival, prompt_len, max_new, cancel;
    int64_t id = -1;
  };
  std::vector<Req> reqs;
  Req r;
  while (in >> r.arrival >> r.prompt_len >> r.max_new >> r.cancel) reqs.push_back(r);
  Engine engine(*model, nullptr, ec);
  const int V = model->config().vocab_size;
  std::ofstream out(out_path);
  std::size_t added = 0;
  for (int step = 0; step < 5000 && (added < reqs.size() || !engine.idle()); ++step) {
    for (std::size_t i = 0; i < reqs.size(); ++i) {
      Req& q = reqs[i];
      if (q.id < 0 && q.arrival <= step) {
        std::vector<int32_t> prompt(q.prompt_len);
        for (int j = 0; j < q.prompt_len; ++j) prompt[j] = static_cast<int32_t>((i * 7 + j * 3 + 1) % V);
        SamplingParams sp;
        sp.max_new_tokens = q.max_new;
        sp.ignore_eos = true;
        q.id = engine.add_request(prompt, sp);
        ++added;
      }
      if (q.id >= 0 && q.cancel >= 0 && q.arrival + q.cancel == step) engine.cancel(q.id);
    }
    const auto events = engine.step();
    const EngineStats& st = engine.stats();
    out << "step " << step << "\nevents";
    for (const auto& e : events) out << " " << e.id << ":" << e.tokens.size() << ":" << (e.finished ? 1 : 0);
    out << "\nstats " << st.prefill_tokens << " " << st.decode_rows << " " << st.preemptions << " "
        << st.generated_tokens << "\ncounts " << engine.num_running() << " " << engine.num_waiting() << " "
        << engine.free_blocks() << "\n"
        << engine.debug_state();
  }
  out << "end\n";
  return engine.idle() ? 0 : 3;
}

static int run_uniform(const char* out_path) {
  std::ofstream out(out_path);
  const uint64_t seeds[] = {0ull, 1ull, 7ull, 0x6A09E667F3BCC909ull, 0xFFFFFFFFFFFFFFFFull, 123456789012345ull};
  const int64_t positions[] = {0, 1, 2, 17, 1000, 4095, 1ll << 20, (1ll << 40) + 3};
  for (uint64_t seed : seeds)
    for (int64_t pos : positions)
      for (uint64_t stream = 0; stream < 4; ++stream) {
        const double u = counter_uniform(seed, pos, stream);
        uint64_t bits;
        static_assert(sizeof(bits) == sizeof(u), "double is 64 bits");
        std::memcpy(&bits, &u, sizeof(bits));
        out << seed << " " << pos << " " << stream << " " << std::hex << bits << std::dec << "\n";
      }
  return 0;
}

int main(int argc, char** argv) {
  if (argc == 5 && std::string(argv[1]) == "--sched") return run_sched(argv[2], argv[3], argv[4]);
  if (argc == 3 && std::string(argv[1]) == "--uniform") return run_uniform(argv[2]);
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
