// Times tkran2/bitwise's own model code on the benchmark shape, through its public classes
// (Model::random, KVPool, Runner::forward, argmax_row; src/model.h, src/engine.h), compiled
// unmodified beside this file with the reference's own flags (CMakeLists.txt:15-18).
//
//   ref_bench LAYERS HIDDEN HEADS KV_HEADS HEAD_DIM INTERMEDIATE VOCAB THETA THREADS CTX
//             BATCH STEPS WARMUP PREFILL_TOKENS [POINT_BATCH ...]
//
// Decode: BATCH rows at position CTX - 1, each over a block table of its own (up to eight
// distinct key/value sets, cycled over larger batches, as the timing does not depend on what
// the cache holds), one Runner::forward per step, timed by the host clock after WARMUP steps;
// "e2e" adds the reference's greedy sampler over the logits rows it returns (host tokens in,
// host tokens out: this engine lives on the CPU, no copies to count).  Prefill: one forward
// over PREFILL_TOKENS rows of one sequence, logits at the last.  Prints one line of JSON.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "engine.h"
#include "model.h"

using namespace bw;
using Clock = std::chrono::steady_clock;

static double seconds_since(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

int main(int argc, char** argv) {
  if (argc < 15) {
    std::fprintf(stderr, "usage: ref_bench LAYERS HIDDEN HEADS KV_HEADS HEAD_DIM INTERMEDIATE VOCAB THETA THREADS CTX "
                         "BATCH STEPS WARMUP PREFILL_TOKENS [POINT_BATCH ...]\n");
    return 2;
  }
  ModelConfig cfg;
  cfg.arch = "llama";
  cfg.layers = std::atoi(argv[1]);
  cfg.hidden = std::atoi(argv[2]);
  cfg.heads = std::atoi(argv[3]);
  cfg.kv_heads = std::atoi(argv[4]);
  cfg.head_dim = std::atoi(argv[5]);
  cfg.intermediate = std::atoi(argv[6]);
  cfg.vocab_size = std::atoi(argv[7]);
  cfg.rope_theta = static_cast<float>(std::atof(argv[8]));
  cfg.rms_eps = 1e-5f;
  const int threads = std::atoi(argv[9]), ctx = std::atoi(argv[10]), batch = std::atoi(argv[11]);
  const int steps = std::atoi(argv[12]), warmup = std::atoi(argv[13]), prefill_tokens = std::atoi(argv[14]);
  std::vector<int> points;
  for (int i = 15; i < argc; ++i) points.push_back(std::atoi(argv[i]));

  auto t_build = Clock::now();
  auto model = Model::random(cfg, 1, DType::BF16);  // bf16 weights, fp32 compute: the reference's serving mode
  const double build_s = seconds_since(t_build);
  ThreadPool pool(threads);
  const int bs = 16;
  const int blocks_per_seq = (std::max(ctx, prefill_tokens) + bs - 1) / bs;
  const int sets = 8;
  KVPool kv(model->config(), sets * blocks_per_seq, bs);  // zero-filled
  Runner runner(*model, kv, pool, KernelMode::Invariant);
  std::vector<std::vector<int32_t>> tables(sets, std::vector<int32_t>(blocks_per_seq));
  for (int s = 0; s < sets; ++s)
    for (int b = 0; b < blocks_per_seq; ++b) tables[s][b] = s * blocks_per_seq + b;
  const int V = cfg.vocab_size;

  auto decode = [&](int b, int n_steps, int n_warm, double* e2e_ms) {
    std::vector<BatchRow> rows;
    for (int i = 0; i < b; ++i) rows.push_back({(i * 7919 + 13) % V, ctx - 1, tables[i % sets].data(), true});
    std::vector<int32_t> sampled(b);
    int nl = 0;
    for (int i = 0; i < n_warm; ++i) runner.forward(rows, &nl);
    auto t0 = Clock::now();
    for (int i = 0; i < n_steps; ++i) runner.forward(rows, &nl);
    const double ms = seconds_since(t0) * 1e3 / n_steps;
    if (e2e_ms) {
      auto t1 = Clock::now();
      for (int i = 0; i < n_steps; ++i) {
        const float* logits = runner.forward(rows, &nl);
        for (int r = 0; r < nl; ++r) sampled[r] = argmax_row(logits + static_cast<std::size_t>(r) * V, V);
        for (int r = 0; r < b; ++r) rows[r].token = sampled[r];  // the next step's input, as an engine would feed it
      }
      *e2e_ms = seconds_since(t1) * 1e3 / n_steps;
    }
    return ms;
  };

  double e2e_ms = 0.0;
  const double ms = decode(batch, steps, warmup, &e2e_ms);
  std::printf("{\"ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f, \"build_seconds\": %.2f, \"threads\": %d", ms, e2e_ms,
              build_s, threads);
  for (int pb : points) {
    const double pm = decode(pb, std::max(3, steps / 4), 1, nullptr);
    std::printf(", \"decode_b%d_ms\": %.4f", pb, pm);
  }
  if (prefill_tokens > 0) {
    std::vector<BatchRow> rows;
    for (int i = 0; i < prefill_tokens; ++i)
      rows.push_back({(i * 31 + 7) % V, i, tables[0].data(), i == prefill_tokens - 1});
    int nl = 0;
    auto t0 = Clock::now();
    runner.forward(rows, &nl);
    std::printf(", \"prefill_ms\": %.2f", seconds_since(t0) * 1e3);
  }
  std::printf("}\n");
  return 0;
}
