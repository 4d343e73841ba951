// Kernels that both precisions share: embedding gather into the 32-bit residual stream,
// sampling from 32-bit logits, and the logits fingerprint.
#include <cstdarg>
#include <cstdio>

#include "bw_common.cuh"

namespace bw {
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
}  // namespace bw

BW_API const char* bw_last_error() { return bw::g_error; }

// ---------------------------------------------------------------------------------------
// The failure word (see bw_common.cuh).
namespace bw {
static int* g_failure_word = nullptr;
static bool g_failure_word_owned = false;
int* failure_word() {
  if (!g_failure_word) {
    cudaError_t e = cudaMalloc(&g_failure_word, sizeof(int));
    if (e != cudaSuccess) {
      g_failure_word = nullptr;
      set_error("cannot allocate the failure word: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cudaMemset(g_failure_word, 0, sizeof(int));
    g_failure_word_owned = true;
  }
  return g_failure_word;
}
}  // namespace bw

// The caller's word of device memory (an int that is zero) for this library's kernels to raise
// when a bounded wait runs out; several libraries may share one word. Null: back to a word of
// the library's own.
BW_API void bw_set_failure_word(int* word) {
  if (bw::g_failure_word_owned && bw::g_failure_word) cudaFree(bw::g_failure_word);
  bw::g_failure_word = word;
  bw::g_failure_word_owned = false;
}

// Reads and clears the failure word: 1 (once) when a kernel gave up a bounded wait since the
// last call. A copy of four bytes that waits for the device.
BW_API int bw_device_failure() {
  if (!bw::g_failure_word) return 0;
  int v = 0;
  if (cudaMemcpy(&v, bw::g_failure_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
  if (v) cudaMemset(bw::g_failure_word, 0, sizeof(int));
  return v != 0;
}

// A check of the machinery above that needs no fault: one warp waits, with the helper that
// every kernel uses, for a barrier on which nothing ever arrives, gives up after `polls` polls,
// raises the failure word as the kernels do and returns. result[0] becomes 1 when the wait
// reported success (it must not), 2 when it gave up.
__global__ void bounded_wait_selftest_kernel(uint32_t polls, int* failure, int* result) {
  __shared__ uint64_t bar;
  __shared__ uint32_t gave_up;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&bar))), "r"(1));
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool ok = bw::mbar_wait_bounded(&bar, 0, &gave_up, polls);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (gave_up) atomicExch(failure, 1);
    result[0] = ok ? 1 : 2;
  }
}

BW_API int bw_selftest_bounded_wait(unsigned polls, int* result, cudaStream_t stream) {
  if (polls > 1000000u) {
    bw::set_error("bounded-wait self-test: %u polls is more than a test needs (at most 1000000)", polls);
    return -1;
  }
  int* word = bw::failure_word();
  if (!word) return -1;
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(polls, word, result);
  return bw::launch_status();
}

// ---------------------------------------------------------------------------------------
// Embedding: x[r][:] = E[token_r][:], widened to float (src/model.cpp:233-239,274).

template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                  float* __restrict__ out, int n, int width) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const T* src = table + static_cast<size_t>(tokens[r]) * width;
  float* dst = out + static_cast<size_t>(r) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = static_cast<float>(src[i]);
}

BW_API int bw_embed_rows(const void* table, int table_is_bf16, const int* tokens, float* out, int n,
                         int width, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_is_bf16)
    bw::launch_pdl(embed_rows_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(table), tokens, out, n, width);
  else
    bw::launch_pdl(embed_rows_kernel<float>, dim3(n), dim3(threads), 0, stream, static_cast<const float*>(table), tokens, out, n, width);
  return bw::launch_status();
}

// ---------------------------------------------------------------------------------------
// Tokens that the step before sampled and the host has not read yet go from the sampler's
// output straight into this step's token list: tokens[rows[i]] = values[src[i]].
__global__ void patch_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ rows, const int* __restrict__ src,
                                    const int* __restrict__ values, int count) {
  bw::pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) tokens[rows[i]] = values[src[i]];
}

BW_API int bw_patch_tokens(int* tokens, const int* rows, const int* src, const int* values, int count, cudaStream_t stream) {
  if (count <= 0) return 0;
  bw::launch_pdl(patch_tokens_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, tokens, rows, src, values, count);
  return bw::launch_status();
}

// ---------------------------------------------------------------------------------------
// Sampling. One block per logits row.
//   temperature <= 0: the first index of the maximum (src/engine.cpp:40-45).
//   otherwise: w_i = exp((l_i - max) / T) in 32-bit, total and running sums in 64-bit in
//   vocabulary order, the first i with cum > u * total, skipping w_i <= 0, else the last
//   positive one (src/engine.cpp:50-80).  The 64-bit sums are formed per contiguous
//   segment of the vocabulary (one per thread) and chained over the segments in order; the
//   reference adds strictly one by one, which differs from this by 64-bit rounding only.
constexpr int kSampleThreads = 512;

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                   const double* __restrict__ uniform, int* __restrict__ out_token) {
  bw::pdl_enter();
  const int row = blockIdx.x;
  const float* l = logits + static_cast<size_t>(row) * vocab;
  const int tid = threadIdx.x;
  __shared__ float s_val[kSampleThreads];
  __shared__ int s_idx[kSampleThreads];
  __shared__ double s_sum[kSampleThreads];
  __shared__ double s_total;
  __shared__ int s_pick;
  __shared__ int s_last;

  // maximum and its first index
  float best = -INFINITY;
  int best_i = -1;
  for (int i = tid; i < vocab; i += kSampleThreads) {
    const float v = l[i];
    if (best_i < 0 || v > best) {  // indices come in increasing order: ">" keeps the first maximum
      best = v;
      best_i = i;
    }
  }
  s_val[tid] = best;
  s_idx[tid] = best_i;
  __syncthreads();
  for (int s = kSampleThreads / 2; s > 0; s >>= 1) {
    if (tid < s) {
      const float ov = s_val[tid + s];
      const int oi = s_idx[tid + s];
      const int mi = s_idx[tid];
      if (oi >= 0 && (mi < 0 || ov > s_val[tid] || (ov == s_val[tid] && oi < mi))) {
        s_val[tid] = ov;
        s_idx[tid] = oi;
      }
    }
    __syncthreads();
  }
  const float mx = s_val[0];
  const int arg = s_idx[0];
  __syncthreads();  // s_idx is reused below
  const float temp = temperature[row];
  if (!(temp > 0.0f)) {
    if (tid == 0) out_token[row] = arg;
    return;
  }

  // contiguous segment of this thread
  const int seg = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int lo = min(vocab, tid * seg), hi = min(vocab, lo + seg);
  double local = 0.0;
  int last_pos = -1;
  for (int i = lo; i < hi; ++i) {
    const float w = bw::det_expf(__fdiv_rn(__fsub_rn(l[i], mx), temp));
    if (w > 0.0f) last_pos = i;
    local += static_cast<double>(w);
  }
  s_sum[tid] = local;
  s_idx[tid] = last_pos;
  if (tid == 0) s_pick = 0x7fffffff;
  __syncthreads();
  if (tid == 0) {  // exclusive prefix over segments, in order
    double run = 0.0;
    int lastp = 0;
    for (int t = 0; t < kSampleThreads; ++t) {
      const double v = s_sum[t];
      s_sum[t] = run;
      run += v;
      if (s_idx[t] >= 0) lastp = s_idx[t];
    }
    s_last = lastp;
    s_total = run;
  }
  __syncthreads();
  const double total = s_total;
  const double target = uniform[row] * total;
  double cum = s_sum[tid];
  for (int i = lo; i < hi; ++i) {
    const float w = bw::det_expf(__fdiv_rn(__fsub_rn(l[i], mx), temp));
    if (w <= 0.0f) continue;
    cum += static_cast<double>(w);
    if (cum > target) {
      atomicMin(&s_pick, i);
      break;
    }
  }
  __syncthreads();
  if (tid == 0) out_token[row] = (s_pick != 0x7fffffff) ? s_pick : s_last;
}

BW_API int bw_sample_rows(const float* logits, int rows, int vocab, const float* temperature,
                          const double* uniform, int* out_token, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) {
    bw::set_error("sample_rows: vocabulary size %d", vocab);
    return -1;
  }
  bw::launch_pdl(sample_rows_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, logits, vocab, temperature, uniform, out_token);
  return bw::launch_status();
}

// ---------------------------------------------------------------------------------------
// Logits fingerprint: the reference chains an FNV-style hash over the raw bits of every
// sampled-from logits row (src/engine.cpp:18-29): for each 8-byte word h = (h ^ w) * prime,
// trailing bytes one by one, then the splitmix64 finaliser.  The chain is serial by
// definition.  state[slot[r]] holds the running hash.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// One warp per row: the lanes fetch 32 consecutive words at a time (one coalesced read, the
// next group already on its way) and every lane runs the same chain over them, taking word j
// from lane j; no lane waits for memory inside the chain. The chain itself is written in 32-bit
// halves: the prime is 2^40 + 0x1B3, so with t = h ^ w the new low half is t.lo * 0x1B3 and the
// new high half hi(t.lo * 0x1B3) + t.hi * 0x1B3 + (t.lo << 8): two dependent instructions a
// word on each half instead of the chain of a general 64-bit product.
struct Hash64 {
  uint32_t lo, hi;
};
__device__ __forceinline__ void hash_step(Hash64& h, uint32_t w_lo, uint32_t w_hi) {
  const uint32_t t_lo = h.lo ^ w_lo, t_hi = h.hi ^ w_hi;
  h.lo = t_lo * 0x1B3u;
  h.hi = __umulhi(t_lo, 0x1B3u) + (t_lo << 8) + t_hi * 0x1B3u;
}

__global__ void __launch_bounds__(32)
fingerprint_rows_kernel(const float* __restrict__ logits, int rows, int vocab, const int* __restrict__ slot,
                        unsigned long long* __restrict__ state) {
  bw::pdl_enter();
  const int r = blockIdx.x, lane = threadIdx.x;
  if (r >= rows) return;
  const uint32_t* w = reinterpret_cast<const uint32_t*>(logits + static_cast<size_t>(r) * vocab);
  const uint64_t h0 = state[slot[r]];
  Hash64 h{static_cast<uint32_t>(h0), static_cast<uint32_t>(h0 >> 32)};
  const int words = vocab / 2;  // whole 8-byte words
  auto fetch = [&](int base) -> uint2 {
    const int i = base + lane;
    if (i >= words) return make_uint2(0u, 0u);
    return *reinterpret_cast<const uint2*>(w + 2 * i);  // rows of an even vocabulary start on 8 bytes
  };
  const bool aligned8 = (reinterpret_cast<uintptr_t>(w) & 7) == 0;
  if (aligned8) {
    uint2 cur = fetch(0);
    for (int base = 0; base < words; base += 32) {
      const uint2 nxt = fetch(base + 32);
      const int count = min(32, words - base);
      if (count == 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) hash_step(h, __shfl_sync(0xffffffffu, cur.x, j), __shfl_sync(0xffffffffu, cur.y, j));
      } else {
        for (int j = 0; j < count; ++j) hash_step(h, __shfl_sync(0xffffffffu, cur.x, j), __shfl_sync(0xffffffffu, cur.y, j));
      }
      cur = nxt;
    }
  } else {
    for (int i = 0; i < words; ++i) hash_step(h, w[2 * i], w[2 * i + 1]);
  }
  if (vocab & 1) {
    const uint32_t v = w[vocab - 1];
    for (int b = 0; b < 4; ++b) hash_step(h, (v >> (8 * b)) & 0xffu, 0u);
  }
  if (lane == 0) state[slot[r]] = mix64(static_cast<uint64_t>(h.lo) | (static_cast<uint64_t>(h.hi) << 32));
}

BW_API int bw_fingerprint_rows(const float* logits, int rows, int vocab, const int* slot,
                               unsigned long long* state, cudaStream_t stream) {
  if (rows <= 0) return 0;
  bw::launch_pdl(fingerprint_rows_kernel, dim3(rows), dim3(32), 0, stream, logits, rows, vocab, slot, state);
  return bw::launch_status();
}
