// Serving-path kernels around the matrix products: RMSNorm (32-bit statistic, bfloat16
// out), rotary encoding with the cache write, SwiGLU. Activations between kernels are
// bfloat16; the residual stream and every reduction are float32. Each output depends on
// its own row only, and its reduction order is fixed by the row width, never by the batch.
#include "bw_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// RMSNorm: y = (x * inv) * w, inv = 1 / sqrt(mean(x^2) + eps) (src/kernels.cpp:264-271),
// one block per output row. Thread t sums elements t, t + T, ... in order; the partial sums
// are combined by a fixed shuffle tree and then across warps in warp order.
constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bf16_kernel(const float* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                    const int* __restrict__ rows, int width, float eps) {
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + static_cast<size_t>(src) * width;
  __nv_bfloat16* yr = y + static_cast<size_t>(r) * width;
  __shared__ float red[kNormThreads / 32];
  float acc = 0.0f;
  for (int i = threadIdx.x; i < width; i += kNormThreads) {
    const float v = xr[i];
    acc = fmaf(v, v, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) ss += red[i];
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int i = threadIdx.x; i < width; i += kNormThreads) yr[i] = __float2bfloat16_rn((xr[i] * inv) * w[i]);
}

// ---------------------------------------------------------------------------------------
// Rotary encoding (rotate-half pairs, src/kernels.cpp:273-289) in float32 on bfloat16
// values, rounded once; then K and V of the row go into the paged cache
// (src/model.cpp:285-297). With a null table nothing is rotated.
__global__ void rope_cache_bf16_kernel(__nv_bfloat16* qkv, int row_stride, const int* __restrict__ pos,
                                       const int* __restrict__ row_seq, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int* __restrict__ block_table,
                                       int max_blocks, __nv_bfloat16* kcache, __nv_bfloat16* vcache, int heads,
                                       int kv_heads, int hd, int page, int write_kv) {
  const int r = blockIdx.x;
  const int half = hd >> 1;
  const int p = pos[r];
  __nv_bfloat16* row = qkv + static_cast<size_t>(r) * row_stride;
  const float* c = cos_t ? cos_t + static_cast<size_t>(p) * half : nullptr;
  const float* s = sin_t ? sin_t + static_cast<size_t>(p) * half : nullptr;
  if (c) {
    const int q_items = heads * half;
    for (int it = threadIdx.x; it < q_items; it += blockDim.x) {
      const int h = it / half, i = it - h * half;
      __nv_bfloat16* v = row + h * hd;
      const float x1 = __bfloat162float(v[i]), x2 = __bfloat162float(v[i + half]);
      v[i] = __float2bfloat16_rn(x1 * c[i] - x2 * s[i]);
      v[i + half] = __float2bfloat16_rn(x2 * c[i] + x1 * s[i]);
    }
  }
  if (!write_kv) return;
  const int blk = block_table[static_cast<size_t>(row_seq[r]) * max_blocks + p / page];
  const int slot = p % page;
  const __nv_bfloat16* k = row + heads * hd;
  const __nv_bfloat16* vv = k + kv_heads * hd;
  const int k_items = kv_heads * half;
  for (int it = threadIdx.x; it < k_items; it += blockDim.x) {
    const int h = it / half, i = it - h * half;
    const size_t dst = ((static_cast<size_t>(blk) * kv_heads + h) * page + slot) * hd;
    const float x1 = __bfloat162float(k[h * hd + i]), x2 = __bfloat162float(k[h * hd + i + half]);
    if (c) {
      kcache[dst + i] = __float2bfloat16_rn(x1 * c[i] - x2 * s[i]);
      kcache[dst + i + half] = __float2bfloat16_rn(x2 * c[i] + x1 * s[i]);
    } else {
      kcache[dst + i] = k[h * hd + i];
      kcache[dst + i + half] = k[h * hd + i + half];
    }
    vcache[dst + i] = vv[h * hd + i];
    vcache[dst + i + half] = vv[h * hd + i + half];
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU on rows laid out [gate | up]: h = (g * sigmoid(g)) * u in float32 (src/kernels.cpp:291-298).
__global__ void swiglu_bf16_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                   int n, int inter) {
  const size_t total = static_cast<size_t>(n) * inter;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / inter;
    const int i = static_cast<int>(idx - r * inter);
    const float g = __bfloat162float(gate_up[r * 2 * inter + i]);
    const float u = __bfloat162float(gate_up[r * 2 * inter + inter + i]);
    const float sig = 1.0f / (1.0f + bw::det_expf(-g));
    out[idx] = __float2bfloat16_rn((g * sig) * u);
  }
}

}  // namespace

BW_API int bw_bf16_rmsnorm(const float* x, const float* weight, __nv_bfloat16* y, const int* rows, int n,
                           int width, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) {
    bw::set_error("rmsnorm: width %d", width);
    return -1;
  }
  rmsnorm_bf16_kernel<<<n, kNormThreads, 0, stream>>>(x, weight, y, rows, width, eps);
  return bw::launch_status();
}

BW_API int bw_bf16_rope_cache(__nv_bfloat16* qkv, int row_stride, const int* pos, const int* row_seq,
                              const float* cos_t, const float* sin_t, const int* block_table, int max_blocks,
                              __nv_bfloat16* kcache, __nv_bfloat16* vcache, int n, int heads, int kv_heads, int hd,
                              int page, int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd % 2) {
    bw::set_error("rope: head size %d is odd", hd);
    return -1;
  }
  rope_cache_bf16_kernel<<<n, 128, 0, stream>>>(qkv, row_stride, pos, row_seq, cos_t, sin_t, block_table, max_blocks,
                                                kcache, vcache, heads, kv_heads, hd, page, write_kv);
  return bw::launch_status();
}

BW_API int bw_bf16_swiglu(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int n, int inter, cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  const size_t total = static_cast<size_t>(n) * inter;
  const unsigned blocks = static_cast<unsigned>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  swiglu_bf16_kernel<<<blocks, 256, 0, stream>>>(gate_up, out, n, inter);
  return bw::launch_status();
}
