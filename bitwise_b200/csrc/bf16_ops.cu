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
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + static_cast<size_t>(src) * width;
  __nv_bfloat16* yr = y + static_cast<size_t>(r) * width;
  __shared__ float red[kNormThreads / 32];
  // A thread's elements are threadIdx.x, + kNormThreads, ...: eight of them (a row of 2,048 in one
  // go) are asked for before the first is used, and the weights with them, so that a row costs one
  // round trip to memory instead of one per element. The sums keep their order.
  constexpr int kBatch = 8;
  float acc = 0.0f;
  float v[kBatch], g[kBatch];
  const bool one_go = width <= kBatch * kNormThreads;
  for (int base = 0; base < width; base += kBatch * kNormThreads) {
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = base + threadIdx.x + j * kNormThreads;
      v[j] = i < width ? xr[i] : 0.0f;
      if (one_go) g[j] = i < width ? w[i] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (base + threadIdx.x + j * kNormThreads < width) acc = __fmaf_rn(v[j], v[j], acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) ss = __fadd_rn(ss, red[i]);
  const float inv = bw::rms_scale(ss, width, eps);
  if (one_go) {
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = threadIdx.x + j * kNormThreads;
      if (i < width) yr[i] = __float2bfloat16_rn(bw::rms_apply(v[j], inv, g[j]));
    }
  } else {
    for (int i = threadIdx.x; i < width; i += kNormThreads) yr[i] = __float2bfloat16_rn(bw::rms_apply(xr[i], inv, w[i]));
  }
}

// ---------------------------------------------------------------------------------------
// Rotary encoding (rotate-half pairs, src/kernels.cpp:273-289) in float32 on bfloat16
// values, rounded once; then K and V of the row go into the paged cache
// (src/model.cpp:285-297). With a null table nothing is rotated. One thread per 8 pairs
// (16-byte accesses): blockIdx.x is the row, blockIdx.y * blockDim.x + threadIdx.x the item,
// first the items of the query heads, then those of the key heads (which also carry the
// values). The head size is a multiple of 16, so half a head is a whole number of items.
__device__ __forceinline__ void rotate8(const uint4& a, const uint4& b, const float* c, const float* s, uint4& ra,
                                        uint4& rb) {
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
  __nv_bfloat162* oa = reinterpret_cast<__nv_bfloat162*>(&ra);
  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 x1 = __bfloat1622float2(a2[e]), x2 = __bfloat1622float2(b2[e]);
    const float c0 = c[2 * e], c1 = c[2 * e + 1], s0 = s[2 * e], s1 = s[2 * e + 1];
    oa[e] = __floats2bfloat162_rn(__fsub_rn(__fmul_rn(x1.x, c0), __fmul_rn(x2.x, s0)),
                                  __fsub_rn(__fmul_rn(x1.y, c1), __fmul_rn(x2.y, s1)));
    ob[e] = __floats2bfloat162_rn(__fadd_rn(__fmul_rn(x2.x, c0), __fmul_rn(x1.x, s0)),
                                  __fadd_rn(__fmul_rn(x2.y, c1), __fmul_rn(x1.y, s1)));
  }
}

__global__ void rope_cache_bf16_kernel(__nv_bfloat16* qkv, int row_stride, const int* __restrict__ pos,
                                       const int* __restrict__ row_seq, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int* __restrict__ block_table,
                                       int max_blocks, __nv_bfloat16* kcache, __nv_bfloat16* vcache, int heads,
                                       int kv_heads, int hd, int page, int write_kv) {
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int half = hd >> 1, per_head = half >> 3;  // items of 8 pairs per head
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int q_items = heads * per_head, k_items = write_kv ? kv_heads * per_head : 0;
  if (item >= q_items + k_items) return;
  const int p = pos[r];
  __nv_bfloat16* row = qkv + static_cast<size_t>(r) * row_stride;
  const bool is_q = item < q_items;
  const int local = is_q ? item : item - q_items;
  const int h = local / per_head, i = (local - h * per_head) * 8;
  float c[8], s[8];
  if (cos_t) {
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(p) * half + i);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(p) * half + i);
    *reinterpret_cast<float4*>(c) = c4[0], *reinterpret_cast<float4*>(c + 4) = c4[1];
    *reinterpret_cast<float4*>(s) = s4[0], *reinterpret_cast<float4*>(s + 4) = s4[1];
  }
  if (is_q) {
    if (!cos_t) return;
    __nv_bfloat16* v = row + h * hd + i;
    const uint4 a = *reinterpret_cast<const uint4*>(v), b = *reinterpret_cast<const uint4*>(v + half);
    uint4 ra, rb;
    rotate8(a, b, c, s, ra, rb);
    *reinterpret_cast<uint4*>(v) = ra;
    *reinterpret_cast<uint4*>(v + half) = rb;
    return;
  }
  const int blk = block_table[static_cast<size_t>(row_seq[r]) * max_blocks + p / page];
  const int slot = p % page;
  const __nv_bfloat16* k = row + heads * hd + h * hd + i;
  const __nv_bfloat16* vv = k + kv_heads * hd;
  const size_t dst = ((static_cast<size_t>(blk) * kv_heads + h) * page + slot) * hd + i;
  uint4 a = *reinterpret_cast<const uint4*>(k), b = *reinterpret_cast<const uint4*>(k + half);
  if (cos_t) {
    uint4 ra, rb;
    rotate8(a, b, c, s, ra, rb);
    a = ra, b = rb;
  }
  *reinterpret_cast<uint4*>(kcache + dst) = a;
  *reinterpret_cast<uint4*>(kcache + dst + half) = b;
  *reinterpret_cast<uint4*>(vcache + dst) = *reinterpret_cast<const uint4*>(vv);
  *reinterpret_cast<uint4*>(vcache + dst + half) = *reinterpret_cast<const uint4*>(vv + half);
}

// ---------------------------------------------------------------------------------------
// SwiGLU on rows laid out [gate | up]: h = (g * sigmoid(g)) * u in float32 (src/kernels.cpp:291-298).
// blockIdx.y is the row; a thread handles 8 consecutive columns when the row width allows
// 16-byte accesses, else one column.
using bw::swiglu_one;

__global__ void swiglu_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int inter) {
  bw::pdl_enter();
  const int r = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= inter) return;
  const __nv_bfloat16* g = gate_up + static_cast<size_t>(r) * 2 * inter + c;
  const uint4 gv = *reinterpret_cast<const uint4*>(g);
  const uint4 uv = *reinterpret_cast<const uint4*>(g + inter);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
  __align__(16) __nv_bfloat162 o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 gf = __bfloat1622float2(g2[e]), uf = __bfloat1622float2(u2[e]);
    o[e] = __floats2bfloat162_rn(swiglu_one(gf.x, uf.x), swiglu_one(gf.y, uf.y));
  }
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * inter + c) = *reinterpret_cast<const uint4*>(o);
}

__global__ void swiglu_bf16_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                   int inter) {
  bw::pdl_enter();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= inter) return;
  const __nv_bfloat16* g = gate_up + static_cast<size_t>(r) * 2 * inter + c;
  out[static_cast<size_t>(r) * inter + c] =
      __float2bfloat16_rn(swiglu_one(__bfloat162float(g[0]), __bfloat162float(g[inter])));
}

}  // namespace

BW_API int bw_bf16_rmsnorm(const float* x, const float* weight, __nv_bfloat16* y, const int* rows, int n,
                           int width, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) {
    bw::set_error("rmsnorm: width %d", width);
    return -1;
  }
  bw::launch_pdl(rmsnorm_bf16_kernel, dim3(n), dim3(kNormThreads), 0, stream, x, weight, y, rows, width, eps);
  return bw::launch_status();
}

BW_API int bw_bf16_rope_cache(__nv_bfloat16* qkv, int row_stride, const int* pos, const int* row_seq,
                              const float* cos_t, const float* sin_t, const int* block_table, int max_blocks,
                              __nv_bfloat16* kcache, __nv_bfloat16* vcache, int n, int heads, int kv_heads, int hd,
                              int page, int write_kv, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd % 16 || row_stride % 8) {
    bw::set_error("rope: head size %d must be a multiple of 16 and the row stride %d of 8", hd, row_stride);
    return -1;
  }
  const int items = (heads + (write_kv ? kv_heads : 0)) * (hd / 16);
  const int threads = items >= 128 ? 128 : 64;
  dim3 grid(n, (items + threads - 1) / threads);
  if (grid.y > 65535u) {
    bw::set_error("rope: %d heads exceed the grid limit", heads);
    return -1;
  }
  bw::launch_pdl(rope_cache_bf16_kernel, dim3(grid), dim3(threads), 0, stream, qkv, row_stride, pos, row_seq, cos_t, sin_t, block_table,
                                                       max_blocks, kcache, vcache, heads, kv_heads, hd, page, write_kv);
  return bw::launch_status();
}

BW_API int bw_bf16_swiglu(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int n, int inter, cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  if (n > 65535) {  // rows ride on blockIdx.y; split very tall inputs
    for (int r = 0; r < n; r += 65535) {
      const int cnt = n - r < 65535 ? n - r : 65535;
      const int rc = bw_bf16_swiglu(gate_up + static_cast<size_t>(r) * 2 * inter, out + static_cast<size_t>(r) * inter,
                                    cnt, inter, stream);
      if (rc) return rc;
    }
    return 0;
  }
  const bool vec = inter % 8 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0;
  if (vec) {
    const int threads = 128;
    dim3 grid((inter / 8 + threads - 1) / threads, n);
    bw::launch_pdl(swiglu_bf16_vec_kernel, dim3(grid), dim3(threads), 0, stream, gate_up, out, inter);
  } else {
    const int threads = 256;
    dim3 grid((inter + threads - 1) / threads, n);
    bw::launch_pdl(swiglu_bf16_kernel, dim3(grid), dim3(threads), 0, stream, gate_up, out, inter);
  }
  return bw::launch_status();
}
