// The true 32-bit path: every kernel of the model in IEEE float32 with the reference's
// reduction orders, so that its results equal a plain fixed-order CPU implementation bit
// for bit, however the work is cut into steps and batches.
//
//   matrix product  one fused-multiply-add chain k = 0..K-1 per output   (src/kernels.cpp:236-244)
//   sum of squares / dot product   16 lane-wise chains, then a fixed tree (src/kernels.cpp:57-64,86-100)
//   attention       two passes over the keys in key order, global max     (src/kernels.cpp:312-338)
//
// No tensor cores here (tf32 is not float32). Explicit __f*_rn intrinsics keep the compiler
// from contracting or reassociating anything.
#include "bw_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// RMSNorm: ss = dot16(x, x); inv = 1 / sqrt(ss / width + eps); y = (x * inv) * w
// (src/kernels.cpp:264-271). One warp per output row; lanes 0..15 run the 16 chains.
constexpr int kNormWarps = 4;

__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_exact_kernel(const float* __restrict__ x, const float* __restrict__ w, float* y,
                     const int* __restrict__ rows, int n, int width, float eps) {
  const int r = blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  if (r >= n) return;
  const int lane = threadIdx.x & 31;
  const int src = rows ? rows[r] : r;
  const float* xr = x + static_cast<size_t>(src) * width;
  float* yr = y + static_cast<size_t>(r) * width;
  float acc = 0.0f;
  if (lane < 16) {
#pragma unroll 8
    for (int i = lane; i < width; i += 16) {
      const float v = xr[i];
      acc = __fmaf_rn(v, v, acc);
    }
  }
  acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8, 16));
  acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4, 16));
  acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2, 16));
  acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1, 16));
  const float ss = __shfl_sync(0xffffffffu, acc, 0);
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(width)), eps)));
  for (int i = lane; i < width; i += 32) yr[i] = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
}

// ---------------------------------------------------------------------------------------
// Matrix product y[m][n] = sum_k x[m][k] * W[n][k], one chain per output. Tiles only decide
// which outputs are computed side by side; zero padding past K adds fma(0, 0, acc) = acc.
constexpr int kGemmBN = 64;
constexpr int kGemmBK = 16;

template <int BM>
__global__ void __launch_bounds__(256)
gemm_exact_kernel(const float* __restrict__ X, const float* __restrict__ W, float* Y,
                  const float* residual, int M, int N, int K) {
  constexpr int TM = BM / 16;
  __shared__ float As[kGemmBK][BM + 1];
  __shared__ __align__(16) float Ws[kGemmBK][kGemmBN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * kGemmBN;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += kGemmBK) {
    // X tile: BM x 16
    if (BM == 64) {
      const int row = tid >> 2, kq = (tid & 3) * 4;
      const int gm = m0 + row;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gk = k0 + kq + i;
        As[kq + i][row] = (gm < M && gk < K) ? X[static_cast<size_t>(gm) * K + gk] : 0.0f;
      }
    } else {
      const int row = tid >> 4, kk = tid & 15;
      const int gm = m0 + row, gk = k0 + kk;
      if (row < BM) As[kk][row] = (gm < M && gk < K) ? X[static_cast<size_t>(gm) * K + gk] : 0.0f;
    }
    {  // W tile: 64 x 16
      const int row = tid >> 2, kq = (tid & 3) * 4;
      const int gn = n0 + row;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int gk = k0 + kq + i;
        Ws[kq + i][row] = (gn < N && gk < K) ? W[static_cast<size_t>(gn) * K + gk] : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kGemmBK; ++k) {
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const float a = As[k][ty * TM + i];
        acc[i][0] = __fmaf_rn(a, b.x, acc[i][0]);
        acc[i][1] = __fmaf_rn(a, b.y, acc[i][1]);
        acc[i][2] = __fmaf_rn(a, b.z, acc[i][2]);
        acc[i][3] = __fmaf_rn(a, b.w, acc[i][3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      const size_t o = static_cast<size_t>(gm) * N + gn;
      Y[o] = residual ? __fadd_rn(residual[o], acc[i][j]) : acc[i][j];
    }
  }
}

// ---------------------------------------------------------------------------------------
// The same product for large batches (prefill) whose rows start on 16 bytes: tiles of
// 128 x 128 outputs, a thread carries 8 x 8 of them (each still one chain, k ascending), so that
// four 16-byte reads from shared memory feed 64 multiply-adds; the next k-tile is fetched
// into registers while this one is used, and two buffers in shared memory leave one barrier
// per k-tile.
constexpr int kBigBM = 128, kBigBN = 128, kBigBK = 16;

__global__ void __launch_bounds__(256, 2)
gemm_exact_big_kernel(const float* __restrict__ X, const float* __restrict__ W, float* Y, const float* residual, int M,
                      int N, int K) {
  __shared__ __align__(16) float As[2][kBigBK][kBigBM + 4];
  __shared__ __align__(16) float Bs[2][kBigBK][kBigBN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // columns 4 tx .. + 3 and 64 + 4 tx .. + 3, rows 8 ty .. + 7
  const int m0 = blockIdx.y * kBigBM, n0 = blockIdx.x * kBigBN;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
  // a thread fetches two 16-byte pieces of x and two of W per k-tile: piece p = tid + 256 i is
  // row p / 4, k-quarter p % 4
  float4 xa[2], wb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int pc = tid + 256 * i, row = pc >> 2, gk = k0 + (pc & 3) * 4;
      const int gm = m0 + row, gn = n0 + row;
      xa[i] = (gm < M && gk < K) ? *reinterpret_cast<const float4*>(X + static_cast<size_t>(gm) * K + gk)
                                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // K is a multiple of 4
      wb[i] = (gn < N && gk < K) ? *reinterpret_cast<const float4*>(W + static_cast<size_t>(gn) * K + gk)
                                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int pc = tid + 256 * i, row = pc >> 2, kq = (pc & 3) * 4;
      As[buf][kq + 0][row] = xa[i].x, As[buf][kq + 1][row] = xa[i].y;
      As[buf][kq + 2][row] = xa[i].z, As[buf][kq + 3][row] = xa[i].w;
      Bs[buf][kq + 0][row] = wb[i].x, Bs[buf][kq + 1][row] = wb[i].y;
      Bs[buf][kq + 2][row] = wb[i].z, Bs[buf][kq + 3][row] = wb[i].w;
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  const int tiles = (K + kBigBK - 1) / kBigBK;
  for (int t = 0; t < tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < tiles) fetch((t + 1) * kBigBK);
#pragma unroll
    for (int k = 0; k < kBigBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 8 + 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    if (t + 1 < tiles) stash(buf ^ 1);  // nobody reads that buffer: its tile was used before the last barrier
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + ty * 8 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn >= N) continue;
      const size_t o = static_cast<size_t>(gm) * N + gn;
      Y[o] = residual ? __fadd_rn(residual[o], acc[i][j]) : acc[i][j];
    }
  }
}

// ---------------------------------------------------------------------------------------
// The same product for steps of few rows (decode steps, up to 16 rows), where the weights are
// all that is read: one chain per output as above (a thread carries two rows of one column,
// k ascending, fma after fma), but tiles of 16 columns, so that every SM streams weights (a
// product with 2,048 columns is 128 blocks instead of 32), and the tiles of W and x come
// through a ring of cp.async stages instead of a load, a barrier, the arithmetic and a
// barrier in turn. Shared memory holds a stage as [k / 4][column or row][4 values]: a lane's
// 16-byte read of its column meets no other lane's bank, the rows of x are broadcast.
constexpr int kRowsBN = 16;      // columns per block
constexpr int kRowsBK = 64;      // k per stage
constexpr int kRowsStages = 6;

__device__ __forceinline__ void cp_async16_f32(void* dst, const void* src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // 0: zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

template <int R>  // rows of the tile: 8 or 16
__global__ void __launch_bounds__(kRowsBN * R / 2)
gemm_exact_rows_kernel(const float* __restrict__ X, const float* __restrict__ W, float* Y, const float* residual, int M,
                       int N, int K) {
  constexpr int kThreads = kRowsBN * R / 2;
  __shared__ __align__(16) float Ws[kRowsStages][kRowsBK / 4][kRowsBN][4];
  __shared__ __align__(16) float Xs[kRowsStages][kRowsBK / 4][R][4];
  const int tid = threadIdx.x;
  const int col = tid % kRowsBN, rp = tid / kRowsBN;  // this thread's column and pair of rows
  const int n0 = blockIdx.x * kRowsBN;
  const int stages_total = (K + kRowsBK - 1) / kRowsBK;
  auto load_stage = [&](int st) {
    const int slot = st % kRowsStages, k0 = st * kRowsBK;
    for (int idx = tid; idx < kRowsBN * (kRowsBK / 4); idx += kThreads) {
      const int c = idx / (kRowsBK / 4), k4 = idx % (kRowsBK / 4);  // a thread walks k: 16 bytes after 16 bytes of a row
      const int gn = n0 + c, gk = k0 + k4 * 4;
      const bool ok = gn < N && gk < K;  // K is a multiple of 4
      cp_async16_f32(&Ws[slot][k4][c][0], W + (ok ? static_cast<size_t>(gn) * K + gk : 0), ok);
    }
    for (int idx = tid; idx < R * (kRowsBK / 4); idx += kThreads) {
      const int r = idx / (kRowsBK / 4), k4 = idx % (kRowsBK / 4);
      const int gk = k0 + k4 * 4;
      const bool ok = r < M && gk < K;
      cp_async16_f32(&Xs[slot][k4][r][0], X + (ok ? static_cast<size_t>(r) * K + gk : 0), ok);
    }
  };
  for (int st = 0; st < kRowsStages - 1; ++st) {
    if (st < stages_total) load_stage(st);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  float acc0 = 0.0f, acc1 = 0.0f;
  for (int st = 0; st < stages_total; ++st) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kRowsStages - 2));
    __syncthreads();  // stage st has landed for every thread; the slot of stage st - 1 is free
    if (st + kRowsStages - 1 < stages_total) load_stage(st + kRowsStages - 1);
    asm volatile("cp.async.commit_group;\n" ::);
    const int slot = st % kRowsStages;
#pragma unroll
    for (int k4 = 0; k4 < kRowsBK / 4; ++k4) {
      const float4 w = *reinterpret_cast<const float4*>(&Ws[slot][k4][col][0]);
      const float4 a = *reinterpret_cast<const float4*>(&Xs[slot][k4][2 * rp][0]);
      const float4 b = *reinterpret_cast<const float4*>(&Xs[slot][k4][2 * rp + 1][0]);
      acc0 = __fmaf_rn(a.x, w.x, acc0), acc1 = __fmaf_rn(b.x, w.x, acc1);
      acc0 = __fmaf_rn(a.y, w.y, acc0), acc1 = __fmaf_rn(b.y, w.y, acc1);
      acc0 = __fmaf_rn(a.z, w.z, acc0), acc1 = __fmaf_rn(b.z, w.z, acc1);
      acc0 = __fmaf_rn(a.w, w.w, acc0), acc1 = __fmaf_rn(b.w, w.w, acc1);
    }
  }
  const int gn = n0 + col;
  if (gn >= N) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int gm = 2 * rp + i;
    if (gm >= M) continue;
    const size_t o = static_cast<size_t>(gm) * N + gn;
    const float v = i ? acc1 : acc0;
    Y[o] = residual ? __fadd_rn(residual[o], v) : v;
  }
}

// ---------------------------------------------------------------------------------------
// Rotary encoding in the rotate-half pairing (i, i + hd/2) with separate roundings of the
// products (src/kernels.cpp:273-289), then the write of K and V into the paged cache
// (src/model.cpp:285-297). cos/sin come from a host-built table [position][hd/2]. Queries
// are rotated in place; the rotated key goes to the cache only.
__global__ void rope_cache_exact_kernel(float* qkv, int row_stride, const int* __restrict__ pos,
                                        const int* __restrict__ row_seq,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                        const int* __restrict__ block_table, int max_blocks,
                                        float* kcache, float* vcache, int heads, int kv_heads, int hd,
                                        int page, int write_kv) {
  const int r = blockIdx.x;
  const int half = hd >> 1;
  const int p = pos[r];
  float* row = qkv + static_cast<size_t>(r) * row_stride;
  const bool rotate = cos_t != nullptr;  // a null table leaves q and k as they are
  const float* c = rotate ? cos_t + static_cast<size_t>(p) * half : nullptr;
  const float* s = rotate ? sin_t + static_cast<size_t>(p) * half : nullptr;
  const int q_items = rotate ? heads * half : 0;
  for (int it = threadIdx.x; it < q_items; it += blockDim.x) {
    const int h = it / half, i = it - h * half;
    float* v = row + h * hd;
    const float x1 = v[i], x2 = v[i + half];
    v[i] = __fsub_rn(__fmul_rn(x1, c[i]), __fmul_rn(x2, s[i]));
    v[i + half] = __fadd_rn(__fmul_rn(x2, c[i]), __fmul_rn(x1, s[i]));
  }
  if (!write_kv) return;
  const int blk = block_table[static_cast<size_t>(row_seq[r]) * max_blocks + p / page];
  const int slot = p % page;
  const float* k = row + heads * hd;
  const float* vv = k + kv_heads * hd;
  const int k_items = kv_heads * half;
  for (int it = threadIdx.x; it < k_items; it += blockDim.x) {
    const int h = it / half, i = it - h * half;
    const size_t dst = ((static_cast<size_t>(blk) * kv_heads + h) * page + slot) * hd;
    const float x1 = k[h * hd + i], x2 = k[h * hd + i + half];
    kcache[dst + i] = rotate ? __fsub_rn(__fmul_rn(x1, c[i]), __fmul_rn(x2, s[i])) : x1;
    kcache[dst + i + half] = rotate ? __fadd_rn(__fmul_rn(x2, c[i]), __fmul_rn(x1, s[i])) : x2;
    vcache[dst + i] = vv[h * hd + i];
    vcache[dst + i + half] = vv[h * hd + i + half];
  }
}

// ---------------------------------------------------------------------------------------
// Attention over the cache, one block per (row, head): scores s_j = dot16(q, K_j) * scale
// with the global maximum, then in key order e_j = exp(s_j - max), sum += e_j,
// acc[d] = fma(e_j, V_j[d], acc[d]); finally o[d] = acc[d] * (1 / sum)
// (src/kernels.cpp:312-338,361-364). `window` > 0 limits the keys to the last `window`
// positions. Every thread carries the running sum itself, so all hold the same value.
constexpr int kAttnThreads = 128;
constexpr int kAttnTileKeys = 64;  // keys per tile of values in shared memory

template <bool STAGED>
__global__ void __launch_bounds__(kAttnThreads)
attention_exact_kernel(const float* __restrict__ qkv, int q_stride, const float* __restrict__ kcache,
                       const float* __restrict__ vcache, const int* __restrict__ block_table,
                       int max_blocks, const int* __restrict__ row_seq, const int* __restrict__ pos,
                       float* __restrict__ out, int out_stride, int heads, int kv_heads, int hd, int page,
                       int window, float scale, int score_floats) {
  extern __shared__ __align__(16) float smem[];
  float* q = smem;          // [hd]
  float* scores = smem + hd;  // [len]
  __shared__ float red[kAttnThreads / 32];
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int p = pos[r];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int len = p - lo + 1;
  const int g = h / (heads / kv_heads);
  const int* table = block_table + static_cast<size_t>(row_seq[r]) * max_blocks;
  const float* qg = qkv + static_cast<size_t>(r) * q_stride + h * hd;
  for (int i = tid; i < hd; i += kAttnThreads) q[i] = qg[i];
  __syncthreads();

  float mx = -INFINITY;
  for (int j = lo + tid; j <= p; j += kAttnThreads) {
    const float* kp = kcache + ((static_cast<size_t>(table[j / page]) * kv_heads + g) * page + j % page) * hd;
    float lane[16];
#pragma unroll
    for (int l = 0; l < 16; ++l) lane[l] = 0.0f;
    for (int i = 0; i < hd; i += 16) {
      const float4* k4 = reinterpret_cast<const float4*>(kp + i);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const float4 kk = k4[v];
        lane[4 * v + 0] = __fmaf_rn(q[i + 4 * v + 0], kk.x, lane[4 * v + 0]);
        lane[4 * v + 1] = __fmaf_rn(q[i + 4 * v + 1], kk.y, lane[4 * v + 1]);
        lane[4 * v + 2] = __fmaf_rn(q[i + 4 * v + 2], kk.z, lane[4 * v + 2]);
        lane[4 * v + 3] = __fmaf_rn(q[i + 4 * v + 3], kk.w, lane[4 * v + 3]);
      }
    }
    const float s = __fmul_rn(bw::tree16(lane), scale);
    scores[j - lo] = s;
    mx = fmaxf(mx, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < kAttnThreads / 32; ++w) mx = fmaxf(mx, red[w]);
  for (int j = tid; j < len; j += kAttnThreads) scores[j] = bw::det_expf(__fsub_rn(scores[j], mx));
  __syncthreads();

  // Second pass, in key order: thread d walks the keys for output element d: sum += e,
  // acc = fma(e, v, acc). With many blocks (prefill) it reads the values straight from the
  // cache: other blocks hide the latency of its loads.
  if (!STAGED) {
    for (int d = tid; d < hd; d += kAttnThreads) {
      float acc = 0.0f, sum = 0.0f;
      int j = lo;
      while (j <= p) {
        const int b = j / page;
        const int first = j - b * page;
        const int last = (p - b * page < page - 1) ? p - b * page : page - 1;
        const float* vp = vcache + ((static_cast<size_t>(table[b]) * kv_heads + g) * page) * hd + d;
#pragma unroll 4
        for (int s = first; s <= last; ++s) {
          const float e = scores[j - lo + (s - first)];
          sum = __fadd_rn(sum, e);
          acc = __fmaf_rn(e, vp[static_cast<size_t>(s) * hd], acc);
        }
        j += last - first + 1;
      }
      out[static_cast<size_t>(r) * out_stride + h * hd + d] = __fmul_rn(acc, __fdiv_rn(1.0f, sum));
    }
    return;
  }
  // With few blocks (decode steps) a walk through the cache is a chain of load latencies. The
  // values then come through shared memory in tiles of 64 keys that all threads fetch
  // together (cp.async, the next tile on its way while this one is used); the same operations
  // in the same order.
  float* vt = scores + score_floats;  // [2][kAttnTileKeys][hd]
  constexpr int kMaxD = 256 / kAttnThreads;  // output elements per thread (head sizes up to 256)
  float acc[kMaxD], sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxD; ++i) acc[i] = 0.0f;
  const int tiles = (len + kAttnTileKeys - 1) / kAttnTileKeys;
  const int pieces = hd / 4;  // 16-byte pieces of a value row
  auto fetch = [&](int t) {
    float* dst = vt + (t & 1) * kAttnTileKeys * hd;
    for (int idx = tid; idx < kAttnTileKeys * pieces; idx += kAttnThreads) {
      const int key = idx / pieces, piece = idx - key * pieces;
      const int j = lo + t * kAttnTileKeys + key;
      const bool ok = j <= p;
      const float* src = vcache;
      if (ok) src += ((static_cast<size_t>(table[j / page]) * kv_heads + g) * page + j % page) * hd + piece * 4;
      const unsigned d32 = static_cast<unsigned>(__cvta_generic_to_shared(dst + key * hd + piece * 4));
      const int bytes = ok ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d32), "l"(src), "r"(bytes));
    }
  };
  fetch(0);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int t = 0; t < tiles; ++t) {
    if (t + 1 < tiles) fetch(t + 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const float* v = vt + (t & 1) * kAttnTileKeys * hd;
    const int keys = min(kAttnTileKeys, len - t * kAttnTileKeys);
    const float* e_t = scores + t * kAttnTileKeys;
#pragma unroll 8
    for (int s2 = 0; s2 < keys; ++s2) {
      const float e = e_t[s2];
      sum = __fadd_rn(sum, e);
#pragma unroll
      for (int i = 0; i < kMaxD; ++i) {
        const int d = tid + i * kAttnThreads;
        if (d < hd) acc[i] = __fmaf_rn(e, v[s2 * hd + d], acc[i]);
      }
    }
    __syncthreads();  // the tile may be overwritten by the fetch after next
  }
  const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
  for (int i = 0; i < kMaxD; ++i) {
    const int d = tid + i * kAttnThreads;
    if (d < hd) out[static_cast<size_t>(r) * out_stride + h * hd + d] = __fmul_rn(acc[i], inv);
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU on rows laid out [gate | up]: h = (g * (1 / (1 + exp(-g)))) * u (src/kernels.cpp:291-298).
__global__ void swiglu_exact_kernel(const float* __restrict__ gate_up, float* __restrict__ out, int n, int inter) {
  const size_t total = static_cast<size_t>(n) * inter;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = idx / inter;
    const int i = static_cast<int>(idx - r * inter);
    const float g = gate_up[r * 2 * inter + i];
    const float u = gate_up[r * 2 * inter + inter + i];
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, bw::det_expf(-g)));
    out[idx] = __fmul_rn(__fmul_rn(g, sig), u);
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Exported entry points.

BW_API int bw_f32_rmsnorm(const float* x, const float* weight, float* y, const int* rows, int n, int width,
                          float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) {
    bw::set_error("rmsnorm: width %d", width);
    return -1;
  }
  rmsnorm_exact_kernel<<<(n + kNormWarps - 1) / kNormWarps, kNormWarps * 32, 0, stream>>>(x, weight, y, rows, n,
                                                                                          width, eps);
  return bw::launch_status();
}

BW_API int bw_f32_linear(const float* x, const float* w, float* y, const float* residual, int m, int n, int k,
                         cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0) {
    bw::set_error("linear: inner size %d", k);
    return -1;
  }
  const unsigned gx = (n + kGemmBN - 1) / kGemmBN;
  if (m <= 16 && k % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    const unsigned blocks = (n + kRowsBN - 1) / kRowsBN;  // rows that start on 16 bytes: the streaming tile
    if (m <= 8)
      gemm_exact_rows_kernel<8><<<blocks, kRowsBN * 4, 0, stream>>>(x, w, y, residual, m, n, k);
    else
      gemm_exact_rows_kernel<16><<<blocks, kRowsBN * 8, 0, stream>>>(x, w, y, residual, m, n, k);
  } else if (m <= 16) {
    gemm_exact_kernel<16><<<dim3(gx, (m + 15) / 16), 256, 0, stream>>>(x, w, y, residual, m, n, k);
  } else if (m > 64 && k % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    const unsigned gy = (m + kBigBM - 1) / kBigBM;
    if (gy > 65535u) {
      bw::set_error("linear: %d rows exceed the grid limit", m);
      return -1;
    }
    gemm_exact_big_kernel<<<dim3((n + kBigBN - 1) / kBigBN, gy), 256, 0, stream>>>(x, w, y, residual, m, n, k);
  } else {
    const unsigned gy = (m + 63) / 64;
    if (gy > 65535u) {
      bw::set_error("linear: %d rows exceed the grid limit", m);
      return -1;
    }
    gemm_exact_kernel<64><<<dim3(gx, gy), 256, 0, stream>>>(x, w, y, residual, m, n, k);
  }
  return bw::launch_status();
}

BW_API int bw_f32_rope_cache(float* qkv, int row_stride, const int* pos, const int* row_seq, const float* cos_t,
                             const float* sin_t, const int* block_table, int max_blocks, float* kcache,
                             float* vcache, int n, int heads, int kv_heads, int hd, int page, int write_kv,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd % 2) {
    bw::set_error("rope: head size %d is odd", hd);
    return -1;
  }
  rope_cache_exact_kernel<<<n, 128, 0, stream>>>(qkv, row_stride, pos, row_seq, cos_t, sin_t, block_table,
                                                 max_blocks, kcache, vcache, heads, kv_heads, hd, page, write_kv);
  return bw::launch_status();
}

BW_API int bw_f32_attention(const float* qkv, int q_stride, const float* kcache, const float* vcache,
                            const int* block_table, int max_blocks, const int* row_seq, const int* pos,
                            float* out, int out_stride, int n, int heads, int kv_heads, int hd, int page,
                            int window, int max_keys, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd % 16 || hd <= 0) {
    bw::set_error("attention: head size %d is not a multiple of 16", hd);
    return -1;
  }
  if (heads % kv_heads) {
    bw::set_error("attention: %d heads are not a multiple of %d key/value heads", heads, kv_heads);
    return -1;
  }
  if (hd > 256) {
    bw::set_error("attention (32-bit): head size %d exceeds 256", hd);
    return -1;
  }
  const int score_floats = (max_keys + 3) / 4 * 4;  // keeps the value tiles behind the scores on 16 bytes
  const bool staged = static_cast<long long>(n) * heads <= 148 * 16;  // few blocks: a decode step
  const size_t smem = (static_cast<size_t>(hd) + score_floats + (staged ? 2 * kAttnTileKeys * hd : 0)) * sizeof(float);
  if (smem > 220 * 1024) {
    bw::set_error("attention (32-bit): %d keys exceed the shared-memory score buffer", max_keys);
    return -1;
  }
  if (heads > 65535) {
    bw::set_error("attention: %d heads exceed the grid limit", heads);
    return -1;
  }
  static bool configured = false;
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_exact_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         220 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_exact_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) {
      bw::set_error("attention: cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  if (staged)
    attention_exact_kernel<true><<<dim3(n, heads), kAttnThreads, smem, stream>>>(
        qkv, q_stride, kcache, vcache, block_table, max_blocks, row_seq, pos, out, out_stride, heads, kv_heads, hd,
        page, window, scale, score_floats);
  else
    attention_exact_kernel<false><<<dim3(n, heads), kAttnThreads, smem, stream>>>(
        qkv, q_stride, kcache, vcache, block_table, max_blocks, row_seq, pos, out, out_stride, heads, kv_heads, hd,
        page, window, scale, score_floats);
  return bw::launch_status();
}

BW_API int bw_f32_swiglu(const float* gate_up, float* out, int n, int inter, cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  const size_t total = static_cast<size_t>(n) * inter;
  const unsigned blocks = static_cast<unsigned>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  swiglu_exact_kernel<<<blocks, 256, 0, stream>>>(gate_up, out, n, inter);
  return bw::launch_status();
}
