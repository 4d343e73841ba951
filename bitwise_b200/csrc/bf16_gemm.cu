// bfloat16 matrix product y[m][n] = sum_k x[m][k] * W[n][k] (+ residual) with float32
// accumulation, for every projection of the model (the reference's hand-written matmul,
// src/kernels.cpp:196-259, is its counterpart).
//
// One summation order for every shape. The inner dimension is cut into chunks of 2048
// elements at fixed positions. Inside a chunk the products are accumulated by the tensor
// core in steps of 16 along k, ascending. The chunk sums are added in float32 in ascending
// chunk order, p0, then + p1, then + p2 ..., and the residual last. A large batch walks the
// chunks inside one thread block; a small batch gives every chunk to a thread block of its
// own (so that a product with few output columns still fills the machine) and the block
// that finishes last adds the stored chunk sums in the same order. Either way a given row
// gets the same bits whatever else is in the batch and however the prompt was cut, the way
// the reference's one-chain-per-output rule does for its CPU kernels (src/kernels.h:4-12).
#include "bw_common.cuh"

namespace {

constexpr int BK = 64;        // k elements per shared-memory tile (128 bytes per row)
constexpr int kChunk = 512;   // canonical summation chunk along k
constexpr int kTilesPerChunk = kChunk / BK;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of the 16-byte piece `piece` (0..7) of row `row` in a [rows][64] bf16 tile,
// xor-swizzled so that eight consecutive rows of one piece fall into distinct banks
__device__ __forceinline__ uint32_t tile_offset(int row, int piece) {
  return static_cast<uint32_t>(row * 128 + ((piece ^ (row & 7)) << 4));
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool SPLIT>
__global__ void __launch_bounds__(WARPS_M * WARPS_N * 32)
gemm_bf16_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, void* Y, int y_is_f32,
                 const float* residual, int M, int N, int K, int aligned, float* partials, int* counters) {
  bw::pdl_enter();
  constexpr int THREADS = WARPS_M * WARPS_N * 32;
  constexpr int WTM = BM / WARPS_M, WTN = BN / WARPS_N;
  constexpr int MI = WTM / 16, NI = WTN / 8;
  static_assert(NI % 2 == 0, "warp tile must hold pairs of 8-column blocks");
  constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warp_m = warp / WARPS_N, warp_n = warp % WARPS_N;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int num_chunks = (K + kChunk - 1) / kChunk;
  const int chunk_first = SPLIT ? static_cast<int>(blockIdx.z) : 0;
  const int chunk_last = SPLIT ? chunk_first : num_chunks - 1;
  const int k_begin = chunk_first * kChunk;
  const int k_end = min(K, (chunk_last + 1) * kChunk);
  const int ntiles = (k_end - k_begin + BK - 1) / BK;

  float total[MI][NI][4];
  float part[MI][NI][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) total[i][j][e] = part[i][j][e] = 0.0f;

  auto load_tile = [&](int stage, int kt) {
    unsigned char* sa = smem + stage * STAGE_BYTES;
    unsigned char* sb = sa + A_BYTES;
    const int k0 = k_begin + kt * BK;
    if (aligned) {
      for (int idx = tid; idx < BM * 8; idx += THREADS) {
        const int row = idx >> 3, piece = idx & 7;
        const int gm = m0 + row, gk = k0 + piece * 8;
        const bool ok = gm < M && gk < k_end;
        cp_async16(smem_u32(sa + tile_offset(row, piece)), X + (ok ? static_cast<size_t>(gm) * K + gk : 0), ok);
      }
      for (int idx = tid; idx < BN * 8; idx += THREADS) {
        const int row = idx >> 3, piece = idx & 7;
        const int gn = n0 + row, gk = k0 + piece * 8;
        const bool ok = gn < N && gk < k_end;
        cp_async16(smem_u32(sb + tile_offset(row, piece)), W + (ok ? static_cast<size_t>(gn) * K + gk : 0), ok);
      }
    } else {  // rows that do not start on 16 bytes: element loads with bounds checks
      for (int idx = tid; idx < (BM + BN) * 8; idx += THREADS) {
        const bool is_a = idx < BM * 8;
        const int li = is_a ? idx : idx - BM * 8;
        const int row = li >> 3, piece = li & 7;
        const int g = (is_a ? m0 : n0) + row;
        const bool row_ok = is_a ? g < M : g < N;
        const __nv_bfloat16* src = (is_a ? X : W) + static_cast<size_t>(row_ok ? g : 0) * K;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int gk = k0 + piece * 8 + e;
          v[e] = (row_ok && gk < k_end) ? src[gk] : __float2bfloat16_rn(0.0f);
        }
        *reinterpret_cast<uint4*>((is_a ? sa : sb) + tile_offset(row, piece)) = *reinterpret_cast<const uint4*>(v);
      }
    }
  };

  auto compute_tile = [&](int stage) {
    const unsigned char* sa = smem + stage * STAGE_BYTES;
    const unsigned char* sb = sa + A_BYTES;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t a[MI][4];
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const int row = warp_m * WTM + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int piece = kk * 2 + (lane >> 4);
        ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3], smem_u32(sa + tile_offset(row, piece)));
      }
#pragma unroll
      for (int jp = 0; jp < NI / 2; ++jp) {
        uint32_t b[4];
        const int row = warp_n * WTN + jp * 16 + (lane & 7) + (lane >> 4) * 8;
        const int piece = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b[0], b[1], b[2], b[3], smem_u32(sb + tile_offset(row, piece)));
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          mma_bf16(part[i][2 * jp], a[i], b[0], b[1]);
          mma_bf16(part[i][2 * jp + 1], a[i], b[2], b[3]);
        }
      }
    }
  };

  auto close_chunk = [&](bool first) {
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          total[i][j][e] = first ? part[i][j][e] : total[i][j][e] + part[i][j][e];
          part[i][j][e] = 0.0f;
        }
  };

  if (aligned) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s < ntiles) load_tile(s, s);
      cp_async_commit();
    }
    for (int kt = 0; kt < ntiles; ++kt) {
      cp_async_wait<STAGES - 2>();
      __syncthreads();
      const int nxt = kt + STAGES - 1;
      if (nxt < ntiles) load_tile(nxt % STAGES, nxt);
      cp_async_commit();
      compute_tile(kt % STAGES);
      if ((kt + 1) % kTilesPerChunk == 0 || kt + 1 == ntiles) close_chunk(kt < kTilesPerChunk);
    }
    cp_async_wait<0>();
  } else {
    for (int kt = 0; kt < ntiles; ++kt) {
      __syncthreads();
      load_tile(0, kt);
      __syncthreads();
      compute_tile(0);
      if ((kt + 1) % kTilesPerChunk == 0 || kt + 1 == ntiles) close_chunk(kt < kTilesPerChunk);
    }
  }

  // ---- epilogue -------------------------------------------------------------------------
  const int row_base = m0 + warp_m * WTM + (lane >> 2);
  const int col_base = n0 + warp_n * WTN + 2 * (lane & 3);
  auto store_out = [&](int gm, int gn, float v) {
    const size_t o = static_cast<size_t>(gm) * N + gn;
    if (residual) v = residual[o] + v;
    if (y_is_f32)
      static_cast<float*>(Y)[o] = v;
    else
      static_cast<__nv_bfloat16*>(Y)[o] = __float2bfloat16_rn(v);
  };

  if (!SPLIT || num_chunks == 1) {
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gm = row_base + i * 16 + (e >> 1) * 8;
          const int gn = col_base + j * 8 + (e & 1);
          if (gm < M && gn < N) store_out(gm, gn, total[i][j][e]);
        }
    return;
  }

  // one chunk per block: store the chunk sum, the last block of this output tile adds them
  {
    float* mine = partials + static_cast<size_t>(blockIdx.z) * M * N;
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gm = row_base + i * 16 + (e >> 1) * 8;
          const int gn = col_base + j * 8 + (e & 1);
          if (gm < M && gn < N) __stcg(mine + static_cast<size_t>(gm) * N + gn, total[i][j][e]);
        }
  }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
  if (tid == 0) {
    const int seen = atomicAdd(&counters[tile_id], 1);
    s_last = (seen == num_chunks - 1);
    if (s_last) counters[tile_id] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int rows_here = min(BM, M - m0), cols_here = min(BN, N - n0);
  for (int idx = tid; idx < rows_here * cols_here; idx += THREADS) {
    const int gm = m0 + idx / cols_here, gn = n0 + idx % cols_here;
    const size_t o = static_cast<size_t>(gm) * N + gn;
    float v = __ldcg(partials + o);
    for (int c = 1; c < num_chunks; ++c) v = v + __ldcg(partials + static_cast<size_t>(c) * M * N + o);
    store_out(gm, gn, v);
  }
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool SPLIT>
int launch(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32, const float* residual, int m,
           int n, int k, float* partials, int* counters, cudaStream_t stream) {
  constexpr int THREADS = WARPS_M * WARPS_N * 32;
  const int aligned = (k % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  const int stages = aligned ? STAGES : 1;
  const size_t smem = static_cast<size_t>(stages) * (BM + BN) * 128;
  auto kernel = gemm_bf16_kernel<BM, BN, WARPS_M, WARPS_N, STAGES, SPLIT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         STAGES * (BM + BN) * 128);
    if (e != cudaSuccess) {
      bw::set_error("linear: cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  const int chunks = (k + kChunk - 1) / kChunk;
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM, SPLIT ? chunks : 1);
  if (grid.y > 65535u) {
    bw::set_error("linear: %d rows exceed the grid limit", m);
    return -1;
  }
  bw::launch_pdl(kernel, dim3(grid), dim3(THREADS), smem, stream, x, w, y, y_is_f32, residual, m, n, k, aligned, partials, counters);
  return bw::launch_status();
}

}  // namespace

// The tcgen05 / TMA variant (bf16_gemm_tc.cu), same summation order, for every shape whose
// rows start on 16 bytes.
BW_API int bw_bf16_linear_tc_usable(const void* x, const void* w, int k);
BW_API int bw_bf16_linear_tc_splits(int m, int n, int k);
BW_API int bw_bf16_linear_tc_may_split(int m, int n, int k);
BW_API long long bw_bf16_linear_tc_scratch_floats(int m, int n, int k);
BW_API int bw_bf16_linear_tc_counters(int n);
BW_API int bw_bf16_linear_tc(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32,
                             const float* residual, int m, int n, int k, float* partials, int* counters,
                             cudaStream_t stream);

// Rows up to which the legacy tile runs with one thread block per chunk.
constexpr int kSplitMaxRows = 64;
constexpr int kSplitBN = 64;

// Scratch that a product of this shape may need (chunk sums and per-tile counters), whichever
// variant runs it: the caller provides at least this much.
BW_API long long bw_bf16_linear_scratch_floats(int m, int n, int k) {
  const long long chunks = (k + kChunk - 1) / kChunk;
  const bool tc = bw_bf16_linear_tc_may_split(m, n, k) != 0;
  const bool legacy = m <= kSplitMaxRows && chunks > 1 && (n + kSplitBN - 1) / kSplitBN < 2 * 148;
  return (tc || legacy) ? chunks * m * n : 0;
}

BW_API int bw_bf16_linear_counters(int n) { return (n + kSplitBN - 1) / kSplitBN; }

BW_API int bw_bf16_linear_split_rows() { return 128; }

// One entry for every bfloat16 product. `use_legacy` != 0 forces the mma.sync tile (tests
// compare the two variants bit for bit); otherwise the tcgen05 kernel runs whenever the rows
// start on 16 bytes, and the legacy tile takes the remaining shapes (an inner size that is no
// multiple of 8).
BW_API int bw_bf16_linear(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32,
                          const float* residual, int m, int n, int k, float* partials, int* counters,
                          int use_legacy, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0) {
    bw::set_error("linear: inner size %d", k);
    return -1;
  }
  if (!use_legacy && bw_bf16_linear_tc_usable(x, w, k))
    return bw_bf16_linear_tc(x, w, y, y_is_f32, residual, m, n, k, partials, counters, stream);
  if (m > kSplitMaxRows)
    return launch<128, 128, 4, 4, 3, false>(x, w, y, y_is_f32, residual, m, n, k, nullptr, nullptr, stream);
  const int chunks = (k + kChunk - 1) / kChunk;
  const int tiles = (n + kSplitBN - 1) / kSplitBN;
  const bool split = chunks > 1 && tiles < 2 * 148 && partials != nullptr && counters != nullptr;
  if (split) return launch<64, kSplitBN, 2, 2, 4, true>(x, w, y, y_is_f32, residual, m, n, k, partials, counters, stream);
  return launch<64, kSplitBN, 2, 2, 4, false>(x, w, y, y_is_f32, residual, m, n, k, nullptr, nullptr, stream);
}
