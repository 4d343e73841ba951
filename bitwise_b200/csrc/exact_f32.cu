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
#include <cuda.h>

#include "bw_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// RMSNorm: ss = dot16(x, x); inv = 1 / sqrt(ss / width + eps); y = (x * inv) * w
// (src/kernels.cpp:264-271). One warp per output row; lanes 0..15 run the 16 chains.
// The row is brought into shared memory by the whole warp first (whole lines, all loads in
// flight together), so that the chains, which are what the time of a step of few rows hangs on,
// read shared memory instead of waiting for global memory eight values at a time.
constexpr int kNormWarps = 4;
constexpr int kNormStaged = 4096;  // widths up to this are staged; wider rows are read in place

__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_exact_kernel(const float* __restrict__ x, const float* __restrict__ w, float* y,
                     const int* __restrict__ rows, int n, int width, float eps) {
  extern __shared__ __align__(16) float norm_rows[];  // [kNormWarps][width] when the width is staged
  const int warp = threadIdx.x >> 5;
  const int r = blockIdx.x * (static_cast<int>(blockDim.x) >> 5) + warp;
  if (r >= n) return;
  const int lane = threadIdx.x & 31;
  const int src = rows ? rows[r] : r;
  const float* xr = x + static_cast<size_t>(src) * width;
  float* yr = y + static_cast<size_t>(r) * width;
  const bool staged = width <= kNormStaged;
  if (staged) {
    float* mine = norm_rows + warp * width;
#pragma unroll 16
    for (int i = lane; i < width; i += 32) mine[i] = xr[i];
    __syncwarp();
    xr = mine;
  }
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
#pragma unroll 4
  for (int i = lane; i < width; i += 32) yr[i] = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
}

// The same for steps of few rows: a block per row. All threads bring the row into shared memory
// (every load of the row in flight at once), lanes 0..15 of the first warp run the chains, all
// threads write the result: the row's time is one trip to memory and the chain.
constexpr int kNormRowThreads = 128;

__global__ void __launch_bounds__(kNormRowThreads)
rmsnorm_exact_row_kernel(const float* __restrict__ x, const float* __restrict__ w, float* y,
                         const int* __restrict__ rows, int width, float eps) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float norm_row[];  // [width], then the scale
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* xr = x + static_cast<size_t>(rows ? rows[r] : r) * width;
  float* yr = y + static_cast<size_t>(r) * width;
#pragma unroll 8
  for (int i = tid; i < width; i += kNormRowThreads) norm_row[i] = xr[i];
  __syncthreads();
  if (tid < 32) {
    float acc = 0.0f;
    if (tid < 16) {
#pragma unroll 8
      for (int i = tid; i < width; i += 16) {
        const float v = norm_row[i];
        acc = __fmaf_rn(v, v, acc);
      }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8, 16));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4, 16));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2, 16));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1, 16));
    if (tid == 0)
      norm_row[width] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(acc, static_cast<float>(width)), eps)));
  }
  __syncthreads();
  const float inv = norm_row[width];
#pragma unroll 8
  for (int i = tid; i < width; i += kNormRowThreads) yr[i] = __fmul_rn(__fmul_rn(norm_row[i], inv), w[i]);
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
// all that is read: one chain per output as above (k ascending, fma after fma). The tiles of W
// and x come through a ring of stages that a warp of its own requests; blocks stay for the
// whole launch, one on an SM, and walk tiles of TC columns one after the other, the ring
// running on from tile to tile.
//
// What bounds such a product on an SM, beside the weights' way from memory, is the way from
// shared memory into registers: 32 bytes a cycle for each of the SM's four schedulers, so that
// a warp's read of 16 bytes per lane takes 16 cycles (8 when all lanes read one address), far
// more than the multiply-adds it feeds unless a lane keeps several outputs: with RM rows and
// CN columns per lane, CN reads of W and RM reads of x feed 4 RM CN multiply-adds. And a chain
// takes 4 cycles per value of k whatever else happens. So the shape follows the product's
// width (the host's choice, see rows_plan): a narrow product is cut into tiles of 16 columns,
// one output per lane (lanes 0-15 and 16-31 of a warp carry two rows of the same 16 columns),
// so that every SM has a tile and the time is the chains' own; a wide one into tiles of 128
// columns with 4 rows x 2 columns per lane, which reads each value of W from shared memory
// once per 4 rows. A tile is carried by one chain warp per scheduler (two with 16 rows).
//
// A stage is LINES lines of 32 values of k: one TMA box of W ([LINES][TC columns][32 values],
// a three-dimensional view of the row-major matrix, written with the 128-byte swizzle so that
// the lanes of a quarter warp meet in no bank) and one of x ([LINES][R rows][32 values],
// plain: a warp reads one or two addresses of it at a time). What lies outside the matrices
// arrives as zeros; lines beyond k are not walked. The chain warps ask for the next stage's
// barrier before they start on this one, so that the answer (some hundred cycles even when the
// stage is there) comes while they compute. Every wait is bounded (bw_common.cuh).
constexpr int kRowsTileK = 32;    // values of k in a 128-byte line

template <int R, int RM, int CN, bool HALF, int CG, int LINES>
struct RowsShape {
  static constexpr int kLaneCols = HALF ? 16 : 32;           // columns that the lanes of a warp spread over
  static constexpr int kWarpRows = HALF ? 2 * RM : RM;       // rows that a warp carries
  static constexpr int kRowGroups = R / kWarpRows;
  static constexpr int kChainWarps = CG * kRowGroups;
  static constexpr int kTileCols = CG * CN * kLaneCols;
  static constexpr int kWBytes = LINES * kTileCols * 128, kXBytes = LINES * R * 128;
  static constexpr int kStageBytes = kWBytes + kXBytes;
  static constexpr int kThreads = (kChainWarps + 1) * 32;
  static_assert(R % kWarpRows == 0 && kTileCols % 8 == 0 && kTileCols <= 256, "tile shape");
  static_assert(kStageBytes % 1024 == 0, "the swizzle of W wants stages that start on 1,024 bytes");
};

__device__ __forceinline__ unsigned smem_addr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// asks once whether phase `parity` of the barrier is over
__device__ __forceinline__ bool bar_try(uint64_t* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// one box of the view (32 values, rows, lines): rows from `row` on, lines from `line` on
__device__ __forceinline__ void tma_box3(void* dst, const CUtensorMap* map, int row, int line, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_addr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(row), "r"(line), "r"(smem_addr(bar))
      : "memory");
}

// the multiply-adds of one line of k: 8 pieces of 16 bytes of this lane's CN columns against its RM rows
template <int RM, int CN>
__device__ __forceinline__ void rows_line(const unsigned char* wl, const unsigned char* xl, unsigned swz, float (&acc)[RM][CN]) {
#pragma unroll
  for (int p = 0; p < 8; ++p) {  // the 16-byte pieces of a swizzled line sit at piece ^ (row % 8)
    float4 w[CN], x[RM];
#pragma unroll
    for (int c = 0; c < CN; ++c) w[c] = *reinterpret_cast<const float4*>(wl + c * (32 * 128) + ((p << 4) ^ swz));
#pragma unroll
    for (int r = 0; r < RM; ++r) x[r] = *reinterpret_cast<const float4*>(xl + r * 128 + p * 16);
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < CN; ++c) acc[r][c] = __fmaf_rn(x[r].x, w[c].x, acc[r][c]);
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < CN; ++c) acc[r][c] = __fmaf_rn(x[r].y, w[c].y, acc[r][c]);
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < CN; ++c) acc[r][c] = __fmaf_rn(x[r].z, w[c].z, acc[r][c]);
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < CN; ++c) acc[r][c] = __fmaf_rn(x[r].w, w[c].w, acc[r][c]);
  }
}

template <int R, int RM, int CN, bool HALF, int CG, int LINES>
__global__ void __launch_bounds__(RowsShape<R, RM, CN, HALF, CG, LINES>::kThreads)
gemm_exact_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, float* Y,
                       const float* residual, int M, int N, int K, int stages, int* failure) {
  using S = RowsShape<R, RM, CN, HALF, CG, LINES>;
  extern __shared__ __align__(1024) unsigned char rows_raw[];
  unsigned char* base = bw::smem_align_1024(rows_raw);
  uint64_t* full = reinterpret_cast<uint64_t*>(base + stages * S::kStageBytes);  // a stage: W, then x
  uint64_t* empty = full + stages;
  volatile unsigned* gave_up = reinterpret_cast<volatile unsigned*>(failure);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lines_total = K / kRowsTileK;
  const int stages_per_tile = (lines_total + LINES - 1) / LINES;
  const int tiles = (N + S::kTileCols - 1) / S::kTileCols;
  const int my_tiles = (tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  if (tid == 0) {
    for (int s2 = 0; s2 < stages; ++s2) {
      bar_init(full + s2, 1);
      bar_init(empty + s2, S::kChainWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bw::pdl_launch();
  if (warp == S::kChainWarps) {  // the requesting warp
    if (lane == 0) {
      // The weights of the ring's first round do not depend on the kernel before this one: they
      // are asked for at once, the rows of x after the wait for that kernel.
      const int total = my_tiles * stages_per_tile;
      const int first = total < stages ? total : stages;
      {
        int t = 0, st = 0;
        for (int i = 0; i < first; ++i) {
          const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * S::kTileCols;
          bar_expect(full + i, S::kStageBytes);
          tma_box3(base + i * S::kStageBytes, &map_w, n0, st * LINES, full + i);
          if (++st == stages_per_tile) st = 0, ++t;
        }
      }
      bw::pdl_wait();
      int slot = 0, round = 0, it = 0;
      for (int t = 0; t < my_tiles; ++t) {
        const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * S::kTileCols;
        for (int st = 0; st < stages_per_tile; ++st, ++it) {
          unsigned char* stage = base + slot * S::kStageBytes;
          if (it >= first) {
            if (!bw::mbar_wait_bounded_idle(empty + slot, (round - 1) & 1, gave_up)) return;
            bar_expect(full + slot, S::kStageBytes);
            tma_box3(stage, &map_w, n0, st * LINES, full + slot);
          }
          tma_box3(stage + S::kWBytes, &map_x, 0, st * LINES, full + slot);
          if (++slot == stages) slot = 0, ++round;
        }
      }
    }
    return;
  }
  bw::pdl_wait();
  const int cg = warp % CG, rg = warp / CG;
  const int col = cg * (CN * S::kLaneCols) + (HALF ? (lane & 15) : lane);      // this lane's first column of the tile
  const int row0 = rg * S::kWarpRows + (HALF ? (lane >> 4) * RM : 0);            // and its first row
  const unsigned w_lane = col * 128, swz = (col & 7) << 4;
  if (!bw::mbar_wait_bounded(full, 0, gave_up)) return;
  int slot = 0, round = 0;
  for (int t = 0; t < my_tiles; ++t) {
    float acc[RM][CN];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < CN; ++c) acc[r][c] = 0.0f;
    for (int st = 0; st < stages_per_tile; ++st) {
      int next = slot + 1, next_round = round;
      if (next == stages) next = 0, ++next_round;
      const bool more = st + 1 < stages_per_tile || t + 1 < my_tiles;
      const bool next_there = more && bar_try(full + next, next_round & 1);  // answered while this stage is walked
      const unsigned char* wl = base + slot * S::kStageBytes + w_lane;
      const unsigned char* xl = base + slot * S::kStageBytes + S::kWBytes + row0 * 128;
      if (lines_total - st * LINES >= LINES) {
#pragma unroll
        for (int line = 0; line < LINES; ++line)
          rows_line<RM, CN>(wl + line * (S::kTileCols * 128), xl + line * (R * 128), swz, acc);
      } else {
        for (int line = 0; line < lines_total - st * LINES; ++line)
          rows_line<RM, CN>(wl + line * (S::kTileCols * 128), xl + line * (R * 128), swz, acc);
      }
      __syncwarp();
      if (lane == 0) bar_arrive(empty + slot);  // this warp has read the stage
      if (more && !next_there && !bw::mbar_wait_bounded(full + next, next_round & 1, gave_up)) return;
      slot = next, round = next_round;
    }
    const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * S::kTileCols;
#pragma unroll
    for (int c = 0; c < CN; ++c) {
      const int gn = n0 + col + c * 32;
      if (gn >= N) continue;
#pragma unroll
      for (int r = 0; r < RM; ++r) {
        const int gm = row0 + r;
        if (gm >= M) continue;
        const size_t o = static_cast<size_t>(gm) * N + gn;
        Y[o] = residual ? __fadd_rn(residual[o], acc[r][c]) : acc[r][c];
      }
    }
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
  bw::pdl_enter();
  const int r = blockIdx.x;
  const int half = hd >> 1;
  const int p = pos[r];
  float* row = qkv + static_cast<size_t>(r) * row_stride;
  const bool rotate = cos_t != nullptr;  // a null table leaves q and k as they are
  const float* c = rotate ? cos_t + static_cast<size_t>(p) * half : nullptr;
  const float* s = rotate ? sin_t + static_cast<size_t>(p) * half : nullptr;
  // A thread's pairs are read four at a time before any of them is written: the row is rotated
  // in place, and a write between the reads would keep them from being in flight together.
  const int q_items = rotate ? heads * half : 0;
  const int step = static_cast<int>(blockDim.x);
  for (int it0 = threadIdx.x; it0 < q_items; it0 += 4 * step) {
    float x1[4], x2[4], cc[4], ss[4];
    int at[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int it = it0 + u * step;
      at[u] = -1;
      if (it < q_items) {
        const int h = it / half, i = it - h * half;
        at[u] = h * hd + i;
        x1[u] = row[at[u]], x2[u] = row[at[u] + half], cc[u] = c[i], ss[u] = s[i];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (at[u] < 0) continue;
      row[at[u]] = __fsub_rn(__fmul_rn(x1[u], cc[u]), __fmul_rn(x2[u], ss[u]));
      row[at[u] + half] = __fadd_rn(__fmul_rn(x2[u], cc[u]), __fmul_rn(x1[u], ss[u]));
    }
  }
  if (!write_kv) return;
  const int blk = block_table[static_cast<size_t>(row_seq[r]) * max_blocks + p / page];
  const int slot = p % page;
  const float* k = row + heads * hd;
  const float* vv = k + kv_heads * hd;
  const int k_items = kv_heads * half;
  for (int it0 = threadIdx.x; it0 < k_items; it0 += 4 * step) {
    float x1[4], x2[4], v1[4], v2[4], cc[4], ss[4];
    size_t dst[4];
    bool ok[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int it = it0 + u * step;
      ok[u] = it < k_items;
      if (ok[u]) {
        const int h = it / half, i = it - h * half;
        dst[u] = ((static_cast<size_t>(blk) * kv_heads + h) * page + slot) * hd + i;
        x1[u] = k[h * hd + i], x2[u] = k[h * hd + i + half];
        v1[u] = vv[h * hd + i], v2[u] = vv[h * hd + i + half];
        cc[u] = rotate ? c[i] : 1.0f, ss[u] = rotate ? s[i] : 0.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!ok[u]) continue;
      kcache[dst[u]] = rotate ? __fsub_rn(__fmul_rn(x1[u], cc[u]), __fmul_rn(x2[u], ss[u])) : x1[u];
      kcache[dst[u] + half] = rotate ? __fadd_rn(__fmul_rn(x2[u], cc[u]), __fmul_rn(x1[u], ss[u])) : x2[u];
      vcache[dst[u]] = v1[u];
      vcache[dst[u] + half] = v2[u];
    }
  }
}

// ---------------------------------------------------------------------------------------
// Attention over the cache (src/kernels.cpp:312-338,361-364). For a query at position p of a
// sequence and a head h (key/value head g = h / (heads / kv_heads)):
//   pass 1   s_j = dot16(q, K_j) * scale for the keys j = lo .. p, mx = max_j s_j
//   pass 2   in key order: e_j = exp(s_j - mx); sum += e_j; acc[d] = fma(e_j, V_j[d], acc[d])
//   out[d] = acc[d] * (1 / sum)
// lo = max(0, p - window + 1) when window > 0, else 0. Which thread computes which score, and
// how many queries share a block, is free: a score is one dot16, the maximum does not depend
// on the order, and the chains of pass 2 (one per output element, plus the sum) are walked by
// one thread each, in key order. Two forms:
//   * tiles of up to 16 consecutive query rows of a sequence (prompt portions): a block per
//     (tile, head) walks the keys twice in tiles that all its rows share; the scores are
//     computed again in the second walk (the same instructions, so the same bits) instead of
//     being kept, so that the context is not limited by shared memory;
//   * single rows (decode steps): the scores of a row are spread over many blocks and stored,
//     a second kernel streams the values through a ring in shared memory.

// 16 lane-wise chains of a dot product, kept apart: lane[i % 16] = fma(a[i], b[i], lane[i % 16])
// for i ascending (src/kernels.cpp:86-100); bw::tree16 folds them.
constexpr int kTileRows = 16;       // query rows of a tile
constexpr int kTileThreads = 128;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // 0: zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}

template <int HD>
struct TileGeometry {
  static constexpr int KT = HD <= 64 ? 64 : 32;         // keys per tile
  static constexpr int KPT = KT / 32;                   // keys per thread when scores are computed
  static constexpr int KStride = HD + 4;                // floats per key row in shared memory: a lane's 16-byte
                                                        // read of its key meets no other lane's bank
  static constexpr int HDP = HD <= 16 ? 16 : HD <= 32 ? 32 : HD <= 64 ? 64 : HD <= 128 ? 128 : 256;
  static constexpr int TD = HDP < kTileThreads ? HDP : kTileThreads;  // threads side by side along d in pass 2
  static constexpr int DPT = HDP / TD;                  // output columns per thread
  static constexpr int RG = kTileThreads / TD;          // groups of rows
  static constexpr int RPT = kTileRows / RG;            // rows per thread
  static constexpr int QFloats = kTileRows * HD;
  static constexpr int KFloats = KT * KStride;
  static constexpr int VFloats = KT * HD;
  static constexpr int EFloats = KT * kTileRows;
  static constexpr int SmemFloats = QFloats + 2 * KFloats + 2 * VFloats + EFloats + 2 * kTileRows;
};

// Scores of this thread's pairs (4 rows of its warp x KPT keys of its lane) against the tile in
// shared memory: s[rr][c] = dot16(Q[4 w + rr], K[lane + 32 c]) * scale.
template <int HD>
__device__ __forceinline__ void tile_scores(const float* __restrict__ qs, const float* __restrict__ ks, int warp, int lane,
                                            float scale, float (&s)[4][TileGeometry<HD>::KPT]) {
  using G = TileGeometry<HD>;
  float acc[4][G::KPT][16];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr)
#pragma unroll
    for (int c = 0; c < G::KPT; ++c)
#pragma unroll
      for (int l = 0; l < 16; ++l) acc[rr][c][l] = 0.0f;
#pragma unroll
  for (int i4 = 0; i4 < HD / 4; ++i4) {
    float4 q[4], k[G::KPT];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) q[rr] = *reinterpret_cast<const float4*>(qs + (4 * warp + rr) * HD + 4 * i4);
#pragma unroll
    for (int c = 0; c < G::KPT; ++c) k[c] = *reinterpret_cast<const float4*>(ks + (lane + 32 * c) * G::KStride + 4 * i4);
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int c = 0; c < G::KPT; ++c) {
        float* a = acc[rr][c] + 4 * (i4 & 3);
        a[0] = __fmaf_rn(q[rr].x, k[c].x, a[0]);
        a[1] = __fmaf_rn(q[rr].y, k[c].y, a[1]);
        a[2] = __fmaf_rn(q[rr].z, k[c].z, a[2]);
        a[3] = __fmaf_rn(q[rr].w, k[c].w, a[3]);
      }
  }
#pragma unroll
  for (int rr = 0; rr < 4; ++rr)
#pragma unroll
    for (int c = 0; c < G::KPT; ++c) s[rr][c] = __fmul_rn(bw::tree16(acc[rr][c]), scale);
}

template <int HD>
__global__ void __launch_bounds__(kTileThreads)
attention_tiles_exact_kernel(const float* __restrict__ qkv, int q_stride, const float* __restrict__ kcache,
                             const float* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                             const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                             const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                             const int* __restrict__ seq_row0, float* __restrict__ out, int out_stride, int heads,
                             int kv_heads, int page, int window, float scale) {
  using G = TileGeometry<HD>;
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                       // [16][HD]
  float* kbuf = qs + G::QFloats;          // [2][KT][KStride]
  float* vbuf = kbuf + 2 * G::KFloats;    // [2][KT][HD]
  float* es = vbuf + 2 * G::VFloats;      // [KT][16]: weights of the tile in hand, by key
  float* row_max = es + G::EFloats;       // [16]
  float* row_inv = row_max + kTileRows;   // [16]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.y, h = blockIdx.x;  // heads fastest: the host lists the longest tiles first
  const int g = h / (heads / kv_heads);
  const int seq = tile_seq[tile], row0 = tile_row0[tile], nrows = tile_rows[tile];
  const int p_first = seq_pos0[seq] + (row0 - seq_row0[seq]);  // position of the tile's first query row
  const int p_last = p_first + nrows - 1;
  const int* table = block_table + static_cast<size_t>(seq) * max_blocks;
  auto first_key = [&](int p) { return (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0; };
  const int kv_lo = (first_key(p_first) / G::KT) * G::KT;
  const int ntiles = (p_last + 1 - kv_lo + G::KT - 1) / G::KT;

  for (int idx = tid; idx < kTileRows * (HD / 4); idx += kTileThreads) {
    const int r = idx / (HD / 4), piece = idx - r * (HD / 4);
    const bool ok = r < nrows;
    cp_async16(qs + r * HD + 4 * piece, qkv + static_cast<size_t>(row0 + (ok ? r : 0)) * q_stride + h * HD + 4 * piece, ok);
  }
  // keys (and values) of tile t into buffer t % 2; keys beyond the last query's position are zeros.
  // A thread keeps its 16-byte piece of a row and walks the keys.
  const int page_shift = (page & (page - 1)) == 0 ? __ffs(page) - 1 : -1;
  constexpr int kPieces = HD / 4, kKeysPerPass = kTileThreads / kPieces;
  const int my_piece = tid % kPieces, my_key0 = tid / kPieces;
  auto load_tile = [&](int t, bool with_values) {
    if (my_key0 >= kKeysPerPass) return;  // threads beyond a whole number of keys sit out
    float* kd = kbuf + (t & 1) * G::KFloats;
    float* vd = vbuf + (t & 1) * G::VFloats;
    for (int key = my_key0; key < G::KT; key += kKeysPerPass) {
      const int j = kv_lo + t * G::KT + key;
      const bool ok = j <= p_last;
      size_t off = 0;
      if (ok) {
        const int blk = page_shift >= 0 ? j >> page_shift : j / page;
        off = ((static_cast<size_t>(table[blk]) * kv_heads + g) * page + (j - blk * page)) * HD + 4 * my_piece;
      }
      cp_async16(kd + key * G::KStride + 4 * my_piece, kcache + off, ok);
      if (with_values) cp_async16(vd + key * HD + 4 * my_piece, vcache + off, ok);
    }
  };
  // this thread's rows when scores are computed, their positions and first keys
  int pos_r[4], lo_r[4];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int r = 4 * warp + rr;
    pos_r[rr] = r < nrows ? p_first + r : -1;  // a row beyond the tile sees no key
    lo_r[rr] = first_key(pos_r[rr]);
  }

  // ---- first walk: the maximum of every row's scores
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  load_tile(0, false);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) load_tile(t + 1, false);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    float s[4][G::KPT];
    tile_scores<HD>(qs, kbuf + (t & 1) * G::KFloats, warp, lane, scale, s);
    const int j0 = kv_lo + t * G::KT;
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int c = 0; c < G::KPT; ++c) {
        const int j = j0 + lane + 32 * c;
        if (j >= lo_r[rr] && j <= pos_r[rr]) mx[rr] = fmaxf(mx[rr], s[rr][c]);
      }
    __syncthreads();  // the buffer may be refilled
  }
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], o));
  }

  // ---- second walk: weights, their sum and the weighted values, in key order
  const int dcol = tid % G::TD, rg = tid / G::TD;  // pass 2: this thread's first output column and group of rows
  float acc[G::RPT][G::DPT];
#pragma unroll
  for (int i = 0; i < G::RPT; ++i)
#pragma unroll
    for (int dd = 0; dd < G::DPT; ++dd) acc[i][dd] = 0.0f;
  float sum = 0.0f;                                 // of row rg * RPT + dcol, for dcol < RPT
  const int sum_row = rg * G::RPT + (dcol < G::RPT ? dcol : 0);
  const int sum_pos = sum_row < nrows ? p_first + sum_row : -1, sum_lo = first_key(sum_pos);
  int pos2[G::RPT], lo2[G::RPT];
#pragma unroll
  for (int i = 0; i < G::RPT; ++i) {
    const int r = rg * G::RPT + i;
    pos2[i] = r < nrows ? p_first + r : -1;
    lo2[i] = first_key(pos2[i]);
  }
  const int lo_all = first_key(p_last);  // a key from here on is in every row's window
  load_tile(0, true);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) load_tile(t + 1, true);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const int j0 = kv_lo + t * G::KT;
    {
      float s[4][G::KPT];
      tile_scores<HD>(qs, kbuf + (t & 1) * G::KFloats, warp, lane, scale, s);
#pragma unroll
      for (int c = 0; c < G::KPT; ++c) {
        float4 e;
        e.x = bw::det_expf(__fsub_rn(s[0][c], mx[0]));
        e.y = bw::det_expf(__fsub_rn(s[1][c], mx[1]));
        e.z = bw::det_expf(__fsub_rn(s[2][c], mx[2]));
        e.w = bw::det_expf(__fsub_rn(s[3][c], mx[3]));
        *reinterpret_cast<float4*>(es + (lane + 32 * c) * kTileRows + 4 * warp) = e;
      }
    }
    __syncthreads();
    const float* vt = vbuf + (t & 1) * G::VFloats;
    const int keys = min(G::KT, p_last + 1 - j0);
    const bool all_in = nrows == kTileRows && j0 >= lo_all && j0 + G::KT - 1 <= p_first;
    if (dcol < HD || G::TD * (G::DPT - 1) + dcol < HD || dcol < G::RPT) {
      if (all_in) {
#pragma unroll 4
        for (int kk = 0; kk < G::KT; ++kk) {
          float e[G::RPT], v[G::DPT];
#pragma unroll
          for (int i = 0; i < G::RPT; ++i) e[i] = es[kk * kTileRows + rg * G::RPT + i];
#pragma unroll
          for (int dd = 0; dd < G::DPT; ++dd) v[dd] = (dcol + G::TD * dd < HD) ? vt[kk * HD + dcol + G::TD * dd] : 0.0f;
          if (dcol < G::RPT) sum = __fadd_rn(sum, es[kk * kTileRows + sum_row]);
#pragma unroll
          for (int i = 0; i < G::RPT; ++i)
#pragma unroll
            for (int dd = 0; dd < G::DPT; ++dd) acc[i][dd] = __fmaf_rn(e[i], v[dd], acc[i][dd]);
        }
      } else {
        for (int kk = 0; kk < keys; ++kk) {
          const int j = j0 + kk;
          float v[G::DPT];
#pragma unroll
          for (int dd = 0; dd < G::DPT; ++dd) v[dd] = (dcol + G::TD * dd < HD) ? vt[kk * HD + dcol + G::TD * dd] : 0.0f;
          if (dcol < G::RPT && j >= sum_lo && j <= sum_pos) sum = __fadd_rn(sum, es[kk * kTileRows + sum_row]);
#pragma unroll
          for (int i = 0; i < G::RPT; ++i) {
            if (j < lo2[i] || j > pos2[i]) continue;
            const float e = es[kk * kTileRows + rg * G::RPT + i];
#pragma unroll
            for (int dd = 0; dd < G::DPT; ++dd) acc[i][dd] = __fmaf_rn(e, v[dd], acc[i][dd]);
          }
        }
      }
    }
    __syncthreads();  // the buffers and the weights may be overwritten
  }
  if (dcol < G::RPT) row_inv[rg * G::RPT + dcol] = __fdiv_rn(1.0f, sum);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < G::RPT; ++i) {
    const int r = rg * G::RPT + i;
    if (r >= nrows) continue;
#pragma unroll
    for (int dd = 0; dd < G::DPT; ++dd) {
      const int d = dcol + G::TD * dd;
      if (d < HD) out[static_cast<size_t>(row0 + r) * out_stride + h * HD + d] = __fmul_rn(acc[i][dd], row_inv[r]);
    }
  }
}

// ---- single rows: scores by many blocks -------------------------------------------------------
// A block takes kScoreKeys consecutive keys of one (row, head) and computes
// s_j = dot16(q, K_j) * scale for each; the block's maximum goes to its own place.
// scores[(row * heads + h) * score_stride + j], chunk_max[(row * heads + h) * chunks + chunk].
// Four neighbouring threads share a key: thread c of the four carries the partial sums 4c .. 4c+3
// of the sixteen (the values of k at 16 i + 4c + {0..3}), so that a warp's load covers eight keys
// in pieces of 64 consecutive bytes instead of 32 keys in pieces of 16, and the sixteen sums meet
// through two exchanges in the order of bw::tree16: (l, l + 8), then (l, l + 4), then the last two.
constexpr int kScoreThreads = 256;
constexpr int kScoreKeys = 256;

__global__ void __launch_bounds__(kScoreThreads)
attention_scores_exact_kernel(const float* __restrict__ qkv, int q_stride, const float* __restrict__ kcache,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_seq,
                              const int* __restrict__ pos, int heads, int kv_heads, int hd, int page, int window,
                              float scale, float* __restrict__ scores, int score_stride,
                              float* __restrict__ chunk_max, int chunks) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float smem[];
  float* q = smem;  // [hd]
  __shared__ float red[kScoreThreads / 32];
  const int r = blockIdx.x, h = blockIdx.y, chunk = blockIdx.z, tid = threadIdx.x;
  const int p = pos[r];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int c0 = chunk * kScoreKeys;
  if (c0 > p || c0 + kScoreKeys <= lo) return;  // no key of the row's range in this chunk
  const int g = h / (heads / kv_heads);
  const int* table = block_table + static_cast<size_t>(row_seq[r]) * max_blocks;
  const float* qg = qkv + static_cast<size_t>(r) * q_stride + h * hd;
  for (int i = tid; i < hd; i += kScoreThreads) q[i] = qg[i];
  __syncthreads();
  float* out = scores + (static_cast<size_t>(r) * heads + h) * score_stride;
  const int c = tid & 3;  // which four of the sixteen partial sums
  float mx = -INFINITY;
#pragma unroll 2
  for (int j = c0 + (tid >> 2); j < c0 + kScoreKeys; j += kScoreThreads / 4) {
    const bool in_range = j >= lo && j <= p;  // the four threads of a key agree, whole warps may not
    const int jj = in_range ? j : p;
    const float* kp = kcache + ((static_cast<size_t>(table[jj / page]) * kv_heads + g) * page + jj % page) * hd + 4 * c;
    float4 part = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int i = 0; i < hd; i += 16) {
      const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
      const float4 q4 = *reinterpret_cast<const float4*>(q + i + 4 * c);
      part.x = __fmaf_rn(q4.x, k4.x, part.x), part.y = __fmaf_rn(q4.y, k4.y, part.y);
      part.z = __fmaf_rn(q4.z, k4.z, part.z), part.w = __fmaf_rn(q4.w, k4.w, part.w);
    }
    // sums l and l + 8 lie two threads apart, their sums l and l + 4 one thread apart
    part.x = __fadd_rn(part.x, __shfl_xor_sync(0xffffffffu, part.x, 2));
    part.y = __fadd_rn(part.y, __shfl_xor_sync(0xffffffffu, part.y, 2));
    part.z = __fadd_rn(part.z, __shfl_xor_sync(0xffffffffu, part.z, 2));
    part.w = __fadd_rn(part.w, __shfl_xor_sync(0xffffffffu, part.w, 2));
    part.x = __fadd_rn(part.x, __shfl_xor_sync(0xffffffffu, part.x, 1));
    part.y = __fadd_rn(part.y, __shfl_xor_sync(0xffffffffu, part.y, 1));
    part.z = __fadd_rn(part.z, __shfl_xor_sync(0xffffffffu, part.z, 1));
    part.w = __fadd_rn(part.w, __shfl_xor_sync(0xffffffffu, part.w, 1));
    const float sc = __fmul_rn(__fadd_rn(__fadd_rn(part.x, part.z), __fadd_rn(part.y, part.w)), scale);
    if (in_range) {
      if (c == 0) out[j] = sc;
      mx = fmaxf(mx, sc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
#pragma unroll
    for (int w = 1; w < kScoreThreads / 32; ++w) m = fmaxf(m, red[w]);
    chunk_max[(static_cast<size_t>(r) * heads + h) * chunks + chunk] = m;
  }
}

// ---- single rows: the chains of pass 2 -------------------------------------------------------
// A block per (row, head, slice of the output columns): the weights e_j = exp(s_j - mx) of
// the whole row are put into shared memory first (all threads, any order: each is a function
// of its own score), then the values stream through a ring of tiles of 64 keys and thread d
// walks the keys in order: sum += e_j, acc = fma(e_j, V_j[d], acc). Every chain thread carries
// the sum itself. The warps that hold chain threads do nothing but walk the chains: a thread
// that also computed addresses and issued copies would stretch the chain that the kernel's time
// hangs on. Two forms of the copying:
//   * by pages (whole value rows, a page size that divides 64, no window): one more warp
//     requests a page of a head, which lies in one piece, as one bulk copy counted on the
//     tile's barrier; the chain warps hand a tile back through a second barrier;
//   * by 16-byte pieces (any page size, slices of the rows, windows): the block's other warps
//     copy with cp.async, a thread keeps its piece of a row and walks the keys.
constexpr int kValueTile = 64;
constexpr int kValueMaxStages = 6;
constexpr int kValueMaxSlice = 128;  // output columns per block at most
constexpr int kValueStages = 4;      // of the form that copies by pieces
constexpr int kValueThreads = 256;   // of the form that copies by pieces: the first `dslice` walk the chains

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// the keys of one tile for output column d: `e_t` the tile's weights, `v` the tile's values at column d
__device__ __forceinline__ void value_chain(const float* __restrict__ e_t, const float* __restrict__ v, int dslice, int keys,
                                            float& sum, float& acc) {
  if (keys == kValueTile) {
    // eight keys' weights and values are read while the eight before them are chained in
    float4 e0 = *reinterpret_cast<const float4*>(e_t), e1 = *reinterpret_cast<const float4*>(e_t + 4);  // tiles start on 16 bytes
    float vv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) vv[i] = v[i * dslice];
#pragma unroll
    for (int s8 = 0; s8 < kValueTile; s8 += 8) {
      float4 n0 = e0, n1 = e1;
      float vn[8];
      if (s8 + 8 < kValueTile) {
        n0 = *reinterpret_cast<const float4*>(e_t + s8 + 8), n1 = *reinterpret_cast<const float4*>(e_t + s8 + 12);
#pragma unroll
        for (int i = 0; i < 8; ++i) vn[i] = v[(s8 + 8 + i) * dslice];
      }
      sum = __fadd_rn(sum, e0.x), acc = __fmaf_rn(e0.x, vv[0], acc);
      sum = __fadd_rn(sum, e0.y), acc = __fmaf_rn(e0.y, vv[1], acc);
      sum = __fadd_rn(sum, e0.z), acc = __fmaf_rn(e0.z, vv[2], acc);
      sum = __fadd_rn(sum, e0.w), acc = __fmaf_rn(e0.w, vv[3], acc);
      sum = __fadd_rn(sum, e1.x), acc = __fmaf_rn(e1.x, vv[4], acc);
      sum = __fadd_rn(sum, e1.y), acc = __fmaf_rn(e1.y, vv[5], acc);
      sum = __fadd_rn(sum, e1.z), acc = __fmaf_rn(e1.z, vv[6], acc);
      sum = __fadd_rn(sum, e1.w), acc = __fmaf_rn(e1.w, vv[7], acc);
      if (s8 + 8 < kValueTile) {
        e0 = n0, e1 = n1;
#pragma unroll
        for (int i = 0; i < 8; ++i) vv[i] = vn[i];
      }
    }
  } else {
    for (int s2 = 0; s2 < keys; ++s2) {
      const float e = e_t[s2];
      sum = __fadd_rn(sum, e);
      acc = __fmaf_rn(e, v[s2 * dslice], acc);
    }
  }
}

// The same for a thread that carries two neighbouring outputs (a read of 8 bytes per key): two
// chains that do not wait for one another, half as many warps on the way from shared memory.
__device__ __forceinline__ void value_chain2(const float* __restrict__ e_t, const float* __restrict__ v, int dslice, int keys,
                                             float& sum, float2& acc) {
  if (keys == kValueTile) {
    float4 e0 = *reinterpret_cast<const float4*>(e_t), e1 = *reinterpret_cast<const float4*>(e_t + 4);
    float2 vv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) vv[i] = *reinterpret_cast<const float2*>(v + i * dslice);
#pragma unroll
    for (int s8 = 0; s8 < kValueTile; s8 += 8) {
      float4 n0 = e0, n1 = e1;
      float2 vn[8];
      if (s8 + 8 < kValueTile) {
        n0 = *reinterpret_cast<const float4*>(e_t + s8 + 8), n1 = *reinterpret_cast<const float4*>(e_t + s8 + 12);
#pragma unroll
        for (int i = 0; i < 8; ++i) vn[i] = *reinterpret_cast<const float2*>(v + (s8 + 8 + i) * dslice);
      }
      const float e[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sum = __fadd_rn(sum, e[i]);
        acc.x = __fmaf_rn(e[i], vv[i].x, acc.x), acc.y = __fmaf_rn(e[i], vv[i].y, acc.y);
      }
      if (s8 + 8 < kValueTile) {
        e0 = n0, e1 = n1;
#pragma unroll
        for (int i = 0; i < 8; ++i) vv[i] = vn[i];
      }
    }
  } else {
    for (int s2 = 0; s2 < keys; ++s2) {
      const float e = e_t[s2];
      const float2 x = *reinterpret_cast<const float2*>(v + s2 * dslice);
      sum = __fadd_rn(sum, e);
      acc.x = __fmaf_rn(e, x.x, acc.x), acc.y = __fmaf_rn(e, x.y, acc.y);
    }
  }
}

// the weights of a row into shared memory, by `count` threads of which this is number `tid`
__device__ __forceinline__ void row_weights(float* es, const float* __restrict__ scores, const float* __restrict__ cm,
                                            int lo, int p, int tid, int count) {
  // The chunks' maxima and the scores come from memory that another kernel just wrote: many
  // loads are asked for before the first is used, or every one of them would cost a round trip.
  float mx = -INFINITY;
  for (int c = lo / kScoreKeys + (tid & 31); c <= p / kScoreKeys; c += 32) mx = fmaxf(mx, cm[c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));  // a maximum has no order
  const int n = p - lo + 1;
  for (int j0 = tid; j0 < n; j0 += 16 * count) {
    float s[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int j = j0 + u * count;
      s[u] = j < n ? scores[lo + j] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int j = j0 + u * count;
      if (j < n) es[j] = bw::det_expf(__fsub_rn(s[u], mx));
    }
  }
}

__global__ void __launch_bounds__(kValueMaxSlice + 32)
attention_values_paged_exact_kernel(const float* __restrict__ scores, int score_stride, const float* __restrict__ chunk_max,
                                    int chunks, const float* __restrict__ vcache, const int* __restrict__ block_table,
                                    int max_blocks, const int* __restrict__ row_seq, const int* __restrict__ pos,
                                    float* __restrict__ out, int out_stride, int heads, int kv_heads, int hd, int page,
                                    int weight_floats, int stages, int* failure) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float smem[];
  float* es = smem;                    // [len] weights of the row
  float* vt = smem + weight_floats;    // [stages][kValueTile][hd]
  uint64_t* full = reinterpret_cast<uint64_t*>(vt + stages * kValueTile * hd);
  uint64_t* empty = full + stages;
  volatile unsigned* gave_up = reinterpret_cast<volatile unsigned*>(failure);
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int workers = static_cast<int>(blockDim.x) - 32;  // whole warps of chain threads, then the requesting warp
  const int p = pos[r];
  const int len = p + 1;
  const int g = h / (heads / kv_heads);
  const int* table = block_table + static_cast<size_t>(row_seq[r]) * max_blocks;
  const int tiles = (len + kValueTile - 1) / kValueTile;
  if (tid == 0) {
    for (int s2 = 0; s2 < stages; ++s2) {
      bar_init(full + s2, 1);
      bar_init(empty + s2, workers / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (tid >= workers) {
    // the requesting warp: lane l brings page l of a tile (a page of a head lies in one piece)
    const int pages_per_tile = kValueTile / page;
    const unsigned page_bytes = static_cast<unsigned>(page) * hd * 4u;
    for (int t = 0; t < tiles; ++t) {
      const int slot = t % stages;
      if (t >= stages && !bw::mbar_wait_bounded_idle(empty + slot, ((t / stages) - 1) & 1, gave_up)) break;
      const int keys = min(kValueTile, len - t * kValueTile);
      const int pages = (keys + page - 1) / page;  // the last page is copied whole: it is the request's own
      if (lane == 0) bar_expect(full + slot, page_bytes * pages);
      __syncwarp();
      for (int pg = lane; pg < pages; pg += 32) {
        const int blk = t * pages_per_tile + pg;
        const size_t off = (static_cast<size_t>(table[blk]) * kv_heads + g) * page * hd;
        bulk_copy(vt + (slot * kValueTile + pg * page) * hd, vcache + off, page_bytes, full + slot);
      }
    }
    return;
  }
  row_weights(es, scores + (static_cast<size_t>(r) * heads + h) * score_stride,
              chunk_max + (static_cast<size_t>(r) * heads + h) * chunks, 0, p, tid, workers);
  asm volatile("bar.sync 1, %0;" ::"r"(workers) : "memory");  // the chain warps only: the requesting warp is elsewhere
  const int d = 2 * tid;  // this thread's two outputs
  float2 acc = make_float2(0.0f, 0.0f);
  float sum = 0.0f;
  for (int t = 0; t < tiles; ++t) {
    const int slot = t % stages;
    if (!bw::mbar_wait_bounded(full + slot, (t / stages) & 1, gave_up)) break;
    if (d < hd) value_chain2(es + t * kValueTile, vt + slot * kValueTile * hd + d, hd, min(kValueTile, len - t * kValueTile), sum, acc);
    __syncwarp();
    if (lane == 0) bar_arrive(empty + slot);  // this warp has read the tile
  }
  if (d < hd) {
    const float inv = __fdiv_rn(1.0f, sum);
    *reinterpret_cast<float2*>(out + static_cast<size_t>(r) * out_stride + h * hd + d) = make_float2(__fmul_rn(acc.x, inv), __fmul_rn(acc.y, inv));
  }
}

__global__ void __launch_bounds__(kValueThreads)
attention_values_exact_kernel(const float* __restrict__ scores, int score_stride, const float* __restrict__ chunk_max,
                              int chunks, const float* __restrict__ vcache, const int* __restrict__ block_table,
                              int max_blocks, const int* __restrict__ row_seq, const int* __restrict__ pos,
                              float* __restrict__ out, int out_stride, int heads, int kv_heads, int hd, int dslice,
                              int page, int window, int weight_floats) {
  bw::pdl_enter();
  extern __shared__ __align__(16) float smem[];
  float* es = smem;                    // [len] weights of the row
  float* vt = smem + weight_floats;    // [kValueStages][kValueTile][dslice]
  const int r = blockIdx.x, h = blockIdx.y, d0 = blockIdx.z * dslice, tid = threadIdx.x;
  const int p = pos[r];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int len = p - lo + 1;
  const int g = h / (heads / kv_heads);
  const int* table = block_table + static_cast<size_t>(row_seq[r]) * max_blocks;
  const int pieces = dslice / 4;  // 16-byte pieces of this block's part of a value row
  const int tiles = (len + kValueTile - 1) / kValueTile;
  const int workers = (dslice + 31) / 32 * 32, copiers = kValueThreads - workers;
  const bool copier = tid >= workers;
  const int ctid = tid - workers;
  const int page_shift = (page & (page - 1)) == 0 ? __ffs(page) - 1 : -1;
  const int keys_per_pass = copiers / pieces, my_piece = ctid % pieces, my_key0 = ctid / pieces;
  auto fetch = [&](int t) {
    if (!copier || my_key0 >= keys_per_pass) return;  // threads beyond a whole number of keys sit out
    float* dst = vt + (t % kValueStages) * kValueTile * dslice + 4 * my_piece;
    for (int key = my_key0; key < kValueTile; key += keys_per_pass) {
      const int j = lo + t * kValueTile + key;
      const bool ok = j <= p;
      size_t off = 0;
      if (ok) {
        const int blk = page_shift >= 0 ? j >> page_shift : j / page;
        off = ((static_cast<size_t>(table[blk]) * kv_heads + g) * page + (j - blk * page)) * hd + d0 + 4 * my_piece;
      }
      cp_async16(dst + key * dslice, vcache + off, ok);
    }
  };
  // the values do not wait for the weights: the ring is filled first
  for (int t = 0; t < kValueStages - 1; ++t) {
    if (t < tiles) fetch(t);
    asm volatile("cp.async.commit_group;\n" ::);
  }
  row_weights(es, scores + (static_cast<size_t>(r) * heads + h) * score_stride,
              chunk_max + (static_cast<size_t>(r) * heads + h) * chunks, lo, p, tid, kValueThreads);
  const int d = tid;  // column d0 + d of the output, for d < dslice
  float acc = 0.0f, sum = 0.0f;
  for (int t = 0; t < tiles; ++t) {
    if (copier) asm volatile("cp.async.wait_group %0;\n" ::"n"(kValueStages - 2));
    __syncthreads();  // tile t has landed (every copier waited for its own copies) and, at t = 0, the
                      // weights are written; the buffer of tile t - 1 is free
    if (copier) {
      if (t + kValueStages - 1 < tiles) fetch(t + kValueStages - 1);
      asm volatile("cp.async.commit_group;\n" ::);
      continue;
    }
    if (d < dslice)
      value_chain(es + t * kValueTile, vt + (t % kValueStages) * kValueTile * dslice + d, dslice,
                  min(kValueTile, len - t * kValueTile), sum, acc);
  }
  if (d < dslice) out[static_cast<size_t>(r) * out_stride + h * hd + d0 + d] = __fmul_rn(acc, __fdiv_rn(1.0f, sum));
}

// ---------------------------------------------------------------------------------------
// SwiGLU on rows laid out [gate | up]: h = (g * (1 / (1 + exp(-g)))) * u (src/kernels.cpp:291-298).
__global__ void swiglu_exact_kernel(const float* __restrict__ gate_up, float* __restrict__ out, int n, int inter) {
  bw::pdl_enter();
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
// Tensor maps for the streaming tile of few rows: a row-major float32 matrix [rows][k] seen as
// (32 values, rows, k / 32 lines), boxes of box_lines lines x box_rows rows, with the 128-byte
// swizzle or plain, zeros outside.
namespace {
typedef CUresult (*EncodeTiledF32)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledF32 f32_encoder() {
  static EncodeTiledF32 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledF32>(p);
  }
  return fn;
}
bool f32_rows_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows, int box_lines, bool swizzled) {
  EncodeTiledF32 enc = f32_encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {kRowsTileK, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k / kRowsTileK)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 4, kRowsTileK * 4};
  const cuuint32_t box[3] = {kRowsTileK, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_lines)};
  const cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// The streaming tile's width for a product (16, 32, 64 or 128 columns; the kernel's shape follows
// from it) and the stages of its ring.
struct RowsPlan {
  int tile_cols, stages;
};
int g_forced_tile_cols = 0, g_forced_stages = 0;

// lines of k in a stage, by tile width: stages of 16 to 40 KB
constexpr int rows_lines(int tile_cols) { return tile_cols == 16 ? 8 : tile_cols == 128 ? 2 : 4; }

RowsPlan rows_plan(int rows, int n, int k) {
  const int sms = sm_count();
  // Cycles that a tile's chain warps take per four values of k (the inner loop alone, measured on
  // a B200 with 8 rows; with 16 rows two warps share a scheduler and all of them double), times
  // the tiles that the busiest SM walks: the narrowest tile for narrow products, where the
  // chains' own length counts, the widest where there is a tile or more for every SM. The
  // choice this makes was the fastest of the four widths for every product of the two model
  // shapes that bench.py knows (measured with bw_f32_force_rows_plan).
  const int widths[4] = {16, 32, 64, 128};
  const int cycles[4] = {20, 34, 48, 76};
  int best = 0;
  long long best_cost = 0;
  for (int i = 0; i < 4; ++i) {
    const int tiles = (n + widths[i] - 1) / widths[i];
    const long long cost = static_cast<long long>((tiles + sms - 1) / sms) * cycles[i];
    if (i == 0 || cost < best_cost) best = i, best_cost = cost;
  }
  RowsPlan p;
  p.tile_cols = widths[best];
  if (g_forced_tile_cols == 16 || g_forced_tile_cols == 32 || g_forced_tile_cols == 64 || g_forced_tile_cols == 128)
    p.tile_cols = g_forced_tile_cols;
  const int stage_bytes = rows_lines(p.tile_cols) * (p.tile_cols + rows) * 128;
  p.stages = (225 * 1024) / (stage_bytes + 16);
  p.stages = p.stages > 12 ? 12 : p.stages;
  if (g_forced_stages >= 2 && g_forced_stages < p.stages) p.stages = g_forced_stages;
  return p;
}

template <int R, int RM, int CN, bool HALF, int CG, int LINES>
int launch_rows(const CUtensorMap& map_x, const CUtensorMap& map_w, float* y, const float* residual, int m, int n, int k,
                int stages, int* word, cudaStream_t stream) {
  using S = RowsShape<R, RM, CN, HALF, CG, LINES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_exact_rows_kernel<R, RM, CN, HALF, CG, LINES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      bw::set_error("linear (32-bit): cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  const int tiles = (n + S::kTileCols - 1) / S::kTileCols;
  const int sms = sm_count();
  const int smem = stages * (S::kStageBytes + 16) + 1024;
  cudaError_t le = bw::launch_pdl(gemm_exact_rows_kernel<R, RM, CN, HALF, CG, LINES>, dim3(tiles < sms ? tiles : sms), dim3(S::kThreads),
                                  static_cast<size_t>(smem), stream, map_x, map_w, y, residual, m, n, k, stages, word);
  if (le != cudaSuccess) {
    bw::set_error("linear (32-bit): launch failed: %s", cudaGetErrorString(le));
    return static_cast<int>(le);
  }
  return bw::launch_status();
}
}  // namespace

// For measurements and tests: fixes the streaming tile's width (16, 32, 64 or 128 columns) and
// the stages of its ring for the products that follow (0: the library's own choice).
BW_API void bw_f32_force_rows_plan(int tile_cols, int stages) { g_forced_tile_cols = tile_cols, g_forced_stages = stages; }

// ---------------------------------------------------------------------------------------
// Exported entry points.

BW_API int bw_f32_rmsnorm(const float* x, const float* weight, float* y, const int* rows, int n, int width,
                          float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0) {
    bw::set_error("rmsnorm: width %d", width);
    return -1;
  }
  const size_t smem = width <= kNormStaged ? static_cast<size_t>(kNormWarps) * width * sizeof(float) : 0;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kNormWarps * kNormStaged * static_cast<int>(sizeof(float)));
    if (e != cudaSuccess) {
      bw::set_error("rmsnorm: cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  if (n <= 64 && width < 12000)  // few rows (a decode step): a block per row
    bw::launch_pdl(rmsnorm_exact_row_kernel, dim3(n), dim3(kNormRowThreads), (width + 4) * sizeof(float), stream, x, weight, y, rows, width, eps);
  else
    rmsnorm_exact_kernel<<<(n + kNormWarps - 1) / kNormWarps, kNormWarps * 32, smem, stream>>>(x, weight, y, rows, n, width, eps);
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
  if (m <= 16 && k % kRowsTileK == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
      f32_encoder() != nullptr) {
    // rows that are whole 128-byte lines: the streaming tile
    const int rows = m <= 8 ? 8 : 16;
    const RowsPlan plan = rows_plan(rows, n, k);
    const int lines = rows_lines(plan.tile_cols);
    int* word = bw::failure_word();
    if (!word) return -1;
    CUtensorMap map_x, map_w;
    if (!f32_rows_map(&map_x, x, m, k, rows, lines, false) || !f32_rows_map(&map_w, w, n, k, plan.tile_cols, lines, true)) {
      bw::set_error("linear (32-bit): cuTensorMapEncodeTiled refused [%d x %d] / [%d x %d]", m, k, n, k);
      return -1;
    }
    // rows, rows and columns per lane, half-warp layout, column groups of warps, lines per stage
#define BW_ROWS(TC_, R_, RM_, CN_, HALF_, CG_)                                                                        \
  if (plan.tile_cols == TC_ && rows == R_)                                                                            \
    return launch_rows<R_, RM_, CN_, HALF_, CG_, rows_lines(TC_)>(map_x, map_w, y, residual, m, n, k, plan.stages, word, stream);
    BW_ROWS(16, 8, 1, 1, true, 1)
    BW_ROWS(32, 8, 2, 1, false, 1)
    BW_ROWS(64, 8, 4, 1, false, 2)
    BW_ROWS(128, 8, 4, 2, false, 2)
    BW_ROWS(16, 16, 1, 1, true, 1)
    BW_ROWS(32, 16, 2, 1, false, 1)
    BW_ROWS(64, 16, 4, 1, false, 2)
    BW_ROWS(128, 16, 4, 2, false, 2)
#undef BW_ROWS
    bw::set_error("linear (32-bit): no streaming tile of %d columns for %d rows", plan.tile_cols, rows);
    return -1;
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
  // a thread per pair of the widest part (at most 1,024): a step of few rows is a chain of round trips to
  // memory (position, then the row, the table's line and the block, then the writes), not a stream
  int threads = (heads > kv_heads ? heads : kv_heads) * (hd / 2);
  threads = threads > 1024 ? 1024 : threads < 128 ? 128 : (threads + 31) / 32 * 32;
  if (n > 64) threads = 128;
  bw::launch_pdl(rope_cache_exact_kernel, dim3(n), dim3(threads), 0, stream, qkv, row_stride, pos, row_seq, cos_t, sin_t,
                 block_table, max_blocks, kcache, vcache, heads, kv_heads, hd, page, write_kv);
  return bw::launch_status();
}

// Floats of scratch that a step of single rows needs (scores and the chunks' maxima).
BW_API long long bw_f32_attention_scratch_floats(int n, int heads, int max_keys) {
  const long long stride = (static_cast<long long>(max_keys) + kScoreKeys - 1) / kScoreKeys * kScoreKeys;
  return static_cast<long long>(n) * heads * (stride + stride / kScoreKeys);
}

namespace {

template <int HD>
int launch_attention_tiles(const float* qkv, int q_stride, const float* kcache, const float* vcache, const int* block_table,
                           int max_blocks, const int* tile_seq, const int* tile_row0, const int* tile_rows, int num_tiles,
                           const int* seq_pos0, const int* seq_row0, float* out, int out_stride, int heads, int kv_heads,
                           int page, int window, float scale, cudaStream_t stream) {
  using G = TileGeometry<HD>;
  constexpr int smem = G::SmemFloats * static_cast<int>(sizeof(float));
  static_assert(smem <= 227 * 1024, "the tiles do not fit into shared memory");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tiles_exact_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      bw::set_error("attention (32-bit): cannot raise shared memory to %d: %s", smem, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  attention_tiles_exact_kernel<HD><<<dim3(heads, num_tiles), kTileThreads, smem, stream>>>(
      qkv, q_stride, kcache, vcache, block_table, max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out,
      out_stride, heads, kv_heads, page, window, scale);
  return bw::launch_status();
}

}  // namespace

// Query rows in a tile of the tiled form (what callers cut a step's rows into).
BW_API int bw_f32_attention_tile_rows() { return kTileRows; }

// out[r, h] = attention of row r's query over the cached keys of its sequence.
//   tiles given (num_tiles > 0) and some tile has more than one row: every tile (up to 16
//     consecutive rows of one sequence) is a block per head;
//   otherwise (single rows, in any order): scores by many blocks into `scratch`
//     (bw_f32_attention_scratch_floats), then the chains.
BW_API int bw_f32_attention(const float* qkv, int q_stride, const float* kcache, const float* vcache,
                            const int* block_table, int max_blocks, const int* row_seq, const int* pos,
                            const int* tile_seq, const int* tile_row0, const int* tile_rows, int num_tiles,
                            const int* seq_pos0, const int* seq_row0, float* out, int out_stride, int n, int heads,
                            int kv_heads, int hd, int page, int window, int max_keys, float scale, float* scratch,
                            long long scratch_floats, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd % 16 || hd <= 0 || hd > 256) {
    bw::set_error("attention (32-bit): head size %d is not a multiple of 16 up to 256", hd);
    return -1;
  }
  if (kv_heads <= 0 || heads % kv_heads) {
    bw::set_error("attention: %d heads are not a multiple of %d key/value heads", heads, kv_heads);
    return -1;
  }
  if (heads > 65535 || page <= 0 || q_stride % 4 || (reinterpret_cast<uintptr_t>(qkv) & 15) ||
      (reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15)) {
    bw::set_error("attention (32-bit): %d heads, page %d, row stride %d: rows must start on 16 bytes", heads, page, q_stride);
    return -1;
  }
  if (num_tiles > 0 && num_tiles < n) {  // prompt portions (perhaps beside single rows)
    if (num_tiles > 65535) {
      bw::set_error("attention (32-bit): %d query tiles exceed the grid limit", num_tiles);
      return -1;
    }
#define BW_TILES(HD_)                                                                                                  \
  case HD_:                                                                                                            \
    return launch_attention_tiles<HD_>(qkv, q_stride, kcache, vcache, block_table, max_blocks, tile_seq, tile_row0,   \
                                       tile_rows, num_tiles, seq_pos0, seq_row0, out, out_stride, heads, kv_heads,    \
                                       page, window, scale, stream)
    switch (hd) {
      BW_TILES(16);
      BW_TILES(32);
      BW_TILES(48);
      BW_TILES(64);
      BW_TILES(80);
      BW_TILES(96);
      BW_TILES(112);
      BW_TILES(128);
      BW_TILES(144);
      BW_TILES(160);
      BW_TILES(176);
      BW_TILES(192);
      BW_TILES(208);
      BW_TILES(224);
      BW_TILES(240);
      BW_TILES(256);
    }
#undef BW_TILES
    return -1;
  }
  // single rows
  const int score_stride = (max_keys + kScoreKeys - 1) / kScoreKeys * kScoreKeys;
  const int chunks = score_stride / kScoreKeys;
  if (!scratch || scratch_floats < bw_f32_attention_scratch_floats(n, heads, max_keys)) {
    bw::set_error("attention (32-bit): %lld floats of scratch for %d rows, %d heads, %d keys are too few", scratch_floats,
                  n, heads, max_keys);
    return -1;
  }
  if (chunks > 65535) {
    bw::set_error("attention (32-bit): %d keys exceed the grid limit", max_keys);
    return -1;
  }
  float* scores = scratch;
  float* chunk_max = scratch + static_cast<size_t>(n) * heads * score_stride;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  bw::launch_pdl(attention_scores_exact_kernel, dim3(n, heads, chunks), dim3(kScoreThreads), hd * sizeof(float), stream, qkv,
                 q_stride, kcache, block_table, max_blocks, row_seq, pos, heads, kv_heads, hd, page, window, scale, scores,
                 score_stride, chunk_max, chunks);
  const int weight_floats = (max_keys + 3) / 4 * 4;  // keeps the value tiles behind the weights on 16 bytes
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_values_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_values_paged_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) {
      bw::set_error("attention (32-bit): cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  // Whole value rows by pages, when there are (row, head) pairs enough to give every SM a stream
  // of values, a page of a head is a piece of a kilobyte or more, pages divide a tile, and no
  // window cuts into a page.
  const bool by_page = static_cast<long long>(n) * heads >= sms && hd <= kValueMaxSlice && window <= 0 &&
                       kValueTile % page == 0 && static_cast<long long>(page) * hd * 4 >= 1024;
  if (by_page) {
    // as many tiles on their way as 96 KB hold, six at most, two at least
    int stages = (96 * 1024) / (kValueTile * hd * static_cast<int>(sizeof(float)));
    stages = stages > kValueMaxStages ? kValueMaxStages : stages < 2 ? 2 : stages;
    const size_t smem = (static_cast<size_t>(weight_floats) + static_cast<size_t>(stages) * kValueTile * hd) * sizeof(float) +
                        2 * stages * sizeof(uint64_t);
    int* word = bw::failure_word();
    if (!word) return -1;
    if (smem <= 220 * 1024) {
      bw::launch_pdl(attention_values_paged_exact_kernel, dim3(n, heads), dim3((hd / 2 + 31) / 32 * 32 + 32), smem, stream,
                     scores, score_stride, chunk_max, chunks, vcache, block_table, max_blocks, row_seq, pos, out, out_stride,
                     heads, kv_heads, hd, page, weight_floats, stages, word);
      return bw::launch_status();
    }
  }
  // columns of the output per block: all of them, or fewer when there are too few (row, head)
  // pairs to give every SM a stream of values, and never more than a block has chain threads
  int dsplit = 1;
  while (hd / dsplit > kValueMaxSlice) dsplit *= 2;
  while (dsplit < 4 && static_cast<long long>(n) * heads * dsplit < sms && (hd / (2 * dsplit)) % 4 == 0 &&
         hd % (2 * dsplit) == 0)
    dsplit *= 2;
  if (hd % dsplit || (hd / dsplit) % 4) {
    bw::set_error("attention (32-bit): head size %d cannot be cut into %d slices of whole 16 bytes", hd, dsplit);
    return -1;
  }
  const int dslice = hd / dsplit;
  const size_t smem = (static_cast<size_t>(weight_floats) + static_cast<size_t>(kValueStages) * kValueTile * dslice) * sizeof(float);
  if (smem > 220 * 1024) {
    bw::set_error("attention (32-bit): %d keys exceed the shared-memory buffer of a row's weights", max_keys);
    return -1;
  }
  bw::launch_pdl(attention_values_exact_kernel, dim3(n, heads, dsplit), dim3(kValueThreads), smem, stream, scores,
                 score_stride, chunk_max, chunks, vcache, block_table, max_blocks, row_seq, pos, out, out_stride, heads,
                 kv_heads, hd, dslice, page, window, weight_floats);
  return bw::launch_status();
}

BW_API int bw_f32_swiglu(const float* gate_up, float* out, int n, int inter, cudaStream_t stream) {
  if (n <= 0 || inter <= 0) return 0;
  const size_t total = static_cast<size_t>(n) * inter;
  const unsigned blocks = static_cast<unsigned>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  bw::launch_pdl(swiglu_exact_kernel, dim3(blocks), dim3(256), 0, stream, gate_up, out, n, inter);
  return bw::launch_status();
}
