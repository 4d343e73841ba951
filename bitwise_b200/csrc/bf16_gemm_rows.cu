// bfloat16 matrix product for steps of few rows (decode steps, up to 16 rows):
// y[m][n] = sum_k x[m][k] * W[n][k], then what follows it (a float32 residual sum, the
// rounding to bfloat16, or SwiGLU of interleaved gate/up weights), in ONE kernel.
//
// Why a kernel of its own beside the tcgen05 one (bf16_gemm_tc.cu). With a handful of rows a
// product is a stream of weights, not arithmetic: what counts is how soon every byte of W is
// requested and how short the chain from the last byte to the stored output is. On the
// tcgen05 path a chunk of 512 k-elements is 32 MMAs that each wait about 100 ns for the one
// before (the accumulator dependency), 3.2 us per chunk however narrow the tile, and the
// chunk sums of a product that is split over the machine pass through scratch memory and a
// second kernel. Here a block per SM stays for the whole product and walks output tiles of 8
// or 16 columns. Four warps share the chunks of 8 columns (warp w takes chunks w, w + 4, ...);
// a work item is (tile, chunk): 8 KB of W per 8 columns, fetched by ONE TMA copy (a box of
// 8 rows x 8 k-tiles of 64, 128-byte swizzle) into the warp's own ring of buffers, two items
// ahead of the arithmetic (the first ones before the wait for the kernel before this one:
// weights do not depend on it). The step's rows of x are loaded once per block and stay in
// shared memory. An item's 32 k-steps run on mma.sync (m16n8k16: a dependent step every 28
// cycles, measured; a tile of 16 columns has a second set of four warps for its second half,
// so that every warp runs one chain). The chunk sums of a tile meet in shared memory, are
// added in ascending order and leave as finished outputs. No scratch, no second kernel.
//
// Same bits as every other variant of the product (tested against them): inside a chunk the
// tensor core accumulates from zero in k-steps of 16, ascending; chunk sums are added in
// float32, ascending; the residual last. That order depends on k alone, which is the
// reference's rule (src/kernels.h:4-12: one chain per output, whatever the batch).
#include <cuda.h>

#include "bw_common.cuh"

namespace {

constexpr int kChunk = 512;            // canonical summation chunk along k (as in bf16_gemm_tc.cu)
constexpr int kTileK = 64;             // k-elements of a shared-memory line (128 bytes, swizzled)
constexpr int kTilesPerChunk = kChunk / kTileK;
constexpr int kGroupBytes = 8 * kChunk * 2;  // 8 rows x one chunk: [k-tile][row][128 bytes]
constexpr int kWarps = 4;              // warps per group of 8 columns; chunk c belongs to warp c % kWarps of the group
constexpr int kStages = 2;             // buffers in a warp's ring of W items
constexpr int kSmemLimit = 227 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for a phase of a barrier; when the limit runs out the thread raises the
// library's failure word and the kernel goes on (its outputs are then worthless, and the host
// learns of it).
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, int* failure) {
  bw::mbar_wait_bounded(bar, parity, reinterpret_cast<volatile uint32_t*>(failure));
}
// One box of the view (64 k-elements, rows, k-tiles) of a row-major matrix: the box's rows
// from `row` on, 8 k-tiles from `ktile` on, laid out [k-tile][row][128 bytes] with the
// 128-byte swizzle; what lies outside the matrix arrives as zeros. The first coordinate is 0.
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, int row, int ktile, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(row), "r"(ktile), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// EPI 0: y = product in bfloat16.  EPI 1: W holds gate/up rows interleaved in blocks of 64 and
// y[m][n / 2] = SwiGLU (bfloat16); a tile is 8 outputs (8 gate rows and their 8 up rows, NT 2).
// EPI 2: y = (residual +) product in float32.
// EPI 3: W is the fused q/k/v projection; the tile's two groups are the two halves of a head
// (columns i .. i + 7 and i + hd / 2 .. of it), so that a thread holds both partners of a
// rotation: the outputs are rounded to bfloat16, q and k are rotated by their row's position,
// q goes to y, k and v go straight into their page of the cache (what rope_cache_bf16_kernel
// does to a stored product, with its arithmetic: same bits).
// ROWS16: up to 16 rows (else up to 8: the upper half of the tensor core's 16 rows is zero).
// NT: groups of 8 output columns per tile (1 or 2), each with kWarps warps of its own.
//
// Shared memory (1024-byte aligned for the swizzle): the rows of x [chunk][k-tile][R][128 B],
// the rings [warp][stage][k-tile][8][128 B], the barriers, and the chunk sums of two tiles in
// turn [2][chunk][NT][R][8].
struct RopeCache {
  const int* pos;            // position of every row
  const int* row_seq;        // its sequence's row of the block table
  const float* cos_t;        // [positions][hd / 2], or null: nothing is rotated
  const float* sin_t;
  const int* block_table;
  int max_blocks;
  __nv_bfloat16* kcache;     // [pages][kv_heads][page][hd]
  __nv_bfloat16* vcache;
  int heads, kv_heads, hd, page, write_kv;
};

template <int EPI, bool ROWS16, int NT>
__global__ void __launch_bounds__(NT * kWarps * 32)
linear_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, void* Y,
                   const float* residual, int M, int N, int K, int tiles, RopeCache rc, int* failure) {
  static_assert(EPI != 3 || NT == 2, "a rotation needs both halves of a head in the tile");
  constexpr int R = ROWS16 ? 16 : 8;
  constexpr int kItemBytes = kGroupBytes;  // what a warp fetches per (tile, chunk): its group's 8 rows
  constexpr int kThreads = NT * kWarps * 32;
  constexpr int kXChunkBytes = R * kChunk * 2;
  constexpr int kOutputs = R * NT * 8;                                // outputs of a tile, chunk sums of one chunk
  constexpr int kMine = (kOutputs + kThreads - 1) / kThreads;         // outputs per thread in the epilogue
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = bw::smem_align_1024(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp_all = tid >> 5;
  const int grp = warp_all / kWarps, warp = warp_all % kWarps;  // group of 8 columns; which chunks of it
  const int num_chunks = (K + kChunk - 1) / kChunk;
  unsigned char* xs = smem;
  unsigned char* ring = xs + num_chunks * kXChunkBytes + warp_all * (kStages * kItemBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(xs + num_chunks * kXChunkBytes + NT * kWarps * kStages * kItemBytes);
  uint64_t* wbar = bars + warp_all * kStages;            // one barrier per buffer of this warp's ring
  uint64_t* xbar = bars + NT * kWarps * kStages + warp;  // the chunks of x that this warp works on
  float* part = reinterpret_cast<float*>(bars + NT * kWarps * kStages + kWarps);

  if (tid == 0) {
    for (int i = 0; i < NT * kWarps * kStages + kWarps; ++i) mbar_init(bars + i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // This warp's items: for tile = blockIdx.x, + gridDim.x, ...: chunks warp, warp + kWarps, ...
  const int my_chunks = warp < num_chunks ? (num_chunks - warp + kWarps - 1) / kWarps : 0;
  // Requests item (tile, chunk) into buffer `stage`: one box of this warp's group of 8 rows of W
  // (with interleaved gate/up weights the up rows of 8 outputs lie 64 rows after their gate rows).
  auto request = [&](int tile, int chunk, int stage) {
    if (lane == 0) {
      int row;
      if (EPI == 1) {
        const int c0 = tile * 8;
        row = 128 * (c0 >> 6) + (c0 & 63) + 64 * grp;
      } else if (EPI == 3) {
        const int per_head = rc.hd >> 4;  // tiles per head
        const int head = tile / per_head;
        row = head * rc.hd + grp * (rc.hd >> 1) + (tile - head * per_head) * 8;
      } else {
        row = (tile * NT + grp) * 8;
      }
      mbar_expect_tx(wbar + stage, kItemBytes);
      tma_load_box(ring + stage * kItemBytes, &map_w, row, chunk * kTilesPerChunk, wbar + stage);
    }
  };

  // the first items of the ring: weights do not depend on the kernel before this one
  int req_tile = blockIdx.x, req_cc = 0;  // next item to request: tile and index among this warp's chunks
  if (my_chunks > 0) {
    for (int s = 0; s < kStages && req_tile < tiles; ++s) {
      request(req_tile, warp + req_cc * kWarps, s);
      if (++req_cc == my_chunks) req_cc = 0, req_tile += gridDim.x;
    }
  }
  bw::pdl_launch();
  bw::pdl_wait();
  // x, once per block: the warps of the first group bring the chunks they work on, which are
  // those of their namesakes in the other group too (rows beyond the step's arrive as zeros)
  if (my_chunks > 0) {
    if (lane == 0 && grp == 0) {
      mbar_expect_tx(xbar, static_cast<uint32_t>(my_chunks * kXChunkBytes));
      for (int cc = 0; cc < my_chunks; ++cc) {
        const int chunk = warp + cc * kWarps;
        tma_load_box(xs + chunk * kXChunkBytes, &map_x, 0, chunk * kTilesPerChunk, xbar);
      }
    }
    mbar_wait(xbar, 0, failure);
  }

  // Shared-memory addresses of this lane's ldmatrix rows. A line of 128 bytes holds 64
  // k-elements of one row; its 16-byte pieces are swizzled with the row's low three bits.
  // W (and x with up to 8 rows): one ldmatrix brings rows 0-7 of four k-blocks of 8, both halves
  // of two k-steps; lane l addresses row l % 8 of k-block l / 8.
  const int lrow = lane & 7, lblk = lane >> 3;
  const uint32_t b_off = lrow * 128;
  // x with 16 rows: a: rows 0-7 / 8-15 of k 0-7, then of k 8-15 of one step
  const int arow = ROWS16 ? lrow + ((lane >> 3) & 1) * 8 : lrow;
  const int ablk = ROWS16 ? (lane >> 4) : lblk;
  const uint32_t a_off = arow * 128;

  uint32_t used = 0;  // items consumed by this warp
  int flip = 0;       // which half of the chunk sums this tile uses
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, flip ^= 1) {
    // the residual of this thread's outputs is asked for now and used after the arithmetic
    float res[kMine];
#pragma unroll
    for (int e = 0; e < kMine; ++e) {
      res[e] = 0.0f;
      if (EPI == 2 && residual) {
        const int o = tid + e * kThreads;
        const int r = o / (NT * 8), n = tile * (NT * 8) + o % (NT * 8);
        if (o < kOutputs && r < M && n < N) res[e] = residual[static_cast<size_t>(r) * N + n];
      }
    }
    float* sums = part + flip * num_chunks * kOutputs;
    for (int cc = 0; cc < my_chunks; ++cc, ++used) {
      const int chunk = warp + cc * kWarps;
      const int stage = used % kStages;
      const uint32_t wb = smem_u32(ring + stage * kItemBytes) + b_off;
      const uint32_t xa = smem_u32(xs + chunk * kXChunkBytes) + a_off;
      mbar_wait(wbar + stage, (used / kStages) & 1, failure);
      const int k_here = min(kChunk, K - chunk * kChunk);
      const int pairs = (k_here / kTileK) * 2;  // pairs of k-steps of 16 (k is a multiple of 64)
      float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      // fragments of pair p: k-tile p / 2, k-blocks 4 (p % 2) .. + 3 of it; those of the next
      // pair are fetched before this pair's MMAs are issued
      uint32_t a[2][ROWS16 ? 8 : 4], b[2][4];
      auto fetch = [&](int p, int slot) {
        const int kt = p >> 1, q0 = (p & 1) * 4;
        if (ROWS16) {
          uint32_t lo[4], hi[4];
          ldmatrix_x4(lo, xa + kt * (R * 128) + (((q0 + ablk) ^ lrow) << 4));
          ldmatrix_x4(hi, xa + kt * (R * 128) + (((q0 + 2 + ablk) ^ lrow) << 4));
#pragma unroll
          for (int e = 0; e < 4; ++e) a[slot][e] = lo[e], a[slot][4 + e] = hi[e];
        } else {
          uint32_t v[4];
          ldmatrix_x4(v, xa + kt * (R * 128) + (((q0 + ablk) ^ lrow) << 4));
#pragma unroll
          for (int e = 0; e < 4; ++e) a[slot][e] = v[e];
        }
        ldmatrix_x4(b[slot], wb + kt * 1024 + (((q0 + lblk) ^ lrow) << 4));
      };
      auto steps = [&](int slot) {
        if (ROWS16) {
          mma_bf16(d, a[slot][0], a[slot][1], a[slot][2], a[slot][3], b[slot][0], b[slot][1]);
          mma_bf16(d, a[slot][4], a[slot][5], a[slot][6], a[slot][7], b[slot][2], b[slot][3]);
        } else {
          mma_bf16(d, a[slot][0], 0u, a[slot][1], 0u, b[slot][0], b[slot][1]);
          mma_bf16(d, a[slot][2], 0u, a[slot][3], 0u, b[slot][2], b[slot][3]);
        }
      };
      fetch(0, 0);
      for (int p = 0; p < pairs; p += 2) {  // pairs is even
        fetch(p + 1, 1);
        steps(0);
        if (p + 2 < pairs) fetch(p + 2, 0);
        steps(1);
      }
      // The buffer is free: the item two ahead takes it. Every ldmatrix of this item has
      // delivered (the MMAs that consumed them were issued), so the copy may overwrite it.
      __syncwarp();
      if (req_tile < tiles) {
        request(req_tile, warp + req_cc * kWarps, stage);
        if (++req_cc == my_chunks) req_cc = 0, req_tile += gridDim.x;
      }
      // chunk sums: d[0..1] are columns 2 (lane % 4) + {0, 1} of row lane / 4 of this group,
      // d[2..3] of row lane / 4 + 8
      {
        float* mine = sums + chunk * kOutputs + grp * (R * 8) + (lane >> 2) * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2*>(mine) = make_float2(d[0], d[1]);
        if (ROWS16) *reinterpret_cast<float2*>(mine + 64) = make_float2(d[2], d[3]);
      }
    }
    __syncthreads();  // the chunk sums of this tile are complete (the next tile writes the other half)

    // the ordered sum of the chunk sums, then what follows the product
    auto chunk_sum = [&](int t, int r, int j) {
      const float* p = sums + t * (R * 8) + r * 8 + j;
      float v = p[0];
      for (int c = 1; c < num_chunks; ++c) v = v + p[c * kOutputs];
      return v;
    };
    if (EPI == 3) {
      const int per_head = rc.hd >> 4, half = rc.hd >> 1;
      const int head = tile / per_head, i0 = (tile - head * per_head) * 8;  // head among q, k, v heads
      for (int o = tid; o < R * 8; o += kThreads) {
        const int r = o >> 3, i = i0 + (o & 7);
        if (r >= M) continue;
        const float x1 = __bfloat162float(__float2bfloat16_rn(chunk_sum(0, r, o & 7)));
        const float x2 = __bfloat162float(__float2bfloat16_rn(chunk_sum(1, r, o & 7)));
        const int p = rc.pos[r];
        float o1 = x1, o2 = x2;
        if (rc.cos_t && head < rc.heads + rc.kv_heads) {
          const float c = rc.cos_t[static_cast<size_t>(p) * half + i], sn = rc.sin_t[static_cast<size_t>(p) * half + i];
          o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
          o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
        }
        if (head < rc.heads) {
          __nv_bfloat16* q = static_cast<__nv_bfloat16*>(Y) + static_cast<size_t>(r) * N + head * rc.hd + i;
          q[0] = __float2bfloat16_rn(o1);
          q[half] = __float2bfloat16_rn(o2);
        } else if (rc.write_kv) {
          const bool is_k = head < rc.heads + rc.kv_heads;
          const int kvh = head - rc.heads - (is_k ? 0 : rc.kv_heads);
          const int blk = rc.block_table[static_cast<size_t>(rc.row_seq[r]) * rc.max_blocks + p / rc.page];
          __nv_bfloat16* dst = (is_k ? rc.kcache : rc.vcache) +
                               ((static_cast<size_t>(blk) * rc.kv_heads + kvh) * rc.page + p % rc.page) * rc.hd + i;
          dst[0] = __float2bfloat16_rn(o1);
          dst[half] = __float2bfloat16_rn(o2);
        }
      }
    } else if (EPI == 1) {
      const int inter = N / 2;
      for (int o = tid; o < R * 8; o += kThreads) {
        const int r = o >> 3, j = o & 7;
        if (r >= M) continue;
        const float g = __bfloat162float(__float2bfloat16_rn(chunk_sum(0, r, j)));
        const float u = __bfloat162float(__float2bfloat16_rn(chunk_sum(1, r, j)));
        static_cast<__nv_bfloat16*>(Y)[static_cast<size_t>(r) * inter + tile * 8 + j] =
            __float2bfloat16_rn(bw::swiglu_one(g, u));
      }
    } else {
#pragma unroll
      for (int e = 0; e < kMine; ++e) {
        const int o = tid + e * kThreads;
        const int r = o / (NT * 8), cj = o % (NT * 8);
        const int n = tile * (NT * 8) + cj;
        if (o >= kOutputs || r >= M || n >= N) continue;
        float v = chunk_sum(cj >> 3, r, cj & 7);
        const size_t at = static_cast<size_t>(r) * N + n;
        if (EPI == 2) {
          if (residual) v = res[e] + v;
          static_cast<float*>(Y)[at] = v;
        } else {
          static_cast<__nv_bfloat16*>(Y)[at] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

int g_rows_enabled = 1;

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled rows_encoder() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

// The view (64 k-elements, rows, k-tiles of 64) of a row-major [rows][k] bfloat16 matrix, k a
// multiple of 64; a box takes `box_rows` rows and the 8 k-tiles of a chunk.
bool rows_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  EncodeTiled enc = rows_encoder();
  if (!enc) return false;
  const cuuint64_t dims[3] = {kTileK, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k / kTileK)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 2, kTileK * 2};
  const cuuint32_t box[3] = {kTileK, static_cast<cuuint32_t>(box_rows), kTilesPerChunk};
  const cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct RowsShape {
  int nt, rows16, tiles;
  size_t smem;
  unsigned grid;
};

int rows_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

// How a product of m rows runs here, or false when it has to take another path (more than 16
// rows, k no multiple of 64, or k so long that the step's rows of x do not fit into shared
// memory beside the rings).
bool rows_shape(int m, int n, int k, bool swiglu, RowsShape* s) {
  if (m < 1 || m > 16 || k < kTileK || k % kTileK || n < 1) return false;
  const long long chunks = (k + kChunk - 1) / kChunk;
  s->rows16 = m > 8;
  const int R = s->rows16 ? 16 : 8;
  for (int nt = 2; nt >= 1; --nt) {
    if (swiglu && nt != 2) break;
    const long long smem = 1024 + chunks * R * kChunk * 2 + static_cast<long long>(kWarps) * kStages * nt * kGroupBytes +
                           (nt * kWarps * kStages + kWarps) * 8 + 2 * chunks * nt * R * 8 * 4;
    if (smem > kSmemLimit) continue;
    const long long tiles = swiglu ? n / 16 : (n + nt * 8 - 1) / (nt * 8);
    if (tiles > 0x7fffffffLL) return false;
    const long long resident = static_cast<long long>(rows_sm_count()) * (kSmemLimit / smem);
    s->nt = nt;
    s->tiles = static_cast<int>(tiles);
    s->smem = static_cast<size_t>(smem);
    s->grid = static_cast<unsigned>(tiles < resident ? tiles : resident);
    return true;
  }
  return false;
}

template <int EPI, bool ROWS16, int NT>
int launch_rows(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, const float* residual, int m, int n, int k,
                const RowsShape& s, cudaStream_t stream, const RopeCache& rc = RopeCache{}) {
  auto kernel = linear_rows_kernel<EPI, ROWS16, NT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) {
      bw::set_error("linear (few rows): cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  CUtensorMap map_x, map_w;
  if (!rows_map(&map_x, x, m, k, ROWS16 ? 16 : 8) || !rows_map(&map_w, w, n, k, 8)) {
    bw::set_error("linear (few rows): cuTensorMapEncodeTiled refused [%d x %d] / [%d x %d]", m, k, n, k);
    return -1;
  }
  int* word = bw::failure_word();
  if (!word) return -1;
  bw::launch_pdl(kernel, dim3(s.grid), dim3(NT * kWarps * 32), s.smem, stream, map_x, map_w, y, residual, m, n, k, s.tiles, rc,
                 word);
  return bw::launch_status();
}

template <int EPI>
int launch_rows_epi(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, const float* residual, int m, int n, int k,
                    const RowsShape& s, cudaStream_t stream) {
  if (s.nt == 2)
    return s.rows16 ? launch_rows<EPI, true, 2>(x, w, y, residual, m, n, k, s, stream)
                    : launch_rows<EPI, false, 2>(x, w, y, residual, m, n, k, s, stream);
  if (EPI == 1) return -1;  // SwiGLU tiles always hold two groups
  return s.rows16 ? launch_rows<EPI == 1 ? 0 : EPI, true, 1>(x, w, y, residual, m, n, k, s, stream)
                  : launch_rows<EPI == 1 ? 0 : EPI, false, 1>(x, w, y, residual, m, n, k, s, stream);
}

}  // namespace

// Switches this path off (0) or on (1, the default); returns the previous setting. Tests and
// measurements compare it with the tcgen05 path bit for bit.
BW_API int bw_bf16_linear_rows_enable(int on) {
  const int before = g_rows_enabled;
  g_rows_enabled = on ? 1 : 0;
  return before;
}

// Whether a product of this shape runs on this path (rows that start on 16 bytes, at most 16
// rows, k a multiple of 64 and short enough for the step's rows of x to stay in shared memory).
BW_API int bw_bf16_linear_rows_usable(const void* x, const void* w, int m, int n, int k, int swiglu) {
  RowsShape s;
  return g_rows_enabled && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0) &&
         (!swiglu || n % 128 == 0) && rows_shape(m, n, k, swiglu != 0, &s) && rows_encoder() != nullptr;
}

// y_kind 0: y bfloat16 [m][n].  1: SwiGLU of interleaved gate/up weights, y bfloat16 [m][n / 2].
// 2: y float32 [m][n] = (residual +) product; y may alias residual.
BW_API int bw_bf16_linear_rows(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_kind, const float* residual,
                               int m, int n, int k, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  RowsShape s;
  if (!bw_bf16_linear_rows_usable(x, w, m, n, k, y_kind == 1) || !rows_shape(m, n, k, y_kind == 1, &s)) {
    bw::set_error("linear (few rows): shape [%d x %d] x [%d x %d] is not for this path", m, k, n, k);
    return -1;
  }
  if (y_kind == 1) return launch_rows_epi<1>(x, w, y, nullptr, m, n, k, s, stream);
  if (y_kind == 2) return launch_rows_epi<2>(x, w, y, residual, m, n, k, s, stream);
  return launch_rows_epi<0>(x, w, y, nullptr, m, n, k, s, stream);
}

// Whether the fused q/k/v projection of a step can rotate and store its outputs itself
// (bw_bf16_linear_rows_rope): a shape of this path whose tiles hold both halves of a head.
BW_API int bw_bf16_linear_rows_rope_usable(const void* x, const void* w, int m, int n, int k, int heads, int kv_heads,
                                           int hd) {
  RowsShape s;
  return g_rows_enabled && hd >= 16 && hd % 16 == 0 && heads > 0 && kv_heads > 0 && n == (heads + 2 * kv_heads) * hd &&
         (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0) &&
         rows_shape(m, n, k, true, &s) && rows_encoder() != nullptr;
}

// qkv = x W^T for the fused q/k/v weights, then what bw_bf16_rope_cache does to it, in the same
// kernel: q rotated into qkv[:, :heads * hd]; k rotated and v as it is into the pages
// block_table[row_seq[r]][pos[r] / page] of the cache (not when write_kv is 0; the k and v
// columns of qkv are not written). cos_t / sin_t null: nothing is rotated.
BW_API int bw_bf16_linear_rows_rope(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* qkv, int m, int n, int k,
                                    const int* pos, const int* row_seq, const float* cos_t, const float* sin_t,
                                    const int* block_table, int max_blocks, __nv_bfloat16* kcache, __nv_bfloat16* vcache,
                                    int heads, int kv_heads, int hd, int page, int write_kv, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  RowsShape s;
  if (!bw_bf16_linear_rows_rope_usable(x, w, m, n, k, heads, kv_heads, hd) || !rows_shape(m, n, k, true, &s) || page <= 0) {
    bw::set_error("linear with rotation (few rows): shape [%d x %d] x [%d x %d], %d/%d heads of %d is not for this path", m,
                  k, n, k, heads, kv_heads, hd);
    return -1;
  }
  const RopeCache rc{pos, row_seq, cos_t, sin_t, block_table, max_blocks, kcache, vcache, heads, kv_heads, hd, page, write_kv};
  return s.rows16 ? launch_rows<3, true, 2>(x, w, qkv, nullptr, m, n, k, s, stream, rc)
                  : launch_rows<3, false, 2>(x, w, qkv, nullptr, m, n, k, s, stream, rc);
}
