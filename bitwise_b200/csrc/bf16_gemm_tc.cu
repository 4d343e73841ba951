// The bfloat16 matrix product on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands brought into shared memory by TMA. One summation
// order for every batch size: chunks of 512 along k at fixed positions, inside a chunk the
// tensor core accumulates in steps of 16 along k, the chunk sums are added in float32 in
// ascending order. A product with many output tiles walks the chunks of a tile inside one
// block ("whole" mode). A product with few output tiles and few rows (decode steps) gives
// every (tile, chunk) pair to a block as a work item of its own ("split" mode), so that the
// weights stream from all SMs; the chunk sums go to scratch memory and a second small kernel
// adds them in the same ascending order.
//
// One thread block computes one 128 x 128 output tile with six warps:
//   warp 0   one thread issues the TMA loads of the x tile and the W tile, 64 k-elements per
//            stage (128-byte rows, 128-byte swizzle), into a ring of stages
//   warp 1   one thread issues tcgen05.mma (M 128, N 128, K 16, four per stage) into one of
//            two accumulators in tensor memory; a commit frees the stage, and at the end of a
//            chunk another commit hands the accumulator to the epilogue
//   warps 2-5  read the finished chunk sum from tensor memory (each thread one row, 32 columns
//            at a time) and add it to the running total in registers, while the tensor core
//            already works on the next chunk in the other accumulator; after the last chunk
//            they add the residual and store.
// The kernel is persistent: one block per SM (6 stages of 32 KB) takes output tiles round-robin,
// and because loads, MMAs and the epilogue each walk the tile sequence on their own, the store
// of one tile overlaps the main loop of the next.
//
// Every wait on an mbarrier is bounded: after a limit the thread raises a flag in global
// memory and the block drains and returns instead of hanging; the host reports the flag.
#include <cuda.h>

#include "bw_common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64;  // BN: columns one epilogue thread carries; a wide tile has 2 BN
constexpr int kChunk = 512;
constexpr int kTilesPerChunk = kChunk / BK;
constexpr int kSmemBudget = 200 * 1024;        // ring of stages (plus barriers) per block

// The x tile of a stage holds A_ROWS rows: 128 for large batches, fewer for small ones. The
// tensor core always reads 128 rows; with a shorter tile the rows beyond it are whatever lies
// behind in shared memory (the ring is padded so that the read stays inside the block's
// allocation). Rows are independent in a matrix product, so this only fills accumulator
// lanes that are never read, and it leaves room for more stages: a decode step is bound by
// how many bytes of weights an SM keeps in flight.
//
// The W tile of a stage holds w_rows rows: 128 (256 for a wide tile), or fewer, in steps of
// 16, when a product has too few columns to give every SM a 128-column tile: a decode step
// then runs more, narrower tiles instead of cutting k further.
constexpr int kMaxStages = 32;
struct RingShape {
  int tile_bytes_x, stage_bytes, stages, pad_bytes, ring_bytes;
};
__host__ __device__ inline RingShape ring_shape(int a_rows, int w_rows) {
  RingShape r;
  r.tile_bytes_x = a_rows * BK * 2;
  r.stage_bytes = r.tile_bytes_x + w_rows * BK * 2;
  r.pad_bytes = (BM - a_rows) * BK * 2;  // behind the last stage
  const int fit = (kSmemBudget - r.pad_bytes) / r.stage_bytes;
  r.stages = fit > kMaxStages ? kMaxStages : fit;
  r.ring_bytes = r.stages * r.stage_bytes + r.pad_bytes;
  return r;
}

struct __align__(8) Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false when the limit ran out (or another thread of the block already gave up).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* failed) {
  return bw::mbar_wait_bounded(bar, parity, failed);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, written by
// TMA with the 128-byte swizzle: start address / 16 in bits 0-13, leading byte offset (unused
// for swizzled K-major layouts, set to 1) in bits 16-29, stride byte offset 1024 / 16 (eight
// rows of 128 bytes) in bits 32-45, descriptor version 1 in bits 46-47, layout type 2
// (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor of kind::f16: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9
// and 10-12 = 1), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- two blocks on one tile (cta_group::2) ----------------------------------------------
// A cluster of two blocks computes a 256 x 256 tile: each block loads 128 rows of x and 128
// rows of W per stage; one tcgen05.mma issued by the block of rank 0 reads both blocks'
// shared memory (M 256: 128 rows per block, N 256: 128 W rows from each block) and writes
// each block's 128 x 256 part into that block's own tensor memory. Per flop a block takes
// in a third less from shared memory than with a 128 x 256 tile of its own.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of the same shared-memory location in the block of the given rank
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a block of the pair; the bytes are counted on the barrier at `bar_cluster_addr`,
// which lies in the block of rank 0
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>((2 * BM) >> 4) << 24);
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at the same offset in both blocks of the pair once the MMAs issued
// so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 32-byte accesses: a thread of the epilogue owns a row, so a warp's store touches 32 rows;
// whole 32-byte sectors keep the memory system from merging partial ones.
__device__ __forceinline__ void st256(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void ld256(const void* p, uint32_t (&v)[8]) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Second half of split mode: y[m][n] = residual + ((p0 + p1) + p2) + ..., the chunk sums taken
// in ascending order. One thread per output; the loads of eight chunks are issued together,
// the additions stay in order.
__global__ void reduce_chunks_kernel(const float* __restrict__ partials, int num_chunks, void* Y, int y_is_f32,
                                     const float* residual, int M, int N) {
  bw::pdl_enter();
  const size_t total = static_cast<size_t>(M) * N;
  const size_t o = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (o >= total) return;
  float v = 0.0f;
  for (int c0 = 0; c0 < num_chunks; c0 += 8) {
    float p[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] = (c0 + e < num_chunks) ? __ldcg(partials + (c0 + e) * total + o) : 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (c0 + e < num_chunks) v = (c0 + e == 0) ? p[e] : v + p[e];
  }
  if (residual) v = residual[o] + v;
  if (y_is_f32)
    static_cast<float*>(Y)[o] = v;
  else
    static_cast<__nv_bfloat16*>(Y)[o] = __float2bfloat16_rn(v);
}

// The ordered sum of the chunk sums of one output (shared by the reduce kernels below).
__device__ __forceinline__ float ordered_chunk_sum(const float* __restrict__ partials, int num_chunks, size_t plane,
                                                   size_t o) {
  float v = 0.0f;
  for (int c0 = 0; c0 < num_chunks; c0 += 8) {
    float p[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] = (c0 + e < num_chunks) ? __ldcg(partials + (c0 + e) * plane + o) : 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (c0 + e < num_chunks) v = (c0 + e == 0) ? p[e] : v + p[e];
  }
  return v;
}

// Split mode of the gate/up product with SwiGLU: weights are interleaved in blocks of 64 rows
// (64 gate rows, then the 64 up rows of the same indices), so output c of a row takes the
// gate at column 128 (c / 64) + c % 64 and the up value 64 columns further. Gate and up are
// rounded to bfloat16 first, as if the product had been stored, then combined.
__global__ void reduce_swiglu_kernel(const float* __restrict__ partials, int num_chunks, __nv_bfloat16* __restrict__ H,
                                     int M, int N) {
  bw::pdl_enter();
  const int inter = N / 2;
  const size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<size_t>(M) * inter) return;
  const int r = static_cast<int>(idx / inter), c = static_cast<int>(idx - static_cast<size_t>(r) * inter);
  const size_t plane = static_cast<size_t>(M) * N;
  const size_t og = static_cast<size_t>(r) * N + 128 * (c / 64) + (c % 64);
  const float g = __bfloat162float(__float2bfloat16_rn(ordered_chunk_sum(partials, num_chunks, plane, og)));
  const float u = __bfloat162float(__float2bfloat16_rn(ordered_chunk_sum(partials, num_chunks, plane, og + 64)));
  H[idx] = __float2bfloat16_rn(bw::swiglu_one(g, u));
}

// EPI 0: y = product in bfloat16.  EPI 2: y = (residual +) product in float32.  EPI 1 (whole
// mode only): the product is the interleaved gate/up projection and y[m][n / 2] = SwiGLU of it
// (bfloat16). In split mode the kernel writes chunk sums and the second kernel finishes.
//
// A wide tile has no path for pieces that are cut by the matrix edge or that do not start on
// 32 bytes (the path costs registers that the totals need): the host gives wide tiles only
// products with n a multiple of 64 and outputs that start on 32 bytes.
//
// WIDE: the output tile is 128 x 256 instead of 128 x 128 and sixteen epilogue warps share it
// (one row x 64 columns per thread). A wide tile needs a third less operand traffic per flop.
// Large batches are bound by how fast a chunk sum leaves tensor memory: the tensor core may
// start chunk c + 2 only when the epilogue has read chunk c out of that accumulator, so the
// read is spread over many warps, 32 columns per tcgen05.ld, and the totals of a thread (64)
// stay in registers.
//
// PAIR (with WIDE, whole mode): two blocks of a cluster share a 256 x 256 tile, see above.
template <bool SPLIT, int A_ROWS, int EPI, bool WIDE, bool PAIR>
__global__ void __launch_bounds__(WIDE ? 384 : 192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, void* Y,
               int y_is_f32, const float* residual, int M, int N, int K, int* error_flag, float* partials, int bn) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the swizzled tiles want 1024-byte alignment
  unsigned char* tiles = bw::smem_align_1024(smem_raw);
  static_assert(!PAIR || (WIDE && !SPLIT && A_ROWS == BM), "a pair works on wide tiles in whole mode");
  constexpr int BNT = WIDE ? 2 * BN : BN;   // columns of this block's accumulators
  constexpr int BNW = PAIR ? BN : BNT;      // W rows this block loads per stage
  constexpr int BMT = PAIR ? 2 * BM : BM;   // rows of a work item's output tile
  constexpr int kEpiWarps = WIDE ? 8 : 4;
  constexpr int kFirstEpiWarp = WIDE ? 4 : 2;  // wide: warps 0-3 are one warpgroup (loader, MMA, two idle)
  constexpr int PW = 64;                    // columns of one of the two pieces an epilogue thread owns
  constexpr int LDW = WIDE ? 64 : 32;       // columns per tcgen05.ld (what the register budget allows)
  constexpr int kTmemColsT = 2 * BNT;  // two accumulators
  const int bt = WIDE ? BNT : bn;           // columns of a work item's tile (bn: 16 .. 128 in steps of 16)
  const RingShape ring = ring_shape(A_ROWS, WIDE ? BNW : bn);
  const int kStages = ring.stages, kStageBytes = ring.stage_bytes, kTileBytesX = ring.tile_bytes_x;
  Barriers* bars = reinterpret_cast<Barriers*>(tiles + ring.ring_bytes);
  volatile uint32_t* failed = &bars->failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = (K + BK - 1) / BK;          // k-tiles of one output tile
  const int num_chunks = (K + kChunk - 1) / kChunk;
  const int m_blocks = (M + BMT - 1) / BMT, n_blocks = (N + bt - 1) / bt;
  // a pair is one worker: both blocks walk the same items, each on its own 128 rows
  const uint32_t rank = PAIR ? cluster_rank() : 0;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // Work items are dealt round-robin to the resident blocks and the three roles below walk
  // the same sequence of items. Whole mode: item t is the output tile with rows of block
  // t % m_blocks and columns of block t / m_blocks, all its chunks (blocks that run at the same
  // time share W tiles through L2). Split mode (one block of rows): item t is chunk
  // t % num_chunks of the output tile with columns of block t / num_chunks.
  const int out_tiles = SPLIT ? n_blocks * num_chunks : m_blocks * n_blocks;
  auto item_m0 = [&](int t) { return SPLIT ? 0 : (t % m_blocks) * BMT + static_cast<int>(rank) * BM; };
  auto item_n0 = [&](int t) { return SPLIT ? (t / num_chunks) * bt : (t / m_blocks) * bt; };
  auto item_c0 = [&](int t) { return SPLIT ? t % num_chunks : 0; };
  auto item_c1 = [&](int t) { return SPLIT ? t % num_chunks + 1 : num_chunks; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], PAIR ? 2 * kEpiWarps : kEpiWarps);  // one arrival per epilogue warp
    }
    bars->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // this warp owns the tensor-memory allocation (in a pair: the same warp of both blocks)
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                   "n"(kTmemColsT)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                   "n"(kTmemColsT)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  fence_before_sync();
  if (PAIR)
    cluster_sync_all();  // the other block's barriers exist before anything arrives on them
  else
    __syncthreads();
  fence_after_sync();
  // Barriers and tensor memory are set up. The next kernel may be set up from now on; this
  // one waits for the kernel before it where it first touches data that kernel may have
  // written: the loader before its first x tile, the epilogue before it reads or writes.
  bw::pdl_launch();
  const uint32_t tmem_base = bars->tmem_base;
  // Wide tiles: the epilogue threads carry 128 running totals and the values in flight from
  // tensor memory; the loader and MMA warps need little. Registers move from the first
  // warpgroup to the two epilogue warpgroups (384 threads start with 168 each).
  if (warp < kFirstEpiWarp) {
  if (WIDE) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: the W tiles of the first
      // round of the ring are requested at once, the wait for the previous kernel comes
      // after, then the x tiles of those stages follow. Later stages load both together.
      uint32_t it = 0;  // k-tiles issued so far, over all output tiles of this block
      bool ok = true, waited = false;
      // In a pair both blocks' loads are counted on the "full" barrier of rank 0, which
      // expects the bytes of both; each block waits on its own "empty" barrier.
      auto expect = [&](int s) {
        if (!PAIR)
          mbar_expect_tx(&bars->full[s], kStageBytes);
        else if (rank == 0)
          mbar_expect_tx(&bars->full[s], 2 * kStageBytes);
      };
      auto load = [&](void* dst, const CUtensorMap* map, int x, int y, int s) {
        if (PAIR)
          tma_load_2d_pair(dst, map, x, y, peer_addr(smem_u32(&bars->full[s]), 0));
        else
          tma_load_2d(dst, map, x, y, &bars->full[s]);
      };
      for (int tile = worker; tile < out_tiles && ok; tile += workers) {
        const int m0 = item_m0(tile), n0 = item_n0(tile) + (PAIR ? static_cast<int>(rank) * BN : 0);
        const int kt0 = item_c0(tile) * kTilesPerChunk, kt1 = min(num_tiles, item_c1(tile) * kTilesPerChunk);
        int kt = kt0;
        if (!waited) {  // first item of this block
          const int early = min(kt1 - kt0, kStages);
          for (int e = 0; e < early; ++e) {
            unsigned char* a = tiles + e * kStageBytes;
            expect(e);
            load(a + kTileBytesX, &map_w, (kt0 + e) * BK, n0, e);
          }
          bw::pdl_wait();
          waited = true;
          for (int e = 0; e < early; ++e) load(tiles + e * kStageBytes, &map_x, (kt0 + e) * BK, m0, e);
          kt += early;
          it += early;
        }
        for (; kt < kt1; ++kt, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          if (round > 0 && !mbar_wait(&bars->empty[s], (round - 1) & 1, failed)) {
            ok = false;
            break;
          }
          unsigned char* a = tiles + s * kStageBytes;
          expect(s);
          load(a, &map_x, kt * BK, m0, s);
          load(a + kTileBytesX, &map_w, kt * BK, n0, s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // in a pair the block of rank 0 issues for both
      uint32_t it = 0, gc = 0;  // k-tiles and chunks consumed so far
      bool ok = true;
      for (int tile = worker; tile < out_tiles && ok; tile += workers) {
        for (int c = item_c0(tile); c < item_c1(tile) && ok; ++c, ++gc) {
          const int buf = gc & 1;
          const uint32_t use = gc >> 1;  // how often this accumulator was used before
          if (use > 0 && !mbar_wait(&bars->acc_empty[buf], (use - 1) & 1, failed)) {
            ok = false;
            break;
          }
          fence_after_sync();
          const uint32_t d = tmem_base + buf * BNT;
          const int t_begin = c * kTilesPerChunk, t_end = min(num_tiles, t_begin + kTilesPerChunk);
          for (int kt = t_begin; kt < t_end; ++kt, ++it) {
            const int s = it % kStages;
            if (!mbar_wait(&bars->full[s], (it / kStages) & 1, failed)) {
              ok = false;
              break;
            }
            fence_after_sync();
            const uint32_t a_addr = smem_u32(tiles + s * kStageBytes);
            const uint64_t adesc = make_desc(a_addr), bdesc = make_desc(a_addr + kTileBytesX);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              // 16 k-elements are 32 bytes: the start address field moves by 2 (units of 16 bytes)
              const uint32_t acc = (kt > t_begin || k > 0) ? 1u : 0u;
              if (PAIR)
                umma_pair(d, adesc + 2 * k, bdesc + 2 * k, instr_desc_pair(BNT), acc);
              else
                umma(d, adesc + 2 * k, bdesc + 2 * k, instr_desc(bt), acc);
            }
            // the stage may be refilled once these MMAs are done
            if (PAIR)
              umma_commit_pair(&bars->empty[s]);
            else
              umma_commit(&bars->empty[s]);
          }
          if (ok) {
            if (PAIR)
              umma_commit_pair(&bars->acc_full[buf]);
            else
              umma_commit(&bars->acc_full[buf]);
          }
        }
      }
    }
  }
  } else {
    if (WIDE) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // epilogue: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31. A thread owns one
    // row of the tile and the two halves (pieces of 64 columns) of a 128-column block of it;
    // a wide tile has two such blocks, one per group of four warps. With interleaved gate/up
    // weights the first piece holds gates and the second the up values of the same outputs.
    bw::pdl_wait();
    const int quarter = warp & 3;
    const int et = quarter * 32 + lane;  // 0..127: this thread's row of the tile
    const int blk = (warp - kFirstEpiWarp) >> 2;  // 0, or 0..1 in a wide tile
    constexpr int half = 0;
    const int off0 = blk * BN, off1 = off0 + BN / 2;  // column offsets of the pieces in the tile
    float total[2 * PW];
    uint32_t gc = 0;
    bool ok = true;
    for (int tile = worker; tile < out_tiles && ok; tile += workers) {
      const int m0 = item_m0(tile), n0 = item_n0(tile);
      const int row = m0 + et;
      for (int c = item_c0(tile); c < item_c1(tile) && ok; ++c, ++gc) {
        const int buf = gc & 1;
        if (!mbar_wait(&bars->acc_full[buf], (gc >> 1) & 1, failed)) {
          ok = false;
          break;
        }
        fence_after_sync();
        if (!SPLIT || quarter * 32 < M) {  // in split mode warps whose rows are all padding read nothing
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BNT;
#pragma unroll
          for (int piece = 0; piece < 2; ++piece) {
#pragma unroll
            for (int g = 0; g < PW / LDW; ++g) {
              if (!WIDE && (piece ? off1 : off0) + g * LDW >= bt) continue;  // a narrow tile ends here
              float v[LDW];
              tmem_ld(taddr + (piece ? off1 : off0) + g * LDW, v);
#pragma unroll
              for (int j = 0; j < LDW; ++j) {
                float& t = total[piece * PW + g * LDW + j];
                t = (SPLIT || c == 0) ? v[j] : t + v[j];
              }
            }
          }
        }
        fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR)
            mbar_arrive_cluster(peer_addr(smem_u32(&bars->acc_empty[buf]), 0));
          else
            mbar_arrive(&bars->acc_empty[buf]);
        }
      }
      if (!ok) break;
      if (row >= M) continue;
      if (SPLIT && num_chunks > 1) {
        // this item's chunk sum goes to scratch; a second kernel adds the chunk sums in order
        const int chunk = item_c0(tile);
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
          const int col0 = n0 + (piece ? off1 : off0);
          const int cols = min(PW, min(N, n0 + bt) - col0);
          float* mine = partials + (static_cast<size_t>(chunk) * M + row) * N + col0;
          if (cols == PW && (N & 7) == 0 && (reinterpret_cast<uintptr_t>(partials) & 31) == 0) {
#pragma unroll
            for (int j = 0; j < PW; j += 8) {
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(total[piece * PW + j + e]);
              st256(mine + j, o);
            }
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j)
              if (!WIDE && j < cols) __stcg(mine + j, total[piece * PW + j]);
          }
        }
        continue;
      }
      if (EPI == 1) {
        // the first piece holds gate rows, the second the up rows of the same indices; both
        // are rounded to bfloat16 first, as if the product had been stored
        if (n0 + off0 >= N) continue;
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(Y) + static_cast<size_t>(row) * (N / 2) + (n0 + blk * BN) / 2 + half * PW;
        const bool wide_store = (reinterpret_cast<uintptr_t>(Y) & 31) == 0;  // rows are N bytes, N % 128 == 0
#pragma unroll
        for (int j = 0; j < PW; j += 16) {
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float g0 = __bfloat162float(__float2bfloat16_rn(total[j + 2 * e]));
            const float g1 = __bfloat162float(__float2bfloat16_rn(total[j + 2 * e + 1]));
            const float u0 = __bfloat162float(__float2bfloat16_rn(total[PW + j + 2 * e]));
            const float u1 = __bfloat162float(__float2bfloat16_rn(total[PW + j + 2 * e + 1]));
            o[e] = pack_bf16(bw::swiglu_one(g0, u0), bw::swiglu_one(g1, u1));
          }
          if (wide_store) {
            st256(out + j, o);
          } else {
            *reinterpret_cast<uint4*>(out + j) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(out + j + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        continue;
      }
#pragma unroll
      for (int piece = 0; piece < 2; ++piece) {
        const int col0 = n0 + (piece ? off1 : off0);
        const int cols = min(PW, min(N, n0 + bt) - col0);  // may be <= 0 in a narrow or a last, partial tile
        if (cols <= 0) continue;
        const size_t base = static_cast<size_t>(row) * N + col0;
        if (EPI == 2) {
          float* out = static_cast<float*>(Y) + base;
          const float* res = residual ? residual + base : nullptr;
          if (cols == PW && (N & 7) == 0 && (reinterpret_cast<uintptr_t>(Y) & 31) == 0 &&
              (reinterpret_cast<uintptr_t>(residual) & 31) == 0) {
#pragma unroll
            for (int j = 0; j < PW; j += 8) {
              uint32_t o[8];
              if (res) {
                ld256(res + j, o);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) + total[piece * PW + j + e]);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(total[piece * PW + j + e]);
              }
              st256(out + j, o);
            }
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j)  // static indices keep the totals in registers
              if (!WIDE && j < cols) out[j] = res ? res[j] + total[piece * PW + j] : total[piece * PW + j];
          }
        } else {
          __nv_bfloat16* out = static_cast<__nv_bfloat16*>(Y) + base;
          if (cols == PW && (N & 15) == 0 && (reinterpret_cast<uintptr_t>(Y) & 31) == 0) {
#pragma unroll
            for (int j = 0; j < PW; j += 16) {
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = pack_bf16(total[piece * PW + j + 2 * e], total[piece * PW + j + 2 * e + 1]);
              st256(out + j, o);
            }
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j)
              if (!WIDE && j < cols) out[j] = __float2bfloat16_rn(total[piece * PW + j]);
          }
        }
      }
    }
  }

  fence_before_sync();
  if (PAIR)
    cluster_sync_all();  // neither block leaves while the other may still read its memory or signal it
  else
    __syncthreads();
  if (warp == 1) {
    __syncwarp();
    fence_after_sync();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(kTmemColsT) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(kTmemColsT) : "memory");
  }
  if (threadIdx.x == 0 && bars->failed) atomicExch(error_flag, 1);
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
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

// rows x k bf16, row-major; box of box_rows rows x 64 k-elements, 128-byte swizzle, zero fill outside
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows = BM) {
  EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int g_pair_tiles = 1;         // large batches: two blocks per 256 x 256 tile (0: one block per 128 x 256 tile)

}  // namespace

// Whether this product can run on the tcgen05 path: rows that start on 16 bytes (TMA).
BW_API int bw_bf16_linear_tc_usable(const void* x, const void* w, int k) {
  return (k % 8 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0) &&
         encoder() != nullptr;
}

// Large batches run two blocks per tile (1, the default) or one (0); both give the same bits.
// Returns the previous setting. For tests and measurements.
BW_API int bw_bf16_linear_tc_pair_tiles(int on) {
  const int before = g_pair_tiles;
  g_pair_tiles = on ? 1 : 0;
  return before;
}

// Scratch of split mode: chunk sums [chunks][m][n] float32 and one counter per column block.
BW_API long long bw_bf16_linear_tc_scratch_floats(int m, int n, int k) {
  return static_cast<long long>((k + kChunk - 1) / kChunk) * m * n;
}
BW_API int bw_bf16_linear_tc_counters(int n) { return (n + BN - 1) / BN; }

// Split mode is chosen from the shape alone: one block of rows, more than one chunk, and too
// few output tiles to occupy the machine. Both modes give the same bits.
namespace {

constexpr int kMaxDevices = 64;  // per-device state below is kept for device ordinals up to this

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

int sm_count_of_device() {
  static int sm_count[kMaxDevices] = {0};
  const int dev = current_device();
  if (!sm_count[dev]) {
    cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sm_count[dev] <= 0) sm_count[dev] = 148;
  }
  return sm_count[dev];
}

// How a product with one block of rows (m <= 128) runs. A tcgen05.mma that adds to the
// accumulator of the one before it starts only when that one is done, about 100 ns later
// whatever the tile's width, so a block's time is the number of such steps it issues one
// after the other: 32 per chunk of 512. The plan minimises (rounds of the SMs over the work
// items) x (steps per item): items are output tiles (all chunks inside, "whole") or (tile,
// chunk) pairs ("split", which adds a second kernel and the traffic of the chunk sums);
// tiles are 16 .. 128 columns wide in steps of 16, or 256. Of equal plans the one with the
// narrower tiles wins (more SMs stream weights). Every plan gives the same bits.
struct Plan {
  bool split;
  int bn;
};
int g_tile_width = 0;  // 0: chosen from the shape; else forced (tests, measurements)
int g_force_mode = 0;  // 0: chosen; 1: whole; 2: split where it is possible

constexpr int kMaxSplitColumns = 16384;  // bounds the scratch of the chunk sums

Plan plan_rows(int m, int n, int k, bool swiglu, int sms, bool allow_wide = true) {
  const int chunks = (k + kChunk - 1) / kChunk;
  const int steps_chunk = kChunk / 16;
  const bool may_split = m <= BM && chunks > 1 && n <= kMaxSplitColumns;
  Plan best{false, BN};
  double best_cost = -1.0;
  for (int mode = 0; mode < 2; ++mode) {
    if (mode == 1 && !may_split) continue;
    if (g_force_mode == 1 && mode == 1) continue;
    if (g_force_mode == 2 && mode == 0 && may_split) continue;
    for (int bn = 16; bn <= 2 * BN; bn = (bn < BN ? bn + 16 : 2 * bn)) {
      if (swiglu && bn < BN) continue;  // gate and up of an output lie 64 columns apart
      if (bn > BN && (!allow_wide || n % 64)) continue;
      if (g_tile_width && bn != g_tile_width && !(swiglu && g_tile_width < BN && bn == BN)) continue;
      const long long tiles = (n + bn - 1) / bn;
      const long long items = mode ? tiles * chunks : tiles;
      const long long rounds = (items + sms - 1) / sms;
      double cost = static_cast<double>(rounds) * (mode ? steps_chunk : steps_chunk * chunks);
      // the second kernel, and writing and reading the chunk sums (8 bytes each at about 3 TB/s)
      if (mode) cost += 20.0 + 2.67e-5 * chunks * static_cast<double>(m) * n;
      if (best_cost < 0 || cost < best_cost - 1e-9) best = Plan{mode == 1, bn}, best_cost = cost;
    }
  }
  return best;
}

}  // namespace

// Steps of few rows take the streaming kernel of bf16_gemm_rows.cu (same bits), unless a test
// or a measurement forces a plan of this file's kernel.
BW_API int bw_bf16_linear_rows_usable(const void* x, const void* w, int m, int n, int k, int swiglu);
BW_API int bw_bf16_linear_rows(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_kind, const float* residual,
                               int m, int n, int k, cudaStream_t stream);
namespace {
bool rows_path_takes(int m, int n, int k, int swiglu, const void* x = nullptr, const void* w = nullptr) {
  return g_tile_width == 0 && g_force_mode == 0 && bw_bf16_linear_rows_usable(x, w, m, n, k, swiglu) != 0;
}
}  // namespace

// Forces the width of the output tiles of small batches (a multiple of 16 up to 128, or 256;
// 0: chosen from the shape) and the mode (0 chosen, 1 whole, 2 split where possible). Every
// combination gives the same bits. For tests and measurements.
BW_API void bw_bf16_linear_tc_force(int bn, int mode) {
  if (bn == 0 || bn == 2 * BN || (bn % 16 == 0 && bn >= 16 && bn <= BN)) g_tile_width = bn;
  if (mode >= 0 && mode <= 2) g_force_mode = mode;
}

// Whether a plain product of this shape is split along k (then it needs scratch).
BW_API int bw_bf16_linear_tc_splits(int m, int n, int k) {
  return m <= BM && plan_rows(m, n, k, false, sm_count_of_device()).split;
}
// Whether some plan may split it (what callers size the scratch by).
BW_API int bw_bf16_linear_tc_may_split(int m, int n, int k) { return m <= BM && k > kChunk && n <= kMaxSplitColumns; }
// Kernels that one call launches (1, or 2 when the product is split): callers count launches.
BW_API int bw_bf16_linear_tc_kernels(int m, int n, int k, int swiglu, int has_scratch) {
  if (rows_path_takes(m, n, k, swiglu)) return 1;
  return (m <= BM && has_scratch && plan_rows(m, n, k, swiglu != 0, sm_count_of_device()).split) ? 2 : 1;
}

namespace {

// What follows the product: nothing, or SwiGLU.
struct Fused {
  int mode = 0;  // 0 none, 2 swiglu (y is [m][n / 2] bfloat16)
};

// Once per device and kernel variant: the shared-memory limit of the kernel is raised and, for
// the variant that runs pairs of blocks, the number of pairs the device runs at a time is
// asked. Neither allocates. Returns 0 or an error; *pairs receives the number of pairs.
template <bool SPLIT, int A_ROWS, int EPI, bool WIDE, bool PAIR = false>
int configure_tc(int* pairs = nullptr) {
  constexpr int smem_max = kSmemBudget + sizeof(Barriers) + 1024;
  constexpr int threads = WIDE ? 384 : 192;
  static_assert(smem_max <= 227 * 1024, "ring does not fit");
  static bool configured[kMaxDevices] = {false};
  static int max_pairs[kMaxDevices] = {0};  // pairs that the device runs at the same time
  const int dev = current_device();
  auto kernel = gemm_tc_kernel<SPLIT, A_ROWS, EPI, WIDE, PAIR>;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
    if (e != cudaSuccess) {
      bw::set_error("linear (tcgen05): cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    if (PAIR) {
      constexpr int BNW = BN;
      const RingShape ring = ring_shape(A_ROWS, BNW);
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(2 * (sm_count_of_device() / 2));
      probe.blockDim = dim3(threads);
      probe.dynamicSmemBytes = ring.ring_bytes + static_cast<int>(sizeof(Barriers)) + 1024;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
      probe.attrs = attr;
      probe.numAttrs = 1;
      e = cudaOccupancyMaxActiveClusters(&max_pairs[dev], kernel, &probe);
      if (e != cudaSuccess || max_pairs[dev] <= 0) {
        bw::set_error("linear (tcgen05): the device offers no cluster of two blocks for this kernel: %s",
                      cudaGetErrorString(e));
        cudaGetLastError();
        return e != cudaSuccess ? static_cast<int>(e) : -1;
      }
    }
    configured[dev] = true;
  }
  if (pairs) *pairs = max_pairs[dev];
  return 0;
}

template <bool SPLIT, int A_ROWS, int EPI, bool WIDE, bool PAIR = false>
int launch_tc(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32, const float* residual, int m, int n,
              int k, int* error_word, float* partials, const Fused& fused, cudaStream_t stream, int narrow_bn = BN) {
  constexpr int BNT = WIDE ? 2 * BN : BN;
  constexpr int BNW = PAIR ? BN : BNT;
  constexpr int BMT = PAIR ? 2 * BM : BM;
  constexpr int threads = WIDE ? 384 : 192;
  const int chunks = (k + kChunk - 1) / kChunk;
  const int bn = WIDE ? BNT : narrow_bn;
  const RingShape ring = ring_shape(A_ROWS, WIDE ? BNW : bn);
  const int smem = ring.ring_bytes + static_cast<int>(sizeof(Barriers)) + 1024;
  auto kernel = gemm_tc_kernel<SPLIT, A_ROWS, EPI, WIDE, PAIR>;
  int max_pairs = 0;
  if (const int rc = configure_tc<SPLIT, A_ROWS, EPI, WIDE, PAIR>(&max_pairs)) return rc;
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, x, m, k, A_ROWS) || !make_map(&map_w, w, n, k, WIDE ? BNW : bn)) {
    bw::set_error("linear (tcgen05): cuTensorMapEncodeTiled refused [%d x %d] / [%d x %d]", m, k, n, k);
    return -1;
  }
  const int n_blocks = (n + bn - 1) / bn, m_blocks = (m + BMT - 1) / BMT;
  const long long items = SPLIT ? static_cast<long long>(n_blocks) * chunks : static_cast<long long>(n_blocks) * m_blocks;
  if (PAIR) {
    const unsigned pairs = static_cast<unsigned>(items < max_pairs ? items : max_pairs);
    bw::launch_pdl_cluster2(kernel, dim3(2 * pairs), dim3(threads), smem, stream, map_x, map_w, y, y_is_f32, residual, m,
                            n, k, error_word, partials, bn);
    return bw::launch_status();
  }
  const int sms = sm_count_of_device();
  const unsigned grid = static_cast<unsigned>(items < sms ? items : sms);
  bw::launch_pdl(kernel, dim3(grid), dim3(threads), smem, stream, map_x, map_w, y, y_is_f32, residual, m, n, k,
                 error_word, partials, bn);
  if (SPLIT) {
    const size_t outputs = static_cast<size_t>(m) * n;
    if (fused.mode == 2)
      bw::launch_pdl(reduce_swiglu_kernel, dim3(static_cast<unsigned>((outputs / 2 + 255) / 256)), dim3(256), 0, stream, 
          partials, chunks, static_cast<__nv_bfloat16*>(y), m, n);
    else
      bw::launch_pdl(reduce_chunks_kernel, dim3(static_cast<unsigned>((outputs + 255) / 256)), dim3(256), 0, stream, partials, chunks, y,
                                                                                            y_is_f32, residual, m, n);
  }
  return bw::launch_status();
}

// picks the x-tile height from the batch size, and for small batches the plan
template <int EPI>
int launch_tc_rows(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32, const float* residual, int m,
                   int n, int k, int* error_word, float* partials, const Fused& fused, cudaStream_t stream) {
#define BW_LAUNCH(SPLIT_, ROWS_, EPI_, WIDE_) \
  launch_tc<SPLIT_, ROWS_, EPI_, WIDE_>(x, w, y, y_is_f32, residual, m, n, k, error_word, partials, fused, stream, plan.bn)
#define BW_LAUNCH_ROWS(SPLIT_, EPI_, WIDE_)                        \
  (m <= 16   ? BW_LAUNCH(SPLIT_, 16, EPI_, WIDE_)                  \
   : m <= 32 ? BW_LAUNCH(SPLIT_, 32, EPI_, WIDE_)                  \
   : m <= 64 ? BW_LAUNCH(SPLIT_, 64, EPI_, WIDE_)                  \
             : BW_LAUNCH(SPLIT_, 128, EPI_, WIDE_))
  // wide tiles want whole pieces of 64 columns and 32-byte stores
  const bool wide_ok = n % 64 == 0 && reinterpret_cast<uintptr_t>(y) % 32 == 0 &&
                       reinterpret_cast<uintptr_t>(residual) % 32 == 0 && reinterpret_cast<uintptr_t>(partials) % 32 == 0;
  if (m <= BM) {
    Plan plan = plan_rows(m, n, k, fused.mode == 2, sm_count_of_device(), wide_ok);
    if (!partials) plan = Plan{false, plan.split ? BN : plan.bn};
    const bool wide = plan.bn > BN;
    if (plan.split) return wide ? BW_LAUNCH_ROWS(true, 0, true) : BW_LAUNCH_ROWS(true, 0, false);
    return wide ? BW_LAUNCH_ROWS(false, EPI, true) : BW_LAUNCH_ROWS(false, EPI, false);
  }
#undef BW_LAUNCH_ROWS
#undef BW_LAUNCH
  if (!wide_ok)
    return launch_tc<false, 128, EPI, false>(x, w, y, y_is_f32, residual, m, n, k, error_word, nullptr, fused, stream);
  if (g_pair_tiles)
    return launch_tc<false, 128, EPI, true, true>(x, w, y, y_is_f32, residual, m, n, k, error_word, nullptr, fused, stream);
  return launch_tc<false, 128, EPI, true>(x, w, y, y_is_f32, residual, m, n, k, error_word, nullptr, fused, stream);
}

// Every kernel variant that launch_tc_rows<EPI> can choose, configured for the current device.
template <int EPI>
int configure_reachable() {
  int rc = 0;
#define BW_CONF(...) if (!rc) rc = configure_tc<__VA_ARGS__>()
#define BW_CONF_ROWS(SPLIT_, EPI_, WIDE_) \
  BW_CONF(SPLIT_, 16, EPI_, WIDE_);      \
  BW_CONF(SPLIT_, 32, EPI_, WIDE_);      \
  BW_CONF(SPLIT_, 64, EPI_, WIDE_);      \
  BW_CONF(SPLIT_, 128, EPI_, WIDE_)
  BW_CONF_ROWS(true, 0, true);
  BW_CONF_ROWS(true, 0, false);
  BW_CONF_ROWS(false, EPI, true);
  BW_CONF_ROWS(false, EPI, false);
  BW_CONF(false, 128, EPI, true, true);
#undef BW_CONF_ROWS
#undef BW_CONF
  return rc;
}

}  // namespace

BW_API int bw_bf16_linear_tc(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32,
                             const float* residual, int m, int n, int k, float* partials, int* counters,
                             cudaStream_t stream) {
  (void)counters;
  if (m <= 0 || n <= 0) return 0;
  if (!bw_bf16_linear_tc_usable(x, w, k)) {
    bw::set_error("linear (tcgen05): rows must start on 16 bytes (k %% 8 == 0) and the driver must offer tensor maps");
    return -1;
  }
  if (rows_path_takes(m, n, k, 0, x, w)) return bw_bf16_linear_rows(x, w, y, y_is_f32 ? 2 : 0, residual, m, n, k, stream);
  int* word = bw::failure_word();
  if (!word) return -1;
  const Fused none;
  if (y_is_f32) return launch_tc_rows<2>(x, w, y, 1, residual, m, n, k, word, partials, none, stream);
  return launch_tc_rows<0>(x, w, y, 0, nullptr, m, n, k, word, partials, none, stream);
}

// h[m][n / 2] = SwiGLU of x W^T for gate/up weights interleaved in blocks of 64 rows
// (n a multiple of 128).
BW_API int bw_bf16_linear_tc_swiglu(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* h, int m, int n, int k,
                                    float* partials, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (n % 128 || !bw_bf16_linear_tc_usable(x, w, k)) {
    bw::set_error("linear + SwiGLU: needs n %% 128 == 0 (got %d) and rows that start on 16 bytes", n);
    return -1;
  }
  if (rows_path_takes(m, n, k, 1, x, w)) return bw_bf16_linear_rows(x, w, h, 1, nullptr, m, n, k, stream);
  int* word = bw::failure_word();
  if (!word) return -1;
  Fused f;
  f.mode = 2;
  return launch_tc_rows<1>(x, w, h, 0, nullptr, m, n, k, word, partials, f, stream);
}

// ---------------------------------------------------------------------------------------
// The entry point that allocates nothing (declared in bw_noalloc.h, which says whom it is
// for).  Same kernels as above; the scratch of split mode and the word that bounded waits
// raise live in file-scope device arrays instead of memory from cudaMalloc.
#include "bw_noalloc.h"

namespace {

// In host code these names are stand-ins, not device addresses: the address that a kernel
// may use comes from cudaGetSymbolAddress, once per device (below).
static __device__ __align__(256) float g_noalloc_scratch[BW_NOALLOC_MAX_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_error[64];

float* g_noalloc_scratch_ptr[kMaxDevices] = {nullptr};
int* g_noalloc_error_ptr[kMaxDevices] = {nullptr};

}  // namespace

// Floats of the library's scratch array that a product of this shape uses: chunks of 512 along
// k times m times n when the product is split along k, else 0.
BW_API long long bw_bf16_linear_noalloc_scratch_floats(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0 || !bw_bf16_linear_tc_splits(m, n, k)) return 0;
  return static_cast<long long>((k + kChunk - 1) / kChunk) * m * n;
}

BW_API int bw_bf16_linear_noalloc(const __nv_bfloat16* x, const __nv_bfloat16* w, void* y, int y_is_f32,
                                  const float* residual, int m, int n, int k, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0) {
    bw::set_error("linear (no allocation): inner size %d", k);
    return -1;
  }
  if (!bw_bf16_linear_tc_usable(x, w, k)) {
    bw::set_error("linear (no allocation): rows must start on 16 bytes (k %% 8 == 0) and the driver must offer tensor maps");
    return -1;
  }
  if (residual && !y_is_f32) {
    bw::set_error("linear (no allocation): a residual needs a float32 output");
    return -1;
  }
  const long long need = bw_bf16_linear_noalloc_scratch_floats(m, n, k);
  const bool split = need > 0;
  if (need > BW_NOALLOC_MAX_SCRATCH_FLOATS) {
    bw::set_error("linear (no allocation): [%d x %d] x [%d x %d] needs %lld floats of scratch, the library holds %d",
                  m, k, n, k, need, BW_NOALLOC_MAX_SCRATCH_FLOATS);
    return -2;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    bw::set_error("linear (no allocation): cannot use device %d: %s", dev, cudaGetErrorString(e));
    return e != cudaSuccess ? static_cast<int>(e) : -1;
  }
  if (!g_noalloc_scratch_ptr[dev]) {
    // set-up, once per device, with that device current
    float* sp = nullptr;
    int* ep = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&sp), g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ep), g_noalloc_error);
    if (e != cudaSuccess) {
      bw::set_error("linear (no allocation): set-up on device %d failed: %s", dev, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    // every kernel variant that a later call may pick gets its shared-memory limit now, so that
    // no later call has set-up left to do, whatever its shape
    if (const int rc = configure_reachable<0>()) return rc;
    if (const int rc = configure_reachable<2>()) return rc;
    g_noalloc_error_ptr[dev] = ep;  // the array is zero when the library is loaded; kernels only ever set word 0
    g_noalloc_scratch_ptr[dev] = sp;
  }
  // Nothing in the scratch has to start at zero: every chunk sum that the second kernel reads
  // is written by the first one in this same call.
  float* scratch = split ? g_noalloc_scratch_ptr[dev] : nullptr;
  if (y_is_f32)
    return launch_tc_rows<2>(x, w, y, 1, residual, m, n, k, g_noalloc_error_ptr[dev], scratch, Fused(), stream);
  return launch_tc_rows<0>(x, w, y, 0, nullptr, m, n, k, g_noalloc_error_ptr[dev], scratch, Fused(), stream);
}

// Reads and clears the word that a kernel launched by bw_bf16_linear_noalloc raises when one
// of its bounded waits ran out (a copy of four bytes; nothing is allocated).
BW_API int bw_bf16_linear_noalloc_failed() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || !g_noalloc_error_ptr[dev]) return 0;
  int v = 0;
  cudaMemcpy(&v, g_noalloc_error_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(g_noalloc_error_ptr[dev], 0, sizeof(int));
  return v;
}
