// Prefill attention on the fifth-generation tensor cores, for head sizes 64 and 128.
//
// Same arithmetic, in the same order, as attention_whole_kernel / attention_split_kernel in
// bf16_attention.cu (key tiles of 64 at fixed positions; per tile and row the maximum, the sum
// of the weights and the unnormalised output with bfloat16 weights; ordered merge), so the
// three kernels give the same bits. What changes is where the work runs:
//   warp 0     brings Q (once) and the key/value tiles of the paged cache into shared memory
//              with TMA (128-byte swizzle), one box per page and piece, the lanes asking for
//              one box each
//   warp 1     one thread issues tcgen05.mma: S = Q K^T (128 stacked rows x 64 keys, K-major
//              operands) into one of two S buffers in tensor memory, and O_t = P V (P from
//              shared memory, V as an MN-major operand) into one of two O buffers
//   warps 2-5  one thread per stacked row: read the S row from tensor memory, scale, mask,
//              maximum, weights, sum; write the bfloat16 weights as the next A operand into
//              shared memory; later read the O_t row and merge it into the running state in
//              registers; finally normalise and store
// A head of 128 is two pieces of 64 along d: Q, K and V tiles are kept piece by piece (a row of
// a piece is one 128-byte swizzled line), the scores add up over the pieces' k-steps in order,
// and the output takes one MMA per 16 keys over all 128 columns (the pieces of V are the
// swizzle atoms of one MN-major operand, a piece apart).
// What the tensor core does is handed out by one thread, and every instruction or barrier
// operation costs that thread about a hundred cycles, which is what a tile's time is made of
// (measured with time stamps: 21 such operations and 2,500 cycles per tile of 64 keys at head
// size 128, where the arithmetic needs 500). So that thread waits only for what nothing else
// implies (keys landed, weights written: the buffers of S and O are free by then, see below)
// and announces the output and the freed stage with one commit.
// At head size 64 two blocks share an SM (256 tensor-memory columns and about 100 KB each), so
// one block's softmax overlaps the other's MMAs; at 128 a block has the SM to itself (384 of
// the 512 columns, 170 KB) and overlaps its own stages. Every mbarrier wait is bounded
// (bw_common.cuh).
#include <cuda.h>

#include "bw_common.cuh"

#ifndef BW_HEAD_DIM
#error "compile with -DBW_HEAD_DIM=<head size>"
#endif

#if BW_HEAD_DIM == 64 || BW_HEAD_DIM == 128

namespace {

constexpr int HD = BW_HEAD_DIM;
constexpr int kPieces = HD / 64;  // 64-wide pieces of a head along d
constexpr int kTileM = 128;   // stacked rows per block
constexpr int kTileKV = 64;   // keys per tile
constexpr int kStages = 3;    // key/value tiles in flight (a fourth at head size 128 fits and was slower end to end)  // key/value tiles in flight (at 64 two blocks share an SM's shared memory)
constexpr int kThreads = 192;
constexpr int kQPiece = kTileM * 128;          // 16 KB: one piece of the Q tile
constexpr int kKPiece = kTileKV * 128;         // 8 KB: one piece of a K (or V) tile
constexpr int kQBytes = kPieces * kQPiece;
constexpr int kKBytes = kPieces * kKPiece;
constexpr int kPBytes = kTileM * 128;          // 16 KB per weight buffer
constexpr int kOCol = 128;                     // S0 S1 at columns 0 and 64, O0 O1 at 128 and 128 + HD
constexpr int kTmemCols = HD == 64 ? 256 : 512;

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t kv_full[kStages], pv_done[kStages];  // a tile's keys and values have landed; its output is formed
  uint64_t s_full[2], p_ready[2];
  uint32_t tmem_base;
  uint32_t failed;
};
constexpr int kMaxTablePages = 2048;  // page ids of the block's key range, staged in shared memory

constexpr int kSmemBytes = kQBytes + kStages * 2 * kKBytes + 2 * kPBytes + sizeof(Barriers) + kMaxTablePages * 4 + 1024;

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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* failed) {
  return bw::mbar_wait_bounded(bar, parity, failed);
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}
// descriptor of a 128-byte-swizzled tile with 8-row groups 1024 bytes apart (K-major tiles of
// Q, K and P; the MN-major V tile has the same numbers: 64 contiguous d, groups of 8 keys)
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// The same for the whole MN-major V tile of a head wider than 64: its 64-wide pieces lie a piece
// (kKPiece bytes) apart, which is the leading-dimension offset between the swizzle atoms along d.
__device__ __forceinline__ uint64_t make_desc_wide(uint32_t smem_addr, uint32_t piece_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(piece_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// kind::f16, D float32, A and B bfloat16, M 128, N 64; bit 16 set: B is MN-major (N = HD: all of
// a head's columns in one instruction, an instruction's issue costs its thread about a hundred cycles)
constexpr uint32_t kDescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kDescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((static_cast<uint32_t>(HD) >> 3) << 17) | ((128u >> 4) << 24);

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
// 64 consecutive columns of this thread's lane: one load instruction and one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// the merge of bf16_attention.cu, word for word
struct MergeWeights {
  float a, b, mx;
};
__device__ __forceinline__ MergeWeights merge_weights(float M, float m) {
  MergeWeights w;
  w.mx = fmaxf(M, m);
  const float ref = (w.mx == -INFINITY) ? 0.0f : w.mx;
  w.a = bw::exp2_approx(__fsub_rn(M, ref));
  w.b = bw::exp2_approx(__fsub_rn(m, ref));
  return w;
}
__device__ __forceinline__ float merge_value(float X, float x, const MergeWeights& w) {
  return __fmaf_rn(x, w.b, __fmul_rn(X, w.a));
}

__global__ void __launch_bounds__(kThreads)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                    const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                    const int* __restrict__ seq_row0, __nv_bfloat16* __restrict__ out, int out_stride, int heads,
                    int kv_heads, int page, int window, float scale_log2, int* error_flag) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = bw::smem_align_1024(smem_raw);
  unsigned char* sq = base;
  unsigned char* skv = sq + kQBytes;                    // stage s: K at skv + s * 2 * kKBytes, V kKBytes behind
  unsigned char* sp = skv + kStages * 2 * kKBytes;      // two weight buffers
  Barriers* bars = reinterpret_cast<Barriers*>(sp + 2 * kPBytes);
  int* spages = reinterpret_cast<int*>(bars + 1);
  volatile uint32_t* failed = &bars->failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->pv_done[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->p_ready[b], 4);
    }
    bars->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "n"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  bw::pdl_enter();

  // The host lists the tiles with the most keys first, and blocks are handed out with
  // blockIdx.x running fastest: the heads of the longest tile start first, then those of the
  // next one, so the long blocks do not start late and stretch the tail of the launch.
  const int tile = blockIdx.y, g = blockIdx.x;
  const int group = heads / kv_heads;
  const int seq = tile_seq[tile], row0 = tile_row0[tile], nrows = tile_rows[tile];
  const int mrows = nrows * group;
  const int p_first = seq_pos0[seq] + (row0 - seq_row0[seq]);
  const int p_last = p_first + nrows - 1;
  const int kv_lo = (window > 0 && p_first - window + 1 > 0) ? ((p_first - window + 1) / kTileKV) * kTileKV : 0;
  const int kv_hi = p_last + 1;
  const int ntiles = (kv_hi - kv_lo + kTileKV - 1) / kTileKV;
  const int pages_per_tile = kTileKV / page;

  if (warp == 0) {
    // the page ids of this block's key range go to shared memory first (one coalesced read),
    // so that the loop below does not wait for a table entry per page
    const int* table = block_table + static_cast<size_t>(seq) * max_blocks;
    const int first_page = kv_lo / page, last_page = (kv_hi - 1) / page;
    const int staged = min(last_page - first_page + 1, kMaxTablePages);
    for (int i = lane; i < staged; i += 32) spages[i] = table[first_page + i];
    __syncwarp();
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, kQBytes);
      for (int i = 0; i < kPieces; ++i) tma_load_4d(sq + i * kQPiece, &map_q, 64 * i, 0, g, row0, &bars->q_full);
    }
    // A tile of keys and values is pages x pieces x 2 copies (16 at head size 128 with pages of 16),
    // and the issue of one holds its thread for a hundred cycles or more: the lanes issue one each,
    // side by side, or the copies of a tile would take longer to ask for than the tile takes to use.
    const int copies = pages_per_tile * kPieces * 2;
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % kStages;
      int ok = 1;
      if (lane == 0) {
        if (t >= kStages && !mbar_wait(&bars->pv_done[s], ((t / kStages) - 1) & 1, failed)) ok = 0;
        if (ok) mbar_expect_tx(&bars->kv_full[s], 2 * kKBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      unsigned char* k = skv + s * 2 * kKBytes;
      const int j0 = kv_lo + t * kTileKV;
      for (int c = lane; c < copies; c += 32) {
        const int pg = c / (kPieces * 2), i = (c >> 1) % kPieces, is_v = c & 1;
        const int j = j0 + pg * page;
        // pages wholly beyond the last key are not in the table: any valid page will do, its keys are masked
        const int pi = min(j / page, last_page) - first_page;
        const int blk = pi < staged ? spages[pi] : table[first_page + pi];
        tma_load_4d(k + is_v * kKBytes + i * kKPiece + pg * page * 128, is_v ? &map_v : &map_k, 64 * i, 0, g, blk,
                    &bars->kv_full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(&bars->q_full, 0, failed);
      fence_after_sync();
      const uint32_t q_addr = smem_u32(sq);
      auto issue_qk = [&](int t) -> bool {
        const int s = t % kStages, b = t & 1;
        if (!mbar_wait(&bars->kv_full[s], (t / kStages) & 1, failed)) return false;
        // The scores' buffer was read by the softmax of tile t - 2 before that tile's weights were
        // announced, and this thread saw that announcement before it formed tile t - 2's output:
        // no barrier of its own (a wait costs this thread a hundred cycles even when it is over,
        // and the tensor core's work is handed out by this one thread).
        fence_after_sync();
        const uint32_t k_addr = smem_u32(skv + s * 2 * kKBytes);
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {  // d ascending: piece after piece, 16 values a step
          const uint64_t qdesc = make_desc(q_addr + i * kQPiece), kdesc = make_desc(k_addr + i * kKPiece);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma(tmem_base + b * 64, qdesc + 2 * k, kdesc + 2 * k, kDescQK, (i | k) > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[b]);
        return true;
      };
      if (ok && ntiles > 0) ok = issue_qk(0);
      for (int t = 0; t < ntiles && ok; ++t) {
        const int s = t % kStages, b = t & 1;
        if (t + 1 < ntiles) ok = issue_qk(t + 1);  // the next tile's scores are computed while this one's weights are formed
        if (!ok) break;
        if (!mbar_wait(&bars->p_ready[b], (t >> 1) & 1, failed)) break;
        // the output buffer was merged (tile t - 2) before the softmax of this tile began: same argument
        fence_after_sync();
        const uint64_t pdesc = make_desc(smem_u32(sp + b * kPBytes));
        const uint32_t v_addr = smem_u32(skv + s * 2 * kKBytes + kKBytes);
        const uint64_t vdesc = kPieces == 1 ? make_desc(v_addr) : make_desc_wide(v_addr, kKPiece);
#pragma unroll
        for (int k = 0; k < kTileKV / 16; ++k)  // 16 keys: 32 bytes along a row of P, two 8-key groups (2048 bytes) of V
          umma(tmem_base + kOCol + b * HD, pdesc + 2 * k, vdesc + 128 * k, kDescPV, k > 0 ? 1u : 0u);
        umma_commit(&bars->pv_done[s]);  // the output is there, and the stage may be filled again
      }
    }
  } else {
    // one thread per stacked row; warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    const int pos = (m < mrows) ? p_first + m / group : p_last;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float o_tot[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_tot[i] = 0.0f;
    float M = -INFINITY, L = 0.0f, prev_max = -INFINITY, prev_sum = 0.0f;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      const int b = t & 1;
      const int j0 = kv_lo + t * kTileKV;
      if (!mbar_wait(&bars->s_full[b], (t >> 1) & 1, failed)) {
        ok = false;
        break;
      }
      fence_after_sync();
      float s[kTileKV];
      tmem_ld64(lane_addr + b * 64, s);
      fence_before_sync();
      // mask, maximum of the raw scores (the mask test is skipped for tiles inside the row's
      // range), then weights e = 2^(s * scale - ref) with one fused multiply-add per key
      float tmax = -INFINITY;
      const bool inside = j0 + kTileKV - 1 <= pos && j0 >= first;
      if (!inside) {
#pragma unroll
        for (int i = 0; i < kTileKV; ++i) {
          const int j = j0 + i;
          s[i] = (j <= pos && j >= first) ? s[i] : -INFINITY;
        }
      }
      {  // the maximum is exact in any order: four independent chains instead of one of 64
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < kTileKV; i += 4) {
          m4[0] = fmaxf(m4[0], s[i]);
          m4[1] = fmaxf(m4[1], s[i + 1]);
          m4[2] = fmaxf(m4[2], s[i + 2]);
          m4[3] = fmaxf(m4[3], s[i + 3]);
        }
        tmax = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      tmax = __fmul_rn(tmax, scale_log2);
      const float nref = (tmax == -INFINITY) ? 0.0f : -tmax;
      // their sum in the order of the other kernels: key j belongs to quad lane (j % 8) / 2; a
      // quad lane adds its pairs for j / 8 ascending; then (a0 + a1) + (a2 + a3)
      float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t packed[kTileKV / 2];
#pragma unroll
      for (int nb = 0; nb < kTileKV / 8; ++nb)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float e0 = bw::exp2_approx(__fmaf_rn(s[nb * 8 + 2 * q], scale_log2, nref));
          const float e1 = bw::exp2_approx(__fmaf_rn(s[nb * 8 + 2 * q + 1], scale_log2, nref));
          part[q] = __fadd_rn(part[q], __fadd_rn(e0, e1));
          __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
          packed[nb * 4 + q] = *reinterpret_cast<uint32_t*>(&pr);
        }
      const float tsum = __fadd_rn(__fadd_rn(part[0], part[1]), __fadd_rn(part[2], part[3]));
      // the row of P: 64 bfloat16 = eight 16-byte pieces, swizzled like a TMA-written tile
      unsigned char* prow = sp + b * kPBytes + m * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (m & 7)) << 4)) =
            make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the writes visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready[b]);

      // the output of the tile before this one is merged now, while the tensor core forms this
      // tile's output from the weights just written
      if (t > 0) {
        const int pb = (t - 1) & 1;
        if (!mbar_wait(&bars->pv_done[(t - 1) % kStages], ((t - 1) / kStages) & 1, failed)) {
          ok = false;
          break;
        }
        fence_after_sync();
        const MergeWeights w = merge_weights(M, prev_max);
        M = w.mx;
        L = merge_value(L, prev_sum, w);
#pragma unroll
        for (int pc = 0; pc < kPieces; ++pc) {
          float v[64];
          tmem_ld64(lane_addr + kOCol + pb * HD + 64 * pc, v);
#pragma unroll
          for (int i = 0; i < 64; ++i) o_tot[64 * pc + i] = merge_value(o_tot[64 * pc + i], v[i], w);
        }
        fence_before_sync();
      }
      prev_max = tmax;
      prev_sum = tsum;
    }
    if (ok && ntiles > 0) {  // the last tile's output
      const int pb = (ntiles - 1) & 1;
      if (mbar_wait(&bars->pv_done[(ntiles - 1) % kStages], ((ntiles - 1) / kStages) & 1, failed)) {
        fence_after_sync();
        const MergeWeights w = merge_weights(M, prev_max);
        M = w.mx;
        L = merge_value(L, prev_sum, w);
#pragma unroll
        for (int pc = 0; pc < kPieces; ++pc) {
          float v[64];
          tmem_ld64(lane_addr + kOCol + pb * HD + 64 * pc, v);
#pragma unroll
          for (int i = 0; i < 64; ++i) o_tot[64 * pc + i] = merge_value(o_tot[64 * pc + i], v[i], w);
        }
      } else {
        ok = false;
      }
    }
    if (ok && m < mrows) {
      const int qr = m / group, hq = m - qr * group;
      __nv_bfloat16* dst = out + static_cast<size_t>(row0 + qr) * out_stride + (g * group + hq) * HD;
      const float inv = __fdiv_rn(1.0f, L);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        __align__(16) __nv_bfloat162 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = __floats2bfloat162_rn(__fmul_rn(o_tot[c * 8 + 2 * e], inv), __fmul_rn(o_tot[c * 8 + 2 * e + 1], inv));
        *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(o);
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && bars->failed) atomicExch(error_flag, 1);
}

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

bool make_map4(CUtensorMap* map, const void* base, const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3],
               const cuuint32_t (&box)[4]) {
  EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Query rows per block, or 0 when this kernel cannot take the shape: head size 64 or 128, a page size
// that divides 64, a group of heads that divides 128, rows that start on 16 bytes.
BW_API int bw_bf16_attention_tc_tile_rows(int heads, int kv_heads, int hd, int page, int q_stride) {
  if (hd != HD || kv_heads <= 0 || heads % kv_heads) return 0;
  const int group = heads / kv_heads;
  if (group > kTileM || kTileM % group || page <= 0 || kTileKV % page || q_stride % 8 || !encoder()) return 0;
  return kTileM / group;
}

BW_API int bw_bf16_attention_tc(const __nv_bfloat16* qkv, int q_stride, const __nv_bfloat16* kcache,
                                const __nv_bfloat16* vcache, int num_pages, const int* block_table, int max_blocks,
                                const int* tile_seq, const int* tile_row0, const int* tile_rows, int num_tiles,
                                const int* seq_pos0, const int* seq_row0, __nv_bfloat16* out, int out_stride, int n,
                                int heads, int kv_heads, int hd, int page, int window, float scale,
                                cudaStream_t stream) {
  if (n <= 0 || num_tiles <= 0) return 0;
  if (num_tiles > 65535) {
    bw::set_error("attention (tcgen05): %d query tiles exceed the grid limit", num_tiles);
    return -1;
  }
  const int tile_rows_q = bw_bf16_attention_tc_tile_rows(heads, kv_heads, hd, page, q_stride);
  if (!tile_rows_q || out_stride % 8) {
    bw::set_error("attention (tcgen05): unsupported shape (heads %d/%d, head size %d, page %d)", heads, kv_heads, hd, page);
    return -1;
  }
  const int group = heads / kv_heads;
  int* word = bw::failure_word();
  if (!word) return -1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      bw::set_error("attention (tcgen05): cannot raise shared memory: %s", cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  {  // queries: [token][kv head][head of the group][d], box = 128 stacked rows of one kv head
    const cuuint64_t dims[4] = {HD, static_cast<cuuint64_t>(group), static_cast<cuuint64_t>(kv_heads),
                                static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[3] = {HD * 2, static_cast<cuuint64_t>(group) * HD * 2, static_cast<cuuint64_t>(q_stride) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(group), 1, static_cast<cuuint32_t>(kTileM / group)};  // one piece
    if (!make_map4(&map_q, qkv, dims, strides, box)) {
      bw::set_error("attention (tcgen05): cuTensorMapEncodeTiled refused the query map");
      return -1;
    }
  }
  {  // cache: [page][kv head][slot][d], box = one page of one kv head
    const cuuint64_t dims[4] = {HD, static_cast<cuuint64_t>(page), static_cast<cuuint64_t>(kv_heads),
                                static_cast<cuuint64_t>(num_pages)};
    const cuuint64_t strides[3] = {HD * 2, static_cast<cuuint64_t>(page) * HD * 2,
                                   static_cast<cuuint64_t>(kv_heads) * page * HD * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(page), 1, 1};  // one piece of a page
    if (!make_map4(&map_k, kcache, dims, strides, box) || !make_map4(&map_v, vcache, dims, strides, box)) {
      bw::set_error("attention (tcgen05): cuTensorMapEncodeTiled refused the cache map");
      return -1;
    }
  }
  const float scale_log2 = scale * 1.44269504088896341f;
  bw::launch_pdl(attention_tc_kernel, dim3(kv_heads, num_tiles), dim3(kThreads), kSmemBytes, stream, map_q, map_k, map_v,
                 block_table, max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out, out_stride, heads,
                 kv_heads, page, window, scale_log2, word);
  return bw::launch_status();
}

#else  // other head sizes use the kernels of bf16_attention.cu

BW_API int bw_bf16_attention_tc_tile_rows(int, int, int, int, int) { return 0; }

#endif
