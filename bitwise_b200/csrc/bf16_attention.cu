// bfloat16 attention over the paged cache for prefill portions and decoded tokens alike.
//
// One kernel serves every row of a step (the reference likewise has one paged_attention for
// all rows, src/kernels.cpp:342-368). A thread block takes a tile of consecutive query rows
// of ONE sequence and one key/value head; the query heads that share this key/value head
// (src/kernels.cpp:346: kv head = h / (heads / kv_heads)) are stacked with the rows, so the
// tile's keys and values are read once for the whole group.
//
// One summation order for every shape. Keys are cut into tiles of 64 at fixed absolute
// positions [64 t, 64 t + 64). Each tile gives, per query row, the maximum of its scores, the
// sum of exp(score - maximum) and the unnormalised output sum(exp(...) v) (scores, maximum,
// sum and output in float32; the weights are rounded to bfloat16 for the value product). The
// tile results are merged in ascending tile order by one written-down formula (merge_weights
// / merge_value below). A prefill portion walks its tiles inside one block; a decode step,
// which has few query rows and long contexts, gives every tile to a block of one warp (so
// that the cache streams from all SMs; the tile arrives by cp.async, at head size 64 as TMA
// page boxes, and for steps of many rows through the rings of persistent blocks), and a
// second kernel merges the stored tile results in the same order. A row's arithmetic depends only on its own query,
// its position and the cached keys: tiles that lie wholly outside a row's range merge as an
// exact no-op, so the result does not depend on which other rows share the block, on how the
// prompt was cut, on the batch, or on which pages hold the keys.
#include <cuda.h>

#include "bw_common.cuh"

#ifndef BW_HEAD_DIM
#error "compile with -DBW_HEAD_DIM=<head size, a multiple of 16>"
#endif

namespace {

constexpr int HD = BW_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int kTileM = 64;    // stacked (query row, head of the group) rows per block
constexpr int kTileKV = 64;   // keys per tile
// Key tiles per block in split mode, one per warp. One: a block is a single warp with its own
// 16 KB of keys and values, a dozen of them share an SM, and each leaves as soon as its tile
// is done, so loads stay in flight all the time (with four warps per block that wait for each
// other the same kernel was a tenth slower).
constexpr int kSplitWarps = 1;
constexpr int kThreads = 128;
// Rows of Q, K and V tiles in shared memory. When a row is a whole number of 128-byte lines
// the 16-byte pieces of a line are xor-swizzled with the row number; other head sizes get 16
// bytes of padding per row. Either way eight consecutive rows of one piece fall into
// distinct banks for ldmatrix.
constexpr bool kSwizzle = (HD % 64 == 0);
constexpr int kRowBytes = kSwizzle ? HD * 2 : HD * 2 + 16;
__device__ __forceinline__ int piece_offset(int row, int piece) {
  return row * kRowBytes + (kSwizzle ? (((piece & ~7) | ((piece ^ row) & 7)) << 4) : (piece << 4));
}
constexpr int kQBytes = kTileM * kRowBytes;
constexpr int kKVBytes = kTileKV * kRowBytes;
constexpr int kPieces = HD / 8;             // 16-byte pieces per row

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
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Merge of a tile result (m, l, o) into the running state (M, L, O): the new maximum, both
// sides rescaled to it. Maxima are in the base-2 exponent domain. A side that has seen no key
// (maximum -inf) gets weight 0 through a zero reference instead of inf - inf.
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

// What one warp holds of a tile result: rows lane / 4 ("lo") and lane / 4 + 8 ("hi") of its 16
// stacked rows; o[i][0..1] are columns 8 i + 2 (lane % 4) + {0, 1} of row lo, o[i][2..3] of row hi.
struct TileResult {
  float o[HD / 8][4];
  float max_lo, max_hi, sum_lo, sum_hi;
};

// One tile of 64 keys for the 16 stacked rows of one warp: S = Q K^T (scaled to the base-2
// domain), mask, maximum, weights, sum, o = P V from zero. sq points at the warp's 16 rows of
// Q, sk / sv at the tile's keys and values in shared memory (padded rows of kRowBytes).
// Both modes call this one function, so a tile gives the same bits in both.
__device__ __forceinline__ void attend_tile(const unsigned char* sq, const unsigned char* sk, const unsigned char* sv,
                                            int lane, int j0, int pos_lo, int pos_hi, int first_lo, int first_hi,
                                            float scale_log2, TileResult& r) {
  float s[kTileKV / 8][4];
#pragma unroll
  for (int i = 0; i < kTileKV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
  // The fragments of a k-step are all fetched before its MMAs are issued (the statements keep
  // their order in the machine code): the loads' latencies overlap instead of adding up.
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    uint32_t a[4];
    {
      const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(a, smem_u32(sq + piece_offset(row, kk * 2 + (lane >> 4))));
    }
    uint32_t b[kTileKV / 16][4];
#pragma unroll
    for (int np = 0; np < kTileKV / 16; ++np) {
      const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
      ldmatrix_x4(b[np], smem_u32(sk + piece_offset(key, kk * 2 + ((lane >> 3) & 1))));
    }
#pragma unroll
    for (int np = 0; np < kTileKV / 16; ++np) {
      mma_bf16(s[2 * np], a, b[np][0], b[np][1]);
      mma_bf16(s[2 * np + 1], a, b[np][2], b[np][3]);
    }
  }
  // maximum of the raw scores (scaling by a positive factor commutes with the maximum), then
  // weights e = 2^(s * scale - ref) with one fused multiply-add per key
  float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
  // a tile that lies wholly inside both rows' ranges needs no per-key test (same values either way)
  const bool inside = j0 + kTileKV - 1 <= min(pos_lo, pos_hi) && j0 >= max(first_lo, first_hi);
  if (inside) {
#pragma unroll
    for (int nb = 0; nb < kTileKV / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (e >= 2) tmax_hi = fmaxf(tmax_hi, s[nb][e]); else tmax_lo = fmaxf(tmax_lo, s[nb][e]);
      }
  } else {
#pragma unroll
    for (int nb = 0; nb < kTileKV / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nb * 8 + 2 * (lane & 3) + (e & 1);
        const bool hi = e >= 2;
        const bool ok = hi ? (j <= pos_hi && j >= first_hi) : (j <= pos_lo && j >= first_lo);
        const float v = ok ? s[nb][e] : -INFINITY;
        s[nb][e] = v;
        if (hi) tmax_hi = fmaxf(tmax_hi, v); else tmax_lo = fmaxf(tmax_lo, v);
      }
  }
  tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
  tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
  tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
  tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
  tmax_lo = __fmul_rn(tmax_lo, scale_log2);
  tmax_hi = __fmul_rn(tmax_hi, scale_log2);
  // a row with no key in this tile keeps a zero reference so that 2^(-inf - ref) = 0
  const float nref_lo = (tmax_lo == -INFINITY) ? 0.0f : -tmax_lo;
  const float nref_hi = (tmax_hi == -INFINITY) ? 0.0f : -tmax_hi;
  float tsum_lo = 0.0f, tsum_hi = 0.0f;
  uint32_t p[kTileKV / 16][4];
#pragma unroll
  for (int nb = 0; nb < kTileKV / 8; ++nb) {
    const float e0 = bw::exp2_approx(__fmaf_rn(s[nb][0], scale_log2, nref_lo));
    const float e1 = bw::exp2_approx(__fmaf_rn(s[nb][1], scale_log2, nref_lo));
    const float e2 = bw::exp2_approx(__fmaf_rn(s[nb][2], scale_log2, nref_hi));
    const float e3 = bw::exp2_approx(__fmaf_rn(s[nb][3], scale_log2, nref_hi));
    tsum_lo = __fadd_rn(tsum_lo, __fadd_rn(e0, e1));
    tsum_hi = __fadd_rn(tsum_hi, __fadd_rn(e2, e3));
    p[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16(e0, e1);
    p[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(e2, e3);
  }
  tsum_lo = __fadd_rn(tsum_lo, __shfl_xor_sync(0xffffffffu, tsum_lo, 1));
  tsum_lo = __fadd_rn(tsum_lo, __shfl_xor_sync(0xffffffffu, tsum_lo, 2));
  tsum_hi = __fadd_rn(tsum_hi, __shfl_xor_sync(0xffffffffu, tsum_hi, 1));
  tsum_hi = __fadd_rn(tsum_hi, __shfl_xor_sync(0xffffffffu, tsum_hi, 2));
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) r.o[i][e] = 0.0f;
#pragma unroll
  for (int kp = 0; kp < kTileKV / 16; ++kp) {
    // four value fragments at a time: fetched together, then their MMAs
#pragma unroll
    for (int d0 = 0; d0 < HD / 16; d0 += 4) {
      uint32_t b[4][4];
#pragma unroll
      for (int dd = 0; dd < 4; ++dd) {
        if (d0 + dd < HD / 16) {
          const int key = kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(b[dd], smem_u32(sv + piece_offset(key, (d0 + dd) * 2 + (lane >> 4))));
        }
      }
#pragma unroll
      for (int dd = 0; dd < 4; ++dd) {
        if (d0 + dd < HD / 16) {
          mma_bf16(r.o[2 * (d0 + dd)], p[kp], b[dd][0], b[dd][1]);
          mma_bf16(r.o[2 * (d0 + dd) + 1], p[kp], b[dd][2], b[dd][3]);
        }
      }
    }
  }
  r.max_lo = tmax_lo;
  r.max_hi = tmax_hi;
  r.sum_lo = tsum_lo;
  r.sum_hi = tsum_hi;
}

// cp.async of `count` threads (whole warps): one tile of keys and values from the
// paged cache into shared memory; keys at or beyond kv_hi are zero-filled. A thread keeps its
// 16-byte piece and walks the keys; page_shift is log2(page) when the page size is a power of
// two, else -1. The page ids of the tile are read first, one per lane, and handed round by
// shuffle: a table entry read inside the walk would put a round trip to memory (a few hundred
// cycles, one after the other) before every pair of copies, and the issue of a tile's copies
// took three times as long as the tile's arithmetic.
__device__ __forceinline__ void load_kv_tile(unsigned char* sk, unsigned char* sv, const __nv_bfloat16* kcache,
                                             const __nv_bfloat16* vcache, const int* table, int page, int page_shift,
                                             int kv_heads, int g, int j0, int kv_hi, int t, int count) {
  const int piece = t % kPieces;
  const int keys_per_pass = count / kPieces;  // threads beyond a whole number of keys copy nothing
  const bool copies = t < keys_per_pass * kPieces;
  // tiles start on multiples of kTileKV: with a power-of-two page of at most kTileKV keys a tile is
  // whole pages, at most 32 of them when a page has two keys or more
  const bool by_lane = page_shift >= 1 && page <= kTileKV;
  int my_page = 0;
  if (by_lane) {
    const int lane = t & 31, first = j0 >> page_shift;
    if (lane < (kTileKV >> page_shift) && ((first + lane) << page_shift) < kv_hi) my_page = table[first + lane];
  }
  const int passes = (kTileKV + keys_per_pass - 1) / keys_per_pass;  // the same for every thread: all lanes meet in the shuffle
  for (int i = 0; i < passes; ++i) {
    const int key = t / kPieces + i * keys_per_pass;
    const bool in_tile = copies && key < kTileKV;
    const int j = j0 + (in_tile ? key : 0);
    const bool ok = in_tile && j < kv_hi;
    int page_id = 0, slot = 0;
    if (by_lane) {
      page_id = __shfl_sync(0xffffffffu, my_page, (j - j0) >> page_shift);
      slot = j & (page - 1);
    } else if (ok) {
      const int blk = page_shift >= 0 ? j >> page_shift : j / page;
      slot = page_shift >= 0 ? j & (page - 1) : j - blk * page;
      page_id = table[blk];
    }
    if (!in_tile) continue;
    const size_t off = ok ? ((static_cast<size_t>(page_id) * kv_heads + g) * page + slot) * HD + piece * 8 : 0;
    cp_async16(smem_u32(sk + piece_offset(key, piece)), kcache + off, ok);
    cp_async16(smem_u32(sv + piece_offset(key, piece)), vcache + off, ok);
  }
}

// ---------------------------------------------------------------------------------------
// Whole mode: a block takes a tile of up to 64 stacked rows (query rows of one sequence x the
// heads of one group) and walks the key tiles in order, two tiles of keys in flight.
constexpr int kStages = 2;

__global__ void __launch_bounds__(kThreads)
attention_whole_kernel(const __nv_bfloat16* __restrict__ qkv, int q_stride, const __nv_bfloat16* __restrict__ kcache,
                       const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                       const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                       const int* __restrict__ seq_row0, __nv_bfloat16* __restrict__ out, int out_stride, int heads,
                       int kv_heads, int page, int page_shift, int window, float scale_log2) {
  bw::pdl_enter();
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sq = smem;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.y, g = blockIdx.x;  // heads fastest: the host lists the longest tiles first
  const int group = heads / kv_heads;
  const int seq = tile_seq[tile], row0 = tile_row0[tile], nrows = tile_rows[tile];
  const int mrows = nrows * group;  // stacked rows in use (<= 64)
  const int p_first = seq_pos0[seq] + (row0 - seq_row0[seq]);  // position of the tile's first query row
  const int p_last = p_first + nrows - 1;
  const int* table = block_table + static_cast<size_t>(seq) * max_blocks;

  // stacked row m = (query row m / group, head g * group + m % group)
  for (int idx = tid; idx < kTileM * kPieces; idx += kThreads) {
    const int m = idx / kPieces, piece = idx - m * kPieces;
    const bool ok = m < mrows;
    const int qr = ok ? m / group : 0, hq = ok ? m - qr * group : 0;
    const __nv_bfloat16* src = qkv + static_cast<size_t>(row0 + qr) * q_stride + (g * group + hq) * HD + piece * 8;
    cp_async16(smem_u32(sq + piece_offset(m, piece)), src, ok);
  }
  cp_async_commit();

  const int kv_lo = (window > 0 && p_first - window + 1 > 0) ? ((p_first - window + 1) / kTileKV) * kTileKV : 0;
  const int kv_hi = p_last + 1;  // keys [kv_lo, kv_hi) are walked
  const int ntiles = (kv_hi - kv_lo + kTileKV - 1) / kTileKV;
  auto stage_k = [&](int st) { return smem + kQBytes + st * 2 * kKVBytes; };

  load_kv_tile(stage_k(0), stage_k(0) + kKVBytes, kcache, vcache, table, page, page_shift, kv_heads, g, kv_lo, kv_hi, tid,
               kThreads);
  cp_async_commit();

  const int m_lo = warp * 16 + (lane >> 2), m_hi = m_lo + 8;
  const int pos_lo = (m_lo < mrows) ? p_first + m_lo / group : p_last;
  const int pos_hi = (m_hi < mrows) ? p_first + m_hi / group : p_last;
  const int first_lo = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
  const int first_hi = (window > 0 && pos_hi - window + 1 > 0) ? pos_hi - window + 1 : 0;
  const bool warp_active = warp * 16 < mrows;

  float o_tot[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_tot[i][e] = 0.0f;
  float M_lo = -INFINITY, M_hi = -INFINITY, L_lo = 0.0f, L_hi = 0.0f;

  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles)
      load_kv_tile(stage_k((t + 1) & 1), stage_k((t + 1) & 1) + kKVBytes, kcache, vcache, table, page, page_shift, kv_heads, g,
                   kv_lo + (t + 1) * kTileKV, kv_hi, tid, kThreads);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (warp_active) {
      TileResult r;
      attend_tile(sq + warp * 16 * kRowBytes, stage_k(t & 1), stage_k(t & 1) + kKVBytes, lane, kv_lo + t * kTileKV, pos_lo,
                  pos_hi, first_lo, first_hi, scale_log2, r);
      const MergeWeights wl = merge_weights(M_lo, r.max_lo), wh = merge_weights(M_hi, r.max_hi);
      M_lo = wl.mx;
      M_hi = wh.mx;
      L_lo = merge_value(L_lo, r.sum_lo, wl);
      L_hi = merge_value(L_hi, r.sum_hi, wh);
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_tot[i][0] = merge_value(o_tot[i][0], r.o[i][0], wl);
        o_tot[i][1] = merge_value(o_tot[i][1], r.o[i][1], wl);
        o_tot[i][2] = merge_value(o_tot[i][2], r.o[i][2], wh);
        o_tot[i][3] = merge_value(o_tot[i][3], r.o[i][3], wh);
      }
    }
    __syncthreads();
  }

  if (!warp_active) return;
  const float inv_lo = __fdiv_rn(1.0f, L_lo), inv_hi = __fdiv_rn(1.0f, L_hi);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = half ? m_hi : m_lo;
    if (m >= mrows) continue;
    const int qr = m / group, hq = m - qr * group;
    __nv_bfloat16* dst = out + static_cast<size_t>(row0 + qr) * out_stride + (g * group + hq) * HD + 2 * (lane & 3);
    const float inv = half ? inv_hi : inv_lo;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const uint32_t v = pack_bf16(__fmul_rn(o_tot[i][half * 2], inv), __fmul_rn(o_tot[i][half * 2 + 1], inv));
      *reinterpret_cast<uint32_t*>(dst + i * 8) = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Split mode (decode steps: one query row per sequence, at most 16 stacked rows): a block
// takes (row, key/value head, kSplitWarps consecutive key tiles), each warp one tile of its
// own: it loads the tile, computes the tile result and stores it. Record layout per (row,
// head, tile): o[HD], maximum, sum.
constexpr int kSplitQBytes = 16 * kRowBytes;

__global__ void __launch_bounds__(kSplitWarps * 32)
attention_split_kernel(const __nv_bfloat16* __restrict__ qkv, int q_stride, const __nv_bfloat16* __restrict__ kcache,
                       const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ row_seq, const int* __restrict__ pos, int heads, int kv_heads, int page,
                       int page_shift, int window, float scale_log2, float* __restrict__ tile_out, int max_tiles) {
  // The step's index arrays (positions, row -> sequence, block tables) were copied to the
  // device before the step's first kernel, and the keys and values of a tile that ends before
  // the row's own position were stored by earlier steps: those loads are issued before the
  // wait for the previous kernel (which stores this step's key and value and rotates q), so
  // they overlap its tail.
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sq = smem;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x, g = blockIdx.y;
  const int group = heads / kv_heads;  // stacked rows in use (<= 16)
  const int p = pos[row];
  const int first = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int t = blockIdx.z * kSplitWarps + warp;  // this warp's key tile
  const int block_first_tile = blockIdx.z * kSplitWarps;
  if (block_first_tile * kTileKV > p || (block_first_tile + kSplitWarps) * kTileKV <= first) {
    bw::pdl_enter();
    return;  // nothing in range
  }
  const int* table = block_table + static_cast<size_t>(row_seq[row]) * max_blocks;
  const bool mine = t * kTileKV <= p && (t + 1) * kTileKV > first;  // the tile holds a key of the row's range
  const bool settled = (t + 1) * kTileKV <= p;                      // all of it was stored by earlier steps
  unsigned char* sk = smem + kSplitQBytes + warp * 2 * kKVBytes;
  unsigned char* sv = sk + kKVBytes;
  if (mine && settled)
    load_kv_tile(sk, sv, kcache, vcache, table, page, page_shift, kv_heads, g, t * kTileKV, p + 1, lane, 32);
  bw::pdl_enter();

  for (int idx = tid; idx < 16 * kPieces; idx += kSplitWarps * 32) {
    const int m = idx / kPieces, piece = idx - m * kPieces;
    const bool ok = m < group;
    const __nv_bfloat16* src = qkv + static_cast<size_t>(row) * q_stride + (g * group + (ok ? m : 0)) * HD + piece * 8;
    cp_async16(smem_u32(sq + piece_offset(m, piece)), src, ok);
  }
  if (mine && !settled)
    load_kv_tile(sk, sv, kcache, vcache, table, page, page_shift, kv_heads, g, t * kTileKV, p + 1, lane, 32);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();  // Q was loaded by all warps
  if (!mine) return;

  TileResult r;
  attend_tile(sq, sk, sv, lane, t * kTileKV, p, p, first, first, scale_log2, r);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = (lane >> 2) + half * 8;
    if (m >= group) continue;
    float* dst = tile_out + ((static_cast<size_t>(row) * heads + (g * group + m)) * max_tiles + t) * (HD + 2);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<float2*>(dst + i * 8 + 2 * (lane & 3)) = make_float2(r.o[i][half * 2], r.o[i][half * 2 + 1]);
    if ((lane & 3) == 0) {
      dst[HD] = half ? r.max_hi : r.max_lo;
      dst[HD + 1] = half ? r.sum_hi : r.sum_lo;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Split mode for head size 64, as a stream (decode steps, where the cache is all that is read).
// One block per SM stays for the whole launch; each of its warps walks work items (row,
// key/value head, key tile) and keeps a ring of three of them in shared memory. An item is
// fetched by TMA: the page of a head is one box of 2 KB (a row of 64 values is a 128-byte line,
// and the 128-byte swizzle of the copy is the layout that attend_tile reads), so a tile of keys
// and values is eight copies instead of a thousand 16-byte ones, and the query row is one
// more. Tiles that earlier steps stored are requested before the wait for the kernel before
// this one. The arithmetic and the records are those of attention_split_kernel (same bits).
#if BW_HEAD_DIM == 64
constexpr int kStreamWarps = 6;
constexpr int kStreamStages = 2;
constexpr int kStreamMaxRows = 512;  // rows of a step whose positions fit into shared memory beside the rings
constexpr int kStreamQBytes = 16 * 128;                       // 16 stacked rows; a step's row fills `group` of them
constexpr int kStreamItemBytes = kStreamQBytes + 2 * kKVBytes;  // 18 KB, a multiple of 1024

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// raises the bytes that the barrier's current phase expects, without arriving
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// gives up after a limit and raises the library's failure word: the outputs of this launch are
// then worthless, and the host learns of it
__device__ __forceinline__ void mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* failure) {
  bw::mbar_wait_bounded(bar, parity, reinterpret_cast<volatile uint32_t*>(failure));
}
__device__ __forceinline__ void tma_box_4d(void* dst, const CUtensorMap* map, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(0), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// map_q: [row][kv head][head of the group][64], box = the group's heads of one row and kv head.
// map_k / map_v: [page][kv head][slot][64], box = one page of one kv head.
//
// Work items are the (row, key tile) pairs that hold a key of the row's range, in row order,
// times the key/value heads, heads fastest (neighbouring items read neighbouring heads of the
// same pages). Warp w of block b takes items b * kStreamWarps + w, + gridDim.x * kStreamWarps, ...
// Positions, the rows' sequences and the running count of tiles per row are put into shared
// memory once, so that finding an item costs no trip to global memory; the page numbers of
// an item are fetched one item before they are needed.
__global__ void __launch_bounds__(kStreamWarps * 32)
attention_stream_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ row_seq, const int* __restrict__ pos, int n, int heads, int kv_heads,
                        int page, int window, float scale_log2, float* __restrict__ tile_out, int max_tiles,
                        int* failure) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = bw::smem_align_1024(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = heads / kv_heads;
  unsigned char* ring = smem + warp * (kStreamStages * kStreamItemBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStreamWarps * kStreamStages * kStreamItemBytes) + warp * kStreamStages;
  int* s_cum = reinterpret_cast<int*>(smem + kStreamWarps * kStreamStages * (kStreamItemBytes + 8));  // [n + 1] tiles before row r
  int* s_pos = s_cum + n + 1;
  int* s_seq = s_pos + n;
  const int pages_per_tile = kTileKV / page;
  const int stride = static_cast<int>(gridDim.x) * kStreamWarps;

  // rows of the query tiles beyond the group stay zero for the whole launch
  for (int s = 0; s < kStreamStages; ++s)
    for (int b = lane * 16; b < kStreamQBytes; b += 32 * 16)
      *reinterpret_cast<uint4*>(ring + s * kStreamItemBytes + b) = make_uint4(0u, 0u, 0u, 0u);
  if (lane == 0) {
    for (int s = 0; s < kStreamStages; ++s) mbar_init(bars + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the zeros above were written through the generic proxy; the copies go through the async one
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  auto first_key = [&](int p) { return (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0; };
  // positions and sequences were copied to the device before the step's first kernel
  for (int r = tid; r < n; r += kStreamWarps * 32) {
    const int p = pos[r];
    s_pos[r] = p;
    s_seq[r] = row_seq[r];
    s_cum[r + 1] = p / kTileKV - first_key(p) / kTileKV + 1;  // tiles of row r, summed up below
  }
  __syncthreads();
  if (warp == 0) {  // running sum over the rows, 32 at a time
    int base = 0;
    for (int r0 = 0; r0 < n; r0 += 32) {
      int v = r0 + lane < n ? s_cum[r0 + lane + 1] : 0;
      for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += u;
      }
      if (r0 + lane < n) s_cum[r0 + lane + 1] = base + v;
      base += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) s_cum[0] = 0;
  }
  __syncthreads();
  const int total = s_cum[n] * kv_heads;

  struct Item {
    int row, g, t, p;
  };
  // item `id` (< total); `row` is a cursor that only moves forward
  auto find_item = [&](int id, int& row, Item& it) {
    const int j = id / kv_heads;
    it.g = id - j * kv_heads;
    while (j >= s_cum[row + 1]) ++row;
    it.row = row;
    it.p = s_pos[row];
    it.t = first_key(it.p) / kTileKV + (j - s_cum[row]);
  };
  // the page of the item's tile that lane `lane` (< pages_per_tile) looks up
  auto lookup_page = [&](const Item& it) {
    // pages wholly beyond the last key are not in the table: any valid page will do, its keys are masked
    const int blk = min((it.t * kTileKV) / page + lane, it.p / page);
    return block_table[static_cast<size_t>(s_seq[it.row]) * max_blocks + blk];
  };
  // requests keys and values of an item, given the pages that lanes 0 .. pages_per_tile - 1 hold
  auto request_kv = [&](const Item& it, int my_page, unsigned char* buf, uint64_t* bar) {
    for (int pg = 0; pg < pages_per_tile; ++pg) {
      const int blk = __shfl_sync(0xffffffffu, my_page, pg);
      if (lane == 0) {
        tma_box_4d(buf + kStreamQBytes + pg * page * 128, &map_k, it.g, blk, bar);
        tma_box_4d(buf + kStreamQBytes + kKVBytes + pg * page * 128, &map_v, it.g, blk, bar);
      }
    }
  };
  const uint32_t q_bytes = static_cast<uint32_t>(group) * 128, kv_bytes = 2 * kKVBytes;

  // The ring's first items. Keys and values that earlier steps stored do not depend on the
  // kernel before this one (which rotates q and stores this step's key and value).
  int req_id = static_cast<int>(blockIdx.x) * kStreamWarps + warp, req_row = 0;
  Item first_items[kStreamStages];
  int first_pages[kStreamStages];
  bool early[kStreamStages];
  int primed = 0;
  for (; primed < kStreamStages && req_id < total; ++primed, req_id += stride) {
    Item& it = first_items[primed];
    find_item(req_id, req_row, it);
    first_pages[primed] = lane < pages_per_tile ? lookup_page(it) : 0;
    early[primed] = (it.t + 1) * kTileKV <= it.p;
    if (early[primed]) {
      if (lane == 0) mbar_expect_tx(bars + primed, kv_bytes);
      __syncwarp();
      request_kv(it, first_pages[primed], ring + primed * kStreamItemBytes, bars + primed);
    }
  }
  bw::pdl_launch();
  bw::pdl_wait();
  for (int s = 0; s < primed; ++s) {
    const Item& it = first_items[s];
    unsigned char* buf = ring + s * kStreamItemBytes;
    if (lane == 0) {
      mbar_arrive_expect_tx(bars + s, early[s] ? q_bytes : q_bytes + kv_bytes);
      tma_box_4d(buf, &map_q, it.g, it.row, bars + s);
    }
    __syncwarp();
    if (!early[s]) request_kv(it, first_pages[s], buf, bars + s);
  }
  // the item that the next request will bring, and its pages
  Item nx;
  int nx_page = 0;
  bool nx_ok = req_id < total;
  if (nx_ok) {
    find_item(req_id, req_row, nx);
    nx_page = lane < pages_per_tile ? lookup_page(nx) : 0;
  }

  int use_row = 0;
  uint32_t used = 0;
  for (int use_id = static_cast<int>(blockIdx.x) * kStreamWarps + warp; use_id < total; use_id += stride, ++used) {
    Item it;
    find_item(use_id, use_row, it);
    const int first = first_key(it.p);
    const int stage = used % kStreamStages;
    unsigned char* buf = ring + stage * kStreamItemBytes;
    mbar_wait_bounded(bars + stage, (used / kStreamStages) & 1, failure);
    TileResult r;
    attend_tile(buf, buf + kStreamQBytes, buf + kStreamQBytes + kKVBytes, lane, it.t * kTileKV, it.p, it.p, first, first,
                scale_log2, r);
    // the buffer is free (every ldmatrix of the item has delivered): the next item of the ring
    // takes it; the pages of the one after are looked up now and used a whole item later
    __syncwarp();
    if (nx_ok) {
      if (lane == 0) {
        mbar_arrive_expect_tx(bars + stage, q_bytes + kv_bytes);
        tma_box_4d(buf, &map_q, nx.g, nx.row, bars + stage);
      }
      __syncwarp();
      request_kv(nx, nx_page, buf, bars + stage);
      req_id += stride;
      nx_ok = req_id < total;
      if (nx_ok) {
        find_item(req_id, req_row, nx);
        nx_page = lane < pages_per_tile ? lookup_page(nx) : 0;
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = (lane >> 2) + half * 8;
      if (m >= group) continue;
      float* dst = tile_out + ((static_cast<size_t>(it.row) * heads + (it.g * group + m)) * max_tiles + it.t) * (HD + 2);
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * (lane & 3)) = make_float2(r.o[i][half * 2], r.o[i][half * 2 + 1]);
      if ((lane & 3) == 0) {
        dst[HD] = half ? r.max_hi : r.max_lo;
        dst[HD + 1] = half ? r.sum_hi : r.sum_lo;
      }
    }
  }
}

// The per-tile blocks of attention_split_kernel (one warp, one key tile, a dozen blocks on an SM)
// with the tile's keys and values fetched as TMA boxes: a page of a head is one box, eight
// boxes a tile, asked for by one lane, instead of 32 warp-wide cp.async of four lines each
// (whose issue was a third of a block's time). The query row still comes by cp.async, the
// arithmetic and the record are attend_tile's: same bits. For steps of fewer rows than the
// streaming kernel above is worth its set-up for.
__global__ void __launch_bounds__(32)
attention_tile_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const __nv_bfloat16* __restrict__ qkv, int q_stride, const int* __restrict__ block_table,
                          int max_blocks, const int* __restrict__ row_seq, const int* __restrict__ pos, int heads,
                          int kv_heads, int page, int window, float scale_log2, float* __restrict__ tile_out, int max_tiles,
                          int* failure) {
  extern __shared__ __align__(1024) unsigned char tile_raw[];
  unsigned char* base = bw::smem_align_1024(tile_raw);
  unsigned char* sq = base;                  // 16 stacked rows of 128 bytes
  unsigned char* sk = base + kStreamQBytes;  // the boxes' swizzle is the layout that attend_tile reads
  unsigned char* sv = sk + kKVBytes;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sv + kKVBytes);
  const int lane = threadIdx.x;
  const int row = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int group = heads / kv_heads;
  const int p = pos[row];
  const int first = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  if (t * kTileKV > p || (t + 1) * kTileKV <= first) {
    bw::pdl_enter();
    return;  // no key of the row's range in this tile
  }
  if (lane == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int* table = block_table + static_cast<size_t>(row_seq[row]) * max_blocks;
  const int pages_per_tile = kTileKV / page;
  // pages wholly beyond the row's last key are not in the table: the last page stands in, its keys are masked
  const int my_page = lane < pages_per_tile ? table[min(t * pages_per_tile + lane, p / page)] : 0;
  const bool settled = (t + 1) * kTileKV <= p;  // all of the tile was stored by earlier steps
  auto request = [&]() {
    if (lane == 0) mbar_arrive_expect_tx(bar, 2 * kKVBytes);
    __syncwarp();
    for (int pg = 0; pg < pages_per_tile; ++pg) {
      const int blk = __shfl_sync(0xffffffffu, my_page, pg);
      if (lane == 0) {
        tma_box_4d(sk + pg * page * 128, &map_k, g, blk, bar);
        tma_box_4d(sv + pg * page * 128, &map_v, g, blk, bar);
      }
    }
  };
  if (settled) request();  // before the wait for the kernel that rotates q and stores this step's key and value
  bw::pdl_enter();
  for (int idx = lane; idx < 16 * kPieces; idx += 32) {
    const int m = idx / kPieces, piece = idx - m * kPieces;
    const bool ok = m < group;
    const __nv_bfloat16* src = qkv + static_cast<size_t>(row) * q_stride + (g * group + (ok ? m : 0)) * HD + piece * 8;
    cp_async16(smem_u32(sq + piece_offset(m, piece)), src, ok);
  }
  cp_async_commit();
  if (!settled) request();
  cp_async_wait<0>();
  if (!bw::mbar_wait_bounded(bar, 0, reinterpret_cast<volatile uint32_t*>(failure))) return;
  __syncwarp();

  TileResult r;
  attend_tile(sq, sk, sv, lane, t * kTileKV, p, p, first, first, scale_log2, r);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = (lane >> 2) + half * 8;
    if (m >= group) continue;
    float* dst = tile_out + ((static_cast<size_t>(row) * heads + (g * group + m)) * max_tiles + t) * (HD + 2);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<float2*>(dst + i * 8 + 2 * (lane & 3)) = make_float2(r.o[i][half * 2], r.o[i][half * 2 + 1]);
    if ((lane & 3) == 0) {
      dst[HD] = half ? r.max_hi : r.max_lo;
      dst[HD + 1] = half ? r.sum_hi : r.sum_lo;
    }
  }
}
#endif  // BW_HEAD_DIM == 64

// Second half of split mode: per (row, head) the tile results are merged in ascending tile
// order with the same formula as in whole mode; thread d carries output element d. The records
// of up to kMergeBatch tiles are brought into shared memory by all threads together (one
// round trip to memory instead of one per tile), then each thread walks them in order.
constexpr int kMergeBatch = (10 * 1024) / (HD + 2) > 64 ? 64 : (10 * 1024) / (HD + 2);  // at most 40 KB of records
constexpr int kMergeThreads = HD < 64 ? 64 : HD;

__global__ void __launch_bounds__(kMergeThreads)
merge_tiles_kernel(const float* __restrict__ tile_out, int max_tiles, const int* __restrict__ pos,
                   __nv_bfloat16* __restrict__ out, int out_stride, int heads, int window) {
  __shared__ float rec[kMergeBatch * (HD + 2)];
  const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int p = pos[r];  // copied before the step began
  const int t_first = (window > 0 && p - window + 1 > 0) ? (p - window + 1) / kTileKV : 0;
  const int t_last = p / kTileKV;
  const float* src = tile_out + (static_cast<size_t>(r) * heads + h) * max_tiles * (HD + 2);
  bw::pdl_enter();
  float M = -INFINITY, L = 0.0f, O = 0.0f;
  for (int t0 = t_first; t0 <= t_last; t0 += kMergeBatch) {
    const int count = min(kMergeBatch, t_last + 1 - t0);
    const int floats = count * (HD + 2);
    const float* from = src + static_cast<size_t>(t0) * (HD + 2);
    if (t0 > t_first) __syncthreads();  // the previous batch has been read
    for (int i = d; i < floats; i += kMergeThreads) rec[i] = __ldcg(from + i);
    __syncthreads();
    if (d < HD) {
      for (int t = 0; t < count; ++t) {
        const float* s0 = rec + t * (HD + 2);
        const MergeWeights w = merge_weights(M, s0[HD]);
        M = w.mx, L = merge_value(L, s0[HD + 1], w), O = merge_value(O, s0[d], w);
      }
    }
  }
  if (d < HD) out[static_cast<size_t>(r) * out_stride + h * HD + d] = __float2bfloat16_rn(__fmul_rn(O, __fdiv_rn(1.0f, L)));
}

}  // namespace

BW_API int bw_bf16_attention_head_dim() { return HD; }

// Floats of scratch that split mode needs for `n` rows whose longest context is `max_keys`.
BW_API long long bw_bf16_attention_scratch_floats(int n, int heads, int max_keys) {
  const long long tiles = (max_keys + kTileKV - 1) / kTileKV;
  return static_cast<long long>(n) * heads * tiles * (HD + 2);
}

BW_API int bw_bf16_attention(const __nv_bfloat16* qkv, int q_stride, const __nv_bfloat16* kcache,
                             const __nv_bfloat16* vcache, const int* block_table, int max_blocks,
                             const int* tile_seq, const int* tile_row0, const int* tile_rows, int num_tiles,
                             const int* seq_pos0, const int* seq_row0, const int* row_seq, const int* pos,
                             __nv_bfloat16* out, int out_stride, int n, int heads, int kv_heads, int hd, int page,
                             int window, float scale, int max_keys, float* scratch, cudaStream_t stream) {
  if (n <= 0 || num_tiles <= 0) return 0;
  if (hd != HD) {
    bw::set_error("attention: this library was compiled for head size %d, got %d", HD, hd);
    return -1;
  }
  if (heads % kv_heads || heads / kv_heads > kTileM) {
    bw::set_error("attention: %d heads over %d key/value heads (group must divide and be at most %d)", heads,
                  kv_heads, kTileM);
    return -1;
  }
  if (q_stride % 8 || out_stride % 2) {
    bw::set_error("attention: row strides %d / %d are not aligned for 16-byte loads", q_stride, out_stride);
    return -1;
  }
  if (kv_heads > 65535 || heads > 65535 || num_tiles > 65535) {
    bw::set_error("attention: %d heads or %d query tiles exceed the grid limit", heads, num_tiles);
    return -1;
  }
  const float scale_log2 = scale * 1.44269504088896341f;
  int page_shift = -1;
  for (int b = 0; b < 30; ++b)
    if ((1 << b) == page) page_shift = b;
  const int key_tiles = (max_keys + kTileKV - 1) / kTileKV;
  constexpr int split_smem = kSplitQBytes + kSplitWarps * 2 * kKVBytes;
  // decode steps (every query tile a single row) over more than a few key tiles run split, if
  // the caller gave scratch and a group fits one warp; both ways give the same bits
  const bool split = scratch != nullptr && n == num_tiles && key_tiles > 2 && heads / kv_heads <= 16 &&
                     split_smem <= 200 * 1024 && (key_tiles + kSplitWarps - 1) / kSplitWarps <= 65535;
  static bool configured[2] = {false, false};
  if (split) {
    if (!configured[1]) {
      cudaError_t e = cudaFuncSetAttribute(attention_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, split_smem);
      if (e != cudaSuccess) {
        bw::set_error("attention: cannot raise shared memory to %d: %s", split_smem, cudaGetErrorString(e));
        return static_cast<int>(e);
      }
      configured[1] = true;
    }
    bw::launch_pdl(attention_split_kernel, dim3(dim3(n, kv_heads, (key_tiles + kSplitWarps - 1) / kSplitWarps)), dim3(kSplitWarps * 32), split_smem, stream, qkv, q_stride, kcache, vcache, block_table, max_blocks, row_seq, pos, heads,
                                       kv_heads, page, page_shift, window, scale_log2, scratch, key_tiles);
    bw::launch_pdl(merge_tiles_kernel, dim3(dim3(n, heads)), dim3(kMergeThreads), 0, stream, scratch, key_tiles, pos, out, out_stride, heads, window);
  } else {
    constexpr int smem = kQBytes + kStages * 2 * kKVBytes;
    if (!configured[0]) {
      cudaError_t e = cudaFuncSetAttribute(attention_whole_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        bw::set_error("attention: cannot raise shared memory to %d: %s", smem, cudaGetErrorString(e));
        return static_cast<int>(e);
      }
      configured[0] = true;
    }
    bw::launch_pdl(attention_whole_kernel, dim3(dim3(kv_heads, num_tiles)), dim3(kThreads), smem, stream, 
        qkv, q_stride, kcache, vcache, block_table, max_blocks, tile_seq, tile_row0, tile_rows, seq_pos0, seq_row0, out,
        out_stride, heads, kv_heads, page, page_shift, window, scale_log2);
  }
  return bw::launch_status();
}

#if BW_HEAD_DIM == 64
namespace {
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled stream_encoder() {
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
bool stream_map(CUtensorMap* map, const void* base, const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3],
                const cuuint32_t (&box)[4]) {
  EncodeTiled enc = stream_encoder();
  if (!enc) return false;
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
int g_stream_mode = 1;  // 0 never, 1 for steps of many rows, 2 whenever the shape allows
constexpr int kStreamMinRows = 32;
}  // namespace

// How decode steps fetch the cache where the shape allows TMA boxes: 0 never (the cp.async blocks
// of attention_split_kernel), 1 (the default) the streaming kernel for steps of 32 rows or more
// and a block per key tile fed by boxes for fewer (measured on B200: with few rows the set-up of
// a persistent block costs more than its steadier stream of loads gains), 2 the streaming kernel
// whenever the shape allows. Returns the previous setting. Tests compare the kernels bit for bit.
BW_API int bw_bf16_attention_stream_mode(int mode) {
  const int before = g_stream_mode;
  if (mode >= 0 && mode <= 2) g_stream_mode = mode;
  return before;
}

// Whether decode steps of this shape can take bw_bf16_attention_stream: head size 64, pages of 8
// keys or more that divide a tile of 64, a group of at most 16 heads, rows that start on 16
// bytes, and a step of at most 512 rows.
BW_API int bw_bf16_attention_stream_usable(int n, int heads, int kv_heads, int hd, int page, int q_stride) {
  if (!g_stream_mode || hd != HD || kv_heads <= 0 || heads % kv_heads || n > kStreamMaxRows) return 0;
  const int group = heads / kv_heads;
  return group <= 16 && page >= 8 && kTileKV % page == 0 && q_stride % 8 == 0 && stream_encoder() != nullptr;
}

// A decode step (one query row per sequence): tile results by the streaming kernel, then the
// ordered merge. `scratch` as for bw_bf16_attention (bw_bf16_attention_scratch_floats).
BW_API int bw_bf16_attention_stream(const __nv_bfloat16* qkv, int q_stride, const __nv_bfloat16* kcache,
                                    const __nv_bfloat16* vcache, int num_pages, const int* block_table, int max_blocks,
                                    const int* row_seq, const int* pos, __nv_bfloat16* out, int out_stride, int n,
                                    int heads, int kv_heads, int hd, int page, int window, float scale, int max_keys,
                                    float* scratch, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!bw_bf16_attention_stream_usable(n, heads, kv_heads, hd, page, q_stride) || !scratch || out_stride % 2) {
    bw::set_error("attention (stream): unsupported shape (heads %d/%d, head size %d, page %d)", heads, kv_heads, hd, page);
    return -1;
  }
  const int key_tiles = (max_keys + kTileKV - 1) / kTileKV;
  const long long items = static_cast<long long>(n) * kv_heads * key_tiles;
  if (items > 0x3fffffffLL || heads > 65535 || n > kStreamMaxRows) {
    bw::set_error("attention (stream): %lld work items exceed the limit", items);
    return -1;
  }
  const int group = heads / kv_heads;
  const int smem = kStreamWarps * kStreamStages * (kStreamItemBytes + 8) + (3 * n + 1) * 4 + 1024;
  constexpr int smem_max = kStreamWarps * kStreamStages * (kStreamItemBytes + 8) + (3 * kStreamMaxRows + 1) * 4 + 1024;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
    if (e != cudaSuccess) {
      bw::set_error("attention (stream): cannot raise shared memory to %d: %s", smem_max, cudaGetErrorString(e));
      return static_cast<int>(e);
    }
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    configured = true;
  }
  CUtensorMap map_q, map_k, map_v;
  {  // queries: [row][kv head][head of the group][d], box = the group's heads of one row
    const cuuint64_t dims[4] = {HD, static_cast<cuuint64_t>(group), static_cast<cuuint64_t>(kv_heads),
                                static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[3] = {HD * 2, static_cast<cuuint64_t>(group) * HD * 2, static_cast<cuuint64_t>(q_stride) * 2};
    const cuuint32_t box[4] = {HD, static_cast<cuuint32_t>(group), 1, 1};
    if (!stream_map(&map_q, qkv, dims, strides, box)) {
      bw::set_error("attention (stream): cuTensorMapEncodeTiled refused the query map");
      return -1;
    }
  }
  {  // cache: [page][kv head][slot][d], box = one page of one kv head
    const cuuint64_t dims[4] = {HD, static_cast<cuuint64_t>(page), static_cast<cuuint64_t>(kv_heads),
                                static_cast<cuuint64_t>(num_pages)};
    const cuuint64_t strides[3] = {HD * 2, static_cast<cuuint64_t>(page) * HD * 2,
                                   static_cast<cuuint64_t>(kv_heads) * page * HD * 2};
    const cuuint32_t box[4] = {HD, static_cast<cuuint32_t>(page), 1, 1};
    if (!stream_map(&map_k, kcache, dims, strides, box) || !stream_map(&map_v, vcache, dims, strides, box)) {
      bw::set_error("attention (stream): cuTensorMapEncodeTiled refused the cache map");
      return -1;
    }
  }
  int* word = bw::failure_word();
  if (!word) return -1;
  const float scale_log2 = scale * 1.44269504088896341f;
  if (g_stream_mode == 1 && n < kStreamMinRows) {  // few rows: a block per key tile, fed by the same boxes
    constexpr int tile_smem = kStreamItemBytes + 8 + 1024;
    if (key_tiles > 65535 || kv_heads > 65535) {
      bw::set_error("attention: %d key tiles or %d key/value heads exceed the grid limit", key_tiles, kv_heads);
      return -1;
    }
    bw::launch_pdl(attention_tile_tma_kernel, dim3(n, kv_heads, key_tiles), dim3(32), tile_smem, stream, map_k, map_v, qkv,
                   q_stride, block_table, max_blocks, row_seq, pos, heads, kv_heads, page, window, scale_log2, scratch,
                   key_tiles, word);
    bw::launch_pdl(merge_tiles_kernel, dim3(dim3(n, heads)), dim3(kMergeThreads), 0, stream, scratch, key_tiles, pos, out,
                   out_stride, heads, window);
    return bw::launch_status();
  }
  const long long warps_needed = (items + 0) / 1;
  const unsigned grid = static_cast<unsigned>(
      warps_needed < static_cast<long long>(sms) * kStreamWarps ? (warps_needed + kStreamWarps - 1) / kStreamWarps : sms);
  bw::launch_pdl(attention_stream_kernel, dim3(grid), dim3(kStreamWarps * 32), smem, stream, map_q, map_k, map_v,
                 block_table, max_blocks, row_seq, pos, n, heads, kv_heads, page, window, scale_log2, scratch, key_tiles,
                 word);
  bw::launch_pdl(merge_tiles_kernel, dim3(dim3(n, heads)), dim3(kMergeThreads), 0, stream, scratch, key_tiles, pos, out,
                 out_stride, heads, window);
  return bw::launch_status();
}
#else
BW_API int bw_bf16_attention_stream_mode(int) { return 0; }
BW_API int bw_bf16_attention_stream_usable(int, int, int, int, int, int) { return 0; }
#endif
