// bfloat16 attention over the paged cache for prefill portions and decoded tokens alike.
//
// One kernel serves every row of a step (the reference likewise has one paged_attention for
// all rows, src/kernels.cpp:342-368). A thread block takes a tile of consecutive query rows
// of ONE sequence and one key/value head; the query heads that share this key/value head
// (src/kernels.cpp:346: kv head = h / (heads / kv_heads)) are stacked with the rows, so the
// tile's keys and values are read once for the whole group.
//
// One summation order for every shape. Keys are cut into chunks of 256 at fixed absolute
// positions. Inside a chunk the keys are walked in tiles of 64 with a running maximum and
// running sum per query row (scores, maximum, sum and the output accumulator in float32; the
// softmax weights are rounded to bfloat16 for the value product). The chunk results
// (maximum, sum, unnormalised output) are merged in ascending chunk order by one written-down
// formula (merge_state below). A prefill portion walks its chunks inside one block; a decode
// step, which has few query rows and long contexts, gives every chunk to a block of its own
// (so that the cache streams from all SMs) and a second kernel merges the stored chunk
// results in the same order. A row's arithmetic depends only on its own query, its position
// and the cached keys: tiles and chunks that lie wholly outside a row's range leave its state
// untouched bit for bit, so the result does not depend on which other rows share the block,
// on how the prompt was cut, on the batch, or on which pages hold the keys.
#include "bw_common.cuh"

#ifndef BW_HEAD_DIM
#error "compile with -DBW_HEAD_DIM=<head size, a multiple of 16>"
#endif

namespace {

constexpr int HD = BW_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int kTileM = 64;    // stacked (query row, head of the group) rows per block
constexpr int kTileKV = 64;   // keys per tile
constexpr int kChunkKV = 256; // keys per chunk of the summation order
static_assert(kChunkKV % kTileKV == 0, "a chunk is a whole number of tiles");
constexpr int kThreads = 128;
constexpr int kRowElems = HD + 8;           // padded row: 16 bytes of padding keep ldmatrix conflict-free
constexpr int kRowBytes = kRowElems * 2;
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

// Merge of a chunk result (m, l, o) into the running state (M, L, O): the new maximum, both
// sides rescaled to it. Maxima are in the base-2 exponent domain. A side that has seen no key
// (maximum -inf) gets weight 0 through a zero reference instead of inf - inf.
struct MergeWeights {
  float a, b, mx;
};
__device__ __forceinline__ MergeWeights merge_weights(float M, float m) {
  MergeWeights w;
  w.mx = fmaxf(M, m);
  const float ref = (w.mx == -INFINITY) ? 0.0f : w.mx;
  w.a = exp2f(__fsub_rn(M, ref));
  w.b = exp2f(__fsub_rn(m, ref));
  return w;
}
__device__ __forceinline__ float merge_value(float X, float x, const MergeWeights& w) {
  return __fmaf_rn(x, w.b, __fmul_rn(X, w.a));
}

// STAGES key/value tiles are in flight or in use at a time: two for prefill portions (more
// blocks per SM), four for decode steps, where a block has little arithmetic per tile and
// the time goes to waiting for memory. The arithmetic does not depend on STAGES.
template <int STAGES, bool SPLIT>
__global__ void __launch_bounds__(kThreads)
attention_bf16_kernel(const __nv_bfloat16* __restrict__ qkv, int q_stride, const __nv_bfloat16* __restrict__ kcache,
                      const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                      const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                      const int* __restrict__ tile_rows, const int* __restrict__ seq_pos0,
                      const int* __restrict__ seq_row0, __nv_bfloat16* __restrict__ out, int out_stride, int heads,
                      int kv_heads, int page, int window, float scale_log2, float* __restrict__ chunk_out,
                      int max_chunks) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sq = smem;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x, g = blockIdx.y;
  const int group = heads / kv_heads;
  const int seq = tile_seq[tile], row0 = tile_row0[tile], nrows = tile_rows[tile];
  const int mrows = nrows * group;  // stacked rows in use (<= 64)
  const int p_first = seq_pos0[seq] + (row0 - seq_row0[seq]);  // position of the tile's first query row
  const int p_last = p_first + nrows - 1;
  const int* table = block_table + static_cast<size_t>(seq) * max_blocks;

  // keys [kv_lo, kv_hi) are walked; kv_lo is a multiple of the tile size, in split mode the
  // range is cut to this block's chunk
  int kv_lo = (window > 0 && p_first - window + 1 > 0) ? ((p_first - window + 1) / kTileKV) * kTileKV : 0;
  int kv_hi = p_last + 1;
  if (SPLIT) {
    const int c = blockIdx.z;
    kv_lo = max(kv_lo, c * kChunkKV);
    kv_hi = min(kv_hi, (c + 1) * kChunkKV);
    if (kv_hi <= kv_lo) return;  // this chunk lies outside the tile's range: nothing is stored for it
  }
  const int ntiles = (kv_hi - kv_lo + kTileKV - 1) / kTileKV;

  // ---- stage Q: stacked row m = (query row m / group, head g * group + m % group) ----------
  for (int idx = tid; idx < kTileM * kPieces; idx += kThreads) {
    const int m = idx / kPieces, piece = idx - m * kPieces;
    const bool ok = m < mrows;
    const int qr = ok ? m / group : 0, hq = ok ? m - qr * group : 0;
    const __nv_bfloat16* src = qkv + static_cast<size_t>(row0 + qr) * q_stride + (g * group + hq) * HD + piece * 8;
    cp_async16(smem_u32(sq + m * kRowBytes + piece * 16), src, ok);
  }
  cp_async_commit();

  auto load_kv = [&](int stage, int t) {
    unsigned char* sk = smem + kQBytes + stage * 2 * kKVBytes;
    unsigned char* sv = sk + kKVBytes;
    const int j0 = kv_lo + t * kTileKV;
    for (int idx = tid; idx < kTileKV * kPieces; idx += kThreads) {
      const int key = idx / kPieces, piece = idx - key * kPieces;
      const int j = j0 + key;
      const bool ok = j < kv_hi;
      size_t off = 0;
      if (ok) off = ((static_cast<size_t>(table[j / page]) * kv_heads + g) * page + (j % page)) * HD + piece * 8;
      cp_async16(smem_u32(sk + key * kRowBytes + piece * 16), kcache + off, ok);
      cp_async16(smem_u32(sv + key * kRowBytes + piece * 16), vcache + off, ok);
    }
  };

#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < ntiles) load_kv(st, st);
    cp_async_commit();
  }

  // per-thread rows of the warp's 16-row slice: r_lo = lane / 4, r_hi = r_lo + 8
  const int m_lo = warp * 16 + (lane >> 2), m_hi = m_lo + 8;
  const int pos_lo = (m_lo < mrows) ? p_first + m_lo / group : p_last;
  const int pos_hi = (m_hi < mrows) ? p_first + m_hi / group : p_last;
  const int first_lo = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
  const int first_hi = (window > 0 && pos_hi - window + 1 > 0) ? pos_hi - window + 1 : 0;
  const bool warp_active = warp * 16 < mrows;

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[i][e] = 0.0f;
  float max_lo = -INFINITY, max_hi = -INFINITY, sum_lo = 0.0f, sum_hi = 0.0f;
  // running state over the chunks (whole mode only)
  float o_tot[SPLIT ? 1 : HD / 8][4];
  float Mt_lo = -INFINITY, Mt_hi = -INFINITY, Lt_lo = 0.0f, Lt_hi = 0.0f;
  if (!SPLIT) {
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o_tot[i][e] = 0.0f;
  }

  for (int t = 0; t < ntiles; ++t) {
    if (t + STAGES - 1 < ntiles) load_kv((t + STAGES - 1) % STAGES, t + STAGES - 1);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (warp_active) {
      const unsigned char* sk = smem + kQBytes + (t % STAGES) * 2 * kKVBytes;
      const unsigned char* sv = sk + kKVBytes;
      const int j0 = kv_lo + t * kTileKV;

      // ---- S = Q K^T for 16 stacked rows x 64 keys ------------------------------------------
      float s[kTileKV / 8][4];
#pragma unroll
      for (int i = 0; i < kTileKV / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4];
        {
          const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(a, smem_u32(sq + row * kRowBytes + (kk * 2 + (lane >> 4)) * 16));
        }
#pragma unroll
        for (int np = 0; np < kTileKV / 16; ++np) {
          uint32_t b[4];
          const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
          ldmatrix_x4(b, smem_u32(sk + key * kRowBytes + (kk * 2 + ((lane >> 3) & 1)) * 16));
          mma_bf16(s[2 * np], a, b[0], b[1]);
          mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
      }

      // ---- mask, running maximum ---------------------------------------------------------------
      float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < kTileKV / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + nb * 8 + 2 * (lane & 3) + (e & 1);
          const bool hi = e >= 2;
          const bool ok = hi ? (j <= pos_hi && j >= first_hi) : (j <= pos_lo && j >= first_lo);
          const float v = ok ? s[nb][e] * scale_log2 : -INFINITY;
          s[nb][e] = v;
          if (hi) tmax_hi = fmaxf(tmax_hi, v); else tmax_lo = fmaxf(tmax_lo, v);
        }
      tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
      tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
      tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
      tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
      const float new_lo = fmaxf(max_lo, tmax_lo), new_hi = fmaxf(max_hi, tmax_hi);
      // a row that has seen no key yet keeps a zero reference so that exp2(-inf - ref) = 0
      const float ref_lo = (new_lo == -INFINITY) ? 0.0f : new_lo;
      const float ref_hi = (new_hi == -INFINITY) ? 0.0f : new_hi;
      const float alpha_lo = exp2f(max_lo - ref_lo), alpha_hi = exp2f(max_hi - ref_hi);
      max_lo = new_lo;
      max_hi = new_hi;

      // ---- weights, running sum, P as the A operand ---------------------------------------------
      float tsum_lo = 0.0f, tsum_hi = 0.0f;
      uint32_t p[kTileKV / 16][4];
#pragma unroll
      for (int nb = 0; nb < kTileKV / 8; ++nb) {
        const float e0 = exp2f(s[nb][0] - ref_lo), e1 = exp2f(s[nb][1] - ref_lo);
        const float e2 = exp2f(s[nb][2] - ref_hi), e3 = exp2f(s[nb][3] - ref_hi);
        tsum_lo += e0 + e1;
        tsum_hi += e2 + e3;
        p[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16(e0, e1);
        p[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      tsum_lo += __shfl_xor_sync(0xffffffffu, tsum_lo, 1);
      tsum_lo += __shfl_xor_sync(0xffffffffu, tsum_lo, 2);
      tsum_hi += __shfl_xor_sync(0xffffffffu, tsum_hi, 1);
      tsum_hi += __shfl_xor_sync(0xffffffffu, tsum_hi, 2);
      sum_lo = sum_lo * alpha_lo + tsum_lo;
      sum_hi = sum_hi * alpha_hi + tsum_hi;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_acc[i][0] *= alpha_lo;
        o_acc[i][1] *= alpha_lo;
        o_acc[i][2] *= alpha_hi;
        o_acc[i][3] *= alpha_hi;
      }

      // ---- O += P V -----------------------------------------------------------------------------
#pragma unroll
      for (int kp = 0; kp < kTileKV / 16; ++kp) {
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t b[4];
          const int key = kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(b, smem_u32(sv + key * kRowBytes + (dp * 2 + (lane >> 4)) * 16));
          mma_bf16(o_acc[2 * dp], p[kp], b[0], b[1]);
          mma_bf16(o_acc[2 * dp + 1], p[kp], b[2], b[3]);
        }
      }

      // ---- end of a chunk: merge it into the running state and start afresh --------------------
      if (!SPLIT && (((j0 + kTileKV) % kChunkKV) == 0 || t + 1 == ntiles)) {
        const MergeWeights wl = merge_weights(Mt_lo, max_lo), wh = merge_weights(Mt_hi, max_hi);
        Mt_lo = wl.mx;
        Mt_hi = wh.mx;
        Lt_lo = merge_value(Lt_lo, sum_lo, wl);
        Lt_hi = merge_value(Lt_hi, sum_hi, wh);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o_tot[i][0] = merge_value(o_tot[i][0], o_acc[i][0], wl);
          o_tot[i][1] = merge_value(o_tot[i][1], o_acc[i][1], wl);
          o_tot[i][2] = merge_value(o_tot[i][2], o_acc[i][2], wh);
          o_tot[i][3] = merge_value(o_tot[i][3], o_acc[i][3], wh);
          o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
        }
        max_lo = max_hi = -INFINITY;
        sum_lo = sum_hi = 0.0f;
      }
    }
    __syncthreads();
  }

  if (!warp_active) return;
  if (SPLIT) {
    // ---- store this chunk's result: o[HD], then maximum and sum, per (row, head, chunk) ---------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = half ? m_hi : m_lo;
      if (m >= mrows) continue;
      const int qr = m / group, hq = m - qr * group;
      float* dst = chunk_out + ((static_cast<size_t>(row0 + qr) * heads + (g * group + hq)) * max_chunks + blockIdx.z) *
                                   (HD + 2);
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * (lane & 3)) = make_float2(o_acc[i][half * 2], o_acc[i][half * 2 + 1]);
      if ((lane & 3) == 0) {
        dst[HD] = half ? max_hi : max_lo;
        dst[HD + 1] = half ? sum_hi : sum_lo;
      }
    }
    return;
  }
  // ---- normalise and store ---------------------------------------------------------------------
  const float inv_lo = __fdiv_rn(1.0f, Lt_lo), inv_hi = __fdiv_rn(1.0f, Lt_hi);
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

// Second half of split mode: per (row, head) the chunk results are merged in ascending chunk
// order with the same formula as above; thread d carries output element d.
__global__ void merge_chunks_kernel(const float* __restrict__ chunk_out, int max_chunks, const int* __restrict__ pos,
                                    __nv_bfloat16* __restrict__ out, int out_stride, int heads, int window) {
  const int r = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int p = pos[r];
  const int c_first = (window > 0 && p - window + 1 > 0) ? (p - window + 1) / kChunkKV : 0;
  const int c_last = p / kChunkKV;
  const float* src = chunk_out + (static_cast<size_t>(r) * heads + h) * max_chunks * (HD + 2);
  float M = -INFINITY, L = 0.0f, O = 0.0f;
  for (int c = c_first; c <= c_last; ++c) {
    const float* s = src + static_cast<size_t>(c) * (HD + 2);
    const MergeWeights w = merge_weights(M, s[HD]);
    M = w.mx;
    L = merge_value(L, s[HD + 1], w);
    O = merge_value(O, s[d], w);
  }
  out[static_cast<size_t>(r) * out_stride + h * HD + d] = __float2bfloat16_rn(__fmul_rn(O, __fdiv_rn(1.0f, L)));
}

}  // namespace

BW_API int bw_bf16_attention_head_dim() { return HD; }

// Floats of scratch that split mode needs for `n` rows whose longest context is `max_keys`.
BW_API long long bw_bf16_attention_scratch_floats(int n, int heads, int max_keys) {
  const long long chunks = (max_keys + kChunkKV - 1) / kChunkKV;
  return static_cast<long long>(n) * heads * chunks * (HD + 2);
}

BW_API int bw_bf16_attention(const __nv_bfloat16* qkv, int q_stride, const __nv_bfloat16* kcache,
                             const __nv_bfloat16* vcache, const int* block_table, int max_blocks,
                             const int* tile_seq, const int* tile_row0, const int* tile_rows, int num_tiles,
                             const int* seq_pos0, const int* seq_row0, const int* pos, __nv_bfloat16* out,
                             int out_stride, int n, int heads, int kv_heads, int hd, int page, int window,
                             float scale, int max_keys, float* scratch, cudaStream_t stream) {
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
  if (kv_heads > 65535 || heads > 65535) {
    bw::set_error("attention: %d heads exceed the grid limit", heads);
    return -1;
  }
  const float scale_log2 = scale * 1.44269504088896341f;
  const int chunks = (max_keys + kChunkKV - 1) / kChunkKV;
  // decode steps (every tile a single row) with more than one chunk run split, if the caller
  // gave scratch; both ways give the same bits
  const bool split = scratch != nullptr && n == num_tiles && chunks > 1 && chunks <= 65535;
  static bool configured[2] = {false, false};
  auto run = [&](auto kernel, int stages, int which, dim3 grid, float* chunk_out) -> int {
    const int smem = kQBytes + stages * 2 * kKVBytes;
    if (!configured[which]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        bw::set_error("attention: cannot raise shared memory to %d: %s", smem, cudaGetErrorString(e));
        return static_cast<int>(e);
      }
      configured[which] = true;
    }
    kernel<<<grid, kThreads, smem, stream>>>(qkv, q_stride, kcache, vcache, block_table, max_blocks, tile_seq,
                                             tile_row0, tile_rows, seq_pos0, seq_row0, out, out_stride, heads, kv_heads,
                                             page, window, scale_log2, chunk_out, chunks);
    return 0;
  };
  if (split) {
    const int rc = run(attention_bf16_kernel<3, true>, 3, 1, dim3(num_tiles, kv_heads, chunks), scratch);
    if (rc) return rc;
    merge_chunks_kernel<<<dim3(n, heads), HD, 0, stream>>>(scratch, chunks, pos, out, out_stride, heads, window);
  } else {
    const int rc = run(attention_bf16_kernel<2, false>, 2, 0, dim3(num_tiles, kv_heads), nullptr);
    if (rc) return rc;
  }
  return bw::launch_status();
}
