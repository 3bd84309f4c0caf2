// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16, fp32 accumulation)
// for the forms the other tensor-core kernels do not take: keys and values of different sizes, keys
// of any multiple of 16 up to 1024 (a latent row), values that are the first columns of the keys'
// own rows, a sink score per head in the softmax's denominator, and a distance bias with a slope per
// head.  Prompt portions and single decoded tokens alike.
//
// A block takes R = 16 MT query rows that share one key/value head (MT = 1: four warps, for steps of
// single tokens; MT = 2 or 4: eight or sixteen warps, for prompt portions, with two buffers for the
// chunk's rows where shared memory allows, so that the next chunk is copied while this one is multiplied): with G = nq / nkv query heads per
// key/value head, the rows are (token, head in group) pairs, R / G tokens by G heads when G divides
// R, or R of the G heads of one token when R divides G.  It walks the request's keys in chunks of 64
// (cut at absolute multiples of 64): the chunk's rows are gathered from their pages into shared
// memory (un-permuted); each group of four warps owns 16 of the rows, and in it warp w computes the
// scores of keys 16 w .. 16 w + 15 (S = Q K^T), the four exchange row maxima and sums and the bf16
// weights through shared memory, and each then adds P V for its quarter of the value columns to
// accumulators in registers.  Scores, the softmax and all sums are fp32; the weights are rounded to
// bf16 for the second product.
//
// With n_splits > 1 the keys of every tile are cut into that many runs of whole chunks, one block
// each; the blocks leave unnormalised sums with their maxima and denominators in `part_o` / `part_ml`
// and attention_rows_merge_kernel adds them up (and the sink) in a fixed order.
//
// Layouts as in attention_generic.cu: q [tokens, q_stride], out [tokens, out_stride], kcache
// [pages, nkv, page_size, d], vcache [pages, nkv, page_size, dv] (null with v_prefix), block tables
// and the per-request lists of a step; tile_req / tile_tok0 list tiles of `tile_tokens` tokens.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define ROWS 16      // rows of one group of four warps
#define CHUNK 64
#define QUARTERS 4   // warps of a group: each takes a quarter of a chunk's keys and of the value columns
#define PAD 8   // bf16 elements behind every shared-memory row: rows stay 16-byte aligned, banks spread

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two 8x8 matrices, transposed: lanes 0..7 give the row addresses of the first, 8..15 of the second
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The CHUNK cache rows listed in rowbase (element offset / width; -1: none, zeros) into shared memory
// rows of `pitch` elements, their 16-byte pieces un-permuted (piece c of a row at in-page offset t
// lies at piece c ^ (t & mask)).
template <int NT>
__device__ __forceinline__ void gather_rows(bf16* __restrict__ dst, int pitch, const bf16* __restrict__ cache, int width,
                                            int mask, const int* __restrict__ rowbase, const int* __restrict__ rowoff,
                                            int tid) {
  const int pieces = width >> 3, total = CHUNK * pieces;
  for (int i0 = tid; i0 < total; i0 += 4 * NT) {
    uint4 v[4];
    int where[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = i0 + u * NT;
      v[u] = make_uint4(0, 0, 0, 0);
      where[u] = -1;
      if (idx < total) {
        const int jj = idx / pieces, c = idx - jj * pieces;
        where[u] = jj * pitch + c * 8;
        const int base = rowbase[jj];
        if (base >= 0) v[u] = *reinterpret_cast<const uint4*>(cache + (size_t)base * width + ((c ^ (rowoff[jj] & mask)) << 3));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (where[u] >= 0) *reinterpret_cast<uint4*>(dst + where[u]) = v[u];
  }
}

// The same gather as asynchronous copies (cp.async, 16 bytes each; a row that is not there is filled
// with zeros by a copy of no bytes): the caller commits the group and waits for it later.
template <int NT>
__device__ __forceinline__ void gather_rows_async(bf16* __restrict__ dst, int pitch, const bf16* __restrict__ cache,
                                                  int width, int mask, const int* __restrict__ rowbase,
                                                  const int* __restrict__ rowoff, int tid) {
  const int pieces = width >> 3, total = CHUNK * pieces;
  for (int idx = tid; idx < total; idx += NT) {
    const int jj = idx / pieces, c = idx - jj * pieces;
    const int base = rowbase[jj];
    const bf16* src = base >= 0 ? cache + (size_t)base * width + ((c ^ (rowoff[jj] & mask)) << 3) : cache;
    const unsigned to = (unsigned)__cvta_generic_to_shared(dst + jj * pitch + c * 8);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(to), "l"(src), "r"(base >= 0 ? 16 : 0) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// Which token (within the tile) and which head a row of a tile of R rows stands for.
struct RowMap {
  int G, R, kvh, hs;
  __device__ __forceinline__ int token(int r) const { return G >= R ? 0 : r / G; }
  __device__ __forceinline__ int head(int r) const { return G >= R ? kvh * G + hs * R + r : kvh * G + r % G; }
};

// DVW: value columns per warp that the accumulators have room for (dv <= 4 * DVW).  DB: two buffers for
// the chunk's rows; the next chunk is copied (cp.async) while this one is multiplied.
template <int DVW, int MT, bool DB>
__global__ void __launch_bounds__(QUARTERS * MT * 32)
attention_rows_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                      const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ table_rows,
                      int page_size, const int* __restrict__ q_start, const int* __restrict__ q_len,
                      const int* __restrict__ kv_len, const int* __restrict__ tile_req,
                      const int* __restrict__ tile_tok0, int tile_tokens, int nq, int nkv, int d, int dv, float scale,
                      const float* __restrict__ sinks, const float* __restrict__ slopes, int v_prefix,
                      int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
  mi_pdl_enter();
  constexpr int R = ROWS * MT, NW = QUARTERS * MT, NT = NW * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dp = d + PAD, dvp = dv + PAD;
  constexpr int STAGES = DB ? 2 : 1;
  const int stage_elems = CHUNK * dp + (v_prefix ? 0 : CHUNK * dvp);   // a chunk's keys [CHUNK][dp], then its values [CHUNK][dvp]
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [R][dp]
  bf16* KV = Qs + R * dp;                                       // [STAGES][stage_elems]
  bf16* Ps = KV + STAGES * stage_elems;                         // [R][CHUNK + PAD]
  float* wmax = reinterpret_cast<float*>(Ps + R * (CHUNK + PAD));      // [QUARTERS][R]
  float* wsum = wmax + QUARTERS * R;                            // [QUARTERS][R]
  int* rowbase_all = reinterpret_cast<int*>(wsum + QUARTERS * R);      // [STAGES][CHUNK] cache row of each key, -1: none
  int* rowoff_all = rowbase_all + STAGES * CHUNK;               // [STAGES][CHUNK] in-page offset of each key

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = (tid >> 5) % QUARTERS, mt = (tid >> 5) / QUARTERS;   // the quarter, and which 16 rows
  const int g = lane >> 2, t4 = lane & 3;                      // the fragment's row (and row + 8) and column pair
  const int G = nq / nkv;
  const int head_tiles = G >= R ? G / R : 1;
  int bid = blockIdx.x;
  const int split = bid % n_splits;
  bid /= n_splits;
  const int hs = bid % head_tiles;
  bid /= head_tiles;
  const int kvh = bid % nkv;
  const int tile = bid / nkv;
  const int b = tile_req[tile], tok0 = tile_tok0[tile];
  const int ql = q_len[b], kl = kv_len[b], qs = q_start[b];
  const int trow = table_rows ? table_rows[b] : b;
  const int nt = min(tile_tokens, ql - tok0);                   // tokens of this tile
  const int p0 = kl - ql + tok0;                                // position of the tile's first token
  const int j_end = p0 + nt;                                    // one past the last key any row sees

  const RowMap rows{G, R, kvh, hs};
  auto row_token = [&](int r) { return rows.token(r); };
  auto row_head = [&](int r) { return rows.head(r); };
  // this block's run of keys: whole chunks, the same cut for every row of the tile
  const int chunks_all = (j_end + CHUNK - 1) / CHUNK, chunks_mine = (chunks_all + n_splits - 1) / n_splits;
  const int j_begin = split * chunks_mine * CHUNK, j_stop = min(j_end, (split + 1) * chunks_mine * CHUNK);

  // ---- the queries: 16-byte pieces, zero for rows without a token
  const int pieces = d >> 3;
  for (int idx = tid; idx < R * pieces; idx += NT) {
    const int r = idx / pieces, c = idx - r * pieces;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row_token(r) < nt)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(qs + tok0 + row_token(r)) * q_stride + row_head(r) * d + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * dp + c * 8) = v;
  }

  // per thread: the two rows of its fragments
  const int r_lo = mt * ROWS + g, r_hi = r_lo + 8;
  const bool ok_lo = row_token(r_lo) < nt, ok_hi = row_token(r_hi) < nt;
  const int pos_lo = p0 + row_token(r_lo), pos_hi = p0 + row_token(r_hi);
  const float slope_lo = slopes ? slopes[row_head(r_lo)] : 0.f, slope_hi = slopes ? slopes[row_head(r_hi)] : 0.f;
  constexpr float LOG2E = 1.4426950408889634f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;     // running maximum (in units of log2) and sum
  float acc[DVW / 8][4];
#pragma unroll
  for (int n = 0; n < DVW / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const int col0 = warp * (dv / QUARTERS);                      // this warp's value columns
  const int ntiles_v = (dv / QUARTERS) >> 3;
  const int mk = mi_swizzle_mask_rows(d, 2), mv = mi_swizzle_mask_rows(dv, 2);
  const int vpitch = v_prefix ? dp : dvp;
  // where the 64 keys from j0 on lie in the cache (threads 0..63), into list `which`
  auto list_rows = [&](int j0, int which) {
    if (tid < CHUNK) {
      const int j = j0 + tid;
      int base = -1;
      if (j < j_stop) {
        const int page = block_table[(size_t)trow * bt_stride + j / page_size];
        base = (page * nkv + kvh) * page_size + j % page_size;
      }
      rowbase_all[which * CHUNK + tid] = base;
      rowoff_all[which * CHUNK + tid] = j % page_size;
    }
  };
  auto copy_chunk = [&](int which) {     // asynchronous copies of the chunk listed in `which` into buffer `which`
    bf16* kdst = KV + which * stage_elems;
    gather_rows_async<NT>(kdst, dp, kcache, d, mk, rowbase_all + which * CHUNK, rowoff_all + which * CHUNK, tid);
    if (!v_prefix)
      gather_rows_async<NT>(kdst + CHUNK * dp, dvp, vcache, dv, mv, rowbase_all + which * CHUNK, rowoff_all + which * CHUNK, tid);
    cp_async_commit();
  };
  if (DB && j_begin < j_stop) {
    list_rows(j_begin, 0);
    __syncthreads();
    copy_chunk(0);
    list_rows(j_begin + CHUNK, 1);
  }

  int it = 0;
  for (int j0 = j_begin; j0 < j_stop; j0 += CHUNK, ++it) {
    const int cur = DB ? (it & 1) : 0;
    const bf16* Ks = KV + cur * stage_elems;
    const bf16* Vrows = v_prefix ? Ks : Ks + CHUNK * dp;
    if (DB) {
      cp_async_wait_all();
      __syncthreads();          // this chunk has landed, the next one's rows are listed, the chunk before is consumed
      if (j0 + CHUNK < j_stop) copy_chunk(cur ^ 1);
      list_rows(j0 + 2 * CHUNK, cur);      // read after the next iteration's barrier (this chunk's list has done its work)
    } else {
      __syncthreads();                                          // the chunk before is consumed (first time: Qs written)
      list_rows(j0, 0);
      __syncthreads();
      // four 16-byte pieces per thread are asked for before the first is stored, so that they fly together
      bf16* kdst = KV;
      gather_rows<NT>(kdst, dp, kcache, d, mk, rowbase_all, rowoff_all, tid);
      if (!v_prefix) gather_rows<NT>(kdst + CHUNK * dp, dvp, vcache, dv, mv, rowbase_all, rowoff_all, tid);
      __syncthreads();
    }

    // ---- S = Q K^T for this warp's 16 keys: two tiles of 8 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    // one ldmatrix.x4 per operand and step of 16 dimensions.  A: lanes 0..15 address rows 0..15 at
    // dimension k0, lanes 16..31 the same rows at k0 + 8 (matrices a0, a1, a2, a3 in that order).  B: lanes
    // 0..7 keys 0..7 at k0, 8..15 the same keys at k0 + 8, 16..31 likewise for keys 8..15 (b0, b1 of the
    // first eight keys, then of the second eight).
    const uint32_t qaddr = (uint32_t)__cvta_generic_to_shared(Qs + (mt * ROWS + (lane & 15)) * dp + ((lane >> 4) << 3));
    const uint32_t kaddr = (uint32_t)__cvta_generic_to_shared(
        Ks + (warp * 16 + ((lane >> 4) << 3) + (lane & 7)) * dp + (((lane >> 3) & 1) << 3));
    for (int k0 = 0; k0 < d; k0 += 16) {
      uint32_t a[4], bfrag[4];
      ldmatrix_x4(a, qaddr + k0 * 2);
      ldmatrix_x4(bfrag, kaddr + k0 * 2);
      mma_bf16(s[0], a, bfrag[0], bfrag[1]);
      mma_bf16(s[1], a, bfrag[2], bfrag[3]);
    }
    // ---- scale, distance bias, mask; everything in units of log2
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + warp * 16 + n * 8 + 2 * t4 + (e & 1);
        const bool hi = e >= 2;
        const int pos = hi ? pos_hi : pos_lo;
        const bool ok = (hi ? ok_hi : ok_lo) && j <= pos;
        const float v = ok ? (s[n][e] * scale - (hi ? slope_hi : slope_lo) * (float)(pos - j)) * LOG2E : -INFINITY;
        s[n][e] = v;
        if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    if (t4 == 0) {
      wmax[warp * R + r_lo] = mx_lo;
      wmax[warp * R + r_hi] = mx_hi;
    }
    __syncthreads();
    float cm_lo = wmax[r_lo], cm_hi = wmax[r_hi];
#pragma unroll
    for (int w = 1; w < QUARTERS; ++w) {
      cm_lo = fmaxf(cm_lo, wmax[w * R + r_lo]);
      cm_hi = fmaxf(cm_hi, wmax[w * R + r_hi]);
    }
    const float mn_lo = fmaxf(m_lo, cm_lo), mn_hi = fmaxf(m_hi, cm_hi);
    const float al_lo = mn_lo == -INFINITY ? 1.f : exp2f(m_lo - mn_lo);      // m = -inf gives 0
    const float al_hi = mn_hi == -INFINITY ? 1.f : exp2f(m_hi - mn_hi);
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0v = mn_lo == -INFINITY ? 0.f : exp2f(s[n][0] - mn_lo), p1v = mn_lo == -INFINITY ? 0.f : exp2f(s[n][1] - mn_lo);
      const float p2v = mn_hi == -INFINITY ? 0.f : exp2f(s[n][2] - mn_hi), p3v = mn_hi == -INFINITY ? 0.f : exp2f(s[n][3] - mn_hi);
      const uint32_t w_lo = pack_bf16(p0v, p1v), w_hi = pack_bf16(p2v, p3v);
      // the sums count the weights as the second product will read them: rounded to bf16
      const float2 f_lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w_lo));
      const float2 f_hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w_hi));
      ps_lo += f_lo.x + f_lo.y;
      ps_hi += f_hi.x + f_hi.y;
      const int col = warp * 16 + n * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(Ps + r_lo * (CHUNK + PAD) + col) = w_lo;
      *reinterpret_cast<uint32_t*>(Ps + r_hi * (CHUNK + PAD) + col) = w_hi;
    }
    ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 1);
    ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 2);
    ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 1);
    ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 2);
    if (t4 == 0) {
      wsum[warp * R + r_lo] = ps_lo;
      wsum[warp * R + r_hi] = ps_hi;
    }
    __syncthreads();
    l_lo = l_lo * al_lo + ((wsum[r_lo] + wsum[R + r_lo]) + (wsum[2 * R + r_lo] + wsum[3 * R + r_lo]));
    l_hi = l_hi * al_hi + ((wsum[r_hi] + wsum[R + r_hi]) + (wsum[2 * R + r_hi] + wsum[3 * R + r_hi]));
    m_lo = mn_lo;
    m_hi = mn_hi;

    // ---- O = alpha O + P V for this warp's value columns
#pragma unroll
    for (int n = 0; n < DVW / 8; ++n) {
      acc[n][0] *= al_lo; acc[n][1] *= al_lo;
      acc[n][2] *= al_hi; acc[n][3] *= al_hi;
    }
    const bf16* pa = Ps + r_lo * (CHUNK + PAD) + 2 * t4;
#pragma unroll
    for (int k0 = 0; k0 < CHUNK; k0 += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(pa + k0);
      a[1] = *reinterpret_cast<const uint32_t*>(pa + 8 * (CHUNK + PAD) + k0);
      a[2] = *reinterpret_cast<const uint32_t*>(pa + k0 + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(pa + 8 * (CHUNK + PAD) + k0 + 8);
      const bf16* vrow = Vrows + (k0 + (lane & 15)) * vpitch + col0;      // lanes 0..15: the 16 keys of this step
#pragma unroll
      for (int n = 0; n < DVW / 8; ++n) {
        if (n < ntiles_v) {
          uint32_t b0, b1;
          ldmatrix_x2_trans(b0, b1, vrow + n * 8);
          mma_bf16(acc[n], a, b0, b1);
        }
      }
    }
  }

  if (n_splits > 1) {
    // ---- one of several runs of keys: unnormalised sums, maximum and denominator for the merge
    const size_t unit = (size_t)(blockIdx.x / n_splits) * n_splits + split;
    float* po = part_o + unit * R * dv;
    float* pml = part_ml + unit * R * 2;
#pragma unroll
    for (int n = 0; n < DVW / 8; ++n) {
      if (n < ntiles_v) {
        const int col = col0 + n * 8 + 2 * t4;
        *reinterpret_cast<float2*>(po + (size_t)r_lo * dv + col) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2*>(po + (size_t)r_hi * dv + col) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    if (warp == 0 && t4 == 0) {
      pml[2 * r_lo] = m_lo; pml[2 * r_lo + 1] = l_lo;
      pml[2 * r_hi] = m_hi; pml[2 * r_hi + 1] = l_hi;
    }
    return;
  }
  // ---- the sink joins the denominator once; then the rows are written
  if (sinks) {
    const float sk_lo = sinks[row_head(ok_lo ? r_lo : 0)] * LOG2E, sk_hi = sinks[row_head(ok_hi ? r_hi : 0)] * LOG2E;
    const float mf_lo = fmaxf(m_lo, sk_lo), mf_hi = fmaxf(m_hi, sk_hi);
    const float keep_lo = m_lo == -INFINITY ? 0.f : exp2f(m_lo - mf_lo), keep_hi = m_hi == -INFINITY ? 0.f : exp2f(m_hi - mf_hi);
    l_lo = l_lo * keep_lo + exp2f(sk_lo - mf_lo);
    l_hi = l_hi * keep_hi + exp2f(sk_hi - mf_hi);
#pragma unroll
    for (int n = 0; n < DVW / 8; ++n) {
      acc[n][0] *= keep_lo; acc[n][1] *= keep_lo;
      acc[n][2] *= keep_hi; acc[n][3] *= keep_hi;
    }
  }
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int n = 0; n < DVW / 8; ++n) {
    if (n < ntiles_v) {
      const int col = col0 + n * 8 + 2 * t4;
      if (ok_lo)
        *reinterpret_cast<uint32_t*>(out + (size_t)(qs + tok0 + row_token(r_lo)) * out_stride + row_head(r_lo) * dv + col) =
            pack_bf16(acc[n][0] * inv_lo, acc[n][1] * inv_lo);
      if (ok_hi)
        *reinterpret_cast<uint32_t*>(out + (size_t)(qs + tok0 + row_token(r_hi)) * out_stride + row_head(r_hi) * dv + col) =
            pack_bf16(acc[n][2] * inv_hi, acc[n][3] * inv_hi);
    }
  }
}

// Adds up the runs of keys of every row: grid = units x R rows, one block per row.  The weight of
// every run (2^(its maximum - the row's maximum)) is worked out once, into shared memory.
#define MERGE_MAX_SPLITS 64
__global__ void __launch_bounds__(128)
attention_rows_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                            int out_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
                            const int* __restrict__ tile_req, const int* __restrict__ tile_tok0, int tile_tokens,
                            int nq, int nkv, int dv, const float* __restrict__ sinks, int n_splits, int R) {
  mi_pdl_enter();
  __shared__ float weight[MERGE_MAX_SPLITS];
  __shared__ float inv_l;
  constexpr float LOG2E = 1.4426950408889634f;
  const int r = blockIdx.x % R;
  int bid = blockIdx.x / R;
  const int unit = bid;
  const int G = nq / nkv;
  const int head_tiles = G >= R ? G / R : 1;
  const int hs = bid % head_tiles;
  bid /= head_tiles;
  const int kvh = bid % nkv;
  const int tile = bid / nkv;
  const RowMap rows{G, R, kvh, hs};
  const int b = tile_req[tile], tok0 = tile_tok0[tile];
  const int nt = min(tile_tokens, q_len[b] - tok0);
  if (rows.token(r) >= nt) return;
  const int head = rows.head(r);
  const float* pml = part_ml + ((size_t)unit * n_splits * R + r) * 2;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, pml[(size_t)s * R * 2]);
    m = mi_warp_max(m);
    const float sink2 = sinks ? sinks[head] * LOG2E : -INFINITY;
    const float mf = fmaxf(m, sink2);
    float l = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 32) {     // runs in ascending order: lanes, then the warp's fixed tree
      const int s = s0 + lane;
      float w = 0.f, part = 0.f;
      if (s < n_splits) {
        const float ms = pml[(size_t)s * R * 2];
        w = ms == -INFINITY ? 0.f : exp2f(ms - mf);
        part = pml[(size_t)s * R * 2 + 1] * w;
        weight[s] = w;
      }
      l += mi_warp_sum(part);
    }
    if (sinks) l += exp2f(sink2 - mf);
    if (lane == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
  }
  __syncthreads();
  const float inv = inv_l;
  bf16* o = out + (size_t)(q_start[b] + tok0 + rows.token(r)) * out_stride + head * dv;
  const float* po = part_o + ((size_t)unit * n_splits * R + r) * dv;
  // every run has written its sums (zeros where it had no keys), so all of them are read: four columns
  // per thread, eight runs in flight
  for (int c = threadIdx.x * 4; c < dv; c += blockDim.x * 4) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 8 <= n_splits; s += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const float4*>(po + (size_t)(s + u) * R * dv + c);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float w = weight[s + u];
        sum.x += v[u].x * w; sum.y += v[u].y * w; sum.z += v[u].z * w; sum.w += v[u].w * w;
      }
    }
    for (; s < n_splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(po + (size_t)s * R * dv + c);
      const float w = weight[s];
      sum.x += v.x * w; sum.y += v.y * w; sum.z += v.z * w; sum.w += v.w * w;
    }
    *reinterpret_cast<uint2*>(o + c) = make_uint2(pack_bf16(sum.x * inv, sum.y * inv), pack_bf16(sum.z * inv, sum.w * inv));
  }
}

// Tokens per tile of `rows` rows for a group of G query heads per key/value head, or 0 when the
// kernel does not take the group size.
extern "C" int mi_attention_rows_tile_tokens(int G, int rows) {
  if (G <= 0 || (rows != ROWS && rows != 2 * ROWS && rows != 4 * ROWS)) return 0;
  if (G >= rows) return G % rows == 0 ? 1 : 0;
  return rows % G == 0 ? rows / G : 0;
}

extern "C" int mi_attention_rows_supported(int nq, int nkv, int d, int dv, int v_prefix) {
  if (nq <= 0 || nkv <= 0 || nq % nkv) return 0;
  if (!mi_attention_rows_tile_tokens(nq / nkv, ROWS)) return 0;
  if (d < 16 || d % 16 || d > 1024 || dv < 32 || dv % 32 || dv > 512) return 0;
  if (v_prefix && dv > d) return 0;
  return 1;
}

// Floats of part_o and of part_ml that a launch with these numbers needs.
extern "C" int mi_attention_rows_scratch(int n_tiles, int rows, int nq, int nkv, int dv, int n_splits,
                                         long long* o_floats, long long* ml_floats) {
  const int G = nq / nkv;
  const long long units = (long long)n_tiles * nkv * (G >= rows ? G / rows : 1);
  *o_floats = n_splits > 1 ? units * n_splits * rows * dv : 0;
  *ml_floats = n_splits > 1 ? units * n_splits * rows * 2 : 0;
  return 0;
}

extern "C" int mi_attention_rows(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                 const void* vcache, const int* block_table, int bt_stride, const int* table_rows,
                                 int page_size, const int* q_start, const int* q_len, const int* kv_len,
                                 const int* tile_req, const int* tile_tok0, int n_tiles, int tile_tokens, int rows,
                                 int nq, int nkv, int d, int dv, float scale, const float* sinks, const float* slopes,
                                 int v_prefix, int n_splits, float* part_o, float* part_ml, int stages,
                                 cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (stages != 1 && stages != 2) MI_REFUSE("attention_rows: one or two buffers for a chunk, not %d", stages);
  if ((rows == 2 * ROWS && stages != 2) || (rows == ROWS && stages != 1))
    MI_REFUSE("attention_rows: blocks of %d rows with %d buffers are not built", rows, stages);
  if (!mi_attention_rows_supported(nq, nkv, d, dv, v_prefix))
    MI_REFUSE("attention_rows: sizes not taken (heads %d over %d, keys %d, values %d)", nq, nkv, d, dv);
  const int G = nq / nkv;
  if (!mi_attention_rows_tile_tokens(G, rows) || tile_tokens != mi_attention_rows_tile_tokens(G, rows))
    MI_REFUSE("attention_rows: tiles of %d tokens and %d rows do not fit a group of %d heads", tile_tokens, rows, G);
  if (page_size <= 0) MI_REFUSE("attention_rows: bad page size %d", page_size);
  if (!v_prefix && !vcache) MI_REFUSE("attention_rows: no value cache");
  if (n_splits < 1 || n_splits > MERGE_MAX_SPLITS || (n_splits > 1 && (!part_o || !part_ml)))
    MI_REFUSE("attention_rows: 1 to %d runs of keys, and scratch for more than one", MERGE_MAX_SPLITS);
  if (!mi_aligned(q, 16) || !mi_aligned(kcache, 16) || !mi_aligned(vcache, 16) || !mi_aligned(out, 4) ||
      !mi_aligned(part_o, 16) || q_stride % 8 || out_stride % 2 || (n_splits > 1 && (!mi_aligned(out, 8) || out_stride % 4)))
    MI_REFUSE("attention_rows: q and the caches must be 16-byte aligned with rows of whole 16-byte pieces");
  const long long units = (long long)n_tiles * nkv * (G >= rows ? G / rows : 1);
  const long long blocks = units * n_splits;
  if (blocks > 0x7fffffffLL || units * rows > 0x7fffffffLL) MI_REFUSE("attention_rows: too many blocks for one launch");
  const size_t smem = ((size_t)rows * (d + PAD) +
                       (size_t)stages * ((size_t)CHUNK * (d + PAD) + (v_prefix ? 0 : (size_t)CHUNK * (dv + PAD))) +
                       (size_t)rows * (CHUNK + PAD)) * sizeof(bf16) +
                      2 * QUARTERS * rows * sizeof(float) + (size_t)stages * 2 * CHUNK * sizeof(int);
  if (smem > 227 * 1024) MI_REFUSE("attention_rows: keys of %d and values of %d do not fit in shared memory", d, dv);
#define MI_GO(DVW, MT, DB)                                                                                      \
  do {                                                                                                          \
    auto kern = attention_rows_kernel<DVW, MT, DB>;                                                             \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      if (e != cudaSuccess) return (int)e;                                                                      \
    }                                                                                                           \
    MI_LAUNCH(kern, (unsigned)blocks, QUARTERS * MT * 32, smem, stream, (const bf16*)q, q_stride, (bf16*)out,    \
              out_stride, (const bf16*)kcache, (const bf16*)vcache, block_table, bt_stride, table_rows, page_size, \
              q_start, q_len, kv_len, tile_req, tile_tok0, tile_tokens, nq, nkv, d, dv, scale, sinks, slopes,    \
              v_prefix, n_splits, part_o, part_ml);                                                             \
  } while (0)
  if (rows == ROWS) {
    if (dv <= 128) MI_GO(32, 1, false);
    else if (dv <= 256) MI_GO(64, 1, false);
    else MI_GO(128, 1, false);
  } else if (rows == 2 * ROWS) {
    if (dv <= 128) MI_GO(32, 2, true);
    else if (dv <= 256) MI_GO(64, 2, true);
    else MI_GO(128, 2, true);
  } else if (stages == 2) {
    if (dv <= 128) MI_GO(32, 4, true);
    else if (dv <= 256) MI_GO(64, 4, true);
    else MI_GO(128, 4, true);
  } else {
    if (dv <= 128) MI_GO(32, 4, false);
    else if (dv <= 256) MI_GO(64, 4, false);
    else MI_GO(128, 4, false);
  }
#undef MI_GO
  {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      snprintf(g_mi_error, sizeof(g_mi_error), "CUDA: %s", cudaGetErrorString(e));
      return (int)e;
    }
  }
  if (n_splits > 1)
    MI_LAUNCH(attention_rows_merge_kernel, (unsigned)(units * rows), 128, 0, stream, (const float*)part_o,
              (const float*)part_ml, (bf16*)out, out_stride, q_start, q_len, tile_req, tile_tok0, tile_tokens, nq, nkv,
              dv, sinks, n_splits, rows);
  MI_RETURN_LAUNCH_STATUS();
}
