// Latent attention on the tensor cores (bfloat16 cache): the kernel of attention_latent.cu with mma.sync.
//
// The queries are R-wide vectors in the latent space, one per (token, head); keys and values are the cached
// latents themselves, shared by all heads.  So the heads of a token are rows of one tile: a block takes BM = 16
// or 64 consecutive (token, head) rows of one request, holds them as bfloat16 in shared memory, and walks the
// request's pages in tiles of 64 latents that it copies once (cp.async, two buffers) and uses twice:
//
//   S = Q C^T      [BM x 64], summed over R       mma.m16n8k16, C read as the col-major operand
//   P = softmax tile by tile in float32 (running maximum and sum per row, rows rescaled when the maximum moves)
//   O += P C       [BM x R], summed over 64 keys  the same tile read as the row-major operand (ldmatrix.trans)
//
// The eight warps share S by (row tile, key group) and O by columns: every warp owns R/8 columns of all rows,
// so O never leaves its registers.  S, P and the rows' maxima, sums and rescale factors pass through shared
// memory.  R is padded with zero columns to a multiple of 64.  With few tiles and long contexts the keys of a
// tile are cut into splits (blockIdx.y) whose unnormalised sums a second kernel merges.
//
// Scores, maxima, sums and O are float32; Q and P enter the products rounded to bfloat16, C is bfloat16 as
// cached.  Causal: key j is visible to a row whose token is at position p iff j <= p.
//
// Options: a cached row may be wider than the latent (R columns, of which the first `vrank` are the latent that
// serves as value; the rest, a rotated key part that all heads share, enters the scores only: O is formed over
// all R columns and the first vrank are written).  window > 0 hides keys j <= p - window, and the tiles wholly
// behind the window of a tile's first row are never read.  sink ([n_heads] or null): one more term exp(sink[h])
// without a value in the denominator, added once, at the end (by the merge kernel when the keys are split).
#include "common.cuh"

namespace {
constexpr int PAD = 8;            // bfloat16 elements of padding per shared-memory row (keeps ldmatrix conflict-free)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x2(unsigned (&r)[2], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned (&r)[2], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct HeadLayout { long long row, head; };

struct LatentTiles {
  const int* block_tables;    // [n_entries, bt_stride]
  int bt_stride;
  const int* tile_entry;      // [n_tiles]
  const int* tile_row0;       // [n_tiles] first (token, head) row of the tile within its entry, a multiple of BM
  const int* entry_q_start;
  const int* entry_q_len;
  const int* entry_ctx_start;
};

// MT: row tiles of 16 per block (BM = 16 MT); RT: R padded to 64 RT columns; NARROW: tiles of 32 latents instead of
// 64, so that two blocks of 16 rows fit an SM at every rank (taken when there are more blocks than SMs).
template <int MT, int RT, bool NARROW>
__global__ void __launch_bounds__(256)
attn_latent_mma_kernel(const float* __restrict__ q, HeadLayout ql, bf16* __restrict__ out, HeadLayout ol,
                       const bf16* __restrict__ cache, long long page_stride, int page_size, int page_shift,
                       LatentTiles b, int n_heads, int rank, float scale, int n_splits,
                       float* __restrict__ part_o, float* __restrict__ part_ml, int vrank, int window,
                       const float* __restrict__ sink) {
  constexpr bool BY_R = MT <= 2 && RT >= 2;
  constexpr int BN = NARROW ? 32 : 64;
  constexpr int BM = 16 * MT, RP = 64 * RT, LD = RP + PAD, LDP = BN + PAD, LDS = BN + 4;
  // S is shared out over the 8 warps in one of two ways.  By keys (NP == 1): a warp takes one row tile and MT of the 8
  // key tiles over all of R.  By R (NP > 1, taken for the low tiles of decode steps where the sums over R would
  // otherwise be one long chain of dependent products): a warp takes one row tile, all 8 key tiles and 1/NP of R,
  // and the NP partial scores are added when the softmax reads them.
  constexpr int NP = BY_R ? 8 / MT : 1;
  constexpr int NT_S = BY_R ? BN / 8 : MT;
  pdl_enter();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                    // [BM][LD]
  bf16* cs = qs + BM * LD;                                          // [2][BN][LD]
  bf16* ps = cs + 2 * BN * LD;                                      // [BM][LDP]
  float* ss = reinterpret_cast<float*>(ps + BM * LDP);              // [NP][BM][LDS]
  float* row_m = ss + NP * BM * LDS;                                // [BM]
  float* row_l = row_m + BM;
  float* row_a = row_l + BM;
  int* row_pos = reinterpret_cast<int*>(row_a + BM);                // [BM] position of each row's token, -1 = no such row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int e = b.tile_entry[tile];
  const int row0 = b.tile_row0[tile];
  const int q_len = b.entry_q_len[e];
  const int n_rows = min(BM, q_len * n_heads - row0);               // rows of the tile that exist
  const int tok0 = b.entry_q_start[e], pos0 = b.entry_ctx_start[e];
  const int* bt = b.block_tables + (size_t)e * b.bt_stride;
  const int last_tok = (row0 + n_rows - 1) / n_heads;
  const int kend = pos0 + last_tok;                                 // last key any row of the tile may see
  const int key_tiles = kend / BN + 1;
  const int kt_first = window > 0 ? max(0, pos0 + row0 / n_heads - window + 1) / BN : 0;     // tiles before it lie behind every row's window
  const int per = (key_tiles - kt_first + n_splits - 1) / n_splits;
  const int kt_lo = kt_first + split * per, kt_hi = min(key_tiles, kt_lo + per);

  // zero the padding columns once (no copy ever touches them), load Q as bfloat16
  for (int idx = tid; idx < (BM + 2 * BN) * (LD - rank); idx += blockDim.x) {
    const int r = idx / (LD - rank), c = rank + idx % (LD - rank);
    qs[r * LD + c] = __float2bfloat16_rn(0.0f);                     // qs and cs are contiguous: r runs over both
  }
  if (((ql.row | ql.head) & 3) == 0 && ((uintptr_t)q & 15) == 0) {
    // sixteen threads a row, 16 bytes a load: one division per row instead of two per element
    for (int r = tid >> 4; r < BM; r += 16) {
      const int rr = row0 + r, t = rr / n_heads, h = rr - t * n_heads;
      const float4* src = reinterpret_cast<const float4*>(q + (size_t)(tok0 + t) * ql.row + (size_t)h * ql.head);
      for (int c = tid & 15; c < (rank >> 2); c += 16) {
        const float4 v = r < n_rows ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&lo);
        u.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(qs + r * LD + 4 * c) = u;
      }
    }
  } else {
    for (int idx = tid; idx < BM * rank; idx += blockDim.x) {
      const int r = idx / rank, d = idx - r * rank;
      float v = 0.0f;
      if (r < n_rows) {
        const int rr = row0 + r, t = rr / n_heads, h = rr - t * n_heads;
        v = q[(size_t)(tok0 + t) * ql.row + (size_t)h * ql.head + d];
      }
      qs[r * LD + d] = __float2bfloat16_rn(v);
    }
  }
  for (int r = tid; r < BM; r += blockDim.x) {
    row_m[r] = -INFINITY;
    row_l[r] = 0.0f;
    row_pos[r] = r < n_rows ? pos0 + (row0 + r) / n_heads : -1;
  }

  // a warp copies whole latents (one block-table look-up each), its lanes the 16-byte chunks of one
  auto load_tile = [&](int kt, int buf) {
    bf16* dst = cs + (size_t)buf * BN * LD;
    const int chunks = rank >> 3;
    // the pages of this warp's latents are looked up side by side (one wait for memory, not one per latent)
    int my_page = -1;
    if (lane < BN / 8) {
      const int key = kt * BN + warp + 8 * lane;
      if (key <= kend) my_page = bt[key >> page_shift];
    }
#pragma unroll
    for (int jj = 0; jj < BN / 8; ++jj) {
      const int j = warp + 8 * jj;
      const int key = kt * BN + j;
      const int page = __shfl_sync(0xffffffffu, my_page, jj);
      bf16* d = dst + j * LD;
      if (page >= 0) {
        const bf16* src = cache + (size_t)page * page_stride + (size_t)(key & (page_size - 1)) * rank;
        for (int c = lane; c < chunks; c += 32) cp_async16(d + c * 8, src + c * 8);
      } else {
        for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  float o[MT][RT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < RT; ++n) { o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.0f; }

  const int sm = warp % MT;                                         // this warp's row tile in S
  const int sg = NP > 1 ? 0 : warp / MT;                            // its group of key tiles (by keys)
  const int sp = NP > 1 ? warp / MT : 0;                            // its part of R (by R)
  constexpr int KSTEPS = RP / 16 / NP;                              // steps of 16 columns this warp sums over
  if (kt_lo < kt_hi) load_tile(kt_lo, 0);
  cp_async_commit();
  for (int kt = kt_lo; kt < kt_hi; ++kt) {
    const int buf = (kt - kt_lo) & 1;
    if (kt + 1 < kt_hi) load_tile(kt + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                                // tile kt has landed; Q and the row state are written
    const bf16* ct = cs + (size_t)buf * BN * LD;
    // ---- S = Q C^T for this warp's (row tile, key tiles)
    float s[NT_S][4];
#pragma unroll
    for (int j = 0; j < NT_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
    {
      // fragments of step k + 1 are asked for before the products of step k are issued
      const bf16* qa = qs + (sm * 16 + (lane & 15)) * LD + (lane >> 4) * 8 + sp * KSTEPS * 16;
      const bf16* cb = ct + (sg * NT_S * 8 + (lane & 7)) * LD + ((lane >> 3) & 1) * 8 + sp * KSTEPS * 16;
      unsigned a[2][4], bb[2][NT_S][2];
      ldsm_x4(a[0], qa);
#pragma unroll
      for (int j = 0; j < NT_S; ++j) ldsm_x2(bb[0][j], cb + j * 8 * LD);
#pragma unroll 2
      for (int k = 0; k < KSTEPS; ++k) {
        const int cur = k & 1, nxt = cur ^ 1;
        if (k + 1 < KSTEPS) {
          ldsm_x4(a[nxt], qa + (k + 1) * 16);
#pragma unroll
          for (int j = 0; j < NT_S; ++j) ldsm_x2(bb[nxt][j], cb + j * 8 * LD + (k + 1) * 16);
        }
#pragma unroll
        for (int j = 0; j < NT_S; ++j) mma_bf16(s[j], a[cur], bb[cur][j][0], bb[cur][j][1]);
      }
    }
#pragma unroll
    for (int j = 0; j < NT_S; ++j) {
      const int col = (sg * NT_S + j) * 8 + 2 * tq;
      float* d0 = ss + (sp * BM + sm * 16 + g) * LDS + col;
      float* d1 = ss + (sp * BM + sm * 16 + g + 8) * LDS + col;
      d0[0] = s[j][0]; d0[1] = s[j][1]; d1[0] = s[j][2]; d1[1] = s[j][3];
    }
    __syncthreads();
    // ---- softmax of the tile: a warp takes BM / 8 rows, a lane two keys of a row
    for (int r = warp * (BM / 8); r < (warp + 1) * (BM / 8); ++r) {
      const int p = row_pos[r];                                      // -1 hides every key from a row that does not exist
      constexpr int KPL = BN / 32;                                   // keys a lane
      const int key = kt * BN + KPL * lane;
      const bool v0 = key <= p && (window <= 0 || key > p - window);
      const bool v1 = KPL > 1 && key + 1 <= p && (window <= 0 || key + 1 > p - window);
      float sc0, sc1 = 0.0f;
      if constexpr (KPL == 2) {
        float2 sc = *reinterpret_cast<const float2*>(ss + r * LDS + 2 * lane);
#pragma unroll
        for (int part = 1; part < NP; ++part) {
          const float2 more = *reinterpret_cast<const float2*>(ss + (part * BM + r) * LDS + 2 * lane);
          sc.x += more.x;
          sc.y += more.y;
        }
        sc0 = sc.x;
        sc1 = sc.y;
      } else {
        sc0 = ss[r * LDS + lane];
#pragma unroll
        for (int part = 1; part < NP; ++part) sc0 += ss[(part * BM + r) * LDS + lane];
      }
      const float s0 = v0 ? sc0 * scale : -INFINITY;
      const float s1 = v1 ? sc1 * scale : -INFINITY;
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      float p0 = 0.0f, p1 = 0.0f, alpha = 1.0f;
      if (m_new != -INFINITY) {
        alpha = expf(m_old - m_new);
        p0 = v0 ? expf(s0 - m_new) : 0.0f;
        p1 = v1 ? expf(s1 - m_new) : 0.0f;
      }
      // the sum is taken over the weights as they enter the product
      float sum;
      if constexpr (KPL == 2) {
        const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
        *reinterpret_cast<__nv_bfloat162*>(ps + r * LDP + 2 * lane) = pp;
        sum = warp_sum(__low2float(pp) + __high2float(pp));
      } else {
        const bf16 pb = __float2bfloat16_rn(p0);
        ps[r * LDP + lane] = pb;
        sum = warp_sum(__bfloat162float(pb));
      }
      if (lane == 0) { row_m[r] = m_new; row_l[r] = row_l[r] * alpha + sum; row_a[r] = alpha; }
    }
    __syncthreads();
    // ---- O = O * alpha + P C for this warp's columns
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float a0 = row_a[m * 16 + g], a1 = row_a[m * 16 + g + 8];
#pragma unroll
      for (int n = 0; n < RT; ++n) { o[m][n][0] *= a0; o[m][n][1] *= a0; o[m][n][2] *= a1; o[m][n][3] *= a1; }
    }
    {
      const bf16* pb = ps + (lane & 15) * LDP + (lane >> 4) * 8;
      const bf16* vb = ct + (lane & 15) * LD + warp * RT * 8;
      unsigned bb[2][2];
      ldsm_x2_trans(bb[0], vb);
#pragma unroll
      for (int k = 0; k < BN / 16; ++k) {
        unsigned pa[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) ldsm_x4(pa[m], pb + m * 16 * LDP + k * 16);
#pragma unroll
        for (int n = 0; n < RT; ++n) {
          const int at = k * RT + n, cur = at & 1, nxt = cur ^ 1;
          if (at + 1 < (BN / 16) * RT) {
            const int k2 = (at + 1) / RT, n2 = (at + 1) % RT;
            ldsm_x2_trans(bb[nxt], vb + k2 * 16 * LD + n2 * 8);
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) mma_bf16(o[m][n], pa[m], bb[cur][0], bb[cur][1]);
        }
      }
    }
    __syncthreads();                                                // the tile's buffer, S and P may be written again
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- output: normalised rows, or this split's unnormalised sums with their maxima and sums
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = m * 16 + g + 8 * half;
      if (r >= n_rows) continue;
      const int rr = row0 + r, t = rr / n_heads, h = rr - t * n_heads;
      if (n_splits == 1) {
        float l = row_l[r], keep = 1.0f;
        if (sink) {                // the sink joins the denominator: everything is brought to the larger maximum
          const float mx = fmaxf(row_m[r], sink[h]);
          keep = expf(row_m[r] - mx);
          l = l * keep + expf(sink[h] - mx);
        }
        const float inv = l > 0.0f ? keep / l : 0.0f;
        bf16* orow = out + (size_t)(tok0 + t) * ol.row + (size_t)h * ol.head;
#pragma unroll
        for (int n = 0; n < RT; ++n) {
          const int col = (warp * RT + n) * 8 + 2 * tq;
          if (col < vrank)         // vrank is a multiple of 8: col + 1 < vrank too
            *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(o[m][n][2 * half] * inv, o[m][n][2 * half + 1] * inv);
        }
      } else {
        float* prow = part_o + ((size_t)(tile * n_splits + split) * BM + r) * rank;
#pragma unroll
        for (int n = 0; n < RT; ++n) {
          const int col = (warp * RT + n) * 8 + 2 * tq;
          if (col < rank) { prow[col] = o[m][n][2 * half]; prow[col + 1] = o[m][n][2 * half + 1]; }
        }
      }
    }
  }
  if (n_splits > 1)
    for (int r = tid; r < n_rows; r += blockDim.x) {
      float* ml = part_ml + ((size_t)(tile * n_splits + split) * BM + r) * 2;
      ml[0] = row_m[r];
      ml[1] = row_l[r];
    }
}

// One block per (tile, row): the splits' sums brought to a common maximum and added.  The weight of every split
// (its share of the common sum) is worked out once per row; the sums of the splits are then read side by side.
__global__ void attn_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, HeadLayout ol, LatentTiles b, int n_heads, int rank,
                                         int n_splits, int bm, int vrank, const float* __restrict__ sink) {
  pdl_enter();
  __shared__ float w[64];
  const int tile = blockIdx.x, r = blockIdx.y;
  const int e = b.tile_entry[tile], row0 = b.tile_row0[tile];
  const int rr = row0 + r;
  if (rr >= b.entry_q_len[e] * n_heads) return;
  const int t = rr / n_heads, h = rr - t * n_heads;
  const size_t first = (size_t)tile * n_splits * bm + r;             // split s lies s * bm rows further on
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    if (lane < n_splits) { m0 = part_ml[(first + (size_t)lane * bm) * 2]; l0 = part_ml[(first + (size_t)lane * bm) * 2 + 1]; }
    if (lane + 32 < n_splits) { m1 = part_ml[(first + (size_t)(lane + 32) * bm) * 2]; l1 = part_ml[(first + (size_t)(lane + 32) * bm) * 2 + 1]; }
    const float mx = fmaxf(warp_max(fmaxf(m0, m1)), sink ? sink[h] : -INFINITY);
    const float e0 = m0 == -INFINITY ? 0.0f : expf(m0 - mx), e1 = m1 == -INFINITY ? 0.0f : expf(m1 - mx);
    const float l = warp_sum(l0 * e0 + l1 * e1) + (sink ? expf(sink[h] - mx) : 0.0f);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    w[lane] = e0 * inv;
    w[lane + 32] = e1 * inv;
  }
  __syncthreads();
  bf16* orow = out + (size_t)(b.entry_q_start[e] + t) * ol.row + (size_t)h * ol.head;
  for (int d = threadIdx.x; d < vrank; d += blockDim.x) {
    const float* p = part_o + first * rank + d;
    float acc = 0.0f;
    int s = 0;
    for (; s + 4 <= n_splits; s += 4) {
      const float v0 = p[(size_t)s * bm * rank], v1 = p[(size_t)(s + 1) * bm * rank];
      const float v2 = p[(size_t)(s + 2) * bm * rank], v3 = p[(size_t)(s + 3) * bm * rank];
      acc = fmaf(v3, w[s + 3], fmaf(v2, w[s + 2], fmaf(v1, w[s + 1], fmaf(v0, w[s], acc))));
    }
    for (; s < n_splits; ++s) acc = fmaf(p[(size_t)s * bm * rank], w[s], acc);
    orow[d] = __float2bfloat16_rn(acc);
  }
}

template <int MT, int RT, bool NARROW>
size_t smem_bytes() {
  constexpr bool BY_R = MT <= 2 && RT >= 2;
  constexpr int BM = 16 * MT, LD = 64 * RT + PAD, NP = BY_R ? 8 / MT : 1, BN = NARROW ? 32 : 64;
  return (size_t)(BM + 2 * BN) * LD * 2 + (size_t)BM * (BN + PAD) * 2 + (size_t)NP * BM * (BN + 4) * 4 + (size_t)4 * BM * 4;
}

template <int MT, int RT, bool NARROW>
int launch_mma(const float* q, HeadLayout ql, bf16* out, HeadLayout ol, const bf16* cache, long long page_stride,
               int page_size, LatentTiles b, int n_tiles, int n_heads, int rank, float scale, int n_splits,
               float* part_o, float* part_ml, int vrank, int window, const float* sink, cudaStream_t stream) {
  const size_t smem = smem_bytes<MT, RT, NARROW>();
  auto kern = attn_latent_mma_kernel<MT, RT, NARROW>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  int rc = launch_pdl(kern, dim3(n_tiles, n_splits), dim3(256), smem, stream, q, ql, out, ol, cache, page_stride, page_size,
                      page_shift, b, n_heads, rank, scale, n_splits, part_o, part_ml, vrank, window, sink);
  if (rc) return rc;
  if (n_splits > 1) {
    rc = launch_pdl(attn_latent_merge_kernel, dim3(n_tiles, 16 * MT), dim3(rank > 256 ? 256 : (rank > 64 ? 128 : 64)), 0, stream,
                    (const float*)part_o, (const float*)part_ml, out, ol, b, n_heads, rank, n_splits, 16 * MT, vrank, sink);
    if (rc) return rc;
  }
  return IFX_LAUNCH_CHECK();
}
}  // namespace

// The largest rank the kernel takes (multiples of 8 up to it).
IFX_API int ifx_attn_latent_mma_max_rank() { return 512; }

namespace {
int sm_count_now() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
// Tiles of 16 rows take tiles of 32 latents when there are more blocks than SMs (two blocks then share an SM).
bool narrow_tiles(int blocks) { return blocks > sm_count_now(); }
}  // namespace

// Into how many splits the keys of every tile are cut: enough blocks to fill the GPU (as many as it holds at
// one block an SM), but no split shorter than 256 keys.
IFX_API int ifx_attn_latent_mma_plan(int n_tiles, int bm, int rank, int max_keys) {
  if (n_tiles <= 0) return 1;
  const int sms = sm_count_now();
  const int key_tiles = (max_keys + 63) / 64;
  int splits = sms / n_tiles;                     // one block an SM where the tiles alone do not fill the GPU
  if (splits > key_tiles / 4) splits = key_tiles / 4;      // no split shorter than 256 keys: below that a block's set-up outweighs its tiles
  return splits < 1 ? 1 : (splits > 64 ? 64 : splits);
}

// q float32 and out bfloat16 hold a (token, head) vector at token * row + head * head elements.  Tiles: bm (16 or
// 64) consecutive (token, head) rows of one entry, listed by tile_entry / tile_row0.  n_splits > 1: part_o holds
// n_tiles * n_splits * bm * rank floats, part_ml n_tiles * n_splits * bm * 2.
// vrank (a multiple of 8, at most rank): the first columns of a cached row that are the latent and are written to
// out; window: 0 = none; sink: float32 [n_heads] or null.
IFX_API int ifx_attn_latent_mma_ex(const float* q, long long q_row, long long q_head, void* out, long long o_row,
                                   long long o_head, const void* cache, long long page_stride, int page_size,
                                   const int* block_tables, int bt_stride, const int* tile_entry, const int* tile_row0,
                                   int n_tiles, int bm, const int* entry_q_start, const int* entry_q_len,
                                   const int* entry_ctx_start, int n_heads, int rank, float scale, int n_splits,
                                   float* part_o, float* part_ml, int vrank, int window, const float* sink,
                                   cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (rank < 8 || rank > 512 || rank % 8 || n_heads < 1 || n_splits < 1 || n_splits > 64) return IFX_ERR_UNSUPPORTED;
  if (vrank < 8 || vrank > rank || vrank % 8 || window < 0) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1)) || (page_stride & 7)) return IFX_ERR_UNSUPPORTED;
  if (((uintptr_t)cache & 15) != 0) return IFX_ERR_ALIGNMENT;
  if (n_splits > 1 && (!part_o || !part_ml)) return IFX_ERR_UNSUPPORTED;
  LatentTiles b{block_tables, bt_stride, tile_entry, tile_row0, entry_q_start, entry_q_len, entry_ctx_start};
  HeadLayout ql{q_row, q_head}, ol{o_row, o_head};
  const int rt = (rank + 63) / 64;
#define IFX_LM(MT, RT) return launch_mma<MT, RT, false>(q, ql, (bf16*)out, ol, (const bf16*)cache, page_stride, page_size, b, n_tiles, \
                                                 n_heads, rank, scale, n_splits, part_o, part_ml, vrank, window, sink, stream)
  if (bm == 16 && rt >= 2 && narrow_tiles(n_tiles * n_splits)) {
#define IFX_LN(RT) return launch_mma<1, RT, true>(q, ql, (bf16*)out, ol, (const bf16*)cache, page_stride, page_size, b, n_tiles, \
                                                  n_heads, rank, scale, n_splits, part_o, part_ml, vrank, window, sink, stream)
    if (rt <= 2) IFX_LN(2);
    if (rt <= 4) IFX_LN(4);
    IFX_LN(8);
#undef IFX_LN
  }
  if (bm == 16) {
    if (rt <= 1) IFX_LM(1, 1);
    if (rt <= 2) IFX_LM(1, 2);
    if (rt <= 4) IFX_LM(1, 4);
    IFX_LM(1, 8);
  }
  if (bm == 32) {
    if (rt <= 1) IFX_LM(2, 1);
    if (rt <= 2) IFX_LM(2, 2);
    if (rt <= 4) IFX_LM(2, 4);
    IFX_LM(2, 8);
  }
  if (bm == 64) {
    if (rt <= 1) IFX_LM(4, 1);
    if (rt <= 2) IFX_LM(4, 2);
    if (rt <= 4) IFX_LM(4, 4);
    IFX_LM(4, 8);
  }
#undef IFX_LM
  return IFX_ERR_UNSUPPORTED;
}

IFX_API int ifx_attn_latent_mma(const float* q, long long q_row, long long q_head, void* out, long long o_row,
                                long long o_head, const void* cache, long long page_stride, int page_size,
                                const int* block_tables, int bt_stride, const int* tile_entry, const int* tile_row0,
                                int n_tiles, int bm, const int* entry_q_start, const int* entry_q_len,
                                const int* entry_ctx_start, int n_heads, int rank, float scale, int n_splits,
                                float* part_o, float* part_ml, cudaStream_t stream) {
  return ifx_attn_latent_mma_ex(q, q_row, q_head, out, o_row, o_head, cache, page_stride, page_size, block_tables, bt_stride,
                                tile_entry, tile_row0, n_tiles, bm, entry_q_start, entry_q_len, entry_ctx_start, n_heads, rank,
                                scale, n_splits, part_o, part_ml, rank, 0, nullptr, stream);
}
