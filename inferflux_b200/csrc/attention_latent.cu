// Latent attention: a token caches one latent vector c (rank R) from which every head's keys and values
// follow, k_h = Uk_h c and v_h = Uv_h c.  The products are moved to the query's side,
//
//   score_h(i, j) = q_h(i) . (Uk_h c_j) = (Uk_h^T q_h(i)) . c_j            o_h(i) = Uv_h (sum_j p_h(i, j) c_j)
//
// so the kernel attends over the cached latents alone: its queries are the R-wide vectors Uk_h^T q_h, its keys
// and its values are both c, and its output is the R-wide weighted sum that the caller sends through Uv_h.
// Scores, softmax and sums are float32 (expf, running maximum and sum); causal: key j is visible to the query
// at position p iff j <= p.  No positions enter.
//
// latent_prep turns a token's stacked down projections into what the step needs: the query latent and the
// key/value latent each divided by their root mean square and multiplied by their weights (the key/value
// latent goes straight to the token's place in the paged cache), and the sigmoid of the per-head output gates.
//
// attn_latent_paged: one block takes 16 consecutive new tokens of one request and one head and walks the
// request's pages in tiles of 32 latents that serve as keys and as values.  Tiles start at multiples of 32 and
// are added in index order, so a token's result does not depend on how the prompt was cut.
#include "common.cuh"

namespace {
constexpr int LQ = 16;        // query rows per block (2 per warp, 8 warps)
constexpr int LKEYS = 32;     // latents per tile (one per lane)

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ p, long long p_stride, const float* __restrict__ wq,
                                   const float* __restrict__ wkv, float eps, int q_rank, int kv_rank, int n_heads,
                                   T* __restrict__ cq, T* __restrict__ cache, long long page_stride, int page_size,
                                   const int* __restrict__ slot_map, float* __restrict__ gate) {
  pdl_enter();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* pr = p + (size_t)row * p_stride;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq = fmaf(pr[i], pr[i], sq);
  const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)row * q_rank + i] = Num<T>::from_f(pr[i] * rq * wq[i]);
  const float* pk = pr + q_rank;
  sq = 0.0f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) sq = fmaf(pk[i], pk[i], sq);
  const float rk = 1.0f / sqrtf(block_sum(sq, red) / (float)kv_rank + eps);
  const int slot = slot_map[row];
  if (slot >= 0) {
    T* c = cache + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * kv_rank;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) c[i] = Num<T>::from_f(pk[i] * rk * wkv[i]);
  }
  const float* pg = pk + kv_rank;
  for (int i = threadIdx.x; i < n_heads; i += blockDim.x) gate[(size_t)row * n_heads + i] = sigmoid_f(pg[i]);
}

struct LatentBatch {
  const int* block_tables;    // [n_entries, bt_stride] page of each logical block, -1 = given back
  int bt_stride;
  const int* tile_entry;      // [n_tiles] request entry of each query tile
  const int* tile_q0;         // [n_tiles] first new token (within the entry) of the tile
  const int* entry_q_start;   // [n_entries] row of the entry's first new token in q/out
  const int* entry_q_len;     // [n_entries] new tokens
  const int* entry_ctx_start; // [n_entries] tokens cached before them = position of the first new token
};

// Where a (token, head) vector of `rank` elements lies: token * row + head * head elements from the start.
struct HeadLayout { long long row, head; };

// q float32, out of the cache's type T, each laid out by its HeadLayout.  cache: the run's rows of page 0,
// [slot][kw] within a page.  A cached row is kw wide: its first `rank` elements are the latent, which serves as
// key and as value; the other kw - rank (a rotated key part that all heads share, say) enter the scores only.
// Queries are kw wide, results rank wide.  window > 0 hides keys j <= p - window; sink ([n_heads] or null) puts
// one more term exp(sink[head]) without a value into the softmax's denominator.
template <typename T, int NACC>
__global__ void __launch_bounds__(256)
attn_latent_paged_kernel(const float* __restrict__ q, HeadLayout ql, T* __restrict__ out, HeadLayout ol,
                         const T* __restrict__ cache, long long page_stride, int page_size, int page_shift,
                         LatentBatch b, int rank, int kw, float scale, int window, const float* __restrict__ sink) {
  pdl_enter();
  extern __shared__ float smem[];
  float* qs = smem;                               // [LQ][kw]
  float* cs = qs + LQ * kw;                       // [LKEYS][kw + 1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int e = b.tile_entry[tile];
  const int q0 = b.tile_q0[tile];
  const int rows = min(LQ, b.entry_q_len[e] - q0);
  if (rows <= 0) return;
  const int tok0 = b.entry_q_start[e] + q0;
  const int pos0 = b.entry_ctx_start[e] + q0;
  const int* bt = b.block_tables + (size_t)e * b.bt_stride;

  for (int idx = tid; idx < LQ * kw; idx += blockDim.x) {
    const int r = idx / kw, d = idx - r * kw;
    qs[idx] = r < rows ? q[(size_t)(tok0 + r) * ql.row + (size_t)head * ql.head + d] : 0.0f;
  }

  const int r0 = warp * 2, r1 = r0 + 1;
  // a sink is a key without a value: the running maximum starts at its score and the sum at exp(0)
  const float sink0 = sink ? sink[head] : -INFINITY;
  float m[2] = {sink0, sink0}, l[2] = {sink ? 1.0f : 0.0f, sink ? 1.0f : 0.0f};
  float o[2][NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) { o[0][a] = 0.0f; o[1][a] = 0.0f; }

  const int kend = pos0 + rows - 1;               // last key any row of the tile may see
  const int kstart = window > 0 ? max(0, pos0 - window + 1) & ~(LKEYS - 1) : 0;
  for (int k0 = kstart; k0 <= kend; k0 += LKEYS) {
    __syncthreads();
    for (int idx = tid; idx < LKEYS * kw; idx += blockDim.x) {
      const int j = idx / kw, d = idx - j * kw;
      const int key = k0 + j;
      float c = 0.0f;
      if (key <= kend) {
        const int page = bt[key >> page_shift];
        if (page >= 0) c = Num<T>::to_f(cache[(size_t)page * page_stride + (size_t)(key & (page_size - 1)) * kw + d]);
      }
      cs[j * (kw + 1) + d] = c;
    }
    __syncthreads();
    if (r0 < rows) {                               // warp-uniform
      const bool two = r1 < rows;
      const float* cr = cs + lane * (kw + 1);
      const float* qa = qs + r0 * kw;
      const float* qb = qs + r1 * kw;
      float s0 = 0.0f, s1 = 0.0f;
      for (int d = 0; d < kw; ++d) {
        const float cd = cr[d];
        s0 = fmaf(qa[d], cd, s0);
        s1 = fmaf(qb[d], cd, s1);
      }
      const int key = k0 + lane;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (rr == 1 && !two) break;
        const int p = pos0 + r0 + rr;
        const bool visible = key <= p && (window <= 0 || key > p - window);
        const float s = visible ? (rr ? s1 : s0) * scale : -INFINITY;
        const float m_new = fmaxf(m[rr], warp_max(s));
        if (m_new == -INFINITY) continue;          // nothing visible to this row yet (warp-uniform)
        const float alpha = expf(m[rr] - m_new);   // exp(-inf) = 0 on the first visible tile
        const float pj = visible ? expf(s - m_new) : 0.0f;
        l[rr] = l[rr] * alpha + warp_sum(pj);
        m[rr] = m_new;
#pragma unroll
        for (int a = 0; a < NACC; ++a) o[rr][a] *= alpha;
        for (int j = 0; j < LKEYS; ++j) {
          const float pjj = __shfl_sync(0xffffffffu, pj, j);
          if (pjj == 0.0f) continue;               // warp-uniform; also keeps stale latents out
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            const int d = lane + 32 * a;
            if (d < rank) o[rr][a] = fmaf(pjj, cs[j * (kw + 1) + d], o[rr][a]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = r0 + rr;
    if (r >= rows) continue;
    const float inv = l[rr] > 0.0f ? 1.0f / l[rr] : 0.0f;
    T* orow = out + (size_t)(tok0 + r) * ol.row + (size_t)head * ol.head;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int d = lane + 32 * a;
      if (d < rank) orow[d] = Num<T>::from_f(o[rr][a] * inv);
    }
  }
}

template <typename T, int NACC>
int launch_latent(const float* q, HeadLayout ql, void* out, HeadLayout ol, const void* cache, long long page_stride,
                  int page_size, LatentBatch b, int n_tiles, int n_heads, int rank, int kw, float scale, int window,
                  const float* sink, cudaStream_t stream) {
  const size_t smem = ((size_t)LQ * kw + (size_t)LKEYS * (kw + 1)) * sizeof(float);
  auto kern = attn_latent_paged_kernel<T, NACC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const int rc = launch_pdl(kern, dim3(n_tiles, n_heads), dim3(256), smem, stream, q, ql, (T*)out, ol, (const T*)cache,
                            page_stride, page_size, page_shift, b, rank, kw, scale, window, sink);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

template <typename T>
int dispatch_latent(const float* q, HeadLayout ql, void* out, HeadLayout ol, const void* cache, long long page_stride,
                    int page_size, LatentBatch b, int n_tiles, int n_heads, int rank, int kw, float scale, int window,
                    const float* sink, cudaStream_t stream) {
  const int nacc = (rank + 31) / 32;
#define IFX_LAT(N) return launch_latent<T, N>(q, ql, out, ol, cache, page_stride, page_size, b, n_tiles, n_heads, rank, kw, scale, window, sink, stream)
  if (nacc <= 1) IFX_LAT(1);
  if (nacc <= 2) IFX_LAT(2);
  if (nacc <= 4) IFX_LAT(4);
  if (nacc <= 8) IFX_LAT(8);
  if (nacc <= 16) IFX_LAT(16);
  IFX_LAT(32);
#undef IFX_LAT
}

// A token's stacked float32 sums [q heads (each `dim` plain then `rot` rotating columns) | latent (kv_rank) |
// rotating key part (rot)] become what the step needs: the plain query parts side by side in the engine's type
// (the operand of the product with the keys' up-projection), the rotated query parts as float32 in the last
// `rot` columns of every head's (kv_rank + rot)-wide query row, and in the token's place in the paged cache the
// latent, divided by its root mean square and multiplied by its weight, followed by the rotated key part.
// Neighbouring pairs (2i, 2i + 1) rotate by cos/sin [N, rot / 2].
template <typename T>
__global__ void latent_rope_prep_kernel(const float* __restrict__ p, long long p_stride, const float* __restrict__ wkv,
                                        float eps, int n_heads, int dim, int rot, int kv_rank,
                                        const float* __restrict__ cosv, const float* __restrict__ sinv,
                                        T* __restrict__ q_plain, float* __restrict__ q_rows, long long q_row, long long q_head,
                                        T* __restrict__ cache, long long page_stride, int page_size,
                                        const int* __restrict__ slot_map) {
  pdl_enter();
  __shared__ float red[32];
  const int row = blockIdx.x, half = rot >> 1;
  const float* pr = p + (size_t)row * p_stride;
  const float* cr = cosv + (size_t)row * half;
  const float* sr = sinv + (size_t)row * half;
  const int hw = dim + rot;
  for (int i = threadIdx.x; i < n_heads * dim; i += blockDim.x) {
    const int h = i / dim, d = i - h * dim;
    q_plain[(size_t)row * n_heads * dim + i] = Num<T>::from_f(pr[h * hw + d]);
  }
  for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const float u = pr[h * hw + dim + 2 * j], v = pr[h * hw + dim + 2 * j + 1];
    float* dst = q_rows + (size_t)row * q_row + (size_t)h * q_head + kv_rank + 2 * j;
    dst[0] = u * cr[j] - v * sr[j];
    dst[1] = v * cr[j] + u * sr[j];
  }
  const float* pk = pr + (size_t)n_heads * hw;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) sq = fmaf(pk[i], pk[i], sq);
  const float rk = 1.0f / sqrtf(block_sum(sq, red) / (float)kv_rank + eps);
  const int slot = slot_map[row];
  if (slot >= 0) {
    T* c = cache + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * (kv_rank + rot);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) c[i] = Num<T>::from_f(pk[i] * rk * wkv[i]);
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const float u = pk[kv_rank + 2 * j], v = pk[kv_rank + 2 * j + 1];
      c[kv_rank + 2 * j] = Num<T>::from_f(u * cr[j] - v * sr[j]);
      c[kv_rank + 2 * j + 1] = Num<T>::from_f(v * cr[j] + u * sr[j]);
    }
  }
}
}  // namespace

// p float32 [N, q_rank + kv_rank + n_heads] (row stride p_stride): a token's down projections side by side.
// cq [N, q_rank] and the cache are of dtype; gate float32 [N, n_heads]; slot_map [N] = page * page_size +
// place within the page of each token's latent (-1: not written).
IFX_API int ifx_latent_prep(const float* p, long long p_stride, const float* wq, const float* wkv, float eps, int q_rank,
                            int kv_rank, int n_heads, void* cq, void* cache, int dtype, long long page_stride,
                            int page_size, const int* slot_map, float* gate, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (q_rank < 1 || kv_rank < 1 || n_heads < 1 || page_size < 1) return IFX_ERR_UNSUPPORTED;
  const int widest = q_rank > kv_rank ? q_rank : kv_rank;
  int threads = 64;
  while (threads < 1024 && threads * 4 < widest) threads <<= 1;
  int rc;
  if (dtype == IFX_F32)
    rc = launch_pdl(latent_prep_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, p, p_stride, wq, wkv, eps, q_rank,
                    kv_rank, n_heads, (float*)cq, (float*)cache, page_stride, page_size, slot_map, gate);
  else if (dtype == IFX_BF16)
    rc = launch_pdl(latent_prep_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, p, p_stride, wq, wkv, eps, q_rank,
                    kv_rank, n_heads, (bf16*)cq, (bf16*)cache, page_stride, page_size, slot_map, gate);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}

namespace {
// out[t, h, :] = in[t, h, :] * gate[t, h] (gate null: times 1), from rows laid out by `il` into contiguous [N, heads * width] rows of
// the engine's type: the per-head output gate, the rounding and the gathering of the heads in one pass.  With
// row_entry the kernel takes only the rows of entries that bring more than one token (prompt == 1) or exactly
// one (prompt == 0) and leaves the others as they are.
template <typename TI, typename TO>
__global__ void gate_heads_kernel(const TI* __restrict__ in, HeadLayout il, const float* __restrict__ gate,
                                  TO* __restrict__ out, long long out_stride, int n_heads, int width, const int* __restrict__ row_entry,
                                  const int* __restrict__ entry_q_len, int prompt) {
  pdl_enter();
  const int row = blockIdx.x;
  if (row_entry && (entry_q_len[row_entry[row]] > 1) != (prompt != 0)) return;
  const int total = n_heads * width;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / width, d = i - h * width;
    out[(size_t)row * out_stride + i] = Num<TO>::from_f(Num<TI>::to_f(in[(size_t)row * il.row + (size_t)h * il.head + d]) * (gate ? gate[(size_t)row * n_heads + h] : 1.0f));
  }
}

// out[i, :] = the cached latent of (entry g_entry[i], position g_pos[i]), found through the block tables.
template <typename T>
__global__ void gather_latents_kernel(const T* __restrict__ cache, long long page_stride, int page_size, int page_shift,
                                      int rank, const int* __restrict__ block_tables, int bt_stride,
                                      const int* __restrict__ g_entry, const int* __restrict__ g_pos, T* __restrict__ out) {
  pdl_enter();
  const int row = blockIdx.x;
  const int pos = g_pos[row];
  const int page = block_tables[(size_t)g_entry[row] * bt_stride + (pos >> page_shift)];
  const T* src = cache + (size_t)(page < 0 ? 0 : page) * page_stride + (size_t)(pos & (page_size - 1)) * rank;
  T* dst = out + (size_t)row * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = page < 0 ? Num<T>::from_f(0.0f) : src[i];
}
}  // namespace

// in_dtype / out_dtype: IFX_F32 or IFX_BF16.  row_entry (with entry_q_len) may be null: every row is taken.
IFX_API int ifx_gate_heads(const void* in, int in_dtype, long long in_row, long long in_head, const float* gate, void* out,
                           long long out_stride, int out_dtype, int n_rows, int n_heads, int width, const int* row_entry,
                           const int* entry_q_len, int prompt, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int total = n_heads * width;
  const int threads = total >= 1024 ? 256 : (total >= 256 ? 128 : 64);
  HeadLayout il{in_row, in_head};
  int rc;
#define IFX_GH(TI, TO) rc = launch_pdl(gate_heads_kernel<TI, TO>, dim3(n_rows), dim3(threads), 0, stream, (const TI*)in, il, gate, \
                                       (TO*)out, out_stride, n_heads, width, row_entry, entry_q_len, prompt)
  if (in_dtype == IFX_F32 && out_dtype == IFX_F32) IFX_GH(float, float);
  else if (in_dtype == IFX_F32 && out_dtype == IFX_BF16) IFX_GH(float, bf16);
  else if (in_dtype == IFX_BF16 && out_dtype == IFX_BF16) IFX_GH(bf16, bf16);
  else if (in_dtype == IFX_BF16 && out_dtype == IFX_F32) IFX_GH(bf16, float);
  else return IFX_ERR_UNSUPPORTED;
#undef IFX_GH
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_gather_latents(const void* cache, int dtype, long long page_stride, int page_size, int rank,
                               const int* block_tables, int bt_stride, const int* g_entry, const int* g_pos, void* out,
                               int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (page_size <= 0 || (page_size & (page_size - 1)) || rank < 1) return IFX_ERR_UNSUPPORTED;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const int threads = rank >= 256 ? 128 : 64;
  int rc;
  if (dtype == IFX_F32)
    rc = launch_pdl(gather_latents_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)cache, page_stride,
                    page_size, page_shift, rank, block_tables, bt_stride, g_entry, g_pos, (float*)out);
  else if (dtype == IFX_BF16)
    rc = launch_pdl(gather_latents_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)cache, page_stride,
                    page_size, page_shift, rank, block_tables, bt_stride, g_entry, g_pos, (bf16*)out);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// Query tiles are 16 tokens of one entry: tile_entry / tile_q0 list them.  kw: 1..1024, rank <= kw.  q float32 (kw
// wide) and out (rank wide, of the cache's type) hold a (token, head) vector at token * row + head * head elements.
IFX_API int ifx_attn_latent_paged_ex(const float* q, long long q_row, long long q_head, void* out, long long o_row,
                                     long long o_head, const void* cache, int cache_dtype, long long page_stride,
                                     int page_size, const int* block_tables, int bt_stride, const int* tile_entry,
                                     const int* tile_q0, int n_tiles, const int* entry_q_start, const int* entry_q_len,
                                     const int* entry_ctx_start, int n_heads, int rank, int kw, float scale, int window,
                                     const float* sink, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (rank < 1 || kw < rank || kw > 1024 || n_heads < 1 || n_heads > 65535 || window < 0) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  LatentBatch b{block_tables, bt_stride, tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start};
  HeadLayout ql{q_row, q_head}, ol{o_row, o_head};
  if (cache_dtype == IFX_F32)
    return dispatch_latent<float>(q, ql, out, ol, cache, page_stride, page_size, b, n_tiles, n_heads, rank, kw, scale, window, sink, stream);
  if (cache_dtype == IFX_BF16)
    return dispatch_latent<bf16>(q, ql, out, ol, cache, page_stride, page_size, b, n_tiles, n_heads, rank, kw, scale, window, sink, stream);
  return IFX_ERR_UNSUPPORTED;
}

IFX_API int ifx_attn_latent_paged(const float* q, long long q_row, long long q_head, void* out, long long o_row,
                                  long long o_head, const void* cache, int cache_dtype, long long page_stride,
                                  int page_size, const int* block_tables, int bt_stride, const int* tile_entry,
                                  const int* tile_q0, int n_tiles, const int* entry_q_start, const int* entry_q_len,
                                  const int* entry_ctx_start, int n_heads, int rank, float scale, cudaStream_t stream) {
  return ifx_attn_latent_paged_ex(q, q_row, q_head, out, o_row, o_head, cache, cache_dtype, page_stride, page_size,
                                  block_tables, bt_stride, tile_entry, tile_q0, n_tiles, entry_q_start, entry_q_len,
                                  entry_ctx_start, n_heads, rank, rank, scale, 0, nullptr, stream);
}

// p float32 [N, n_heads * (dim + rot) + kv_rank + rot] (row stride p_stride); q_plain [N, n_heads * dim] and the
// cache (rows of kv_rank + rot) are of dtype; q_rows float32, a (token, head) row at token * q_row + head * q_head.
IFX_API int ifx_latent_rope_prep(const float* p, long long p_stride, const float* wkv, float eps, int n_heads, int dim,
                                 int rot, int kv_rank, const float* cosv, const float* sinv, void* q_plain, float* q_rows,
                                 long long q_row, long long q_head, void* cache, int dtype, long long page_stride,
                                 int page_size, const int* slot_map, int n_rows, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_heads < 1 || dim < 0 || rot < 0 || (rot & 1) || kv_rank < 1 || page_size < 1) return IFX_ERR_UNSUPPORTED;
  const int widest = n_heads * dim > kv_rank ? n_heads * dim : kv_rank;
  int threads = 64;
  while (threads < 1024 && threads * 4 < widest) threads <<= 1;
  int rc;
  if (dtype == IFX_F32)
    rc = launch_pdl(latent_rope_prep_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, p, p_stride, wkv, eps, n_heads, dim,
                    rot, kv_rank, cosv, sinv, (float*)q_plain, q_rows, q_row, q_head, (float*)cache, page_stride, page_size, slot_map);
  else if (dtype == IFX_BF16)
    rc = launch_pdl(latent_rope_prep_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, p, p_stride, wkv, eps, n_heads, dim,
                    rot, kv_rank, cosv, sinv, (bf16*)q_plain, q_rows, q_row, q_head, (bf16*)cache, page_stride, page_size, slot_map);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}
