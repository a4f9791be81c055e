// Paged grouped-query attention over the cache, any element type: the kernel
// of the float32 path, and the plain counterpart of the bfloat16 kernels.
//
// Reference formulas (runtime/backends/cuda/kernels/flash_attention.cu:52-173):
//   kv_head = head / (n_heads / n_kv);  s_j = (q . k_j) * scale  (scale after the dot, :127-141)
//   causal: key j visible to the query at position p iff j <= p (:70-71,85)
//   online softmax in float32 with expf, running max and sum (:143-171);  o = sum p_j v_j / sum p_j
// The reference runs one block per (query, head) over a dense per-sequence
// buffer.  Here one block takes 16 consecutive new tokens of one request and
// one head, reads keys and values through the request's block table in tiles
// of 32 keys, and serves prompt portions (any number of cached tokens before
// them) and single decoded tokens alike.  A window w > 0 hides keys j <= p - w.
//
// A second kernel serves steps' single tokens (attn_single_token_kernel below).
// Options (AttnOptions; all off for plain attention): values of another width than keys (`v_dim`); a cap on
// the scores, s <- cap * tanh(s / cap); kept first tokens, which stay visible behind the window
// (key j visible iff j <= p and (p - j < w or j < keep_first)); a sink, one more term of score 0 and no value
// in the softmax's denominator, p_j = exp(s_j) / (1 + sum exp(s_j)); an output gate, every element of a
// head's result times sigmoid of a float32 row given beside it.
//
// Tiles start at multiples of 32 keys and keys are added in index order, so in
// float32 the result for a token does not depend on how the prompt was cut.
#include "common.cuh"

namespace {
constexpr int BQ = 16;        // query rows per block (2 per warp, 8 warps)
constexpr int BKEYS = 32;     // keys per tile (one per lane)

struct AttnBatch {
  const int* block_tables;    // [n_entries, bt_stride] page of each logical block, -1 = given back
  int bt_stride;
  const int* tile_entry;      // [n_tiles] request entry of each query tile
  const int* tile_q0;         // [n_tiles] first new token (within the entry) of the tile
  const int* entry_q_start;   // [n_entries] row of the entry's first new token in q/out
  const int* entry_q_len;     // [n_entries] new tokens
  const int* entry_ctx_start; // [n_entries] tokens cached before them = position of the first new token
};

struct AttnOptions {
  int v_dim;                  // width of a value head (keys are head_dim wide)
  int v_head_stride;          // elements between the value heads of a page = page_size * v_dim
  float softcap;              // 0 = none
  int keep_first;             // first tokens that stay visible behind the window
  int sink;                   // 1 = the denominator has one more term exp(0)
  const float* gate;          // [N][gate_stride] float32 or null: out *= sigmoid(gate[row][head * v_dim + d])
  int gate_parts; long long gate_part_stride; int gate_stride;
  float q_temp_coef;          // the query at position p counts 1 + coef * ln(floor((p + 1) / every) + 1) times; every = 0: none
  int q_temp_every;
  const float* dist_r1;       // [n_heads] or null: the score of key j loses r1[head] * ln(1 + r2[head] * (p - j))
  const float* dist_r2;
  const float* sink_value;    // [n_heads] or null: with a sink, its score (0 where null)
};

// What the options make of a raw product q . k: the query's temperature, the scale, the cap, the distance's toll.
__device__ __forceinline__ float query_temperature(const AttnOptions& opt, int p) {
  return opt.q_temp_every > 0 ? 1.0f + opt.q_temp_coef * logf((float)((p + 1) / opt.q_temp_every + 1)) : 1.0f;
}
__device__ __forceinline__ float shaped_score(const AttnOptions& opt, float dot, float scale_temp, float r1, float r2, int dist) {
  float sc = dot * scale_temp;
  if (opt.softcap > 0.0f) sc = opt.softcap * tanhf(sc / opt.softcap);
  if (opt.dist_r1) sc -= r1 * log1pf(r2 * (float)dist);
  return sc;
}

template <typename T, int NACC>
__global__ void __launch_bounds__(256)
attn_paged_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                          PagedKV kv, AttnBatch b, int n_heads, int n_kv, int head_dim, float scale, int window,
                          AttnOptions opt) {
  pdl_enter();
  extern __shared__ float smem[];
  const int v_dim = opt.v_dim;
  float* qs = smem;                               // [BQ][head_dim]
  float* ks = qs + BQ * head_dim;                 // [BKEYS][head_dim + 1]
  float* vs = ks + BKEYS * (head_dim + 1);        // [BKEYS][v_dim]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int e = b.tile_entry[tile];
  const int q0 = b.tile_q0[tile];
  const int rows = min(BQ, b.entry_q_len[e] - q0);
  if (rows <= 0) return;
  const int tok0 = b.entry_q_start[e] + q0;
  const int pos0 = b.entry_ctx_start[e] + q0;
  const int kvh = head / (n_heads / n_kv);
  const int* bt = b.block_tables + (size_t)e * b.bt_stride;
  const T* kc = (const T*)kv.k + (size_t)kvh * kv.head_stride;
  const T* vc = (const T*)kv.v + (size_t)kvh * opt.v_head_stride;

  for (int idx = tid; idx < BQ * head_dim; idx += blockDim.x) {
    const int r = idx / head_dim, d = idx - r * head_dim;
    qs[idx] = r < rows ? Num<T>::to_f(q[(size_t)(tok0 + r) * q_stride + (size_t)head * head_dim + d]) : 0.0f;
  }

  const int r0 = warp * 2, r1 = r0 + 1;
  // a sink is a key of score 0 without a value: the running maximum starts at 0 and the sum at exp(0)
  const float sink0 = opt.sink ? (opt.sink_value ? opt.sink_value[head] : 0.0f) : -INFINITY;
  const float toll1 = opt.dist_r1 ? opt.dist_r1[head] : 0.0f, toll2 = opt.dist_r1 ? opt.dist_r2[head] : 0.0f;
  float m[2] = {sink0, sink0}, l[2] = {opt.sink ? 1.0f : 0.0f, opt.sink ? 1.0f : 0.0f};
  float o[2][NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) { o[0][a] = 0.0f; o[1][a] = 0.0f; }

  const int kend = pos0 + rows - 1;               // last key any row of the tile may see
  int kstart = 0;
  if (window > 0) kstart = max(0, pos0 - window + 1) & ~(BKEYS - 1);
  // with kept first tokens the tiles [0, keep_end) come first, then those from kstart on
  const int keep_end = window > 0 ? min((opt.keep_first + BKEYS - 1) & ~(BKEYS - 1), kstart) : 0;

  for (int k0 = keep_end > 0 ? 0 : kstart; k0 <= kend; k0 += BKEYS) {
    if (k0 >= keep_end && k0 < kstart) k0 = kstart;
    __syncthreads();
    for (int idx = tid; idx < BKEYS * head_dim; idx += blockDim.x) {
      const int j = idx / head_dim, d = idx - j * head_dim;
      const int key = k0 + j;
      float kval = 0.0f;
      if (key <= kend) {
        const int page = bt[key >> kv.page_shift];
        if (page >= 0)
          kval = Num<T>::to_f(kc[(size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * head_dim + d]);
      }
      ks[j * (head_dim + 1) + d] = kval;
    }
    for (int idx = tid; idx < BKEYS * v_dim; idx += blockDim.x) {
      const int j = idx / v_dim, d = idx - j * v_dim;
      const int key = k0 + j;
      float vval = 0.0f;
      if (key <= kend) {
        const int page = bt[key >> kv.page_shift];
        if (page >= 0)
          vval = Num<T>::to_f(vc[(size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * v_dim + d]);
      }
      vs[j * v_dim + d] = vval;
    }
    __syncthreads();
    if (r0 < rows) {                               // warp-uniform
      const bool two = r1 < rows;
      const float* kr = ks + lane * (head_dim + 1);
      const float* qa = qs + r0 * head_dim;
      const float* qb = qs + r1 * head_dim;
      float s0 = 0.0f, s1 = 0.0f;
      for (int d = 0; d < head_dim; ++d) {
        const float kd = kr[d];
        s0 = fmaf(qa[d], kd, s0);
        s1 = fmaf(qb[d], kd, s1);
      }
      const int key = k0 + lane;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (rr == 1 && !two) break;
        const int p = pos0 + r0 + rr;
        const bool visible = key <= p && (window <= 0 || key > p - window || key < opt.keep_first);
        const float sc = shaped_score(opt, rr ? s1 : s0, scale * query_temperature(opt, p), toll1, toll2, visible ? p - key : 0);
        const float s = visible ? sc : -INFINITY;
        const float m_new = fmaxf(m[rr], warp_max(s));
        if (m_new == -INFINITY) continue;          // nothing visible to this row yet (warp-uniform)
        const float alpha = expf(m[rr] - m_new);   // exp(-inf) = 0 on the first visible tile
        const float pj = visible ? expf(s - m_new) : 0.0f;
        l[rr] = l[rr] * alpha + warp_sum(pj);
        m[rr] = m_new;
#pragma unroll
        for (int a = 0; a < NACC; ++a) o[rr][a] *= alpha;
        for (int j = 0; j < BKEYS; ++j) {
          const float pjj = __shfl_sync(0xffffffffu, pj, j);
          if (pjj == 0.0f) continue;               // warp-uniform; also keeps stale values out
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            const int d = lane + 32 * a;
            if (d < v_dim) o[rr][a] = fmaf(pjj, vs[j * v_dim + d], o[rr][a]);
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
    T* orow = out + (size_t)(tok0 + r) * out_stride + (size_t)head * v_dim;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int d = lane + 32 * a;
      if (d >= v_dim) continue;
      float y = o[rr][a] * inv;
      if (opt.gate) {
        float g = 0.0f;
        for (int s = 0; s < opt.gate_parts; ++s)
          g += opt.gate[(size_t)s * opt.gate_part_stride + (size_t)(tok0 + r) * opt.gate_stride + (size_t)head * v_dim + d];
        y *= 1.0f / (1.0f + expf(-g));
      }
      orow[d] = Num<T>::from_f(y);
    }
  }
}

// Single tokens: one block a (token, head), its warps take the key tiles of 32 in turn (a lane a key for the
// scores, a lane a few value dimensions for the sum), each warp with a running maximum, sum and result of its
// own that the block merges at the end; keys and values are read straight from the pages.  The same options.
// DEC_WARPS warps a block: 32 where the step's blocks are few (every warp then has about one tile of a window of
// 1,024), 16 where they are many (two blocks share an SM and one's merge overlaps the other's tiles).
template <typename T, int NACC, int DEC_WARPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_single_token_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                         PagedKV kv, AttnBatch b, int n_heads, int n_kv, int head_dim, float scale, int window,
                         AttnOptions opt) {
  pdl_enter();
  extern __shared__ float smem[];
  const int v_dim = opt.v_dim;
  float* qs = smem;                                   // [head_dim]
  float* wm = qs + head_dim;                          // [DEC_WARPS] maxima
  float* wl = wm + DEC_WARPS;                         // [DEC_WARPS] sums
  float* wo = wl + DEC_WARPS;                         // [DEC_WARPS][v_dim]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e = b.tile_entry[blockIdx.x], head = blockIdx.y;
  const int tok = b.entry_q_start[e] + b.tile_q0[blockIdx.x];
  const int p = b.entry_ctx_start[e] + b.tile_q0[blockIdx.x];          // the token's position = its last visible key
  const int kvh = head / (n_heads / n_kv);
  const int* bt = b.block_tables + (size_t)e * b.bt_stride;
  const T* kc = (const T*)kv.k + (size_t)kvh * kv.head_stride;
  const T* vc = (const T*)kv.v + (size_t)kvh * opt.v_head_stride;
  for (int d = tid; d < head_dim; d += blockDim.x) qs[d] = Num<T>::to_f(q[(size_t)tok * q_stride + (size_t)head * head_dim + d]);
  __syncthreads();
  int kstart = 0;
  if (window > 0) kstart = max(0, p - window + 1) & ~(BKEYS - 1);
  const int keep_end = window > 0 ? min((opt.keep_first + BKEYS - 1) & ~(BKEYS - 1), kstart) : 0;
  const int n_keep = keep_end / BKEYS, n_tiles = n_keep + (p - kstart) / BKEYS + 1;
  const float scale_temp = scale * query_temperature(opt, p);
  const float r1 = opt.dist_r1 ? opt.dist_r1[head] : 0.0f, r2 = opt.dist_r1 ? opt.dist_r2[head] : 0.0f;
  float m = -INFINITY, l = 0.0f, o[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) o[a] = 0.0f;
  // which value dimension accumulator a of this lane holds: lane + 32 a, or, where a lane can take 4 neighbouring
  // 16-bit values with one 8-byte load (values 128 or 256 wide), 4 lane + (a mod 4) + 128 (a / 4)
  const bool vec_v = sizeof(T) == 2 && NACC >= 4 && v_dim == 32 * NACC && kv.page_size >= 4;
#define IFX_DIM_OF(a) (vec_v ? 4 * lane + ((a) & 3) + 128 * ((a) >> 2) : lane + 32 * (a))
  for (int it = warp; it < n_tiles; it += DEC_WARPS) {
    const int k0 = it < n_keep ? it * BKEYS : kstart + (it - n_keep) * BKEYS;
    const int key = k0 + lane;
    const bool visible = key <= p && (window <= 0 || key > p - window || key < opt.keep_first);
    const int page = key <= p ? bt[key >> kv.page_shift] : -1;
    float sc = -INFINITY;
    if (visible && page >= 0) {
      const T* kr = kc + (size_t)page * kv.page_stride + (size_t)(key & (kv.page_size - 1)) * head_dim;
      float dot = 0.0f;
      if (sizeof(T) == 2 && (head_dim & 7) == 0 && kv.page_size >= 8) {
        // the key row's 16-byte pieces are asked for eight at a time, and added up in two chains
        float dot2 = 0.0f;
#pragma unroll 8
        for (int d = 0; d < head_dim; d += 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
          const float4 qa = *reinterpret_cast<const float4*>(qs + d), qb = *reinterpret_cast<const float4*>(qs + d + 4);
          const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
          const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
          dot = fmaf(qa.x, f0.x, fmaf(qa.y, f0.y, fmaf(qa.z, f1.x, fmaf(qa.w, f1.y, dot))));
          dot2 = fmaf(qb.x, f2.x, fmaf(qb.y, f2.y, fmaf(qb.z, f3.x, fmaf(qb.w, f3.y, dot2))));
        }
        dot += dot2;
      } else {
        for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], Num<T>::to_f(kr[d]), dot);
      }
      sc = shaped_score(opt, dot, scale_temp, r1, r2, p - key);
    }
    const float m_new = fmaxf(m, warp_max(sc));
    if (m_new == -INFINITY) continue;                 // warp-uniform: nothing visible in this tile
    const float alpha = expf(m - m_new);
    const float pj = sc == -INFINITY ? 0.0f : expf(sc - m_new);
    l = l * alpha + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int a = 0; a < NACC; ++a) o[a] *= alpha;
    // No branch on the weight here: the values of eight keys are asked for together, from an address that is
    // always valid (page 0 stands in for a key that is not visible), and what was read for a key of weight 0 is
    // replaced by zeros before it is used, so stale pages stay out.
    if (vec_v) {
      for (int j0 = 0; j0 < BKEYS; j0 += 8) {
        uint2 raw[8][NACC / 4 > 0 ? NACC / 4 : 1];
        float wj[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          wj[u] = __shfl_sync(0xffffffffu, pj, j0 + u);
          const int pg = __shfl_sync(0xffffffffu, page, j0 + u);
          const T* vr = vc + (size_t)(wj[u] != 0.0f ? pg : 0) * kv.page_stride + (size_t)((k0 + j0 + u) & (kv.page_size - 1)) * v_dim;
#pragma unroll
          for (int a4 = 0; a4 < NACC / 4; ++a4) raw[u][a4] = *reinterpret_cast<const uint2*>(vr + 4 * lane + 128 * a4);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
          for (int a4 = 0; a4 < NACC / 4; ++a4) {
            const uint2 r2 = wj[u] != 0.0f ? raw[u][a4] : make_uint2(0u, 0u);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r2.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r2.y));
            o[4 * a4] = fmaf(wj[u], lo.x, o[4 * a4]);
            o[4 * a4 + 1] = fmaf(wj[u], lo.y, o[4 * a4 + 1]);
            o[4 * a4 + 2] = fmaf(wj[u], hi.x, o[4 * a4 + 2]);
            o[4 * a4 + 3] = fmaf(wj[u], hi.y, o[4 * a4 + 3]);
          }
        }
      }
    } else {
#pragma unroll 4
      for (int j = 0; j < BKEYS; ++j) {
        const float pjj = __shfl_sync(0xffffffffu, pj, j);
        const int pg = __shfl_sync(0xffffffffu, page, j);
        const bool on = pjj != 0.0f;
        const T* vr = vc + (size_t)(on ? pg : 0) * kv.page_stride + (size_t)((k0 + j) & (kv.page_size - 1)) * v_dim;
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          const int d = lane + 32 * a;
          const float vv = d < v_dim ? Num<T>::to_f(vr[d]) : 0.0f;
          o[a] = fmaf(pjj, on ? vv : 0.0f, o[a]);
        }
      }
    }
  }
  if (lane == 0) { wm[warp] = m; wl[warp] = l; }
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int d = IFX_DIM_OF(a);
    if (d < v_dim) wo[warp * v_dim + d] = o[a];
  }
#undef IFX_DIM_OF
  __syncthreads();
  if (warp == 0) {                                    // the merge: warps in index order, the sink as one more term exp(its score)
    const float sink0 = opt.sink ? (opt.sink_value ? opt.sink_value[head] : 0.0f) : -INFINITY;
    float mm = sink0;
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, wm[w]);
    float ll = opt.sink ? expf(sink0 - mm) : 0.0f;
    float f[DEC_WARPS];
    for (int w = 0; w < DEC_WARPS; ++w) {
      f[w] = wm[w] == -INFINITY ? 0.0f : expf(wm[w] - mm);
      ll += wl[w] * f[w];
    }
    const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
    T* orow = out + (size_t)tok * out_stride + (size_t)head * v_dim;
    for (int d = lane; d < v_dim; d += 32) {
      float y = 0.0f;
      for (int w = 0; w < DEC_WARPS; ++w) y = fmaf(wo[w * v_dim + d], f[w], y);
      y *= inv;
      if (opt.gate) {
        float g = 0.0f;
        for (int sl = 0; sl < opt.gate_parts; ++sl)
          g += opt.gate[(size_t)sl * opt.gate_part_stride + (size_t)tok * opt.gate_stride + (size_t)head * v_dim + d];
        y *= 1.0f / (1.0f + expf(-g));
      }
      orow[d] = Num<T>::from_f(y);
    }
  }
}

template <typename T, int NACC, int DEC_WARPS>
int launch_single_w(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                    int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, AttnOptions opt, cudaStream_t stream) {
  const size_t smem = ((size_t)head_dim + 2 * DEC_WARPS + (size_t)DEC_WARPS * opt.v_dim) * sizeof(float);
  const int rc = launch_pdl(attn_single_token_kernel<T, NACC, DEC_WARPS>, dim3(n_tiles, n_heads), dim3(DEC_WARPS * 32), smem, stream,
                            (const T*)q, q_stride, (T*)out, out_stride, kv, b, n_heads, n_kv, head_dim, scale, window, opt);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

template <typename T, int NACC>
int launch_single(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                  int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, AttnOptions opt, cudaStream_t stream) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
  }
  if ((long long)n_tiles * n_heads <= 2ll * sms)
    return launch_single_w<T, NACC, 32>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  return launch_single_w<T, NACC, 16>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
}

template <typename T>
int dispatch_single(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                    int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, AttnOptions opt, cudaStream_t stream) {
  const int nacc = (opt.v_dim + 31) / 32;
  if (nacc <= 1) return launch_single<T, 1>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  if (nacc <= 2) return launch_single<T, 2>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  if (nacc <= 4) return launch_single<T, 4>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  return launch_single<T, 8>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
}

template <typename T, int NACC>
int launch_generic(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                   int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, AttnOptions opt, cudaStream_t stream) {
  const size_t smem = ((size_t)BQ * head_dim + (size_t)BKEYS * (head_dim + 1) + (size_t)BKEYS * opt.v_dim) * sizeof(float);
  auto kern = attn_paged_generic_kernel<T, NACC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_tiles, n_heads);
  const int ifx_rc = launch_pdl(kern, grid, dim3(256), smem, stream, (const T*)q, q_stride, (T*)out, out_stride, kv, b, n_heads, n_kv,
                                head_dim, scale, window, opt);
  return ifx_rc ? ifx_rc : IFX_LAUNCH_CHECK();
}

template <typename T>
int dispatch_generic(const void* q, long long q_stride, void* out, long long out_stride, PagedKV kv, AttnBatch b,
                     int n_tiles, int n_heads, int n_kv, int head_dim, float scale, int window, AttnOptions opt, cudaStream_t stream) {
  const int nacc = (opt.v_dim + 31) / 32;
  if (nacc <= 1) return launch_generic<T, 1>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  if (nacc <= 2) return launch_generic<T, 2>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  if (nacc <= 4) return launch_generic<T, 4>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  return launch_generic<T, 8>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
}
}  // namespace

// Query tiles are 16 tokens of one entry: tile_entry / tile_q0 list them.
// head_dim and v_dim: any positive size up to 256; n_heads must be a multiple of n_kv.  The options are
// those of AttnOptions; gate: float32 slices [gate_parts][N][gate_stride] whose sum is the gate's argument.
// q_temp_every > 0: the query at position p is multiplied by 1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1);
// dist_r1, dist_r2 ([n_heads] float32 or null): the score of key j loses r1 * ln(1 + r2 * (p - j)), after the cap;
// sink_value ([n_heads] float32 or null): the sink's score where it is not 0.
IFX_API int ifx_attn_paged_generic_ex2(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                       void* k_layer, void* v_layer, long long page_stride, int page_size,
                                       const int* block_tables, int bt_stride,
                                       const int* tile_entry, const int* tile_q0, int n_tiles,
                                       const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                       int n_heads, int n_kv, int head_dim, float scale, int window,
                                       int v_dim, float softcap, int keep_first, int sink,
                                       const float* gate, int gate_parts, long long gate_part_stride, int gate_stride,
                                       int single_tokens, float q_temp_coef, int q_temp_every, const float* dist_r1,
                                       const float* dist_r2, const float* sink_value, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim < 1 || head_dim > 256 || v_dim < 1 || v_dim > 256 || n_kv < 1 || n_heads % n_kv) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  if (n_heads > 65535 || keep_first < 0 || softcap < 0.0f) return IFX_ERR_UNSUPPORTED;
  PagedKV kv;
  kv.k = k_layer; kv.v = v_layer; kv.page_stride = page_stride;
  kv.head_stride = page_size * head_dim; kv.page_size = page_size; kv.page_shift = 0;
  while ((1 << kv.page_shift) < page_size) ++kv.page_shift;
  AttnBatch b{block_tables, bt_stride, tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start};
  if (q_temp_every < 0 || (dist_r1 != nullptr) != (dist_r2 != nullptr)) return IFX_ERR_UNSUPPORTED;
  AttnOptions opt{v_dim, page_size * v_dim, softcap, keep_first, sink, gate, gate_parts, gate_part_stride, gate_stride,
                  q_temp_coef, q_temp_every, dist_r1, dist_r2, sink_value};
  if (single_tokens) {            // every tile is one token (tile_q0 = its place in its entry): the kernel for those
    if (dtype == IFX_F32)
      return dispatch_single<float>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
    if (dtype == IFX_BF16)
      return dispatch_single<bf16>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
    return IFX_ERR_UNSUPPORTED;
  }
  if (dtype == IFX_F32)
    return dispatch_generic<float>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  if (dtype == IFX_BF16)
    return dispatch_generic<bf16>(q, q_stride, out, out_stride, kv, b, n_tiles, n_heads, n_kv, head_dim, scale, window, opt, stream);
  return IFX_ERR_UNSUPPORTED;
}

IFX_API int ifx_attn_paged_generic_ex(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                      void* k_layer, void* v_layer, long long page_stride, int page_size,
                                      const int* block_tables, int bt_stride,
                                      const int* tile_entry, const int* tile_q0, int n_tiles,
                                      const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                      int n_heads, int n_kv, int head_dim, float scale, int window,
                                      int v_dim, float softcap, int keep_first, int sink,
                                      const float* gate, int gate_parts, long long gate_part_stride, int gate_stride,
                                      int single_tokens, cudaStream_t stream) {
  return ifx_attn_paged_generic_ex2(q, q_stride, out, out_stride, dtype, k_layer, v_layer, page_stride, page_size,
                                    block_tables, bt_stride, tile_entry, tile_q0, n_tiles, entry_q_start, entry_q_len,
                                    entry_ctx_start, n_heads, n_kv, head_dim, scale, window, v_dim, softcap, keep_first,
                                    sink, gate, gate_parts, gate_part_stride, gate_stride, single_tokens, 0.0f, 0,
                                    nullptr, nullptr, nullptr, stream);
}

IFX_API int ifx_attn_paged_generic(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                   void* k_layer, void* v_layer, long long page_stride, int page_size,
                                   const int* block_tables, int bt_stride,
                                   const int* tile_entry, const int* tile_q0, int n_tiles,
                                   const int* entry_q_start, const int* entry_q_len, const int* entry_ctx_start,
                                   int n_heads, int n_kv, int head_dim, float scale, int window,
                                   cudaStream_t stream) {
  return ifx_attn_paged_generic_ex(q, q_stride, out, out_stride, dtype, k_layer, v_layer, page_stride, page_size,
                                   block_tables, bt_stride, tile_entry, tile_q0, n_tiles, entry_q_start, entry_q_len,
                                   entry_ctx_start, n_heads, n_kv, head_dim, scale, window, head_dim, 0.0f, 0, 0,
                                   nullptr, 0, 0, 0, 0, stream);
}
