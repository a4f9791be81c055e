// Routed experts: every token runs `top` of `experts` small feed-forwards and adds their results, weighted.
//
//   z = the router's float32 logits of a token;  chosen = the `top` largest (lowest index first among equals);
//   weight_k = exp(z_k) / sum over the chosen exp(z)                                           (route)
//   the (token, choice) pairs are sorted by expert into tiles of TILE rows, each tile one expert's (group)
//   act = silu(x Wg_e^T) * (x Wu_e^T)   per tile, rows gathered from the tokens                 (expert_product)
//   y   = act Wd_e^T                    per tile, float32
//   out[token] = sum_k weight_k y[pair]  in the order of the choices                            (combine)
//
// Nothing here visits the host: the number of tiles that a step can need at most (pairs / TILE + experts) is
// launched, and tiles beyond those in use return at once.  A pair's result does not depend on where in a tile
// it lands (every output element adds its K products in index order), so the sort's order does not show.
// The products are FFMA with float32 sums for either element type.
#include "common.cuh"

namespace {
constexpr int MAX_TOP = 64;
// what a tile product does with its sums: nothing; W_e = [gate rows; up rows] and out = silu(gate) * up; out = relu(sum)^2
constexpr int MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_RELU2 = 2;

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int n_tokens, int experts, int top, int over_all, float scale,
                 int* __restrict__ chosen, float* __restrict__ weights) {
  pdl_enter();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * experts;
  int ids[MAX_TOP]; float vals[MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY; int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      bool taken = false;
      for (int u = 0; u < k; ++u) taken |= ids[u] == e;
      const float v = z[e];
      if (!taken && (v > best || (v == best && e < arg))) { best = v; arg = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    ids[k] = arg; vals[k] = best;
  }
  if (over_all) {
    // scores are the softmax over every expert; a chosen one's weight is its score over the chosen scores' sum
    float all = 0.0f;
    for (int e = lane; e < experts; e += 32) all += expf(z[e] - vals[0]);
    all = warp_sum(all);
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) sum += expf(vals[k] - vals[0]) / all;
    for (int k = lane; k < top; k += 32) {
      chosen[(size_t)t * top + k] = ids[k];
      weights[(size_t)t * top + k] = expf(vals[k] - vals[0]) / all / (sum + 1e-20f) * scale;
    }
    return;
  }
  float sum = 0.0f;
  for (int k = 0; k < top; ++k) sum += expf(vals[k] - vals[0]);      // vals[0] is the largest
  for (int k = lane; k < top; k += 32) {
    chosen[(size_t)t * top + k] = ids[k];
    weights[(size_t)t * top + k] = expf(vals[k] - vals[0]) / sum * scale;
  }
}

// One block: counts per expert, tiles per expert, a place for every pair.
//   tile_expert[max_tiles]: the expert of each tile or -1;  sorted_pair[max_tiles * tile]: the pair at each sorted
//   row or -1;  pair_row[pairs]: the sorted row of each pair.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int pairs, int experts, int tile, int max_tiles,
                 int* __restrict__ tile_expert, int* __restrict__ sorted_pair, int* __restrict__ pair_row) {
  pdl_enter();
  extern __shared__ int sm[];
  int* count = sm;                 // [experts]
  int* first = count + experts;    // [experts] first sorted row of the expert
  int* cursor = first + experts;   // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) sorted_pair[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&count[chosen[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = t * tile;
      const int n = (count[e] + tile - 1) / tile;
      for (int k = 0; k < n; ++k) tile_expert[t + k] = e;
      t += n;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    const int r = first[e] + atomicAdd(&cursor[e], 1);
    sorted_pair[r] = i;
    pair_row[i] = r;
  }
}

// C tile = A rows (gathered) x W_e^T.  SWIGLU: W_e is [2 * n_out][K] (gate rows, then up rows) and the tile's
// columns are n_out wide: out = silu(gate) * up in TO.  Otherwise W_e is [n_out][K] and out is float32.
// BM = 16 * TM rows a tile.
template <typename TA, typename TW, typename TO, int TM, int MODE>
__global__ void __launch_bounds__(256)
moe_product_kernel(const TA* __restrict__ A, long long lda, int gather_div /* 0: rows are sorted rows; else token = pair / gather_div */,
                   const TW* __restrict__ W, const int* __restrict__ tile_expert, const int* __restrict__ sorted_pair,
                   TO* __restrict__ C, long long ldc, int n_out, int K) {
  constexpr bool SWIGLU = MODE == MODE_SWIGLU;
  constexpr int BM = 16 * TM, BN = 64, BK = 16;
  constexpr int TN = SWIGLU ? 2 : 4;                // per thread: TM x TN outputs (SWIGLU: of gate and of up each)
  pdl_enter();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int rows[BM];
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int cols = SWIGLU ? BN / 2 : BN;            // output columns per block
  const int n0 = blockIdx.x * cols;
  const TW* We = W + (size_t)e * (SWIGLU ? 2 : 1) * n_out * K;
  if (tid < BM) {
    const int pair = sorted_pair[tile * BM + tid];
    rows[tid] = pair < 0 ? -1 : (gather_div ? pair / gather_div : tile * BM + tid);
  }
  __syncthreads();
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += 256) {
      const int r = idx / BK, k = idx - r * BK;
      const int src = rows[r];
      As[k][r] = (src >= 0 && k0 + k < K) ? Num<TA>::to_f(A[(size_t)src * lda + k0 + k]) : 0.0f;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int c = idx / BK, k = idx - c * BK;
      int wrow;                                      // which row of W_e feeds the tile's local column c
      if (SWIGLU) wrow = c < cols ? n0 + c : n_out + n0 + (c - cols);
      else wrow = n0 + c;
      const bool ok = (SWIGLU ? (c < cols ? n0 + c : n0 + c - cols) : n0 + c) < n_out && k0 + k < K;
      Ws[k][c] = ok ? Num<TW>::to_f(We[(size_t)wrow * K + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
      if (SWIGLU) {
        w[0] = Ws[kk][tx * 2]; w[1] = Ws[kk][tx * 2 + 1]; w[2] = Ws[kk][cols + tx * 2]; w[3] = Ws[kk][cols + tx * 2 + 1];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (rows[r] < 0) continue;
    TO* crow = C + (size_t)(tile * BM + r) * ldc;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= n_out) continue;
      if (SWIGLU) {
        const float g = acc[i][j], u = acc[i][2 + j];
        crow[n] = Num<TO>::from_f(g / (1.0f + expf(-g)) * u);
      } else if (MODE == MODE_RELU2) {
        const float r = fmaxf(acc[i][j], 0.0f);
        crow[n] = Num<TO>::from_f(r * r);
      } else {
        crow[n] = Num<TO>::from_f(acc[i][j]);
      }
    }
  }
}

// The same tile product for bfloat16 and short tiles (16 rows: steps of single tokens) on tensor cores: the 16 rows
// are the rows of one m16n8k16 MMA, a warp owns 16 of the block's 64 rows of W_e (SwiGLU: 8 gate rows and the 8 up
// rows that belong to them), operands go through shared memory 64 K at a time by 16-byte loads.  Such a step is
// bound by reading the chosen experts' weights once; the arithmetic of the FFMA tiles above took three times as long.
__device__ __forceinline__ void moe_mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TO, int MODE>
__global__ void __launch_bounds__(128)
moe_product_mma_kernel(const bf16* __restrict__ A, long long lda, int gather_div, const bf16* __restrict__ W,
                       const int* __restrict__ tile_expert, const int* __restrict__ sorted_pair, TO* __restrict__ C,
                       long long ldc, int n_out, int K) {
  constexpr bool SWIGLU = MODE == MODE_SWIGLU;
  constexpr int BM = 16, BN = 64, BK = 64, LD = BK + 8;
  pdl_enter();
  __shared__ __align__(16) bf16 As[BM][LD];
  __shared__ __align__(16) bf16 Ws[BN][LD];
  __shared__ int rows[BM];
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  constexpr int cols = SWIGLU ? BN / 2 : BN;
  const int n0 = blockIdx.x * cols;
  const bf16* We = W + (size_t)e * (SWIGLU ? 2 : 1) * n_out * K;
  if (tid < BM) {
    const int pair = sorted_pair[tile * BM + tid];
    rows[tid] = pair < 0 ? -1 : (gather_div ? pair / gather_div : tile * BM + tid);
  }
  __syncthreads();
  // the two rows of W_e's tile that feed this thread's two accumulators, and which output columns they are
  const int r0 = SWIGLU ? 8 * warp + g : 16 * warp + g;
  const int r1 = SWIGLU ? cols + 8 * warp + g : 16 * warp + 8 + g;
  float acc0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int r = tid >> 3, c8 = (tid & 7) * 8;
      const int src = rows[r];
      *reinterpret_cast<uint4*>(&As[r][c8]) = (src >= 0 && k0 + c8 < K)
          ? *reinterpret_cast<const uint4*>(A + (size_t)src * lda + k0 + c8) : zero;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = tid + 128 * i, c = v >> 3, c8 = (v & 7) * 8;
      const int col = SWIGLU ? (c < cols ? n0 + c : n0 + c - cols) : n0 + c;        // the output column this row of the tile feeds
      const int wrow = SWIGLU && c >= cols ? n_out + col : col;
      *reinterpret_cast<uint4*>(&Ws[c][c8]) = (col < n_out && k0 + c8 < K)
          ? *reinterpret_cast<const uint4*>(We + (size_t)wrow * K + k0 + c8) : zero;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      unsigned a[4];
      a[0] = *reinterpret_cast<const unsigned*>(&As[g][kk + 2 * t]);
      a[1] = *reinterpret_cast<const unsigned*>(&As[g + 8][kk + 2 * t]);
      a[2] = *reinterpret_cast<const unsigned*>(&As[g][kk + 8 + 2 * t]);
      a[3] = *reinterpret_cast<const unsigned*>(&As[g + 8][kk + 8 + 2 * t]);
      moe_mma_bf16(acc0, a, *reinterpret_cast<const unsigned*>(&Ws[r0][kk + 2 * t]),
                   *reinterpret_cast<const unsigned*>(&Ws[r0][kk + 8 + 2 * t]));
      moe_mma_bf16(acc1, a, *reinterpret_cast<const unsigned*>(&Ws[r1][kk + 2 * t]),
                   *reinterpret_cast<const unsigned*>(&Ws[r1][kk + 8 + 2 * t]));
    }
    __syncthreads();
  }
  // accumulator layout: [0], [1] = row g, columns 2t and 2t + 1; [2], [3] = row g + 8, the same columns
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    if (rows[r] < 0) continue;
    TO* crow = C + (size_t)(tile * BM + r) * ldc;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (SWIGLU) {
        const int n = n0 + 8 * warp + 2 * t + j;
        const float gt = acc0[2 * h + j], up = acc1[2 * h + j];
        if (n < n_out) crow[n] = Num<TO>::from_f(gt / (1.0f + expf(-gt)) * up);
      } else {
        const int na = n0 + 16 * warp + 2 * t + j, nb = na + 8;
        float va = acc0[2 * h + j], vb = acc1[2 * h + j];
        if (MODE == MODE_RELU2) { va = fmaxf(va, 0.0f); va *= va; vb = fmaxf(vb, 0.0f); vb *= vb; }
        if (na < n_out) crow[na] = Num<TO>::from_f(va);
        if (nb < n_out) crow[nb] = Num<TO>::from_f(vb);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ weights,
                   float* __restrict__ out, int hidden, int top) {
  pdl_enter();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(size_t)t * top + k], y[(size_t)pair_row[(size_t)t * top + k] * hidden + i], acc);
    out[(size_t)t * hidden + i] = acc;
  }
}

// act: MODE_SWIGLU (w_up = [gate rows; up rows] of every expert) or MODE_RELU2 (w_up = up rows alone)
int launch_products_mma(const void* x, const void* w_up, const void* w_down, const int* tile_expert, const int* sorted_pair,
                        void* act_out, float* y, int max_tiles, int hidden, int ff, int top, int act, cudaStream_t stream) {
  int rc = act == MODE_SWIGLU
      ? launch_pdl(moe_product_mma_kernel<bf16, MODE_SWIGLU>, dim3((ff + 31) / 32, max_tiles), dim3(128), 0, stream,
                   (const bf16*)x, (long long)hidden, top, (const bf16*)w_up, tile_expert, sorted_pair, (bf16*)act_out,
                   (long long)ff, ff, hidden)
      : launch_pdl(moe_product_mma_kernel<bf16, MODE_RELU2>, dim3((ff + 63) / 64, max_tiles), dim3(128), 0, stream,
                   (const bf16*)x, (long long)hidden, top, (const bf16*)w_up, tile_expert, sorted_pair, (bf16*)act_out,
                   (long long)ff, ff, hidden);
  if (rc) return rc;
  return launch_pdl(moe_product_mma_kernel<float, MODE_PLAIN>, dim3((hidden + 63) / 64, max_tiles), dim3(128), 0, stream,
                    (const bf16*)act_out, (long long)ff, 0, (const bf16*)w_down, tile_expert, sorted_pair, y, (long long)hidden,
                    hidden, ff);
}

template <typename T, int TM>
int launch_products(const void* x, const void* w_up, const void* w_down, const int* tile_expert, const int* sorted_pair,
                    void* act_out, float* y, int max_tiles, int hidden, int ff, int top, int act, cudaStream_t stream) {
  int rc = act == MODE_SWIGLU
      ? launch_pdl(moe_product_kernel<T, T, T, TM, MODE_SWIGLU>, dim3((ff + 31) / 32, max_tiles), dim3(256), 0, stream,
                   (const T*)x, (long long)hidden, top, (const T*)w_up, tile_expert, sorted_pair, (T*)act_out,
                   (long long)ff, ff, hidden)
      : launch_pdl(moe_product_kernel<T, T, T, TM, MODE_RELU2>, dim3((ff + 63) / 64, max_tiles), dim3(256), 0, stream,
                   (const T*)x, (long long)hidden, top, (const T*)w_up, tile_expert, sorted_pair, (T*)act_out,
                   (long long)ff, ff, hidden);
  if (rc) return rc;
  return launch_pdl(moe_product_kernel<T, T, float, TM, MODE_PLAIN>, dim3((hidden + 63) / 64, max_tiles), dim3(256), 0, stream,
                    (const T*)act_out, (long long)ff, 0, (const T*)w_down, tile_expert, sorted_pair, y, (long long)hidden,
                    hidden, ff);
}
}  // namespace

// xs[r] = x[pair / top] for the pair at sorted row r, zeros where a row holds no pair
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ sorted_pair, T* __restrict__ xs, int hidden, int top) {
  pdl_enter();
  const int r = blockIdx.x;
  const int pair = sorted_pair[r];
  const T* src = pair >= 0 ? x + (size_t)(pair / top) * hidden : nullptr;
  T* dst = xs + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src ? src[i] : Num<T>::from_f(0.0f);
}

// The sort alone (for callers that run the tiles' products with a kernel of their own): tile = rows per tile.
IFX_API int ifx_moe_group(const int* chosen, int pairs, int experts, int tile, int max_tiles, int* tile_expert,
                          int* sorted_pair, int* pair_row, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (tile < 1 || max_tiles < pairs / tile + experts || experts > 4096) return IFX_ERR_UNSUPPORTED;
  const int rc = launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)3 * experts * sizeof(int), stream, chosen, pairs,
                            experts, tile, max_tiles, tile_expert, sorted_pair, pair_row);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_moe_gather_rows(const void* x, int dtype, const int* sorted_pair, void* xs, int rows, int hidden, int top,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int rc = dtype == IFX_BF16
      ? launch_pdl(moe_gather_rows_kernel<bf16>, dim3(rows), dim3(256), 0, stream, (const bf16*)x, sorted_pair, (bf16*)xs, hidden, top)
      : launch_pdl(moe_gather_rows_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)x, sorted_pair, (float*)xs, hidden, top);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_moe_combine(const float* y, const int* pair_row, const float* weights, float* out, int n_tokens, int hidden,
                            int top, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int rc = launch_pdl(moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, y, pair_row, weights, out, hidden, top);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// over_all 0: weights are the softmax over the chosen logits alone; 1: the softmax over every expert's logit, the
// chosen ones' scores divided by their sum (+ 1e-20).  Either is multiplied by scale.
IFX_API int ifx_moe_route(const float* logits, int n_tokens, int experts, int top, int over_all, float scale, int* chosen,
                          float* weights, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (top < 1 || top > MAX_TOP || top > experts) return IFX_ERR_UNSUPPORTED;
  const int rc = launch_pdl(moe_route_kernel, dim3((n_tokens + 7) / 8), dim3(256), 0, stream, logits, n_tokens, experts, top,
                            over_all, scale, chosen, weights);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// Rows per tile for a step of n_tokens * top pairs: few pairs (single-token steps) take short tiles.
IFX_API int ifx_moe_tile_rows(int pairs) { return pairs <= 256 ? 16 : 64; }

// act 1: w_gate_up [experts][2 ff][hidden] and silu(gate) * up; act 2: w_gate_up [experts][ff][hidden] (up rows alone) and
// relu(up)^2.
// x [N][hidden], w_gate_up [experts][2 ff][hidden], w_down [experts][hidden][ff] of one element type `dtype`;
// act [max_tiles * tile][ff] of that type, y [max_tiles * tile][hidden] float32, out [N][hidden] float32.
// max_tiles >= pairs / tile + experts, tile = ifx_moe_tile_rows(pairs).
IFX_API int ifx_moe_experts(const void* x, int dtype, const void* w_gate_up, const void* w_down, const int* chosen,
                            const float* weights, int n_tokens, int hidden, int ff, int experts, int top, int activation, int tile,
                            int max_tiles, int* tile_expert, int* sorted_pair, int* pair_row, void* act, float* y,
                            float* out, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int pairs = n_tokens * top;
  if ((tile != 16 && tile != 64) || max_tiles < pairs / tile + experts || experts > 4096) return IFX_ERR_UNSUPPORTED;
  if (activation != MODE_SWIGLU && activation != MODE_RELU2) return IFX_ERR_UNSUPPORTED;
  int rc = launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)3 * experts * sizeof(int), stream, chosen, pairs, experts,
                      tile, max_tiles, tile_expert, sorted_pair, pair_row);
  if (rc) return rc;
  if (dtype == IFX_F32)
    rc = tile == 16 ? launch_products<float, 1>(x, w_gate_up, w_down, tile_expert, sorted_pair, act, y, max_tiles, hidden, ff, top, activation, stream)
                    : launch_products<float, 4>(x, w_gate_up, w_down, tile_expert, sorted_pair, act, y, max_tiles, hidden, ff, top, activation, stream);
  else if (dtype == IFX_BF16 && tile == 16 && hidden % 8 == 0 && ff % 8 == 0 &&
           (((uintptr_t)x | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)act) & 15) == 0)
    rc = launch_products_mma(x, w_gate_up, w_down, tile_expert, sorted_pair, act, y, max_tiles, hidden, ff, top, activation, stream);
  else if (dtype == IFX_BF16)
    rc = tile == 16 ? launch_products<bf16, 1>(x, w_gate_up, w_down, tile_expert, sorted_pair, act, y, max_tiles, hidden, ff, top, activation, stream)
                    : launch_products<bf16, 4>(x, w_gate_up, w_down, tile_expert, sorted_pair, act, y, max_tiles, hidden, ff, top, activation, stream);
  else
    return IFX_ERR_UNSUPPORTED;
  if (rc) return rc;
  rc = launch_pdl(moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)y, (const int*)pair_row, weights, out,
                  hidden, top);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
