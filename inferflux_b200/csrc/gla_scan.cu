// Gated linear attention: per head a float32 state S [dim x vdim] that every token first shrinks row by row and
// then adds to,
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          o_t = S_t^T (q_t * q_scale)
//   alpha_t = sigmoid(z_t + bias)^(1 / tau)          one decay per head and key channel, in (0, 1)
//
// with z the float32 sums of a small projection of the token.  The decay is worked out in float32 as
// exp(log_sigmoid(z + bias) / tau), log_sigmoid(x) = min(x, 0) - log1p(exp(-|x|)); state, decays and sums are float32
// whatever the engine's type.  The state starts at zero with the sequence (the slot is zeroed when a request takes
// it), is read from the request's state slot at the start of its portion and written back at its end, so a prompt
// may be cut anywhere.
//
// A block takes one (head, entry, 32 value columns) and walks the entry's tokens in order.  A thread holds, of one
// value column, the state rows 4 (g + 4 i) .. + 3 for its row group g in 0..3 (NI groups of four rows, in
// registers); the four threads of a column add their parts of o_t by shuffles.  Tokens are staged 16 (8 for the widest heads) at a time in
// shared memory (q, k, the decays worked out on the way in, and the block's 32 value columns), rows padded with zeros
// to a multiple of 16, so that the inner loop is 16-byte shared loads and fused multiply-adds alone.
#include "common.cuh"

namespace {
constexpr int GLA_COLS = 32;       // value columns a block

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

template <int NI>
__global__ void __launch_bounds__(128)
gla_scan_kernel(const float* __restrict__ proj, long long proj_stride, int q_col, int k_col, int v_col,
                const float* __restrict__ z, long long z_stride, const float* __restrict__ z_bias, float inv_tau,
                float q_scale, float* __restrict__ state, const int* __restrict__ entry_q_start,
                const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot, float* __restrict__ out,
                long long out_stride, int heads, int dim, int vdim) {
  pdl_enter();
  constexpr int DP = 16 * NI;                              // rows, padded
  constexpr int GLA_TOKENS = NI > 12 ? 8 : 16;             // tokens staged at a time (what 48 KB of shared memory hold)
  __shared__ __align__(16) float qs[GLA_TOKENS][DP], ks[GLA_TOKENS][DP], as[GLA_TOKENS][DP];
  __shared__ float vs[GLA_TOKENS][GLA_COLS];
  const int head = blockIdx.x, e = blockIdx.y, c0 = blockIdx.z * GLA_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane & 3;
  const int col = c0 + warp * 8 + (lane >> 2);
  const bool col_ok = col < vdim;
  const int n = entry_q_len[e], t0 = entry_q_start[e], slot = entry_slot[e];
  float* sp = state + ((size_t)slot * heads + head) * dim * vdim;
  float s[NI][4];
#pragma unroll
  for (int i = 0; i < NI; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = 4 * (g + 4 * i) + j;
      s[i][j] = (col_ok && r < dim) ? sp[(size_t)r * vdim + col] : 0.0f;
    }
  for (int base = 0; base < n; base += GLA_TOKENS) {
    const int cnt = min(GLA_TOKENS, n - base);
    __syncthreads();
    for (int idx = tid; idx < cnt * DP; idx += blockDim.x) {
      const int t = idx / DP, d = idx - t * DP;
      float qv = 0.0f, kv = 0.0f, av = 0.0f;
      if (d < dim) {
        const float* pr = proj + (size_t)(t0 + base + t) * proj_stride + (size_t)head * dim + d;
        qv = pr[q_col] * q_scale;
        kv = pr[k_col];
        av = expf(log_sigmoid_f(z[(size_t)(t0 + base + t) * z_stride + (size_t)head * dim + d] + z_bias[head * dim + d]) * inv_tau);
      }
      qs[t][d] = qv; ks[t][d] = kv; as[t][d] = av;
    }
    for (int idx = tid; idx < cnt * GLA_COLS; idx += blockDim.x) {
      const int t = idx / GLA_COLS, c = idx - t * GLA_COLS;
      vs[t][c] = c0 + c < vdim ? proj[(size_t)(t0 + base + t) * proj_stride + v_col + (size_t)head * vdim + c0 + c] : 0.0f;
    }
    __syncthreads();
    for (int t = 0; t < cnt; ++t) {
      const float v = vs[t][warp * 8 + (lane >> 2)];
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int at = 4 * (g + 4 * i);
        const float4 a4 = *reinterpret_cast<const float4*>(&as[t][at]);
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][at]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][at]);
        s[i][0] = fmaf(a4.x, s[i][0], k4.x * v);
        s[i][1] = fmaf(a4.y, s[i][1], k4.y * v);
        s[i][2] = fmaf(a4.z, s[i][2], k4.z * v);
        s[i][3] = fmaf(a4.w, s[i][3], k4.w * v);
        acc0 = fmaf(s[i][0], q4.x, fmaf(s[i][1], q4.y, acc0));
        acc1 = fmaf(s[i][2], q4.z, fmaf(s[i][3], q4.w, acc1));
      }
      float acc = acc0 + acc1;
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (g == 0 && col_ok) out[(size_t)(t0 + base + t) * out_stride + (size_t)head * vdim + col] = acc;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = 4 * (g + 4 * i) + j;
        if (r < dim) sp[(size_t)r * vdim + col] = s[i][j];
      }
  }
}

template <int NI>
int launch_gla(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, const float* z, long long z_stride,
               const float* z_bias, float inv_tau, float q_scale, float* state, const int* entry_q_start,
               const int* entry_q_len, const int* entry_slot, int n_entries, float* out, long long out_stride, int heads,
               int dim, int vdim, cudaStream_t stream) {
  const dim3 grid(heads, n_entries, (vdim + GLA_COLS - 1) / GLA_COLS);
  const int rc = launch_pdl(gla_scan_kernel<NI>, grid, dim3(128), 0, stream, proj, proj_stride, q_col, k_col, v_col, z, z_stride,
                            z_bias, inv_tau, q_scale, state, entry_q_start, entry_q_len, entry_slot, out, out_stride, heads,
                            dim, vdim);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// proj float32 rows hold q and k (heads * dim each) and v (heads * vdim) from the given columns; z float32 rows
// [N, heads * dim]; z_bias float32 [heads * dim]; state float32 [slots, heads, dim, vdim]; out float32 rows
// [N, heads * vdim].  dim up to 256.
IFX_API int ifx_gla_scan(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, const float* z,
                         long long z_stride, const float* z_bias, float inv_tau, float q_scale, float* state,
                         const int* entry_q_start, const int* entry_q_len, const int* entry_slot, int n_entries, float* out,
                         long long out_stride, int heads, int dim, int vdim, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || heads > 65535 || dim < 1 || dim > 256 || vdim < 1 || n_entries > 65535) return IFX_ERR_UNSUPPORTED;
  const int ni = (dim + 15) / 16;
#define IFX_GLA(NI) return launch_gla<NI>(proj, proj_stride, q_col, k_col, v_col, z, z_stride, z_bias, inv_tau, q_scale, state, \
                                          entry_q_start, entry_q_len, entry_slot, n_entries, out, out_stride, heads, dim, vdim, stream)
  if (ni <= 1) IFX_GLA(1);
  if (ni <= 2) IFX_GLA(2);
  if (ni <= 3) IFX_GLA(3);
  if (ni <= 4) IFX_GLA(4);
  if (ni <= 6) IFX_GLA(6);
  if (ni <= 8) IFX_GLA(8);
  if (ni <= 12) IFX_GLA(12);
  IFX_GLA(16);
#undef IFX_GLA
}
