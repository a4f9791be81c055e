// The generalized delta rule: a linear-attention state with a decay per key channel and a removal along the unit key,
// everything float32.  Per head, with S [dim x vdim] (zero at the start of a sequence):
//
//   w_t = exp(-decay_scale * sigmoid(wraw_t + w0))          decay per key channel, in (exp(-decay_scale), 1)
//   a_t = sigmoid(araw_t + ab)                              removal rate per key channel
//   u_t = k_t / sqrt(sum(k_t^2) + key_eps)                  the unit key of the head
//   S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T        both terms read the old state
//   o_t = S_t^T r_t
//
// The scan runs a block per (head, entry, block of value columns); a thread owns one value column and every LN-th
// key row of it (R rows in registers).  A token costs one reduction over the key rows for u^T S, the update, and a
// second reduction for the output.  Tokens are staged through shared memory TC at a time, where the decay, the
// removal rate and the unit key are computed once per block.  The state of a sequence lives in its slot as
// [heads][vdim][dim] float32, read at the start of an entry and written at its end, so a prompt may be cut
// anywhere and a decoded token is the same kernel with one token.
//
// The finish brings every head's output to unit root mean square, multiplies by a weight over all heads and by
// sigmoid(gate), and rounds once into the engine's type.
#include "common.cuh"

namespace {
constexpr int R = 16;           // key rows a thread holds
constexpr int TC = 8;           // tokens staged at a time

struct DeltaArgs {
  const float* proj; long long stride; int r_col, k_col, v_col, a_col;   // float32 rows: r, k, v heads and raw removal rates
  const float* wraw; long long w_stride;                                 // raw decays [row][heads * dim]
  const float* w0; const float* ab;                                      // [heads * dim]
  float* state;                                                          // [slots][heads][vdim][dim]
  const int* entry_q_start; const int* entry_q_len; const int* entry_slot;
  float* out; long long out_stride;                                      // [row][heads * vdim]
  int heads, dim, vdim, ln, cols_per_block;
  float decay_scale, key_eps;
};

__global__ void __launch_bounds__(1024)
delta_rule_scan_kernel(DeltaArgs p) {
  extern __shared__ float sm[];
  const int LN = p.ln, NP = R * LN, PB = p.cols_per_block;
  float* rs = sm;                       // [TC][NP]
  float* ks = rs + TC * NP;             // [TC][NP]
  float* us = ks + TC * NP;             // [TC][NP]  unit key
  float* ws = us + TC * NP;             // [TC][NP]  decay
  float* as = ws + TC * NP;             // [TC][NP]  removal rate times unit key
  float* vs = as + TC * NP;             // [TC][PB]
  pdl_enter();
  const int h = blockIdx.x, e = blockIdx.y, p0 = blockIdx.z * PB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int pl = tid / LN, ln = tid - pl * LN;
  const int col = p0 + pl;
  const bool valid = pl < PB && col < p.vdim;
  const int r0 = p.entry_q_start[e], len = p.entry_q_len[e];
  const int hd = h * p.dim;
  float* st = p.state + (((size_t)p.entry_slot[e] * p.heads + h) * p.vdim + (valid ? col : 0)) * p.dim;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = i * LN + ln;
    S[i] = (valid && n < p.dim) ? st[n] : 0.0f;
  }
  for (int t0 = 0; t0 < len; t0 += TC) {
    const int nt = min(TC, len - t0);
    __syncthreads();
    for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
      const int tt = idx / NP, n = idx - tt * NP;
      const size_t row = (size_t)(r0 + t0 + tt);
      const bool on = n < p.dim;
      const float* pr = p.proj + row * p.stride;
      rs[idx] = on ? pr[p.r_col + hd + n] : 0.0f;
      ks[idx] = on ? pr[p.k_col + hd + n] : 0.0f;
      const float wr = on ? p.wraw[row * p.w_stride + hd + n] + p.w0[hd + n] : 0.0f;
      ws[idx] = on ? expf(-p.decay_scale / (1.0f + expf(-wr))) : 0.0f;
      const float ar = on ? pr[p.a_col + hd + n] + p.ab[hd + n] : 0.0f;
      as[idx] = on ? 1.0f / (1.0f + expf(-ar)) : 0.0f;
    }
    for (int idx = tid; idx < nt * PB; idx += blockDim.x) {
      const int tt = idx / PB, c = idx - tt * PB;
      vs[idx] = p0 + c < p.vdim ? p.proj[(size_t)(r0 + t0 + tt) * p.stride + p.v_col + h * p.vdim + p0 + c] : 0.0f;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += nwarps) {            // the unit key: a warp a token, a fixed order of additions
      float ss = 0.0f;
      for (int n = lane; n < NP; n += 32) ss = fmaf(ks[tt * NP + n], ks[tt * NP + n], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + p.key_eps);
      for (int n = lane; n < NP; n += 32) {
        const float u = ks[tt * NP + n] * inv;
        us[tt * NP + n] = u;
        as[tt * NP + n] *= u;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* u = us + tt * NP + ln;
      const float* w = ws + tt * NP + ln;
      const float* au = as + tt * NP + ln;
      const float* k = ks + tt * NP + ln;
      const float* r = rs + tt * NP + ln;
      const float v = pl < PB ? vs[tt * PB + pl] : 0.0f;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < R; ++i) dot = fmaf(u[i * LN], S[i], dot);
      for (int o = LN >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      float y = 0.0f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] = fmaf(w[i * LN], S[i], fmaf(k[i * LN], v, -au[i * LN] * dot));
        y = fmaf(S[i], r[i * LN], y);
      }
      for (int o = LN >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (valid && ln == 0) p.out[(size_t)(r0 + t0 + tt) * p.out_stride + h * p.vdim + col] = y;
    }
  }
  if (valid) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = i * LN + ln;
      if (n < p.dim) st[n] = S[i];
    }
  }
}

// out[t][h] = o[t][h] / sqrt(mean(o[t][h]^2) + eps) * w[h] * gate(g[t][h]); a warp a (token, head).
// gate: 0 none, 1 sigmoid, 2 silu.  w may be null.
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, long long o_stride, const float* __restrict__ g, long long g_stride,
                      const float* __restrict__ w, TO* __restrict__ out, long long out_stride, int n_rows, int heads,
                      int vdim, float eps, int gate) {
  pdl_enter();
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_rows * heads) return;
  const int t = idx / heads, h = idx - t * heads;
  const float* src = o + (size_t)t * o_stride + (size_t)h * vdim;
  float ss = 0.0f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  const float* gr = g ? g + (size_t)t * g_stride + (size_t)h * vdim : nullptr;
  TO* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
  for (int i = lane; i < vdim; i += 32) {
    float v = src[i] * inv;
    if (w) v *= w[h * vdim + i];
    if (gate == 1) v *= 1.0f / (1.0f + expf(-gr[i]));
    else if (gate == 2) v *= gr[i] / (1.0f + expf(-gr[i]));
    dst[i] = Num<TO>::from_f(v);
  }
}
}  // namespace

// proj float32 rows hold r, k, v heads and the raw removal rates from the given columns on; wraw float32 rows the raw
// decays; state float32 [slots][heads][vdim][dim]; out float32 rows of heads * vdim.
IFX_API int ifx_delta_rule_scan(const float* proj, long long stride, int r_col, int k_col, int v_col, int a_col,
                                const float* wraw, long long w_stride, const float* w0, const float* ab, float* state,
                                const int* entry_q_start, const int* entry_q_len, const int* entry_slot, int n_entries,
                                float* out, long long out_stride, int heads, int dim, int vdim, float decay_scale,
                                float key_eps, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || dim < 1 || dim > R * 32 || vdim < 1 || n_entries > 65535) return IFX_ERR_UNSUPPORTED;
  int ln = 1;
  while (R * ln < dim) ln <<= 1;
  int pb = 256 / ln;                      // blocks of at most 256 threads: more blocks to spread over the SMs
  if (pb > vdim) pb = vdim;
  if (pb > 16 && heads * n_entries * ((vdim + pb - 1) / pb) < 148) pb = 16;
  const int threads = (pb * ln + 31) / 32 * 32;
  DeltaArgs p{proj, stride, r_col, k_col, v_col, a_col, wraw, w_stride, w0, ab, state, entry_q_start, entry_q_len, entry_slot,
              out, out_stride, heads, dim, vdim, ln, pb, decay_scale, key_eps};
  const size_t smem = (size_t)TC * (5 * R * ln + pb) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(delta_rule_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int rc = launch_pdl(delta_rule_scan_kernel, dim3(heads, n_entries, (vdim + pb - 1) / pb), dim3(threads), smem, stream, p);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// o float32 [n][heads * vdim] (rows o_stride apart), g float32 rows (the gate's sums, g_stride apart) or null, w float32
// [heads * vdim] or null; out rows of either type.
IFX_API int ifx_head_norm_gate(const float* o, long long o_stride, const float* g, long long g_stride, const float* w,
                               void* out, int out_dtype, long long out_stride, int n_rows, int heads, int vdim, float eps,
                               int gate, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (heads < 1 || vdim < 1 || gate < 0 || gate > 2 || (gate && !g)) return IFX_ERR_UNSUPPORTED;
  const long long warps = (long long)n_rows * heads;
  const int blocks = (int)((warps + 7) / 8);
  int rc;
  if (out_dtype == IFX_BF16)
    rc = launch_pdl(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, o, o_stride, g, g_stride, w, (bf16*)out,
                    out_stride, n_rows, heads, vdim, eps, gate);
  else if (out_dtype == IFX_F32)
    rc = launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, o, o_stride, g, g_stride, w, (float*)out,
                    out_stride, n_rows, heads, vdim, eps, gate);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}
