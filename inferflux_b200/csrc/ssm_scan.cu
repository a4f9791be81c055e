// A selective state-space layer's two time-dependent steps, everything float32:
//
//   causal convolution   y_t[c] = act(b[c] + sum_{j < taps} w[c][j] * u_{t - taps + 1 + j}[c]),  u = 0 ahead of a
//                        sequence's first token; the last taps-1 inputs of every sequence live in its state slot
//                        ("tail") and are brought up to date by a second kernel after all rows have been read
//   scan                 per head h (its B and C from group h / (heads / groups)):
//                          dt_t = softplus(raw_t[h] + dt_bias[h])          (no clamp)
//                          S_t  = exp(-exp(A_log[h]) dt_t) S_{t-1} + dt_t B_t x_t^T        S: [state x vdim]
//                          y_t  = S_t^T C_t + D[h] x_t
//
// The scan runs a block per (entry, head, block of value columns); a thread owns one value column and every
// LN-th state row of it (R rows in registers), so a token costs R multiply-adds for the state, R for the result
// and log2(LN) shuffles.  Tokens are staged through shared memory TC at a time.  The state of a sequence lives in
// its slot as [heads][vdim][state] float32, is read at the start of the entry and written at its end, so a
// prompt may be cut anywhere and a decoded token is the same kernel with one token.
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 16;
constexpr int R = 16;           // state rows a thread holds
constexpr int TC = 16;          // tokens staged at a time

struct ConvArgs {
  const float* in; long long in_stride; int col0;       // u = in[row][col0 + c]
  const float* w; const float* bias; int taps;          // w [channels][taps]
  float* tail;                                          // [slots][taps-1][channels]
  const int* row_entry; const int* entry_q_start; const int* entry_q_len; const int* entry_slot;
  float* out; long long out_stride; int channels; int act;   // act 0: none, 1: silu
};

__global__ void __launch_bounds__(256)
causal_conv_kernel(ConvArgs p) {
  pdl_enter();
  const int row = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.channels) return;
  const int e = p.row_entry[row];
  const int i = row - p.entry_q_start[e];
  const int keep = p.taps - 1;
  const float* tail = p.tail ? p.tail + (size_t)p.entry_slot[e] * keep * p.channels : nullptr;
  float y = p.bias ? p.bias[c] : 0.0f;
  const float* w = p.w + (size_t)c * p.taps;
  for (int j = 0; j < p.taps; ++j) {
    const int m = i - keep + j;                        // which token of the entry, negative = before this step
    const float u = m >= 0 ? p.in[(size_t)(row - (i - m)) * p.in_stride + p.col0 + c]
                           : tail[(size_t)(keep + m) * p.channels + c];
    y = fmaf(w[j], u, y);
  }
  if (p.act == 1) y = y / (1.0f + expf(-y));
  p.out[(size_t)row * p.out_stride + c] = y;
}

// After the rows have been read: the tail becomes the last taps-1 rows of (old tail ++ the entry's new inputs).
__global__ void __launch_bounds__(256)
causal_conv_tail_kernel(ConvArgs p) {
  pdl_enter();
  const int e = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.channels) return;
  const int keep = p.taps - 1, len = p.entry_q_len[e], r0 = p.entry_q_start[e];
  float* tail = p.tail + (size_t)p.entry_slot[e] * keep * p.channels;
  float v[MAX_TAPS];
  for (int s = 0; s < keep; ++s) {
    const int m = len + s;                             // index into (old tail ++ new rows)
    v[s] = m < keep ? tail[(size_t)m * p.channels + c] : p.in[(size_t)(r0 + m - keep) * p.in_stride + p.col0 + c];
  }
  for (int s = 0; s < keep; ++s) tail[(size_t)s * p.channels + c] = v[s];
}

struct SsmArgs {
  const float* xbc; long long xbc_stride; int x_col, b_col, c_col;     // convolved x, B, C rows
  const float* dt; long long dt_stride;                                // raw dt, [row][head]
  const float* dt_bias; const float* a_log; const float* d_skip;       // [heads]
  float* state;                                                        // [slots][heads][vdim][n_state]
  const int* entry_q_start; const int* entry_q_len; const int* entry_slot;
  float* out; long long out_stride;                                    // [row][heads * vdim]
  int heads, groups, vdim, n_state, ln, cols_per_block;
};

__global__ void __launch_bounds__(1024)
ssm_scan_kernel(SsmArgs p) {
  extern __shared__ float sm[];
  const int LN = p.ln, NP = R * LN, PB = p.cols_per_block;
  float* Bs = sm;                       // [TC][NP]
  float* Cs = Bs + TC * NP;             // [TC][NP]
  float* xs = Cs + TC * NP;             // [TC][PB]
  float* dts = xs + TC * PB;            // [TC]
  float* decs = dts + TC;               // [TC]
  pdl_enter();
  const int h = blockIdx.x, e = blockIdx.y, p0 = blockIdx.z * PB;
  const int tid = threadIdx.x;
  const int pl = tid / LN, ln = tid - pl * LN;
  const int col = p0 + pl;
  const bool valid = pl < PB && col < p.vdim;
  const int g = h / (p.heads / p.groups);
  const int r0 = p.entry_q_start[e], len = p.entry_q_len[e];
  const float bias = p.dt_bias[h], neg_a = -expf(p.a_log[h]), dskip = p.d_skip[h];
  float* st = p.state + (((size_t)p.entry_slot[e] * p.heads + h) * p.vdim + (valid ? col : 0)) * p.n_state;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = i * LN + ln;
    S[i] = (valid && n < p.n_state) ? st[n] : 0.0f;
  }
  for (int t0 = 0; t0 < len; t0 += TC) {
    const int nt = min(TC, len - t0);
    __syncthreads();
    for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
      const int tt = idx / NP, n = idx - tt * NP;
      const float* row = p.xbc + (size_t)(r0 + t0 + tt) * p.xbc_stride;
      const bool on = n < p.n_state;
      Bs[idx] = on ? row[p.b_col + g * p.n_state + n] : 0.0f;
      Cs[idx] = on ? row[p.c_col + g * p.n_state + n] : 0.0f;
    }
    for (int idx = tid; idx < nt * PB; idx += blockDim.x) {
      const int tt = idx / PB, c = idx - tt * PB;
      xs[idx] = p0 + c < p.vdim ? p.xbc[(size_t)(r0 + t0 + tt) * p.xbc_stride + p.x_col + h * p.vdim + p0 + c] : 0.0f;
    }
    if (tid < nt) {
      const float raw = p.dt[(size_t)(r0 + t0 + tid) * p.dt_stride + h] + bias;
      const float dtv = raw > 20.0f ? raw : log1pf(expf(raw));
      dts[tid] = dtv;
      decs[tid] = expf(neg_a * dtv);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dtv = dts[tt], dec = decs[tt];
      const float xv = pl < PB ? xs[tt * PB + pl] : 0.0f;
      const float bx = dtv * xv;
      const float* b = Bs + tt * NP + ln;
      const float* c = Cs + tt * NP + ln;
      float y = 0.0f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] = fmaf(dec, S[i], bx * b[i * LN]);
        y = fmaf(S[i], c[i * LN], y);
      }
      for (int o = LN >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (valid && ln == 0) p.out[(size_t)(r0 + t0 + tt) * p.out_stride + h * p.vdim + col] = fmaf(dskip, xv, y);
    }
  }
  if (valid) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = i * LN + ln;
      if (n < p.n_state) st[n] = S[i];
    }
  }
}
}  // namespace

// out[row][c] = act(bias[c] + the convolution of column col0 + c of `in` over time), see the header.  tail may be
// null when taps is 1.  The tail is brought up to date by the second launch.
IFX_API int ifx_causal_conv(const float* in, long long in_stride, int col0, const float* w, const float* bias, int taps,
                            float* tail, const int* row_entry, const int* entry_q_start, const int* entry_q_len,
                            const int* entry_slot, int n_rows, int n_entries, float* out, long long out_stride,
                            int channels, int act, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS || channels < 1 || (taps > 1 && !tail) || act < 0 || act > 1) return IFX_ERR_UNSUPPORTED;
  ConvArgs p{in, in_stride, col0, w, bias, taps, tail, row_entry, entry_q_start, entry_q_len, entry_slot, out, out_stride,
             channels, act};
  int rc = launch_pdl(causal_conv_kernel, dim3(n_rows, (channels + 255) / 256), dim3(256), 0, stream, p);
  if (!rc && taps > 1)
    rc = launch_pdl(causal_conv_tail_kernel, dim3(n_entries, (channels + 255) / 256), dim3(256), 0, stream, p);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_ssm_scan(const float* xbc, long long xbc_stride, int x_col, int b_col, int c_col, const float* dt,
                         long long dt_stride, const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                         const int* entry_q_start, const int* entry_q_len, const int* entry_slot, int n_entries,
                         float* out, long long out_stride, int heads, int groups, int vdim, int n_state,
                         cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || vdim < 1 || n_state < 1 || n_state > R * 32 || heads > 65535 * 32)
    return IFX_ERR_UNSUPPORTED;
  int ln = 1;
  while (R * ln < n_state) ln <<= 1;
  int pb = 1024 / ln;
  if (pb > vdim) pb = vdim;
  // blocks of at most 256 threads where the columns allow it: more blocks to spread over the SMs
  while (pb * ln > 256 && pb % 2 == 0 && pb > 8) pb >>= 1;
  const int threads = (pb * ln + 31) / 32 * 32;
  SsmArgs p{xbc, xbc_stride, x_col, b_col, c_col, dt, dt_stride, dt_bias, a_log, d_skip, state, entry_q_start, entry_q_len,
            entry_slot, out, out_stride, heads, groups, vdim, n_state, ln, pb};
  const size_t smem = ((size_t)TC * (2 * R * ln + pb) + 2 * TC) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(ssm_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int rc = launch_pdl(ssm_scan_kernel, dim3(heads, n_entries, (vdim + pb - 1) / pb), dim3(threads), smem, stream, p);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

namespace {
// out[t][g] = N(y[t][g] * silu(z[t][g])) * w[g] over each of `groups` equal parts of a row, N(v) = v / sqrt(mean(v^2) + eps).
// A block a (row, group); the gate comes ahead of the norm.
template <typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, long long y_stride, const float* __restrict__ z, long long z_stride,
                        const float* __restrict__ w, TO* __restrict__ out, long long out_stride, int group_width, float eps) {
  __shared__ float scratch[32];
  pdl_enter();
  const int t = blockIdx.x, c0 = blockIdx.y * group_width;
  const float* yr = y + (size_t)t * y_stride + c0;
  const float* zr = z + (size_t)t * z_stride + c0;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
    const float g = zr[i];
    const float v = yr[i] * (g / (1.0f + expf(-g)));
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)group_width + eps);
  TO* o = out + (size_t)t * out_stride + c0;
  for (int i = threadIdx.x; i < group_width; i += blockDim.x) {
    const float g = zr[i];
    const float v = yr[i] * (g / (1.0f + expf(-g)));
    o[i] = Num<TO>::from_f(v * inv * w[c0 + i]);
  }
}
}  // namespace

// y float32 [n][groups * group_width] (rows y_stride apart), z float32 rows z_stride apart (the gate's sums), w float32
// [groups * group_width]; out rows of either type.  The number of threads depends on the group's width alone.
IFX_API int ifx_gated_group_norm(const float* y, long long y_stride, const float* z, long long z_stride, const float* w,
                                 void* out, int out_dtype, long long out_stride, int n_rows, int groups, int group_width,
                                 float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (groups < 1 || groups > 65535 || group_width < 1) return IFX_ERR_UNSUPPORTED;
  const int threads = group_width >= 256 ? 256 : (group_width + 31) / 32 * 32;
  int rc;
  if (out_dtype == IFX_BF16)
    rc = launch_pdl(gated_group_norm_kernel<bf16>, dim3(n_rows, groups), dim3(threads), 0, stream, y, y_stride, z, z_stride, w,
                    (bf16*)out, out_stride, group_width, eps);
  else if (out_dtype == IFX_F32)
    rc = launch_pdl(gated_group_norm_kernel<float>, dim3(n_rows, groups), dim3(threads), 0, stream, y, y_stride, z, z_stride, w,
                    (float*)out, out_stride, group_width, eps);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}
