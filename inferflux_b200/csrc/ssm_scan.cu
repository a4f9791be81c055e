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
// LN-th group of four state rows of it (R rows in registers, read from shared memory 16 bytes at a time), so a token costs R multiply-adds for the state, R for the result
// and log2(LN) shuffles.  Tokens are staged through shared memory a chunk at a time in two buffers: asynchronous
// copies bring the next chunk's rows while the block works through the present one.  The state of a sequence lives in
// its slot as [heads][vdim][state] float32, is read at the start of the entry and written at its end, so a
// prompt may be cut anywhere and a decoded token is the same kernel with one token.
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 16;
constexpr int R = 16;           // state rows a thread holds
constexpr int MAX_TC = 16;      // tokens staged at a time at most

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
  int heads, groups, vdim, n_state, cols_per_block, tc, vec;   // vec: every staged row starts 16-byte aligned
};

template <int LN>
__global__ void __launch_bounds__(512)
ssm_scan_kernel(SsmArgs p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = R * LN;
  const int PB = p.cols_per_block, TC = p.tc;
  const int BUF = (TC * (2 * NP + PB + 2) + 3) & ~3;   // per buffer (16-byte aligned): B, C [TC][NP], x [TC][PB], dt and the decay [TC]
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
  float S[R];                              // S[4 j + c] is state row 4 (j LN + ln) + c: a 16-byte load per four rows
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = 4 * ((i >> 2) * LN + ln) + (i & 3);
    S[i] = (valid && n < p.n_state) ? st[n] : 0.0f;
  }
  // the rows of the tokens from t0 on, asked for (asynchronous copies); rows past the state's size are zeros
  auto stage = [&](int t0, float* buf) {
    const int nt = min(TC, len - t0);
    float* Bs = buf; float* Cs = Bs + TC * NP; float* xs = Cs + TC * NP; float* dts = xs + TC * PB;
    if (p.vec) {
      for (int idx = tid; idx < nt * (NP / 4); idx += blockDim.x) {
        const int tt = idx / (NP / 4), n = 4 * (idx - tt * (NP / 4));
        const float* row = p.xbc + (size_t)(r0 + t0 + tt) * p.xbc_stride + g * p.n_state + n;
        if (n < p.n_state) {
          cp_async_f32x4(Bs + tt * NP + n, row + p.b_col);
          cp_async_f32x4(Cs + tt * NP + n, row + p.c_col);
        } else {
          *reinterpret_cast<float4*>(Bs + tt * NP + n) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          *reinterpret_cast<float4*>(Cs + tt * NP + n) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
      }
      const int pq = PB >> 2;
      for (int idx = tid; idx < nt * pq; idx += blockDim.x) {
        const int tt = idx / pq, c = 4 * (idx - tt * pq);
        if (p0 + c < p.vdim) cp_async_f32x4(xs + tt * PB + c, p.xbc + (size_t)(r0 + t0 + tt) * p.xbc_stride + p.x_col + h * p.vdim + p0 + c);
        else *reinterpret_cast<float4*>(xs + tt * PB + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    } else {
      for (int idx = tid; idx < nt * NP; idx += blockDim.x) {
        const int tt = idx / NP, n = idx - tt * NP;
        const float* row = p.xbc + (size_t)(r0 + t0 + tt) * p.xbc_stride + g * p.n_state + n;
        if (n < p.n_state) {
          cp_async_f32(Bs + idx, row + p.b_col);
          cp_async_f32(Cs + idx, row + p.c_col);
        } else {
          Bs[idx] = Cs[idx] = 0.0f;
        }
      }
      for (int idx = tid; idx < nt * PB; idx += blockDim.x) {
        const int tt = idx / PB, c = idx - tt * PB;
        if (p0 + c < p.vdim) cp_async_f32(xs + idx, p.xbc + (size_t)(r0 + t0 + tt) * p.xbc_stride + p.x_col + h * p.vdim + p0 + c);
        else xs[idx] = 0.0f;
      }
    }
    for (int tt = tid; tt < nt; tt += blockDim.x) cp_async_f32(dts + tt, p.dt + (size_t)(r0 + t0 + tt) * p.dt_stride + h);
    cp_async_commit();
  };
  // once the copies are in: the step size and the decay of every staged token
  auto prepare = [&](int nt, float* buf) {
    float* dts = buf + TC * (2 * NP + PB); float* decs = dts + TC;
    for (int tt = tid; tt < nt; tt += blockDim.x) {
      const float raw = dts[tt] + bias;
      const float dtv = raw > 20.0f ? raw : log1pf(expf(raw));
      dts[tt] = dtv;
      decs[tt] = expf(neg_a * dtv);
    }
  };
  if (len > 0) {
    stage(0, sm);
    cp_async_wait_all();
    __syncthreads();
    prepare(min(TC, len), sm);
    __syncthreads();
  }
  int which = 0;
  for (int t0 = 0; t0 < len; t0 += TC, which ^= 1) {
    const int nt = min(TC, len - t0);
    const bool more = t0 + TC < len;
    float* cur = sm + which * BUF;
    float* nxt = sm + (which ^ 1) * BUF;          // last read two chunks ago, before the barriers of the last turn
    if (more) stage(t0 + TC, nxt);
    const float* Bs = cur; const float* Cs = Bs + TC * NP; const float* xs = Cs + TC * NP; const float* dts = xs + TC * PB;
    const float* decs = dts + TC;
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float dtv = dts[tt], dec = decs[tt];
      const float xv = pl < PB ? xs[tt * PB + pl] : 0.0f;
      const float bx = dtv * xv;
      const float4* b4 = reinterpret_cast<const float4*>(Bs + tt * NP) + ln;
      const float4* c4 = reinterpret_cast<const float4*>(Cs + tt * NP) + ln;
      float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;      // four chains: no addition waits on the one before it
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 b = b4[j * LN], c = c4[j * LN];
        S[4 * j] = fmaf(dec, S[4 * j], bx * b.x);
        S[4 * j + 1] = fmaf(dec, S[4 * j + 1], bx * b.y);
        S[4 * j + 2] = fmaf(dec, S[4 * j + 2], bx * b.z);
        S[4 * j + 3] = fmaf(dec, S[4 * j + 3], bx * b.w);
        y0 = fmaf(S[4 * j], c.x, y0);
        y1 = fmaf(S[4 * j + 1], c.y, y1);
        y2 = fmaf(S[4 * j + 2], c.z, y2);
        y3 = fmaf(S[4 * j + 3], c.w, y3);
      }
      float yo = (y0 + y1) + (y2 + y3);
      for (int o = LN >> 1; o > 0; o >>= 1) yo += __shfl_xor_sync(0xffffffffu, yo, o);
      if (valid && ln == 0) p.out[(size_t)(r0 + t0 + tt) * p.out_stride + h * p.vdim + col] = fmaf(dskip, xv, yo);
    }
    if (more) {
      cp_async_wait_all();
      __syncthreads();
      prepare(min(TC, len - t0 - TC), nxt);
      __syncthreads();
    }
  }
  if (valid) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = 4 * ((i >> 2) * LN + ln) + (i & 3);
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
                         int n_rows, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || vdim < 1 || n_state < 1 || n_state > R * 32 || heads > 65535 * 32)
    return IFX_ERR_UNSUPPORTED;
  int ln = 1;
  while (R * ln < n_state) ln <<= 1;
  int pb = 512 / ln;
  if (pb > vdim) pb = vdim;
  // blocks of at most 256 threads where the columns allow it: more blocks to spread over the SMs
  while (pb * ln > 256 && pb % 2 == 0 && pb > 8) pb >>= 1;
  const int threads = (pb * ln + 31) / 32 * 32;
  int tc = n_rows <= n_entries ? 1 : MAX_TC;      // single tokens stage one
  while (tc > 1 && (size_t)2 * (tc * (2 * R * ln + pb + 2) + 3) * sizeof(float) > 96 * 1024) tc >>= 1;
  const int vec = !((n_state | vdim | pb | x_col | b_col | c_col) & 3) && !(xbc_stride & 3) && !((uintptr_t)xbc & 15);
  SsmArgs p{xbc, xbc_stride, x_col, b_col, c_col, dt, dt_stride, dt_bias, a_log, d_skip, state, entry_q_start, entry_q_len,
            entry_slot, out, out_stride, heads, groups, vdim, n_state, pb, tc, vec};
  const size_t smem = (size_t)2 * (tc * (2 * R * ln + pb + 2) + 3) * sizeof(float);
  const dim3 grid(heads, n_entries, (vdim + pb - 1) / pb), block(threads);
  int rc = IFX_ERR_UNSUPPORTED;
#define IFX_SSM_CASE(L)                                                                                             \
  case L: {                                                                                                         \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t err = cudaFuncSetAttribute(ssm_scan_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (err != cudaSuccess) return (int)err;                                                                      \
    }                                                                                                               \
    rc = launch_pdl(ssm_scan_kernel<L>, grid, block, smem, stream, p);                                              \
  } break;
  switch (ln) { IFX_SSM_CASE(1) IFX_SSM_CASE(2) IFX_SSM_CASE(4) IFX_SSM_CASE(8) IFX_SSM_CASE(16) IFX_SSM_CASE(32) }
#undef IFX_SSM_CASE
  return rc ? rc : IFX_LAUNCH_CHECK();
}

namespace {
// out[t][g] = N(y[t][g] * silu(z[t][g])) * w[g] over each of `groups` equal parts of a row, N(v) = v / sqrt(mean(v^2) + eps).
// A block a (row, group); the gate comes ahead of the norm.  A thread keeps its first eight gated values between
// the sum of squares and the result, so that their loads are asked for together and nothing is computed twice.
template <typename TO>
__global__ void __launch_bounds__(1024)
gated_group_norm_kernel(const float* __restrict__ y, long long y_stride, const float* __restrict__ z, long long z_stride,
                        const float* __restrict__ w, TO* __restrict__ out, long long out_stride, int group_width, float eps) {
  __shared__ float scratch[32];
  constexpr int KEEP = 8;
  pdl_enter();
  const int t = blockIdx.x, c0 = blockIdx.y * group_width;
  const float* yr = y + (size_t)t * y_stride + c0;
  const float* zr = z + (size_t)t * z_stride + c0;
  float keep[KEEP];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    const float g = i < group_width ? zr[i] : 0.0f;
    const float v = i < group_width ? yr[i] * (g / (1.0f + expf(-g))) : 0.0f;
    keep[j] = v;
    ss = fmaf(v, v, ss);
  }
  for (int i = threadIdx.x + KEEP * blockDim.x; i < group_width; i += blockDim.x) {
    const float g = zr[i];
    const float v = yr[i] * (g / (1.0f + expf(-g)));
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)group_width + eps);
  TO* o = out + (size_t)t * out_stride + c0;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < group_width) o[i] = Num<TO>::from_f(keep[j] * inv * w[c0 + i]);
  }
  for (int i = threadIdx.x + KEEP * blockDim.x; i < group_width; i += blockDim.x) {
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
  const int threads = group_width >= 4096 ? 1024 : group_width >= 1024 ? 512 : group_width >= 256 ? 256 : (group_width + 31) / 32 * 32;
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
