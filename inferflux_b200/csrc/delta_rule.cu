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
// fourth group of four key rows of it (R rows in registers, read from shared memory 16 bytes at a time).  A token costs one reduction over the key rows for u^T S, the update, and a
// second reduction for the output; the sums run in four chains so that no addition waits on the one before it.
// Tokens are staged through shared memory a chunk at a time in two buffers: while the block works through one
// chunk, asynchronous copies bring the next chunk's rows.  The decay, the unit key and the removal rate times the unit
// key come, in a step with portions, from a kernel ahead of the scan that computes them for all rows at once (a warp
// a row and head), and the copies are issued by two warps of their own behind the scanning ones: the scan is a chain
// from token to token, so its warps are best left alone on their schedulers.  In a step of single tokens the
// scanning warps compute the three themselves, a warp a token.  The state of a sequence lives in its slot
// as [heads][vdim][dim] float32, read at the start of an entry and written at its end, so a prompt may be cut
// anywhere and a decoded token is the same kernel with one token.
//
// The finish brings every head's output to unit root mean square, multiplies by a weight over all heads and by
// sigmoid(gate), and rounds once into the engine's type.
#include "common.cuh"

namespace {
constexpr int R = 16;           // key rows a thread holds
constexpr int MAX_TC = 16;      // tokens staged at a time at most

struct DeltaArgs {
  const float* proj; long long stride; int r_col, k_col, v_col, a_col;   // float32 rows: r, k, v heads and raw removal rates
  const float* wraw; long long w_stride;                                 // raw decays [row][heads * dim]
  const float* w0; const float* ab;                                      // [heads * dim]
  float* state;                                                          // [slots][heads][vdim][dim]
  const int* entry_q_start; const int* entry_q_len; const int* entry_slot;
  float* out; long long out_stride;                                      // [row][heads * vdim]
  int heads, dim, vdim, cols_per_block, tc, vec;    // vec: every staged row starts 16-byte aligned
  int helpers;                                      // threads behind the scanning ones that only stage (and prepare)
  const float* prep; long long prep_stride;         // [row][unit key | decay | rate times unit key], each heads * dim, or null
  float decay_scale, key_eps;
};

template <int LN>
__global__ void __launch_bounds__(512)
delta_rule_scan_kernel(DeltaArgs p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = R * LN;
  const int PB = p.cols_per_block, TC = p.tc;
  const int BUF = (TC * (5 * NP + PB) + 3) & ~3;   // per buffer (16-byte aligned): r, k, unit key, decay, removal rate [TC][NP] each, v [TC][PB]
  pdl_enter();
  const int h = blockIdx.x, e = blockIdx.y, p0 = blockIdx.z * PB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int pl = tid / LN, ln = tid - pl * LN;
  const int col = p0 + pl;
  const bool valid = pl < PB && col < p.vdim;
  const int r0 = p.entry_q_start[e], len = p.entry_q_len[e];
  const int hd = h * p.dim;
  const int scanning = blockDim.x - p.helpers;
  float* st = p.state + (((size_t)p.entry_slot[e] * p.heads + h) * p.vdim + (valid ? col : 0)) * p.dim;
  float S[R];                              // S[4 j + c] is key row 4 (j LN + ln) + c: a 16-byte load per four rows
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = 4 * ((i >> 2) * LN + ln) + (i & 3);
    S[i] = (valid && n < p.dim) ? st[n] : 0.0f;
  }
  // the raw rows of the tokens from t0 on, asked for; rows past the head's size are zeros
  auto stage = [&](int t0, float* buf, int wtid, int wthreads) {
    const int nt = min(TC, len - t0);
    float* rs = buf; float* ks = rs + TC * NP; float* us = ks + TC * NP; float* ws = us + TC * NP; float* as = ws + TC * NP;
    float* vs = as + TC * NP;
    const int width = p.heads * p.dim;
    if (p.vec) {
      for (int idx = wtid; idx < nt * (NP / 4); idx += wthreads) {
        const int tt = idx / (NP / 4), n = 4 * (idx - tt * (NP / 4)), at = tt * NP + n;
        const size_t row = (size_t)(r0 + t0 + tt);
        if (n < p.dim) {
          const float* pr = p.proj + row * p.stride + hd + n;
          cp_async_f32x4(rs + at, pr + p.r_col);
          cp_async_f32x4(ks + at, pr + p.k_col);
          if (p.prep) {
            const float* pp = p.prep + row * p.prep_stride + hd + n;
            cp_async_f32x4(us + at, pp);
            cp_async_f32x4(ws + at, pp + width);
            cp_async_f32x4(as + at, pp + 2 * width);
          } else {
            cp_async_f32x4(as + at, pr + p.a_col);
            cp_async_f32x4(ws + at, p.wraw + row * p.w_stride + hd + n);
          }
        } else {
          const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          *reinterpret_cast<float4*>(rs + at) = *reinterpret_cast<float4*>(ks + at) = zero;
          *reinterpret_cast<float4*>(as + at) = *reinterpret_cast<float4*>(ws + at) = zero;
          *reinterpret_cast<float4*>(us + at) = zero;
        }
      }
      const int pq = PB >> 2;
      for (int idx = wtid; idx < nt * pq; idx += wthreads) {
        const int tt = idx / pq, c = 4 * (idx - tt * pq);
        if (p0 + c < p.vdim) cp_async_f32x4(vs + tt * PB + c, p.proj + (size_t)(r0 + t0 + tt) * p.stride + p.v_col + h * p.vdim + p0 + c);
        else *reinterpret_cast<float4*>(vs + tt * PB + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    } else {
      for (int idx = wtid; idx < nt * NP; idx += wthreads) {
        const int tt = idx / NP, n = idx - tt * NP;
        const size_t row = (size_t)(r0 + t0 + tt);
        if (n < p.dim) {
          const float* pr = p.proj + row * p.stride + hd + n;
          cp_async_f32(rs + idx, pr + p.r_col);
          cp_async_f32(ks + idx, pr + p.k_col);
          if (p.prep) {
            const float* pp = p.prep + row * p.prep_stride + hd + n;
            cp_async_f32(us + idx, pp);
            cp_async_f32(ws + idx, pp + width);
            cp_async_f32(as + idx, pp + 2 * width);
          } else {
            cp_async_f32(as + idx, pr + p.a_col);
            cp_async_f32(ws + idx, p.wraw + row * p.w_stride + hd + n);
          }
        } else {
          rs[idx] = ks[idx] = us[idx] = as[idx] = ws[idx] = 0.0f;
        }
      }
      for (int idx = wtid; idx < nt * PB; idx += wthreads) {
        const int tt = idx / PB, c = idx - tt * PB;
        if (p0 + c < p.vdim) cp_async_f32(vs + idx, p.proj + (size_t)(r0 + t0 + tt) * p.stride + p.v_col + h * p.vdim + p0 + c);
        else vs[idx] = 0.0f;
      }
    }
    cp_async_commit();
  };
  // once the copies are in: a warp a token, the unit key (a fixed order of additions), the decay, the removal rate
  auto prepare = [&](int nt, float* buf, int wwarp, int wwarps) {
    if (p.prep) return;                                      // a kernel ahead of this one has done it for all rows
    float* ks = buf + TC * NP; float* us = ks + TC * NP; float* ws = us + TC * NP; float* as = ws + TC * NP;
    for (int tt = wwarp; tt < nt; tt += wwarps) {
      float ss = 0.0f;
      for (int n = lane; n < NP; n += 32) ss = fmaf(ks[tt * NP + n], ks[tt * NP + n], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + p.key_eps);
      for (int n = lane; n < NP; n += 32) {
        const int i = tt * NP + n;
        const float u = ks[i] * inv;
        us[i] = u;
        if (n < p.dim) {
          ws[i] = expf(-p.decay_scale / (1.0f + expf(-(ws[i] + p.w0[hd + n]))));
          as[i] = u / (1.0f + expf(-(as[i] + p.ab[hd + n])));
        }
      }
    }
  };
  if (len > 0) {
    stage(0, sm, tid, blockDim.x);
    cp_async_wait_all();
    __syncthreads();
    prepare(min(TC, len), sm, warp, nwarps);
    __syncthreads();
  }
  int which = 0;
  for (int t0 = 0; t0 < len; t0 += TC, which ^= 1) {
    const int nt = min(TC, len - t0);
    const bool more = t0 + TC < len;
    float* cur = sm + which * BUF;
    float* nxt = sm + (which ^ 1) * BUF;          // last read two chunks ago, before the barriers of the last turn
    if (p.helpers) {
      // the threads behind the scanning ones bring and prepare the next chunk meanwhile; all meet at the turn's end
      if (tid >= scanning) {
        if (more) {
          stage(t0 + TC, nxt, tid - scanning, p.helpers);
          cp_async_wait_all();
          if (!p.prep) {
            asm volatile("bar.sync 1, %0;\n" ::"r"(p.helpers) : "memory");
            prepare(min(TC, len - t0 - TC), nxt, warp - (scanning >> 5), p.helpers >> 5);
          }
        }
        __syncthreads();
        continue;
      }
    } else if (more) {
      stage(t0 + TC, nxt, tid, blockDim.x);
    }
    const float* rs = cur; const float* ks = rs + TC * NP; const float* us = ks + TC * NP; const float* ws = us + TC * NP;
    const float* as = ws + TC * NP; const float* vs = as + TC * NP;
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {
      const float4* u4 = reinterpret_cast<const float4*>(us + tt * NP) + ln;
      const float4* w4 = reinterpret_cast<const float4*>(ws + tt * NP) + ln;
      const float4* a4 = reinterpret_cast<const float4*>(as + tt * NP) + ln;
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * NP) + ln;
      const float4* r4 = reinterpret_cast<const float4*>(rs + tt * NP) + ln;
      const float v = pl < PB ? vs[tt * PB + pl] : 0.0f;
      float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 u = u4[j * LN];
        d0 = fmaf(u.x, S[4 * j], d0);
        d1 = fmaf(u.y, S[4 * j + 1], d1);
        d2 = fmaf(u.z, S[4 * j + 2], d2);
        d3 = fmaf(u.w, S[4 * j + 3], d3);
      }
      float dot = (d0 + d1) + (d2 + d3);
      for (int o = LN >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 w = w4[j * LN], k = k4[j * LN], au = a4[j * LN], r = r4[j * LN];
        S[4 * j] = fmaf(w.x, S[4 * j], fmaf(k.x, v, -au.x * dot));
        S[4 * j + 1] = fmaf(w.y, S[4 * j + 1], fmaf(k.y, v, -au.y * dot));
        S[4 * j + 2] = fmaf(w.z, S[4 * j + 2], fmaf(k.z, v, -au.z * dot));
        S[4 * j + 3] = fmaf(w.w, S[4 * j + 3], fmaf(k.w, v, -au.w * dot));
        y0 = fmaf(S[4 * j], r.x, y0);
        y1 = fmaf(S[4 * j + 1], r.y, y1);
        y2 = fmaf(S[4 * j + 2], r.z, y2);
        y3 = fmaf(S[4 * j + 3], r.w, y3);
      }
      float yo = (y0 + y1) + (y2 + y3);
      for (int o = LN >> 1; o > 0; o >>= 1) yo += __shfl_xor_sync(0xffffffffu, yo, o);
      if (valid && ln == 0) p.out[(size_t)(r0 + t0 + tt) * p.out_stride + h * p.vdim + col] = yo;
    }
    if (p.helpers) {
      __syncthreads();
    } else if (more) {
      cp_async_wait_all();
      __syncthreads();
      prepare(min(TC, len - t0 - TC), nxt, warp, nwarps);
      __syncthreads();
    }
  }
  if (valid) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = 4 * ((i >> 2) * LN + ln) + (i & 3);
      if (n < p.dim) st[n] = S[i];
    }
  }
}

// What the scan needs of every (row, head) besides r, k and v, for all rows of a step at once (a warp each): the
// unit key, the decay and the removal rate times the unit key, [row][3][heads * dim].
__global__ void __launch_bounds__(256)
delta_prepare_kernel(DeltaArgs p, float* __restrict__ prep, int n_rows) {
  pdl_enter();
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= n_rows * p.heads) return;
  const int row = idx / p.heads, h = idx - row * p.heads, hd = h * p.dim, width = p.heads * p.dim;
  const float* pr = p.proj + (size_t)row * p.stride + hd;
  const float* wr = p.wraw + (size_t)row * p.w_stride + hd;
  float* dst = prep + (size_t)row * p.prep_stride + hd;
  float ss = 0.0f;
  for (int n = lane; n < p.dim; n += 32) ss = fmaf(pr[p.k_col + n], pr[p.k_col + n], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + p.key_eps);
  for (int n = lane; n < p.dim; n += 32) {
    const float u = pr[p.k_col + n] * inv;
    dst[n] = u;
    dst[width + n] = expf(-p.decay_scale / (1.0f + expf(-(wr[n] + p.w0[hd + n]))));
    dst[2 * width + n] = u / (1.0f + expf(-(pr[p.a_col + n] + p.ab[hd + n])));
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
                                float key_eps, int n_rows, float* prep, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || dim < 1 || dim > R * 32 || vdim < 1 || n_entries > 65535) return IFX_ERR_UNSUPPORTED;
  int ln = 1;
  while (R * ln < dim) ln <<= 1;
  int pb = 256 / ln;                      // blocks of at most 256 threads: more blocks to spread over the SMs
  if (pb > vdim) pb = vdim;
  // small blocks where the heads alone do not fill the SMs; a step with portions gets two more warps a block that
  // stage and prepare the chunk after the one being scanned
  int helpers = n_rows <= n_entries ? 0 : 64;
  if (pb > 16 && heads * n_entries * ((vdim + pb - 1) / pb) < 148) pb = 16;
  const int threads = (pb * ln + 31) / 32 * 32 + helpers;
  int tc = n_rows <= n_entries ? 1 : MAX_TC;
  while (tc > 1 && (size_t)2 * (tc * (5 * R * ln + pb) + 3) * sizeof(float) > 96 * 1024) tc >>= 1;
  const int vec = !((dim | vdim | pb | r_col | k_col | v_col | a_col) & 3) && !((stride | w_stride) & 3) &&
                  !(((uintptr_t)proj | (uintptr_t)wraw) & 15);
  DeltaArgs p{proj, stride, r_col, k_col, v_col, a_col, wraw, w_stride, w0, ab, state, entry_q_start, entry_q_len, entry_slot,
              out, out_stride, heads, dim, vdim, pb, tc, vec, helpers, nullptr, 0, decay_scale, key_eps};
  if (prep && tc > 1) {
    p.prep = prep;
    p.prep_stride = 3LL * heads * dim;
    if ((uintptr_t)prep & 15) p.vec = 0;
    const long long warps = (long long)n_rows * heads;
    const int prc = launch_pdl(delta_prepare_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, p, prep, n_rows);
    if (prc) return prc;
  }
  const size_t smem = (size_t)2 * (tc * (5 * R * ln + pb) + 3) * sizeof(float);
  const dim3 grid(heads, n_entries, (vdim + pb - 1) / pb), block(threads);
  int rc = IFX_ERR_UNSUPPORTED;
#define IFX_DELTA_CASE(L)                                                                                           \
  case L: {                                                                                                         \
    if (smem > 48 * 1024) {                                                                                         \
      cudaError_t err = cudaFuncSetAttribute(delta_rule_scan_kernel<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (err != cudaSuccess) return (int)err;                                                                      \
    }                                                                                                               \
    rc = launch_pdl(delta_rule_scan_kernel<L>, grid, block, smem, stream, p);                                       \
  } break;
  switch (ln) { IFX_DELTA_CASE(1) IFX_DELTA_CASE(2) IFX_DELTA_CASE(4) IFX_DELTA_CASE(8) IFX_DELTA_CASE(16) IFX_DELTA_CASE(32) }
#undef IFX_DELTA_CASE
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
