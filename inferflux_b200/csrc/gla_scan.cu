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
// The recurrence is linear in S, so a long portion is cut into segments of 64 tokens that run side by side: (1) every
// segment's own end state from zero and the product of its decays, (2) per request and head the segments' starting
// states one after the other, S_start(s + 1) = A_s S_start(s) + L_s (the last goes to the slot), (3) every segment
// again from its true starting state, now writing o.  Steps whose entries all fit one segment (all steps of single
// tokens) run the plain walk from the slot alone.
//
// A block takes one (head, entry or segment, 32 value columns) and walks its tokens in order.  A thread holds, of one
// value column, the state rows 4 (g + 4 i) .. + 3 for its row group g in 0..3 (NI groups of four rows, in
// registers); the four threads of a column add their parts of o_t by shuffles.  Tokens are staged 16 (8 for the widest heads) at a time in
// shared memory (q, k, the decays worked out on the way in, and the block's 32 value columns), rows padded with zeros
// to a multiple of 16, so that the inner loop is 16-byte shared loads and fused multiply-adds alone.
#include "common.cuh"

namespace {
constexpr int GLA_COLS = 32;       // value columns a block

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

constexpr int GLA_SEGMENT = 64;    // tokens a segment
// What a launch does.  WALK: an entry's tokens from the slot's state back into the slot, writing o.  LOCAL: a segment
// from zero, leaving its end state and the product of its decays.  FINISH: a segment from its starting state, writing o.
constexpr int GLA_WALK = 0, GLA_LOCAL = 1, GLA_FINISH = 2;

struct GlaSegments {
  const int* seg_entry;       // [n_segments] the entry of each segment
  const int* seg_t0;          // [n_segments] its first token within the entry
  float* seg_state;           // [n_segments, heads, dim, vdim] LOCAL: end state from zero; after the carry: starting state
  float* seg_decay;           // [n_segments, heads, dim] product of the segment's decays
};

template <int NI, int MODE>
__global__ void __launch_bounds__(128)
gla_scan_kernel(const float* __restrict__ proj, long long proj_stride, int q_col, int k_col, int v_col,
                const float* __restrict__ z, long long z_stride, const float* __restrict__ z_bias, float inv_tau,
                float q_scale, float* __restrict__ state, const int* __restrict__ entry_q_start,
                const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot, float* __restrict__ out,
                long long out_stride, int heads, int dim, int vdim, GlaSegments sg) {
  pdl_enter();
  constexpr int DP = 16 * NI;                              // rows, padded
  constexpr int GLA_TOKENS = NI > 12 ? 8 : 16;             // tokens staged at a time (what 48 KB of shared memory hold)
  __shared__ __align__(16) float qs[GLA_TOKENS][DP], ks[GLA_TOKENS][DP], as[GLA_TOKENS][DP];
  __shared__ float vs[GLA_TOKENS][GLA_COLS];
  const int head = blockIdx.x, c0 = blockIdx.z * GLA_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane & 3;
  const int col = c0 + warp * 8 + (lane >> 2);
  const bool col_ok = col < vdim;
  int e = blockIdx.y, n, t0;
  float* sp;                                               // where the state comes from (and, WALK, goes back to)
  if (MODE == GLA_WALK) {
    n = entry_q_len[e];
    t0 = entry_q_start[e];
    sp = state + ((size_t)entry_slot[e] * heads + head) * dim * vdim;
  } else {
    const int seg = blockIdx.y;
    e = sg.seg_entry[seg];
    n = min(GLA_SEGMENT, entry_q_len[e] - sg.seg_t0[seg]);
    t0 = entry_q_start[e] + sg.seg_t0[seg];
    sp = sg.seg_state + ((size_t)seg * heads + head) * dim * vdim;
  }
  float s[NI][4], ap[MODE == GLA_LOCAL ? NI : 1][4];
#pragma unroll
  for (int i = 0; i < NI; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = 4 * (g + 4 * i) + j;
      s[i][j] = (MODE != GLA_LOCAL && col_ok && r < dim) ? sp[(size_t)r * vdim + col] : 0.0f;
      if (MODE == GLA_LOCAL) ap[i][j] = 1.0f;
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
        if (MODE == GLA_LOCAL) {
          ap[i][0] *= a4.x; ap[i][1] *= a4.y; ap[i][2] *= a4.z; ap[i][3] *= a4.w;
        } else {
          acc0 = fmaf(s[i][0], q4.x, fmaf(s[i][1], q4.y, acc0));
          acc1 = fmaf(s[i][2], q4.z, fmaf(s[i][3], q4.w, acc1));
        }
      }
      if (MODE != GLA_LOCAL) {
        float acc = acc0 + acc1;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (g == 0 && col_ok) out[(size_t)(t0 + base + t) * out_stride + (size_t)head * vdim + col] = acc;
      }
    }
  }
  if (MODE == GLA_FINISH) return;                          // the carry has already sent the entry's last state to the slot
  if (MODE == GLA_LOCAL && blockIdx.z == 0 && warp == 0 && (lane >> 2) == 0) {     // one column's threads hold every row's product
    float* dp = sg.seg_decay + ((size_t)blockIdx.y * heads + head) * dim;
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = 4 * (g + 4 * i) + j;
        if (r < dim) dp[r] = ap[i][j];
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

// The segments' starting states, one after the other: a thread an element of the state of one (entry, head).  The
// buffer holds a segment's end state from zero on the way in and its starting state on the way out; the state
// behind the entry's last segment goes to the slot.
__global__ void gla_carry_kernel(GlaSegments sg, const int* __restrict__ entry_first_seg, const int* __restrict__ entry_q_len,
                                 const int* __restrict__ entry_slot, float* __restrict__ state, int heads, int dim, int vdim) {
  pdl_enter();
  const int head = blockIdx.x, e = blockIdx.y;
  const int idx = blockIdx.z * blockDim.x + threadIdx.x;
  if (idx >= dim * vdim) return;
  const int row = idx / vdim;
  const int first = entry_first_seg[e], count = (entry_q_len[e] + GLA_SEGMENT - 1) / GLA_SEGMENT;
  float* sp = state + ((size_t)entry_slot[e] * heads + head) * dim * vdim + idx;
  float cur = *sp;
  for (int s0 = 0; s0 < count; s0 += 4) {                  // four segments' sums and decays asked for together
    float local[4], decay[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int seg = first + s0 + u;
      local[u] = s0 + u < count ? sg.seg_state[((size_t)seg * heads + head) * dim * vdim + idx] : 0.0f;
      decay[u] = s0 + u < count ? sg.seg_decay[((size_t)seg * heads + head) * dim + row] : 1.0f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (s0 + u >= count) break;
      sg.seg_state[((size_t)(first + s0 + u) * heads + head) * dim * vdim + idx] = cur;
      cur = fmaf(decay[u], cur, local[u]);
    }
  }
  *sp = cur;
}

template <int NI>
int launch_gla(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, const float* z, long long z_stride,
               const float* z_bias, float inv_tau, float q_scale, float* state, const int* entry_q_start,
               const int* entry_q_len, const int* entry_slot, int n_entries, float* out, long long out_stride, int heads,
               int dim, int vdim, GlaSegments sg, int n_segments, const int* entry_first_seg, cudaStream_t stream) {
  const int vblocks = (vdim + GLA_COLS - 1) / GLA_COLS;
  int rc;
#define IFX_GLA_RUN(MODE, count)                                                                                          \
  launch_pdl(gla_scan_kernel<NI, MODE>, dim3(heads, count, vblocks), dim3(128), 0, stream, proj, proj_stride, q_col, k_col, \
             v_col, z, z_stride, z_bias, inv_tau, q_scale, state, entry_q_start, entry_q_len, entry_slot, out, out_stride,  \
             heads, dim, vdim, sg)
  if (n_segments <= 0) {
    rc = IFX_GLA_RUN(GLA_WALK, n_entries);
    return rc ? rc : IFX_LAUNCH_CHECK();
  }
  if ((rc = IFX_GLA_RUN(GLA_LOCAL, n_segments))) return rc;
  if ((rc = launch_pdl(gla_carry_kernel, dim3(heads, n_entries, (dim * vdim + 255) / 256), dim3(256), 0, stream, sg, entry_first_seg,
                       entry_q_len, entry_slot, state, heads, dim, vdim))) return rc;
  rc = IFX_GLA_RUN(GLA_FINISH, n_segments);
#undef IFX_GLA_RUN
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// proj float32 rows hold q and k (heads * dim each) and v (heads * vdim) from the given columns; z float32 rows
// [N, heads * dim]; z_bias float32 [heads * dim]; state float32 [slots, heads, dim, vdim]; out float32 rows
// [N, heads * vdim].  dim up to 256.  n_segments > 0: the step is cut into that many segments of
// ifx_gla_segment() tokens (seg_entry, seg_t0: each one's entry and first token within it; entry_first_seg: each
// entry's first segment; seg_state float32 [n_segments, heads, dim, vdim] and seg_decay [n_segments, heads, dim] are
// scratch) that run side by side; 0: every entry is walked from its slot by one block per head and 32 value columns.
IFX_API int ifx_gla_segment() { return GLA_SEGMENT; }

IFX_API int ifx_gla_scan(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, const float* z,
                         long long z_stride, const float* z_bias, float inv_tau, float q_scale, float* state,
                         const int* entry_q_start, const int* entry_q_len, const int* entry_slot, int n_entries, float* out,
                         long long out_stride, int heads, int dim, int vdim, const int* seg_entry, const int* seg_t0,
                         const int* entry_first_seg, int n_segments, float* seg_state, float* seg_decay,
                         cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (heads < 1 || heads > 65535 || dim < 1 || dim > 256 || vdim < 1 || n_entries > 65535 || n_segments > 65535) return IFX_ERR_UNSUPPORTED;
  if (n_segments > 0 && (!seg_entry || !seg_t0 || !entry_first_seg || !seg_state || !seg_decay)) return IFX_ERR_UNSUPPORTED;
  GlaSegments sg{seg_entry, seg_t0, seg_state, seg_decay};
  const int ni = (dim + 15) / 16;
#define IFX_GLA(NI) return launch_gla<NI>(proj, proj_stride, q_col, k_col, v_col, z, z_stride, z_bias, inv_tau, q_scale, state, \
                                          entry_q_start, entry_q_len, entry_slot, n_entries, out, out_stride, heads, dim, vdim, \
                                          sg, n_segments, entry_first_seg, stream)
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
