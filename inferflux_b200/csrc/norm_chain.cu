// A chain of root-mean-square norms around the residual sum, one block a row, everything float32:
//
//   ya = sum of a's slices                       (a mixer's or feed-forward's float32 sums)
//   if wa:  ya = N(ya) * wa                      N(v) = v / sqrt(mean(v^2) + eps) over the row
//   if b:   yb likewise with wb;  y = (ya + yb) / 2     (two branches side by side)      else y = ya
//   if w_post:  y = N(y) * w_post                (a norm behind the sublayer)
//   r = residual + y;   residual = r             (unless `rows` picks rows: then the residual stays)
//   if out:  out = N(r) * w_next                 (the norm ahead of the next sublayer, engine type)
//            or, without w_next, out = r          (a sublayer that reads the stream itself: its rounding alone)
//
// Blocks that sandwich every sublayer between two norms, and mixers whose result is the mean of two normed
// branches, run all of their row-wise arithmetic here in one pass over the row.  The number of threads
// depends on the row length alone and every sum is added in a fixed order, so a row's result does not
// depend on what else is in the batch.
#include "common.cuh"

namespace {
struct ChainArgs {
  const float* a; int a_parts; long long a_stride; const float* wa;
  const float* b; int b_parts; long long b_stride; const float* wb;
  const float* w_post;
  float* residual;
  const float* w_next;
  void* out;
  const int* rows;
  int hidden;
  float eps;
};

template <typename TO>
__global__ void __launch_bounds__(1024)
norm_chain_kernel(ChainArgs p) {
  extern __shared__ float row[];                  // [hidden]: y
  __shared__ float scratch[32];
  pdl_enter();
  const int H = p.hidden;
  const int out_row = blockIdx.x;
  const int r = p.rows ? p.rows[out_row] : out_row;
  const float inv_h = 1.0f / (float)H;
  // branch a
  float ss = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = 0.0f;
    if (p.a) for (int s = 0; s < p.a_parts; ++s) v += p.a[(size_t)s * p.a_stride + (size_t)r * H + i];
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (p.wa) {
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) * inv_h + p.eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = row[i] * inv * p.wa[i];
  }
  if (p.b) {
    float sb = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = 0.0f;
      for (int s = 0; s < p.b_parts; ++s) v += p.b[(size_t)s * p.b_stride + (size_t)r * H + i];
      sb = fmaf(v, v, sb);
    }
    const float inv = p.wb ? 1.0f / sqrtf(block_sum(sb, scratch) * inv_h + p.eps) : 1.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = 0.0f;
      for (int s = 0; s < p.b_parts; ++s) v += p.b[(size_t)s * p.b_stride + (size_t)r * H + i];
      v = p.wb ? v * inv * p.wb[i] : v;
      row[i] = 0.5f * (row[i] + v);
    }
  }
  if (p.w_post) {
    float sy = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) sy = fmaf(row[i], row[i], sy);
    const float inv = 1.0f / sqrtf(block_sum(sy, scratch) * inv_h + p.eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = row[i] * inv * p.w_post[i];
  }
  float sr = 0.0f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = p.residual[(size_t)r * H + i] + row[i];
    if (!p.rows) p.residual[(size_t)r * H + i] = v;
    row[i] = v;
    sr = fmaf(v, v, sr);
  }
  if (p.out && p.w_next) {
    const float inv = 1.0f / sqrtf(block_sum(sr, scratch) * inv_h + p.eps);
    TO* o = (TO*)p.out + (size_t)out_row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = Num<TO>::from_f(row[i] * inv * p.w_next[i]);
  } else if (p.out) {
    TO* o = (TO*)p.out + (size_t)out_row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = Num<TO>::from_f(row[i]);
  }
}
// The same with the row in registers: row lengths that are multiples of 4 up to 4 x 4 x 1,024, a thread holding up
// to four groups of 4 neighbouring elements, every access 16 bytes wide, each input read once.
__device__ __forceinline__ float4 sum_slices4(const float* base, int parts, long long stride, size_t at) {
  float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < parts; ++s) {
    const float4 u = *reinterpret_cast<const float4*>(base + (size_t)s * stride + at);
    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
  }
  return v;
}
__device__ __forceinline__ float sq4(float4 v) { return fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))); }
__device__ __forceinline__ float4 scale4(float4 v, float f, const float* w) {
  const float4 u = *reinterpret_cast<const float4*>(w);
  return make_float4(v.x * f * u.x, v.y * f * u.y, v.z * f * u.z, v.w * f * u.w);
}

template <typename TO, int G>
__global__ void __launch_bounds__(1024)
norm_chain_vec_kernel(ChainArgs p) {
  __shared__ float scratch[32];
  pdl_enter();
  const int H = p.hidden;
  const int out_row = blockIdx.x;
  const int r = p.rows ? p.rows[out_row] : out_row;
  const float inv_h = 1.0f / (float)H;
  float4 y[G];
  bool on[G];
  float ss = 0.0f;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int i = 4 * (threadIdx.x + g * blockDim.x);
    on[g] = i < H;
    y[g] = on[g] && p.a ? sum_slices4(p.a, p.a_parts, p.a_stride, (size_t)r * H + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    ss += sq4(y[g]);
  }
  if (p.wa) {
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) * inv_h + p.eps);
#pragma unroll
    for (int g = 0; g < G; ++g) if (on[g]) y[g] = scale4(y[g], inv, p.wa + 4 * (threadIdx.x + g * blockDim.x));
  }
  if (p.b) {
    float4 z[G];
    float sb = 0.0f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      z[g] = on[g] ? sum_slices4(p.b, p.b_parts, p.b_stride, (size_t)r * H + 4 * (threadIdx.x + g * blockDim.x))
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      sb += sq4(z[g]);
    }
    const float inv = p.wb ? 1.0f / sqrtf(block_sum(sb, scratch) * inv_h + p.eps) : 1.0f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!on[g]) continue;
      if (p.wb) z[g] = scale4(z[g], inv, p.wb + 4 * (threadIdx.x + g * blockDim.x));
      y[g] = make_float4(0.5f * (y[g].x + z[g].x), 0.5f * (y[g].y + z[g].y), 0.5f * (y[g].z + z[g].z), 0.5f * (y[g].w + z[g].w));
    }
  }
  if (p.w_post) {
    float sy = 0.0f;
#pragma unroll
    for (int g = 0; g < G; ++g) sy += sq4(y[g]);
    const float inv = 1.0f / sqrtf(block_sum(sy, scratch) * inv_h + p.eps);
#pragma unroll
    for (int g = 0; g < G; ++g) if (on[g]) y[g] = scale4(y[g], inv, p.w_post + 4 * (threadIdx.x + g * blockDim.x));
  }
  float sr = 0.0f;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (!on[g]) continue;
    float* rp = p.residual + (size_t)r * H + 4 * (threadIdx.x + g * blockDim.x);
    const float4 u = *reinterpret_cast<const float4*>(rp);
    y[g] = make_float4(u.x + y[g].x, u.y + y[g].y, u.z + y[g].z, u.w + y[g].w);
    if (!p.rows) *reinterpret_cast<float4*>(rp) = y[g];
    sr += sq4(y[g]);
  }
  if (p.out) {
    const float inv = p.w_next ? 1.0f / sqrtf(block_sum(sr, scratch) * inv_h + p.eps) : 1.0f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (!on[g]) continue;
      const int i = 4 * (threadIdx.x + g * blockDim.x);
      const float4 v = p.w_next ? scale4(y[g], inv, p.w_next + i) : y[g];
      TO* o = (TO*)p.out + (size_t)out_row * H + i;
      o[0] = Num<TO>::from_f(v.x); o[1] = Num<TO>::from_f(v.y); o[2] = Num<TO>::from_f(v.z); o[3] = Num<TO>::from_f(v.w);
    }
  }
}

template <typename TO>
int launch_chain_vec(const ChainArgs& p, int n_rows, cudaStream_t stream) {
  const int quads = p.hidden / 4;
  int threads = quads < 64 ? 64 : (quads > 1024 ? 1024 : (quads + 31) / 32 * 32);       // by the row length alone
  const int groups = (quads + threads - 1) / threads;
  if (groups <= 1) return launch_pdl(norm_chain_vec_kernel<TO, 1>, dim3(n_rows), dim3(threads), 0, stream, p);
  if (groups <= 2) return launch_pdl(norm_chain_vec_kernel<TO, 2>, dim3(n_rows), dim3(threads), 0, stream, p);
  return launch_pdl(norm_chain_vec_kernel<TO, 4>, dim3(n_rows), dim3(threads), 0, stream, p);
}
}  // namespace

IFX_API int ifx_norm_chain(const float* a, int a_parts, long long a_stride, const float* wa,
                           const float* b, int b_parts, long long b_stride, const float* wb,
                           const float* w_post, float* residual, const float* w_next, void* out, int out_dtype,
                           const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden < 1 || hidden > 49152) return IFX_ERR_UNSUPPORTED;
  ChainArgs p{a, a_parts, a_stride, wa, b, b_parts, b_stride, wb, w_post, residual, w_next, out, rows, hidden, eps};
  const uintptr_t ptrs = (uintptr_t)a | (uintptr_t)wa | (uintptr_t)b | (uintptr_t)wb | (uintptr_t)w_post | (uintptr_t)residual |
                         (uintptr_t)w_next;
  if (!(hidden & 3) && hidden <= 16384 && !(ptrs & 15) && !(a_stride & 3) && !(b_stride & 3)) {
    const int rc = out_dtype == IFX_BF16 ? launch_chain_vec<bf16>(p, n_rows, stream) : launch_chain_vec<float>(p, n_rows, stream);
    return rc ? rc : IFX_LAUNCH_CHECK();
  }
  int threads = (hidden + 3) / 4;                 // by the row length alone
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : (threads + 31) / 32 * 32);
  const size_t smem = (size_t)hidden * sizeof(float);
  auto kern = out_dtype == IFX_BF16 ? norm_chain_kernel<bf16> : norm_chain_kernel<float>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, p);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
