// RMS norm over equal consecutive parts of a row, fused with the sum into the float32 stream:
//
//   r = residual + sa * (a_0 + a_1 + ...) + sb * (b_0 + b_1 + ...)        (either addend may be absent)
//   out[i] = r[i] / sqrt(mean(r[part of i]^2) + eps) * weight[i]
//
// The row is cut into `groups` parts of hidden / groups elements; every part is divided by its own root mean
// square.  groups = 1 is the plain RMS norm.  The two addends, each given as float32 or bfloat16 slices whose sum
// it is and each with a factor of its own, are what a layer with two mixers side by side hands on
// (sa * left + sb * right): the weighted sum, the sum into the stream and the norm are one pass.
//
// One block per output row; the row lies in shared memory between the passes.  A part's squares are added by one
// warp, lane by lane and then over the warp, so the order of additions depends on the part's length alone, never on
// what else is in the batch.  Source row = rows ? rows[blockIdx.x] : blockIdx.x; in that gather mode the stream is
// left untouched.
#include "common.cuh"

namespace {
template <typename TD>
__device__ __forceinline__ float slices_sum(const TD* d, int parts, long long stride) {
  float v = 0.0f;
  for (int p = 0; p < parts; ++p) v += Num<TD>::to_f(d[(size_t)p * stride]);
  return v;
}

template <typename T> struct GnOut4;
template <> struct GnOut4<float> {
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct GnOut4<bf16> {
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename TD, typename TO, bool VEC>
__global__ void add_group_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ a, int a_parts,
                                         long long a_stride, float a_scale, const TD* __restrict__ b, int b_parts,
                                         long long b_stride, float b_scale, const float* __restrict__ weight, float eps,
                                         int groups, TO* __restrict__ out, const int* __restrict__ rows, int hidden,
                                         int write_residual) {
  pdl_enter();
  extern __shared__ __align__(16) float gn_smem[];
  float* row_buf = gn_smem;                 // [hidden]
  float* rstd = gn_smem + hidden;           // [groups]
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (VEC) {                                // hidden a multiple of 4, float32 addends, everything on 16-byte boundaries
    const float* ar = a ? reinterpret_cast<const float*>(a) + (size_t)src * hidden : nullptr;
    const float* br = b ? reinterpret_cast<const float*>(b) + (size_t)src * hidden : nullptr;
    for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
      float4 v = *reinterpret_cast<const float4*>(r + i);
      if (a || b) {
        float4 sa = make_float4(0.f, 0.f, 0.f, 0.f), sb = sa;
        for (int p = 0; ar && p < a_parts; ++p) {
          const float4 t = *reinterpret_cast<const float4*>(ar + (size_t)p * a_stride + i);
          sa.x += t.x; sa.y += t.y; sa.z += t.z; sa.w += t.w;
        }
        for (int p = 0; br && p < b_parts; ++p) {
          const float4 t = *reinterpret_cast<const float4*>(br + (size_t)p * b_stride + i);
          sb.x += t.x; sb.y += t.y; sb.z += t.z; sb.w += t.w;
        }
        v.x += fmaf(b_scale, sb.x, a_scale * sa.x); v.y += fmaf(b_scale, sb.y, a_scale * sa.y);
        v.z += fmaf(b_scale, sb.z, a_scale * sa.z); v.w += fmaf(b_scale, sb.w, a_scale * sa.w);
        if (write_residual) *reinterpret_cast<float4*>(r + i) = v;
      }
      *reinterpret_cast<float4*>(row_buf + i) = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = r[i];
      float add = 0.0f;
      if (a) add = a_scale * slices_sum<TD>(a + (size_t)src * hidden + i, a_parts, a_stride);
      if (b) add = fmaf(b_scale, slices_sum<TD>(b + (size_t)src * hidden + i, b_parts, b_stride), add);
      if (a || b) v += add;
      row_buf[i] = v;
      if (write_residual && (a || b)) r[i] = v;
    }
  }
  __syncthreads();
  if (!out) return;
  const int gs = hidden / groups;
  for (int g = warp; g < groups; g += nwarps) {
    const float* part = row_buf + (size_t)g * gs;
    float ss = 0.0f;
    for (int i = lane; i < gs; i += 32) ss = fmaf(part[i], part[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  TO* o = out + (size_t)blockIdx.x * hidden;
  if (VEC && (gs & 3) == 0) {
    for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(row_buf + i), w = *reinterpret_cast<const float4*>(weight + i);
      const float rs = rstd[i / gs];
      GnOut4<TO>::store(o + i, make_float4(v.x * rs * w.x, v.y * rs * w.y, v.z * rs * w.z, v.w * rs * w.w));
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = Num<TO>::from_f(row_buf[i] * rstd[i / gs] * weight[i]);
}

template <typename TD, typename TO>
int launch_group_norm(float* residual, const void* a, int a_parts, long long a_stride, float a_scale, const void* b,
                      int b_parts, long long b_stride, float b_scale, const float* weight, float eps, int groups,
                      void* out, const int* rows, int n_rows, int hidden, int write_residual, cudaStream_t stream) {
  const size_t smem = ((size_t)hidden + groups) * sizeof(float);
  if (smem > 200 * 1024) return IFX_ERR_UNSUPPORTED;
  // 16-byte accesses where everything allows them; the order of every addition is the same in both shapes
  const bool vec = sizeof(TD) == 4 && hidden % 4 == 0 && (a_stride & 3) == 0 && (b_stride & 3) == 0 &&
                   (((uintptr_t)residual | (uintptr_t)a | (uintptr_t)b | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  auto kern = vec ? add_group_rmsnorm_kernel<TD, TO, true> : add_group_rmsnorm_kernel<TD, TO, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < hidden) threads <<= 1;
  const int rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, residual, (const TD*)a, a_parts, a_stride, a_scale,
                            (const TD*)b, b_parts, b_stride, b_scale, weight, eps, groups, (TO*)out, rows, hidden, write_residual);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// delta_dtype (of a and b) / out_dtype: IFX_F32 or IFX_BF16.  a, b and out may be null; a_parts / b_parts slices
// lie a_stride / b_stride elements apart.  groups must divide hidden.
IFX_API int ifx_add_group_rmsnorm(float* residual, const void* a, int a_parts, long long a_stride, float a_scale,
                                  const void* b, int b_parts, long long b_stride, float b_scale, int delta_dtype,
                                  const float* weight, float eps, int groups, void* out, int out_dtype, const int* rows,
                                  int n_rows, int hidden, int write_residual, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (rows && write_residual) return IFX_ERR_UNSUPPORTED;
  if (groups < 1 || hidden < 1 || hidden % groups) return IFX_ERR_UNSUPPORTED;
  if (a_parts < 1) a_parts = 1;
  if (b_parts < 1) b_parts = 1;
#define IFX_GN(TD, TO) return launch_group_norm<TD, TO>(residual, a, a_parts, a_stride, a_scale, b, b_parts, b_stride, b_scale, weight, \
                                                        eps, groups, out, rows, n_rows, hidden, write_residual, stream)
  if (delta_dtype == IFX_F32 && out_dtype == IFX_F32) IFX_GN(float, float);
  if (delta_dtype == IFX_F32 && out_dtype == IFX_BF16) IFX_GN(float, bf16);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_BF16) IFX_GN(bf16, bf16);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_F32) IFX_GN(bf16, float);
#undef IFX_GN
  return IFX_ERR_UNSUPPORTED;
}

namespace {
// A gated feed-forward's activation over float32 sums with clamped inputs:
//   g = min(zg + bg, limit), u = clamp(zu + bu, -limit, limit), out = g * sigmoid(alpha * g) * (u + shift)
// z holds gate columns first, then up columns, as `parts` slices that are added first.
template <typename T>
__global__ void glu_clamped_kernel(const float* __restrict__ z, int parts, long long part_stride, const float* __restrict__ bias,
                                   T* __restrict__ out, long long total, int inter, float limit, float alpha, float shift) {
  pdl_enter();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long m = idx / inter;
    const int i = (int)(idx - m * inter);
    const float* zr = z + m * 2 * inter;
    float g = bias ? bias[i] : 0.0f, u = bias ? bias[inter + i] : 0.0f;
    float sg = 0.0f, su = 0.0f;
    for (int p = 0; p < parts; ++p) { sg += zr[(size_t)p * part_stride + i]; su += zr[(size_t)p * part_stride + inter + i]; }
    g = fminf(sg + g, limit);
    u = fminf(fmaxf(su + u, -limit), limit);
    out[idx] = Num<T>::from_f(g / (1.0f + expf(-alpha * g)) * (u + shift));     // as glu_one below
  }
}

template <typename T> struct Out4;
template <> struct Out4<float> {
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Out4<bf16> {
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};
__device__ __forceinline__ float glu_one(float g, float u, float limit, float alpha, float shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + shift);
}
// The same, four neighbouring columns a thread with 16-byte loads: inter a multiple of 4, pointers on 16-byte boundaries.
template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(const float* __restrict__ z, int parts, long long part_stride, const float* __restrict__ bias,
                       T* __restrict__ out, int inter, float limit, float alpha, float shift) {
  pdl_enter();
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= inter) return;
  const size_t m = blockIdx.y;
  const float* zr = z + m * 2 * inter + i;
  float4 g = bias ? *reinterpret_cast<const float4*>(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 u = bias ? *reinterpret_cast<const float4*>(bias + inter + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 sg = make_float4(0.f, 0.f, 0.f, 0.f), su = sg;
  for (int p = 0; p < parts; ++p) {
    const float4 a = *reinterpret_cast<const float4*>(zr + (size_t)p * part_stride);
    const float4 b = *reinterpret_cast<const float4*>(zr + (size_t)p * part_stride + inter);
    sg.x += a.x; sg.y += a.y; sg.z += a.z; sg.w += a.w;
    su.x += b.x; su.y += b.y; su.z += b.z; su.w += b.w;
  }
  Out4<T>::store(out + m * inter + i, make_float4(glu_one(sg.x + g.x, su.x + u.x, limit, alpha, shift), glu_one(sg.y + g.y, su.y + u.y, limit, alpha, shift),
                                                  glu_one(sg.z + g.z, su.z + u.z, limit, alpha, shift), glu_one(sg.w + g.w, su.w + u.w, limit, alpha, shift)));
}
}  // namespace

// z float32 [parts][M][2 * inter]; bias float32 [2 * inter] or null; out [M][inter] of out_dtype.
IFX_API int ifx_glu_clamped(const float* z, int parts, long long part_stride, const float* bias, void* out, int out_dtype,
                            int m, int inter, float limit, float alpha, float shift, cudaStream_t stream) {
  if (m <= 0 || inter <= 0) return 0;
  if (parts < 1) return IFX_ERR_UNSUPPORTED;
  if (inter % 4 == 0 && (part_stride & 3) == 0 && m <= 65535 &&
      (((uintptr_t)z | (uintptr_t)bias | (uintptr_t)out) & 15) == 0) {
    const dim3 grid((inter / 4 + 255) / 256, m);
    int rcv;
    if (out_dtype == IFX_F32)
      rcv = launch_pdl(glu_clamped_vec_kernel<float>, grid, dim3(256), 0, stream, z, parts, part_stride, bias, (float*)out, inter, limit, alpha, shift);
    else if (out_dtype == IFX_BF16)
      rcv = launch_pdl(glu_clamped_vec_kernel<bf16>, grid, dim3(256), 0, stream, z, parts, part_stride, bias, (bf16*)out, inter, limit, alpha, shift);
    else
      return IFX_ERR_UNSUPPORTED;
    return rcv ? rcv : IFX_LAUNCH_CHECK();
  }
  const long long total = (long long)m * inter;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  int rc;
  if (out_dtype == IFX_F32)
    rc = launch_pdl(glu_clamped_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, z, parts, part_stride, bias, (float*)out,
                    total, inter, limit, alpha, shift);
  else if (out_dtype == IFX_BF16)
    rc = launch_pdl(glu_clamped_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, stream, z, parts, part_stride, bias, (bf16*)out,
                    total, inter, limit, alpha, shift);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}
