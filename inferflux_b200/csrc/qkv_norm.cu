// What lies between the stacked q, k, v projection and attention in designs that norm the projections, one block a
// token, everything float32:
//
//   q <- N(q) * wq over ALL of the token's query columns at once (heads * dim), k <- N(k) * wk likewise
//        (N(v) = v / sqrt(mean(v^2) + eps); either weight may be absent: then that projection stays as it is)
//   rotation of the first 2 * rot_half dimensions of every query and key head, pairs (i, i + rot_half) or (2i, 2i + 1)
//   v <- v / sqrt(mean over the head (v^2) + eps)   per key/value head, no weight          (v_norm)
//   value mixing: mode 1 stores the token's values in v_first; mode 2 computes v <- (1 - lambda) v + lambda v_first
//   q goes to q_out, k and v into the paged cache at slot_map.
//
// The projection arrives as float32 sums [N][W] (or slices [P][N][W] to be added): q heads, k heads, v heads side by side.
#include "common.cuh"

namespace {
struct QkvNormArgs {
  const float* proj; int parts; long long part_stride; int width;
  const float* wq; const float* wk; float eps;
  const float* cos_t; const float* sin_t; int rot_half; int layout;      // layout 0: halves, 1: neighbours
  int n_heads, n_kv, dim, vdim;
  int v_norm; int mix_mode; const float* lambda; float* v_first;        // v_first [N][n_kv * vdim]
  void* q_out; const int* slot_map; void* k_cache; void* v_cache; long long page_stride; int page_size, page_shift;
};

template <typename T>
__global__ void __launch_bounds__(256)
qkv_norm_rope_kernel(QkvNormArgs p) {
  extern __shared__ float row[];                   // [channels]
  __shared__ float scratch[32];
  pdl_enter();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int qw = p.n_heads * p.dim, kw = p.n_kv * p.dim, vw = p.n_kv * p.vdim;
  const int channels = qw + kw + vw;
  float ssq = 0.0f, ssk = 0.0f;
  for (int c = tid; c < channels; c += blockDim.x) {
    float v = 0.0f;
    for (int s = 0; s < p.parts; ++s) v += p.proj[(size_t)s * p.part_stride + (size_t)t * p.width + c];
    row[c] = v;
    if (c < qw) ssq = fmaf(v, v, ssq);
    else if (c < qw + kw) ssk = fmaf(v, v, ssk);
  }
  const float inv_q = p.wq ? 1.0f / sqrtf(block_sum(ssq, scratch) / (float)qw + p.eps) : 1.0f;
  const float inv_k = p.wk ? 1.0f / sqrtf(block_sum(ssk, scratch) / (float)kw + p.eps) : 1.0f;
  __syncthreads();
  if (p.wq) for (int c = tid; c < qw; c += blockDim.x) row[c] = row[c] * inv_q * p.wq[c];
  if (p.wk) for (int c = tid; c < kw; c += blockDim.x) row[qw + c] = row[qw + c] * inv_k * p.wk[c];
  __syncthreads();
  // rotation: one thread a pair
  if (p.rot_half > 0) {
    const int pairs = (p.n_heads + p.n_kv) * p.rot_half;
    for (int i = tid; i < pairs; i += blockDim.x) {
      const int head = i / p.rot_half, j = i - head * p.rot_half;
      const int a = head * p.dim + (p.layout == 0 ? j : 2 * j);
      const int b = p.layout == 0 ? a + p.rot_half : a + 1;
      const float cs = p.cos_t[(size_t)t * p.rot_half + j], sn = p.sin_t[(size_t)t * p.rot_half + j];
      const float u = row[a], v = row[b];
      row[a] = u * cs - v * sn;
      row[b] = v * cs + u * sn;
    }
  }
  // values: a warp a head
  const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const float lam = p.mix_mode == 2 ? p.lambda[0] : 0.0f;
  for (int h = warp; h < p.n_kv; h += nwarps) {
    float* v = row + qw + kw + h * p.vdim;
    float inv = 1.0f;
    if (p.v_norm) {
      float ss = 0.0f;
      for (int i = lane; i < p.vdim; i += 32) ss = fmaf(v[i], v[i], ss);
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.vdim + p.eps);
    }
    float* vf = p.v_first ? p.v_first + (size_t)t * vw + h * p.vdim : nullptr;
    for (int i = lane; i < p.vdim; i += 32) {
      float y = v[i] * inv;
      if (p.mix_mode == 1) vf[i] = y;
      else if (p.mix_mode == 2) y = (1.0f - lam) * y + lam * vf[i];
      v[i] = y;
    }
  }
  __syncthreads();
  T* q = (T*)p.q_out + (size_t)t * qw;
  for (int c = tid; c < qw; c += blockDim.x) q[c] = Num<T>::from_f(row[c]);
  const int where = p.slot_map ? p.slot_map[t] : -1;
  if (where < 0) return;
  const int page = where >> p.page_shift, off = where & (p.page_size - 1);
  T* kc = (T*)p.k_cache + (size_t)page * p.page_stride;
  T* vc = (T*)p.v_cache + (size_t)page * p.page_stride;
  for (int c = tid; c < kw; c += blockDim.x) {
    const int h = c / p.dim, d = c - h * p.dim;
    kc[((size_t)h * p.page_size + off) * p.dim + d] = Num<T>::from_f(row[qw + c]);
  }
  for (int c = tid; c < vw; c += blockDim.x) {
    const int h = c / p.vdim, d = c - h * p.vdim;
    vc[((size_t)h * p.page_size + off) * p.vdim + d] = Num<T>::from_f(row[qw + kw + c]);
  }
}
}  // namespace

IFX_API int ifx_qkv_norm_rope_write(const float* proj, int parts, long long part_stride, int width, const float* wq,
                                    const float* wk, float eps, const float* cos_t, const float* sin_t, int rot_half,
                                    int layout, int n_heads, int n_kv, int dim, int vdim, int v_norm, int mix_mode,
                                    const float* lambda, float* v_first, void* q_out, int dtype, const int* slot_map,
                                    void* k_cache, void* v_cache, long long page_stride, int page_size, int n_tokens,
                                    cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (page_size <= 0 || (page_size & (page_size - 1)) || n_heads < 1 || n_kv < 1 || dim < 1 || vdim < 1) return IFX_ERR_UNSUPPORTED;
  if (rot_half < 0 || 2 * rot_half > dim || mix_mode < 0 || mix_mode > 2 || (mix_mode && !v_first) || (mix_mode == 2 && !lambda))
    return IFX_ERR_UNSUPPORTED;
  const int channels = (n_heads + n_kv) * dim + n_kv * vdim;
  if (channels > width) return IFX_ERR_UNSUPPORTED;
  QkvNormArgs p{proj, parts, part_stride, width, wq, wk, eps, cos_t, sin_t, rot_half, layout, n_heads, n_kv, dim, vdim,
                v_norm, mix_mode, lambda, v_first, q_out, slot_map, k_cache, v_cache, page_stride, page_size, 0};
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  const size_t smem = (size_t)channels * sizeof(float);
  auto kern = dtype == IFX_BF16 ? qkv_norm_rope_kernel<bf16> : qkv_norm_rope_kernel<float>;
  if (dtype != IFX_BF16 && dtype != IFX_F32) return IFX_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int rc = launch_pdl(kern, dim3(n_tokens), dim3(256), smem, stream, p);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
