// A branch that is normalised before it joins the residual stream:
//
//   y = branch * rsqrt(mean(branch^2) + eps_b) * post_w (* layer_scale)
//   x = resid + y                      (written back to resid unless `rows` selects rows)
//   out = x * rsqrt(mean(x^2) + eps_n) * next_w          (when a norm follows)
//
// in one pass: the norm after a sublayer, the per-channel layer scale, the 32-bit residual sum
// and the norm in front of the next sublayer.  Statistics, sums and the residual stream are
// float32; `out` is rounded once to the activation type.  The branch comes in the activation
// type or as float32 partial sums [parts, tokens, hidden] of a split-K product.
#include "common.cuh"

namespace tk {

template <typename T>
__global__ void branch_norm_add_kernel(float* __restrict__ resid, const T* __restrict__ branch,
                                       const float* __restrict__ parts, int n_parts, size_t part_stride,
                                       const float* __restrict__ post_w, const float* __restrict__ layer_scale,
                                       const float* __restrict__ next_w, T* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps_b, float eps_n) {
  extern __shared__ float row[];          // the branch, then the new residual row
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * hidden;
  float ss = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float b;
    if (branch != nullptr) {
      b = to_f32<T>(branch[(size_t)r * hidden + h]);
    } else {
      b = 0.0f;
      for (int s = 0; s < n_parts; ++s) b += parts[(size_t)s * part_stride + (size_t)r * hidden + h];
    }
    row[h] = b;
    ss += b * b;
  }
  ss = block_sum(ss, scratch);
  const float rstd_b = rsqrtf(ss / (float)hidden + eps_b);
  float ss2 = 0.0f;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
    float y = row[h] * rstd_b;
    if (post_w != nullptr) y *= post_w[h];
    if (layer_scale != nullptr) y *= layer_scale[h];
    const float v = x[h] + y;
    if (rows == nullptr) x[h] = v;
    row[h] = v;
    ss2 += v * v;
  }
  if (out == nullptr) return;
  ss2 = block_sum(ss2, scratch);
  const float rstd = rsqrtf(ss2 / (float)hidden + eps_n);
  T* o = out + (size_t)i * hidden;
  for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = from_f32<T>(row[h] * rstd * next_w[h]);
}

}  // namespace tk

TK_API int tk_branch_norm_add(float* resid, const void* branch, const float* parts, int n_parts,
                              long long part_stride, const float* post_w, const float* layer_scale,
                              const float* next_w, void* out, const int* rows, int n_rows, int hidden,
                              float eps_b, float eps_n, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden < 1 || hidden > 12288 || (branch == nullptr) == (parts == nullptr) || (out != nullptr && next_w == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::branch_norm_add_kernel<T>, dim3((unsigned)n_rows), dim3(threads),
                                   (size_t)hidden * sizeof(float), stream, resid, (const T*)branch, parts, n_parts,
                                   (size_t)part_stride, post_w, layer_scale, next_w, (T*)out, rows, hidden, eps_b,
                                   eps_n));
  return (int)e;
}
