// Gated linear attention: a matrix-valued recurrent state per (request, head) with a decay per
// key channel,
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        S: [key_dim, value_dim], float32
//   o_t = S_t^T q_t
//
// and what surrounds it: the decays from a low-rank projection,
//   log alpha = log(sigmoid(W_2 a + b)) / tau,   a = the rank-r projection of the layer input,
// and the output stage, an RMS norm of every head's o over value_dim with one weight vector
// shared by the heads, times silu(gate).
//
// The state, the decays and their logarithms, the recurrence and the norm are float32 in every
// engine dtype.  A request's tokens are walked in order by the blocks that own its state, so the
// result at a position is bit-equal however the prompt was cut into steps and whatever else is
// in the batch: the state is read at the start of a step's portion and stored at its end.
//
// The inputs are columns of one stacked projection output [tokens, row_stride] (in the
// activation type, or float32 partial sums [parts, tokens, row_stride] of a split-K product).
#include "common.cuh"

namespace tk {

struct GlaInput {
  const void* x;            // [n_tokens, row_stride] activation type, or null
  const float* parts;       // [n_parts, n_tokens, row_stride] float32, or null
  int n_parts;
  int row_stride;
  long long part_stride;
};

template <typename T>
__device__ __forceinline__ float gla_ld(const GlaInput& in, size_t off) {
  if (in.parts == nullptr) return to_f32<T>(((const T*)in.x)[off]);
  float acc = 0.0f;
  for (int s = 0; s < in.n_parts; ++s) acc += in.parts[(size_t)s * in.part_stride + off];
  return acc;
}

// log_alpha[t, c] = logsigmoid(sum_j a[t, j] * w2[c, j] + bias[c]) / tau
template <typename T>
__global__ void gla_decay_kernel(GlaInput in, int a_off, const T* __restrict__ w2, const float* __restrict__ bias,
                                 float* __restrict__ log_alpha, int n_tokens, int channels, int rank, float inv_tau) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * channels) return;
  const int t = (int)(idx / channels), c = (int)(idx - (long long)t * channels);
  float z = 0.0f;
  const size_t row = (size_t)t * in.row_stride + a_off;
  for (int j = 0; j < rank; ++j) z += gla_ld<T>(in, row + j) * to_f32<T>(w2[(size_t)c * rank + j]);
  if (bias != nullptr) z += bias[c];
  // log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|))
  log_alpha[idx] = (fminf(z, 0.0f) - log1pf(expf(-fabsf(z)))) * inv_tau;
}

constexpr int kGlaRows = 16;      // rows of the state (key channels) that one thread keeps in registers
constexpr int kGlaBatch = 8;      // tokens staged in shared memory at a time
constexpr int kGlaCols = 32;      // value channels per block: one per lane

struct GlaScanParams {
  GlaInput in;
  int q_off, k_off, v_off;  // first column of q, k and v in a row
  const float* log_alpha;   // [n_tokens, heads * key_dim]
  float* state;             // [n_slots, heads, key_dim, value_dim]
  float* out;               // [n_tokens, heads, value_dim]
  const int* req_q_start;
  const int* req_q_len;
  const int* req_slot;
  int* err;
  int n_tokens, n_slots, heads, key_dim, value_dim;
  float q_scale;
};

// One block per (request, head, 32 value channels); warp w keeps rows 16 w .. 16 w + 15 of the
// block's 32 columns of the state in registers, a lane per column.
template <typename T>
__global__ void gla_scan_kernel(GlaScanParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kGlaCols;
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5, n_parts = blockDim.x >> 5;
  const int dkp = n_parts * kGlaRows;
  float* sq = smem;
  float* sk = sq + kGlaBatch * dkp;
  float* sa = sk + kGlaBatch * dkp;
  float* sv = sa + kGlaBatch * dkp;
  float* so = sv + kGlaBatch * kGlaCols;
  const int dk = p.key_dim, dv = p.value_dim;
  const int slot = p.req_slot[r];
  const int q0 = p.req_q_start[r], n = p.req_q_len[r];
  if (slot < 0 || slot >= p.n_slots || q0 < 0 || n < 0 || q0 + n > p.n_tokens) {
    if (threadIdx.x == 0) set_error(p.err, kErrRequest, r, slot, q0);
    return;
  }
  const int j = j0 + lane;
  float* srow = p.state + (((size_t)slot * p.heads + h) * dk + (size_t)part * kGlaRows) * dv + j;
  float s[kGlaRows];
#pragma unroll
  for (int ii = 0; ii < kGlaRows; ++ii) {
    s[ii] = (j < dv && part * kGlaRows + ii < dk) ? srow[(size_t)ii * dv] : 0.0f;
  }
  for (int t0 = 0; t0 < n; t0 += kGlaBatch) {
    const int nb = min(kGlaBatch, n - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nb * dkp; idx += blockDim.x) {
      const int tb = idx / dkp, i = idx - tb * dkp;
      const size_t tok = (size_t)(q0 + t0 + tb);
      float q = 0.0f, k = 0.0f, a = 0.0f;
      if (i < dk) {
        q = gla_ld<T>(p.in, tok * p.in.row_stride + p.q_off + h * dk + i) * p.q_scale;
        k = gla_ld<T>(p.in, tok * p.in.row_stride + p.k_off + h * dk + i);
        a = expf(p.log_alpha[(tok * p.heads + h) * dk + i]);
      }
      sq[idx] = q; sk[idx] = k; sa[idx] = a;
    }
    for (int idx = threadIdx.x; idx < nb * kGlaCols; idx += blockDim.x) {
      const int tb = idx / kGlaCols, c = idx - tb * kGlaCols;
      const size_t tok = (size_t)(q0 + t0 + tb);
      sv[idx] = (j0 + c < dv) ? gla_ld<T>(p.in, tok * p.in.row_stride + p.v_off + h * dv + j0 + c) : 0.0f;
    }
    __syncthreads();
    for (int tb = 0; tb < nb; ++tb) {
      const float v = sv[tb * kGlaCols + lane];
      const float4* q4 = reinterpret_cast<const float4*>(sq + tb * dkp + part * kGlaRows);
      const float4* k4 = reinterpret_cast<const float4*>(sk + tb * dkp + part * kGlaRows);
      const float4* a4 = reinterpret_cast<const float4*>(sa + tb * dkp + part * kGlaRows);
      float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
      for (int g = 0; g < kGlaRows / 4; ++g) {
        const float4 q = q4[g], k = k4[g], a = a4[g];
        s[4 * g + 0] = a.x * s[4 * g + 0] + k.x * v;
        s[4 * g + 1] = a.y * s[4 * g + 1] + k.y * v;
        s[4 * g + 2] = a.z * s[4 * g + 2] + k.z * v;
        s[4 * g + 3] = a.w * s[4 * g + 3] + k.w * v;
        o0 += q.x * s[4 * g + 0]; o1 += q.y * s[4 * g + 1];
        o0 += q.z * s[4 * g + 2]; o1 += q.w * s[4 * g + 3];
      }
      so[(tb * n_parts + part) * kGlaCols + lane] = o0 + o1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nb * kGlaCols; idx += blockDim.x) {
      const int tb = idx / kGlaCols, c = idx - tb * kGlaCols;
      if (j0 + c >= dv) continue;
      float o = 0.0f;
      for (int w = 0; w < n_parts; ++w) o += so[(tb * n_parts + w) * kGlaCols + c];
      p.out[((size_t)(q0 + t0 + tb) * p.heads + h) * dv + j0 + c] = o;
    }
  }
#pragma unroll
  for (int ii = 0; ii < kGlaRows; ++ii) {
    if (j < dv && part * kGlaRows + ii < dk) srow[(size_t)ii * dv] = s[ii];
  }
}

// y[t, h, e] = o[t, h, e] * rsqrt(mean_e o^2 + eps) * w[e] * silu(g[t, h, e]);   one warp per (token, head)
template <typename T>
__global__ void gla_out_kernel(const float* __restrict__ o, GlaInput in, int g_off, const float* __restrict__ w,
                               T* __restrict__ y, int n_tokens, int heads, int dv, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float* orow = o + (size_t)item * dv;
  float ss = 0.0f;
  for (int e = lane; e < dv; e += 32) ss += orow[e] * orow[e];
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dv + eps);
  for (int e = lane; e < dv; e += 32) {
    float v = orow[e] * rstd;
    if (w != nullptr) v *= w[e];
    if (g_off >= 0) {
      const float g = gla_ld<T>(in, (size_t)t * in.row_stride + g_off + h * dv + e);
      v *= g / (1.0f + expf(-g));
    }
    y[(size_t)item * dv + e] = from_f32<T>(v);
  }
}

}  // namespace tk

static tk::GlaInput gla_input(const void* x, const float* parts, int n_parts, int n_tokens, int row_stride) {
  tk::GlaInput in;
  in.x = x; in.parts = parts; in.n_parts = n_parts; in.row_stride = row_stride;
  in.part_stride = (long long)n_tokens * row_stride;
  return in;
}

TK_API int tk_gla_decay(const void* x, const float* parts, int n_parts, int row_stride, int a_off,
                        const void* w2, const float* bias, float* log_alpha, int n_tokens, int channels,
                        int rank, float tau, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (channels < 1 || rank < 1 || !(tau > 0.0f) || (x == nullptr) == (parts == nullptr)) return (int)cudaErrorInvalidValue;
  const long long total = (long long)n_tokens * channels;
  const tk::GlaInput in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::gla_decay_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                   in, a_off, (const T*)w2, bias, log_alpha, n_tokens, channels, rank, 1.0f / tau));
  return (int)e;
}

TK_API int tk_gla_scan(const void* x, const float* parts, int n_parts, int row_stride, int q_off, int k_off,
                       int v_off, const float* log_alpha, float* state, float* out, const int* req_q_start,
                       const int* req_q_len, const int* req_slot, int* err, int n_tokens, int n_reqs, int n_slots,
                       int heads, int key_dim, int value_dim, float q_scale, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  const int n_warps = (key_dim + tk::kGlaRows - 1) / tk::kGlaRows;
  if (key_dim < 1 || value_dim < 1 || n_warps > 32 || heads < 1 || heads > 65535 ||
      (x == nullptr) == (parts == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::GlaScanParams p;
  p.in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.log_alpha = log_alpha; p.state = state; p.out = out;
  p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_slot = req_slot; p.err = err;
  p.n_tokens = n_tokens; p.n_slots = n_slots; p.heads = heads; p.key_dim = key_dim; p.value_dim = value_dim;
  p.q_scale = q_scale;
  const int col_tiles = (value_dim + tk::kGlaCols - 1) / tk::kGlaCols;
  if (col_tiles > 65535) return (int)cudaErrorInvalidValue;
  const int dkp = n_warps * tk::kGlaRows;
  const size_t smem = sizeof(float) * ((size_t)3 * tk::kGlaBatch * dkp + tk::kGlaBatch * tk::kGlaCols +
                                       (size_t)tk::kGlaBatch * n_warps * tk::kGlaCols);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(tk::gla_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (e == cudaSuccess) {
      e = tk::launch(tk::gla_scan_kernel<T>, dim3((unsigned)n_reqs, (unsigned)heads, (unsigned)col_tiles),
                     dim3(n_warps * 32), smem, stream, p);
    }
  });
  return (int)e;
}

TK_API int tk_gla_out(const float* o, const void* x, const float* parts, int n_parts, int row_stride, int g_off,
                      const float* w, void* y, int n_tokens, int heads, int value_dim, float eps, int dtype,
                      cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads < 1 || value_dim < 1 || (g_off >= 0 && (x == nullptr) == (parts == nullptr))) return (int)cudaErrorInvalidValue;
  const tk::GlaInput in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  const long long items = (long long)n_tokens * heads;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::gla_out_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, o, in,
                                   g_off, w, (T*)y, n_tokens, heads, value_dim, eps));
  return (int)e;
}
