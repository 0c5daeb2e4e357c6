// Latent attention: what stands between the input projections and the attention kernel, and
// between the attention kernel and the output projection, when all heads' keys and values are
// products of one latent vector per token.
//
// A token's cache row is  [ c (rank) | k_rot (rot) ]:
//   c     = x_c * rsqrt(mean(x_c^2) + eps) * w_c        the latent, RMS-normed with a plain weight
//   k_rot = the rotated key part that all heads share: neighbouring pairs (x[2i], x[2i+1]) of its
//           first rot_pairs * 2 elements turn by the angle of the token's position (the table holds
//           cos and sin, already multiplied by any magnitude factor); the rest passes unchanged
// and the scores are taken in the latent space: with q_abs[h] = W_uk[h]^T q_nope[h] (a product of
// its own, given here as float32 [heads, tokens, rank])
//   q_lat[t, h] = [ q_abs[h, t] | rotated q_rot[t, h] ]      float32
//   score = q_lat . row * scale,   out_lat = sum_j p_j c_j,   o[h] = W_uv[h] out_lat[h].
// A design whose queries go through a latent of their own gets that latent normed here too.
//
// latent_prepare_kernel does all of that in one launch (block y = 0: the token's cache row and the
// query latent; block y = 1 + h: the query row of head h).  heads_gate_kernel brings the per-head
// output [heads, tokens, v] back to token-major rows and applies the sigmoid gate.
// Norm statistics, angles and rotations are float32; rows are rounded once on store.
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

struct LatentPrepareParams {
  StackedInput in;            // the stacked input projection of the step's tokens
  int kv_off;                 // columns [kv_off, kv_off + rank + rot): latent input | rotated key part
  int q_off;                  // head h's rotated query part: columns q_off + h * q_head_cols + q_rot_off + [0, rot)
  int q_head_cols, q_rot_off;
  int cq_off, cq_rank;        // columns of the query latent's input (cq_rank 0: none)
  const float* kv_norm_w;     // [rank]
  const float* cq_norm_w;     // [cq_rank]
  void* cq_out;               // [n_tokens, cq_rank] activation type
  const float* q_abs;         // [heads, n_tokens, rank] float32, or null (no query rows are assembled)
  float* q_lat;               // [n_tokens, heads, rank + rot] float32
  void* cache;                // [num_pages, 1, page_size, rank + rot]
  const float2* rope_table;   // [n_tokens, rot_pairs] or null
  const int* positions;
  const int* tok_req;
  const int* req_slot;
  const int* block_table;
  const int* req_q_len;
  const int* req_kv_len;
  int* err;
  int n_tokens, n_reqs, heads, rank, rot, rot_pairs;
  int page_size, max_pages, num_pages;
  float eps;
};

template <typename T>
__global__ void latent_prepare_kernel(LatentPrepareParams p) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t row = (size_t)t * p.in.row_stride;
  const float2* tab = p.rope_table != nullptr ? p.rope_table + (size_t)t * p.rot_pairs : nullptr;
  const int width = p.rank + p.rot;

  if (blockIdx.y > 0) {
    // the query row of one head: the absorbed part as it is, the rotated part turned
    const int h = blockIdx.y - 1;
    float* dst = p.q_lat + ((size_t)t * p.heads + h) * width;
    const float* src = p.q_abs + ((size_t)h * p.n_tokens + t) * p.rank;
    for (int e = threadIdx.x; e < p.rank; e += blockDim.x) dst[e] = src[e];
    const size_t qo = row + p.q_off + (size_t)h * p.q_head_cols + p.q_rot_off;
    for (int i = threadIdx.x; 2 * i < p.rot; i += blockDim.x) {
      const float u = stacked_ld<T>(p.in, qo + 2 * i);
      const bool pair = 2 * i + 1 < p.rot;
      const float w = pair ? stacked_ld<T>(p.in, qo + 2 * i + 1) : 0.0f;
      float2 cs = make_float2(1.0f, 0.0f);
      if (tab != nullptr && i < p.rot_pairs) cs = tab[i];
      dst[p.rank + 2 * i] = u * cs.x - w * cs.y;
      if (pair) dst[p.rank + 2 * i + 1] = w * cs.x + u * cs.y;
    }
    return;
  }

  // the query latent, normed (its product with the up-projection comes after this kernel)
  if (p.cq_rank > 0) {
    float ss = 0.0f;
    for (int e = threadIdx.x; e < p.cq_rank; e += blockDim.x) {
      const float x = stacked_ld<T>(p.in, row + p.cq_off + e);
      ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)p.cq_rank + p.eps);
    T* dst = (T*)p.cq_out + (size_t)t * p.cq_rank;
    for (int e = threadIdx.x; e < p.cq_rank; e += blockDim.x) {
      dst[e] = from_f32<T>(stacked_ld<T>(p.in, row + p.cq_off + e) * rstd * p.cq_norm_w[e]);
    }
  }

  // the token's cache row
  const int pos = p.positions[t];
  const int r = p.tok_req[t];
  if (pos < 0) { if (threadIdx.x == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
  if (r < 0 || r >= p.n_reqs) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  const int pidx = pos / p.page_size;
  const int slot = pos - pidx * p.page_size;
  const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
  if (page < 0 || page >= p.num_pages) { if (threadIdx.x == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
  T* dst = (T*)p.cache + ((size_t)page * p.page_size + slot) * width;
  // the request's last token of this step clears the rest of a page that was begun in this step, so
  // that a live page never holds stale values behind the last position
  if (p.req_kv_len != nullptr) {
    const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
    if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) {
      const int rest = (p.page_size - 1 - slot) * width;
      for (int e = threadIdx.x; e < rest; e += blockDim.x) dst[width + e] = from_f32<T>(0.0f);
    }
  }
  float ss = 0.0f;
  for (int e = threadIdx.x; e < p.rank; e += blockDim.x) {
    const float x = stacked_ld<T>(p.in, row + p.kv_off + e);
    ss += x * x;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)p.rank + p.eps);
  for (int e = threadIdx.x; e < p.rank; e += blockDim.x) {
    dst[e] = from_f32<T>(stacked_ld<T>(p.in, row + p.kv_off + e) * rstd * p.kv_norm_w[e]);
  }
  const size_t ko = row + p.kv_off + p.rank;
  for (int i = threadIdx.x; 2 * i < p.rot; i += blockDim.x) {
    const float u = stacked_ld<T>(p.in, ko + 2 * i);
    const bool pair = 2 * i + 1 < p.rot;
    const float w = pair ? stacked_ld<T>(p.in, ko + 2 * i + 1) : 0.0f;
    float2 cs = make_float2(1.0f, 0.0f);
    if (tab != nullptr && i < p.rot_pairs) cs = tab[i];
    dst[p.rank + 2 * i] = from_f32<T>(u * cs.x - w * cs.y);
    if (pair) dst[p.rank + 2 * i + 1] = from_f32<T>(w * cs.x + u * cs.y);
  }
}

// y[t, h * dv + e] = x[h, t, e] * sigmoid(gate[t, g_off + h * dv + e])   (no gate: g_off < 0)
template <typename T>
__global__ void heads_gate_kernel(const T* __restrict__ x, StackedInput gate, int g_off, T* __restrict__ y,
                                  int n_tokens, int heads, int dv) {
  pdl_trigger();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)n_tokens * heads * dv;
  if (idx >= total) return;
  const int cols = heads * dv;
  const int t = (int)(idx / cols);
  const int c = (int)(idx - (long long)t * cols);
  const int h = c / dv, e = c - h * dv;
  float v = to_f32<T>(x[((size_t)h * n_tokens + t) * dv + e]);
  if (g_off >= 0) {
    const float g = stacked_ld<T>(gate, (size_t)t * gate.row_stride + g_off + c);
    v *= 1.0f / (1.0f + expf(-g));
  }
  y[idx] = from_f32<T>(v);
}

}  // namespace tk

TK_API int tk_latent_prepare(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                             int kv_off, int q_off, int q_head_cols, int q_rot_off, int cq_off, int cq_rank,
                             const float* kv_norm_w, const float* cq_norm_w, void* cq_out, const float* q_abs,
                             float* q_lat, void* cache, const float* rope_table, const int* positions,
                             const int* tok_req, const int* req_slot, const int* block_table, const int* req_q_len,
                             const int* req_kv_len, int* err, int n_tokens, int n_reqs, int heads, int rank, int rot,
                             int rot_pairs, int page_size, int max_pages, int num_pages, float eps, int dtype,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || rank < 1 || rot < 0 || 2 * rot_pairs > rot || heads < 0 || heads > 65534 ||
      (rot_pairs > 0 && rope_table == nullptr) || (cq_rank > 0 && (cq_out == nullptr || cq_norm_w == nullptr)) ||
      (q_abs != nullptr && q_lat == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::LatentPrepareParams p;
  p.in.x = x; p.in.parts = parts; p.in.n_parts = n_parts; p.in.row_stride = row_stride; p.in.part_stride = part_stride;
  p.kv_off = kv_off; p.q_off = q_off; p.q_head_cols = q_head_cols; p.q_rot_off = q_rot_off;
  p.cq_off = cq_off; p.cq_rank = cq_rank; p.kv_norm_w = kv_norm_w; p.cq_norm_w = cq_norm_w; p.cq_out = cq_out;
  p.q_abs = q_abs; p.q_lat = q_lat; p.cache = cache; p.rope_table = (const float2*)rope_table;
  p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot; p.block_table = block_table;
  p.req_q_len = req_q_len; p.req_kv_len = req_kv_len; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.heads = heads; p.rank = rank; p.rot = rot; p.rot_pairs = rot_pairs;
  p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.eps = eps;
  const int widest = rank > cq_rank ? rank : cq_rank;
  const int threads = widest >= 256 ? 256 : (widest >= 128 ? 128 : 64);
  dim3 grid(n_tokens, q_abs != nullptr ? 1 + heads : 1);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::latent_prepare_kernel<T>, grid, dim3(threads), 0, stream, p));
  return (int)e;
}

TK_API int tk_heads_gate(const void* x, const void* gate, const float* gate_parts, int n_parts, long long part_stride,
                         int row_stride, int g_off, void* y, int n_tokens, int heads, int dv, int dtype,
                         cudaStream_t stream) {
  if (n_tokens <= 0 || heads <= 0 || dv <= 0) return 0;
  if (g_off >= 0 && (gate == nullptr) == (gate_parts == nullptr)) return (int)cudaErrorInvalidValue;
  tk::StackedInput in;
  in.x = gate; in.parts = gate_parts; in.n_parts = n_parts; in.row_stride = row_stride; in.part_stride = part_stride;
  const long long total = (long long)n_tokens * heads * dv;
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::heads_gate_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                   (const T*)x, in, g_off, (T*)y, n_tokens, heads, dv));
  return (int)e;
}
