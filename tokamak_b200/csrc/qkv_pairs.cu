// Preparation of queries, keys and values whose key and value heads may differ in size:
// rotation of neighbouring pairs over the first `rotary_dim` elements of every query and key
// head, an optional unit RMS norm of each rotated head (no weight), an optional blend of the
// values with the values that an earlier layer produced for the same token, and the write of
// keys and values into their pages.
//
//   pair (u, w) = (x[2i], x[2i+1]) at angle a:   (u cos a - w sin a,  w cos a + u sin a)
//   unit norm:   x / sqrt(mean(x^2) + eps)       over the head, after the rotation
//   value blend: v = (1 - lambda) v + lambda v_first
//
// Everything is computed in float32 and rounded once on store.  One warp per (token, head);
// a row of the input holds the query heads, then the key heads, then the value heads.
#include "common.cuh"

namespace tk {

struct QkvPairsParams {
  const void* qkv;          // [n_tokens, row_stride]
  const float* qkv_parts;   // or float32 partial sums [n_parts, n_tokens, row_stride]
  int n_parts;
  void* q_out;              // [n_tokens, n_q_heads, k_dim]
  void* k_cache;            // [num_pages, n_kv_heads, page_size, k_dim]
  void* v_cache;            // [num_pages, n_kv_heads, page_size, v_dim]
  const int* positions;
  const int* tok_req;
  const int* req_slot;
  const int* block_table;
  const int* req_q_len;     // or null: see the clearing of a page's rest below
  const int* req_kv_len;
  const float2* rope_table; // [n_tokens, rotary_dim / 2] (cos, sin) or null
  const float* v_first_in;  // [n_tokens, n_kv_heads * v_dim] float32, or null: no blend
  const float* v_lambda;    // one float on the device
  float* v_first_out;       // [n_tokens, n_kv_heads * v_dim] float32, or null: the raw values of this layer
  int* err;
  int n_tokens, n_reqs, n_q_heads, n_kv_heads, k_dim, v_dim, rotary_dim;
  int row_stride, page_size, max_pages, num_pages;
  int unit_norm;
  float eps;
};

constexpr int kPairsIter = 4;     // pairs per lane: head sizes up to 256

template <typename T>
__device__ __forceinline__ float2 load_pair(const QkvPairsParams& p, size_t off) {
  if (p.qkv_parts == nullptr) {
    const T* src = (const T*)p.qkv + off;
    return make_float2(to_f32<T>(src[0]), to_f32<T>(src[1]));
  }
  float2 acc = make_float2(0.0f, 0.0f);
  const size_t part_stride = (size_t)p.n_tokens * p.row_stride;
  for (int s = 0; s < p.n_parts; ++s) {
    const float* src = p.qkv_parts + (size_t)s * part_stride + off;
    acc.x += src[0]; acc.y += src[1];
  }
  return acc;
}

template <typename T>
__global__ void qkv_pairs_kernel(QkvPairsParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads_total = p.n_q_heads + 2 * p.n_kv_heads;
  const int t = blockIdx.x;
  const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (h >= heads_total) return;
  int kind, head;     // 0 = q, 1 = k, 2 = v
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }
  const int d = (kind == 2) ? p.v_dim : p.k_dim;
  const size_t src_off = (size_t)t * p.row_stride +
      (kind == 0 ? (size_t)head * p.k_dim
                 : kind == 1 ? (size_t)(p.n_q_heads + head) * p.k_dim
                             : (size_t)(p.n_q_heads + p.n_kv_heads) * p.k_dim + (size_t)head * p.v_dim);

  T* dst;
  int zero_rows = 0;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
  } else {
    const int pos = p.positions[t];
    const int r = p.tok_req[t];
    if (pos < 0) { if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
    if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    const int slot = pos - pidx * p.page_size;
    const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
    if (page < 0 || page >= p.num_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + (((size_t)page * p.n_kv_heads + head) * p.page_size + slot) * d;
    // the request's last token of this step clears the rest of a page that was begun in this step, so
    // that a live page never holds stale values behind the last position
    if (p.req_kv_len != nullptr) {
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
    }
  }
  for (int z = 1; z <= zero_rows; ++z) {
    for (int e = lane; e < d; e += 32) dst[(size_t)z * d + e] = from_f32<T>(0.0f);
  }

  if (kind == 2) {
    const float lam = (p.v_first_in != nullptr) ? *p.v_lambda : 0.0f;
    for (int e = 2 * lane; e < d; e += 64) {
      float2 x = load_pair<T>(p, src_off + e);
      const size_t vo = ((size_t)t * p.n_kv_heads + head) * d + e;
      if (p.v_first_out != nullptr) { p.v_first_out[vo] = x.x; p.v_first_out[vo + 1] = x.y; }
      if (p.v_first_in != nullptr) {
        x.x = (1.0f - lam) * x.x + lam * p.v_first_in[vo];
        x.y = (1.0f - lam) * x.y + lam * p.v_first_in[vo + 1];
      }
      dst[e] = from_f32<T>(x.x); dst[e + 1] = from_f32<T>(x.y);
    }
    return;
  }

  float2 x[kPairsIter];
  float ss = 0.0f;
  const float2* tab = p.rope_table ? p.rope_table + (size_t)t * (p.rotary_dim >> 1) : nullptr;
#pragma unroll
  for (int k = 0; k < kPairsIter; ++k) {
    const int e = 2 * lane + 64 * k;
    x[k] = make_float2(0.0f, 0.0f);
    if (e < d) {
      const float2 in = load_pair<T>(p, src_off + e);
      if (tab != nullptr && e < p.rotary_dim) {
        const float2 cs = tab[e >> 1];
        x[k].x = in.x * cs.x - in.y * cs.y;
        x[k].y = in.y * cs.x + in.x * cs.y;
      } else {
        x[k] = in;
      }
      ss += x[k].x * x[k].x + x[k].y * x[k].y;
    }
  }
  float rstd = 1.0f;
  if (p.unit_norm) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)d + p.eps);
  }
#pragma unroll
  for (int k = 0; k < kPairsIter; ++k) {
    const int e = 2 * lane + 64 * k;
    if (e < d) { dst[e] = from_f32<T>(x[k].x * rstd); dst[e + 1] = from_f32<T>(x[k].y * rstd); }
  }
}

// Eight neighbouring elements (the address is a multiple of eight elements).
template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void st8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// The same for head sizes and a rotated part that are multiples of 8 and an input in the activation
// type: a lane takes eight neighbouring elements (four pairs), so every access is 16 or 32 bytes.
// One warp per (token, head); heads of up to 256 elements.
template <typename T>
__global__ void qkv_pairs_vec_kernel(QkvPairsParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads_total = p.n_q_heads + 2 * p.n_kv_heads;
  const int t = blockIdx.x;
  const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (h >= heads_total) return;
  int kind, head;     // 0 = q, 1 = k, 2 = v
  if (h < p.n_q_heads) { kind = 0; head = h; }
  else if (h < p.n_q_heads + p.n_kv_heads) { kind = 1; head = h - p.n_q_heads; }
  else { kind = 2; head = h - p.n_q_heads - p.n_kv_heads; }
  const int d = (kind == 2) ? p.v_dim : p.k_dim;
  const T* src = (const T*)p.qkv + (size_t)t * p.row_stride +
      (kind == 0 ? (size_t)head * p.k_dim
                 : kind == 1 ? (size_t)(p.n_q_heads + head) * p.k_dim
                             : (size_t)(p.n_q_heads + p.n_kv_heads) * p.k_dim + (size_t)head * p.v_dim);
  const int e = 8 * lane;
  const bool mine = e < d;
  float x[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  if (mine) ld8<T>(src + e, x);       // asked for before the page is looked up

  T* dst;
  int zero_rows = 0;
  if (kind == 0) {
    dst = (T*)p.q_out + ((size_t)t * p.n_q_heads + head) * d;
  } else {
    const int pos = p.positions[t];
    const int r = p.tok_req[t];
    if (pos < 0) { if (lane == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
    if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    const int pidx = pos / p.page_size;
    const int slot = pos - pidx * p.page_size;
    const int page = (pidx < p.max_pages) ? p.block_table[(size_t)p.req_slot[r] * p.max_pages + pidx] : -1;
    if (page < 0 || page >= p.num_pages) { if (lane == 0) set_error(p.err, kErrPage, t, pidx, page); return; }
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + (((size_t)page * p.n_kv_heads + head) * p.page_size + slot) * d;
    if (p.req_kv_len != nullptr) {      // see the general kernel: the rest of a page begun in this step is cleared
      const int kv_len = p.req_kv_len[r], q_len = p.req_q_len[r];
      if (pos == kv_len - 1 && pos - slot >= kv_len - q_len) zero_rows = p.page_size - 1 - slot;
    }
  }
  if (mine) {
    const float zeros[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    for (int z = 1; z <= zero_rows; ++z) st8<T>(dst + (size_t)z * d + e, zeros);
  }

  if (kind == 2) {
    if (!mine) return;
    const size_t vo = ((size_t)t * p.n_kv_heads + head) * d + e;
    if (p.v_first_out != nullptr) st8<float>(p.v_first_out + vo, x);
    if (p.v_first_in != nullptr) {
      const float lam = *p.v_lambda;
      float f[8];
      ld8<float>(p.v_first_in + vo, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = (1.0f - lam) * x[i] + lam * f[i];
    }
    st8<T>(dst + e, x);
    return;
  }

  float ss = 0.0f;
  if (mine) {
    if (p.rope_table != nullptr && e < p.rotary_dim) {
      float cs[8];      // (cos, sin) of the lane's four pairs
      ld8<float>(reinterpret_cast<const float*>(p.rope_table + (size_t)t * (p.rotary_dim >> 1) + (e >> 1)), cs);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float u = x[2 * i], w = x[2 * i + 1];
        x[2 * i] = u * cs[2 * i] - w * cs[2 * i + 1];
        x[2 * i + 1] = w * cs[2 * i] + u * cs[2 * i + 1];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
  }
  if (p.unit_norm) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)d + p.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] *= rstd;
  }
  if (mine) st8<T>(dst + e, x);
}

}  // namespace tk

TK_API int tk_qkv_pairs(const void* qkv, const float* qkv_parts, int n_parts, void* q_out, void* k_cache,
                        void* v_cache, const int* positions, const int* tok_req, const int* req_slot,
                        const int* block_table, const int* req_q_len, const int* req_kv_len,
                        const float* rope_table, const float* v_first_in, const float* v_lambda,
                        float* v_first_out, int* err, int n_tokens, int n_reqs, int n_q_heads, int n_kv_heads,
                        int k_dim, int v_dim, int rotary_dim, int row_stride, int page_size, int max_pages,
                        int num_pages, int unit_norm, float eps, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (k_dim < 2 || k_dim % 2 || k_dim > 64 * tk::kPairsIter || v_dim < 2 || v_dim % 2 || rotary_dim < 0 ||
      rotary_dim % 2 || rotary_dim > k_dim || (rotary_dim > 0 && rope_table == nullptr) ||
      (v_first_in != nullptr && v_lambda == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::QkvPairsParams p;
  p.qkv = qkv; p.qkv_parts = qkv_parts; p.n_parts = n_parts; p.q_out = q_out; p.k_cache = k_cache;
  p.v_cache = v_cache; p.positions = positions; p.tok_req = tok_req; p.req_slot = req_slot;
  p.block_table = block_table; p.req_q_len = req_q_len; p.req_kv_len = req_kv_len;
  p.rope_table = (const float2*)rope_table; p.v_first_in = v_first_in; p.v_lambda = v_lambda;
  p.v_first_out = v_first_out; p.err = err; p.n_tokens = n_tokens; p.n_reqs = n_reqs;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.k_dim = k_dim; p.v_dim = v_dim;
  p.rotary_dim = rotary_dim; p.row_stride = row_stride; p.page_size = page_size; p.max_pages = max_pages;
  p.num_pages = num_pages; p.unit_norm = unit_norm; p.eps = eps;
  const int heads_total = n_q_heads + 2 * n_kv_heads;
  const int warps = 4;
  const int groups = (heads_total + warps - 1) / warps;
  if (groups > 65535) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  if (qkv_parts == nullptr && k_dim % 8 == 0 && v_dim % 8 == 0 && rotary_dim % 8 == 0 && v_dim <= 256 && row_stride % 8 == 0) {
    TK_DISPATCH_DTYPE(dtype, T,
                      e = tk::launch(tk::qkv_pairs_vec_kernel<T>, dim3((unsigned)n_tokens, (unsigned)groups),
                                     dim3(warps * 32), 0, stream, p));
    return (int)e;
  }
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::qkv_pairs_kernel<T>, dim3((unsigned)n_tokens, (unsigned)groups),
                                   dim3(warps * 32), 0, stream, p));
  return (int)e;
}
