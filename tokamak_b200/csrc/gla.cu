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
#include "mma_utils.cuh"

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

// What the recurrence reads, float32 whatever the engine's dtype: a row per (token, head) of
//   q * q_scale [dks] | k [dks] | alpha [dks] | v [dvs]
// with dks = key_dim and dvs = value_dim rounded up to a multiple of 4 (16 bytes), the padding zero,
// and alpha = sigmoid(sum_j a[t, j] w2[c, j] + bias[c]) ^ (1 / tau), computed through its logarithm
// log(sigmoid(z)) = min(z, 0) - log1p(exp(-|z|)).  One thread per element.
template <typename T>
__global__ void gla_prepare_kernel(GlaInput in, int q_off, int k_off, int v_off, int a_off, const T* __restrict__ w2,
                                   const float* __restrict__ bias, float* __restrict__ prep, int n_tokens, int heads,
                                   int dk, int dv, int dks, int dvs, int rank, float inv_tau, float q_scale) {
  pdl_trigger();
  pdl_wait();
  const int per = dks + dvs;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * heads * per) return;
  const long long th = idx / per;
  const int e = (int)(idx - th * per);
  const int t = (int)(th / heads), h = (int)(th - (long long)t * heads);
  const size_t row = (size_t)t * in.row_stride;
  float* out = prep + (size_t)th * (3 * dks + dvs);
  if (e >= dks) {
    const int c = e - dks;
    out[3 * dks + c] = c < dv ? gla_ld<T>(in, row + v_off + h * dv + c) : 0.0f;
    return;
  }
  if (e >= dk) { out[e] = 0.0f; out[dks + e] = 0.0f; out[2 * dks + e] = 0.0f; return; }
  const int ch = h * dk + e;
  float z = 0.0f;
  for (int j = 0; j < rank; ++j) z += gla_ld<T>(in, row + a_off + j) * to_f32<T>(w2[(size_t)ch * rank + j]);
  if (bias != nullptr) z += bias[ch];
  out[e] = gla_ld<T>(in, row + q_off + ch) * q_scale;
  out[dks + e] = gla_ld<T>(in, row + k_off + ch);
  out[2 * dks + e] = expf((fminf(z, 0.0f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

constexpr int kGlaRows = 8;       // rows of the state (key channels) that one thread keeps in registers
constexpr int kGlaBatch = 32;     // tokens staged in shared memory at a time, times the row groups of a warp
constexpr int kGlaMaxWarps = 16;  // warps of a block
constexpr int kGlaMaxKey = 256;   // key_dim: 16 warps of 16 rows at 16 columns a block; at 32 columns a block 128

struct GlaScanParams {
  const float* prep;        // [n_tokens, heads, 3 dks + dvs], see gla_prepare_kernel
  float* state;             // [n_slots, heads, key_dim, value_dim]
  float* out;               // [n_tokens, heads, value_dim]
  const int* req_q_start;
  const int* req_q_len;
  const int* req_slot;
  int* err;
  int n_tokens, n_slots, heads, key_dim, value_dim, dks, dvs;
};

// One block per (request, head, kCols value channels).  A warp's lanes are kCols columns times
// 32 / kCols groups of eight rows; a thread keeps its eight rows of one column of the state in
// registers and walks the request's tokens in order.  The host picks kCols so that the grid covers
// the SMs: a prompt alone has only heads * value_dim columns to share out.  Tokens are staged a
// batch at a time by asynchronous 16-byte copies into one of two buffers in shared memory: while
// one batch is worked through, the next is on its way (the chain of tokens is what bounds a
// prompt, so no load may stand in it).  A token's output is the sum of the eight-row groups'
// partial sums in the order of the rows, whatever kCols is, so the result does not depend on the
// split.
template <int kCols>
__global__ void __launch_bounds__(kGlaMaxWarps * 32, 1) gla_scan_kernel(GlaScanParams p) {
  constexpr int kGroups = 32 / kCols;               // row groups of a warp
  constexpr int kBatch = kGlaBatch / kGroups;       // tokens of a batch
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int col = lane % kCols, group = warp * kGroups + lane / kCols, n_groups = n_warps * kGroups;
  const int dkp = n_groups * kGlaRows;                      // a staged row: key channels, padded with zeros
  const int per_buf = 3 * kBatch * dkp + kBatch * kCols;    // q, k, alpha [kBatch][dkp] and v [kBatch][kCols]
  float* so = smem + 2 * per_buf;                           // partial outputs [kBatch][n_groups][kCols]
  for (int i = threadIdx.x; i < 2 * per_buf; i += blockDim.x) smem[i] = 0.0f;
  __syncthreads();
  pdl_wait();
  const int dk = p.key_dim, dv = p.value_dim;
  const int slot = p.req_slot[r];
  const int q0 = p.req_q_start[r], n = p.req_q_len[r];
  if (slot < 0 || slot >= p.n_slots || q0 < 0 || n < 0 || q0 + n > p.n_tokens) {
    if (threadIdx.x == 0) set_error(p.err, kErrRequest, r, slot, q0);
    return;
  }
  const int j = j0 + col;
  float* srow = p.state + (((size_t)slot * p.heads + h) * dk + (size_t)group * kGlaRows) * dv + j;
  float2 s[kGlaRows / 2];       // rows in pairs: two multiply-adds an instruction
#pragma unroll
  for (int ii = 0; ii < kGlaRows; ++ii) {
    const float v0 = (j < dv && group * kGlaRows + ii < dk) ? srow[(size_t)ii * dv] : 0.0f;
    if (ii & 1) s[ii / 2].y = v0; else s[ii / 2].x = v0;
  }

  // A warp copies the tokens warp, warp + n_warps, ... of a batch, a lane 16 bytes at a time.
  const int prep_row = 3 * p.dks + p.dvs, chunks = p.dks / 4;
  auto copy = [&](int t0, float* buf) {
    const int nb = min(kBatch, n - t0);
    for (int tb = warp; tb < nb; tb += n_warps) {
      const float* src = p.prep + ((size_t)(q0 + t0 + tb) * p.heads + h) * prep_row;
      for (int c = lane; c < chunks; c += 32) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
          cp_async16(smem_u32(buf + (a * kBatch + tb) * dkp + 4 * c), src + a * p.dks + 4 * c, true);
        }
      }
      if (lane < kCols / 4) {
        const bool live = j0 + 4 * lane < p.dvs;
        cp_async16(smem_u32(buf + 3 * kBatch * dkp + tb * kCols + 4 * lane), src + 3 * p.dks + (live ? j0 + 4 * lane : 0), live);
      }
    }
    cp_async_commit();
  };

  if (n > 0) copy(0, smem);
  int cur = 0;
  for (int t0 = 0; t0 < n; t0 += kBatch) {
    const int nb = min(kBatch, n - t0);
    const float* buf = smem + cur * per_buf;
    cp_async_wait<0>();
    __syncthreads();          // this batch has landed; everyone is done with the other buffer and with so
    if (t0 + kBatch < n) copy(t0 + kBatch, smem + (cur ^ 1) * per_buf);
    const float* sq = buf + group * kGlaRows; const float* sk = sq + kBatch * dkp; const float* sa = sk + kBatch * dkp;
    const float* sv = buf + 3 * kBatch * dkp + col;
    // One token: its q, k and decays come from registers that were loaded while the token before was
    // worked on (the loads of shared memory would otherwise stand in the chain of tokens), and the next
    // token's are loaded first of all.
    float4 q[kGlaRows / 4], k[kGlaRows / 4], a[kGlaRows / 4];
    float v;
    auto load = [&](int tb) {
      v = sv[tb * kCols];
#pragma unroll
      for (int g = 0; g < kGlaRows / 4; ++g) {
        q[g] = reinterpret_cast<const float4*>(sq + tb * dkp)[g];
        k[g] = reinterpret_cast<const float4*>(sk + tb * dkp)[g];
        a[g] = reinterpret_cast<const float4*>(sa + tb * dkp)[g];
      }
    };
    auto token = [&](int tb, bool more) {
      float4 qc[kGlaRows / 4], kc[kGlaRows / 4], ac[kGlaRows / 4];
      const float vc = v;
#pragma unroll
      for (int g = 0; g < kGlaRows / 4; ++g) { qc[g] = q[g]; kc[g] = k[g]; ac[g] = a[g]; }
      if (more) load(tb + 1);
      const float2 v2 = make_float2(vc, vc);
      float2 o01 = make_float2(0.0f, 0.0f), o23 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int g = 0; g < kGlaRows / 4; ++g) {
        s[2 * g] = fma2(make_float2(ac[g].x, ac[g].y), s[2 * g], mul2(make_float2(kc[g].x, kc[g].y), v2));
        s[2 * g + 1] = fma2(make_float2(ac[g].z, ac[g].w), s[2 * g + 1], mul2(make_float2(kc[g].z, kc[g].w), v2));
        o01 = fma2(make_float2(qc[g].x, qc[g].y), s[2 * g], o01);
        o23 = fma2(make_float2(qc[g].z, qc[g].w), s[2 * g + 1], o23);
      }
      so[(tb * n_groups + group) * kCols + col] = (o01.x + o01.y) + (o23.x + o23.y);
    };
    load(0);
    if (nb == kBatch) {       // a full batch: a loop of known length
#pragma unroll 4
      for (int tb = 0; tb < kBatch; ++tb) token(tb, tb + 1 < kBatch);
    } else {
      for (int tb = 0; tb < nb; ++tb) token(tb, tb + 1 < nb);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nb * kCols; idx += blockDim.x) {
      const int tb = idx / kCols, c = idx % kCols;
      if (j0 + c >= dv) continue;
      float o = 0.0f;
      for (int w = 0; w < n_groups; ++w) o += so[(tb * n_groups + w) * kCols + c];
      p.out[((size_t)(q0 + t0 + tb) * p.heads + h) * dv + j0 + c] = o;
    }
    cur ^= 1;
  }
#pragma unroll
  for (int ii = 0; ii < kGlaRows; ++ii) {
    if (j < dv && group * kGlaRows + ii < dk) srow[(size_t)ii * dv] = (ii & 1) ? s[ii / 2].y : s[ii / 2].x;
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

// prep: float32 [n_tokens, heads, 3 dks + dvs] with dks, dvs = key_dim, value_dim rounded up to a multiple of 4.
TK_API int tk_gla_prepare(const void* x, const float* parts, int n_parts, int row_stride, int q_off, int k_off,
                          int v_off, int a_off, const void* w2, const float* bias, float* prep, int n_tokens,
                          int heads, int key_dim, int value_dim, int rank, float tau, float q_scale, int dtype,
                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads < 1 || key_dim < 1 || value_dim < 1 || rank < 1 || !(tau > 0.0f) || (x == nullptr) == (parts == nullptr)) {
    return (int)cudaErrorInvalidValue;
  }
  const int dks = (key_dim + 3) / 4 * 4, dvs = (value_dim + 3) / 4 * 4;
  const long long total = (long long)n_tokens * heads * (dks + dvs);
  const tk::GlaInput in = gla_input(x, parts, n_parts, n_tokens, row_stride);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::gla_prepare_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                   in, q_off, k_off, v_off, a_off, (const T*)w2, bias, prep, n_tokens, heads, key_dim,
                                   value_dim, dks, dvs, rank, 1.0f / tau, q_scale));
  return (int)e;
}

template <int kCols>
static cudaError_t gla_scan_launch(const tk::GlaScanParams& p, int n_reqs, cudaStream_t stream) {
  constexpr int kGroups = 32 / kCols, kBatch = tk::kGlaBatch / kGroups;
  const int n_warps = (p.key_dim + tk::kGlaRows * kGroups - 1) / (tk::kGlaRows * kGroups);
  const int n_groups = n_warps * kGroups, dkp = n_groups * tk::kGlaRows;
  const int col_tiles = (p.value_dim + kCols - 1) / kCols;
  if (n_warps > tk::kGlaMaxWarps || col_tiles > 65535) return cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (2 * ((size_t)3 * kBatch * dkp + kBatch * kCols) + (size_t)kBatch * n_groups * kCols);
  cudaError_t e = cudaSuccess;
  if (smem > 48 * 1024) {
    e = cudaFuncSetAttribute(tk::gla_scan_kernel<kCols>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return tk::launch(tk::gla_scan_kernel<kCols>, dim3((unsigned)n_reqs, (unsigned)p.heads, (unsigned)col_tiles),
                    dim3(n_warps * 32), smem, stream, p);
}

static int gla_sm_count() {
  static int sm_count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 0;
  if (sms == 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) sm_count[dev] = sms;
  }
  return sms;
}

// cols: value channels per block (32, 16 or 8), or 0 for the widest split whose grid still has a block
// for every SM.
TK_API int tk_gla_scan(const float* prep, float* state, float* out, const int* req_q_start, const int* req_q_len,
                       const int* req_slot, int* err, int n_tokens, int n_reqs, int n_slots, int heads, int key_dim,
                       int value_dim, int cols, cudaStream_t stream) {
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  if (key_dim < 1 || key_dim > tk::kGlaMaxKey || value_dim < 1 || heads < 1 || heads > 65535 || prep == nullptr ||
      (cols != 0 && cols != 8 && cols != 16 && cols != 32)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::GlaScanParams p;
  p.prep = prep; p.state = state; p.out = out;
  p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_slot = req_slot; p.err = err;
  p.n_tokens = n_tokens; p.n_slots = n_slots; p.heads = heads; p.key_dim = key_dim; p.value_dim = value_dim;
  p.dks = (key_dim + 3) / 4 * 4; p.dvs = (value_dim + 3) / 4 * 4;
  if (cols == 0) {
    const long long sms = gla_sm_count();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    const long long columns = (long long)n_reqs * heads * value_dim;
    cols = columns >= 32 * sms ? 32 : columns >= 16 * sms ? 16 : 8;
  }
  if (cols == 32 && key_dim > tk::kGlaMaxWarps * tk::kGlaRows) cols = 16;     // eight rows a warp: 128 rows a block
  const cudaError_t e = cols == 32 ? gla_scan_launch<32>(p, n_reqs, stream)
                        : cols == 16 ? gla_scan_launch<16>(p, n_reqs, stream) : gla_scan_launch<8>(p, n_reqs, stream);
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
