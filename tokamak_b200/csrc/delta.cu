// Gated delta rule: a matrix-valued recurrent state per (request, head) that is decayed by one
// number per token and head and corrected, under the token's key, towards the token's value:
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          S: [key_dim, value_dim]
//
// and what feeds it.  q, k and v are columns of one stacked projection that pass a short causal
// convolution over time per channel (taps [channels, K], the last tap weighs the current token) and
// silu; q and k heads are then scaled to unit length, x / sqrt(sum(x^2) + eps), q also by q_scale;
// value head h reads q/k head h / (heads / kv_heads).  Per token and head, from two more columns,
//   beta = sigmoid(b),    g = exp(-exp(A_log[h]) * softplus(a + dt_bias[h])).
//
// A request's record in the state pool is  [ S: heads * key_dim * value_dim | tail: (K - 1) * channels ],
// float32: the state and the last K - 1 inputs of the convolution (oldest first; zeros for a request
// that has just begun).  Three kernels: delta_prepare_kernel (convolution, silu, unit norm, beta, g;
// float32 outputs), delta_tail_kernel (moves the convolution's tail on), delta_scan_kernel (the
// recurrence).  Everything but the stacked projection itself is float32 in every engine dtype.  A
// request's tokens are walked in order by the blocks that own its state with the same operations
// in the same order wherever a step begins, so a position's result does not depend on how the
// prompt was cut or on what else is in the batch.
#include "common.cuh"
#include "stacked_input.cuh"

namespace tk {

constexpr int kDeltaMaxTaps = 8;
constexpr int kDeltaPrepWarps = 4;

struct DeltaPrepareParams {
  StackedInput in;
  int q_off, k_off, v_off, b_off, a_off;   // first columns of the pieces of a row
  const float* taps;          // [channels, n_taps]: q channels, k channels, v channels
  const float* a_log;         // [heads]
  const float* dt_bias;       // [heads]
  float* state;               // the pool of records
  long long rec_stride;       // floats per record
  long long tail_off;         // where the tail starts inside a record
  const int* tok_req;
  const int* req_q_start;
  const int* req_slot;
  float* q_out;               // [n_tokens, kv_heads, key_dim]
  float* k_out;               // [n_tokens, kv_heads, key_dim]
  float* v_out;               // [n_tokens, heads, value_dim]
  float* beta_out;            // [n_tokens, heads]
  float* g_out;               // [n_tokens, heads]
  int* err;
  int n_tokens, n_reqs, n_slots, heads, kv_heads, dk, dv, n_taps;
  int move_tail;              // every request brings one token: the thread that reads a channel's tail also moves it on
  int per_warp;               // a warp a unit (many tokens) or a block a unit (few)
  float unit_eps, q_scale;
};

// One head unit of one token at a time; the units of a token are its q heads, its k heads, its v heads.
// Two shapes of the same arithmetic: with many tokens a warp takes a unit (lanes over the channels, 32 at a
// time), with few a whole block does (a thread a channel, so that the channels' loads of taps, inputs and
// tail wait for memory side by side instead of in turn).  The sum of squares of a q or k head is formed the
// same way in both: every aligned group of 32 channels by a warp's butterfly, the groups added in ascending
// order; a position's inputs are therefore the same bits whichever shape a step takes.
template <typename T>
__global__ void delta_prepare_kernel(DeltaPrepareParams p) {
  __shared__ float s_group[8];        // key_dim <= 256: at most 8 groups
  pdl_trigger();
  pdl_wait();
  const bool per_warp = p.per_warp != 0;
  const int lane = per_warp ? (threadIdx.x & 31) : threadIdx.x;         // place among the unit's threads
  const int stride = per_warp ? 32 : blockDim.x;
  const int t = blockIdx.x;
  const int unit = per_warp ? blockIdx.y * kDeltaPrepWarps + (threadIdx.x >> 5) : blockIdx.y;
  const int units = 2 * p.kv_heads + p.heads;
  if (unit >= units) return;          // whole warps of the last block of the per-warp shape
  int kind, head;      // 0 = q, 1 = k, 2 = v
  if (unit < p.kv_heads) { kind = 0; head = unit; }
  else if (unit < 2 * p.kv_heads) { kind = 1; head = unit - p.kv_heads; }
  else { kind = 2; head = unit - 2 * p.kv_heads; }
  const int d = kind == 2 ? p.dv : p.dk;
  const int hk = p.kv_heads * p.dk;
  const int chan0 = kind == 0 ? head * p.dk : kind == 1 ? hk + head * p.dk : 2 * hk + head * p.dv;
  const int col0 = kind == 0 ? p.q_off + head * p.dk : kind == 1 ? p.k_off + head * p.dk : p.v_off + head * p.dv;
  const int channels = 2 * hk + p.heads * p.dv;
  const int r = p.tok_req[t];
  if (r < 0 || r >= p.n_reqs) { if (lane == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  const int slot = p.req_slot[r];
  if (slot < 0 || slot >= p.n_slots) { if (lane == 0) set_error(p.err, kErrRequest, t, slot, p.n_slots); return; }
  const int i = t - p.req_q_start[r];          // place of the token among its request's tokens of this step
  float* tail = p.state + (size_t)slot * p.rec_stride + p.tail_off;
  const int K = p.n_taps;

  float* dst = kind == 0 ? p.q_out + ((size_t)t * p.kv_heads + head) * p.dk
             : kind == 1 ? p.k_out + ((size_t)t * p.kv_heads + head) * p.dk
                         : p.v_out + ((size_t)t * p.heads + head) * p.dv;
  // one channel: convolution over the step's rows and the tail, silu, the value stored; returns it
  auto channel = [&](int e) -> float {
    const float* w = p.taps + (size_t)(chan0 + e) * K;
    float acc = 0.0f;
    for (int j = 0; j < K; ++j) {
      const int s = i - (K - 1) + j;           // the input's place in this step; negative: before it
      const float x = s >= 0 ? stacked_ld<T>(p.in, (size_t)(t - i + s) * p.in.row_stride + col0 + e)
                             : tail[(size_t)(K - 1 + s) * channels + chan0 + e];
      acc += w[j] * x;
    }
    if (p.move_tail) {
      // the request's only token of this step: nobody else reads this channel's tail, which now ends with the token's input
      float* tc = tail + chan0 + e;
      for (int j = 0; j + 2 < K; ++j) tc[(size_t)j * channels] = tc[(size_t)(j + 1) * channels];
      if (K > 1) tc[(size_t)(K - 2) * channels] = stacked_ld<T>(p.in, (size_t)t * p.in.row_stride + col0 + e);
    }
    const float y = acc / (1.0f + expf(-acc));
    dst[e] = y;
    return y;
  };
  float ss = 0.0f;
  if (kind == 2) {
    for (int e = lane; e < d; e += stride) channel(e);
  } else if (per_warp) {
    // a q or k head has at most 8 groups of 32 channels: their sums of squares are formed after the loop, in order
    float sq[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int e = lane + 32 * it;
      sq[it] = 0.0f;
      if (e < d) { const float y = channel(e); sq[it] = y * y; }
    }
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      if (32 * it < d) ss += warp_sum(sq[it]);
    }
  } else {
    const int e = lane;                          // key_dim <= the block's threads: one round
    float y = 0.0f;
    if (e < d) y = channel(e);
    const float group = warp_sum(y * y);         // channels 32 g .. 32 g + 31, g = e / 32 (the same in a warp)
    if ((threadIdx.x & 31) == 0 && e < d) s_group[e >> 5] = group;
  }
  if (kind != 2) {
    if (!per_warp) {
      __syncthreads();       // kind and d are the block's: every thread comes here
      for (int gi = 0; gi < (d + 31) / 32; ++gi) ss += s_group[gi];
    }
    const float f = rsqrtf(ss + p.unit_eps) * (kind == 0 ? p.q_scale : 1.0f);
    for (int e = lane; e < d; e += stride) dst[e] *= f;     // each thread rescales what it wrote itself
  } else if (lane == 0) {
    const size_t row = (size_t)t * p.in.row_stride;
    const float b = stacked_ld<T>(p.in, row + p.b_off + head);
    const float a = stacked_ld<T>(p.in, row + p.a_off + head) + p.dt_bias[head];
    const float sp = a > 20.0f ? a : log1pf(expf(a));
    p.beta_out[(size_t)t * p.heads + head] = 1.0f / (1.0f + expf(-b));
    p.g_out[(size_t)t * p.heads + head] = expf(-expf(p.a_log[head]) * sp);
  }
}

// The record's tail after the step: the last K - 1 inputs of every channel.  One thread per
// (request, channel) reads what it needs of the old tail before it writes.
template <typename T>
__global__ void delta_tail_kernel(StackedInput in, int q_off, int k_off, int v_off, float* __restrict__ state,
                                  long long rec_stride, long long tail_off, const int* __restrict__ req_q_start,
                                  const int* __restrict__ req_q_len, const int* __restrict__ req_slot, int n_slots,
                                  int hk, int hv, int n_taps) {
  pdl_trigger();
  pdl_wait();
  const int channels = 2 * hk + hv;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= channels) return;
  const int slot = req_slot[r];
  if (slot < 0 || slot >= n_slots) return;            // reported by the kernel before
  const int col = c < hk ? q_off + c : c < 2 * hk ? k_off + (c - hk) : v_off + (c - 2 * hk);
  const int n = req_q_len[r], t0 = req_q_start[r];
  float* tail = state + (size_t)slot * rec_stride + tail_off;
  const int K = n_taps;
  float keep[kDeltaMaxTaps];
#pragma unroll
  for (int j = 0; j < kDeltaMaxTaps - 1; ++j) {
    if (j < K - 1) {
      const int s = n - (K - 1) + j;
      keep[j] = s >= 0 ? stacked_ld<T>(in, (size_t)(t0 + s) * in.row_stride + col) : tail[(size_t)(K - 1 + s) * channels + c];
    }
  }
#pragma unroll
  for (int j = 0; j < kDeltaMaxTaps - 1; ++j) {
    if (j < K - 1) tail[(size_t)j * channels + c] = keep[j];
  }
}

constexpr int kDeltaWarps = 8;
constexpr int kDeltaBatch = 8;       // tokens staged in shared memory at a time (one per warp for the k.q products)

struct DeltaScanParams {
  const float* q;     // [n_tokens, kv_heads, dk]
  const float* k;
  const float* v;     // [n_tokens, heads, dv]
  const float* beta;  // [n_tokens, heads]
  const float* g;
  float* state;       // records; S of head h at h * dk * dv, row-major [dk, dv]
  long long rec_stride;
  float* out;         // [n_tokens, heads, dv]
  const int* req_q_start;
  const int* req_q_len;
  const int* req_slot;
  int* err;
  int n_reqs, n_slots, heads, kv_heads, dk, dv;
};

__device__ __forceinline__ void cp_async16f(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}

// One block per (request, head, kDeltaWarps * 2 kCP value channels); every warp owns kCP pairs of
// neighbouring columns of the state for itself: lane -> (pair = lane % kCP, row group = lane / kCP), a
// thread keeps kRows rows of its two columns in registers as float2, so that every multiply-add is one
// packed instruction on both columns and a row's k and q are loaded once for the two.  Per token every
// thread forms its share of S^T k and S^T q from the decayed state, the shares of a column meet over
// shuffles inside the warp (a fixed order), and since
//   o = (g S + k u^T)^T q = (g S)^T q + u (k . q)
// one meeting per token is enough.  No barrier stands between two tokens: the warps of a block only
// share the staging of the inputs, which come in batches of kDeltaBatch tokens through shared memory,
// the next batch on its way (cp.async) while this one is worked through.
template <int kCP, int kRows>
__global__ void __launch_bounds__(kDeltaWarps * 32) delta_scan_kernel(DeltaScanParams p) {
  constexpr int kGroups = 32 / kCP;                    // row groups of a warp
  constexpr int kRowsAll = kGroups * kRows;            // rows a warp can hold (>= dk)
  constexpr int kCols = kDeltaWarps * 2 * kCP;         // columns of a block
  __shared__ __align__(16) float s_q[2][kDeltaBatch][kRowsAll];
  __shared__ __align__(16) float s_k[2][kDeltaBatch][kRowsAll];
  __shared__ __align__(8) float s_v[2][kDeltaBatch][kCols];
  __shared__ float s_beta[2][kDeltaBatch], s_g[2][kDeltaBatch], s_kq[2][kDeltaBatch];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = lane % kCP, sub = lane / kCP;
  const int row0 = sub * kRows;
  const int r = blockIdx.z, h = blockIdx.y;
  const int c0 = blockIdx.x * kCols;
  const int bcol = 2 * (warp * kCP + pair);            // this thread's first column within the block
  const int hk = h / (p.heads / p.kv_heads);
  const int n = p.req_q_len[r], t0 = p.req_q_start[r];
  const int slot = p.req_slot[r];
  if (slot < 0 || slot >= p.n_slots) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, r, slot, p.n_slots); return; }
  const int dk = p.dk, dv = p.dv;
  const bool ok0 = c0 + bcol < dv, ok1 = c0 + bcol + 1 < dv;
  float* S = p.state + (size_t)slot * p.rec_stride + (size_t)h * dk * dv + c0 + bcol;

  float2 st[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const bool row_ok = row0 + i < dk;
    st[i].x = (ok0 && row_ok) ? S[(size_t)(row0 + i) * dv] : 0.0f;
    st[i].y = (ok1 && row_ok) ? S[(size_t)(row0 + i) * dv + 1] : 0.0f;
  }
  // rows beyond dk read q = k = 0 from shared memory and stay zero; so do columns beyond dv (v = 0)
  for (int e = threadIdx.x; e < 2 * kDeltaBatch * kRowsAll; e += blockDim.x) {
    (&s_q[0][0][0])[e] = 0.0f;
    (&s_k[0][0][0])[e] = 0.0f;
  }
  for (int e = threadIdx.x; e < 2 * kDeltaBatch * kCols; e += blockDim.x) (&s_v[0][0][0])[e] = 0.0f;
  __syncthreads();

  // q and k rows in 16-byte pieces where the rows allow it (key_dim a multiple of 4, the arrays aligned)
  const bool vec = (dk & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k)) & 15) == 0;
  auto stage = [&](int b0, int buf) {
    const int cnt = min(kDeltaBatch, n - b0);
    if (vec) {
      const int quads = dk >> 2;
      for (int e = threadIdx.x; e < cnt * quads; e += blockDim.x) {
        const int i = e / quads, x = (e - i * quads) * 4;
        const size_t src = ((size_t)(t0 + b0 + i) * p.kv_heads + hk) * dk + x;
        cp_async16f(&s_q[buf][i][x], p.q + src);
        cp_async16f(&s_k[buf][i][x], p.k + src);
      }
    } else {
      for (int e = threadIdx.x; e < cnt * dk; e += blockDim.x) {
        const int i = e / dk, x = e - i * dk;
        const size_t src = ((size_t)(t0 + b0 + i) * p.kv_heads + hk) * dk + x;
        cp_async4(&s_q[buf][i][x], p.q + src);
        cp_async4(&s_k[buf][i][x], p.k + src);
      }
    }
    for (int e = threadIdx.x; e < cnt * kCols; e += blockDim.x) {
      const int i = e / kCols, x = e - i * kCols;
      if (c0 + x < dv) cp_async4(&s_v[buf][i][x], p.v + ((size_t)(t0 + b0 + i) * p.heads + h) * dv + c0 + x);
    }
    if (threadIdx.x < cnt) {
      cp_async4(&s_beta[buf][threadIdx.x], p.beta + (size_t)(t0 + b0 + threadIdx.x) * p.heads + h);
      cp_async4(&s_g[buf][threadIdx.x], p.g + (size_t)(t0 + b0 + threadIdx.x) * p.heads + h);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  if (n > 0) stage(0, 0);
  for (int b0 = 0, buf = 0; b0 < n; b0 += kDeltaBatch, buf ^= 1) {
    const int cnt = min(kDeltaBatch, n - b0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();          // this batch is there, and every warp has left the buffer that is staged next
    if (b0 + kDeltaBatch < n) stage(b0 + kDeltaBatch, buf ^ 1);
    // k . q of every staged token: one warp a token, lanes over the rows, added in a fixed order
    if (warp < cnt) {
      float d = 0.0f;
      for (int x = lane; x < dk; x += 32) d += s_k[buf][warp][x] * s_q[buf][warp][x];
      d = warp_sum(d);
      if (lane == 0) s_kq[buf][warp] = d;
    }
    __syncthreads();
    const float* kq_row = &s_k[buf][0][row0];
    const float* qq_row = &s_q[buf][0][row0];
    float* out_row = p.out + ((size_t)(t0 + b0) * p.heads + h) * dv + c0 + bcol;
#pragma unroll 4
    for (int i = 0; i < cnt; ++i, kq_row += kRowsAll, qq_row += kRowsAll, out_row += (size_t)p.heads * dv) {
      const float gt = s_g[buf][i];
      const float2 g2 = make_float2(gt, gt);
      float2 kk[kRows];
      float2 a2 = make_float2(0.0f, 0.0f), b2 = a2, a3 = a2, b3 = a2;
#pragma unroll
      for (int x = 0; x < kRows; x += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kq_row + x);
        const float4 q4 = *reinterpret_cast<const float4*>(qq_row + x);
        kk[x] = make_float2(k4.x, k4.x); kk[x + 1] = make_float2(k4.y, k4.y);
        kk[x + 2] = make_float2(k4.z, k4.z); kk[x + 3] = make_float2(k4.w, k4.w);
        st[x] = mul2(st[x], g2); st[x + 1] = mul2(st[x + 1], g2);
        st[x + 2] = mul2(st[x + 2], g2); st[x + 3] = mul2(st[x + 3], g2);
        a2 = fma2(st[x], kk[x], a2); a3 = fma2(st[x + 1], kk[x + 1], a3);
        a2 = fma2(st[x + 2], kk[x + 2], a2); a3 = fma2(st[x + 3], kk[x + 3], a3);
        b2 = fma2(st[x], make_float2(q4.x, q4.x), b2); b3 = fma2(st[x + 1], make_float2(q4.y, q4.y), b3);
        b2 = fma2(st[x + 2], make_float2(q4.z, q4.z), b2); b3 = fma2(st[x + 3], make_float2(q4.w, q4.w), b3);
      }
      a2 = add2(a2, a3); b2 = add2(b2, b3);
#pragma unroll
      for (int off = kCP; off < 32; off <<= 1) {
        const float2 ao = make_float2(__shfl_xor_sync(0xffffffffu, a2.x, off), __shfl_xor_sync(0xffffffffu, a2.y, off));
        const float2 bo = make_float2(__shfl_xor_sync(0xffffffffu, b2.x, off), __shfl_xor_sync(0xffffffffu, b2.y, off));
        a2 = add2(a2, ao); b2 = add2(b2, bo);
      }
      const float bt = s_beta[buf][i];
      const float2 v2 = *reinterpret_cast<const float2*>(&s_v[buf][i][bcol]);
      const float2 u2 = make_float2(bt * (v2.x - a2.x), bt * (v2.y - a2.y));
#pragma unroll
      for (int x = 0; x < kRows; ++x) st[x] = fma2(kk[x], u2, st[x]);
      if (sub == 0) {
        const float kq = s_kq[buf][i];
        if (ok0) out_row[0] = b2.x + u2.x * kq;
        if (ok1) out_row[1] = b2.y + u2.y * kq;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    if (row0 + i < dk) {
      if (ok0) S[(size_t)(row0 + i) * dv] = st[i].x;
      if (ok1) S[(size_t)(row0 + i) * dv + 1] = st[i].y;
    }
  }
}

}  // namespace tk

TK_API int tk_delta_prepare(const void* x, const float* parts, int n_parts, long long part_stride, int row_stride,
                            int q_off, int k_off, int v_off, int b_off, int a_off, const float* taps,
                            const float* a_log, const float* dt_bias, float* state, long long rec_stride,
                            long long tail_off, const int* tok_req, const int* req_q_start, const int* req_q_len,
                            const int* req_slot, float* q_out, float* k_out, float* v_out, float* beta_out,
                            float* g_out, int* err, int n_tokens, int n_reqs, int n_slots, int heads, int kv_heads,
                            int dk, int dv, int n_taps, float unit_eps, float q_scale, int dtype, int move_tail_in_place,
                            int shape, cudaStream_t stream) {
  // move_tail_in_place: the caller vouches that every request brings at least one token, so that as many
  // tokens as requests means one token each; the kernel of the inputs then moves the tails on itself
  if (n_tokens <= 0 || n_reqs <= 0) return 0;
  if ((x == nullptr) == (parts == nullptr) || heads < 1 || kv_heads < 1 || heads % kv_heads || dk < 1 || dv < 1 ||
      n_taps < 1 || n_taps > tk::kDeltaMaxTaps || n_reqs > 65535) {
    return (int)cudaErrorInvalidValue;
  }
  tk::DeltaPrepareParams p;
  p.in.x = x; p.in.parts = parts; p.in.n_parts = n_parts; p.in.row_stride = row_stride; p.in.part_stride = part_stride;
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.b_off = b_off; p.a_off = a_off;
  p.taps = taps; p.a_log = a_log; p.dt_bias = dt_bias; p.state = state; p.rec_stride = rec_stride; p.tail_off = tail_off;
  p.tok_req = tok_req; p.req_q_start = req_q_start; p.req_slot = req_slot;
  p.q_out = q_out; p.k_out = k_out; p.v_out = v_out; p.beta_out = beta_out; p.g_out = g_out; p.err = err;
  p.n_tokens = n_tokens; p.n_reqs = n_reqs; p.n_slots = n_slots; p.heads = heads; p.kv_heads = kv_heads;
  p.dk = dk; p.dv = dv; p.n_taps = n_taps; p.unit_eps = unit_eps; p.q_scale = q_scale;
  p.move_tail = (n_tokens == n_reqs && move_tail_in_place) ? 1 : 0;
  const int units = 2 * kv_heads + heads;
  if (units > 65535 || dk > 256) return (int)cudaErrorInvalidValue;
  const int widest = dk > dv ? dk : dv;
  // few tokens: a block a unit, so that a step of single tokens is one memory latency long; many: a warp a unit
  // (shape 1 / 2: the caller's choice, for tests and measurements; both give the same bits)
  p.per_warp = shape == 1 ? 1 : shape == 2 ? 0 : ((long long)n_tokens * units >= 4096 ? 1 : 0);
  const int threads = p.per_warp ? tk::kDeltaPrepWarps * 32 : (widest >= 256 ? 256 : (widest + 31) / 32 * 32);
  dim3 grid(n_tokens, p.per_warp ? (units + tk::kDeltaPrepWarps - 1) / tk::kDeltaPrepWarps : units);
  cudaError_t e = cudaSuccess;
  TK_DISPATCH_DTYPE(dtype, T, e = tk::launch(tk::delta_prepare_kernel<T>, grid, dim3(threads), 0, stream, p));
  if (e != cudaSuccess || n_taps == 1 || p.move_tail) return (int)e;
  const int hk = kv_heads * dk, hv = heads * dv;
  dim3 tgrid((2 * hk + hv + 127) / 128, n_reqs);
  TK_DISPATCH_DTYPE(dtype, T,
                    e = tk::launch(tk::delta_tail_kernel<T>, tgrid, dim3(128), 0, stream, p.in, q_off, k_off, v_off,
                                   state, rec_stride, tail_off, req_q_start, req_q_len, req_slot, n_slots, hk, hv,
                                   n_taps));
  return (int)e;
}

// Columns of the state that one block takes (8 warps of 1, 2 or 4 pairs of columns each): fewer where
// the heads alone would leave the SMs' schedulers without a warp, and never so many that a thread would
// hold more than 32 rows.  It follows from the model's sizes only, never from the batch, so that a
// position's sums are always added in the same order.
TK_API int tk_delta_scan_cols(int heads, int dk, int dv) {
  int cp = 4;
  while (cp > 1 && ((long long)heads * dv / (2 * cp) < 500 || dk * cp / 32 > 32)) cp /= 2;
  return 2 * cp * tk::kDeltaWarps;
}

TK_API int tk_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* g,
                         float* state, long long rec_stride, float* out, const int* req_q_start,
                         const int* req_q_len, const int* req_slot, int* err, int n_reqs, int n_slots, int heads,
                         int kv_heads, int dk, int dv, int cols, cudaStream_t stream) {
  if (n_reqs <= 0) return 0;
  if (cols <= 0) cols = tk_delta_scan_cols(heads, dk, dv);
  if (heads < 1 || kv_heads < 1 || heads % kv_heads || heads > 65535 || n_reqs > 65535 ||
      (cols != 64 && cols != 32 && cols != 16)) {
    return (int)cudaErrorInvalidValue;
  }
  if (dk < 1 || dk > 256) return (int)cudaErrorInvalidValue;      // a warp holds 256 key channels at most
  const int cp = cols / (2 * tk::kDeltaWarps);
  const int groups = 32 / cp;
  const int rows = (dk + groups - 1) / groups;
  tk::DeltaScanParams p;
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.g = g; p.state = state; p.rec_stride = rec_stride; p.out = out;
  p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.req_slot = req_slot; p.err = err;
  p.n_reqs = n_reqs; p.n_slots = n_slots; p.heads = heads; p.kv_heads = kv_heads; p.dk = dk; p.dv = dv;
  dim3 grid((dv + cols - 1) / cols, heads, n_reqs);
  dim3 block(tk::kDeltaWarps * 32);
  cudaError_t e = cudaSuccess;
  // only the shapes that 256 key channels need are built
#define TK_DELTA_LAUNCH(C, R) e = tk::launch(tk::delta_scan_kernel<C, R>, grid, block, 0, stream, p)
  if (cp == 4) {
    if (rows <= 4) TK_DELTA_LAUNCH(4, 4); else if (rows <= 8) TK_DELTA_LAUNCH(4, 8);
    else if (rows <= 16) TK_DELTA_LAUNCH(4, 16); else TK_DELTA_LAUNCH(4, 32);
  } else if (cp == 2) {
    if (rows <= 4) TK_DELTA_LAUNCH(2, 4); else if (rows <= 8) TK_DELTA_LAUNCH(2, 8); else TK_DELTA_LAUNCH(2, 16);
  } else {
    if (rows <= 4) TK_DELTA_LAUNCH(1, 4); else TK_DELTA_LAUNCH(1, 8);
  }
#undef TK_DELTA_LAUNCH
  return (int)e;
}
