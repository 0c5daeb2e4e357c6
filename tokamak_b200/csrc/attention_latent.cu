// Attention over a latent cache on the tensor cores (bfloat16 pages, mma.sync m16n8k16).
//
// All query heads of a token read the same cache rows [c | k_rot] (one "head" of D elements a
// position) and their values are the rows' leading DV elements, so the heads of a token are stacked
// as rows of one query tile: row R of a tile is (token R / H, head R % H), and a tile of keys is
// loaded once for all of them, as keys and as values.
//
// One block = 64 query rows x a range of 64-key tiles.  Eight warps: warp w owns the query rows
// 16 (w % 4) .. + 15 and one half (w / 4) of the value columns; both halves form the scores of their
// rows (the score product is the smaller one: D against DV columns a key), then each multiplies the
// probabilities into its own columns.  Key tiles come page by page through cp.async into a double
// buffer; the queries are converted to bfloat16 into shared memory once.  Scores, running maximum,
// normaliser and the output accumulators are float32.  Keys outside the rows' visible range are
// zero-filled instead of loaded and masked in the scores.
//
// Two work lists.  Prompt portions: (request, 64-token tile) pairs as the step lays them out; block
// y = j of a pair takes rows 64 j .. of the tile's tokens x H rows and every key tile they see, and
// writes the output.  Single tokens: block (item, split) takes the H rows of the token and an equal
// share of its key tiles and writes float32 partial results (maximum, normaliser, unnormalised sums);
// latent_merge_kernel adds the shares up, in their order, together with the sink.  With one split the
// output is written directly.
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

namespace tk {

constexpr int kLaWarps = 8;
constexpr int kLaRows = 64;      // query rows of a block
constexpr int kLaKeys = 64;      // keys of a tile

struct LatentAttnParams {
  const void* q;                 // element (t, h, e) at t * q_tok_stride + h * q_head_stride + e
  __nv_bfloat16* out;            // [n_tokens, H, DV]
  const __nv_bfloat16* cache;    // [num_pages, 1, page_size, D]
  const float* sinks;            // [H] or null
  const int* tiles;              // prompt portions: [n, 2] (request row, 64-token tile); else null
  const int* items;              // single tokens: [n] token indices; else null
  const int* positions;
  const int* tok_req;
  const int* req_q_start;
  const int* req_q_len;
  const int* req_kv_len;
  const int* req_slot;
  const int* block_table;
  float* part_o;                 // [n_items, H, n_splits, DV] float32, or null (direct output)
  float* part_ml;                // [n_items, H, n_splits, 2]: maximum (log2 units), normaliser
  int* err;
  long long q_tok_stride, q_head_stride;
  int n_work, n_reqs, H, D, DV, page_size, max_pages, num_pages, window, n_splits;
  float scale_log2;
};

// Byte offset of the 16-byte chunk `chunk` of row `row`: rows are padded by one chunk, so that with an
// even number of chunks a row the eight rows of an ldmatrix fall into different banks.
__device__ __forceinline__ int la_offset(int row, int chunk, int chunks) { return (row * (chunks + 1) + chunk) * 16; }

template <typename TQ, int kPairs>     // kPairs: pairs of 8-column tiles of the values that one warp accumulates
__global__ void __launch_bounds__(kLaWarps * 32, 1) latent_attention_kernel(LatentAttnParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  const int D = p.D, DV = p.DV, H = p.H;
  const int CH = D / 8;
  const int tile_bytes = kLaKeys * (CH + 1) * 16;
  const uint32_t q_base = smem_u32(smem);
  const uint32_t k_base0 = q_base + kLaRows * (CH + 1) * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int rg = warp & 3, half = warp >> 2;

  // ---- what this block works on
  int tok0, pos0, rows_total, row_first, slot, split = 0, work = blockIdx.x;
  if (p.tiles != nullptr) {
    const int r = p.tiles[2 * work], ti = p.tiles[2 * work + 1];
    if (r < 0 || r >= p.n_reqs) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, work, r, p.n_reqs); return; }
    const int q_len = p.req_q_len[r], kv_len = p.req_kv_len[r];
    const int tokens = min(64, q_len - ti * 64);
    if (tokens <= 0 || kv_len < q_len) { if (threadIdx.x == 0) set_error(p.err, kErrPosition, work, q_len, kv_len); return; }
    tok0 = p.req_q_start[r] + ti * 64;
    pos0 = kv_len - q_len + ti * 64;
    rows_total = tokens * H;
    row_first = blockIdx.y * kLaRows;
    slot = p.req_slot[r];
  } else {
    const int t = p.items[work];
    const int r = p.tok_req[t];
    if (r < 0 || r >= p.n_reqs) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
    tok0 = t;
    pos0 = p.positions[t];
    if (pos0 < 0) { if (threadIdx.x == 0) set_error(p.err, kErrPosition, t, pos0, 0); return; }
    rows_total = H;
    row_first = blockIdx.z * kLaRows;
    split = blockIdx.y;
    slot = p.req_slot[r];
  }
  if (row_first >= rows_total) return;
  const int rows_here = min(kLaRows, rows_total - row_first);
  const int* table = p.block_table + (size_t)slot * p.max_pages;
  const int pos_first = pos0 + row_first / H;                      // position of the block's first row
  const int pos_last = pos0 + (row_first + rows_here - 1) / H;     // and of its last
  const int lo_tile = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
  int first_kt = lo_tile / kLaKeys, last_kt = pos_last / kLaKeys;
  if (p.n_splits > 1) {
    const int n = last_kt - first_kt + 1;
    const int a = first_kt + (int)((long long)n * split / p.n_splits);
    const int b = first_kt + (int)((long long)n * (split + 1) / p.n_splits);
    first_kt = a; last_kt = b - 1;
  }
  const int n_kt = last_kt - first_kt + 1;

  // a warp brings whole rows (keys): one look-up of the page a row, then the row's 16-byte pieces over the lanes
  auto issue_load = [&](int kt, int stage) {
    const uint32_t dst = k_base0 + stage * tile_bytes;
#pragma unroll 4
    for (int row = warp; row < kLaKeys; row += kLaWarps) {
      const int key = kt * kLaKeys + row;
      bool valid = key >= lo_tile && key <= pos_last;
      size_t src_row = 0;
      if (valid) {
        const int pidx = key / p.page_size;
        const int page = (pidx < p.max_pages) ? table[pidx] : -1;
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) set_error(p.err, kErrPage, work, pidx, page);
          valid = false;
        } else {
          src_row = (size_t)page * p.page_size + (key - pidx * p.page_size);
        }
      }
      const __nv_bfloat16* src = p.cache + src_row * D;
      for (int chunk = lane; chunk < CH; chunk += 32) cp_async16(dst + la_offset(row, chunk, CH), src + chunk * 8, valid);
    }
  };
  if (n_kt > 0) issue_load(first_kt, 0);
  cp_async_commit();

  // ---- the queries, as bfloat16 rows of shared memory (rows beyond the block's are zero)
  for (int idx = threadIdx.x; idx < kLaRows * CH; idx += kLaWarps * 32) {
    const int row = idx / CH, chunk = idx - row * CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_here) {
      const int R = row_first + row;
      const TQ* src = (const TQ*)p.q + (size_t)(tok0 + R / H) * p.q_tok_stride + (size_t)(R % H) * p.q_head_stride + chunk * 8;
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = pack_bf16(to_f32<TQ>(src[2 * i]), to_f32<TQ>(src[2 * i + 1]));
      v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(smem + la_offset(row, chunk, CH)) = v;
  }

  // this thread's two rows: 16 rg + g and + 8
  const int rowA = rg * 16 + g, rowB = rowA + 8;
  const bool hasA = rowA < rows_here, hasB = rowB < rows_here;
  const int posA = pos0 + (row_first + rowA) / H, posB = pos0 + (row_first + rowB) / H;
  const int loA = (p.window > 0 && posA - p.window + 1 > 0) ? posA - p.window + 1 : 0;
  const int loB = (p.window > 0 && posB - p.window + 1 > 0) ? posB - p.window + 1 : 0;
  const int pairs_all = DV / 16;
  const int pair0 = half == 0 ? 0 : (pairs_all + 1) / 2;            // this warp's pairs of 8-column tiles
  const int pairs_mine = half == 0 ? (pairs_all + 1) / 2 : pairs_all / 2;

  float o[2 * kPairs][4];
#pragma unroll
  for (int i = 0; i < 2 * kPairs; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};

  for (int it = 0; it < n_kt; ++it) {
    const int kt = first_kt + it;
    if (it + 1 < n_kt) issue_load(kt + 1, (it + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kb = k_base0 + (it & 1) * tile_bytes;

    float s[kLaKeys / 8][4];
#pragma unroll
    for (int nt = 0; nt < kLaKeys / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(q_base + la_offset(rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * ks + (lane >> 4), CH), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < kLaKeys / 16; ++np) {
        const int row = np * 16 + ((lane >> 4) << 3) + (lane & 7);
        const int chunk = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kb + la_offset(row, chunk, CH), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    float mx[2] = {-INFINITY, -INFINITY};
    const int key_first = kt * kLaKeys;
#pragma unroll
    for (int nt = 0; nt < kLaKeys / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_first + nt * 8 + 2 * t4 + (e & 1);
        const bool valid = (e < 2) ? (hasA && key <= posA && key >= loA) : (hasB && key <= posB && key >= loB);
        s[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = (m_new == -INFINITY) ? 0.0f : m_new;
      corr[h] = exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float psum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < kLaKeys / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
        psum[e >> 1] += s[nt][e];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
#pragma unroll
    for (int i = 0; i < 2 * kPairs; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < kLaKeys / 16; ++kk) {
      const uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int c = 0; c < kPairs; ++c) {
        if (c < pairs_mine) {
          const int row = kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          const int chunk = 2 * (pair0 + c) + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(kb + la_offset(row, chunk, CH), b0, b1, b2, b3);
          mma_bf16_16816(o[2 * c], pa0, pa1, pa2, pa3, b0, b1);
          mma_bf16_16816(o[2 * c + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (n_kt <= 0) __syncthreads();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  const int RA = row_first + rowA, RB = row_first + rowB;
  if (p.part_o != nullptr) {
    // a share of the keys: unnormalised sums, maximum and normaliser go to the merging kernel
    const size_t ia = ((size_t)work * H + RA) * p.n_splits + split, ib = ((size_t)work * H + RB) * p.n_splits + split;
    if (half == 0 && t4 == 0) {
      if (hasA) { p.part_ml[2 * ia] = m_run[0]; p.part_ml[2 * ia + 1] = l_run[0]; }
      if (hasB) { p.part_ml[2 * ib] = m_run[1]; p.part_ml[2 * ib + 1] = l_run[1]; }
    }
#pragma unroll
    for (int c = 0; c < 2 * kPairs; ++c) {
      if (c < 2 * pairs_mine) {
        const int col = (2 * pair0 + c) * 8 + 2 * t4;
        if (hasA) *reinterpret_cast<float2*>(p.part_o + ia * DV + col) = make_float2(o[c][0], o[c][1]);
        if (hasB) *reinterpret_cast<float2*>(p.part_o + ib * DV + col) = make_float2(o[c][2], o[c][3]);
      }
    }
    return;
  }
  if (p.sinks != nullptr) {
    // the sink: one more term of the denominator, with no key and no value
    if (hasA) {
      const float sk = p.sinks[RA % H] * 1.4426950408889634f, m = fmaxf(m_run[0], sk);
      const float f = exp2f(m_run[0] - m);
      l_run[0] = l_run[0] * f + exp2f(sk - m);
#pragma unroll
      for (int c = 0; c < 2 * kPairs; ++c) { o[c][0] *= f; o[c][1] *= f; }
    }
    if (hasB) {
      const float sk = p.sinks[RB % H] * 1.4426950408889634f, m = fmaxf(m_run[1], sk);
      const float f = exp2f(m_run[1] - m);
      l_run[1] = l_run[1] * f + exp2f(sk - m);
#pragma unroll
      for (int c = 0; c < 2 * kPairs; ++c) { o[c][2] *= f; o[c][3] *= f; }
    }
  }
  const float invA = hasA ? 1.0f / l_run[0] : 0.0f;
  const float invB = hasB ? 1.0f / l_run[1] : 0.0f;
  __nv_bfloat16* oA = p.out + ((size_t)(tok0 + RA / H) * H + RA % H) * DV;
  __nv_bfloat16* oB = p.out + ((size_t)(tok0 + RB / H) * H + RB % H) * DV;
#pragma unroll
  for (int c = 0; c < 2 * kPairs; ++c) {
    if (c < 2 * pairs_mine) {
      const int col = (2 * pair0 + c) * 8 + 2 * t4;
      if (hasA) *reinterpret_cast<uint32_t*>(oA + col) = pack_bf16(o[c][0] * invA, o[c][1] * invA);
      if (hasB) *reinterpret_cast<uint32_t*>(oB + col) = pack_bf16(o[c][2] * invB, o[c][3] * invB);
    }
  }
}

// Single tokens: 16 query rows (heads of one token) a block, so the rows cannot feed eight warps; the
// keys of a tile do.  Warp w forms the scores of the keys 8 w .. 8 w + 7 for all 16 rows, the warps'
// row maxima and sums meet in shared memory, the probabilities go to shared memory as bfloat16, and
// then warp w multiplies them into its own eighth of the value columns.  A ninth warp brings the key
// tiles in, a bulk copy a row, into two stages; "filled" and "given back" are mbarriers, every wait on
// them is bounded and reports kErrWait.
constexpr int kLdRows = 16;

template <typename TQ, int kPairsW>     // kPairsW: pairs of 8-column tiles of the values that one warp accumulates
__global__ void __launch_bounds__((kLaWarps + 1) * 32, 1) latent_decode_kernel(LatentAttnParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_max[kLaWarps][kLdRows], s_sum[kLaWarps][kLdRows];
  const int D = p.D, DV = p.DV, H = p.H;
  const int CH = D / 8;
  const int tile_bytes = kLaKeys * (CH + 1) * 16;
  const uint32_t q_base = smem_u32(smem);
  const uint32_t p_base = q_base + kLdRows * (CH + 1) * 16;          // probabilities [16][64] bfloat16, rows padded
  const uint32_t k_base0 = p_base + kLdRows * 9 * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int work = blockIdx.x, split = blockIdx.y;
  const int t = p.items[work];
  const int r = p.tok_req[t];
  if (r < 0 || r >= p.n_reqs) { if (threadIdx.x == 0) set_error(p.err, kErrRequest, t, r, p.n_reqs); return; }
  const int pos = p.positions[t];
  if (pos < 0) { if (threadIdx.x == 0) set_error(p.err, kErrPosition, t, pos, 0); return; }
  const int row_first = blockIdx.z * kLdRows;
  const int rows_here = min(kLdRows, H - row_first);
  const int* table = p.block_table + (size_t)p.req_slot[r] * p.max_pages;
  const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  int first_kt = lo / kLaKeys, last_kt = pos / kLaKeys;
  if (p.n_splits > 1) {
    const int n = last_kt - first_kt + 1;
    const int a = first_kt + (int)((long long)n * split / p.n_splits);
    const int b = first_kt + (int)((long long)n * (split + 1) / p.n_splits);
    first_kt = a; last_kt = b - 1;
  }
  const int n_kt = last_kt - first_kt + 1;

  // The keys of a tile come row by row through the copy unit (one bulk copy a row, issued by the lanes of
  // the ninth warp, counted off at the stage's barrier).  Rows outside the visible range are not copied; the
  // working warps clear them before the values are read, and their scores are masked.
  __shared__ __align__(8) unsigned long long s_bar[4];      // stage filled (2), stage given back (2)
  volatile __shared__ int no_abort;
  const uint32_t bars = smem_u32(s_bar);
  if (threadIdx.x == 0) {
    mbar_init(bars, 1); mbar_init(bars + 8, 1);
    mbar_init(bars + 16, kLaWarps); mbar_init(bars + 24, kLaWarps);
    no_abort = 0;
  }
  fence_async_shared();       // the barriers, before the copy unit reports to them
  __syncthreads();
  const uint32_t row_bytes = (uint32_t)D * 2u;
  auto issue_load = [&](int kt, int stage) {
    const uint32_t dst = k_base0 + stage * tile_bytes, bar = bars + 8 * stage;
    const int key0 = kt * kLaKeys;
    const int first = max(lo, key0), last = min(pos, key0 + kLaKeys - 1);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)max(0, last - first + 1) * row_bytes);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < kLaKeys / 32; ++j) {
      const int row = lane + 32 * j, key = key0 + row;
      if (key < first || key > last) continue;
      const int pidx = key / p.page_size;
      const int page = (pidx < p.max_pages) ? table[pidx] : -1;
      size_t src_row = 0;       // a bad page is reported; its row is copied from the pool's first row, so the count holds
      if (page < 0 || page >= p.num_pages) set_error(p.err, kErrPage, t, pidx, page);
      else src_row = (size_t)page * p.page_size + (key - pidx * p.page_size);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                   ::"r"(dst + la_offset(row, 0, CH)), "l"(p.cache + src_row * D), "r"(row_bytes), "r"(bar) : "memory");
    }
  };

  if (warp == kLaWarps) {
    // the warp that brings the keys in: a stage is filled again as soon as all eight working warps gave it back
    for (int it = 0; it < n_kt; ++it) {
      if (it >= 2 && !mbar_wait(bars + 16 + 8 * (it & 1), (uint32_t)((it >> 1) - 1) & 1u, &no_abort)) {
        if (lane == 0) { set_error(p.err, kErrWait, 61, work, it); no_abort = 1; }
        return;
      }
      issue_load(first_kt + it, it & 1);
    }
    return;
  }
  // the queries, as bfloat16 rows of shared memory (rows beyond the block's are zero), while the first keys travel
  for (int idx = threadIdx.x; idx < kLdRows * CH; idx += kLaWarps * 32) {
    const int row = idx / CH, chunk = idx - row * CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_here) {
      const TQ* src = (const TQ*)p.q + (size_t)t * p.q_tok_stride + (size_t)(row_first + row) * p.q_head_stride + chunk * 8;
      uint32_t w[4];
      if (sizeof(TQ) == 4 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const float4 x = reinterpret_cast<const float4*>(src)[0], y = reinterpret_cast<const float4*>(src)[1];
        w[0] = pack_bf16(x.x, x.y); w[1] = pack_bf16(x.z, x.w); w[2] = pack_bf16(y.x, y.y); w[3] = pack_bf16(y.z, y.w);
      } else if (sizeof(TQ) == 2 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const uint4 x = *reinterpret_cast<const uint4*>(src);
        w[0] = x.x; w[1] = x.y; w[2] = x.z; w[3] = x.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = pack_bf16(to_f32<TQ>(src[2 * i]), to_f32<TQ>(src[2 * i + 1]));
      }
      v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(smem + la_offset(row, chunk, CH)) = v;
  }
  asm volatile("bar.sync 1, %0;\n" ::"n"(kLaWarps * 32) : "memory");       // the queries are in place
  const bool hasA = g < rows_here, hasB = g + 8 < rows_here;
  const int pairs_all = DV / 16;
  const int per_warp = (pairs_all + kLaWarps - 1) / kLaWarps;
  const int pair0 = warp * per_warp;
  const int pairs_mine = max(0, min(per_warp, pairs_all - pair0));
  float o[2 * kPairsW][4];
#pragma unroll
  for (int i = 0; i < 2 * kPairsW; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  const int k_steps = D / 16;

  for (int it = 0; it < n_kt; ++it) {
    const int kt = first_kt + it;
    if (!mbar_wait(bars + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, &no_abort)) {
      if (lane == 0) { set_error(p.err, kErrWait, 60, work, it); no_abort = 1; }
    }
    const uint32_t kb = k_base0 + (it & 1) * tile_bytes;
    if (kt * kLaKeys < lo || kt * kLaKeys + kLaKeys - 1 > pos) {
      // the window's first tile or the token's last: rows that were not copied are cleared (their probabilities
      // are zero, but zero times what the stage held before need not be); done before the values are read
      for (int row = warp; row < kLaKeys; row += kLaWarps) {
        const int key = kt * kLaKeys + row;
        if (key < lo || key > pos) {
          for (int chunk = lane; chunk < CH; chunk += 32) {
            *reinterpret_cast<uint4*>(smem + (kb - q_base) + la_offset(row, chunk, CH)) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
    }

    // scores of this warp's eight keys, two steps of 16 elements a load of the keys
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // two chains of products
    {
      uint32_t ka = kb + la_offset(warp * 8 + (lane & 7), lane >> 3, CH);                  // four chunks a load: two steps
      uint32_t qa = q_base + la_offset((lane & 7) + ((lane >> 3) & 1) * 8, lane >> 4, CH);   // two chunks a load: one step
      int ks = 0;
      for (; ks + 1 < k_steps; ks += 2, ka += 64, qa += 64) {
        uint32_t b0, b1, b2, b3, a0, a1, a2, a3;
        ldmatrix_x4(ka, b0, b1, b2, b3);
        ldmatrix_x4(qa, a0, a1, a2, a3);
        mma_bf16_16816(s, a0, a1, a2, a3, b0, b1);
        ldmatrix_x4(qa + 32, a0, a1, a2, a3);
        mma_bf16_16816(s2, a0, a1, a2, a3, b2, b3);
      }
      if (ks < k_steps) {       // an odd number of steps: the last load of the keys reads two chunks twice
        uint32_t b0, b1, b2, b3, a0, a1, a2, a3;
        ldmatrix_x4(kb + la_offset(warp * 8 + (lane & 7), 2 * ks + ((lane >> 3) & 1), CH), b0, b1, b2, b3);
        ldmatrix_x4(qa, a0, a1, a2, a3);
        mma_bf16_16816(s, a0, a1, a2, a3, b0, b1);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] += s2[e];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = kt * kLaKeys + warp * 8 + 2 * t4 + (e & 1);
      const bool valid = ((e < 2) ? hasA : hasB) && key <= pos && key >= lo;
      s[e] = valid ? s[e] * p.scale_log2 : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[e]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    if (t4 == 0) { s_max[warp][g] = mx[0]; s_max[warp][g + 8] = mx[1]; }
    asm volatile("bar.sync 1, %0;\n" ::"n"(kLaWarps * 32) : "memory");     // the eight working warps
    if (no_abort) return;     // a wait ran out somewhere in the block: every working warp sees it here and leaves
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m_new = m_run[h];
#pragma unroll
      for (int w = 0; w < kLaWarps; ++w) m_new = fmaxf(m_new, s_max[w][g + 8 * h]);
      m_use[h] = (m_new == -INFINITY) ? 0.0f : m_new;
      corr[h] = exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float psum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s[e] = exp2f(s[e] - m_use[e >> 1]);
      psum[e >> 1] += s[e];
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
      psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
    }
    if (t4 == 0) { s_sum[warp][g] = psum[0]; s_sum[warp][g + 8] = psum[1]; }
    // probabilities of rows g and g + 8, keys 8 w + 2 t4 and the next one: chunk w of the rows
    *reinterpret_cast<uint32_t*>(smem + (p_base - q_base) + (g * 9 + warp) * 16 + t4 * 4) = pack_bf16(s[0], s[1]);
    *reinterpret_cast<uint32_t*>(smem + (p_base - q_base) + ((g + 8) * 9 + warp) * 16 + t4 * 4) = pack_bf16(s[2], s[3]);
    asm volatile("bar.sync 1, %0;\n" ::"n"(kLaWarps * 32) : "memory");
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float add = 0.0f;
#pragma unroll
      for (int w = 0; w < kLaWarps; ++w) add += s_sum[w][g + 8 * h];
      l_run[h] = l_run[h] * corr[h] + add;
    }
#pragma unroll
    for (int i = 0; i < 2 * kPairsW; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    const uint32_t pa = p_base + (((lane & 7) + ((lane >> 3) & 1) * 8) * 9 + (lane >> 4)) * 16;
    const uint32_t va = kb + la_offset((((lane >> 3) & 1) << 3) + (lane & 7), 2 * pair0 + (lane >> 4), CH);
#pragma unroll
    for (int kk = 0; kk < kLaKeys / 16; ++kk) {
      uint32_t pa0, pa1, pa2, pa3;
      ldmatrix_x4(pa + kk * 32, pa0, pa1, pa2, pa3);
#pragma unroll
      for (int c = 0; c < kPairsW; ++c) {
        if (c < pairs_mine) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(va + kk * 16 * (CH + 1) * 16 + c * 32, b0, b1, b2, b3);
          mma_bf16_16816(o[2 * c], pa0, pa1, pa2, pa3, b0, b1);
          mma_bf16_16816(o[2 * c + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
    }
    fence_async_shared();      // rows this warp cleared, before the copy unit writes the stage again
    __syncwarp();
    if (lane == 0) mbar_arrive(bars + 16 + 8 * (it & 1));      // this warp has read the stage for the last time
  }

  // l_run is the same in every thread that holds a row (all added the same shares in the same order)
  const int RA = row_first + g, RB = RA + 8;
  if (p.part_o != nullptr) {
    const size_t ia = ((size_t)work * H + RA) * p.n_splits + split, ib = ((size_t)work * H + RB) * p.n_splits + split;
    if (warp == 0 && t4 == 0) {
      if (hasA) { p.part_ml[2 * ia] = m_run[0]; p.part_ml[2 * ia + 1] = l_run[0]; }
      if (hasB) { p.part_ml[2 * ib] = m_run[1]; p.part_ml[2 * ib + 1] = l_run[1]; }
    }
#pragma unroll
    for (int c = 0; c < 2 * kPairsW; ++c) {
      if (c < 2 * pairs_mine) {
        const int col = (2 * pair0 + c) * 8 + 2 * t4;
        if (hasA) *reinterpret_cast<float2*>(p.part_o + ia * DV + col) = make_float2(o[c][0], o[c][1]);
        if (hasB) *reinterpret_cast<float2*>(p.part_o + ib * DV + col) = make_float2(o[c][2], o[c][3]);
      }
    }
    return;
  }
  if (p.sinks != nullptr) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (h == 0 ? hasA : hasB) {
        const float sk = p.sinks[h == 0 ? RA : RB] * 1.4426950408889634f, m = fmaxf(m_run[h], sk);
        const float f = exp2f(m_run[h] - m);
        l_run[h] = l_run[h] * f + exp2f(sk - m);
#pragma unroll
        for (int c = 0; c < 2 * kPairsW; ++c) { o[c][2 * h] *= f; o[c][2 * h + 1] *= f; }
      }
    }
  }
  const float invA = hasA ? 1.0f / l_run[0] : 0.0f;
  const float invB = hasB ? 1.0f / l_run[1] : 0.0f;
  __nv_bfloat16* oA = p.out + ((size_t)t * H + RA) * DV;
  __nv_bfloat16* oB = p.out + ((size_t)t * H + RB) * DV;
#pragma unroll
  for (int c = 0; c < 2 * kPairsW; ++c) {
    if (c < 2 * pairs_mine) {
      const int col = (2 * pair0 + c) * 8 + 2 * t4;
      if (hasA) *reinterpret_cast<uint32_t*>(oA + col) = pack_bf16(o[c][0] * invA, o[c][1] * invA);
      if (hasB) *reinterpret_cast<uint32_t*>(oB + col) = pack_bf16(o[c][2] * invB, o[c][3] * invB);
    }
  }
}

// out[t, h, :] = sum_s o_s 2^(m_s - m) / (sum_s l_s 2^(m_s - m) + 2^(sink - m)), the shares in their order.
// One block per (token, head): the shares' maxima and normalisers are fetched side by side, one warp
// turns them into a weight per share, then every thread adds its columns up with the loads of several
// shares on their way at a time.
constexpr int kLaMaxSplits = 128;

__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml,
                                                           const float* __restrict__ sinks, const int* __restrict__ items,
                                                           __nv_bfloat16* __restrict__ out, int H, int DV, int n_splits) {
  __shared__ float s_m[kLaMaxSplits], s_w[kLaMaxSplits];
  pdl_trigger();
  pdl_wait();
  const int item = blockIdx.x / H, h = blockIdx.x % H;
  const size_t base = (size_t)blockIdx.x * n_splits;
  const int lane = threadIdx.x & 31;
  float l_mine = 0.0f;
  if (threadIdx.x < n_splits) {
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + 2 * (base + threadIdx.x));
    s_m[threadIdx.x] = ml.x;
    l_mine = ml.y;
  }
  __syncthreads();
  float m = sinks != nullptr ? sinks[h] * 1.4426950408889634f : -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, s_m[s]);          // every thread the same, from shared memory
  if (threadIdx.x < n_splits) {
    const float ms = s_m[threadIdx.x];
    s_w[threadIdx.x] = ms == -INFINITY ? 0.0f : exp2f(ms - m);
    s_m[threadIdx.x] = ms == -INFINITY ? 0.0f : l_mine * exp2f(ms - m);
  }
  __syncthreads();
  float l = sinks != nullptr ? exp2f(sinks[h] * 1.4426950408889634f - m) : 0.0f;
  for (int s = 0; s < n_splits; ++s) l += s_m[s];                    // in the shares' order
  const float inv = 1.0f / l;
  (void)lane;
  __nv_bfloat16* dst = out + ((size_t)items[item] * H + h) * DV;
  const float* src = part_o + base * DV;
  for (int e = threadIdx.x; e < DV; e += blockDim.x) {
    float acc = 0.0f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) acc = fmaf(src[(size_t)s * DV + e], s_w[s], acc);
    dst[e] = __float2bfloat16_rn(acc * inv);
  }
}

template <typename TQ, int kPairs>
static cudaError_t launch_latent(const LatentAttnParams& p, dim3 grid, cudaStream_t stream) {
  const int smem_bytes = 3 * kLaKeys * (p.D / 8 + 1) * 16;
  static int configured = 0;
  if (configured < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<TQ, kPairs>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes);
    if (e != cudaSuccess) return e;
    configured = smem_bytes;
  }
  return launch(latent_attention_kernel<TQ, kPairs>, grid, dim3(kLaWarps * 32), (size_t)smem_bytes, stream, p);
}

template <typename TQ, int kPairsW>
static cudaError_t launch_latent_decode(const LatentAttnParams& p, dim3 grid, cudaStream_t stream) {
  const int smem_bytes = (2 * kLaKeys + kLdRows) * (p.D / 8 + 1) * 16 + kLdRows * 9 * 16;
  static int configured = 0;
  if (configured < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(latent_decode_kernel<TQ, kPairsW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes);
    if (e != cudaSuccess) return e;
    configured = smem_bytes;
  }
  return launch(latent_decode_kernel<TQ, kPairsW>, grid, dim3((kLaWarps + 1) * 32), (size_t)smem_bytes, stream, p);
}

}  // namespace tk

// Whether the tensor-core kernel takes a latent cache of these sizes: rows and values in whole 16-element
// steps, three tiles of shared memory within an SM's.
TK_API int tk_attention_latent_takes(int d, int dv) {
  return d % 16 == 0 && dv % 16 == 0 && dv >= 16 && dv <= 512 && dv <= d && d <= 576;
}

TK_API int tk_attention_latent(const void* q, void* out, const void* cache, const float* sinks, const int* tiles,
                               const int* items, const int* positions, const int* tok_req, const int* req_q_start,
                               const int* req_q_len, const int* req_kv_len, const int* req_slot, const int* block_table,
                               float* part_o, float* part_ml, int* err, long long q_tok_stride, long long q_head_stride,
                               int q_dtype, int n_work, int n_reqs, int heads, int d, int dv, int page_size, int max_pages,
                               int num_pages, int window, int n_splits, float scale, cudaStream_t stream) {
  if (n_work <= 0) return 0;
  if (!tk_attention_latent_takes(d, dv) || heads < 1 || (tiles == nullptr) == (items == nullptr) || n_splits < 1 ||
      (n_splits > 1 && (part_o == nullptr || part_ml == nullptr || tiles != nullptr)) || n_splits > tk::kLaMaxSplits ||
      (q_dtype != tk::kF32 && q_dtype != tk::kBF16)) {
    return (int)cudaErrorInvalidValue;
  }
  tk::LatentAttnParams p;
  p.q = q; p.out = (__nv_bfloat16*)out; p.cache = (const __nv_bfloat16*)cache; p.sinks = sinks; p.tiles = tiles;
  p.items = items; p.positions = positions; p.tok_req = tok_req; p.req_q_start = req_q_start; p.req_q_len = req_q_len;
  p.req_kv_len = req_kv_len; p.req_slot = req_slot; p.block_table = block_table;
  p.part_o = n_splits > 1 ? part_o : nullptr; p.part_ml = n_splits > 1 ? part_ml : nullptr; p.err = err;
  p.q_tok_stride = q_tok_stride; p.q_head_stride = q_head_stride; p.n_work = n_work; p.n_reqs = n_reqs; p.H = heads;
  p.D = d; p.DV = dv; p.page_size = page_size; p.max_pages = max_pages; p.num_pages = num_pages; p.window = window;
  p.n_splits = n_splits; p.scale_log2 = scale * 1.4426950408889634f;
  const int row_tiles = tiles != nullptr ? heads : (heads + tk::kLdRows - 1) / tk::kLdRows;   // 64 tokens x H rows / 64
  if (row_tiles > 65535) return (int)cudaErrorInvalidValue;
  dim3 grid = tiles != nullptr ? dim3(n_work, row_tiles, 1) : dim3(n_work, n_splits, row_tiles);
  const int pairs_half = (dv / 16 + 1) / 2;
  cudaError_t e;
  if (items != nullptr) {
    const int per_warp = (dv / 16 + tk::kLaWarps - 1) / tk::kLaWarps;
#define TK_LATENT_DEC(TQ)                                                          \
  (per_warp <= 1 ? tk::launch_latent_decode<TQ, 1>(p, grid, stream)                \
   : per_warp <= 2 ? tk::launch_latent_decode<TQ, 2>(p, grid, stream)              \
                   : tk::launch_latent_decode<TQ, 4>(p, grid, stream))
    e = q_dtype == tk::kF32 ? TK_LATENT_DEC(float) : TK_LATENT_DEC(__nv_bfloat16);
#undef TK_LATENT_DEC
    if (e != cudaSuccess || n_splits <= 1) return (int)e;
    e = tk::launch(tk::latent_merge_kernel, dim3((unsigned)(n_work * heads)), dim3(128), 0, stream, (const float*)part_o,
                   (const float*)part_ml, sinks, items, (__nv_bfloat16*)out, heads, dv, n_splits);
    return (int)e;
  }
#define TK_LATENT(TQ)                                                              \
  (pairs_half <= 2 ? tk::launch_latent<TQ, 2>(p, grid, stream)                     \
   : pairs_half <= 4 ? tk::launch_latent<TQ, 4>(p, grid, stream)                   \
   : pairs_half <= 8 ? tk::launch_latent<TQ, 8>(p, grid, stream)                   \
                     : tk::launch_latent<TQ, 16>(p, grid, stream))
  e = q_dtype == tk::kF32 ? TK_LATENT(float) : TK_LATENT(__nv_bfloat16);
#undef TK_LATENT
  if (e != cudaSuccess || n_splits <= 1) return (int)e;
  e = tk::launch(tk::latent_merge_kernel, dim3((unsigned)(n_work * heads)), dim3(128), 0, stream, (const float*)part_o,
                 (const float*)part_ml, sinks, items, (__nv_bfloat16*)out, heads, dv, n_splits);
  return (int)e;
}
