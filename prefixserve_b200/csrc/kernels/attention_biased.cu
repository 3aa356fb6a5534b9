// Causal grouped-query attention over the paged cache for designs whose scores carry more than q.k:
//
//   score(i, j) = (q_i . k_j) * scale + bias[h][min(i - j, reach - 1)]       (bias optional)
//   visible:  j <= i,  j > i - window (window optional),  floor(j / chunk) == floor(i / chunk) (chunk optional);
//             with ``keep_first`` > 0 (and a window, no chunk) the first keep_first keys of the sequence stay visible
//             to every later query, at their true positions: j <= i and (j > i - window or j < keep_first)
//   weights = exp(score) / (sum over visible j of exp(score) + exp(sink[h]))  (sink optional: a term of the
//             denominator that has no key and no value)
//
// Keys and values may have different sizes (dim, vdim); the cache entry holds one row per token and key/value head,
// [num_pages, 1, hkv, page_size, dim + vdim]: the key, then the value.  ``bias`` is a float32 table
// [heads, reach] by distance (whatever maps distances to learned rows has been applied when the table was built;
// distances of reach - 1 and more share the last column).  Positions are absolute, so the chunk grid is counted
// from the start of the sequence however the prompt was cut.
//
// attention_biased_append_kernel splits a fused projection row [q | k | v] into the query tensor and the cache row.
// attention_biased_kernel: a block per (token, query head) walks the visible keys in runs of 32 aligned to absolute
// positions, its four warps taking the runs in turn, a lane per key for the scores (the key row read 16 bytes at a
// time), online softmax per warp, the four shares and the sink (maximum = sink, sum = 1, no value) joined at the end.
// Scores, weights and sums are float32 and the weights are not rounded before they multiply the values.  Float32 and
// bfloat16 storage.
//
// attention_biased_tile_kernel (bfloat16 storage): a block takes 16 consecutive tokens of one request and one
// key/value head, with all the query heads that share it; key/value rows are staged in shared memory once for the
// block, a warp takes (token, head) pairs in turn and walks all runs of its pair in order.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T, typename TKV>
__global__ void attention_biased_append_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ token_item, const int32_t* __restrict__ table,
                                               int table_width, TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv,
                                               int dim, int vdim, int page_size, int num_pages) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int qw = hq * dim, kw = hkv * dim, vw = hkv * vdim;
  const T* row = qkv + (size_t)t * (qw + kw + vw);
  for (int c = threadIdx.x; c < qw; c += blockDim.x) q_out[(size_t)t * qw + c] = row[c];
  const int p = positions[t];
  int page = table[(size_t)token_item[t] * table_width + p / page_size];
  if (page < 0 || page >= num_pages) return;  // tables are checked on the host; never write outside the pool
  const int rw = dim + vdim;
  TKV* dst = kv + ((size_t)page * hkv * page_size + (size_t)(p % page_size)) * rw;
  for (int c = threadIdx.x; c < kw + vw; c += blockDim.x) {
    int g, e;
    if (c < kw) { g = c / dim; e = c - g * dim; }
    else { g = (c - kw) / vdim; e = dim + (c - kw) - g * vdim; }
    dst[(size_t)g * page_size * rw + e] = from_float<TKV>(to_float<T>(row[qw + c]));
  }
}

// q . k over ``dim`` elements, 16 bytes of the key row at a time where ``vec`` says the row allows it.
template <typename TKV>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const TKV* __restrict__ k, int dim, bool vec);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int dim, bool vec) {
  float dot = 0.f;
  if (vec) {
    for (int d = 0; d < dim; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + d);
      dot = fmaf(q[d], kv.x, dot); dot = fmaf(q[d + 1], kv.y, dot); dot = fmaf(q[d + 2], kv.z, dot); dot = fmaf(q[d + 3], kv.w, dot);
    }
  } else {
    for (int d = 0; d < dim; ++d) dot = fmaf(q[d], k[d], dot);
  }
  return dot;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int dim, bool vec) {
  float dot = 0.f;
  if (vec) {
    // four 16-byte pieces of the row are asked for before the first is used (a lane's row is its own: nothing coalesces)
    for (int d0 = 0; d0 < dim; d0 += 32) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) raw[u] = d0 + 8 * u < dim ? *reinterpret_cast<const uint4*>(k + d0 + 8 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (d0 + 8 * u >= dim) break;
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kv = __bfloat1622float2(p2[j]);
          dot = fmaf(q[d0 + 8 * u + 2 * j], kv.x, dot);
          dot = fmaf(q[d0 + 8 * u + 2 * j + 1], kv.y, dot);
        }
      }
    }
  } else {
    for (int d = 0; d < dim; ++d) dot = fmaf(q[d], __bfloat162float(k[d]), dot);
  }
  return dot;
}

// A block per (token, query head); its four warps take the runs of 32 keys in turn (run r of the token, counted from
// the aligned start of its visible keys, goes to warp r mod 4) and keep a running maximum, sum and output each; warp 0
// joins the four in warp order.  Which warp gets which run depends on the token's position and the masks only.
template <typename T, typename TKV>
__global__ void __launch_bounds__(WARPS * 32)
attention_biased_kernel(const T* __restrict__ q, const TKV* __restrict__ kv, const int32_t* __restrict__ table,
                        int table_width, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                        const float* __restrict__ bias, const float* __restrict__ sink, T* __restrict__ out, int T_tokens,
                        int hq, int hkv, int dim, int vdim, int page_size, int window, int chunk, int reach, float scale,
                        const int32_t* __restrict__ item_start, int skip_from, int keep_first, float* __restrict__ partial,
                        int splits) {
  __shared__ __align__(16) float qs[MAX_D];
  __shared__ float part[WARPS][MAX_D + 2];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x / hq, h = blockIdx.x - t * hq;
  const int g = h / (hq / hkv);
  const int p = positions[t];
  const int item = token_item[t];
  // ``splits`` > 1 (steps of few tokens over many keys): blockIdx.y names this block's share of the runs; it leaves its
  // maximum, sum and unnormalised output in ``partial`` [T * hq, splits, vdim + 2] and the merge kernel joins the shares
  const int split = blockIdx.y;
  if (skip_from > 0 && item_start[item + 1] - item_start[item] >= skip_from) return;  // the tiled kernel's token
  const int32_t* pages = table + (size_t)item * table_width;
  const T* qrow = q + ((size_t)t * hq + h) * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) qs[d] = to_float<T>(qrow[d]);
  __syncthreads();

  int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
  // kept first keys: when the window still reaches them the visible keys are one stretch from 0; otherwise their runs
  // (counted from key 0) come before the window's runs, and the keys between the two are never touched
  int kept_runs = 0;
  if (keep_first > 0) {
    if (lo <= keep_first) lo = 0;
    else kept_runs = (keep_first + 31) >> 5;
  }
  const int rw = dim + vdim;
  const size_t head_stride = (size_t)page_size * rw;
  const size_t page_elems = (size_t)hkv * head_stride;
  const float* brow = bias ? bias + (size_t)h * reach : nullptr;
  constexpr int PER16 = 16 / (int)sizeof(TKV);
  const bool vec = dim % PER16 == 0 && rw % PER16 == 0 && (((uintptr_t)kv) & 15) == 0;

  float m = -FLT_MAX, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int run = warp + WARPS * split;; run += WARPS * splits) {
    const bool kept = run < kept_runs;
    const int base = kept ? 32 * run : (lo & ~31) + 32 * (run - kept_runs);
    if (base > p) break;
    const int key = base + lane;
    const bool live = kept ? key < keep_first : (key >= lo && key <= p);
    long long off = -1;
    float s = -FLT_MAX;
    if (live) {
      const int page = pages[key / page_size];
      off = (long long)((size_t)page * page_elems + (size_t)g * head_stride + (size_t)(key % page_size) * rw);
      s = dot_row<TKV>(qs, kv + off, dim, vec) * scale;
      if (brow) s += brow[min(p - key, reach - 1)];
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);
    const float pr = live ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    const int n_live = kept ? min(32, keep_first - base) : min(32, p - base + 1);
    // eight keys at a time: their value rows are asked for together, then added in key order
    for (int j0 = 0; j0 < n_live; j0 += 8) {
      float pj[8];
      long long oj[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        pj[k] = __shfl_sync(0xffffffffu, pr, (j0 + k) & 31);
        oj[k] = __shfl_sync(0xffffffffu, off, (j0 + k) & 31);
      }
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) {
          float v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = oj[k] >= 0 ? to_float<TKV>(kv[oj[k] + dim + d]) : 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[i] = fmaf(pj[k], v[k], acc[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) part[warp][d] = acc[i];
  }
  if (lane == 0) { part[warp][MAX_D] = m; part[warp][MAX_D + 1] = l; }
  __syncthreads();
  if (warp != 0) return;
  // join: the sink first (maximum = sink, sum = 1, no value; with split keys it joins in the merge kernel), then the warps in order
  const bool sink_here = sink && splits == 1;
  float M = sink_here ? sink[h] : -FLT_MAX, L = sink_here ? 1.f : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;
  for (int w = 0; w < WARPS; ++w) {
    const float mw = part[w][MAX_D], lw = part[w][MAX_D + 1];
    if (lw == 0.f) continue;  // a warp without keys
    const float m_new = fmaxf(M, mw);
    const float a = expf(M - m_new), b2 = expf(mw - m_new);
    L = L * a + lw * b2;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < vdim) acc[i] = acc[i] * a + part[w][d] * b2;
    }
    M = m_new;
  }
  if (splits > 1) {
    float* mine = partial + (((size_t)t * hq + h) * splits + split) * (vdim + 2);
    if (lane == 0) { mine[0] = M; mine[1] = L; }
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < vdim) mine[2 + d] = acc[i];
    }
    return;
  }
  const float inv = 1.f / L;
  T* orow = out + ((size_t)t * hq + h) * vdim;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// Joins the shares of the blocks that split a (token, head)'s runs among them, in split order, the sink first.
constexpr int MAX_KEY_SPLITS = 16;

template <typename T>
__global__ void __launch_bounds__(32)
attention_biased_merge_kernel(const float* __restrict__ partial, const float* __restrict__ sink, T* __restrict__ out, int hq,
                              int vdim, int splits) {
  pdl_trigger();
  pdl_wait();
  const size_t unit = blockIdx.x;  // token * hq + head
  const int lane = threadIdx.x, h = (int)(unit % hq);
  const float* mine = partial + unit * splits * (vdim + 2);
  // every share's maximum and sum are asked for at once, then every share's output: nothing here waits for a share before
  // it asks for the next
  float ms[MAX_KEY_SPLITS], ls[MAX_KEY_SPLITS];
#pragma unroll
  for (int s = 0; s < MAX_KEY_SPLITS; ++s) {
    ms[s] = s < splits ? mine[(size_t)s * (vdim + 2)] : -FLT_MAX;
    ls[s] = s < splits ? mine[(size_t)s * (vdim + 2) + 1] : 0.f;
  }
  float M = sink ? sink[h] : -FLT_MAX;
#pragma unroll
  for (int s = 0; s < MAX_KEY_SPLITS; ++s)
    if (ls[s] > 0.f) M = fmaxf(M, ms[s]);  // (a share without keys has a sum of zero)
  float L = sink ? expf(sink[h] - M) : 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;
#pragma unroll
  for (int s = 0; s < MAX_KEY_SPLITS; ++s) {
    if (s >= splits) break;
    const float f = ls[s] > 0.f ? expf(ms[s] - M) : 0.f;
    L += ls[s] * f;
    const float* share = mine + (size_t)s * (vdim + 2) + 2;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < vdim) acc[i] = fmaf(share[d], f, acc[i]);
    }
  }
  const float inv = 1.f / L;
  T* orow = out + unit * vdim;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// Prompt portions in bfloat16: a block = up to TILE_T consecutive tokens of one item x one key/value head.  The keys a
// tile can see lie in [lo of its first token, position of its last]; they are brought into shared memory 32 at a time
// (the same absolute runs of 32 the kernel above walks), transposed so that a lane's key is a column, and every
// (token, query head) pair of the tile, one warp each in turn, works on the staged run.
constexpr int TILE_T = 16;
constexpr int TILE_WARPS = 8;

template <int DP, int VP>  // key and value sizes rounded up to 32, 64, 128 or 256
__global__ void __launch_bounds__(TILE_WARPS * 32)
attention_biased_tile_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                             const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ positions,
                             const int32_t* __restrict__ item_start, int items, int min_tokens, const float* __restrict__ bias,
                             const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, int hq, int hkv, int dim, int vdim,
                             int page_size, int window, int chunk, int reach, float scale, int keep_first) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  // tiles are numbered through the portions of at least ``min_tokens`` tokens, in order
  int item = -1, t0 = 0;
  for (int i = 0, left = blockIdx.x; i < items; ++i) {
    const int a = item_start[i], n = item_start[i + 1] - a;
    if (n < min_tokens) continue;
    const int tiles = (n + TILE_T - 1) / TILE_T;
    if (left < tiles) { item = i; t0 = a + left * TILE_T; break; }
    left -= tiles;
  }
  if (item < 0) return;
  const int g = blockIdx.y, share = hq / hkv;
  const int nt = min(TILE_T, item_start[item + 1] - t0);
  const int pairs = nt * share;  // (token, head of the group) units of this block
  float* ks = smem;                               // [DP][33] one run of keys, transposed
  float* vs = ks + DP * 33;                       // [32][VP]
  float* qs = vs + 32 * VP;                       // [TILE_T * share][DP]
  float* st = qs + (size_t)TILE_T * share * DP;   // per unit: m, l
  float* accs = st + 2 * TILE_T * share;          // [TILE_T * share][VP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rw = dim + vdim;
  const size_t head_stride = (size_t)page_size * rw;
  const size_t page_elems = (size_t)hkv * head_stride;
  const int32_t* pages = table + (size_t)item * table_width;
  const int p_first = positions[t0], p_last = p_first + nt - 1;
  for (int i = threadIdx.x; i < pairs * DP; i += blockDim.x) {
    const int u = i / DP, d = i - u * DP;
    const int tt = u / share, hh = g * share + (u - tt * share);
    qs[i] = d < dim ? __bfloat162float(q[((size_t)(t0 + tt) * hq + hh) * dim + d]) : 0.f;
  }
  for (int i = threadIdx.x; i < pairs * VP; i += blockDim.x) accs[i] = 0.f;
  for (int u = threadIdx.x; u < pairs; u += blockDim.x) {
    const int hh = g * share + u % share;
    st[2 * u] = sink ? sink[hh] : -FLT_MAX;
    st[2 * u + 1] = sink ? 1.f : 0.f;
  }
  int lo_tile = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  if (chunk > 0) lo_tile = max(lo_tile, (p_first / chunk) * chunk);
  // kept first keys: one stretch from 0 while the tile's first token still reaches them; else their runs come first
  // (then every token of the tile has a gap between the kept keys and its window)
  int kept_runs = 0;
  if (keep_first > 0) {
    if (lo_tile <= keep_first) lo_tile = 0;
    else kept_runs = (keep_first + 31) >> 5;
  }
  for (int run = 0;; ++run) {
    const bool kept = run < kept_runs;
    const int base = kept ? 32 * run : (lo_tile & ~31) + 32 * (run - kept_runs);
    if (base > p_last) break;
    __syncthreads();
    // stage the run: keys transposed, values as rows; a key beyond the tile's last position is left as zeros
    for (int i = threadIdx.x; i < 32 * (DP + VP) / 2; i += blockDim.x) {
      const int j = i / ((DP + VP) / 2), e = 2 * (i - j * ((DP + VP) / 2));
      const int key = base + j;
      float a = 0.f, b = 0.f;
      const bool is_key = e < DP;
      const int col = is_key ? e : e - DP;
      const int width = is_key ? dim : vdim;
      if ((kept ? key < keep_first : (key >= lo_tile && key <= p_last)) && col < width) {
        const int page = pages[key / page_size];
        const __nv_bfloat16* src = kv + (size_t)page * page_elems + (size_t)g * head_stride + (size_t)(key % page_size) * rw +
                                   (is_key ? 0 : dim) + col;
        a = __bfloat162float(src[0]);
        if (col + 1 < width) b = __bfloat162float(src[1]);
      }
      if (is_key) { ks[col * 33 + j] = a; ks[(col + 1) * 33 + j] = b; }
      else { vs[j * VP + col] = a; vs[j * VP + col + 1] = b; }
    }
    __syncthreads();
    for (int u = warp; u < pairs; u += TILE_WARPS) {
      const int tt = u / share, hh = g * share + (u - tt * share);
      const int p = p_first + tt;
      if (base > p) continue;
      int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
      if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
      if (keep_first > 0 && lo <= keep_first) lo = 0;
      // (a tile whose first token still reaches the kept keys has no kept runs, but a later token's window may
      // already start beyond them: such a token sees the kept keys inside the ordinary runs)
      const bool inline_kept = kept_runs == 0 && keep_first > 0;  // the kept keys lie inside the ordinary runs
      if (!kept && base + 31 < lo && !(inline_kept && base < keep_first)) continue;
      const int key = base + lane;
      const bool live = kept ? key < keep_first : (key <= p && (key >= lo || (inline_kept && key < keep_first)));
      float s = -FLT_MAX;
      if (live) {
        const float* qq = qs + (size_t)u * DP;
        float dot = 0.f;
        for (int d = 0; d < dim; ++d) dot = fmaf(qq[d], ks[d * 33 + lane], dot);
        s = dot * scale;
        if (bias) s += bias[(size_t)hh * reach + min(p - key, reach - 1)];
      }
      float m = st[2 * u], l = st[2 * u + 1];
      const float m_new = fmaxf(m, warp_max(s));
      const float alpha = expf(m - m_new);
      const float pr = live ? expf(s - m_new) : 0.f;
      l = l * alpha + warp_sum(pr);
      __syncwarp();
      if (lane == 0) { st[2 * u] = m_new; st[2 * u + 1] = l; }
      float* acc = accs + (size_t)u * VP;
      float a[VP / 32];
#pragma unroll
      for (int i = 0; i < VP / 32; ++i) a[i] = acc[lane + 32 * i] * alpha;
      const int n_live = kept ? min(32, keep_first - base) : min(32, p - base + 1);
      const int j0 = (kept || (inline_kept && base < keep_first)) ? 0 : max(0, lo - base);
      for (int j = j0; j < n_live; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
        for (int i = 0; i < VP / 32; ++i) a[i] = fmaf(pj, vs[j * VP + lane + 32 * i], a[i]);
      }
#pragma unroll
      for (int i = 0; i < VP / 32; ++i) acc[lane + 32 * i] = a[i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs * VP; i += blockDim.x) {
    const int u = i / VP, d = i - u * VP;
    if (d >= vdim) continue;
    const int tt = u / share, hh = g * share + (u - tt * share);
    out[((size_t)(t0 + tt) * hq + hh) * vdim + d] = __float2bfloat16_rn(accs[i] / st[2 * u + 1]);
  }
}

// Prompt portions in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 sums): a block of four warps takes 64
// consecutive tokens of one request and one query head, a warp 16 of them.  Keys come in blocks of 64 aligned to
// absolute positions: K as [key][d] and V transposed as [v][key] in shared memory (zeros for keys outside the tile's
// reach, so nothing of a page that was never written is read).  S = Q K^T stays in the accumulator registers, where
// scale, bias, masks and the online softmax (started from the sink) are applied in float32; the weights enter the
// second product as the sum of two bfloat16 numbers (p = hi + lo, two instructions), so they keep 16 bits.
constexpr int MMA_ROWS = 64, MMA_KEYS = 64;
constexpr int MMA_BIAS = 2048;  // distances whose bias a block keeps in shared memory

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
  hi = pack_bf16(a, b);
  lo = pack_bf16(a - __bfloat162float(ha), b - __bfloat162float(hb));
}

template <int D, int V>  // key and value sizes rounded up to 64 or 128
__global__ void __launch_bounds__(128)
attention_biased_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                            const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ positions,
                            const int32_t* __restrict__ item_start, int items, int min_tokens, const float* __restrict__ bias,
                            const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, int hq, int hkv, int dim, int vdim,
                            int page_size, int window, int chunk, int reach, float scale, int keep_first) {
  constexpr int KS = D + 8, VS = MMA_KEYS + 8;  // row pitches that keep the fragment loads off each other's banks
  __shared__ __align__(16) __nv_bfloat16 ks[MMA_KEYS * KS];   // keys [key][d]; first the tile's queries [row][d]
  __shared__ __align__(16) __nv_bfloat16 vt[V * VS];          // values transposed [v][key]
  __shared__ float near_bias[MMA_BIAS];                       // the head's bias for the nearest distances
  pdl_wait();
  int item = -1, t0 = 0;
  for (int i = 0, left = blockIdx.x; i < items; ++i) {
    const int a = item_start[i], n = item_start[i + 1] - a;
    if (n < min_tokens) continue;
    const int tiles = (n + MMA_ROWS - 1) / MMA_ROWS;
    if (left < tiles) { item = i; t0 = a + left * MMA_ROWS; break; }
    left -= tiles;
  }
  if (item < 0) return;
  const int h = blockIdx.y, g = h / (hq / hkv);
  const int nt = min(MMA_ROWS, item_start[item + 1] - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int rw = dim + vdim;
  const size_t head_stride = (size_t)page_size * rw, page_elems = (size_t)hkv * head_stride;
  const int32_t* pages = table + (size_t)item * table_width;
  const int p_first = positions[t0], p_last = p_first + nt - 1;

  // the tile's queries through shared memory into fragments
  for (int i = threadIdx.x; i < MMA_ROWS * (D / 8); i += blockDim.x) {
    const int r = i / (D / 8), c = (i - r * (D / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nt && c < dim) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r) * hq + h) * dim + c);
    *reinterpret_cast<uint4*>(&ks[r * KS + c]) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    qf[kk][0] = *reinterpret_cast<const uint32_t*>(&ks[(warp * 16 + gid) * KS + kk * 16 + 2 * tig]);
    qf[kk][1] = *reinterpret_cast<const uint32_t*>(&ks[(warp * 16 + gid + 8) * KS + kk * 16 + 2 * tig]);
    qf[kk][2] = *reinterpret_cast<const uint32_t*>(&ks[(warp * 16 + gid) * KS + kk * 16 + 2 * tig + 8]);
    qf[kk][3] = *reinterpret_cast<const uint32_t*>(&ks[(warp * 16 + gid + 8) * KS + kk * 16 + 2 * tig + 8]);
  }
  // this thread's two rows: positions, lowest visible keys, running maximum and its share of the running sum
  int pos[2], low[2];
  float m[2], l[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    pos[r] = p_first + warp * 16 + gid + 8 * r;
    low[r] = (window > 0 && pos[r] - window + 1 > 0) ? pos[r] - window + 1 : 0;
    if (chunk > 0) low[r] = max(low[r], (pos[r] / chunk) * chunk);
    if (keep_first > 0 && low[r] <= keep_first) low[r] = 0;
    m[r] = sink ? sink[h] : -FLT_MAX;
    l[r] = (sink && tig == 0) ? 1.f : 0.f;
  }
  float o[V / 8][4];
#pragma unroll
  for (int i = 0; i < V / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float* brow = bias ? bias + (size_t)h * reach : nullptr;
  if (brow)
    for (int i = threadIdx.x; i < min(reach, MMA_BIAS); i += 128) near_bias[i] = brow[i];  // visible after the loop's first barrier

  int lo_tile = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  if (chunk > 0) lo_tile = max(lo_tile, (p_first / chunk) * chunk);
  // kept first keys: one stretch from 0 while the tile's first token still reaches them; else their blocks come first
  int kept_blocks = 0;
  if (keep_first > 0) {
    if (lo_tile <= keep_first) lo_tile = 0;
    else kept_blocks = (keep_first + MMA_KEYS - 1) / MMA_KEYS;
  }
  for (int blk = 0;; ++blk) {
    const bool kept = blk < kept_blocks;
    const int base = kept ? MMA_KEYS * blk : (lo_tile & ~(MMA_KEYS - 1)) + MMA_KEYS * (blk - kept_blocks);
    if (base > p_last) break;
    __syncthreads();  // everybody has its query fragments (first round) or is done with the last block
    // every thread asks for all its pieces of the block (page ids first, then the rows) before it stores any
    constexpr int KPIECES = MMA_KEYS * (D / 8) / 128, VPIECES = MMA_KEYS * (V / 8) / 128;
    uint4 kreg[KPIECES], vreg[VPIECES];
#pragma unroll
    for (int u = 0; u < KPIECES; ++u) {
      const int i = threadIdx.x + u * 128;
      const int j = i / (D / 8), c = (i - j * (D / 8)) * 8;
      const int key = base + j;
      kreg[u] = make_uint4(0, 0, 0, 0);
      if ((kept ? key < keep_first : (key >= lo_tile && key <= p_last)) && c < dim)
        kreg[u] = *reinterpret_cast<const uint4*>(kv + (size_t)pages[key / page_size] * page_elems + (size_t)g * head_stride +
                                                  (size_t)(key % page_size) * rw + c);
    }
#pragma unroll
    for (int u = 0; u < VPIECES; ++u) {
      const int i = threadIdx.x + u * 128;
      const int j = i % MMA_KEYS, c = (i / MMA_KEYS) * 8;  // neighbouring lanes: neighbouring keys, the same eight value channels
      const int key = base + j;
      vreg[u] = make_uint4(0, 0, 0, 0);
      if ((kept ? key < keep_first : (key >= lo_tile && key <= p_last)) && c < vdim)
        vreg[u] = *reinterpret_cast<const uint4*>(kv + (size_t)pages[key / page_size] * page_elems + (size_t)g * head_stride +
                                                  (size_t)(key % page_size) * rw + dim + c);
    }
#pragma unroll
    for (int u = 0; u < KPIECES; ++u) {
      const int i = threadIdx.x + u * 128;
      const int j = i / (D / 8), c = (i - j * (D / 8)) * 8;
      *reinterpret_cast<uint4*>(&ks[j * KS + c]) = kreg[u];
    }
#pragma unroll
    for (int u = 0; u < VPIECES; ++u) {
      const int i = threadIdx.x + u * 128;
      const int j = i % MMA_KEYS, c = (i / MMA_KEYS) * 8;
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&vreg[u]);
#pragma unroll
      for (int k = 0; k < 8; ++k) vt[(c + k) * VS + j] = e[k];
    }
    __syncthreads();
    if (warp * 16 >= nt || base > p_first + warp * 16 + 15) continue;  // no rows, or all of them before the block (uniform in the warp)
    // (a kept block lies before every row of a tile that has any: then every row's window starts beyond keep_first)
    float sc[MMA_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < MMA_KEYS / 8; ++n) {
      sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&ks[(n * 8 + gid) * KS + kk * 16 + 2 * tig]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&ks[(n * 8 + gid) * KS + kk * 16 + 2 * tig + 8]);
        mma_16816(sc[n], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
      }
    }
    float top[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
    for (int n = 0; n < MMA_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1, key = base + n * 8 + 2 * tig + (e & 1);
        float v = -INFINITY;
        // (without kept blocks of their own the kept keys lie inside the ordinary blocks: a later row of the tile may
        // see them although its window starts beyond them)
        if (kept ? key < keep_first : (key <= pos[r] && (key >= low[r] || (kept_blocks == 0 && key < keep_first)))) {
          v = sc[n][e] * scale;
          if (brow) {
            const int far = min(pos[r] - key, reach - 1);
            v += far < MMA_BIAS ? near_bias[far] : brow[far];
          }
        }
        sc[n][e] = v;
        top[r] = fmaxf(top[r], v);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
      top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
      const float m_new = fmaxf(m[r], top[r]);
      alpha[r] = expf(m[r] - m_new);
      m[r] = m_new;
      l[r] *= alpha[r];
    }
#pragma unroll
    for (int n = 0; n < MMA_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = expf(sc[n][e] - m[e >> 1]);  // a masked score is -inf: weight 0
        sc[n][e] = pv;
        l[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int i = 0; i < V / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < MMA_KEYS / 16; ++kk) {
      uint32_t hi[4], lo[4];
      split_bf16(sc[2 * kk][0], sc[2 * kk][1], hi[0], lo[0]);
      split_bf16(sc[2 * kk][2], sc[2 * kk][3], hi[1], lo[1]);
      split_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1], hi[2], lo[2]);
      split_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3], hi[3], lo[3]);
#pragma unroll
      for (int nv = 0; nv < V / 8; ++nv) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&vt[(nv * 8 + gid) * VS + kk * 16 + 2 * tig]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&vt[(nv * 8 + gid) * VS + kk * 16 + 2 * tig + 8]);
        mma_16816(o[nv], hi[0], hi[1], hi[2], hi[3], b0, b1);
        mma_16816(o[nv], lo[0], lo[1], lo[2], lo[3], b0, b1);
      }
    }
  }
  pdl_trigger();  // late: blocks of the next kernel waiting beside this one's few warps would only be in their way
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + gid + 8 * r;
    if (row >= nt) continue;
    const float inv = 1.f / l[r];
    __nv_bfloat16* orow = out + ((size_t)(t0 + row) * hq + h) * vdim;
#pragma unroll
    for (int nv = 0; nv < V / 8; ++nv) {
      const int c = nv * 8 + 2 * tig;
      if (c < vdim) *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16(o[nv][2 * r] * inv, o[nv][2 * r + 1] * inv);
    }
  }
}

size_t tile_smem(int dp, int vp, int share) {
  return sizeof(float) * ((size_t)dp * 33 + 32 * (size_t)vp + (size_t)TILE_T * share * dp + 2 * (size_t)TILE_T * share +
                          (size_t)TILE_T * share * vp);
}

PsbPerDevice tile_attr[4][4];

int padded(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : 256; }
int slot_of(int n) { return n == 32 ? 0 : n == 64 ? 1 : n == 128 ? 2 : 3; }

}  // namespace

// (qkv, dtype, positions, token_item, table, table_width, kv, kv_dtype, q_out, T, hq, hkv, dim, vdim, page_size, num_pages, stream)
PSB_API int psb_attention_biased_append(const void* qkv, int dtype, const void* positions, const void* token_item,
                                        const void* table, int table_width, void* kv, int kv_dtype, void* q_out, int T, int hq,
                                        int hkv, int dim, int vdim, int page_size, int num_pages, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 1 || dim < 1 || vdim < 1 || page_size < 1 || table_width < 1 || num_pages < 1)
    PSB_REFUSE("attention_biased_append: bad sizes");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_biased_append_kernel<T_, TKV>, dim3(T), dim3(128), 0, stream, (const T_*)qkv, (const int32_t*)positions,
                 (const int32_t*)token_item, (const int32_t*)table, table_width, (TKV*)kv, (T_*)q_out, hq, hkv, dim, vdim,
                 page_size, num_pages);
    });
  });
  PSB_LAUNCH_CHECK("attention_biased_append");
  return 0;
}

// ``skip_from`` > 0: tokens of portions with at least that many tokens are left to the tiled kernel (item_start needed).
// (q, dtype, kv, kv_dtype, table, table_width, positions, token_item, bias, sink, out, T, hq, hkv, dim, vdim, page_size,
//  window, chunk, reach, scale, item_start, skip_from, keep_first, partial [T * hq, splits, vdim + 2] float32 or null, splits, stream)
PSB_API int psb_attention_biased(const void* q, int dtype, const void* kv, int kv_dtype, const void* table, int table_width,
                                 const void* positions, const void* token_item, const void* bias, const void* sink, void* out,
                                 int T, int hq, int hkv, int dim, int vdim, int page_size, int window, int chunk, int reach,
                                 float scale, const void* item_start, int skip_from, int keep_first, void* partial, int splits,
                                 cudaStream_t stream) {
  if (splits < 1 || splits > MAX_KEY_SPLITS || (splits > 1 && (!partial || skip_from > 0)))
    PSB_REFUSE("attention_biased: 1 to %d shares of the keys (with their scratch, and no tokens left to another kernel), not %d", MAX_KEY_SPLITS, splits);
  if (keep_first < 0 || (keep_first > 0 && (window < 1 || chunk > 0))) PSB_REFUSE("attention_biased: kept first keys go with a window and no chunk mask");
  if (skip_from > 0 && !item_start) PSB_REFUSE("attention_biased: skipping tiled portions needs the item offsets");
  if (T < 0 || hq < 1 || hkv < 1 || hq % hkv) PSB_REFUSE("attention_biased: %d query heads cannot share %d key/value heads", hq, hkv);
  if (dim < 1 || dim > MAX_D || vdim < 1 || vdim > MAX_D) PSB_REFUSE("attention_biased: sizes %d/%d are outside [1, %d]", dim, vdim, MAX_D);
  if (page_size < 1 || table_width < 1) PSB_REFUSE("attention_biased: bad paging (page_size=%d width=%d)", page_size, table_width);
  if (window < 0 || chunk < 0 || (bias && reach < 1)) PSB_REFUSE("attention_biased: negative window or chunk, or an empty bias table");
  if (T == 0) return 0;
  const long long blocks = (long long)T * hq;
  if (blocks > 0x7fffffffLL) PSB_REFUSE("attention_biased: batch too large");
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_biased_kernel<T_, TKV>, dim3((unsigned)blocks, (unsigned)splits), dim3(WARPS * 32), 0, stream, (const T_*)q,
                 (const TKV*)kv, (const int32_t*)table, table_width, (const int32_t*)positions, (const int32_t*)token_item,
                 (const float*)bias, (const float*)sink, (T_*)out, T, hq, hkv, dim, vdim, page_size, window, chunk, reach, scale,
                 (const int32_t*)item_start, skip_from, keep_first, (float*)partial, splits);
    });
  });
  PSB_LAUNCH_CHECK("attention_biased");
  if (splits > 1) {
    PSB_DISPATCH_DTYPE(dtype, T_, {
      psb_launch(attention_biased_merge_kernel<T_>, dim3((unsigned)blocks), dim3(32), 0, stream, (const float*)partial,
                 (const float*)sink, (T_*)out, hq, vdim, splits);
    });
    PSB_LAUNCH_CHECK("attention_biased_merge");
  }
  return 0;
}

// (hq, hkv, dim, vdim) -> 1 if the tensor-core kernel for prompt portions takes the shape
PSB_API int psb_attention_biased_mma_supported(int hq, int hkv, int dim, int vdim) {
  return hq >= 1 && hkv >= 1 && hq % hkv == 0 && dim >= 8 && dim <= 128 && dim % 8 == 0 && vdim >= 8 && vdim <= 128 && vdim % 8 == 0 ? 1 : 0;
}

// The tensor-core kernel over every portion of at least ``min_tokens`` tokens (bfloat16; grid sized by an upper bound on
// the 64-token tiles).  Other tokens are left untouched.
// (q, kv, table, table_width, positions, item_start, items, T, min_tokens, bias, sink, out, hq, hkv, dim, vdim,
//  page_size, window, chunk, reach, scale, keep_first, stream)
PSB_API int psb_attention_biased_mma(const void* q, const void* kv, const void* table, int table_width, const void* positions,
                                     const void* item_start, int items, int T, int min_tokens, const void* bias, const void* sink,
                                     void* out, int hq, int hkv, int dim, int vdim, int page_size, int window, int chunk, int reach,
                                     float scale, int keep_first, cudaStream_t stream) {
  if (!psb_attention_biased_mma_supported(hq, hkv, dim, vdim)) PSB_REFUSE("attention_biased_mma: shape not taken");
  if (keep_first < 0 || (keep_first > 0 && (window < 1 || chunk > 0))) PSB_REFUSE("attention_biased_mma: kept first keys go with a window and no chunk mask");
  if (page_size < 1 || table_width < 1 || window < 0 || chunk < 0 || (bias && reach < 1)) PSB_REFUSE("attention_biased_mma: bad arguments");
  if ((((uintptr_t)q | (uintptr_t)kv) & 15) || hq > 65535) PSB_REFUSE("attention_biased_mma: operands must be 16-byte aligned");
  if (items < 1 || T < 1 || min_tokens < 1) return 0;
  const dim3 grid((T + MMA_ROWS - 1) / MMA_ROWS + items, hq), block(128);
#define MMA_CASE(D_, V_)                                                                                                       \
  psb_launch(attention_biased_mma_kernel<D_, V_>, grid, block, 0, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv,    \
             (const int32_t*)table, table_width, (const int32_t*)positions, (const int32_t*)item_start, items, min_tokens,     \
             (const float*)bias, (const float*)sink, (__nv_bfloat16*)out, hq, hkv, dim, vdim, page_size, window, chunk, reach, \
             scale, keep_first)
  if (dim <= 64 && vdim <= 64) MMA_CASE(64, 64);
  else if (dim <= 64) MMA_CASE(64, 128);
  else if (vdim <= 64) MMA_CASE(128, 64);
  else MMA_CASE(128, 128);
#undef MMA_CASE
  PSB_LAUNCH_CHECK("attention_biased_mma");
  return 0;
}

// () -> tokens a tile of the tiled kernel holds
PSB_API int psb_attention_biased_tile_tokens() { return TILE_T; }

// (hq, hkv, dim, vdim) -> 1 if the tiled kernel takes the shape
PSB_API int psb_attention_biased_tile_supported(int hq, int hkv, int dim, int vdim) {
  if (hq < 1 || hkv < 1 || hq % hkv || dim < 1 || dim > MAX_D || vdim < 1 || vdim > MAX_D) return 0;
  const int dp = padded(dim), vp = padded(vdim);
  return tile_smem(dp, vp, hq / hkv) <= 200 * 1024 ? 1 : 0;
}

// The tiled kernel over every portion of at least ``min_tokens`` tokens (the grid is sized by an upper bound on their
// tiles, so its shape depends on T and the number of items only).  Other tokens are left untouched.
// (q, kv, table, table_width, positions, item_start, items, T, min_tokens, bias, sink, out, hq, hkv, dim, vdim,
//  page_size, window, chunk, reach, scale, keep_first, stream)
PSB_API int psb_attention_biased_tiles(const void* q, const void* kv, const void* table, int table_width, const void* positions,
                                       const void* item_start, int items, int T, int min_tokens,
                                       const void* bias, const void* sink, void* out, int hq, int hkv, int dim, int vdim,
                                       int page_size, int window, int chunk, int reach, float scale, int keep_first,
                                       cudaStream_t stream) {
  if (keep_first < 0 || (keep_first > 0 && (window < 1 || chunk > 0))) PSB_REFUSE("attention_biased_tiles: kept first keys go with a window and no chunk mask");
  if (items < 1 || T < 1 || min_tokens < 1) return 0;
  const int tiles = (T + TILE_T - 1) / TILE_T + items;
  if (!psb_attention_biased_tile_supported(hq, hkv, dim, vdim)) PSB_REFUSE("attention_biased_tiles: shape not taken");
  if (page_size < 1 || table_width < 1 || window < 0 || chunk < 0 || (bias && reach < 1)) PSB_REFUSE("attention_biased_tiles: bad arguments");
  if (hkv > 65535) PSB_REFUSE("attention_biased_tiles: too many key/value heads");
  const int dp = padded(dim), vp = padded(vdim);
  const size_t smem = tile_smem(dp, vp, hq / hkv);
  const dim3 grid(tiles, hkv), block(TILE_WARPS * 32);
#define TILE_CASE(DP_, VP_)                                                                                                    \
  if (dp == DP_ && vp == VP_) {                                                                                                \
    auto kernel = attention_biased_tile_kernel<DP_, VP_>;                                                                      \
    PsbPerDevice& done = tile_attr[slot_of(DP_)][slot_of(VP_)];                                                                \
    if (!done.get()) {                                                                                                         \
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)                \
        PSB_REFUSE("attention_biased_tiles: cannot raise the shared-memory limit");                                            \
      done.set();                                                                                                              \
    }                                                                                                                          \
    psb_launch(kernel, grid, block, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv, (const int32_t*)table,    \
               table_width, (const int32_t*)positions, (const int32_t*)item_start, items, min_tokens,                          \
               (const float*)bias, (const float*)sink, (__nv_bfloat16*)out, hq, hkv, dim, vdim,                                \
               page_size, window, chunk, reach, scale, keep_first);                                                            \
    launched = true;                                                                                                           \
  }
#define TILE_ROW(DP_) TILE_CASE(DP_, 32) TILE_CASE(DP_, 64) TILE_CASE(DP_, 128) TILE_CASE(DP_, 256)
  bool launched = false;
  TILE_ROW(32) TILE_ROW(64) TILE_ROW(128) TILE_ROW(256)
#undef TILE_ROW
#undef TILE_CASE
  if (!launched) PSB_REFUSE("attention_biased_tiles: sizes %d/%d not instantiated", dim, vdim);
  PSB_LAUNCH_CHECK("attention_biased_tiles");
  return 0;
}
