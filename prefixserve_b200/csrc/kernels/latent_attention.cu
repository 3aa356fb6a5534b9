// Attention through a low-rank latent of the keys and values, with one rotated key part shared by all heads.
//
// A token's cache row holds its latent c (``rank`` numbers, already normed) followed by the rotated key part
// (``rot`` numbers): one row per token and layer, whatever the number of heads.  Layout of an entry:
// [num_pages, page_size, rank + rot].  Head h's key would be (U_k[h] c, k_rot) and its value U_v[h] c; instead of
// expanding them, the query is carried into the latent space (q' = U_k[h]^T q_plain, a batched product on the host
// side), so that
//   score(t, j) = (q'_t . c_j + q_rot_t . k_rot_j) * scale,   out_t = sum_j softmax_j(score) c_j,
// and the value matrix is applied once to out_t afterwards.  Key j is visible to the query at position p when
// 0 <= p - j < window (window 0: every earlier key).
//
// latent_prepare_kernel: one row of the fused input projection [query latent | key/value latent | rotated key part |
//   one gate per head] -> the normed query latent (compute type), the cache row (normed latent, rotated key part),
//   sigmoid of the gates (float32).  The norms are x / sqrt(mean(x^2) + eps) * gain in float32.
// latent_query_rotate_kernel: the rotated part of every head's query, turned by the token's position, into the
//   tail of the float32 query rows [T, heads, rank + rot] whose first ``rank`` columns the batched product fills.
// latent_attention_kernel: one block per (token, head) walks the visible keys in runs of 32 aligned to absolute
//   positions, the runs dealt out to its four warps in turn and the four partial results joined in warp order (the
//   order of every sum depends on the token's position only), scores and softmax in float32, the output (times the
//   head's gate) accumulated in registers.
//
// The rotation pairs element 2i with 2i+1 for i < rot_dims/2 (the rest of the rotated part passes through), angle
// tables float32 [positions, rot_dims/2].
#include <cfloat>

#include "common.cuh"

namespace {

__device__ __forceinline__ float block_total(float v, float* scratch) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += scratch[w];
  __syncthreads();
  return total;
}

template <typename T, typename TKV>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ token_item, const int32_t* __restrict__ table,
                                      int table_width, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      const float* __restrict__ gain_q, const float* __restrict__ gain_kv,
                                      T* __restrict__ cq_out, float* __restrict__ gate_out, TKV* __restrict__ cache,
                                      int q_rank, int rank, int rot, int rot_dims, int heads, int page_size,
                                      int num_pages, int max_positions, float eps, long long ld) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;  // ld >= the row's width: the row may be a run of columns of a wider product
  const int pos = positions[t];

  float ss = 0.f;
  for (int j = threadIdx.x; j < q_rank; j += blockDim.x) {
    const float v = to_float<T>(row[j]);
    ss += v * v;
  }
  const float inv_q = q_rank > 0 ? 1.f / sqrtf(block_total(ss, scratch) / (float)q_rank + eps) : 0.f;  // q_rank 0: no query latent in the row
  for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
    cq_out[(size_t)t * q_rank + j] = from_float<T>(gain_q[j] * (to_float<T>(row[j]) * inv_q));

  const T* kvrow = row + q_rank;
  ss = 0.f;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) {
    const float v = to_float<T>(kvrow[j]);
    ss += v * v;
  }
  const float inv_kv = 1.f / sqrtf(block_total(ss, scratch) / (float)rank + eps);

  const int item = token_item[t];
  const int page = pos >= 0 ? table[(size_t)item * table_width + pos / page_size] : -1;
  // the host checks tables before launch; a bad id is skipped rather than written through
  if (page >= 0 && page < num_pages) {
    TKV* dst = cache + ((size_t)page * page_size + (size_t)(pos % page_size)) * (rank + rot);
    for (int j = threadIdx.x; j < rank; j += blockDim.x)
      dst[j] = from_float<TKV>(gain_kv[j] * (to_float<T>(kvrow[j]) * inv_kv));
    const int safe_pos = pos >= max_positions ? max_positions - 1 : pos;
    const int half = rot_dims >> 1;
    const float* c = cos_t + (size_t)safe_pos * half;
    const float* s = sin_t + (size_t)safe_pos * half;
    const T* kr = kvrow + rank;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float o1, o2;
      rotate_pair(to_float<T>(kr[2 * j]), to_float<T>(kr[2 * j + 1]), c[j], s[j], o1, o2);
      dst[rank + 2 * j] = from_float<TKV>(o1);
      dst[rank + 2 * j + 1] = from_float<TKV>(o2);
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) dst[rank + j] = from_float<TKV>(to_float<T>(kr[j]));
  }
  const T* g = kvrow + rank + rot;
  for (int j = threadIdx.x; j < heads; j += blockDim.x) gate_out[(size_t)t * heads + j] = 1.f / (1.f + expf(-to_float<T>(g[j])));
}

template <typename T>
__global__ void latent_query_rotate_kernel(const T* __restrict__ q, const int32_t* __restrict__ positions,
                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                           float* __restrict__ q_lat, int heads, int plain, int rot, int rot_dims, int rank,
                                           int max_positions, long long ldq) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int safe_pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
  const int half = rot_dims >> 1;
  const float* c = cos_t + (size_t)safe_pos * half;
  const float* s = sin_t + (size_t)safe_pos * half;
  const int per_head = half + (rot - rot_dims);  // work items a head: the pairs, then the elements that pass through
  for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, j = idx - h * per_head;
    const T* src = q + (size_t)t * ldq + (size_t)h * (plain + rot) + plain;  // ldq >= heads * (plain + rot)
    float* dst = q_lat + ((size_t)t * heads + h) * (rank + rot) + rank;
    if (j < half) {
      float o1, o2;
      rotate_pair(to_float<T>(src[2 * j]), to_float<T>(src[2 * j + 1]), c[j], s[j], o1, o2);
      dst[2 * j] = o1;
      dst[2 * j + 1] = o2;
    } else {
      const int e = rot_dims + (j - half);
      dst[e] = to_float<T>(src[e]);
    }
  }
}

constexpr int WARPS = 4;

// dot of a float32 query (shared memory) with a cached row, eight elements a load where the row allows it
template <typename TKV>
__device__ __forceinline__ float row_dot(const float* __restrict__ qs, const TKV* __restrict__ krow, int D, bool vec) {
  float dot = 0.f;
  int d = 0;
  if (vec) {
    for (; d + 8 <= D; d += 8) {
      float k[8];
      if constexpr (sizeof(TKV) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          k[2 * i] = f.x;
          k[2 * i + 1] = f.y;
        }
      } else {
        const float4 a = *reinterpret_cast<const float4*>(krow + d), b = *reinterpret_cast<const float4*>(krow + d + 4);
        k[0] = a.x; k[1] = a.y; k[2] = a.z; k[3] = a.w; k[4] = b.x; k[5] = b.y; k[6] = b.z; k[7] = b.w;
      }
      const float4 q0 = *reinterpret_cast<const float4*>(qs + d), q1 = *reinterpret_cast<const float4*>(qs + d + 4);
      dot = fmaf(q0.x, k[0], dot); dot = fmaf(q0.y, k[1], dot); dot = fmaf(q0.z, k[2], dot); dot = fmaf(q0.w, k[3], dot);
      dot = fmaf(q1.x, k[4], dot); dot = fmaf(q1.y, k[5], dot); dot = fmaf(q1.z, k[6], dot); dot = fmaf(q1.w, k[7], dot);
    }
  }
  for (; d < D; ++d) dot = fmaf(qs[d], to_float<TKV>(krow[d]), dot);
  return dot;
}

// One block per (token, head).  Its four warps take the runs of 32 keys in turn (run r goes to warp r mod 4), each
// with a running maximum, sum and output of its own; the four are then joined in warp order.  Lane l of a warp owns
// output columns 2l, 2l+1, 2l+64, ... (pairs, so that a bfloat16 row is read four bytes at a time).
template <typename TKV, typename TO, int NACC>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const float* __restrict__ q_lat, const TKV* __restrict__ cache, const int32_t* __restrict__ table,
                        int table_width, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                        const float* __restrict__ gate, TO* __restrict__ out, int T_tokens, int heads, int rank, int rot,
                        int page_size, int num_pages, int window, float scale, const float* __restrict__ sink) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = rank + rot;
  const int Dpad = (D + 3) & ~3;
  float* qs = smem;                         // [Dpad]
  float* part_ml = smem + Dpad;             // [WARPS][2]
  float* part_o = part_ml + 2 * WARPS;      // [WARPS][rank]
  const int t = blockIdx.x / heads, h = blockIdx.x - t * heads;
  const int p = positions[t];
  const int32_t* pages = table + (size_t)token_item[t] * table_width;
  const float* qrow = q_lat + ((size_t)t * heads + h) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qrow[d];
  __syncthreads();

  const bool vec = (D % 8 == 0);  // rows then start on 16-byte boundaries (the cache's base is aligned by its allocator)
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float m = -FLT_MAX, l = 0.f;
  float acc[NACC][2];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i][0] = acc[i][1] = 0.f;

  for (int base = (lo & ~31) + 32 * warp; base <= p; base += 32 * WARPS) {
    const int key = base + lane;
    const bool live = key >= lo && key <= p;
    long long off = -1;  // element offset of this lane's key row
    float s = -FLT_MAX;
    if (live) {
      const int page = pages[key / page_size];
      if (page >= 0 && page < num_pages) {
        off = ((long long)page * page_size + (key % page_size)) * D;
        s = row_dot<TKV>(qs, cache + off, D, vec) * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);   // first run: exp(-huge) = 0
    const float pr = off >= 0 ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      acc[i][0] *= alpha;
      acc[i][1] *= alpha;
    }
    const int n_live = min(32, p - base + 1);
    for (int j = 0; j < n_live; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pr, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;  // before the window
      const TKV* vrow = cache + oj;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d + 1 < rank) {
          if constexpr (sizeof(TKV) == 2) {
            if ((D & 1) == 0) {
              const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vrow + d));
              acc[i][0] = fmaf(pj, v.x, acc[i][0]);
              acc[i][1] = fmaf(pj, v.y, acc[i][1]);
              continue;
            }
          }
          acc[i][0] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i][0]);
          acc[i][1] = fmaf(pj, to_float<TKV>(vrow[d + 1]), acc[i][1]);
        } else if (d < rank) {
          acc[i][0] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i][0]);
        }
      }
    }
  }
  // join the four warps' partial results in warp order
  if (lane == 0) {
    part_ml[2 * warp] = m;
    part_ml[2 * warp + 1] = l;
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = 2 * lane + 64 * i;
    if (d < rank) part_o[(size_t)warp * rank + d] = acc[i][0];
    if (d + 1 < rank) part_o[(size_t)warp * rank + d + 1] = acc[i][1];
  }
  __syncthreads();
  // ``sink`` (a score per head, optional): one more term of the denominator, without a key or a value
  float m_all = sink ? sink[h] : -FLT_MAX;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, part_ml[2 * w]);
  float f[WARPS], l_all = sink ? expf(sink[h] - m_all) : 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    f[w] = part_ml[2 * w + 1] > 0.f ? expf(part_ml[2 * w] - m_all) : 0.f;
    l_all += part_ml[2 * w + 1] * f[w];
  }
  const float wgt = (gate ? gate[(size_t)t * heads + h] : 1.f) / l_all;
  TO* orow = out + ((size_t)t * heads + h) * rank;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += part_o[(size_t)w * rank + d] * f[w];
    orow[d] = from_float<TO>(v * wgt);
  }
}

// The same attention for bfloat16 rows whose sizes are multiples of eight (the usual case): a warp takes four keys at
// a time and reads each row once, 16 bytes a lane, side by side (lane l holds elements 8l..8l+7, 8(l+32).., of the row
// and of the query); the four scores are finished by a butterfly over the warp, and the weighted sum is accumulated
// from the very registers the scores were computed from.  A block is one token and one head or two (two where the
// head count is even: both use every row the block loads); its eight warps take the groups of four keys in turn,
// counted from the first visible key, and are joined in warp order at the end.
constexpr int ROW_WARPS = 8;
constexpr int GROUP = 4;

template <typename TO, int NP, int HP>
__global__ void __launch_bounds__(ROW_WARPS * 32)
latent_attention_rows_kernel(const float* __restrict__ q_lat, const __nv_bfloat16* __restrict__ cache,
                             const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ positions,
                             const int32_t* __restrict__ token_item, const float* __restrict__ gate, TO* __restrict__ out,
                             float* __restrict__ partial, int heads, int rank, int rot, int page_size, int num_pages,
                             int window, float scale, const float* __restrict__ sink) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = rank + rot, pieces = D >> 3, value_pieces = rank >> 3;
  const int splits = gridDim.y, split = blockIdx.y;  // several blocks may share a (token, heads): each takes every splits-th turn
  float* part_ml = smem;                          // [HP][ROW_WARPS][2]
  float* part_o = smem + 2 * ROW_WARPS * HP;      // [HP][ROW_WARPS][rank]
  const int per_token = heads / HP;               // HP heads of a token share a block and every row it loads
  const int t = blockIdx.x / per_token, h0 = (blockIdx.x - t * per_token) * HP;
  const int p = positions[t];
  const int32_t* pages = table + (size_t)token_item[t] * table_width;
  float q[HP][NP][8];
#pragma unroll
  for (int hh = 0; hh < HP; ++hh) {
    const float* qrow = q_lat + ((size_t)t * heads + h0 + hh) * D;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int c = lane + 32 * i;
      if (c < pieces) {
        const float4 a = *reinterpret_cast<const float4*>(qrow + 8 * c), b = *reinterpret_cast<const float4*>(qrow + 8 * c + 4);
        q[hh][i][0] = a.x * scale; q[hh][i][1] = a.y * scale; q[hh][i][2] = a.z * scale; q[hh][i][3] = a.w * scale;
        q[hh][i][4] = b.x * scale; q[hh][i][5] = b.y * scale; q[hh][i][6] = b.z * scale; q[hh][i][7] = b.w * scale;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) q[hh][i][e] = 0.f;
      }
    }
  }
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int nkeys = p - lo + 1;
  float m[HP], l[HP];
  float acc[HP][NP][8];
#pragma unroll
  for (int hh = 0; hh < HP; ++hh) {
    m[hh] = -FLT_MAX;
    l[hh] = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[hh][i][e] = 0.f;
  }

  for (int g = (split * ROW_WARPS + warp) * GROUP; g < nkeys; g += splits * ROW_WARPS * GROUP) {
    uint4 r[GROUP][NP];
    bool live[GROUP];
#pragma unroll
    for (int k = 0; k < GROUP; ++k) {
      const int key = lo + g + k;
      live[k] = g + k < nkeys;
      const __nv_bfloat16* row = nullptr;
      if (live[k]) {
        const int page = pages[key / page_size];
        live[k] = page >= 0 && page < num_pages;
        if (live[k]) row = cache + ((size_t)page * page_size + (key % page_size)) * D;
      }
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int c = lane + 32 * i;
        r[k][i] = (live[k] && c < pieces) ? *reinterpret_cast<const uint4*>(row + 8 * c) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int hh = 0; hh < HP; ++hh) {
      float s[GROUP];
#pragma unroll
      for (int k = 0; k < GROUP; ++k) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r[k][i]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            dot = fmaf(q[hh][i][2 * e], f.x, dot);
            dot = fmaf(q[hh][i][2 * e + 1], f.y, dot);
          }
        }
        s[k] = dot;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < GROUP; ++k) s[k] += __shfl_xor_sync(0xffffffffu, s[k], o);
      float m_new = m[hh];
#pragma unroll
      for (int k = 0; k < GROUP; ++k) m_new = live[k] ? fmaxf(m_new, s[k]) : m_new;
      const float alpha = expf(m[hh] - m_new);
      float pk[GROUP], add = 0.f;
#pragma unroll
      for (int k = 0; k < GROUP; ++k) {
        pk[k] = live[k] ? expf(s[k] - m_new) : 0.f;
        add += pk[k];
      }
      l[hh] = l[hh] * alpha + add;
      m[hh] = m_new;
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        if (lane + 32 * i < value_pieces) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[hh][i][e] *= alpha;
#pragma unroll
          for (int k = 0; k < GROUP; ++k) {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r[k][i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h2[e]);
              acc[hh][i][2 * e] = fmaf(pk[k], f.x, acc[hh][i][2 * e]);
              acc[hh][i][2 * e + 1] = fmaf(pk[k], f.y, acc[hh][i][2 * e + 1]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int hh = 0; hh < HP; ++hh) {
    if (lane == 0) {
      part_ml[2 * (hh * ROW_WARPS + warp)] = m[hh];
      part_ml[2 * (hh * ROW_WARPS + warp) + 1] = l[hh];
    }
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int c = lane + 32 * i;
      if (c < value_pieces) {
#pragma unroll
        for (int e = 0; e < 8; ++e) part_o[((size_t)hh * ROW_WARPS + warp) * rank + 8 * c + e] = acc[hh][i][e];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < HP; ++hh) {
    const float* ml = part_ml + 2 * hh * ROW_WARPS;
    float m_all = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < ROW_WARPS; ++w) m_all = fmaxf(m_all, ml[2 * w]);
    float f[ROW_WARPS], l_all = 0.f;
#pragma unroll
    for (int w = 0; w < ROW_WARPS; ++w) {
      f[w] = ml[2 * w + 1] > 0.f ? expf(ml[2 * w] - m_all) : 0.f;
      l_all += ml[2 * w + 1] * f[w];
    }
    if (splits > 1) {  // this block's share: maximum, sum and the weighted sum as it stands; the merge kernel joins the shares
      float* mine = partial + (((size_t)t * heads + h0 + hh) * splits + split) * (rank + 2);
      if (threadIdx.x == 0) {
        mine[0] = m_all;
        mine[1] = l_all;
      }
      for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ROW_WARPS; ++w) v += part_o[((size_t)hh * ROW_WARPS + w) * rank + d] * f[w];
        mine[2 + d] = v;
      }
      continue;
    }
    if (sink) {  // the sink joins the denominator where a (token, head)'s keys are whole (else in the merge kernel)
      const float sk = sink[h0 + hh], top = fmaxf(m_all, sk);
      const float down = expf(m_all - top);
      l_all = l_all * down + expf(sk - top);
#pragma unroll
      for (int w = 0; w < ROW_WARPS; ++w) f[w] *= down;
    }
    const float wgt = (gate ? gate[(size_t)t * heads + h0 + hh] : 1.f) / l_all;
    TO* orow = out + ((size_t)t * heads + h0 + hh) * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < ROW_WARPS; ++w) v += part_o[((size_t)hh * ROW_WARPS + w) * rank + d] * f[w];
      orow[d] = from_float<TO>(v * wgt);
    }
  }
}

// Joins the shares of the blocks that split a (token, head)'s keys among them, in split order.
constexpr int MAX_SPLITS = 8;

template <typename TO>
__global__ void latent_attention_merge_kernel(const float* __restrict__ partial, const float* __restrict__ gate,
                                              TO* __restrict__ out, int rank, int splits, const float* __restrict__ sink,
                                              int heads) {
  pdl_trigger();
  pdl_wait();
  const size_t unit = blockIdx.x;  // token * heads + head
  const float* mine = partial + unit * splits * (rank + 2);
  const float sk = sink ? sink[unit % heads] : -FLT_MAX;
  float m_all = sk;
  for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, mine[(size_t)s * (rank + 2)]);
  float f[MAX_SPLITS], l_all = sink ? expf(sk - m_all) : 0.f;
#pragma unroll
  for (int s = 0; s < MAX_SPLITS; ++s) {
    f[s] = 0.f;
    if (s < splits) {
      const float l = mine[(size_t)s * (rank + 2) + 1];
      f[s] = l > 0.f ? expf(mine[(size_t)s * (rank + 2)] - m_all) : 0.f;
      l_all += l * f[s];
    }
  }
  const float wgt = (gate ? gate[unit] : 1.f) / l_all;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s)
      if (s < splits) v += mine[(size_t)s * (rank + 2) + 2 + d] * f[s];
    out[unit * rank + d] = from_float<TO>(v * wgt);
  }
}

// ---- long portions: the band of keys a run of consecutive tokens can see, as matrix products -----------------------
// A run of n consecutive tokens of one request, the first at position p0, sees keys p0 - window + 1 .. p0 + n - 1:
// a band of window + n - 1 rows whatever p0 is.  The rows are gathered from the pages into one matrix (rows before the
// sequence's start are zero and masked), the scores of all (token, head) rows against the band and the weighted
// sums are products on the tensor cores (the library's), and the softmax between them is done here in float32.
// The latent-space query enters its product as bfloat16, like any projection's result; the attention weights enter
// theirs as pairs (hi | lo) of bfloat16 with hi + lo equal to the float32 weight to 16 bits, against the value rows
// stacked twice, so that the weights are not cut to 8 bits on the way.

template <typename TKV>
__global__ void latent_band_gather_kernel(const TKV* __restrict__ cache, const int32_t* __restrict__ table, int table_width,
                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                                          TKV* __restrict__ band, TKV* __restrict__ values2, int t0, int n, int KP, int D,
                                          int rank, int page_size, int num_pages, int window) {
  pdl_trigger();
  pdl_wait();
  const int j = blockIdx.x;
  const int p0 = positions[t0];
  const int kp = p0 - window + 1 + j;
  TKV* dst = band + (size_t)j * D;
  TKV* v1 = values2 + (size_t)j * rank;          // the value part once more, twice: rows j and KP + j of [2 KP, rank],
  TKV* v2 = values2 + (size_t)(KP + j) * rank;   // the other operand of the weights' (hi | lo) pairs
  const TKV* src = nullptr;
  if (kp >= 0 && kp <= p0 + n - 1) {
    const int page = table[(size_t)token_item[t0] * table_width + kp / page_size];
    if (page >= 0 && page < num_pages) src = cache + ((size_t)page * page_size + (kp % page_size)) * D;
  }
  if (D % 8 == 0 && rank % 8 == 0 && sizeof(TKV) == 2) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int d = threadIdx.x; d < D / 8; d += blockDim.x) {
      const uint4 v = src ? reinterpret_cast<const uint4*>(src)[d] : zero;
      reinterpret_cast<uint4*>(dst)[d] = v;
      if (d < rank / 8) {
        reinterpret_cast<uint4*>(v1)[d] = v;
        reinterpret_cast<uint4*>(v2)[d] = v;
      }
    }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const TKV v = src ? src[d] : from_float<TKV>(0.f);
      dst[d] = v;
      if (d < rank) {
        v1[d] = v;
        v2[d] = v;
      }
    }
  }
}

__global__ void split_pairs_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                   size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    if (lo) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
  }
}

// One block per (token, head) row of the score matrix [rows, KP]; writes the softmax weights as (hi | lo) pairs into
// [rows, 2 KP], zero where the key is not visible.  A thread keeps its scores in registers between the passes (up to
// PER each; longer rows are read again).
constexpr int BAND_PER = 16;

__global__ void __launch_bounds__(128)
latent_band_softmax_kernel(const float* __restrict__ scores, const int32_t* __restrict__ positions,
                           __nv_bfloat16* __restrict__ weights, int t0, int heads, int KP, int window, float scale,
                           const float* __restrict__ sink) {
  __shared__ float scratch[8];
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int t = t0 + (int)(row / heads);
  const int p0 = positions[t0], p = positions[t];
  // column j holds key p0 - window + 1 + j; the row sees keys max(0, p - window + 1) .. p
  const int first = max(0, p - window + 1) - (p0 - window + 1), last = p - (p0 - window + 1);
  const float* a = scores + row * KP;
  const bool held = KP <= BAND_PER * 128;
  float v[BAND_PER];
  float m = -FLT_MAX;
  if (held) {
#pragma unroll
    for (int i = 0; i < BAND_PER; ++i) {
      const int j = threadIdx.x + 128 * i;
      v[i] = (j >= first && j <= last) ? a[j] * scale : -FLT_MAX;
      m = fmaxf(m, v[i]);
    }
  } else {
    for (int j = first + threadIdx.x; j <= last; j += blockDim.x) m = fmaxf(m, a[j] * scale);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(scratch[0], scratch[1]), fmaxf(scratch[2], scratch[3]));
  const float sk = sink ? sink[row % heads] : -FLT_MAX;  // a score per head that joins the denominator without a key
  m = fmaxf(m, sk);
  __syncthreads();
  float l = 0.f;
  if (held) {
#pragma unroll
    for (int i = 0; i < BAND_PER; ++i) {
      v[i] = v[i] > -FLT_MAX ? expf(v[i] - m) : 0.f;
      l += v[i];
    }
  } else {
    for (int j = first + threadIdx.x; j <= last; j += blockDim.x) l += expf(a[j] * scale - m);
  }
  l = warp_sum(l);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = l;
  __syncthreads();
  l = (scratch[0] + scratch[1]) + (scratch[2] + scratch[3]);
  if (sink) l += expf(sk - m);
  const float inv = 1.f / l;
  __nv_bfloat16* hi = weights + row * 2 * KP;
  __nv_bfloat16* lo = hi + KP;
  if (held) {
#pragma unroll
    for (int i = 0; i < BAND_PER; ++i) {
      const int j = threadIdx.x + 128 * i;
      if (j < KP) {
        const float w = v[i] * inv;
        const __nv_bfloat16 h = __float2bfloat16_rn(w);
        hi[j] = h;
        lo[j] = __float2bfloat16_rn(w - __bfloat162float(h));
      }
    }
  } else {
    for (int j = threadIdx.x; j < KP; j += blockDim.x) {
      const float w = (j >= first && j <= last) ? expf(a[j] * scale - m) * inv : 0.f;
      const __nv_bfloat16 h = __float2bfloat16_rn(w);
      hi[j] = h;
      lo[j] = __float2bfloat16_rn(w - __bfloat162float(h));
    }
  }
}

template <typename TO>
__global__ void latent_band_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, TO* __restrict__ out,
                                          int rank, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float g = gate ? gate[i / rank] : 1.f;
    out[i] = from_float<TO>(o[i] * g);
  }
}

}  // namespace

PSB_API int psb_latent_prepare(const void* proj, int dtype, const void* positions, const void* token_item, const void* table,
                               int table_width, const void* cos_t, const void* sin_t, const void* gain_q,
                               const void* gain_kv, void* cq_out, void* gate_out, void* cache, int cache_dtype, int T,
                               int q_rank, int rank, int rot, int rot_dims, int heads, int page_size, int num_pages,
                               int max_positions, float eps, long long ld, cudaStream_t stream) {
  if (ld < (long long)q_rank + rank + rot + heads) PSB_REFUSE("latent_prepare: row stride %lld is shorter than the row", ld);
  if (T < 0 || q_rank < 0 || rank < 1 || rot < 0 || heads < 0) PSB_REFUSE("latent_prepare: bad sizes T=%d q_rank=%d rank=%d rot=%d heads=%d", T, q_rank, rank, rot, heads);
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) PSB_REFUSE("latent_prepare: %d rotated dimensions must be even and within the rotated part of %d", rot_dims, rot);
  if (rot_dims > 0 && (!cos_t || !sin_t || max_positions < 1)) PSB_REFUSE("latent_prepare: angle tables missing");
  if (page_size < 1 || num_pages < 1 || table_width < 1) PSB_REFUSE("latent_prepare: bad paging (page_size=%d pages=%d width=%d)", page_size, num_pages, table_width);
  if (!(eps > 0.f)) PSB_REFUSE("latent_prepare: eps must be positive");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(cache_dtype, TKV, {
      psb_launch(latent_prepare_kernel<T_, TKV>, dim3(T), dim3(q_rank + rank >= 1024 ? 512 : 128), 0, stream, (const T_*)proj, (const int32_t*)positions,
                 (const int32_t*)token_item, (const int32_t*)table, table_width, (const float*)cos_t, (const float*)sin_t,
                 (const float*)gain_q, (const float*)gain_kv, (T_*)cq_out, (float*)gate_out, (TKV*)cache, q_rank, rank, rot,
                 rot_dims, heads, page_size, num_pages, max_positions, eps, ld);
    });
  });
  PSB_LAUNCH_CHECK("latent_prepare");
  return 0;
}

PSB_API int psb_latent_query_rotate(const void* q, int dtype, const void* positions, const void* cos_t, const void* sin_t,
                                    void* q_lat, int T, int heads, int plain, int rot, int rot_dims, int rank,
                                    int max_positions, long long ldq, cudaStream_t stream) {
  if (T < 0 || heads < 1 || plain < 1 || rot < 0 || rank < 1) PSB_REFUSE("latent_query_rotate: bad sizes");
  if (ldq < (long long)heads * (plain + rot)) PSB_REFUSE("latent_query_rotate: row stride %lld is shorter than the row", ldq);
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) PSB_REFUSE("latent_query_rotate: %d rotated dimensions must be even and within %d", rot_dims, rot);
  if (rot_dims > 0 && (!cos_t || !sin_t || max_positions < 1)) PSB_REFUSE("latent_query_rotate: angle tables missing");
  if (T == 0 || rot == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    psb_launch(latent_query_rotate_kernel<T_>, dim3(T), dim3(128), 0, stream, (const T_*)q, (const int32_t*)positions,
               (const float*)cos_t, (const float*)sin_t, (float*)q_lat, heads, plain, rot, rot_dims, rank, max_positions, ldq);
  });
  PSB_LAUNCH_CHECK("latent_query_rotate");
  return 0;
}

PSB_API int psb_latent_attention_max_rank() { return 1024; }

// 1 if the kernel that reads four rows side by side takes the case (bfloat16 rows, sizes in multiples of eight)
PSB_API int psb_latent_attention_rows_supported(int cache_dtype, int rank, int rot) {
  return cache_dtype == PSB_BF16 && rank % 8 == 0 && rot % 8 == 0 && rank + rot <= 1024;
}

// ``heads_per_block`` (1 or 2) and ``splits`` (1..8 blocks sharing a (token, heads)'s keys, with ``partial``
// float32 [T, heads, splits, rank + 2] as their meeting place) only matter where that kernel runs.
PSB_API int psb_latent_attention(const void* q_lat, const void* cache, int cache_dtype, const void* table, int table_width,
                                 const void* positions, const void* token_item, const void* gate, void* out, int out_dtype,
                                 int T, int heads, int rank, int rot, int page_size, int num_pages, int window, float scale,
                                 int heads_per_block, int splits, void* partial, const void* sink, cudaStream_t stream) {
  if (T < 0 || heads < 1 || rank < 1 || rot < 0) PSB_REFUSE("latent_attention: bad sizes T=%d heads=%d rank=%d rot=%d", T, heads, rank, rot);
  if (rank > 1024 || rank + rot > 2048) PSB_REFUSE("latent_attention: a latent of %d (+%d rotated) is beyond this kernel (1024, 2048 together)", rank, rot);
  if (page_size < 1 || num_pages < 1 || table_width < 1) PSB_REFUSE("latent_attention: bad paging (page_size=%d pages=%d width=%d)", page_size, num_pages, table_width);
  if (window < 0) PSB_REFUSE("latent_attention: negative window");
  if (T == 0) return 0;
  const long long blocks = (long long)T * heads;
  if (blocks > 0x7fffffffLL) PSB_REFUSE("latent_attention: batch too large");
  if ((uintptr_t)cache & 15) PSB_REFUSE("latent_attention: the cache entry must be 16-byte aligned");
  if (psb_latent_attention_rows_supported(cache_dtype, rank, rot) && ((uintptr_t)q_lat & 15) == 0) {
    // two heads of a token may share a block (and every row it loads) where the head count is even and registers allow
    const int hp = heads_per_block;
    if (hp < 1 || hp > 2 || heads % hp || (hp == 2 && rank + rot > 768)) PSB_REFUSE("latent_attention: %d heads a block do not go with %d heads of %d", hp, heads, rank + rot);
    if (splits < 1 || splits > MAX_SPLITS || (splits > 1 && !partial)) PSB_REFUSE("latent_attention: 1 to %d splits (with their scratch), not %d", MAX_SPLITS, splits);
    const size_t bytes = (size_t)hp * (2 * ROW_WARPS + (size_t)ROW_WARPS * rank) * sizeof(float);
    const int np = (rank + rot + 255) / 256;
    const long long row_blocks = blocks / hp;
#define LATENT_ROWS(NP, HP)                                                                                              \
    do {                                                                                                                 \
      static PsbPerDevice big;                                                                                           \
      PSB_DISPATCH_DTYPE(out_dtype, TO, {                                                                                \
        if (bytes > 48 * 1024 && !big.get()) {                                                                           \
          if (cudaFuncSetAttribute(latent_attention_rows_kernel<TO, NP, HP>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                   96 * 1024) != cudaSuccess)                                                            \
            PSB_REFUSE("latent_attention: cannot reserve %d bytes of shared memory", (int)bytes);                        \
          big.set();                                                                                                     \
        }                                                                                                                \
        psb_launch(latent_attention_rows_kernel<TO, NP, HP>, dim3((unsigned)row_blocks, splits), dim3(ROW_WARPS * 32),   \
                   bytes, stream, (const float*)q_lat, (const __nv_bfloat16*)cache, (const int32_t*)table, table_width,  \
                   (const int32_t*)positions, (const int32_t*)token_item, (const float*)gate, (TO*)out, (float*)partial, \
                   heads, rank, rot, page_size, num_pages, window, scale, (const float*)sink);                           \
      });                                                                                                                \
    } while (0)
    if (hp == 2) {
      if (np == 1) LATENT_ROWS(1, 2); else if (np == 2) LATENT_ROWS(2, 2); else LATENT_ROWS(3, 2);
    } else {
      if (np == 1) LATENT_ROWS(1, 1); else if (np == 2) LATENT_ROWS(2, 1); else if (np == 3) LATENT_ROWS(3, 1); else LATENT_ROWS(4, 1);
    }
#undef LATENT_ROWS
    PSB_LAUNCH_CHECK("latent_attention");
    if (splits > 1) {
      PSB_DISPATCH_DTYPE(out_dtype, TO, {
        psb_launch(latent_attention_merge_kernel<TO>, dim3((unsigned)blocks), dim3(128), 0, stream, (const float*)partial,
                   (const float*)gate, (TO*)out, rank, splits, (const float*)sink, heads);
      });
      PSB_LAUNCH_CHECK("latent_attention_merge");
    }
    return 0;
  }
  const size_t smem = ((size_t)((rank + rot + 3) & ~3) + 2 * WARPS + (size_t)WARPS * rank) * sizeof(float);
#define LATENT_LAUNCH(NACC)                                                                                              \
  PSB_DISPATCH_DTYPE(cache_dtype, TKV, {                                                                                 \
    PSB_DISPATCH_DTYPE(out_dtype, TO, {                                                                                  \
      psb_launch(latent_attention_kernel<TKV, TO, NACC>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, stream,        \
                 (const float*)q_lat, (const TKV*)cache, (const int32_t*)table, table_width, (const int32_t*)positions,  \
                 (const int32_t*)token_item, (const float*)gate, (TO*)out, T, heads, rank, rot, page_size, num_pages,    \
                 window, scale, (const float*)sink);                                                                     \
    });                                                                                                                  \
  })
  if (rank <= 128) { LATENT_LAUNCH(2); }        // NACC pairs of columns a lane: 64 columns each
  else if (rank <= 256) { LATENT_LAUNCH(4); }
  else if (rank <= 512) { LATENT_LAUNCH(8); }
  else { LATENT_LAUNCH(16); }
#undef LATENT_LAUNCH
  PSB_LAUNCH_CHECK("latent_attention");
  return 0;
}

// The band of keys that tokens t0 .. t0+n-1 (one request, consecutive) can see: ``band`` [KP, D] (KP >= window + n - 1)
// and its value part twice over, ``values2`` [2 KP, rank].
PSB_API int psb_latent_band_gather(const void* cache, int dtype, const void* table, int table_width, const void* positions,
                                   const void* token_item, void* band, void* values2, int t0, int n, int KP, int D, int rank,
                                   int page_size, int num_pages, int window, cudaStream_t stream) {
  if (t0 < 0 || n < 1 || window < 1 || KP < window + n - 1 || D < 1 || rank < 1 || rank > D || page_size < 1 || num_pages < 1 || table_width < 1)
    PSB_REFUSE("latent_band_gather: bad sizes t0=%d n=%d window=%d rows=%d D=%d rank=%d", t0, n, window, KP, D, rank);
  if (((uintptr_t)cache | (uintptr_t)band | (uintptr_t)values2) & 15) PSB_REFUSE("latent_band_gather: cache and band must be 16-byte aligned");
  PSB_DISPATCH_DTYPE(dtype, TKV, {
    psb_launch(latent_band_gather_kernel<TKV>, dim3(KP), dim3(64), 0, stream, (const TKV*)cache, (const int32_t*)table,
               table_width, (const int32_t*)positions, (const int32_t*)token_item, (TKV*)band, (TKV*)values2, t0, n, KP, D, rank,
               page_size, num_pages, window);
  });
  PSB_LAUNCH_CHECK("latent_band_gather");
  return 0;
}

// float32 -> bfloat16 (hi) and, if asked for, the bfloat16 nearest to what that rounding lost (lo)
PSB_API int psb_split_pairs(const void* x, void* hi, void* lo, long long total, cudaStream_t stream) {
  if (total < 0) PSB_REFUSE("split_pairs: negative size");
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  psb_launch(split_pairs_kernel, dim3((unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks)), dim3(256), 0, stream, (const float*)x,
             (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, (size_t)total);
  PSB_LAUNCH_CHECK("split_pairs");
  return 0;
}

PSB_API int psb_latent_band_softmax(const void* scores, const void* positions, void* weights, int t0, int n, int heads, int KP,
                                    int window, float scale, const void* sink, cudaStream_t stream) {
  if (t0 < 0 || n < 1 || heads < 1 || window < 1 || KP < window + n - 1) PSB_REFUSE("latent_band_softmax: bad sizes");
  psb_launch(latent_band_softmax_kernel, dim3((unsigned)((long long)n * heads)), dim3(128), 0, stream, (const float*)scores,
             (const int32_t*)positions, (__nv_bfloat16*)weights, t0, heads, KP, window, scale, (const float*)sink);
  PSB_LAUNCH_CHECK("latent_band_softmax");
  return 0;
}

PSB_API int psb_latent_band_finish(const void* o, const void* gate, void* out, int out_dtype, int rank, long long total,
                                   cudaStream_t stream) {
  if (total < 0 || rank < 1) PSB_REFUSE("latent_band_finish: bad sizes");
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  PSB_DISPATCH_DTYPE(out_dtype, TO, {
    psb_launch(latent_band_finish_kernel<TO>, dim3((unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks)), dim3(256), 0, stream,
               (const float*)o, (const float*)gate, (TO*)out, rank, (size_t)total);
  });
  PSB_LAUNCH_CHECK("latent_band_finish");
  return 0;
}
