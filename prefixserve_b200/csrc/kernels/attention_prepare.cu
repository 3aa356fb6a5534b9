// What lies between the fused projection of an attention layer and its scores, for designs that do more to queries
// and keys than rotate them: per token, in one pass over the projection's row [q | k | v] (or [q | k] where the
// projected keys serve as values),
//
//   rotation of the first ``rotary_dim`` elements of every query and key head by the token's absolute position
//     (optional; ``interleaved``: element 2i turns with 2i+1, else i with i + rotary_dim/2);
//   division of every query and key head by the root of (its mean square + eps)   (optional: eps < 0 leaves it out);
//   a factor per query head (optional), so that a head's scores come out multiplied by it;
//   the query written to q_out [T, hq, dim]; the key, then the value, to the token's row of the cache entry
//     [num_pages, 1, hkv, page_size, dim + vdim], the value being the head's own projection or, with
//     ``values_are_keys``, the key as it was projected (before rotation and norm).  With ``split_planes`` (vdim == dim)
//     the entry is [num_pages, 2, hkv, page_size, dim] instead, keys in plane 0 and values in plane 1: the layout of
//     the attention kernels that read keys and values as separate tiles.
//
// Two kernels.  The general one: one block per token, a warp per head in turn; the head lies in the warp's
// shared-memory row between the steps.  The other, for heads of 64, 128 or 256 elements whose rotation (if any) pairs
// neighbours: the head in registers, 32 or 16 lanes a head (every lane a run of elements, which holds whole pairs), one
// wide load and one wide store per lane and row, a warp taking one or several heads.
// Rotation, statistics and factors are float32; storage is float32 or bfloat16.
#include "common.cuh"

namespace {

constexpr int PREP_WARPS = 4;
constexpr int PREP_MAX_D = 256;

template <typename T, typename TKV>
__global__ void __launch_bounds__(PREP_WARPS * 32)
attention_prepare_kernel(const T* __restrict__ proj, long long ld, const int32_t* __restrict__ positions,
                         const int32_t* __restrict__ token_item, const int32_t* __restrict__ table, int table_width,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, const float* __restrict__ head_factor,
                         TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv, int dim, int vdim, int page_size,
                         int num_pages, int max_positions, int rotary_dim, int interleaved, float eps, int values_are_keys,
                         int split_planes, const float* __restrict__ bias, int write_kv) {
  __shared__ float rows[PREP_WARPS][PREP_MAX_D];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qw = hq * dim, kw = hkv * dim;
  const T* row = proj + (size_t)t * ld;  // ld >= the row's width: the projection may be a run of columns of a wider product
  const int p = positions[t];
  const int page = write_kv ? table[(size_t)token_item[t] * table_width + p / page_size] : -1;
  const bool page_ok = page >= 0 && page < num_pages;  // tables are checked on the host; never write outside the pool
  const int rw = dim + vdim;
  const int half = rotary_dim / 2;
  const bool turn = cos_t != nullptr && p >= 0 && p < max_positions;
  const float* cs = turn ? cos_t + (size_t)p * half : nullptr;
  const float* sn = turn ? sin_t + (size_t)p * half : nullptr;
  float* mine = rows[warp];
  // ``bias`` (float32, one number per column of the row, optional) is added to the projection in float32;
  // ``write_kv`` 0: the row holds queries only (a layer that reads another layer's keys and values)
  for (int head = warp; head < hq + (write_kv ? hkv : 0); head += PREP_WARPS) {
    const bool is_q = head < hq;
    const T* src = row + (size_t)head * dim;  // query heads, then key heads, lie one after the other
    for (int d = lane; d < dim; d += 32) mine[d] = to_float<T>(src[d]) + (bias ? bias[(size_t)head * dim + d] : 0.f);
    __syncwarp();
    if (turn) {
      for (int i = lane; i < half; i += 32) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        float o1, o2;
        rotate_pair(mine[a], mine[b], cs[i], sn[i], o1, o2);
        mine[a] = o1;
        mine[b] = o2;
      }
      __syncwarp();
    }
    float factor = 1.f;
    if (eps >= 0.f) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(mine[d], mine[d], ss);
      factor = 1.f / sqrtf(warp_sum(ss) / (float)dim + eps);
    }
    if (is_q) {
      const float f = head_factor ? head_factor[head] : 1.f;
      T* dst = q_out + ((size_t)t * hq + head) * dim;
      for (int d = lane; d < dim; d += 32) dst[d] = from_float<T>(mine[d] * factor * f);
    } else if (page_ok) {
      const int g = head - hq;
      const size_t slot = (size_t)(p % page_size);
      TKV* dst = split_planes ? kv + ((((size_t)page * 2) * hkv + g) * page_size + slot) * dim
                              : kv + (((size_t)page * hkv + g) * page_size + slot) * rw;
      TKV* vdst = split_planes ? dst + (size_t)hkv * page_size * dim : dst + dim;
      for (int d = lane; d < dim; d += 32) dst[d] = from_float<TKV>(mine[d] * factor);
      const T* vsrc = values_are_keys ? src : row + qw + kw + (size_t)g * vdim;
      const float* vb = bias ? (values_are_keys ? bias + (size_t)head * dim : bias + qw + kw + (size_t)g * vdim) : nullptr;
      for (int d = lane; d < vdim; d += 32) vdst[d] = from_float<TKV>(to_float<T>(vsrc[d]) + (vb ? vb[d] : 0.f));
    }
    __syncwarp();
  }
}

// A run of N elements that is loaded and stored as one piece.
template <typename T, int N>
struct alignas(sizeof(T) * N) Run {
  T v[N];
};

// grid: T * groups blocks.  LPH lanes hold a head (32, or 16 for heads of 64 when both head counts are even: then a lane has
// four elements instead of two and a warp takes two heads at a time, which halves the instructions a byte costs); a warp
// takes HPW rounds of 32 / LPH heads: heads (warp index in the token * HPW + round) * (32 / LPH) + lane / LPH.  HPW > 1 (long
// steps): the rows of all of a warp's rounds are asked for together, before any of them is used, so that a lane has
// several loads in flight.  groups = ceil((hq + hkv) / (PREP_WARPS * HPW * 32 / LPH)).  A round lies within the heads or
// beyond them as a whole (the head counts are multiples of 32 / LPH), so the shuffles of a round see all of its lanes.
template <typename T, typename TKV, int DIM, int HPW, int LPH>
__global__ void __launch_bounds__(PREP_WARPS * 32)
attention_prepare_rows_kernel(const T* __restrict__ proj, long long ld, const int32_t* __restrict__ positions,
                              const int32_t* __restrict__ token_item, const int32_t* __restrict__ table, int table_width,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                              const float* __restrict__ head_factor, TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv,
                              int page_size, int num_pages, int max_positions, int rotary_dim, float eps, int values_are_keys,
                              int split_planes, int groups) {
  constexpr int N = DIM / LPH;    // elements a lane holds
  constexpr int HPR = 32 / LPH;   // heads a round
  pdl_trigger();
  const int t = blockIdx.x / groups;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPH, sl = lane % LPH;
  const int head0 = ((blockIdx.x - t * groups) * PREP_WARPS + (threadIdx.x >> 5)) * HPW * HPR;
  // positions and tables are inputs of the step: they may be read before the preceding kernel has finished
  const int p = positions[t];
  const int page = table[(size_t)token_item[t] * table_width + p / page_size];
  pdl_wait();
  const int heads = hq + hkv;
  if (head0 >= heads) return;
  const T* row = proj + (size_t)t * ld;
  Run<T, N> raw[HPW], vin[HPW];
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int head = head0 + i * HPR + sub;
    if (head < heads) raw[i] = *reinterpret_cast<const Run<T, N>*>(row + (size_t)head * DIM + sl * N);
    if (head < heads && head >= hq && !values_are_keys)
      vin[i] = *reinterpret_cast<const Run<T, N>*>(row + (size_t)heads * DIM + (size_t)(head - hq) * DIM + sl * N);
  }
  const bool turn = cos_t != nullptr && p >= 0 && p < max_positions;
  float cs[N / 2], sn[N / 2];
  if (turn) {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const int d = sl * N + i;  // even: the pair (d, d + 1) turns by angle d / 2
      cs[i / 2] = d < rotary_dim ? cos_t[(size_t)p * (rotary_dim / 2) + (d >> 1)] : 1.f;
      sn[i / 2] = d < rotary_dim ? sin_t[(size_t)p * (rotary_dim / 2) + (d >> 1)] : 0.f;
    }
  }
#pragma unroll
  for (int hh = 0; hh < HPW; ++hh) {
    const int head = head0 + hh * HPR + sub;
    if (head0 + hh * HPR >= heads) break;  // the whole round lies beyond the heads
    float x[N];
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = to_float<T>(raw[hh].v[i]);
    if (turn) {
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        if (sl * N + i < rotary_dim) {
          float o1, o2;
          rotate_pair(x[i], x[i + 1], cs[i / 2], sn[i / 2], o1, o2);
          x[i] = o1;
          x[i + 1] = o2;
        }
      }
    }
    float factor = 1.f;
    if (eps >= 0.f) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);  // over the head's lanes
      factor = 1.f / sqrtf(ss / (float)DIM + eps);
    }
    if (head >= heads) continue;  // cannot happen while the head counts are multiples of a round; never store for a head that is not there
    if (head < hq) {
      const float f = head_factor ? head_factor[head] : 1.f;
      Run<T, N> o;
#pragma unroll
      for (int i = 0; i < N; ++i) o.v[i] = from_float<T>(x[i] * factor * f);
      *reinterpret_cast<Run<T, N>*>(q_out + ((size_t)t * hq + head) * DIM + sl * N) = o;
      continue;
    }
    if (page < 0 || page >= num_pages) continue;  // tables are checked on the host; never write outside the pool
    const int g = head - hq;
    const size_t slot = (size_t)(p % page_size);
    TKV* dst = split_planes ? kv + ((((size_t)page * 2) * hkv + g) * page_size + slot) * DIM
                            : kv + (((size_t)page * hkv + g) * page_size + slot) * (2 * DIM);
    TKV* vdst = split_planes ? dst + (size_t)hkv * page_size * DIM : dst + DIM;
    Run<TKV, N> k;
#pragma unroll
    for (int i = 0; i < N; ++i) k.v[i] = from_float<TKV>(x[i] * factor);
    *reinterpret_cast<Run<TKV, N>*>(dst + sl * N) = k;
    const Run<T, N> vsrc = values_are_keys ? raw[hh] : vin[hh];
    Run<TKV, N> v;
#pragma unroll
    for (int i = 0; i < N; ++i) v.v[i] = from_float<TKV>(to_float<T>(vsrc.v[i]));
    *reinterpret_cast<Run<TKV, N>*>(vdst + sl * N) = v;
  }
}

}  // namespace

#define PSB_PREP_ROWS(DD, HH, LL)                                                                                      \
  psb_launch(attention_prepare_rows_kernel<T_, TKV, DD, HH, LL>, dim3((unsigned)blocks), dim3(PREP_WARPS * 32), 0, stream,     \
             (const T_*)proj, ld, (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)table,        \
             table_width, (const float*)cos_t, (const float*)sin_t, (const float*)head_factor, (TKV*)kv, (T_*)q_out,   \
             hq, hkv, page_size, num_pages, max_positions, rotary_dim, eps, values_are_keys, split_planes, groups)

// (proj, ld, dtype, positions, token_item, table, table_width, cos, sin, head_factor, kv, kv_dtype, q_out, T, hq, hkv, dim, vdim,
//  page_size, num_pages, max_positions, rotary_dim, interleaved, eps, values_are_keys, split_planes, bias, write_kv, stream)
PSB_API int psb_attention_prepare(const void* proj, long long ld, int dtype, const void* positions, const void* token_item, const void* table,
                                  int table_width, const void* cos_t, const void* sin_t, const void* head_factor, void* kv,
                                  int kv_dtype, void* q_out, int T, int hq, int hkv, int dim, int vdim, int page_size,
                                  int num_pages, int max_positions, int rotary_dim, int interleaved, float eps,
                                  int values_are_keys, int split_planes, const void* bias, int write_kv, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 1 || dim < 1 || dim > PREP_MAX_D || vdim < 1 || page_size < 1 || (write_kv && (table_width < 1 || num_pages < 1)))
    PSB_REFUSE("attention_prepare: bad sizes (heads %d/%d, sizes %d/%d, at most %d)", hq, hkv, dim, vdim, PREP_MAX_D);
  if (write_kv && (!kv || !table)) PSB_REFUSE("attention_prepare: appending keys and values needs the cache entry and the page table");
  if (ld < (long long)hq * dim + (write_kv ? (long long)hkv * dim + (values_are_keys ? 0 : (long long)hkv * vdim) : 0))
    PSB_REFUSE("attention_prepare: row stride %lld is shorter than the row", ld);
  if (values_are_keys && vdim != dim) PSB_REFUSE("attention_prepare: keys that serve as values need vdim == dim, not %d and %d", vdim, dim);
  if ((cos_t == nullptr) != (sin_t == nullptr)) PSB_REFUSE("attention_prepare: cosines and sines come together");
  if (cos_t && (rotary_dim < 2 || rotary_dim % 2 || rotary_dim > dim || max_positions < 1))
    PSB_REFUSE("attention_prepare: %d rotated elements of %d", rotary_dim, dim);
  if (split_planes && vdim != dim) PSB_REFUSE("attention_prepare: keys and values in planes of their own need vdim == dim, not %d and %d", vdim, dim);
  if (T == 0) return 0;
  // heads in registers: sizes that give every lane an even run, a rotation (if any) of neighbours, rows that allow wide loads
  const bool rows_fit = vdim == dim && (dim == 64 || dim == 128 || dim == 256) && (cos_t == nullptr || interleaved) && !bias && write_kv;
  if (rows_fit) {
    // long steps: four heads a warp, their loads in flight together; short ones: a head a warp, as many warps as there are heads
    const int hpw = (long long)T * (hq + hkv) >= 4096 ? 4 : 1;
    // heads of 64 in pairs (16 lanes a head, four elements a lane) when neither the query nor the key heads leave one over
    const int lph = dim == 64 && hq % 2 == 0 && hkv % 2 == 0 ? 16 : 32;
    const int per_block = PREP_WARPS * hpw * (32 / lph);
    const int groups = (hq + hkv + per_block - 1) / per_block;
    const long long blocks = (long long)T * groups;
    bool done = false;
    PSB_DISPATCH_DTYPE(dtype, T_, {
      PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
        const size_t in_run = sizeof(T_) * (size_t)(dim / lph), out_run = sizeof(TKV) * (size_t)(dim / lph);
        if (blocks <= 0x7fffffffLL && (uintptr_t)proj % in_run == 0 && ((size_t)ld * sizeof(T_)) % in_run == 0 &&
            (uintptr_t)q_out % in_run == 0 && (uintptr_t)kv % out_run == 0) {
          if (hpw == 4) {
            if (dim == 64 && lph == 16) PSB_PREP_ROWS(64, 4, 16); else if (dim == 64) PSB_PREP_ROWS(64, 4, 32);
            else if (dim == 128) PSB_PREP_ROWS(128, 4, 32); else PSB_PREP_ROWS(256, 4, 32);
          } else {
            if (dim == 64 && lph == 16) PSB_PREP_ROWS(64, 1, 16); else if (dim == 64) PSB_PREP_ROWS(64, 1, 32);
            else if (dim == 128) PSB_PREP_ROWS(128, 1, 32); else PSB_PREP_ROWS(256, 1, 32);
          }
          done = true;
        }
      });
    });
    if (done) {
      PSB_LAUNCH_CHECK("attention_prepare");
      return 0;
    }
  }
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_prepare_kernel<T_, TKV>, dim3(T), dim3(PREP_WARPS * 32), 0, stream, (const T_*)proj, ld,
                 (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)table, table_width, (const float*)cos_t,
                 (const float*)sin_t, (const float*)head_factor, (TKV*)kv, (T_*)q_out, hq, hkv, dim, vdim, page_size, num_pages,
                 max_positions, rotary_dim, interleaved, eps, values_are_keys, split_planes, (const float*)bias, write_kv);
    });
  });
  PSB_LAUNCH_CHECK("attention_prepare");
  return 0;
}
