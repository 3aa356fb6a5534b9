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
//     ``values_are_keys``, the key as it was projected (before rotation and norm).
//
// One block per token, a warp per head in turn; the head lies in the warp's shared-memory row between the steps.
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
                         int num_pages, int max_positions, int rotary_dim, int interleaved, float eps, int values_are_keys) {
  __shared__ float rows[PREP_WARPS][PREP_MAX_D];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qw = hq * dim, kw = hkv * dim;
  const T* row = proj + (size_t)t * ld;  // ld >= the row's width: the projection may be a run of columns of a wider product
  const int p = positions[t];
  const int page = table[(size_t)token_item[t] * table_width + p / page_size];
  const bool page_ok = page >= 0 && page < num_pages;  // tables are checked on the host; never write outside the pool
  const int rw = dim + vdim;
  const int half = rotary_dim / 2;
  const bool turn = cos_t != nullptr && p >= 0 && p < max_positions;
  const float* cs = turn ? cos_t + (size_t)p * half : nullptr;
  const float* sn = turn ? sin_t + (size_t)p * half : nullptr;
  float* mine = rows[warp];
  for (int head = warp; head < hq + hkv; head += PREP_WARPS) {
    const bool is_q = head < hq;
    const T* src = row + (size_t)head * dim;  // query heads, then key heads, lie one after the other
    for (int d = lane; d < dim; d += 32) mine[d] = to_float<T>(src[d]);
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
      TKV* dst = kv + (((size_t)page * hkv + g) * page_size + (size_t)(p % page_size)) * rw;
      for (int d = lane; d < dim; d += 32) dst[d] = from_float<TKV>(mine[d] * factor);
      const T* vsrc = values_are_keys ? src : row + qw + kw + (size_t)g * vdim;
      for (int d = lane; d < vdim; d += 32) dst[dim + d] = from_float<TKV>(to_float<T>(vsrc[d]));
    }
    __syncwarp();
  }
}

}  // namespace

// (proj, ld, dtype, positions, token_item, table, table_width, cos, sin, head_factor, kv, kv_dtype, q_out, T, hq, hkv, dim, vdim,
//  page_size, num_pages, max_positions, rotary_dim, interleaved, eps, values_are_keys, stream)
PSB_API int psb_attention_prepare(const void* proj, long long ld, int dtype, const void* positions, const void* token_item, const void* table,
                                  int table_width, const void* cos_t, const void* sin_t, const void* head_factor, void* kv,
                                  int kv_dtype, void* q_out, int T, int hq, int hkv, int dim, int vdim, int page_size,
                                  int num_pages, int max_positions, int rotary_dim, int interleaved, float eps,
                                  int values_are_keys, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 1 || dim < 1 || dim > PREP_MAX_D || vdim < 1 || page_size < 1 || table_width < 1 || num_pages < 1)
    PSB_REFUSE("attention_prepare: bad sizes (heads %d/%d, sizes %d/%d, at most %d)", hq, hkv, dim, vdim, PREP_MAX_D);
  if (ld < (long long)(hq + hkv) * dim + (values_are_keys ? 0 : (long long)hkv * vdim)) PSB_REFUSE("attention_prepare: row stride %lld is shorter than the row", ld);
  if (values_are_keys && vdim != dim) PSB_REFUSE("attention_prepare: keys that serve as values need vdim == dim, not %d and %d", vdim, dim);
  if ((cos_t == nullptr) != (sin_t == nullptr)) PSB_REFUSE("attention_prepare: cosines and sines come together");
  if (cos_t && (rotary_dim < 2 || rotary_dim % 2 || rotary_dim > dim || max_positions < 1))
    PSB_REFUSE("attention_prepare: %d rotated elements of %d", rotary_dim, dim);
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_prepare_kernel<T_, TKV>, dim3(T), dim3(PREP_WARPS * 32), 0, stream, (const T_*)proj, ld,
                 (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)table, table_width, (const float*)cos_t,
                 (const float*)sin_t, (const float*)head_factor, (TKV*)kv, (T_*)q_out, hq, hkv, dim, vdim, page_size, num_pages,
                 max_positions, rotary_dim, interleaved, eps, values_are_keys);
    });
  });
  PSB_LAUNCH_CHECK("attention_prepare");
  return 0;
}
