// A gated recurrence whose gates read only the current token (minGRU), per channel and in float32:
//
//   z_t = sigmoid(pz_t + bz)          u_t = px_t + bx          c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t                          out_t = S_t * silu(pg_t)
//
// pz, px, pg are three runs of W columns of one projection row (row stride ``ld``, so the row may hold more than
// these); S is carried per request in the slot's state (float32, ``state`` + slot * stride) from S = 0.
//
// Since S -> (1 - z) S + z c is a map S -> A S + B and such maps compose, a long portion is cut into chunks that run
// side by side: a first pass reduces every chunk to its (A, B) and notes the state the portion starts from, the
// second folds the maps of the chunks in front of its own and runs the chunk.  Short portions and single tokens take
// the second pass alone, one chunk a portion.  A thread is a channel; the loads of eight tokens are in flight together
// (none depends on S).
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_(float v) { return 1.f / (1.f + expf(-v)); }

// Which portion and which of its chunks a block works on (chunks are numbered through the step's portions in order);
// false beyond the last chunk: the grid is sized by an upper bound.
__device__ __forceinline__ bool gru_find_chunk(const int32_t* __restrict__ item_start, int items, int chunk, int g, int& item,
                                               int& index, int& count) {
  for (int i = 0; i < items; ++i) {
    const int c = (item_start[i + 1] - item_start[i] + chunk - 1) / chunk;
    if (g < c) { item = i; index = g; count = c; return true; }
    g -= c;
  }
  return false;
}

__device__ __forceinline__ void gru_terms(float pz, float px, float bz, float bx, float& keep, float& add) {
  const float z = sigmoid_(pz + bz);
  const float u = px + bx;
  const float c = u >= 0.f ? u + 0.5f : sigmoid_(u);
  keep = 1.f - z;
  add = z * c;
}

constexpr int GRU_UNROLL = 8;

// First pass: carry[chunk] = (A, B) of the chunk from the identity; start[item] = the slot's state as the step found it.
template <typename T>
__global__ void min_gru_chunk_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ bias_z,
                                     const float* __restrict__ bias_x, const float* __restrict__ state, long long stride,
                                     const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots,
                                     float2* __restrict__ carry, float* __restrict__ start, int items, int W, int num_slots,
                                     int chunk) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  int item, index, count;
  if (c >= W || !gru_find_chunk(item_start, items, chunk, blockIdx.y, item, index, count)) return;
  if (index == 0) {
    const int slot = slots[item];
    start[(size_t)item * W + c] = slot >= 0 && slot < num_slots ? state[(size_t)slot * stride + c] : 0.f;
  }
  if (count == 1) return;
  const int t0 = item_start[item] + index * chunk, t1 = min(t0 + chunk, item_start[item + 1]);
  const float bz = bias_z[c], bx = bias_x[c];
  float A = 1.f, B = 0.f;
  for (int t = t0; t < t1; t += GRU_UNROLL) {
    float pz[GRU_UNROLL], px[GRU_UNROLL];
#pragma unroll
    for (int k = 0; k < GRU_UNROLL; ++k) {
      const int tt = t + k < t1 ? t + k : t1 - 1;
      pz[k] = to_float<T>(proj[(size_t)tt * ld + c]);
      px[k] = to_float<T>(proj[(size_t)tt * ld + W + c]);
    }
#pragma unroll
    for (int k = 0; k < GRU_UNROLL; ++k) {
      if (t + k >= t1) break;
      float keep, add;
      gru_terms(pz[k], px[k], bz, bx, keep, add);
      B = fmaf(keep, B, add);
      A *= keep;
    }
  }
  carry[(size_t)blockIdx.y * W + c] = make_float2(A, B);
}

// Second pass (the only one when every portion is one chunk: ``start`` null, the state read from the slot).
template <typename T>
__global__ void min_gru_scan_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ bias_z,
                                    const float* __restrict__ bias_x, float* __restrict__ state, long long stride,
                                    const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots,
                                    const float2* __restrict__ carry, const float* __restrict__ start, T* __restrict__ out,
                                    int items, int W, int num_slots, int chunk) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  int item, index, count;
  if (c >= W || !gru_find_chunk(item_start, items, chunk, blockIdx.y, item, index, count)) return;
  const int slot = slots[item];
  if (slot < 0 || slot >= num_slots) return;  // slots are checked on the host; never touch memory outside the states
  float* mine = state + (size_t)slot * stride + c;
  float S = start ? start[(size_t)item * W + c] : *mine;
  for (int k = 0; k < index; ++k) {  // through the chunks in front of this one
    const float2 ab = carry[(size_t)(blockIdx.y - index + k) * W + c];
    S = fmaf(ab.x, S, ab.y);
  }
  const int t0 = item_start[item] + index * chunk, t1 = min(t0 + chunk, item_start[item + 1]);
  const float bz = bias_z[c], bx = bias_x[c];
  for (int t = t0; t < t1; t += GRU_UNROLL) {
    float pz[GRU_UNROLL], px[GRU_UNROLL], pg[GRU_UNROLL];
#pragma unroll
    for (int k = 0; k < GRU_UNROLL; ++k) {
      const int tt = t + k < t1 ? t + k : t1 - 1;
      pz[k] = to_float<T>(proj[(size_t)tt * ld + c]);
      px[k] = to_float<T>(proj[(size_t)tt * ld + W + c]);
      pg[k] = to_float<T>(proj[(size_t)tt * ld + 2 * W + c]);
    }
#pragma unroll
    for (int k = 0; k < GRU_UNROLL; ++k) {
      if (t + k >= t1) break;
      float keep, add;
      gru_terms(pz[k], px[k], bz, bx, keep, add);
      S = fmaf(keep, S, add);
      out[(size_t)(t + k) * W + c] = from_float<T>(S * (pg[k] * sigmoid_(pg[k])));
    }
  }
  if (index == count - 1) *mine = S;  // the portion's last chunk leaves the state behind
}

}  // namespace

// (proj, ld, dtype, bias_z, bias_x, state, stride, item_start, slots, carry, start, out, items, T, W, num_slots, chunk, stream)
// ``chunk`` >= the longest portion: one pass (carry and start unused); else both passes, carry float2 [T / chunk + items, W]
// and start float32 [items, W].
PSB_API int psb_min_gru(const void* proj, long long ld, int dtype, const void* bias_z, const void* bias_x, void* state,
                        long long stride, const void* item_start, const void* slots, void* carry, void* start, void* out,
                        int items, int T, int W, int num_slots, int chunk, int two_pass, cudaStream_t stream) {
  if (items < 0 || T < 0 || W < 1 || num_slots < 1 || chunk < 1 || ld < 3LL * W || stride < W)
    PSB_REFUSE("min_gru: bad sizes items=%d T=%d W=%d ld=%lld stride=%lld chunk=%d", items, T, W, ld, stride, chunk);
  if (items == 0 || T == 0) return 0;
  const int chunks = T / chunk + items;  // at least the number of chunks of any cutting of T tokens into ``items`` portions
  if (chunks > 65535) PSB_REFUSE("min_gru: %d chunks in one step are too many for this kernel", chunks);
  if (two_pass && (!carry || !start)) PSB_REFUSE("min_gru: portions cut into chunks need the carry and start buffers");
  const int threads = 64;
  const dim3 grid((W + threads - 1) / threads, chunks);
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (two_pass) {
      psb_launch(min_gru_chunk_kernel<T_>, grid, dim3(threads), 0, stream, (const T_*)proj, ld, (const float*)bias_z,
                 (const float*)bias_x, (const float*)state, stride, (const int32_t*)item_start, (const int32_t*)slots,
                 (float2*)carry, (float*)start, items, W, num_slots, chunk);
    }
    psb_launch(min_gru_scan_kernel<T_>, grid, dim3(threads), 0, stream, (const T_*)proj, ld, (const float*)bias_z,
               (const float*)bias_x, (float*)state, stride, (const int32_t*)item_start, (const int32_t*)slots,
               (const float2*)carry, two_pass ? (const float*)start : (const float*)nullptr, (T_*)out, items, W, num_slots, chunk);
  });
  PSB_LAUNCH_CHECK("min_gru");
  return 0;
}
