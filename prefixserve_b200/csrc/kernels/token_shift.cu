// Token shift: what a sublayer reads is moved toward what it read one token earlier, channel by channel,
//
//   y_t = x_t + (x_(t-1) - x_t) * mix        x_(-1) = 0
//
// with x_(t-1) the unshifted row of the token before.  For the first token of a portion that row is not in the step:
// it is carried per request in the slot's state (float32, ``state`` + slot * stride), which the same launch brings up
// to date with the portion's last row.  One block per token; the block of a portion's first token reads the carried
// row and then, thread by thread for the same channels, writes the new one, so nobody reads what has been replaced.
// The interpolation is float32; rows are float32 or bfloat16.  Rows whose width is a multiple of 8 (and 16-byte
// aligned) move in runs of eight channels a thread, one 16-byte load or store per run of bfloat16.
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void run8_load(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void run8_load<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void run8_load<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h2[k]);
    o[2 * k] = f.x; o[2 * k + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void run8_store(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void run8_store<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void run8_store<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// The same as token_shift_kernel below, eight channels a thread and turn.
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_vec_kernel(const T* __restrict__ x, const float* __restrict__ mix, float* __restrict__ state, long long stride,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                       const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots, T* __restrict__ y, int W,
                       int num_slots) {
  pdl_trigger();
  // what the step itself brings (offsets, slots, positions) may be read before the preceding kernel has finished
  const int t = blockIdx.x;
  const int item = token_item[t];
  const int first = item_start[item], last = item_start[item + 1] - 1;
  const int slot = slots[item];
  const bool starts = positions[t] == 0;
  pdl_wait();
  const T* row = x + (size_t)t * W;
  T* out = y + (size_t)t * W;
  if (t != first) {
    const T* before = row - W;
    for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
      float a[8], b[8], m[8];
      run8_load<T>(row + c, a);
      run8_load<T>(before + c, b);
      run8_load<float>(mix + c, m);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] = fmaf(b[k] - a[k], m[k], a[k]);
      run8_store<T>(out + c, a);
    }
    return;
  }
  if (slot < 0 || slot >= num_slots) return;  // slots are checked on the host; never touch memory outside the states
  float* held = state + (size_t)slot * stride;
  const T* newest = x + (size_t)last * W;
  for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
    float a[8], b[8], m[8], n[8];
    run8_load<T>(row + c, a);
    run8_load<T>(newest + c, n);
    run8_load<float>(mix + c, m);
    if (starts) {
#pragma unroll
      for (int k = 0; k < 8; ++k) b[k] = 0.f;
    } else {
      run8_load<float>(held + c, b);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = fmaf(b[k] - a[k], m[k], a[k]);
    run8_store<T>(out + c, a);
    run8_store<float>(held + c, n);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mix, float* __restrict__ state, long long stride,
                   const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                   const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots, T* __restrict__ y, int W,
                   int num_slots) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int item = token_item[t];
  const int first = item_start[item], last = item_start[item + 1] - 1;
  const T* row = x + (size_t)t * W;
  T* out = y + (size_t)t * W;
  if (t != first) {
    const T* before = row - W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      const float a = to_float<T>(row[c]), b = to_float<T>(before[c]);
      out[c] = from_float<T>(fmaf(b - a, mix[c], a));
    }
    return;
  }
  const int slot = slots[item];
  if (slot < 0 || slot >= num_slots) return;  // slots are checked on the host; never touch memory outside the states
  float* held = state + (size_t)slot * stride;
  const bool starts = positions[t] == 0;
  const T* newest = x + (size_t)last * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float a = to_float<T>(row[c]);
    const float b = starts ? 0.f : held[c];
    out[c] = from_float<T>(fmaf(b - a, mix[c], a));
    held[c] = to_float<T>(newest[c]);
  }
}

// Steps of single tokens: the residual sum, the RMS norm in front of the shifted sublayer and the shift in one kernel,
//
//   h_t += delta_t        n_t = round(gain * h_t / rms(h_t))        y_t = n_t + (held - n_t) * mix        held <- n_t
//
// with ``held`` the request's carried row (zero for a sequence's first token) and ``round`` the rounding to the rows'
// type that the norm's own kernel would do, so that a token gets the same y whichever way it went.  A block per token;
// every token of the step is its request's only one, so no block needs another's row.  W % 8 == 0.
template <typename TD, typename TX>
__global__ void __launch_bounds__(256)
add_rmsnorm_shift_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ gain, float eps,
                         const float* __restrict__ mix, float* __restrict__ state, long long stride,
                         const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                         const int32_t* __restrict__ slots, TX* __restrict__ y, int W, int num_slots) {
  __shared__ float sums[8];
  pdl_trigger();
  const int t = blockIdx.x;
  const int slot = slots[token_item[t]];
  const bool starts = positions[t] == 0;
  pdl_wait();
  float* hr = h + (size_t)t * W;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
    float v[8];
    run8_load<float>(hr + c, v);
    if (delta) {
      float d[8];
      run8_load<TD>(delta + (size_t)t * W + c, d);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += d[k];
      run8_store<float>(hr + c, v);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) ss += sums[w];
  const float inv = rsqrtf(ss / (float)W + eps);
  if (slot < 0 || slot >= num_slots) return;  // slots are checked on the host; never touch memory outside the states
  float* held = state + (size_t)slot * stride;
  for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {  // a thread meets the channels it wrote above
    float v[8], g[8], m[8], b[8];
    run8_load<float>(hr + c, v);
    run8_load<float>(gain + c, g);
    run8_load<float>(mix + c, m);
    if (starts) {
#pragma unroll
      for (int k = 0; k < 8; ++k) b[k] = 0.f;
    } else {
      run8_load<float>(held + c, b);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      v[k] = to_float<TX>(from_float<TX>(g[k] * (v[k] * inv)));
      b[k] = fmaf(b[k] - v[k], m[k], v[k]);
    }
    run8_store<TX>(y + (size_t)t * W + c, b);
    run8_store<float>(held + c, v);
  }
}

// out = (gain_a * a / rms(a) + gain_b * b / rms(b)) * weight: two branches that read the same input, each normed over
// the row before they are added.  One block per row, statistics float32, float32 result.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
normed_pair_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ gain_a,
                       const float* __restrict__ gain_b, float* __restrict__ out, int W, float eps, float weight) {
  __shared__ float sums[2][8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const T* ra = a + (size_t)t * W;
  const T* rb = b + (size_t)t * W;
  float sa = 0.f, sb = 0.f;
  if (VEC) {
    // runs of eight channels a thread; the second pass finds the rows in the cache
    for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
      float va[8], vb[8];
      run8_load<T>(ra + c, va);
      run8_load<T>(rb + c, vb);
#pragma unroll
      for (int k = 0; k < 8; ++k) { sa = fmaf(va[k], va[k], sa); sb = fmaf(vb[k], vb[k], sb); }
    }
  } else
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float va = to_float<T>(ra[c]), vb = to_float<T>(rb[c]);
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  sa = warp_sum(sa);
  sb = warp_sum(sb);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sums[0][warp] = sa; sums[1][warp] = sb; }
  __syncthreads();
  sa = sb = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { sa += sums[0][w]; sb += sums[1][w]; }
  const float ia = 1.f / sqrtf(sa / (float)W + eps), ib = 1.f / sqrtf(sb / (float)W + eps);
  if (VEC) {
    for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
      float va[8], vb[8], ga[8], gb[8];
      run8_load<T>(ra + c, va);
      run8_load<T>(rb + c, vb);
      run8_load<float>(gain_a + c, ga);
      run8_load<float>(gain_b + c, gb);
#pragma unroll
      for (int k = 0; k < 8; ++k) va[k] = (ga[k] * (va[k] * ia) + gb[k] * (vb[k] * ib)) * weight;
      run8_store<float>(out + (size_t)t * W + c, va);
    }
    return;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    out[(size_t)t * W + c] = (gain_a[c] * (to_float<T>(ra[c]) * ia) + gain_b[c] * (to_float<T>(rb[c]) * ib)) * weight;
}

}  // namespace

// (x, dtype, mix, state, stride, positions, token_item, item_start, slots, y, T, W, num_slots, stream)
PSB_API int psb_token_shift(const void* x, int dtype, const void* mix, void* state, long long stride, const void* positions,
                            const void* token_item, const void* item_start, const void* slots, void* y, int T, int W,
                            int num_slots, cudaStream_t stream) {
  if (T < 0 || W < 1 || num_slots < 1 || stride < W) PSB_REFUSE("token_shift: bad sizes T=%d W=%d stride=%lld", T, W, stride);
  if (T == 0) return 0;
  const bool vec = W % 8 == 0 && stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)mix | (uintptr_t)state) & 15) == 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (vec)
      psb_launch(token_shift_vec_kernel<T_>, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream, (const T_*)x, (const float*)mix,
                 (float*)state, stride, (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start,
                 (const int32_t*)slots, (T_*)y, W, num_slots);
    else
    psb_launch(token_shift_kernel<T_>, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, stream, (const T_*)x, (const float*)mix,
               (float*)state, stride, (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start,
               (const int32_t*)slots, (T_*)y, W, num_slots);
  });
  PSB_LAUNCH_CHECK("token_shift");
  return 0;
}

// (h, delta, delta_dtype, gain, eps, mix, state, stride, positions, token_item, slots, y, y_dtype, T, W, num_slots, stream)
// Every token of the step must be its request's only one (the caller knows: the step's longest portion is one token).
PSB_API int psb_add_rmsnorm_shift(void* h, const void* delta, int delta_dtype, const void* gain, float eps, const void* mix,
                                  void* state, long long stride, const void* positions, const void* token_item,
                                  const void* slots, void* y, int y_dtype, int T, int W, int num_slots, cudaStream_t stream) {
  if (T < 0 || W < 8 || W % 8 || num_slots < 1 || stride < W || stride % 4) PSB_REFUSE("add_rmsnorm_shift: bad sizes T=%d W=%d stride=%lld", T, W, stride);
  if (!(eps > 0.f)) PSB_REFUSE("add_rmsnorm_shift: eps must be positive");
  if (((uintptr_t)h | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)mix | (uintptr_t)state | (uintptr_t)y) & 15)
    PSB_REFUSE("add_rmsnorm_shift: operands must be 16-byte aligned");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(delta_dtype, TD, {
    PSB_DISPATCH_DTYPE(y_dtype, TX, {
      psb_launch(add_rmsnorm_shift_kernel<TD, TX>, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream, (float*)h, (const TD*)delta,
                 (const float*)gain, eps, (const float*)mix, (float*)state, stride, (const int32_t*)positions,
                 (const int32_t*)token_item, (const int32_t*)slots, (TX*)y, W, num_slots);
    });
  });
  PSB_LAUNCH_CHECK("add_rmsnorm_shift");
  return 0;
}

// (a, b, dtype, gain_a, gain_b, out_f32, T, W, eps, weight, stream)
PSB_API int psb_normed_pair_sum(const void* a, const void* b, int dtype, const void* gain_a, const void* gain_b, void* out,
                                int T, int W, float eps, float weight, cudaStream_t stream) {
  if (T < 0 || W < 1) PSB_REFUSE("normed_pair_sum: bad sizes T=%d W=%d", T, W);
  if (T == 0) return 0;
  const bool vec = W % 8 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)gain_a | (uintptr_t)gain_b | (uintptr_t)out) & 15) == 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (vec)
      psb_launch(normed_pair_sum_kernel<T_, true>, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream, (const T_*)a, (const T_*)b,
                 (const float*)gain_a, (const float*)gain_b, (float*)out, W, eps, weight);
    else
      psb_launch(normed_pair_sum_kernel<T_, false>, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, stream, (const T_*)a, (const T_*)b,
                 (const float*)gain_a, (const float*)gain_b, (float*)out, W, eps, weight);
  });
  PSB_LAUNCH_CHECK("normed_pair_sum");
  return 0;
}
