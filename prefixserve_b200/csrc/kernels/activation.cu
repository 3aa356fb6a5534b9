// Activations of a feed-forward without a gate branch, out = act(x) element by element, float32 arithmetic:
//   silu, gelu_tanh (as in the gated kernels), and xielu with two learned numbers (p, q):
//     z > 0:  softplus(p) z^2 + z/2
//     z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
//   and relu2: max(z, 0)^2.
#include "common.cuh"

namespace {

enum : int { UNARY_SILU = 0, UNARY_GELU_TANH = 1, UNARY_XIELU = 2, UNARY_RELU2 = 3 };

__device__ __forceinline__ float relu2f_(float z) { z = fmaxf(z, 0.f); return z * z; }

__device__ __forceinline__ float softplusf_(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f); }

template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total, int code,
                                 const float* __restrict__ params) {
  pdl_trigger();
  pdl_wait();
  float ap = 0.f, aq = 0.f;
  if (code == UNARY_XIELU) {
    ap = softplusf_(params[0]);
    aq = 0.5f + softplusf_(params[1]);
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float z = to_float<T>(x[i]);
    float v;
    if (code == UNARY_XIELU) v = z > 0.f ? ap * z * z + 0.5f * z : aq * (expm1f(z) - z) + 0.5f * z;
    else if (code == UNARY_RELU2) v = relu2f_(z);
    else v = gate_act(z, code);
    out[i] = from_float<T>(v);
  }
}

// Eight bfloat16 elements a thread (16-byte loads and stores).
__global__ void unary_act_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, size_t vecs, int code,
                                     const float* __restrict__ params) {
  pdl_trigger();
  pdl_wait();
  float ap = 0.f, aq = 0.f;
  if (code == UNARY_XIELU) {
    ap = softplusf_(params[0]);
    aq = 0.5f + softplusf_(params[1]);
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat162* in2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 z = __bfloat1622float2(in2[k]);
      float a, b;
      if (code == UNARY_XIELU) {
        a = z.x > 0.f ? ap * z.x * z.x + 0.5f * z.x : aq * (expm1f(z.x) - z.x) + 0.5f * z.x;
        b = z.y > 0.f ? ap * z.y * z.y + 0.5f * z.y : aq * (expm1f(z.y) - z.y) + 0.5f * z.y;
      } else if (code == UNARY_RELU2) {
        a = relu2f_(z.x);
        b = relu2f_(z.y);
      } else {
        a = gate_act(z.x, code);
        b = gate_act(z.y, code);
      }
      o2[k] = __floats2bfloat162_rn(a, b);
    }
    reinterpret_cast<uint4*>(out)[i] = o4;
  }
}

// out = x * gate, element by element: gate float32 (a sigmoid that somebody has already taken), the product in float32
template <typename TX, typename TO>
__global__ void gate_mul_kernel(const TX* __restrict__ x, const float* __restrict__ gate, TO* __restrict__ out, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<TO>(to_float<TX>(x[i]) * gate[i]);
}

}  // namespace

// (x, x_dtype, gate float32, out, out_dtype, total, stream)
PSB_API int psb_gate_mul(const void* x, int x_dtype, const void* gate, void* out, int out_dtype, long long total, cudaStream_t stream) {
  if (total < 0) PSB_REFUSE("gate_mul: negative size");
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  PSB_DISPATCH_DTYPE(x_dtype, TX, {
    PSB_DISPATCH_DTYPE(out_dtype, TO, {
      psb_launch(gate_mul_kernel<TX, TO>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, stream,
                 (const TX*)x, (const float*)gate, (TO*)out, (size_t)total);
    });
  });
  PSB_LAUNCH_CHECK("gate_mul");
  return 0;
}

PSB_API int psb_unary_act(const void* x, int dtype, void* out, long long total, int code, const void* params,
                          cudaStream_t stream) {
  if (total < 0) PSB_REFUSE("unary_act: negative size");
  if (code < 0 || code > UNARY_RELU2) PSB_REFUSE("unary_act: activation code %d is not built", code);
  if (code == UNARY_XIELU && !params) PSB_REFUSE("unary_act: xielu needs its two numbers");
  if (total == 0) return 0;
  if (dtype == PSB_BF16 && total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const long long vecs = total / 8, vblocks = (vecs + 255) / 256;
    psb_launch(unary_act_vec_kernel, dim3((unsigned)(vblocks > 148 * 16 ? 148 * 16 : vblocks)), dim3(256), 0, stream,
               (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (size_t)vecs, code, (const float*)params);
    PSB_LAUNCH_CHECK("unary_act");
    return 0;
  }
  const long long blocks = (total + 255) / 256;
  PSB_DISPATCH_DTYPE(dtype, T, {
    psb_launch(unary_act_kernel<T>, dim3((unsigned)(blocks > 65535 * 16 ? 65535 * 16 : blocks)), dim3(256), 0, stream,
               (const T*)x, (T*)out, (size_t)total, code, (const float*)params);
  });
  PSB_LAUNCH_CHECK("unary_act");
  return 0;
}
