// Activations of a feed-forward without a gate branch, out = act(x) element by element, float32 arithmetic:
//   silu, gelu_tanh (as in the gated kernels), and xielu with two learned numbers (p, q):
//     z > 0:  softplus(p) z^2 + z/2
//     z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
#include "common.cuh"

namespace {

enum : int { UNARY_SILU = 0, UNARY_GELU_TANH = 1, UNARY_XIELU = 2 };

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
    else v = gate_act(z, code);
    out[i] = from_float<T>(v);
  }
}

}  // namespace

PSB_API int psb_unary_act(const void* x, int dtype, void* out, long long total, int code, const void* params,
                          cudaStream_t stream) {
  if (total < 0) PSB_REFUSE("unary_act: negative size");
  if (code < 0 || code > UNARY_XIELU) PSB_REFUSE("unary_act: activation code %d is not built", code);
  if (code == UNARY_XIELU && !params) PSB_REFUSE("unary_act: xielu needs its two numbers");
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  PSB_DISPATCH_DTYPE(dtype, T, {
    psb_launch(unary_act_kernel<T>, dim3((unsigned)(blocks > 65535 * 16 ? 65535 * 16 : blocks)), dim3(256), 0, stream,
               (const T*)x, (T*)out, (size_t)total, code, (const float*)params);
  });
  PSB_LAUNCH_CHECK("unary_act");
  return 0;
}
