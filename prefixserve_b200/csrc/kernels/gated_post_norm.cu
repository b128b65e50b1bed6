// A sublayer's result joins the residual stream after a gate and a norm of its own:
//   z = y * sigmoid(g + b)            (g: the gate's product with the sublayer's input, b its bias; may be absent)
//   h += mult * gain * z / sqrt(mean(z^2) + eps)
// with h the float32 stream and every step of the arithmetic in float32; only y and g are read in their storage
// type.  The new stream may also be written in the compute type (``copy``) for the products of the next sublayer,
// which reads the stream itself and not a normed form of it.  One block per row; the sum of squares is added up in
// a fixed order, so a row's result does not depend on the batch.
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

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <typename TY, typename TG, typename TX>
__global__ void gated_norm_add_kernel(float* __restrict__ h, const TY* __restrict__ y, const TG* __restrict__ g,
                                      const float* __restrict__ bias, const float* __restrict__ gain,
                                      TX* __restrict__ copy, int H, float eps, float mult) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const size_t r = blockIdx.x;
  const TY* yr = y + r * H;
  const TG* gr = g ? g + r * H : nullptr;
  float* hr = h + r * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float z = to_float<TY>(yr[j]);
    if (gr) z *= sigmoidf_(to_float<TG>(gr[j]) + (bias ? bias[j] : 0.f));
    ss += z * z;
  }
  const float inv = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps);
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float z = to_float<TY>(yr[j]);
    if (gr) z *= sigmoidf_(to_float<TG>(gr[j]) + (bias ? bias[j] : 0.f));
    const float v = hr[j] + mult * (gain[j] * (z * inv));
    hr[j] = v;
    if (copy) copy[r * H + j] = from_float<TX>(v);
  }
}

}  // namespace

PSB_API int psb_gated_norm_add(void* h, const void* y, int y_dtype, const void* g, int g_dtype, const void* bias,
                               const void* gain, void* copy, int copy_dtype, int rows, int H, float eps, float mult,
                               cudaStream_t stream) {
  if (rows < 0 || H < 1) PSB_REFUSE("gated_norm_add: bad sizes rows=%d H=%d", rows, H);
  if (!(eps > 0.f)) PSB_REFUSE("gated_norm_add: eps must be positive");
  if (rows == 0) return 0;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  PSB_DISPATCH_DTYPE(y_dtype, TY, {
    PSB_DISPATCH_DTYPE(g_dtype, TG, {
      PSB_DISPATCH_DTYPE(copy_dtype, TX, {
        psb_launch(gated_norm_add_kernel<TY, TG, TX>, dim3(rows), dim3(threads), 0, stream, (float*)h, (const TY*)y,
                   (const TG*)g, (const float*)bias, (const float*)gain, (TX*)copy, H, eps, mult);
      });
    });
  });
  PSB_LAUNCH_CHECK("gated_norm_add");
  return 0;
}
