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

__device__ __forceinline__ void unpack8(const uint4& raw, float (&o)[8]) {
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h2[k]);
    o[2 * k] = f.x;
    o[2 * k + 1] = f.y;
  }
}

// The same for bfloat16 y and g with H a multiple of 8: every thread keeps its pieces of eight gated values in
// registers between the two passes (PIECES * blockDim * 8 >= H), so y and g are read once.
template <int PIECES>
__global__ void gated_norm_add_vec_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ y,
                                          const __nv_bfloat16* __restrict__ g, const float* __restrict__ bias,
                                          const float* __restrict__ gain, __nv_bfloat16* __restrict__ copy, int H, float eps,
                                          float mult) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const size_t r = blockIdx.x;
  const int vecs = H >> 3;
  float z[PIECES][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PIECES; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < vecs) {
      unpack8(reinterpret_cast<const uint4*>(y + r * H)[v], z[i]);
      if (g) {
        float gg[8];
        unpack8(reinterpret_cast<const uint4*>(g + r * H)[v], gg);
#pragma unroll
        for (int e = 0; e < 8; ++e) z[i][e] *= sigmoidf_(gg[e] + (bias ? bias[8 * v + e] : 0.f));
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += z[i][e] * z[i][e];
    }
  }
  const float inv = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps);
#pragma unroll
  for (int i = 0; i < PIECES; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < vecs) {
      float* hp = h + r * H + 8 * v;
      const float4 a = *reinterpret_cast<const float4*>(hp), b = *reinterpret_cast<const float4*>(hp + 4);
      float o[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] += mult * (gain[8 * v + e] * (z[i][e] * inv));
      *reinterpret_cast<float4*>(hp) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4*>(hp + 4) = make_float4(o[4], o[5], o[6], o[7]);
      if (copy) {
        uint4 raw;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(o[2 * k], o[2 * k + 1]);
        reinterpret_cast<uint4*>(copy + r * H)[v] = raw;
      }
    }
  }
}

}  // namespace

PSB_API int psb_gated_norm_add(void* h, const void* y, int y_dtype, const void* g, int g_dtype, const void* bias,
                               const void* gain, void* copy, int copy_dtype, int rows, int H, float eps, float mult,
                               cudaStream_t stream) {
  if (rows < 0 || H < 1) PSB_REFUSE("gated_norm_add: bad sizes rows=%d H=%d", rows, H);
  if (!(eps > 0.f)) PSB_REFUSE("gated_norm_add: eps must be positive");
  if (rows == 0) return 0;
  if (y_dtype == PSB_BF16 && (!g || g_dtype == PSB_BF16) && (!copy || copy_dtype == PSB_BF16) && H % 8 == 0 && H <= 16384 &&
      (((uintptr_t)h | (uintptr_t)y | (uintptr_t)g | (uintptr_t)copy) & 15) == 0) {
    const int vecs = H / 8;
    const int vthreads = vecs >= 256 ? 256 : (vecs >= 128 ? 128 : 64);
    const int pieces = (vecs + vthreads - 1) / vthreads;
#define GNA_VEC(P)                                                                                                       \
    psb_launch(gated_norm_add_vec_kernel<P>, dim3(rows), dim3(vthreads), 0, stream, (float*)h, (const __nv_bfloat16*)y,  \
               (const __nv_bfloat16*)g, (const float*)bias, (const float*)gain, (__nv_bfloat16*)copy, H, eps, mult)
    if (pieces <= 1) GNA_VEC(1); else if (pieces <= 2) GNA_VEC(2); else if (pieces <= 4) GNA_VEC(4); else GNA_VEC(8);
#undef GNA_VEC
    PSB_LAUNCH_CHECK("gated_norm_add");
    return 0;
  }
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
