// The norm behind a sublayer fused with the norm in front of the next one, for blocks that norm a sublayer's result
// before it joins the stream and norm the stream again before the next sublayer reads it:
//
//   h <- h + gain_post * y / sqrt(mean(y^2) + eps)            (float32 stream, updated in place)
//   x  = gain_pre * h / sqrt(mean(h^2) + eps)                  (optional; in the compute type)
//
// One block per row.  Rows of up to 4,096 numbers live in registers from one read to the last write (the gains are
// asked for ahead of the dependency wait); longer rows keep the new stream row in shared memory between the sum and
// the second norm and read y twice (the second time from the cache).  With ``rows`` the second
// norm is taken of the chosen rows only and written densely (the last use of the stream: the wanted positions);
// the update of the stream is then left out for rows that are not chosen.  Statistics and sums are float32, every
// thread adds the warps' partial sums in the same order.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_total(float v, float* scratch) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += scratch[w];
  return total;
}

template <typename TY, typename TX>
__global__ void __launch_bounds__(256)
norm_add_norm_kernel(float* __restrict__ h, const TY* __restrict__ y, const float* __restrict__ gain_post,
                     const float* __restrict__ gain_pre, const int32_t* __restrict__ rows, TX* __restrict__ x, int H,
                     float eps_post, float eps_pre) {
  extern __shared__ float fresh[];  // [H] the row of the stream after the sum
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (size_t)r * H;
  const TY* yr = y + (size_t)r * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_float<TY>(yr[j]);
    ss = fmaf(v, v, ss);
  }
  const float inv_y = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps_post);
  ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = hr[j] + gain_post[j] * (to_float<TY>(yr[j]) * inv_y);
    if (!rows) hr[j] = v;
    fresh[j] = v;
    ss = fmaf(v, v, ss);
  }
  if (!x) return;
  const float inv_h = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps_pre);
  TX* xr = x + (size_t)i * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) xr[j] = from_float<TX>(gain_pre[j] * (fresh[j] * inv_h));
}

// Rows of up to 256 * ITEMS numbers: everything a thread needs (its share of y, of the stream and of the two gains) is
// asked for at once and kept in registers, so the row is read once and the kernel waits for memory once.
template <typename TY, typename TX, int ITEMS>
__global__ void __launch_bounds__(256)
norm_add_norm_regs_kernel(float* __restrict__ h, const TY* __restrict__ y, const float* __restrict__ gain_post,
                          const float* __restrict__ gain_pre, const int32_t* __restrict__ rows, TX* __restrict__ x, int H,
                          float eps_post, float eps_pre) {
  __shared__ float scratch[32];
  pdl_trigger();
  float gpost[ITEMS], gpre[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {  // weights: before the wait
    const int j = threadIdx.x + 256 * k;
    gpost[k] = j < H ? gain_post[j] : 0.f;
    gpre[k] = (gain_pre && j < H) ? gain_pre[j] : 0.f;
  }
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* hr = h + (size_t)r * H;
  const TY* yr = y + (size_t)r * H;
  float yv[ITEMS], hv[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int j = threadIdx.x + 256 * k;
    yv[k] = j < H ? to_float<TY>(yr[j]) : 0.f;
    hv[k] = j < H ? hr[j] : 0.f;
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) ss = fmaf(yv[k], yv[k], ss);
  const float inv_y = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps_post);
  ss = 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int j = threadIdx.x + 256 * k;
    hv[k] = hv[k] + gpost[k] * (yv[k] * inv_y);
    if (!rows && j < H) hr[j] = hv[k];
    ss = fmaf(hv[k], hv[k], ss);  // beyond H: 0 + 0 * ...
  }
  if (!x) return;
  const float inv_h = 1.f / sqrtf(block_total(ss, scratch) / (float)H + eps_pre);
  TX* xr = x + (size_t)i * H;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int j = threadIdx.x + 256 * k;
    if (j < H) xr[j] = from_float<TX>(gpre[k] * (hv[k] * inv_h));
  }
}

}  // namespace

// (h, y, y_dtype, gain_post, gain_pre, rows, x, x_dtype, n_rows, H, eps_post, eps_pre, stream)
PSB_API int psb_norm_add_norm(void* h, const void* y, int y_dtype, const void* gain_post, const void* gain_pre, const void* rows,
                              void* x, int x_dtype, int n_rows, int H, float eps_post, float eps_pre, cudaStream_t stream) {
  if (n_rows < 0 || H < 1) PSB_REFUSE("norm_add_norm: bad sizes rows=%d H=%d", n_rows, H);
  if ((x == nullptr) != (gain_pre == nullptr)) PSB_REFUSE("norm_add_norm: the second norm needs its gain and its output, or neither");
  if (rows && !x) PSB_REFUSE("norm_add_norm: chosen rows without a second norm do nothing");
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) PSB_REFUSE("norm_add_norm: rows of %d numbers exceed the kernel's shared memory", H);
  if (n_rows == 0) return 0;
  PSB_DISPATCH_DTYPE(y_dtype, TY, {
    PSB_DISPATCH_DTYPE(x_dtype, TX, {
      if (H <= 256 * 4)
        psb_launch(norm_add_norm_regs_kernel<TY, TX, 4>, dim3(n_rows), dim3(256), 0, stream, (float*)h, (const TY*)y,
                   (const float*)gain_post, (const float*)gain_pre, (const int32_t*)rows, (TX*)x, H, eps_post, eps_pre);
      else if (H <= 256 * 16)
        psb_launch(norm_add_norm_regs_kernel<TY, TX, 16>, dim3(n_rows), dim3(256), 0, stream, (float*)h, (const TY*)y,
                   (const float*)gain_post, (const float*)gain_pre, (const int32_t*)rows, (TX*)x, H, eps_post, eps_pre);
      else
        psb_launch(norm_add_norm_kernel<TY, TX>, dim3(n_rows), dim3(256), smem, stream, (float*)h, (const TY*)y,
                   (const float*)gain_post, (const float*)gain_pre, (const int32_t*)rows, (TX*)x, H, eps_post, eps_pre);
    });
  });
  PSB_LAUNCH_CHECK("norm_add_norm");
  return 0;
}
