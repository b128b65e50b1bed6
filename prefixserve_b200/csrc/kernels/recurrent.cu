// A gated linear recurrence with a short causal convolution in front (the recurrent block of Griffin-like models).
//
// Per request and channel c the layer carries a float32 state S and the last K-1 inputs of the convolution; both
// live in the request's slot, ``state`` [num_slots, K, W]: rows 0..K-2 the convolution's inputs at the K-1 positions
// before the next token (oldest first), row K-1 the state S.  A fresh slot is all zeros, which is what the
// convolution reads before the start of a sequence and the recurrence starts from.
//
// The step's fused input projection is [T, 2W]: the gate branch, then the convolution branch (biases not yet
// added).  causal_conv_kernel adds the bias, rounds to the compute type, and convolves:
//   u_t[c] = sum_k w[c][k] x_(t-K+1+k)[c] + b[c]         (w's last column multiplies the current token)
// taking inputs from before the portion out of the slot.  A batched product then gives the pre-activations of the
// two gates, block by block of the channels ([T, blocks, 2 * W/blocks] float32: recurrence gate, input gate), and
// recurrence_scan_kernel runs, one thread per (portion or chunk of it, channel) over its tokens in order:
//   r = sigmoid(.. + br), i = sigmoid(.. + bi), a = exp(-decay * r * softplus(lam)),
//   S = a S + sqrt(1 - a^2) * i * u,        out = S * gelu_tanh(gate branch + bias)
// all in float32; then it leaves S and the portion's last K-1 convolution inputs in the slot (after every block of
// the convolution kernel has finished reading the old ones: a later launch).  A long portion is cut into chunks
// that run side by side: S -> a S + b composes, so a first pass (recurrence_chunk_kernel) reduces every chunk to
// one such map and the second pass folds the maps of the chunks in front of its own before it starts.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float softplusf_(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// CONV_TOKENS: tokens a block of the convolution handles, their look-ups in flight together (8 for prompt portions,
// 1 for a handful of decoded tokens, where the blocks are few as it is)
template <typename T, int CONV_TOKENS>
__global__ void causal_conv_kernel(const T* __restrict__ proj, const float* __restrict__ bias_x,
                                   const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                   const float* __restrict__ state, const int32_t* __restrict__ positions,
                                   const int32_t* __restrict__ token_item, const int32_t* __restrict__ item_start,
                                   const int32_t* __restrict__ slots, T* __restrict__ u_out, int T_tokens, int W, int K,
                                   int num_slots) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int tb = blockIdx.x * CONV_TOKENS;
  int p[CONV_TOKENS], p0[CONV_TOKENS], slot[CONV_TOKENS];
#pragma unroll
  for (int i = 0; i < CONV_TOKENS; ++i) {
    const int t = min(tb + i, T_tokens - 1);
    const int item = token_item[t];
    p[i] = positions[t];
    p0[i] = positions[item_start[item]];  // position of the portion's first token in the step
    const int s = slots[item];
    slot[i] = s < 0 ? 0 : (s >= num_slots ? num_slots - 1 : s);
  }
  if (c >= W) return;
  const float bx = bias_x[c], cb = conv_b[c];
#pragma unroll
  for (int i = 0; i < CONV_TOKENS; ++i) {
    const int t = tb + i;
    if (t >= T_tokens) break;
    const float* tail = state + (size_t)slot[i] * K * W;
    float acc = cb;
    for (int k = 0; k < K; ++k) {
      const int src = p[i] - (K - 1) + k;  // position of the input under tap k
      float x = 0.f;
      if (src >= p0[i]) x = to_float<T>(from_float<T>(to_float<T>(proj[(size_t)(t - (p[i] - src)) * 2 * W + W + c]) + bx));
      else if (src >= 0) x = tail[(size_t)(src - p0[i] + K - 1) * W + c];
      acc = fmaf(conv_w[(size_t)c * K + k], x, acc);
    }
    u_out[(size_t)t * W + c] = from_float<T>(acc);
  }
}

// Which portion and which of its chunks a block works on: chunks of ``chunk`` tokens are numbered through the step's
// portions in order.  False when the number is beyond the last chunk (the grid is sized by an upper bound).
__device__ __forceinline__ bool find_chunk(const int32_t* __restrict__ item_start, int items, int chunk, int g, int& item,
                                           int& index, int& count) {
  for (int i = 0; i < items; ++i) {
    const int n = item_start[i + 1] - item_start[i];
    const int c = (n + chunk - 1) / chunk;
    if (g < c) {
      item = i;
      index = g;
      count = c;
      return true;
    }
    g -= c;
  }
  return false;
}

// First pass over a portion cut into chunks: every chunk's decay product A and its result B from a zero state, so
// that the state entering chunk k is the fold of S -> A_j S + B_j over the chunks before it.  Portions of one chunk
// are skipped (the second pass starts them from the slot's state directly).
template <typename T>
__global__ void recurrence_chunk_kernel(const T* __restrict__ u, const float* __restrict__ gates,
                                        const float* __restrict__ bias_r, const float* __restrict__ bias_i,
                                        const float* __restrict__ lam, const int32_t* __restrict__ item_start,
                                        float2* __restrict__ carry, int items, int W, int block_width, int chunk, float decay) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  int item, index, count;
  if (c >= W || !find_chunk(item_start, items, chunk, blockIdx.y, item, index, count) || count == 1) return;
  const int t0 = item_start[item] + index * chunk, t1 = min(t0 + chunk, item_start[item + 1]);
  const int blk = c / block_width, j = c - blk * block_width;
  const float* g = gates + (size_t)blk * 2 * block_width + j;
  const float br = bias_r[c], bi = bias_i[c];
  const float rate = decay * softplusf_(lam[c]);
  float A = 1.f, B = 0.f;
  constexpr int UNROLL = 8;
  for (int t = t0; t < t1; t += UNROLL) {
    float gr[UNROLL], gi[UNROLL], uu[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {  // the loads of several tokens in flight together
      const int tt = t + k < t1 ? t + k : t1 - 1;
      gr[k] = g[(size_t)tt * 2 * W];
      gi[k] = g[(size_t)tt * 2 * W + block_width];
      uu[k] = to_float<T>(u[(size_t)tt * W + c]);
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      if (t + k >= t1) break;
      const float r = sigmoidf_(gr[k] + br), i = sigmoidf_(gi[k] + bi);
      const float a = expf(-rate * r);
      B = a * B + sqrtf(1.f - a * a) * (i * uu[k]);
      A *= a;
    }
  }
  carry[(size_t)blockIdx.y * W + c] = make_float2(A, B);
}

template <typename T>
__global__ void recurrence_scan_kernel(const T* __restrict__ proj, const T* __restrict__ u, const float* __restrict__ gates,
                                       const float* __restrict__ bias_y, const float* __restrict__ bias_x,
                                       const float* __restrict__ bias_r, const float* __restrict__ bias_i,
                                       const float* __restrict__ lam, float* __restrict__ state,
                                       const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots,
                                       const float2* __restrict__ carry, T* __restrict__ out, int items, int W, int K,
                                       int block_width, int num_slots, int chunk, float decay) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  int item, index, count;
  if (c >= W || !find_chunk(item_start, items, chunk, blockIdx.y, item, index, count)) return;
  const int slot = slots[item];
  if (slot < 0 || slot >= num_slots) return;
  const int t0 = item_start[item] + index * chunk, t1 = min(t0 + chunk, item_start[item + 1]);
  float* mine = state + (size_t)slot * K * W + c;  // this channel's column of the slot
  float S = mine[(size_t)(K - 1) * W];
  for (int k = 0; k < index; ++k) {  // through the chunks before this one
    const float2 ab = carry[(size_t)(blockIdx.y - index + k) * W + c];
    S = ab.x * S + ab.y;
  }
  const int blk = c / block_width, j = c - blk * block_width;
  const float* g = gates + (size_t)blk * 2 * block_width + j;  // + t * 2W: recurrence gate; + block_width: input gate
  const float br = bias_r[c], bi = bias_i[c], by = bias_y[c];
  const float rate = decay * softplusf_(lam[c]);
  constexpr int UNROLL = 8;
  for (int t = t0; t < t1; t += UNROLL) {
    float gr[UNROLL], gi[UNROLL], uu[UNROLL], yy[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {  // the loads of several tokens in flight together: none depends on S
      const int tt = t + k < t1 ? t + k : t1 - 1;
      gr[k] = g[(size_t)tt * 2 * W];
      gi[k] = g[(size_t)tt * 2 * W + block_width];
      uu[k] = to_float<T>(u[(size_t)tt * W + c]);
      yy[k] = to_float<T>(proj[(size_t)tt * 2 * W + c]);
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      if (t + k >= t1) break;
      const float r = sigmoidf_(gr[k] + br), i = sigmoidf_(gi[k] + bi);
      const float a = expf(-rate * r);
      S = a * S + sqrtf(1.f - a * a) * (i * uu[k]);
      const float y = to_float<T>(from_float<T>(gate_act(to_float<T>(from_float<T>(yy[k] + by)), PSB_ACT_GELU_TANH)));
      out[(size_t)(t + k) * W + c] = from_float<T>(S * y);
    }
  }
  if (index != count - 1) return;  // the portion's last chunk leaves the state behind
  mine[(size_t)(K - 1) * W] = S;
  // the convolution's inputs at the last K-1 positions: from this portion where it reaches, else shifted up
  const int n = item_start[item + 1] - item_start[item];
  float keep[MAX_TAPS];
  const float bx = bias_x[c];
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k < K - 1) {
      const int back = K - 1 - k;  // this row is the input ``back`` positions before the next token
      keep[k] = back <= n ? to_float<T>(from_float<T>(to_float<T>(proj[(size_t)(t1 - back) * 2 * W + W + c]) + bx))
                          : mine[(size_t)(k + n) * W];
    }
  }
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k)
    if (k < K - 1) mine[(size_t)k * W] = keep[k];
}

}  // namespace

PSB_API int psb_recurrence_max_taps() { return MAX_TAPS; }

PSB_API int psb_causal_conv(const void* proj, int dtype, const void* bias_x, const void* conv_w, const void* conv_b,
                            const void* state, const void* positions, const void* token_item, const void* item_start,
                            const void* slots, void* u_out, int T, int W, int K, int num_slots, cudaStream_t stream) {
  if (T < 0 || W < 1 || K < 1 || K > MAX_TAPS || num_slots < 1) PSB_REFUSE("causal_conv: bad sizes T=%d W=%d taps=%d (at most %d)", T, W, K, MAX_TAPS);
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (T >= 256) {
      psb_launch(causal_conv_kernel<T_, 8>, dim3((T + 7) / 8, (W + 127) / 128), dim3(128), 0, stream,
                 (const T_*)proj, (const float*)bias_x, (const float*)conv_w, (const float*)conv_b, (const float*)state,
                 (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start, (const int32_t*)slots,
                 (T_*)u_out, T, W, K, num_slots);
    } else {
      psb_launch(causal_conv_kernel<T_, 1>, dim3(T, (W + 127) / 128), dim3(128), 0, stream,
                 (const T_*)proj, (const float*)bias_x, (const float*)conv_w, (const float*)conv_b, (const float*)state,
                 (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start, (const int32_t*)slots,
                 (T_*)u_out, T, W, K, num_slots);
    }
  });
  PSB_LAUNCH_CHECK("causal_conv");
  return 0;
}

PSB_API int psb_recurrence_scan(const void* proj, const void* u, int dtype, const void* gates, const void* bias_y,
                                const void* bias_x, const void* bias_r, const void* bias_i, const void* lam, void* state,
                                const void* item_start, const void* slots, void* carry, void* out, int items, int T, int W,
                                int K, int blocks, int num_slots, int chunk, float decay, cudaStream_t stream) {
  if (items < 0 || T < 0 || W < 1 || K < 1 || K > MAX_TAPS || blocks < 1 || W % blocks || num_slots < 1 || chunk < 1)
    PSB_REFUSE("recurrence_scan: bad sizes items=%d W=%d taps=%d blocks=%d chunk=%d", items, W, K, blocks, chunk);
  if (items == 0 || T == 0) return 0;
  const int chunks = T / chunk + items;  // at least the number of chunks of any cutting of T tokens into ``items`` portions
  if (chunks > 65535) PSB_REFUSE("recurrence_scan: %d chunks in one step are too many for this kernel", chunks);
  if (chunk < T && !carry) PSB_REFUSE("recurrence_scan: portions cut into chunks need the carry buffer");
  const int threads = 64;
  const dim3 grid((W + threads - 1) / threads, chunks);
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (chunk < T) {
      psb_launch(recurrence_chunk_kernel<T_>, grid, dim3(threads), 0, stream, (const T_*)u, (const float*)gates,
                 (const float*)bias_r, (const float*)bias_i, (const float*)lam, (const int32_t*)item_start, (float2*)carry,
                 items, W, W / blocks, chunk, decay);
    }
    psb_launch(recurrence_scan_kernel<T_>, grid, dim3(threads), 0, stream, (const T_*)proj, (const T_*)u,
               (const float*)gates, (const float*)bias_y, (const float*)bias_x, (const float*)bias_r, (const float*)bias_i,
               (const float*)lam, (float*)state, (const int32_t*)item_start, (const int32_t*)slots, (const float2*)carry,
               (T_*)out, items, W, K, W / blocks, num_slots, chunk, decay);
  });
  PSB_LAUNCH_CHECK("recurrence_scan");
  return 0;
}
