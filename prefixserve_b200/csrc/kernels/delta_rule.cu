// The gated delta rule: a linear-attention mixer whose per-head state is a matrix S [dim, vdim] that forgets by a
// per-token decay and is corrected towards each new value.
//
// The step's fused input projection is [T, 2 G dim + 2 H vdim] in the compute type: queries and keys of G groups,
// values of H heads, then the output gate (H vdim).  A second small product gives, in float32, the pre-activations
// of the write strength and of the decay, [T, 2 H].
//
// delta_prepare_kernel (a block per token): every query, key and value channel goes through a short causal
// convolution over its last K inputs (weights [channels, K], the last column the current token's, no bias, zeros
// before the start of the sequence; inputs from before the portion are read from the request's slot) and SiLU.
// Queries and keys are made unit vectors per group, x / sqrt(sum x^2 + 1e-6), queries also times dim^-1/2.  Per
// head, beta = sigmoid(b) and decay = exp(-exp(A_log) softplus(a + dt_bias)).  Everything after the projection is
// float32 and leaves the kernel as float32.
//
// delta_rule_kernel: per request and head, token by token,
//     S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q,
// so the read-out sees the current token's write.  The columns of S (one per value channel) never meet: R lanes of
// a warp hold one column between them (dim / R numbers each, in registers), so a warp carries 32 / R columns, and
// the two dot products of a token are finished by a butterfly among the R lanes.  The order of every sum depends on
// R and dim only, never on the batch.  Queries and keys of a run of tokens are staged in shared memory for the whole
// block.  The state is read from the request's slot at the portion's start and written back at its end; one block
// per request also brings the slot's convolution inputs up to date (the last K-1 rows of the projection, or what
// was there before, moved up, when the portion is shorter).
//
// delta_finish_kernel (a warp per token and head): o / sqrt(mean(o^2) + eps) * gain[vdim] * silu(gate), rounded to
// the compute type for the output projection.
//
// Slot layout (float32): [K-1, C] convolution inputs, oldest first (C = 2 G dim + H vdim), then S as [H, dim, vdim].
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float softplusf_(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ proj, const float* __restrict__ ba, const float* __restrict__ taps,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                     const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots, float* __restrict__ qkv,
                     float* __restrict__ bd, int G, int H, int dim, int vdim, int K, int num_slots, size_t slot_floats) {
  extern __shared__ float row[];  // [C] the token's convolved, activated channels
  __shared__ float factor[64];
  pdl_trigger();
  const int t = blockIdx.x;
  const int C = 2 * G * dim + H * vdim, P = C + H * vdim;
  pdl_wait();
  const int item = token_item[t];
  const int p = positions[t], p0 = positions[item_start[item]];
  int slot = slots[item];
  slot = slot < 0 ? 0 : (slot >= num_slots ? num_slots - 1 : slot);
  const float* tail = state + (size_t)slot * slot_floats;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const int src = p - (K - 1) + k;  // position of the input under tap k
      float x = 0.f;
      if (src >= p0) x = to_float<T>(proj[(size_t)(t - (p - src)) * P + c]);
      else if (src >= 0) x = tail[(size_t)(src - p0 + K - 1) * C + c];
      acc = fmaf(taps[(size_t)c * K + k], x, acc);
    }
    row[c] = siluf_(acc);
  }
  __syncthreads();
  // unit vectors: 2 G groups of dim channels (queries first), a warp per group in turn
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int g0 = 0; g0 < 2 * G; g0 += 64) {
    for (int g = g0 + warp; g < min(2 * G, g0 + 64); g += warps) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(row[g * dim + d], row[g * dim + d], ss);
      ss = warp_sum(ss);
      if (lane == 0) factor[g - g0] = (g < G ? rsqrtf((float)dim) : 1.f) / sqrtf(ss + 1e-6f);
    }
    __syncthreads();
    for (int c = g0 * dim + threadIdx.x; c < min(2 * G, g0 + 64) * dim; c += blockDim.x) row[c] *= factor[c / dim - g0];
    __syncthreads();
  }
  float* out = qkv + (size_t)t * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) out[c] = row[c];
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    bd[(size_t)t * 2 * H + h] = sigmoidf_(ba[(size_t)t * 2 * H + h]);
    bd[(size_t)t * 2 * H + H + h] = expf(-expf(a_log[h]) * softplusf_(ba[(size_t)t * 2 * H + H + h] + dt_bias[h]));
  }
}

constexpr int RULE_WARPS = 4;
constexpr int STAGE_TOKENS = 8;  // tokens whose queries and keys are staged together

// PER: numbers of a column one lane holds; R: lanes per column.  R * PER >= dim.
template <typename T, int PER, int R>
__global__ void __launch_bounds__(RULE_WARPS * 32)
delta_rule_kernel(const float* __restrict__ qkv, const float* __restrict__ bd, const T* __restrict__ proj,
                  float* __restrict__ state, const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots,
                  float* __restrict__ o, int G, int H, int dim, int vdim, int K, int num_slots, size_t slot_floats) {
  __shared__ float qk[STAGE_TOKENS][2][R * PER];
  constexpr int COLS = 32 / R;  // columns a warp holds
  pdl_trigger();
  const int C = 2 * G * dim + H * vdim, P = C + H * vdim;
  const int h = blockIdx.y, item = blockIdx.z;
  const int g = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane % R;
  const int col = (blockIdx.x * RULE_WARPS + warp) * COLS + lane / R;
  const bool live = col < vdim;
  pdl_wait();
  const int t0 = item_start[item], t1 = item_start[item + 1];
  int slot = slots[item];
  slot = slot < 0 ? 0 : (slot >= num_slots ? num_slots - 1 : slot);
  float* base = state + (size_t)slot * slot_floats;
  float* S = base + (size_t)(K - 1) * C + (size_t)h * dim * vdim;
  float s[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int d = r * PER + e;
    s[e] = (live && d < dim) ? S[(size_t)d * vdim + col] : 0.f;
  }
  for (int ts = t0; ts < t1; ts += STAGE_TOKENS) {
    const int n = min(STAGE_TOKENS, t1 - ts);
    __syncthreads();
    for (int i = threadIdx.x; i < n * 2 * R * PER; i += blockDim.x) {
      const int tok = i / (2 * R * PER), rest = i - tok * 2 * R * PER;
      const int which = rest / (R * PER), d = rest - which * R * PER;
      qk[tok][which][d] = d < dim ? qkv[(size_t)(ts + tok) * C + (size_t)which * G * dim + g * dim + d] : 0.f;
    }
    __syncthreads();
    for (int i = 0; i < n; ++i) {
      const int t = ts + i;
      const float beta = bd[(size_t)t * 2 * H + h], dec = bd[(size_t)t * 2 * H + H + h];
      const float v = live ? qkv[(size_t)t * C + 2 * G * dim + h * vdim + col] : 0.f;
      const float* kk = &qk[i][1][r * PER];
      const float* qq = &qk[i][0][r * PER];
      float kd = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        s[e] *= dec;
        kd = fmaf(kk[e], s[e], kd);
      }
#pragma unroll
      for (int off = 1; off < R; off <<= 1) kd += __shfl_xor_sync(0xffffffffu, kd, off);
      const float u = beta * (v - kd);
      float od = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        s[e] = fmaf(kk[e], u, s[e]);
        od = fmaf(qq[e], s[e], od);
      }
#pragma unroll
      for (int off = 1; off < R; off <<= 1) od += __shfl_xor_sync(0xffffffffu, od, off);
      if (live && r == 0) o[((size_t)t * H + h) * vdim + col] = od;
    }
  }
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int d = r * PER + e;
    if (live && d < dim) S[(size_t)d * vdim + col] = s[e];
  }
  // the slot's convolution inputs: the K-1 positions before the next token
  if (blockIdx.x == 0 && h == 0 && K > 1 && t1 > t0) {
    const int n = t1 - t0;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float keep[MAX_TAPS];
#pragma unroll
      for (int k = 0; k < MAX_TAPS; ++k) {
        if (k >= K - 1) break;
        const int back = K - 1 - k;  // this row is the input ``back`` positions before the next token
        keep[k] = back <= n ? to_float<T>(proj[(size_t)(t1 - back) * P + c]) : base[(size_t)(k + n) * C + c];
      }
#pragma unroll
      for (int k = 0; k < MAX_TAPS; ++k) {
        if (k >= K - 1) break;
        base[(size_t)k * C + c] = keep[k];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o, const T* __restrict__ proj, const float* __restrict__ gain,
                    T* __restrict__ out, long long units, int G, int H, int dim, int vdim, float eps) {
  pdl_trigger();
  pdl_wait();
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= units) return;
  const long long t = unit / H;
  const int h = (int)(unit - t * H);
  const int C = 2 * G * dim + H * vdim, P = C + H * vdim;
  const float* orow = o + (size_t)unit * vdim;
  const T* gate = proj + (size_t)t * P + C + (size_t)h * vdim;
  float ss = 0.f;
  for (int j = lane; j < vdim; j += 32) ss = fmaf(orow[j], orow[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  T* orow_out = out + (size_t)unit * vdim;
  for (int j = lane; j < vdim; j += 32) orow_out[j] = from_float<T>(orow[j] * inv * gain[j] * siluf_(to_float<T>(gate[j])));
}

template <typename T, int PER, int R>
void launch_rule(dim3 grid, cudaStream_t stream, const float* qkv, const float* bd, const T* proj, float* state,
                 const int32_t* item_start, const int32_t* slots, float* o, int G, int H, int dim, int vdim, int K,
                 int num_slots, size_t slot_floats) {
  psb_launch(delta_rule_kernel<T, PER, R>, grid, dim3(RULE_WARPS * 32), 0, stream, qkv, bd, proj, state, item_start, slots, o,
             G, H, dim, vdim, K, num_slots, slot_floats);
}

}  // namespace

PSB_API int psb_delta_max_taps() { return MAX_TAPS; }

// (proj, dtype, ba, taps, a_log, dt_bias, state, positions, token_item, item_start, slots, qkv_out, bd_out, T, G, H, dim,
//  vdim, K, num_slots, slot_floats, stream)
PSB_API int psb_delta_prepare(const void* proj, int dtype, const void* ba, const void* taps, const void* a_log,
                              const void* dt_bias, const void* state, const void* positions, const void* token_item,
                              const void* item_start, const void* slots, void* qkv, void* bd, int T, int G, int H, int dim,
                              int vdim, int K, int num_slots, long long slot_floats, cudaStream_t stream) {
  if (T < 0 || G < 1 || H < 1 || H % G || dim < 1 || vdim < 1) PSB_REFUSE("delta_prepare: bad sizes G=%d H=%d dim=%d vdim=%d", G, H, dim, vdim);
  if (K < 1 || K > MAX_TAPS) PSB_REFUSE("delta_prepare: %d taps are outside [1, %d]", K, MAX_TAPS);
  const long long C = 2LL * G * dim + (long long)H * vdim;
  if (slot_floats != (K - 1) * C + (long long)H * dim * vdim) PSB_REFUSE("delta_prepare: a slot of %lld numbers does not fit the sizes", slot_floats);
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 48 * 1024) PSB_REFUSE("delta_prepare: %lld channels exceed the kernel's shared memory", C);
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    psb_launch(delta_prepare_kernel<T_>, dim3(T), dim3(256), smem, stream, (const T_*)proj, (const float*)ba, (const float*)taps,
               (const float*)a_log, (const float*)dt_bias, (const float*)state, (const int32_t*)positions,
               (const int32_t*)token_item, (const int32_t*)item_start, (const int32_t*)slots, (float*)qkv, (float*)bd, G, H, dim,
               vdim, K, num_slots, (size_t)slot_floats);
  });
  PSB_LAUNCH_CHECK("delta_prepare");
  return 0;
}

// (qkv, bd, proj, dtype, state, item_start, slots, o_out, items, G, H, dim, vdim, K, num_slots, slot_floats, lanes, stream)
// ``lanes``: lanes of a warp that share a column of the state (4: a warp reads whole sectors of the state, for steps
// of single tokens; 16: short chains per token, for long portions).
PSB_API int psb_delta_rule(const void* qkv, const void* bd, const void* proj, int dtype, void* state, const void* item_start,
                           const void* slots, void* o, int items, int G, int H, int dim, int vdim, int K, int num_slots,
                           long long slot_floats, int lanes, cudaStream_t stream) {
  if (items < 0 || G < 1 || H < 1 || H % G || dim < 1 || vdim < 1) PSB_REFUSE("delta_rule: bad sizes G=%d H=%d dim=%d vdim=%d", G, H, dim, vdim);
  if (K < 1 || K > MAX_TAPS) PSB_REFUSE("delta_rule: %d taps are outside [1, %d]", K, MAX_TAPS);
  if (lanes != 4 && lanes != 16) PSB_REFUSE("delta_rule: %d lanes a column is not built (4 or 16)", lanes);
  if (dim > 64 * lanes) PSB_REFUSE("delta_rule: key size %d exceeds %d", dim, 64 * lanes);
  if (H > 65535 || items > 65535) PSB_REFUSE("delta_rule: too many heads or requests for one launch");
  if (items == 0) return 0;
  const int per = (dim + lanes - 1) / lanes;
  const int cols = RULE_WARPS * (32 / lanes);
  const dim3 grid((vdim + cols - 1) / cols, H, items);
#define RULE(PER_, R_)                                                                                                \
  launch_rule<T_, PER_, R_>(grid, stream, (const float*)qkv, (const float*)bd, (const T_*)proj, (float*)state,       \
                            (const int32_t*)item_start, (const int32_t*)slots, (float*)o, G, H, dim, vdim, K, num_slots, \
                            (size_t)slot_floats)
  PSB_DISPATCH_DTYPE(dtype, T_, {
    if (lanes == 4) {
      if (per <= 4) RULE(4, 4);
      else if (per <= 8) RULE(8, 4);
      else if (per <= 16) RULE(16, 4);
      else if (per <= 32) RULE(32, 4);
      else RULE(64, 4);
    } else {
      if (per <= 2) RULE(2, 16);
      else if (per <= 4) RULE(4, 16);
      else if (per <= 8) RULE(8, 16);
      else RULE(16, 16);
    }
  });
#undef RULE
  PSB_LAUNCH_CHECK("delta_rule");
  return 0;
}

// (o, proj, dtype, gain, out, T, G, H, dim, vdim, eps, stream)
PSB_API int psb_delta_finish(const void* o, const void* proj, int dtype, const void* gain, void* out, int T, int G, int H,
                             int dim, int vdim, float eps, cudaStream_t stream) {
  if (T < 0 || G < 1 || H < 1 || dim < 1 || vdim < 1) PSB_REFUSE("delta_finish: bad sizes");
  if (T == 0) return 0;
  const long long units = (long long)T * H;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    psb_launch(delta_finish_kernel<T_>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, (const float*)o, (const T_*)proj,
               (const float*)gain, (T_*)out, units, G, H, dim, vdim, eps);
  });
  PSB_LAUNCH_CHECK("delta_finish");
  return 0;
}
