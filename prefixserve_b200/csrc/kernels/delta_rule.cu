// The gated delta rule: a linear-attention mixer whose per-head state is a matrix S [dim, vdim] that forgets by a
// per-token decay and is corrected towards each new value.
//
// The step's fused input projection is [T, 2 G dim + 2 H vdim] in the compute type: queries and keys of G groups,
// values of H heads, then the output gate (H vdim).  A second small product gives, in float32, the pre-activations
// of the write strength and of the decay, [T, 2 H].
//
// delta_prepare_kernel (a block per token and query group, key group or value head): every query, key and value channel goes through a short causal
// convolution over its last K inputs (weights [channels, K], the last column the current token's, no bias, zeros
// before the start of the sequence; inputs from before the portion are read from the request's slot) and SiLU.
// Queries and keys are made unit vectors per group, x / sqrt(sum x^2 + 1e-6), queries also times dim^-1/2.  Per
// head, beta = sigmoid(b) and decay = exp(-exp(A_log) softplus(a + dt_bias)).  Everything after the projection is
// float32 and leaves the kernel as float32.
//
// delta_rule_kernel: per request and head, token by token,
//     S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q,
// so the read-out sees the current token's write (computed as decay (S_old^T q) + (q.k) u, which is the same).  The columns of S (one per value channel) never meet: R lanes of
// a warp hold one column between them (dim / R numbers each, in registers), so a warp carries 32 / R columns, and
// the two dot products of a token are finished by a butterfly among the R lanes.  The order of every sum depends on
// R and dim only, never on the batch.  What a run of tokens brings is staged in shared memory for the whole block, one
// run ahead of the arithmetic.  The state is read from the request's slot at the portion's start and written back at its end; one block
// per request also brings the slot's convolution inputs up to date (the last K-1 rows of the projection, or what
// was there before, moved up, when the portion is shorter).
//
// delta_cross_kernel (a warp per token and head): q.k, and k.k' and q.k' with the key of the token before.
//
// delta_finish_kernel (a warp per token and head): o / sqrt(mean(o^2) + eps) * gain[vdim] * silu(gate), rounded to
// the compute type for the output projection.
//
// Slot layout (float32): [K-1, C] convolution inputs, oldest first (C = 2 G dim + H vdim), then S as [H, dim, vdim].
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
// Per token and head the recurrence is handed five numbers, [T, BD, H]: beta, decay, and three dot products that do
// not depend on the state: q.k of the token, and k.k' and q.k' with the key k' of the token before it in the portion.
constexpr int BD = 5;

__device__ __forceinline__ float softplusf_(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }

// A block per (token, unit); a unit is one query group, one key group (dim channels each) or one value head (vdim).
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* __restrict__ proj, const float* __restrict__ ba, const float* __restrict__ taps,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                     const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots, float* __restrict__ qkv,
                     float* __restrict__ bd, int G, int H, int dim, int vdim, int K, int num_slots, size_t slot_floats,
                     int T_tokens, int tokens_per_block) {
  extern __shared__ float row[];  // the unit's convolved, activated channels
  __shared__ float scratch[4];
  const int unit = blockIdx.y;
  const int C = 2 * G * dim + H * vdim, P = C + H * vdim;
  const int c0 = unit < 2 * G ? unit * dim : 2 * G * dim + (unit - 2 * G) * vdim;
  const int len = unit < 2 * G ? dim : vdim;
  pdl_wait();
  for (int t = blockIdx.x * tokens_per_block; t < min(T_tokens, (blockIdx.x + 1) * tokens_per_block); ++t) {
  __syncthreads();  // the last token's row and sums have been read
  const int item = token_item[t];
  const int p = positions[t], p0 = positions[item_start[item]];
  int slot = slots[item];
  slot = slot < 0 ? 0 : (slot >= num_slots ? num_slots - 1 : slot);
  const float* tail = state + (size_t)slot * slot_floats;
  float ss = 0.f;
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    const int c = c0 + i;
    float x[MAX_TAPS];
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {  // the inputs under the taps, asked for together
      if (k >= K) break;
      const int src = p - (K - 1) + k;
      x[k] = 0.f;
      if (src >= p0) x[k] = to_float<T>(proj[(size_t)(t - (p - src)) * P + c]);
      else if (src >= 0) x[k] = tail[(size_t)(src - p0 + K - 1) * C + c];
    }
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) {
      if (k >= K) break;
      acc = fmaf(taps[(size_t)c * K + k], x[k], acc);
    }
    const float v = siluf_(acc);
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  float factor = 1.f;
  if (unit < 2 * G) {  // unit vectors; queries also times dim^-1/2
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float total = scratch[0] + scratch[1] + scratch[2] + scratch[3];
    factor = (unit < G ? rsqrtf((float)dim) : 1.f) / sqrtf(total + 1e-6f);
  }
  float* out = qkv + (size_t)t * C + c0;
  for (int i = threadIdx.x; i < len; i += blockDim.x) out[i] = row[i] * factor;  // a thread reads back what it wrote
  if (unit == 0) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      bd[(size_t)t * BD * H + h] = sigmoidf_(ba[(size_t)t * 2 * H + h]);
      bd[(size_t)t * BD * H + H + h] = expf(-expf(a_log[h]) * softplusf_(ba[(size_t)t * 2 * H + H + h] + dt_bias[h]));
    }
  }
  }
  // At the end, not at the start: the recurrence behind this kernel has few blocks that live long.  Let in while this
  // kernel's blocks fill the SMs, they crowd onto the few SMs with room and stay there, several to a scheduler; a
  // 2,048-token portion then took 1.4 ms a layer instead of 0.7.
  pdl_trigger();
}

// A warp per (token, head): the three state-free dot products of the unit vectors delta_prepare_kernel left.
__global__ void __launch_bounds__(128)
delta_cross_kernel(const float* __restrict__ qkv, const int32_t* __restrict__ token_item, const int32_t* __restrict__ item_start,
                   float* __restrict__ bd, long long units, int G, int H, int dim, int vdim) {
  pdl_wait();  // (no early trigger: the recurrence comes next, see the end of delta_prepare_kernel)
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= units) return;
  const long long t = unit / H;
  const int h = (int)(unit - t * H), g = h / (H / G);
  const int C = 2 * G * dim + H * vdim;
  const float* q = qkv + (size_t)t * C + (size_t)g * dim;
  const float* k = q + (size_t)G * dim;
  const bool first = t == item_start[token_item[t]];  // no token before it in this step's portion
  const float* kp = first ? k : k - C;
  float qk = 0.f, kk = 0.f, qkp = 0.f;
  for (int d = lane; d < dim; d += 32) {
    const float qv = q[d], kv = k[d], pv = kp[d];
    qk = fmaf(qv, kv, qk);
    kk = fmaf(kv, pv, kk);
    qkp = fmaf(qv, pv, qkp);
  }
  qk = warp_sum(qk); kk = warp_sum(kk); qkp = warp_sum(qkp);
  if (lane == 0) {
    float* out = bd + (size_t)t * BD * H + h;
    out[2 * H] = qk;
    out[3 * H] = first ? 0.f : kk;
    out[4 * H] = first ? 0.f : qkp;
  }
}

constexpr int RULE_WARPS = 4;

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// PER: numbers of a column one lane holds; R: lanes per column.  R * PER >= dim.  What the tokens of a stage bring
// (queries, keys, the block's value columns, beta, decay) is copied into shared memory one stage ahead of the
// arithmetic (cp.async into the other of two buffers), so the chain from token to token never waits for memory.
//
// The chain itself is kept short: with S the state before the token, the sums k.S and q.S (per column) are finished by
// one butterfly, q.k comes ready-made (it does not depend on the state: delta_cross_kernel), and then
//     u = beta (v - dec k.S),   o = dec q.S + (q.k) u,   S <- dec S + k u^T,
// which is the read-out of the updated state written so that it does not wait for the update.  Tokens go two a round
// (see the loop): one butterfly for both.
template <typename T, int PER, int R>
__global__ void __launch_bounds__(RULE_WARPS * 32)
delta_rule_kernel(const float* __restrict__ qkv, const float* __restrict__ bd, const T* __restrict__ proj,
                  float* __restrict__ state, const int32_t* __restrict__ item_start, const int32_t* __restrict__ slots,
                  float* __restrict__ o, int G, int H, int dim, int vdim, int K, int num_slots, size_t slot_floats,
                  int stage_tokens) {
  extern __shared__ __align__(16) float staged[];  // [2][stage_tokens][W]
  constexpr int COLS = 32 / R;  // columns a warp holds
  constexpr int RP = R * PER, BC = RULE_WARPS * COLS, W = (2 * RP + BC + BD + 3) / 4 * 4;
  static_assert(RP % 4 == 0, "queries and keys of a token start on 16 bytes");
  const int C = 2 * G * dim + H * vdim, P = C + H * vdim;
  const int h = blockIdx.y, item = blockIdx.z;
  const int g = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane % R;
  const int col0 = blockIdx.x * BC, in_block = warp * COLS + lane / R;
  const int col = col0 + in_block;
  const bool live = col < vdim;
  // 16-byte copies of queries and keys need their rows on 16 bytes in the [T, C] array
  const bool wide = dim % 4 == 0 && C % 4 == 0 && (((uintptr_t)qkv) & 15) == 0;
  pdl_wait();
  const int t0 = item_start[item], t1 = item_start[item + 1];
  int slot = slots[item];
  slot = slot < 0 ? 0 : (slot >= num_slots ? num_slots - 1 : slot);
  float* base = state + (size_t)slot * slot_floats;
  float* S = base + (size_t)(K - 1) * C + (size_t)h * dim * vdim;

  auto stage = [&](int ts, float* buf) {  // tokens ts .. ts + stage_tokens - 1 (those before t1) into buf
    const int n = min(stage_tokens, t1 - ts);
    if (wide) {
      constexpr int PIECES = 2 * RP / 4;  // 16-byte pieces of a token's queries and keys
      for (int i = threadIdx.x; i < n * PIECES; i += blockDim.x) {
        const int tok = i / PIECES, e = (i - tok * PIECES) * 4;
        const int which = e / RP, d = e - which * RP;
        float* dst = buf + tok * W + e;
        if (d < dim) copy_async16(dst, qkv + (size_t)(ts + tok) * C + (size_t)which * G * dim + g * dim + d);
        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      for (int i = threadIdx.x; i < n * 2 * RP; i += blockDim.x) {
        const int tok = i / (2 * RP), e = i - tok * 2 * RP;
        const int which = e / RP, d = e - which * RP;
        if (d < dim) copy_async4(buf + tok * W + e, qkv + (size_t)(ts + tok) * C + (size_t)which * G * dim + g * dim + d);
        else buf[tok * W + e] = 0.f;
      }
    }
    for (int i = threadIdx.x; i < n * (BC + BD); i += blockDim.x) {
      const int tok = i / (BC + BD), e = i - tok * (BC + BD);
      float* dst = buf + tok * W + 2 * RP + e;
      if (e >= BC) copy_async4(dst, bd + (size_t)(ts + tok) * BD * H + (e - BC) * H + h);
      else if (col0 + e < vdim) copy_async4(dst, qkv + (size_t)(ts + tok) * C + 2 * G * dim + h * vdim + col0 + e);
      else *dst = 0.f;
    }
  };

  if (t1 > t0) stage(t0, staged);
  float s[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int d = r * PER + e;
    s[e] = (live && d < dim) ? S[(size_t)d * vdim + col] : 0.f;
  }
  int which_buf = 0;
  for (int ts = t0; ts < t1; ts += stage_tokens, which_buf ^= 1) {
    const int n = min(stage_tokens, t1 - ts);
    copy_async_wait();
    __syncthreads();  // this stage has landed for everybody, and everybody has left the other buffer
    if (ts + stage_tokens < t1) stage(ts + stage_tokens, staged + (size_t)(which_buf ^ 1) * stage_tokens * W);
    const float* buf = staged + (size_t)which_buf * stage_tokens * W;
    auto load_qk = [&](const float* tokrow, float (&qq)[PER], float (&kk)[PER]) {
      if constexpr (PER % 4 == 0) {
#pragma unroll
        for (int e = 0; e < PER; e += 4) {
          const float4 a = *reinterpret_cast<const float4*>(tokrow + r * PER + e);
          const float4 b4 = *reinterpret_cast<const float4*>(tokrow + RP + r * PER + e);
          qq[e] = a.x; qq[e + 1] = a.y; qq[e + 2] = a.z; qq[e + 3] = a.w;
          kk[e] = b4.x; kk[e + 1] = b4.y; kk[e + 2] = b4.z; kk[e + 3] = b4.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          qq[e] = tokrow[r * PER + e];
          kk[e] = tokrow[RP + r * PER + e];
        }
      }
    };
    int i = 0;
    // Two tokens a round.  With S the state before token a and b = a + 1, the four sums k_a.S, q_a.S, k_b.S, q_b.S are
    // finished by one butterfly; what token b needs of token a's write comes through the state-free products:
    //   u_a = beta_a (v_a - dec_a k_a.S),                              o_a = dec_a q_a.S + (q_a.k_a) u_a,
    //   u_b = beta_b (v_b - dec_b (dec_a k_b.S + (k_a.k_b) u_a)),      o_b = dec_b (dec_a q_b.S + (q_b.k_a) u_a) + (q_b.k_b) u_b,
    //   S <- dec_b dec_a S + k_a (dec_b u_a)^T + k_b u_b^T.
    for (; i + 1 < n; i += 2) {
      const float* ra = buf + i * W;
      const float* rb = ra + W;
      float qa[PER], ka[PER], qb[PER], kb[PER];
      load_qk(ra, qa, ka);
      load_qk(rb, qb, kb);
      const float va = ra[2 * RP + in_block], vb = rb[2 * RP + in_block];
      const float beta_a = ra[2 * RP + BC], dec_a = ra[2 * RP + BC + 1], qk_a = ra[2 * RP + BC + 2];
      const float beta_b = rb[2 * RP + BC], dec_b = rb[2 * RP + BC + 1], qk_b = rb[2 * RP + BC + 2];
      const float kk_ab = rb[2 * RP + BC + 3], qk_ba = rb[2 * RP + BC + 4];
      float kas = 0.f, qas = 0.f, kbs = 0.f, qbs = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        kas = fmaf(ka[e], s[e], kas);
        qas = fmaf(qa[e], s[e], qas);
        kbs = fmaf(kb[e], s[e], kbs);
        qbs = fmaf(qb[e], s[e], qbs);
      }
#pragma unroll
      for (int off = 1; off < R; off <<= 1) {
        kas += __shfl_xor_sync(0xffffffffu, kas, off);
        qas += __shfl_xor_sync(0xffffffffu, qas, off);
        kbs += __shfl_xor_sync(0xffffffffu, kbs, off);
        qbs += __shfl_xor_sync(0xffffffffu, qbs, off);
      }
      const float ua = beta_a * (va - dec_a * kas);
      const float ub = beta_b * (vb - dec_b * fmaf(kk_ab, ua, dec_a * kbs));
      const float dd = dec_b * dec_a, wa = dec_b * ua;
#pragma unroll
      for (int e = 0; e < PER; ++e) s[e] = fmaf(kb[e], ub, fmaf(ka[e], wa, dd * s[e]));
      if (live && r == 0) {
        float* orow = o + ((size_t)(ts + i) * H + h) * vdim + col;
        orow[0] = fmaf(qk_a, ua, dec_a * qas);
        orow[(size_t)H * vdim] = fmaf(qk_b, ub, dec_b * fmaf(qk_ba, ua, dec_a * qbs));
      }
    }
    for (; i < n; ++i) {  // a portion's last token when their number is odd (a single decoded token)
      const float* tokrow = buf + i * W;
      float qq[PER], kk[PER];
      load_qk(tokrow, qq, kk);
      const float v = tokrow[2 * RP + in_block];
      const float beta = tokrow[2 * RP + BC], dec = tokrow[2 * RP + BC + 1], qk = tokrow[2 * RP + BC + 2];
      float ks0 = 0.f, ks1 = 0.f, qs0 = 0.f, qs1 = 0.f;
#pragma unroll
      for (int e = 0; e < PER; e += 2) {
        ks0 = fmaf(kk[e], s[e], ks0);
        qs0 = fmaf(qq[e], s[e], qs0);
        if (e + 1 < PER) {
          ks1 = fmaf(kk[e + 1], s[e + 1], ks1);
          qs1 = fmaf(qq[e + 1], s[e + 1], qs1);
        }
      }
      float ksum = ks0 + ks1, qsum = qs0 + qs1;
#pragma unroll
      for (int off = 1; off < R; off <<= 1) {
        ksum += __shfl_xor_sync(0xffffffffu, ksum, off);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, off);
      }
      const float u = beta * (v - dec * ksum);
#pragma unroll
      for (int e = 0; e < PER; ++e) s[e] = fmaf(kk[e], u, dec * s[e]);
      if (live && r == 0) o[((size_t)(ts + i) * H + h) * vdim + col] = fmaf(qk, u, dec * qsum);
    }
  }
  // Only now may the next kernel's blocks come: this kernel has two warps a scheduler and is bound by their chains of
  // dependent instructions, and the next kernel reads what the last token writes anyway.
  pdl_trigger();
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
  constexpr int W = (2 * R * PER + RULE_WARPS * (32 / R) + BD + 3) / 4 * 4;
  // two buffers within the 48 KB a kernel has without asking: 16 tokens a stage for keys up to 128 numbers, 4 beyond
  const int stage_tokens = 2 * 16 * W * (int)sizeof(float) <= 48 * 1024 ? 16 : 4;
  static_assert(2 * 4 * W * sizeof(float) <= 48 * 1024, "a stage of four tokens fits the default shared memory twice");
  psb_launch(delta_rule_kernel<T, PER, R>, grid, dim3(RULE_WARPS * 32), (size_t)2 * stage_tokens * W * sizeof(float), stream, qkv,
             bd, proj, state, item_start, slots, o, G, H, dim, vdim, K, num_slots, slot_floats, stage_tokens);
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
  const size_t smem = (size_t)(dim > vdim ? dim : vdim) * sizeof(float);
  if (smem > 48 * 1024 || 2 * G + H > 65535) PSB_REFUSE("delta_prepare: sizes exceed the kernel's shared memory or grid");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    const int per_block = T >= 1024 ? 8 : 1;  // long steps: a block stays with its unit for eight tokens
    psb_launch(delta_prepare_kernel<T_>, dim3((T + per_block - 1) / per_block, 2 * G + H), dim3(128), smem, stream, (const T_*)proj,
               (const float*)ba, (const float*)taps, (const float*)a_log, (const float*)dt_bias, (const float*)state,
               (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start, (const int32_t*)slots,
               (float*)qkv, (float*)bd, G, H, dim, vdim, K, num_slots, (size_t)slot_floats, T, per_block);
  });
  PSB_LAUNCH_CHECK("delta_prepare");
  const long long units = (long long)T * H;
  psb_launch(delta_cross_kernel, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, (const float*)qkv, (const int32_t*)token_item,
             (const int32_t*)item_start, (float*)bd, units, G, H, dim, vdim);
  PSB_LAUNCH_CHECK("delta_cross");
  return 0;
}

// (qkv, bd, proj, dtype, state, item_start, slots, o_out, items, G, H, dim, vdim, K, num_slots, slot_floats, lanes, stream)
// ``lanes``: lanes of a warp that share a column of the state (4: a warp reads whole sectors of the state, for steps
// of single tokens; 16 or 32: short chains per token and more warps, for long portions).
PSB_API int psb_delta_rule(const void* qkv, const void* bd, const void* proj, int dtype, void* state, const void* item_start,
                           const void* slots, void* o, int items, int G, int H, int dim, int vdim, int K, int num_slots,
                           long long slot_floats, int lanes, cudaStream_t stream) {
  if (items < 0 || G < 1 || H < 1 || H % G || dim < 1 || vdim < 1) PSB_REFUSE("delta_rule: bad sizes G=%d H=%d dim=%d vdim=%d", G, H, dim, vdim);
  if (K < 1 || K > MAX_TAPS) PSB_REFUSE("delta_rule: %d taps are outside [1, %d]", K, MAX_TAPS);
  if (lanes != 4 && lanes != 16 && lanes != 32) PSB_REFUSE("delta_rule: %d lanes a column is not built (4, 16 or 32)", lanes);
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
    } else if (lanes == 16) {
      if (per <= 2) RULE(2, 16);
      else if (per <= 4) RULE(4, 16);
      else if (per <= 8) RULE(8, 16);
      else RULE(16, 16);
    } else {
      if (per <= 1) RULE(1, 32);
      else if (per <= 2) RULE(2, 32);
      else if (per <= 4) RULE(4, 32);
      else RULE(8, 32);
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
