// Attention through a low-rank latent of the keys and values, with one rotated key part shared by all heads.
//
// A token's cache row holds its latent c (``rank`` numbers, already normed) followed by the rotated key part
// (``rot`` numbers): one row per token and layer, whatever the number of heads.  Layout of an entry:
// [num_pages, page_size, rank + rot].  Head h's key would be (U_k[h] c, k_rot) and its value U_v[h] c; instead of
// expanding them, the query is carried into the latent space (q' = U_k[h]^T q_plain, a batched product on the host
// side), so that
//   score(t, j) = (q'_t . c_j + q_rot_t . k_rot_j) * scale,   out_t = sum_j softmax_j(score) c_j,
// and the value matrix is applied once to out_t afterwards.  Key j is visible to the query at position p when
// 0 <= p - j < window (window 0: every earlier key).
//
// latent_prepare_kernel: one row of the fused input projection [query latent | key/value latent | rotated key part |
//   one gate per head] -> the normed query latent (compute type), the cache row (normed latent, rotated key part),
//   sigmoid of the gates (float32).  The norms are x / sqrt(mean(x^2) + eps) * gain in float32.
// latent_query_rotate_kernel: the rotated part of every head's query, turned by the token's position, into the
//   tail of the float32 query rows [T, heads, rank + rot] whose first ``rank`` columns the batched product fills.
// latent_attention_kernel: one block per (token, head) walks the visible keys in runs of 32 aligned to absolute
//   positions, the runs dealt out to its four warps in turn and the four partial results joined in warp order (the
//   order of every sum depends on the token's position only), scores and softmax in float32, the output (times the
//   head's gate) accumulated in registers.
//
// The rotation pairs element 2i with 2i+1 for i < rot_dims/2 (the rest of the rotated part passes through), angle
// tables float32 [positions, rot_dims/2].
#include <cfloat>

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

template <typename T, typename TKV>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ token_item, const int32_t* __restrict__ table,
                                      int table_width, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      const float* __restrict__ gain_q, const float* __restrict__ gain_kv,
                                      T* __restrict__ cq_out, float* __restrict__ gate_out, TKV* __restrict__ cache,
                                      int q_rank, int rank, int rot, int rot_dims, int heads, int page_size,
                                      int num_pages, int max_positions, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int width = q_rank + rank + rot + heads;
  const T* row = proj + (size_t)t * width;
  const int pos = positions[t];

  float ss = 0.f;
  for (int j = threadIdx.x; j < q_rank; j += blockDim.x) {
    const float v = to_float<T>(row[j]);
    ss += v * v;
  }
  const float inv_q = 1.f / sqrtf(block_total(ss, scratch) / (float)q_rank + eps);
  for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
    cq_out[(size_t)t * q_rank + j] = from_float<T>(gain_q[j] * (to_float<T>(row[j]) * inv_q));

  const T* kvrow = row + q_rank;
  ss = 0.f;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) {
    const float v = to_float<T>(kvrow[j]);
    ss += v * v;
  }
  const float inv_kv = 1.f / sqrtf(block_total(ss, scratch) / (float)rank + eps);

  const int item = token_item[t];
  const int page = pos >= 0 ? table[(size_t)item * table_width + pos / page_size] : -1;
  // the host checks tables before launch; a bad id is skipped rather than written through
  if (page >= 0 && page < num_pages) {
    TKV* dst = cache + ((size_t)page * page_size + (size_t)(pos % page_size)) * (rank + rot);
    for (int j = threadIdx.x; j < rank; j += blockDim.x)
      dst[j] = from_float<TKV>(gain_kv[j] * (to_float<T>(kvrow[j]) * inv_kv));
    const int safe_pos = pos >= max_positions ? max_positions - 1 : pos;
    const int half = rot_dims >> 1;
    const float* c = cos_t + (size_t)safe_pos * half;
    const float* s = sin_t + (size_t)safe_pos * half;
    const T* kr = kvrow + rank;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float o1, o2;
      rotate_pair(to_float<T>(kr[2 * j]), to_float<T>(kr[2 * j + 1]), c[j], s[j], o1, o2);
      dst[rank + 2 * j] = from_float<TKV>(o1);
      dst[rank + 2 * j + 1] = from_float<TKV>(o2);
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) dst[rank + j] = from_float<TKV>(to_float<T>(kr[j]));
  }
  const T* g = kvrow + rank + rot;
  for (int j = threadIdx.x; j < heads; j += blockDim.x) gate_out[(size_t)t * heads + j] = 1.f / (1.f + expf(-to_float<T>(g[j])));
}

template <typename T>
__global__ void latent_query_rotate_kernel(const T* __restrict__ q, const int32_t* __restrict__ positions,
                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                           float* __restrict__ q_lat, int heads, int plain, int rot, int rot_dims, int rank,
                                           int max_positions) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int safe_pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
  const int half = rot_dims >> 1;
  const float* c = cos_t + (size_t)safe_pos * half;
  const float* s = sin_t + (size_t)safe_pos * half;
  const int per_head = half + (rot - rot_dims);  // work items a head: the pairs, then the elements that pass through
  for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, j = idx - h * per_head;
    const T* src = q + ((size_t)t * heads + h) * (plain + rot) + plain;
    float* dst = q_lat + ((size_t)t * heads + h) * (rank + rot) + rank;
    if (j < half) {
      float o1, o2;
      rotate_pair(to_float<T>(src[2 * j]), to_float<T>(src[2 * j + 1]), c[j], s[j], o1, o2);
      dst[2 * j] = o1;
      dst[2 * j + 1] = o2;
    } else {
      const int e = rot_dims + (j - half);
      dst[e] = to_float<T>(src[e]);
    }
  }
}

constexpr int WARPS = 4;

// dot of a float32 query (shared memory) with a cached row, eight elements a load where the row allows it
template <typename TKV>
__device__ __forceinline__ float row_dot(const float* __restrict__ qs, const TKV* __restrict__ krow, int D, bool vec) {
  float dot = 0.f;
  int d = 0;
  if (vec) {
    for (; d + 8 <= D; d += 8) {
      float k[8];
      if constexpr (sizeof(TKV) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          k[2 * i] = f.x;
          k[2 * i + 1] = f.y;
        }
      } else {
        const float4 a = *reinterpret_cast<const float4*>(krow + d), b = *reinterpret_cast<const float4*>(krow + d + 4);
        k[0] = a.x; k[1] = a.y; k[2] = a.z; k[3] = a.w; k[4] = b.x; k[5] = b.y; k[6] = b.z; k[7] = b.w;
      }
      const float4 q0 = *reinterpret_cast<const float4*>(qs + d), q1 = *reinterpret_cast<const float4*>(qs + d + 4);
      dot = fmaf(q0.x, k[0], dot); dot = fmaf(q0.y, k[1], dot); dot = fmaf(q0.z, k[2], dot); dot = fmaf(q0.w, k[3], dot);
      dot = fmaf(q1.x, k[4], dot); dot = fmaf(q1.y, k[5], dot); dot = fmaf(q1.z, k[6], dot); dot = fmaf(q1.w, k[7], dot);
    }
  }
  for (; d < D; ++d) dot = fmaf(qs[d], to_float<TKV>(krow[d]), dot);
  return dot;
}

// One block per (token, head).  Its four warps take the runs of 32 keys in turn (run r goes to warp r mod 4), each
// with a running maximum, sum and output of its own; the four are then joined in warp order.  Lane l of a warp owns
// output columns 2l, 2l+1, 2l+64, ... (pairs, so that a bfloat16 row is read four bytes at a time).
template <typename TKV, typename TO, int NACC>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const float* __restrict__ q_lat, const TKV* __restrict__ cache, const int32_t* __restrict__ table,
                        int table_width, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                        const float* __restrict__ gate, TO* __restrict__ out, int T_tokens, int heads, int rank, int rot,
                        int page_size, int num_pages, int window, float scale) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = rank + rot;
  const int Dpad = (D + 3) & ~3;
  float* qs = smem;                         // [Dpad]
  float* part_ml = smem + Dpad;             // [WARPS][2]
  float* part_o = part_ml + 2 * WARPS;      // [WARPS][rank]
  const int t = blockIdx.x / heads, h = blockIdx.x - t * heads;
  const int p = positions[t];
  const int32_t* pages = table + (size_t)token_item[t] * table_width;
  const float* qrow = q_lat + ((size_t)t * heads + h) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qrow[d];
  __syncthreads();

  const bool vec = (D % 8 == 0);  // rows then start on 16-byte boundaries (the cache's base is aligned by its allocator)
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float m = -FLT_MAX, l = 0.f;
  float acc[NACC][2];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i][0] = acc[i][1] = 0.f;

  for (int base = (lo & ~31) + 32 * warp; base <= p; base += 32 * WARPS) {
    const int key = base + lane;
    const bool live = key >= lo && key <= p;
    long long off = -1;  // element offset of this lane's key row
    float s = -FLT_MAX;
    if (live) {
      const int page = pages[key / page_size];
      if (page >= 0 && page < num_pages) {
        off = ((long long)page * page_size + (key % page_size)) * D;
        s = row_dot<TKV>(qs, cache + off, D, vec) * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);   // first run: exp(-huge) = 0
    const float pr = off >= 0 ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      acc[i][0] *= alpha;
      acc[i][1] *= alpha;
    }
    const int n_live = min(32, p - base + 1);
    for (int j = 0; j < n_live; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pr, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;  // before the window
      const TKV* vrow = cache + oj;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = 2 * lane + 64 * i;
        if (d + 1 < rank) {
          if constexpr (sizeof(TKV) == 2) {
            if ((D & 1) == 0) {
              const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vrow + d));
              acc[i][0] = fmaf(pj, v.x, acc[i][0]);
              acc[i][1] = fmaf(pj, v.y, acc[i][1]);
              continue;
            }
          }
          acc[i][0] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i][0]);
          acc[i][1] = fmaf(pj, to_float<TKV>(vrow[d + 1]), acc[i][1]);
        } else if (d < rank) {
          acc[i][0] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i][0]);
        }
      }
    }
  }
  // join the four warps' partial results in warp order
  if (lane == 0) {
    part_ml[2 * warp] = m;
    part_ml[2 * warp + 1] = l;
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = 2 * lane + 64 * i;
    if (d < rank) part_o[(size_t)warp * rank + d] = acc[i][0];
    if (d + 1 < rank) part_o[(size_t)warp * rank + d + 1] = acc[i][1];
  }
  __syncthreads();
  float m_all = -FLT_MAX;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, part_ml[2 * w]);
  float f[WARPS], l_all = 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    f[w] = part_ml[2 * w + 1] > 0.f ? expf(part_ml[2 * w] - m_all) : 0.f;
    l_all += part_ml[2 * w + 1] * f[w];
  }
  const float wgt = (gate ? gate[(size_t)t * heads + h] : 1.f) / l_all;
  TO* orow = out + ((size_t)t * heads + h) * rank;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += part_o[(size_t)w * rank + d] * f[w];
    orow[d] = from_float<TO>(v * wgt);
  }
}

}  // namespace

PSB_API int psb_latent_prepare(const void* proj, int dtype, const void* positions, const void* token_item, const void* table,
                               int table_width, const void* cos_t, const void* sin_t, const void* gain_q,
                               const void* gain_kv, void* cq_out, void* gate_out, void* cache, int cache_dtype, int T,
                               int q_rank, int rank, int rot, int rot_dims, int heads, int page_size, int num_pages,
                               int max_positions, float eps, cudaStream_t stream) {
  if (T < 0 || q_rank < 1 || rank < 1 || rot < 0 || heads < 0) PSB_REFUSE("latent_prepare: bad sizes T=%d q_rank=%d rank=%d rot=%d heads=%d", T, q_rank, rank, rot, heads);
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) PSB_REFUSE("latent_prepare: %d rotated dimensions must be even and within the rotated part of %d", rot_dims, rot);
  if (rot_dims > 0 && (!cos_t || !sin_t || max_positions < 1)) PSB_REFUSE("latent_prepare: angle tables missing");
  if (page_size < 1 || num_pages < 1 || table_width < 1) PSB_REFUSE("latent_prepare: bad paging (page_size=%d pages=%d width=%d)", page_size, num_pages, table_width);
  if (!(eps > 0.f)) PSB_REFUSE("latent_prepare: eps must be positive");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(cache_dtype, TKV, {
      psb_launch(latent_prepare_kernel<T_, TKV>, dim3(T), dim3(128), 0, stream, (const T_*)proj, (const int32_t*)positions,
                 (const int32_t*)token_item, (const int32_t*)table, table_width, (const float*)cos_t, (const float*)sin_t,
                 (const float*)gain_q, (const float*)gain_kv, (T_*)cq_out, (float*)gate_out, (TKV*)cache, q_rank, rank, rot,
                 rot_dims, heads, page_size, num_pages, max_positions, eps);
    });
  });
  PSB_LAUNCH_CHECK("latent_prepare");
  return 0;
}

PSB_API int psb_latent_query_rotate(const void* q, int dtype, const void* positions, const void* cos_t, const void* sin_t,
                                    void* q_lat, int T, int heads, int plain, int rot, int rot_dims, int rank,
                                    int max_positions, cudaStream_t stream) {
  if (T < 0 || heads < 1 || plain < 1 || rot < 0 || rank < 1) PSB_REFUSE("latent_query_rotate: bad sizes");
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2) PSB_REFUSE("latent_query_rotate: %d rotated dimensions must be even and within %d", rot_dims, rot);
  if (rot_dims > 0 && (!cos_t || !sin_t || max_positions < 1)) PSB_REFUSE("latent_query_rotate: angle tables missing");
  if (T == 0 || rot == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    psb_launch(latent_query_rotate_kernel<T_>, dim3(T), dim3(128), 0, stream, (const T_*)q, (const int32_t*)positions,
               (const float*)cos_t, (const float*)sin_t, (float*)q_lat, heads, plain, rot, rot_dims, rank, max_positions);
  });
  PSB_LAUNCH_CHECK("latent_query_rotate");
  return 0;
}

PSB_API int psb_latent_attention_max_rank() { return 1024; }

PSB_API int psb_latent_attention(const void* q_lat, const void* cache, int cache_dtype, const void* table, int table_width,
                                 const void* positions, const void* token_item, const void* gate, void* out, int out_dtype,
                                 int T, int heads, int rank, int rot, int page_size, int num_pages, int window, float scale,
                                 cudaStream_t stream) {
  if (T < 0 || heads < 1 || rank < 1 || rot < 0) PSB_REFUSE("latent_attention: bad sizes T=%d heads=%d rank=%d rot=%d", T, heads, rank, rot);
  if (rank > 1024 || rank + rot > 2048) PSB_REFUSE("latent_attention: a latent of %d (+%d rotated) is beyond this kernel (1024, 2048 together)", rank, rot);
  if (page_size < 1 || num_pages < 1 || table_width < 1) PSB_REFUSE("latent_attention: bad paging (page_size=%d pages=%d width=%d)", page_size, num_pages, table_width);
  if (window < 0) PSB_REFUSE("latent_attention: negative window");
  if (T == 0) return 0;
  const long long blocks = (long long)T * heads;
  if (blocks > 0x7fffffffLL) PSB_REFUSE("latent_attention: batch too large");
  if ((uintptr_t)cache & 15) PSB_REFUSE("latent_attention: the cache entry must be 16-byte aligned");
  const size_t smem = ((size_t)((rank + rot + 3) & ~3) + 2 * WARPS + (size_t)WARPS * rank) * sizeof(float);
#define LATENT_LAUNCH(NACC)                                                                                              \
  PSB_DISPATCH_DTYPE(cache_dtype, TKV, {                                                                                 \
    PSB_DISPATCH_DTYPE(out_dtype, TO, {                                                                                  \
      psb_launch(latent_attention_kernel<TKV, TO, NACC>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, stream,        \
                 (const float*)q_lat, (const TKV*)cache, (const int32_t*)table, table_width, (const int32_t*)positions,  \
                 (const int32_t*)token_item, (const float*)gate, (TO*)out, T, heads, rank, rot, page_size, num_pages,    \
                 window, scale);                                                                                         \
    });                                                                                                                  \
  })
  if (rank <= 128) { LATENT_LAUNCH(2); }        // NACC pairs of columns a lane: 64 columns each
  else if (rank <= 256) { LATENT_LAUNCH(4); }
  else if (rank <= 512) { LATENT_LAUNCH(8); }
  else { LATENT_LAUNCH(16); }
#undef LATENT_LAUNCH
  PSB_LAUNCH_CHECK("latent_attention");
  return 0;
}
