// Causal grouped-query attention over the paged cache for designs whose scores carry more than q.k:
//
//   score(i, j) = (q_i . k_j) * scale + bias[h][min(i - j, reach - 1)]       (bias optional)
//   visible:  j <= i,  j > i - window (window optional),  floor(j / chunk) == floor(i / chunk) (chunk optional)
//   weights = exp(score) / (sum over visible j of exp(score) + exp(sink[h]))  (sink optional: a term of the
//             denominator that has no key and no value)
//
// Keys and values may have different sizes (dim, vdim); the cache entry holds one row per token and key/value head,
// [num_pages, 1, hkv, page_size, dim + vdim]: the key, then the value.  ``bias`` is a float32 table
// [heads, reach] by distance (whatever maps distances to learned rows has been applied when the table was built;
// distances of reach - 1 and more share the last column).  Positions are absolute, so the chunk grid is counted
// from the start of the sequence however the prompt was cut.
//
// attention_biased_append_kernel splits a fused projection row [q | k | v] into the query tensor and the cache row.
// attention_biased_kernel: a warp per (token, query head) walks the visible keys in runs of 32 aligned to absolute
// positions, a lane per key for the scores, online softmax started from the sink (maximum = sink, sum = 1), the
// output accumulated in registers.  Scores, weights and sums are float32 and the weights are not rounded before
// they multiply the values.  Float32 and bfloat16 storage.
//
// attention_biased_tile_kernel (bfloat16 storage): a block takes 16 consecutive tokens of one request and one
// key/value head, with all the query heads that share it; key/value rows are staged in shared memory once for the
// block, a warp takes (token, head) pairs in turn.  Same arithmetic and order of sums as the kernel above, so both
// give the same numbers for a token.
#include <cfloat>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T, typename TKV>
__global__ void attention_biased_append_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ token_item, const int32_t* __restrict__ table,
                                               int table_width, TKV* __restrict__ kv, T* __restrict__ q_out, int hq, int hkv,
                                               int dim, int vdim, int page_size, int num_pages) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int qw = hq * dim, kw = hkv * dim, vw = hkv * vdim;
  const T* row = qkv + (size_t)t * (qw + kw + vw);
  for (int c = threadIdx.x; c < qw; c += blockDim.x) q_out[(size_t)t * qw + c] = row[c];
  const int p = positions[t];
  int page = table[(size_t)token_item[t] * table_width + p / page_size];
  if (page < 0 || page >= num_pages) return;  // tables are checked on the host; never write outside the pool
  const int rw = dim + vdim;
  TKV* dst = kv + ((size_t)page * hkv * page_size + (size_t)(p % page_size)) * rw;
  for (int c = threadIdx.x; c < kw + vw; c += blockDim.x) {
    int g, e;
    if (c < kw) { g = c / dim; e = c - g * dim; }
    else { g = (c - kw) / vdim; e = dim + (c - kw) - g * vdim; }
    dst[(size_t)g * page_size * rw + e] = from_float<TKV>(to_float<T>(row[qw + c]));
  }
}

template <typename T, typename TKV>
__global__ void __launch_bounds__(WARPS * 32)
attention_biased_kernel(const T* __restrict__ q, const TKV* __restrict__ kv, const int32_t* __restrict__ table,
                        int table_width, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_item,
                        const float* __restrict__ bias, const float* __restrict__ sink, T* __restrict__ out, int T_tokens,
                        int hq, int hkv, int dim, int vdim, int page_size, int window, int chunk, int reach, float scale,
                        const int32_t* __restrict__ item_start, int skip_from) {
  __shared__ float qs[WARPS][MAX_D];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * WARPS + warp;
  if (unit >= (long long)T_tokens * hq) return;
  const int t = (int)(unit / hq), h = (int)(unit - (long long)t * hq);
  const int g = h / (hq / hkv);
  const int p = positions[t];
  const int item = token_item[t];
  if (skip_from > 0 && item_start[item + 1] - item_start[item] >= skip_from) return;  // the tiled kernel's token
  const int32_t* pages = table + (size_t)item * table_width;
  const T* qrow = q + ((size_t)t * hq + h) * dim;
  for (int d = lane; d < dim; d += 32) qs[warp][d] = to_float<T>(qrow[d]);
  __syncwarp();

  int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
  const int rw = dim + vdim;
  const size_t head_stride = (size_t)page_size * rw;
  const size_t page_elems = (size_t)hkv * head_stride;
  const float* brow = bias ? bias + (size_t)h * reach : nullptr;

  float m = -FLT_MAX, l = 0.f;
  if (sink) { m = sink[h]; l = 1.f; }
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int base = lo & ~31; base <= p; base += 32) {
    const int key = base + lane;
    const bool live = key >= lo && key <= p;
    long long off = -1;
    float s = -FLT_MAX;
    if (live) {
      const int page = pages[key / page_size];
      off = (long long)((size_t)page * page_elems + (size_t)g * head_stride + (size_t)(key % page_size) * rw);
      const TKV* krow = kv + off;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qs[warp][d], to_float<TKV>(krow[d]), dot);
      s = dot * scale;
      if (brow) s += brow[min(p - key, reach - 1)];
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);
    const float pr = live ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    const int n_live = min(32, p - base + 1);
    for (int j = 0; j < n_live; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pr, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (oj < 0) continue;
      const TKV* vrow = kv + oj + dim;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) acc[i] = fmaf(pj, to_float<TKV>(vrow[d]), acc[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = out + ((size_t)t * hq + h) * vdim;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// Prompt portions in bfloat16: a block = up to TILE_T consecutive tokens of one item x one key/value head.  The keys a
// tile can see lie in [lo of its first token, position of its last]; they are brought into shared memory 32 at a time
// (the same absolute runs of 32 the kernel above walks), transposed so that a lane's key is a column, and every
// (token, query head) pair of the tile, one warp each in turn, works on the staged run.
constexpr int TILE_T = 16;
constexpr int TILE_WARPS = 8;

template <int DP, int VP>  // key and value sizes rounded up to 32, 64, 128 or 256
__global__ void __launch_bounds__(TILE_WARPS * 32)
attention_biased_tile_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kv,
                             const int32_t* __restrict__ table, int table_width, const int32_t* __restrict__ positions,
                             const int32_t* __restrict__ item_start, int items, int min_tokens, const float* __restrict__ bias,
                             const float* __restrict__ sink, __nv_bfloat16* __restrict__ out, int hq, int hkv, int dim, int vdim,
                             int page_size, int window, int chunk, int reach, float scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  // tiles are numbered through the portions of at least ``min_tokens`` tokens, in order
  int item = -1, t0 = 0;
  for (int i = 0, left = blockIdx.x; i < items; ++i) {
    const int a = item_start[i], n = item_start[i + 1] - a;
    if (n < min_tokens) continue;
    const int tiles = (n + TILE_T - 1) / TILE_T;
    if (left < tiles) { item = i; t0 = a + left * TILE_T; break; }
    left -= tiles;
  }
  if (item < 0) return;
  const int g = blockIdx.y, share = hq / hkv;
  const int nt = min(TILE_T, item_start[item + 1] - t0);
  const int pairs = nt * share;  // (token, head of the group) units of this block
  float* ks = smem;                               // [DP][33] one run of keys, transposed
  float* vs = ks + DP * 33;                       // [32][VP]
  float* qs = vs + 32 * VP;                       // [TILE_T * share][DP]
  float* st = qs + (size_t)TILE_T * share * DP;   // per unit: m, l
  float* accs = st + 2 * TILE_T * share;          // [TILE_T * share][VP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rw = dim + vdim;
  const size_t head_stride = (size_t)page_size * rw;
  const size_t page_elems = (size_t)hkv * head_stride;
  const int32_t* pages = table + (size_t)item * table_width;
  const int p_first = positions[t0], p_last = p_first + nt - 1;
  for (int i = threadIdx.x; i < pairs * DP; i += blockDim.x) {
    const int u = i / DP, d = i - u * DP;
    const int tt = u / share, hh = g * share + (u - tt * share);
    qs[i] = d < dim ? __bfloat162float(q[((size_t)(t0 + tt) * hq + hh) * dim + d]) : 0.f;
  }
  for (int i = threadIdx.x; i < pairs * VP; i += blockDim.x) accs[i] = 0.f;
  for (int u = threadIdx.x; u < pairs; u += blockDim.x) {
    const int hh = g * share + u % share;
    st[2 * u] = sink ? sink[hh] : -FLT_MAX;
    st[2 * u + 1] = sink ? 1.f : 0.f;
  }
  int lo_tile = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  if (chunk > 0) lo_tile = max(lo_tile, (p_first / chunk) * chunk);
  for (int base = lo_tile & ~31; base <= p_last; base += 32) {
    __syncthreads();
    // stage the run: keys transposed, values as rows; a key beyond the tile's last position is left as zeros
    for (int i = threadIdx.x; i < 32 * (DP + VP) / 2; i += blockDim.x) {
      const int j = i / ((DP + VP) / 2), e = 2 * (i - j * ((DP + VP) / 2));
      const int key = base + j;
      float a = 0.f, b = 0.f;
      const bool is_key = e < DP;
      const int col = is_key ? e : e - DP;
      const int width = is_key ? dim : vdim;
      if (key >= lo_tile && key <= p_last && col < width) {
        const int page = pages[key / page_size];
        const __nv_bfloat16* src = kv + (size_t)page * page_elems + (size_t)g * head_stride + (size_t)(key % page_size) * rw +
                                   (is_key ? 0 : dim) + col;
        a = __bfloat162float(src[0]);
        if (col + 1 < width) b = __bfloat162float(src[1]);
      }
      if (is_key) { ks[col * 33 + j] = a; ks[(col + 1) * 33 + j] = b; }
      else { vs[j * VP + col] = a; vs[j * VP + col + 1] = b; }
    }
    __syncthreads();
    for (int u = warp; u < pairs; u += TILE_WARPS) {
      const int tt = u / share, hh = g * share + (u - tt * share);
      const int p = p_first + tt;
      if (base > p) continue;
      int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
      if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
      if (base + 31 < lo) continue;
      const int key = base + lane;
      const bool live = key >= lo && key <= p;
      float s = -FLT_MAX;
      if (live) {
        const float* qq = qs + (size_t)u * DP;
        float dot = 0.f;
        for (int d = 0; d < dim; ++d) dot = fmaf(qq[d], ks[d * 33 + lane], dot);
        s = dot * scale;
        if (bias) s += bias[(size_t)hh * reach + min(p - key, reach - 1)];
      }
      float m = st[2 * u], l = st[2 * u + 1];
      const float m_new = fmaxf(m, warp_max(s));
      const float alpha = expf(m - m_new);
      const float pr = live ? expf(s - m_new) : 0.f;
      l = l * alpha + warp_sum(pr);
      __syncwarp();
      if (lane == 0) { st[2 * u] = m_new; st[2 * u + 1] = l; }
      float* acc = accs + (size_t)u * VP;
      float a[VP / 32];
#pragma unroll
      for (int i = 0; i < VP / 32; ++i) a[i] = acc[lane + 32 * i] * alpha;
      const int n_live = min(32, p - base + 1);
      const int j0 = max(0, lo - base);
      for (int j = j0; j < n_live; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
        for (int i = 0; i < VP / 32; ++i) a[i] = fmaf(pj, vs[j * VP + lane + 32 * i], a[i]);
      }
#pragma unroll
      for (int i = 0; i < VP / 32; ++i) acc[lane + 32 * i] = a[i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs * VP; i += blockDim.x) {
    const int u = i / VP, d = i - u * VP;
    if (d >= vdim) continue;
    const int tt = u / share, hh = g * share + (u - tt * share);
    out[((size_t)(t0 + tt) * hq + hh) * vdim + d] = __float2bfloat16_rn(accs[i] / st[2 * u + 1]);
  }
}

size_t tile_smem(int dp, int vp, int share) {
  return sizeof(float) * ((size_t)dp * 33 + 32 * (size_t)vp + (size_t)TILE_T * share * dp + 2 * (size_t)TILE_T * share +
                          (size_t)TILE_T * share * vp);
}

PsbPerDevice tile_attr[4][4];

int padded(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : 256; }
int slot_of(int n) { return n == 32 ? 0 : n == 64 ? 1 : n == 128 ? 2 : 3; }

}  // namespace

// (qkv, dtype, positions, token_item, table, table_width, kv, kv_dtype, q_out, T, hq, hkv, dim, vdim, page_size, num_pages, stream)
PSB_API int psb_attention_biased_append(const void* qkv, int dtype, const void* positions, const void* token_item,
                                        const void* table, int table_width, void* kv, int kv_dtype, void* q_out, int T, int hq,
                                        int hkv, int dim, int vdim, int page_size, int num_pages, cudaStream_t stream) {
  if (T < 0 || hq < 1 || hkv < 1 || dim < 1 || vdim < 1 || page_size < 1 || table_width < 1 || num_pages < 1)
    PSB_REFUSE("attention_biased_append: bad sizes");
  if (T == 0) return 0;
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_biased_append_kernel<T_, TKV>, dim3(T), dim3(128), 0, stream, (const T_*)qkv, (const int32_t*)positions,
                 (const int32_t*)token_item, (const int32_t*)table, table_width, (TKV*)kv, (T_*)q_out, hq, hkv, dim, vdim,
                 page_size, num_pages);
    });
  });
  PSB_LAUNCH_CHECK("attention_biased_append");
  return 0;
}

// ``skip_from`` > 0: tokens of portions with at least that many tokens are left to the tiled kernel (item_start needed).
// (q, dtype, kv, kv_dtype, table, table_width, positions, token_item, bias, sink, out, T, hq, hkv, dim, vdim, page_size,
//  window, chunk, reach, scale, item_start, skip_from, stream)
PSB_API int psb_attention_biased(const void* q, int dtype, const void* kv, int kv_dtype, const void* table, int table_width,
                                 const void* positions, const void* token_item, const void* bias, const void* sink, void* out,
                                 int T, int hq, int hkv, int dim, int vdim, int page_size, int window, int chunk, int reach,
                                 float scale, const void* item_start, int skip_from, cudaStream_t stream) {
  if (skip_from > 0 && !item_start) PSB_REFUSE("attention_biased: skipping tiled portions needs the item offsets");
  if (T < 0 || hq < 1 || hkv < 1 || hq % hkv) PSB_REFUSE("attention_biased: %d query heads cannot share %d key/value heads", hq, hkv);
  if (dim < 1 || dim > MAX_D || vdim < 1 || vdim > MAX_D) PSB_REFUSE("attention_biased: sizes %d/%d are outside [1, %d]", dim, vdim, MAX_D);
  if (page_size < 1 || table_width < 1) PSB_REFUSE("attention_biased: bad paging (page_size=%d width=%d)", page_size, table_width);
  if (window < 0 || chunk < 0 || (bias && reach < 1)) PSB_REFUSE("attention_biased: negative window or chunk, or an empty bias table");
  if (T == 0) return 0;
  const long long units = (long long)T * hq;
  const long long blocks = (units + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) PSB_REFUSE("attention_biased: batch too large");
  PSB_DISPATCH_DTYPE(dtype, T_, {
    PSB_DISPATCH_DTYPE(kv_dtype, TKV, {
      psb_launch(attention_biased_kernel<T_, TKV>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, (const T_*)q,
                 (const TKV*)kv, (const int32_t*)table, table_width, (const int32_t*)positions, (const int32_t*)token_item,
                 (const float*)bias, (const float*)sink, (T_*)out, T, hq, hkv, dim, vdim, page_size, window, chunk, reach, scale,
                 (const int32_t*)item_start, skip_from);
    });
  });
  PSB_LAUNCH_CHECK("attention_biased");
  return 0;
}

// () -> tokens a tile of the tiled kernel holds
PSB_API int psb_attention_biased_tile_tokens() { return TILE_T; }

// (hq, hkv, dim, vdim) -> 1 if the tiled kernel takes the shape
PSB_API int psb_attention_biased_tile_supported(int hq, int hkv, int dim, int vdim) {
  if (hq < 1 || hkv < 1 || hq % hkv || dim < 1 || dim > MAX_D || vdim < 1 || vdim > MAX_D) return 0;
  const int dp = padded(dim), vp = padded(vdim);
  return tile_smem(dp, vp, hq / hkv) <= 200 * 1024 ? 1 : 0;
}

// The tiled kernel over every portion of at least ``min_tokens`` tokens (the grid is sized by an upper bound on their
// tiles, so its shape depends on T and the number of items only).  Other tokens are left untouched.
// (q, kv, table, table_width, positions, item_start, items, T, min_tokens, bias, sink, out, hq, hkv, dim, vdim,
//  page_size, window, chunk, reach, scale, stream)
PSB_API int psb_attention_biased_tiles(const void* q, const void* kv, const void* table, int table_width, const void* positions,
                                       const void* item_start, int items, int T, int min_tokens,
                                       const void* bias, const void* sink, void* out, int hq, int hkv, int dim, int vdim,
                                       int page_size, int window, int chunk, int reach, float scale, cudaStream_t stream) {
  if (items < 1 || T < 1 || min_tokens < 1) return 0;
  const int tiles = (T + TILE_T - 1) / TILE_T + items;
  if (!psb_attention_biased_tile_supported(hq, hkv, dim, vdim)) PSB_REFUSE("attention_biased_tiles: shape not taken");
  if (page_size < 1 || table_width < 1 || window < 0 || chunk < 0 || (bias && reach < 1)) PSB_REFUSE("attention_biased_tiles: bad arguments");
  if (hkv > 65535) PSB_REFUSE("attention_biased_tiles: too many key/value heads");
  const int dp = padded(dim), vp = padded(vdim);
  const size_t smem = tile_smem(dp, vp, hq / hkv);
  const dim3 grid(tiles, hkv), block(TILE_WARPS * 32);
#define TILE_CASE(DP_, VP_)                                                                                                    \
  if (dp == DP_ && vp == VP_) {                                                                                                \
    auto kernel = attention_biased_tile_kernel<DP_, VP_>;                                                                      \
    PsbPerDevice& done = tile_attr[slot_of(DP_)][slot_of(VP_)];                                                                \
    if (!done.get()) {                                                                                                         \
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)                \
        PSB_REFUSE("attention_biased_tiles: cannot raise the shared-memory limit");                                            \
      done.set();                                                                                                              \
    }                                                                                                                          \
    psb_launch(kernel, grid, block, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv, (const int32_t*)table,    \
               table_width, (const int32_t*)positions, (const int32_t*)item_start, items, min_tokens,                          \
               (const float*)bias, (const float*)sink, (__nv_bfloat16*)out, hq, hkv, dim, vdim,                                \
               page_size, window, chunk, reach, scale);                                                                        \
    launched = true;                                                                                                           \
  }
#define TILE_ROW(DP_) TILE_CASE(DP_, 32) TILE_CASE(DP_, 64) TILE_CASE(DP_, 128) TILE_CASE(DP_, 256)
  bool launched = false;
  TILE_ROW(32) TILE_ROW(64) TILE_ROW(128) TILE_ROW(256)
#undef TILE_ROW
#undef TILE_CASE
  if (!launched) PSB_REFUSE("attention_biased_tiles: sizes %d/%d not instantiated", dim, vdim);
  PSB_LAUNCH_CHECK("attention_biased_tiles");
  return 0;
}
