// Token embedding with a hashed pair embedding added: a token's row of the table plus the row
//   (previous token * mul_prev + token * mul_cur) mod buckets
// of a second table; a sequence's first token (position 0) takes that table's last row, number ``buckets``.  The sum
// is made in float32 and is the start of the residual stream; a copy in the compute type may be written beside it for
// the first sublayer's products.
//
// The previous token of a portion's first token is not in the step: it is kept per request slot (``last_token``
// [num_slots] int32), read here and brought up to date by note_last_token_kernel, a launch of its own so that no
// block of this kernel can still be reading the word it writes.
#include "common.cuh"

namespace {

template <typename TT, typename TX>
__global__ void hashed_embedding_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                                        const int32_t* __restrict__ token_item, const int32_t* __restrict__ item_start,
                                        const int32_t* __restrict__ slots, const int32_t* __restrict__ last_token,
                                        const TT* __restrict__ table, const TT* __restrict__ pair_table,
                                        float* __restrict__ out, TX* __restrict__ copy, int H, int V, int buckets,
                                        long long mul_prev, long long mul_cur, int num_slots) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);  // ids are validated on the host; never read outside the table
  long long bucket = buckets;
  if (positions[t] > 0) {
    const int item = token_item[t];
    long long prev;
    if (t == item_start[item]) {
      int slot = slots[item];
      slot = slot < 0 ? 0 : (slot >= num_slots ? num_slots - 1 : slot);
      prev = last_token[slot];
    } else {
      prev = ids[t - 1];
    }
    bucket = (prev * mul_prev + (long long)id * mul_cur) % buckets;
    if (bucket < 0) bucket += buckets;
  }
  const TT* row = table + (size_t)id * H;
  const TT* pair = pair_table + (size_t)bucket * H;
  float* o = out + (size_t)t * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = to_float<TT>(row[j]) + to_float<TT>(pair[j]);
    o[j] = v;
    if (copy) copy[(size_t)t * H + j] = from_float<TX>(v);
  }
}

__global__ void note_last_token_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ item_start,
                                       const int32_t* __restrict__ slots, int32_t* __restrict__ last_token, int items,
                                       int num_slots) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= items) return;
  const int slot = slots[i];
  if (slot < 0 || slot >= num_slots) return;
  last_token[slot] = ids[item_start[i + 1] - 1];
}

}  // namespace

PSB_API int psb_hashed_embedding(const void* ids, const void* positions, const void* token_item, const void* item_start,
                                 const void* slots, void* last_token, const void* table, const void* pair_table,
                                 int table_dtype, void* out, void* copy, int copy_dtype, int T, int items, int H, int V,
                                 int buckets, long long mul_prev, long long mul_cur, int num_slots, cudaStream_t stream) {
  if (T < 0 || items < 0 || H < 1 || V < 1 || buckets < 1 || num_slots < 1) PSB_REFUSE("hashed_embedding: bad sizes T=%d items=%d H=%d V=%d buckets=%d", T, items, H, V, buckets);
  if (T == 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  PSB_DISPATCH_DTYPE(table_dtype, TT, {
    PSB_DISPATCH_DTYPE(copy_dtype, TX, {
      psb_launch(hashed_embedding_kernel<TT, TX>, dim3(T), dim3(threads), 0, stream, (const int32_t*)ids,
                 (const int32_t*)positions, (const int32_t*)token_item, (const int32_t*)item_start, (const int32_t*)slots,
                 (const int32_t*)last_token, (const TT*)table, (const TT*)pair_table, (float*)out, (TX*)copy, H, V, buckets,
                 mul_prev, mul_cur, num_slots);
    });
  });
  PSB_LAUNCH_CHECK("hashed_embedding");
  psb_launch(note_last_token_kernel, dim3((items + 127) / 128), dim3(128), 0, stream, (const int32_t*)ids,
             (const int32_t*)item_start, (const int32_t*)slots, (int32_t*)last_token, items, num_slots);
  PSB_LAUNCH_CHECK("note_last_token");
  return 0;
}
