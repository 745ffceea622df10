// Paged-cache data movement: K/V scatter, affix relocation with fused RoPE
// re-rotation, and RoPE + scatter for the rows of a forward.  All three are
// HBM-bound byte movers: 16-byte accesses, every K/V byte crosses HBM once.
#include "common.cuh"

namespace acache {

// ------------------------------------------------------------------------------------
// store_kvcache: one item = one 16-byte chunk of one token row (K and V).
template <int VEC>
__global__ void __launch_bounds__(256) store_kvcache_kernel(
    const char* __restrict__ key, int64_t key_stride_b, const char* __restrict__ val, int64_t val_stride_b,
    char* __restrict__ k_cache, char* __restrict__ v_cache, const int32_t* __restrict__ slots, int n_tokens,
    int row_bytes, int64_t num_slots, int32_t* err_flag) {
  const int chunks = row_bytes / VEC;
  const int64_t total = (int64_t)n_tokens * chunks;
  for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < total; it += (int64_t)gridDim.x * blockDim.x) {
    const int tok = (int)(it / chunks);
    const int c = (int)(it - (int64_t)tok * chunks);
    const int slot = slots[tok];
    if (slot == -1) continue;
    if (slot < 0 || slot >= num_slots) {
      if (err_flag) atomicExch(err_flag, 1);
      continue;
    }
    const int64_t dst = (int64_t)slot * row_bytes + (int64_t)c * VEC;
    if (VEC == 16) {
      uint4 a = ld_global_nc(key + tok * key_stride_b + (int64_t)c * 16);
      uint4 b = ld_global_nc(val + tok * val_stride_b + (int64_t)c * 16);
      *reinterpret_cast<uint4*>(k_cache + dst) = a;
      *reinterpret_cast<uint4*>(v_cache + dst) = b;
    } else {  // 2- or 4-byte elements, unaligned rows
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        k_cache[dst + j] = key[tok * key_stride_b + (int64_t)c * VEC + j];
        v_cache[dst + j] = val[tok * val_stride_b + (int64_t)c * VEC + j];
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// Affix relocation.  One item = the pair of 16-byte chunks (d, d + D/2) of one
// (layer, token, kv head) of K plus the same two chunks of V.  The source is read once
// into registers and written once per request with that request's rotation.
template <typename T, typename TR, typename TC>
__global__ void __launch_bounds__(256) relocate_affix_kernel(
    T* __restrict__ k_cache, T* __restrict__ v_cache, int64_t layer_stride, int n_layers, int64_t num_slots,
    int n_kv_heads, int head_dim, const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin,
    int64_t rope_row_stride, int rope_rows, int affix_len, int n_requests, const int32_t* __restrict__ shifts,
    const int32_t* __restrict__ dst_slots, const int32_t* __restrict__ dst_tables, int table_stride, int block_size,
    int32_t* err_flag) {
  constexpr int E = 16 / sizeof(T);
  const int half = head_dim / 2;
  const int cph = half / E;  // chunk pairs per head vector
  const int row = n_kv_heads * head_dim;
  const int64_t per_layer = (int64_t)affix_len * n_kv_heads * cph;
  const int64_t total = per_layer * n_layers;
  for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < total; it += (int64_t)gridDim.x * blockDim.x) {
    const int layer = (int)(it / per_layer);
    int64_t rem = it - (int64_t)layer * per_layer;
    const int tok = (int)(rem / (n_kv_heads * cph));
    const int hc = (int)(rem - (int64_t)tok * (n_kv_heads * cph));
    const int head = hc / cph;
    const int d = (hc - head * cph) * E;
    const int64_t in_row = (int64_t)head * head_dim + d;
    const int64_t src = (int64_t)layer * layer_stride + (int64_t)tok * row + in_row;

    Vec16<T> k1, k2, v1, v2;
    k1.u = ld_global_nc(k_cache + src);
    k2.u = ld_global_nc(k_cache + src + half);
    v1.u = ld_global_nc(v_cache + src);
    v2.u = ld_global_nc(v_cache + src + half);
    float x1[E], x2[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      x1[j] = to_f32<T>(k1.e[j]);
      x2[j] = to_f32<T>(k2.e[j]);
    }

    for (int r = 0; r < n_requests; ++r) {
      const int shift = shifts[r];
      int64_t dslot;
      if (dst_tables != nullptr) {
        const int blk = dst_tables[(int64_t)r * table_stride + tok / block_size];
        dslot = (int64_t)blk * block_size + tok % block_size;
        if (blk < 0) dslot = -1;
      } else {
        dslot = (int64_t)dst_slots[r] + tok;
      }
      if (dslot < affix_len || dslot >= num_slots || shift < 0 || shift >= rope_rows) {
        if (err_flag) atomicExch(err_flag, 1);
        continue;
      }
      const TR* cr = rope_cos + (int64_t)shift * rope_row_stride;
      const TR* sr = rope_sin + (int64_t)shift * rope_row_stride;
      Vec16<T> o1, o2;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float c1 = to_f32<TR>(cr[d + j]), s1 = to_f32<TR>(sr[d + j]);
        const float c2 = to_f32<TR>(cr[d + half + j]), s2 = to_f32<TR>(sr[d + half + j]);
        o1.e[j] = from_f32<T>(rot_lo<TC>(x1[j], x2[j], c1, s1));
        o2.e[j] = from_f32<T>(rot_hi<TC>(x1[j], x2[j], c2, s2));
      }
      const int64_t dst = (int64_t)layer * layer_stride + dslot * row + in_row;
      st_global_cs(k_cache + dst, o1.u);
      st_global_cs(k_cache + dst + half, o2.u);
      st_global_cs(v_cache + dst, v1.u);
      st_global_cs(v_cache + dst + half, v2.u);
    }
  }
}

// ------------------------------------------------------------------------------------
// RoPE of q and k rows in place + scatter of the rotated k and of v into the cache.
template <typename T, typename TR, typename TC>
__global__ void __launch_bounds__(256) rope_store_kernel(
    T* __restrict__ q, int64_t q_stride, T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
    int n_tokens, int n_heads, int n_kv_heads, int head_dim, const int64_t* __restrict__ positions,
    const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin, int64_t rope_row_stride, int rope_rows,
    T* __restrict__ k_cache, T* __restrict__ v_cache, const int32_t* __restrict__ slots, int64_t num_slots,
    int32_t* err_flag) {
  constexpr int E = 16 / sizeof(T);
  const int half = head_dim / 2;
  const int cph = half / E;
  const int heads_all = n_heads + n_kv_heads;
  const int per_tok = heads_all * cph + n_kv_heads * cph;  // rotation items + v-copy items (pairs)
  const int kv_row = n_kv_heads * head_dim;
  const int64_t total = (int64_t)n_tokens * per_tok;
  for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < total; it += (int64_t)gridDim.x * blockDim.x) {
    const int tok = (int)(it / per_tok);
    int w = (int)(it - (int64_t)tok * per_tok);
    int slot = -1;
    if (slots != nullptr) {
      slot = slots[tok];
      if (slot != -1 && (slot < 0 || slot >= num_slots)) {
        if (err_flag) atomicExch(err_flag, 1);
        slot = -1;
      }
    }
    if (w >= heads_all * cph) {  // V copy
      if (slot < 0) continue;
      w -= heads_all * cph;
      const int head = w / cph;
      const int d = (w - head * cph) * E;
      const int64_t off = (int64_t)head * head_dim + d;
      uint4 a = ld_global_nc(v + tok * v_stride + off);
      uint4 b = ld_global_nc(v + tok * v_stride + off + half);
      *reinterpret_cast<uint4*>(v_cache + (int64_t)slot * kv_row + off) = a;
      *reinterpret_cast<uint4*>(v_cache + (int64_t)slot * kv_row + off + half) = b;
      continue;
    }
    const int head = w / cph;
    const int d = (w - head * cph) * E;
    const int64_t pos = positions[tok];
    if (pos < 0 || pos >= rope_rows) {
      if (err_flag) atomicExch(err_flag, 2);
      continue;
    }
    const bool is_k = head >= n_heads;
    T* base = is_k ? (k + tok * k_stride + (int64_t)(head - n_heads) * head_dim + d)
                   : (q + tok * q_stride + (int64_t)head * head_dim + d);
    Vec16<T> a, b, o1, o2;
    a.u = *reinterpret_cast<const uint4*>(base);
    b.u = *reinterpret_cast<const uint4*>(base + half);
    const TR* cr = rope_cos + pos * rope_row_stride;
    const TR* sr = rope_sin + pos * rope_row_stride;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const float x1 = to_f32<T>(a.e[j]), x2 = to_f32<T>(b.e[j]);
      o1.e[j] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + j]), to_f32<TR>(sr[d + j])));
      o2.e[j] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + half + j]), to_f32<TR>(sr[d + half + j])));
    }
    *reinterpret_cast<uint4*>(base) = o1.u;
    *reinterpret_cast<uint4*>(base + half) = o2.u;
    if (is_k && slot >= 0) {
      const int64_t off = (int64_t)slot * kv_row + (int64_t)(head - n_heads) * head_dim + d;
      *reinterpret_cast<uint4*>(k_cache + off) = o1.u;
      *reinterpret_cast<uint4*>(k_cache + off + half) = o2.u;
    }
  }
}

static inline int grid_for(int64_t items, int threads, int ctas_per_sm) {
  int64_t need = (items + threads - 1) / threads;
  int64_t cap = (int64_t)kNumSMs * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

// promote(T, TR): a 16-bit type only when both are the same 16-bit type
template <typename T, typename TR> struct Promote { using type = float; };
template <> struct Promote<__half, __half> { using type = __half; };
template <> struct Promote<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

}  // namespace acache

using namespace acache;

extern "C" int acache_store_kvcache(const void* key, int64_t key_stride, const void* value, int64_t value_stride,
                                    void* k_cache, void* v_cache, const int32_t* slot_mapping, int n_tokens,
                                    int row_elems, int64_t num_slots, int dtype, int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || n_tokens < 0 || row_elems <= 0 || num_slots <= 0) return ACACHE_EINVAL;
  if (n_tokens == 0) return ACACHE_OK;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping) return ACACHE_EINVAL;
  const int es = dtype_bytes(dtype);
  const int row_bytes = row_elems * es;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = row_bytes % 16 == 0 && (key_stride * es) % 16 == 0 && (value_stride * es) % 16 == 0 &&
                   aligned16(key) && aligned16(value) && aligned16(k_cache) && aligned16(v_cache);
  if (vec) {
    const int64_t items = (int64_t)n_tokens * (row_bytes / 16);
    store_kvcache_kernel<16><<<grid_for(items, 256, 8), 256, 0, st>>>(
        (const char*)key, key_stride * es, (const char*)value, value_stride * es, (char*)k_cache, (char*)v_cache,
        slot_mapping, n_tokens, row_bytes, num_slots, err_flag);
  } else if (es == 4) {
    const int64_t items = (int64_t)n_tokens * row_elems;
    store_kvcache_kernel<4><<<grid_for(items, 256, 8), 256, 0, st>>>(
        (const char*)key, key_stride * es, (const char*)value, value_stride * es, (char*)k_cache, (char*)v_cache,
        slot_mapping, n_tokens, row_bytes, num_slots, err_flag);
  } else {
    const int64_t items = (int64_t)n_tokens * row_elems;
    store_kvcache_kernel<2><<<grid_for(items, 256, 8), 256, 0, st>>>(
        (const char*)key, key_stride * es, (const char*)value, value_stride * es, (char*)k_cache, (char*)v_cache,
        slot_mapping, n_tokens, row_bytes, num_slots, err_flag);
  }
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR>
static int launch_relocate(void* k_cache, void* v_cache, int64_t layer_stride, int n_layers, int64_t num_slots,
                           int n_kv_heads, int head_dim, const void* rope_cos, const void* rope_sin,
                           int64_t rope_row_stride, int rope_rows, int affix_len, int n_requests,
                           const int32_t* shifts, const int32_t* dst_slots, const int32_t* dst_tables,
                           int table_stride, int block_size, int32_t* err_flag, cudaStream_t st) {
  using TC = typename Promote<T, TR>::type;
  constexpr int E = 16 / sizeof(T);
  const int64_t items = (int64_t)n_layers * affix_len * n_kv_heads * (head_dim / 2 / E);
  relocate_affix_kernel<T, TR, TC><<<grid_for(items, 256, 8), 256, 0, st>>>(
      (T*)k_cache, (T*)v_cache, layer_stride, n_layers, num_slots, n_kv_heads, head_dim, (const TR*)rope_cos,
      (const TR*)rope_sin, rope_row_stride, rope_rows, affix_len, n_requests, shifts, dst_slots, dst_tables,
      table_stride, block_size, err_flag);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_relocate_affix(void* k_cache, void* v_cache, int64_t layer_stride, int n_layers,
                                     int64_t num_slots, int n_kv_heads, int head_dim, int dtype,
                                     const void* rope_cos, const void* rope_sin, int64_t rope_row_stride,
                                     int rope_rows, int rope_dtype, int affix_len, int n_requests,
                                     const int32_t* shifts, const int32_t* dst_slots,
                                     const int32_t* dst_block_tables, int table_stride, int block_size,
                                     int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (n_layers <= 0 || n_kv_heads <= 0 || head_dim <= 0 || affix_len < 0 || n_requests < 0) return ACACHE_EINVAL;
  if (affix_len == 0 || n_requests == 0) return ACACHE_OK;
  if (!k_cache || !v_cache || !rope_cos || !rope_sin || !shifts) return ACACHE_EINVAL;
  if (dst_block_tables == nullptr && dst_slots == nullptr) return ACACHE_EINVAL;
  if (dst_block_tables != nullptr && (block_size <= 0 || table_stride <= 0)) return ACACHE_EINVAL;
  const int E = 16 / dtype_bytes(dtype);
  if (head_dim % (2 * E) != 0 || layer_stride % E != 0 || !aligned16(k_cache) || !aligned16(v_cache))
    return ACACHE_EUNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define RELOC(T, TR)                                                                                              \
  return launch_relocate<T, TR>(k_cache, v_cache, layer_stride, n_layers, num_slots, n_kv_heads, head_dim,        \
                                rope_cos, rope_sin, rope_row_stride, rope_rows, affix_len, n_requests, shifts,    \
                                dst_slots, dst_block_tables, table_stride, block_size, err_flag, st)
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (rope_dtype == ACACHE_F32) { RELOC(T, float); }
    if (rope_dtype == ACACHE_F16) { RELOC(T, __half); }
    RELOC(T, __nv_bfloat16);
  });
#undef RELOC
  return ACACHE_EINVAL;
}

template <typename T, typename TR>
static int launch_rope_store(void* q, int64_t q_stride, void* k, int64_t k_stride, const void* v, int64_t v_stride,
                             int n_tokens, int n_heads, int n_kv_heads, int head_dim, const int64_t* positions,
                             const void* rope_cos, const void* rope_sin, int64_t rope_row_stride, int rope_rows,
                             void* k_cache, void* v_cache, const int32_t* slots, int64_t num_slots,
                             int32_t* err_flag, cudaStream_t st) {
  using TC = typename Promote<T, TR>::type;
  constexpr int E = 16 / sizeof(T);
  const int cph = head_dim / 2 / E;
  const int64_t items = (int64_t)n_tokens * ((n_heads + 2 * n_kv_heads) * cph);
  rope_store_kernel<T, TR, TC><<<grid_for(items, 256, 8), 256, 0, st>>>(
      (T*)q, q_stride, (T*)k, k_stride, (const T*)v, v_stride, n_tokens, n_heads, n_kv_heads, head_dim, positions,
      (const TR*)rope_cos, (const TR*)rope_sin, rope_row_stride, rope_rows, (T*)k_cache, (T*)v_cache, slots,
      num_slots, err_flag);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_rope_store(void* q, int64_t q_stride, void* k, int64_t k_stride, const void* v,
                                 int64_t v_stride, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                 int dtype, const int64_t* positions, const void* rope_cos, const void* rope_sin,
                                 int64_t rope_row_stride, int rope_rows, int rope_dtype, void* k_cache,
                                 void* v_cache, const int32_t* slot_mapping, int64_t num_slots, int32_t* err_flag,
                                 void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) return ACACHE_EINVAL;
  if (n_tokens == 0) return ACACHE_OK;
  if (!q || !k || !positions || !rope_cos || !rope_sin) return ACACHE_EINVAL;
  if (slot_mapping != nullptr && (!k_cache || !v_cache || !v || num_slots <= 0)) return ACACHE_EINVAL;
  const int E = 16 / dtype_bytes(dtype);
  if (head_dim % (2 * E) != 0 || q_stride % E != 0 || k_stride % E != 0 || (v && v_stride % E != 0) ||
      !aligned16(q) || !aligned16(k) || (v && !aligned16(v)) || (k_cache && !aligned16(k_cache)) ||
      (v_cache && !aligned16(v_cache)))
    return ACACHE_EUNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define ROPE(T, TR)                                                                                              \
  return launch_rope_store<T, TR>(q, q_stride, k, k_stride, v, v_stride, n_tokens, n_heads, n_kv_heads, head_dim, \
                                  positions, rope_cos, rope_sin, rope_row_stride, rope_rows, k_cache, v_cache,   \
                                  slot_mapping, num_slots, err_flag, st)
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (rope_dtype == ACACHE_F32) { ROPE(T, float); }
    if (rope_dtype == ACACHE_F16) { ROPE(T, __half); }
    ROPE(T, __nv_bfloat16);
  });
#undef ROPE
  return ACACHE_EINVAL;
}
