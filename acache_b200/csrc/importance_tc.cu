// Anchor influence score on the tcgen05 tensor cores (bf16/fp16, head_dim 64/128).
//
//   importance[a] += sum over heads h and mask-query rows r of softmax_a(q[r,h] . K'[a] * scale)
//   K' = affix keys of the layer rotated by the table row `affix_shift`, rounded to T.
//
// One CTA (128 threads) = (KV head, tile of 128 virtual rows), a virtual row being a
// (mask query, head-in-GQA-group) pair.  The affix keys are streamed twice in tiles of 64:
//   pass 1: S = Q K'^T (tcgen05.mma, fp32 in TMEM), thread t owns row t and keeps its running
//           maximum and denominator;
//   pass 2: S again, p = exp2(s - m) / l goes transposed to shared memory and 128 threads add up
//           the 64 columns of the tile; the CTA writes its column sums to its own row of
//           `partial`, which importance_reduce_kernel adds in a fixed order (deterministic).
// Keys are staged through registers when they need the rotation, with cp.async otherwise.
// Long affixes are cut into chunks of kChunkTiles tiles that separate CTAs walk (grid.z): a first
// launch runs pass 1 per chunk and leaves every row's (maximum, denominator) per chunk in scratch,
// a second launch folds them per row and runs pass 2 per chunk; each chunk writes its own columns
// of the CTA's partial row, so the reduction that follows is unchanged.
// Every mbarrier wait is bounded.
#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {
int importance_tc_chunks(int affix_len);

namespace tc {

constexpr int IBM = 128, IBN = 64, INT = 128;
constexpr int kChunkTiles = 16;        // 1024 keys per chunk
constexpr int kChunkFrom = 2048;       // affixes longer than this are chunked
enum { kBothPasses = 0, kPassOne = 1, kPassTwo = 2 };
constexpr int kPsLd = 129;  // padded leading dimension of the transposed P tile

template <typename T, typename TR, typename TC, int D>
__global__ void __launch_bounds__(INT) importance_tc_kernel(
    const T* __restrict__ q, int64_t q_stride, const int32_t* __restrict__ q_rows, int n_q, int n_heads, int n_kv_heads,
    const T* __restrict__ affix_k, int64_t k_slot_stride, int affix_len, int affix_shift,
    const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin, int64_t rope_stride, float scale_log2,
    float* __restrict__ partial, int32_t* err_flag, int mode, float* __restrict__ ml,
    const int32_t* __restrict__ req_off, const int32_t* __restrict__ req_shift, int rope_rows) {
  constexpr int CH = D * (int)sizeof(T) / 16;
  constexpr int Q_BYTES = IBM * D * (int)sizeof(T);
  constexpr int K_BYTES = IBN * D * (int)sizeof(T);
  constexpr uint32_t kCols = 64;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sQ = smem_raw;
  uint8_t* sK = sQ + Q_BYTES;                                       // 2 stages
  float* sP = reinterpret_cast<float*>(sK + 2 * K_BYTES);           // [IBN][kPsLd]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + IBN * kPsLd);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int kvh = blockIdx.y;
  const int g = n_heads / n_kv_heads;
  const int m0 = blockIdx.x * IBM;
  // several requests in one launch (unchunked form only): blockIdx.z is the request, its mask
  // rows are q_rows[req_off[z] .. req_off[z + 1]), its rotation row req_shift[z]; its partial rows
  // follow those of the requests before it
  int req = 0;
  if (req_off != nullptr) {
    req = (int)blockIdx.z;
    const int o = req_off[req];
    n_q = max(req_off[req + 1] - o, 0);
    q_rows += o;
    affix_shift = req_shift != nullptr ? req_shift[req] : 0;
    if (affix_shift < 0 || affix_shift >= max(rope_rows, 1)) {
      if (tid == 0 && err_flag) atomicExch(err_flag, 4);
      affix_shift = 0;
    }
  }
  const int vrows = n_q * g;
  float* my_partial = partial + (((int64_t)req * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * affix_len;
  if (m0 >= vrows || (smem_u32(smem_raw) & 1023u) != 0) {
    // the first cannot happen with the launch grid, the second would be a launch error: keep the
    // reduce kernel's input defined (every chunk writes the whole row: same zeros) and report
    if (m0 < vrows && tid == 0 && err_flag) atomicExch(err_flag, 6);
    if (mode != kPassOne)
      for (int a = tid; a < affix_len; a += INT) my_partial[a] = 0.f;
    return;
  }
  const int rows_live = min(IBM, vrows - m0);
  // this CTA's tiles of the affix: all of them, or chunk blockIdx.z
  const int tiles_all = (affix_len + IBN - 1) / IBN;
  const int t0 = mode == kBothPasses ? 0 : (int)blockIdx.z * kChunkTiles;
  const int n_tiles = mode == kBothPasses ? tiles_all : min(kChunkTiles, tiles_all - t0);
  const int n_chunks = req_off != nullptr ? 1 : (int)gridDim.z;
  // (maximum, denominator) of row `tid` for chunk c of this (KV head, row tile)
  float* my_ml = ml + (((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * n_chunks) * (IBM * 2);

  const uint32_t bar_s = smem_u32(&bars[0]);
  if (tid == 0) {
    mbar_init(bar_s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

  // queries: gathered rows of the mask tokens
  for (int id = tid; id < IBM * CH; id += INT) {
    const int r = id / CH, c = id % CH;
    const int v = m0 + r;
    const bool ok = v < vrows;
    const int qrow = ok ? q_rows[v / g] : 0;
    const int head = kvh * g + (ok ? v % g : 0);
    cp_async16(smem_u32(sQ) + swz<D>(IBM, r, c), q + (int64_t)qrow * q_stride + (int64_t)head * D + c * (16 / sizeof(T)), ok);
  }
  // iterations 0..n_tiles-1 are pass 1, n_tiles..2 n_tiles-1 pass 2
  const int it_begin = mode == kPassTwo ? n_tiles : 0;
  const int it_end = mode == kPassOne ? n_tiles : 2 * n_tiles;
  auto load_k = [&](int it) {
    const int tile = t0 + it % n_tiles;
    const int j0 = tile * IBN;
    uint8_t* kb = sK + ((it - it_begin) & 1) * K_BYTES;
    for (int id = tid; id < IBN * CH; id += INT) {
      const int r = id / CH, c = id % CH;
      const int j = j0 + r;
      const bool ok = j < affix_len;
      const T* src = affix_k + (int64_t)(ok ? j : 0) * k_slot_stride + (int64_t)kvh * D + c * (16 / sizeof(T));
      if (affix_shift == 0) {
        cp_async16(smem_u32(kb) + swz<D>(IBN, r, c), src, ok);
      } else if (c < CH / 2) {
        constexpr int E = 16 / sizeof(T);
        Vec16<T> a, bb;
        a.u = make_uint4(0, 0, 0, 0);
        bb.u = a.u;
        if (ok) {
          a.u = *reinterpret_cast<const uint4*>(src);
          bb.u = *reinterpret_cast<const uint4*>(src + D / 2);
          const TR* cr = rope_cos + (int64_t)affix_shift * rope_stride;
          const TR* sr = rope_sin + (int64_t)affix_shift * rope_stride;
          const int d = c * E;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
            a.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), to_f32<TR>(sr[d + e])));
            bb.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), to_f32<TR>(sr[d + D / 2 + e])));
          }
        }
        *reinterpret_cast<uint4*>(kb + swz<D>(IBN, r, c)) = a.u;
        *reinterpret_cast<uint4*>(kb + swz<D>(IBN, r, c + CH / 2)) = bb.u;
      }
    }
  };

  const uint32_t idesc = make_idesc(Fmt<T>::id, 0, IBN, IBM);
  const bool warp_live = warp * 32 < rows_live;
  const bool row_ok = tid < rows_live;
  load_k(it_begin);
  cp_async_commit();

  float m_run = -INFINITY, l_run = 0.f, inv_l = 0.f;
  if (mode == kPassTwo) {   // fold what pass 1 left per chunk, in chunk order
    for (int c = 0; c < n_chunks; ++c) m_run = fmaxf(m_run, my_ml[(c * IBM + tid) * 2]);
    for (int c = 0; c < n_chunks; ++c) {
      const float mc = my_ml[(c * IBM + tid) * 2];
      l_run += mc == -INFINITY ? 0.f : my_ml[(c * IBM + tid) * 2 + 1] * ex2(mc - m_run);
    }
    inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
  }
  bool failed = false;
  uint32_t s[64];
  for (int it = it_begin; it < it_end; ++it) {
    if (it + 1 < it_end) load_k(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();   // also: every thread is done with the previous tile's sP and TMEM scores
    tc_fence_after();
    const int tile = t0 + it % n_tiles;
    const int j0 = tile * IBN;
    const int valid = min(IBN, affix_len - j0);
    const uint32_t kb = smem_u32(sK) + ((it - it_begin) & 1) * K_BYTES;
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t a_off = (ks / 4) * (IBM * 128) + (ks % 4) * 32;
        const uint32_t b_off = (ks / 4) * (IBN * 128) + (ks % 4) * 32;
        mma_ss(tmem_base, make_desc(smem_u32(sQ) + a_off, 16, 1024), make_desc(kb + b_off, 16, 1024), idesc, ks > 0 ? 1u : 0u);
      }
      mma_commit(bar_s);
    }
    const bool ok = mbar_wait(bar_s, (uint32_t)((it - it_begin) & 1));
    tc_fence_after();
    if (mode == kBothPasses && it == n_tiles) inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;   // pass 1 is complete for this row
    if (warp_live) {
      tmem_ld32(t_lane, s);
      tmem_ld32(t_lane + 32, s + 32);
      tmem_wait_ld();
      if (it < n_tiles) {
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < IBN; ++c) {
          const float v = (c < valid) ? __uint_as_float(s[c]) * scale_log2 : -INFINITY;
          s[c] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
        const float m_new = fmaxf(m_run, mx);
        float rs = 0.f;
#pragma unroll
        for (int c = 0; c < IBN; ++c) rs += ex2(__uint_as_float(s[c]) - m_new);
        l_run = l_run * ((m_run == -INFINITY) ? 0.f : ex2(m_run - m_new)) + rs;
        m_run = m_new;
      } else {
#pragma unroll
        for (int c = 0; c < IBN; ++c) {
          const float p = (c < valid && row_ok) ? ex2(fmaf(__uint_as_float(s[c]), scale_log2, -m_run)) * inv_l : 0.f;
          sP[c * kPsLd + tid] = p;
        }
      }
    }
    tc_fence_before();
    if (__syncthreads_or(!ok)) { failed = true; break; }
    if (it >= n_tiles) {
      // column sums of the tile: two threads per column, each over half of the live rows
      const int c = tid & 63, h = tid >> 6;
      const int r0 = h * 64, r1 = min(r0 + 64, rows_live);
      float acc = 0.f;
      for (int r = r0; r < r1; ++r) acc += sP[c * kPsLd + r];
      __shared__ float half_sum[64];
      if (h == 1) half_sum[c] = acc;
      __syncthreads();
      if (h == 0 && c < valid) my_partial[j0 + c] = acc + half_sum[c];
    }
  }
  if (mode == kPassOne) {
    my_ml[((int)blockIdx.z * IBM + tid) * 2] = failed ? -INFINITY : m_run;
    my_ml[((int)blockIdx.z * IBM + tid) * 2 + 1] = failed ? 0.f : l_run;
  }
  if (failed) {
    if (tid == 0 && err_flag) atomicExch(err_flag, 5);
    if (mode != kPassOne)   // this CTA's columns of the partial row
      for (int a = t0 * IBN + tid; a < min(affix_len, (t0 + n_tiles) * IBN); a += INT) my_partial[a] = 0.f;
  }
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

template <typename T, typename TR> struct PromoteI { using type = float; };
template <> struct PromoteI<__half, __half> { using type = __half; };
template <> struct PromoteI<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR, int D>
static int launch_importance_tc(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q, int n_heads,
                                int n_kv_heads, const void* affix_k, int64_t k_slot_stride, int affix_len,
                                int affix_shift, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                                float scale, float* partial, int* n_partials, float* ml, int32_t* err_flag,
                                cudaStream_t st) {
  using TC = typename PromoteI<T, TR>::type;
  constexpr size_t smem = IBM * D * sizeof(T) + 2 * IBN * D * sizeof(T) + IBN * kPsLd * sizeof(float) + 64;
  auto kern = importance_tc_kernel<T, TR, TC, D>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int g = n_heads / n_kv_heads;
  dim3 grid((n_q * g + IBM - 1) / IBM, n_kv_heads);
  const int chunks = importance_tc_chunks(affix_len);
  if (chunks <= 1 || ml == nullptr) {
    kern<<<grid, INT, smem, st>>>((const T*)q, q_stride, q_rows, n_q, n_heads, n_kv_heads, (const T*)affix_k,
                                  k_slot_stride, affix_len, affix_shift, (const TR*)rope_cos, (const TR*)rope_sin,
                                  rope_stride, scale * 1.4426950408889634f, partial, err_flag, kBothPasses, partial,
                                  nullptr, nullptr, 0);
  } else {
    dim3 grid3(grid.x, grid.y, chunks);
    for (int mode = kPassOne; mode <= kPassTwo; ++mode)
      kern<<<grid3, INT, smem, st>>>((const T*)q, q_stride, q_rows, n_q, n_heads, n_kv_heads, (const T*)affix_k,
                                     k_slot_stride, affix_len, affix_shift, (const TR*)rope_cos, (const TR*)rope_sin,
                                     rope_stride, scale * 1.4426950408889634f, partial, err_flag, mode, ml, nullptr, nullptr, 0);
  }
  ACACHE_LAUNCH_CHECK();
  *n_partials = (int)(grid.x * grid.y);
  return ACACHE_OK;
}

// All requests of a probe batch in one launch: grid.z = request.  `partial` gets n_requests groups
// of *n_partials rows each.
template <typename T, typename TR, int D>
static int launch_importance_tc_batched(const void* q, int64_t q_stride, const int32_t* q_rows, const int32_t* req_off,
                                        int n_requests, int max_q, int n_heads, int n_kv_heads, const void* affix_k,
                                        int64_t k_slot_stride, int affix_len, const int32_t* req_shift,
                                        const void* rope_cos, const void* rope_sin, int64_t rope_stride, int rope_rows,
                                        float scale, float* partial, int* n_partials, int32_t* err_flag,
                                        cudaStream_t st) {
  using TC = typename PromoteI<T, TR>::type;
  constexpr size_t smem = IBM * D * sizeof(T) + 2 * IBN * D * sizeof(T) + IBN * kPsLd * sizeof(float) + 64;
  auto kern = importance_tc_kernel<T, TR, TC, D>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int g = n_heads / n_kv_heads;
  dim3 grid((max_q * g + IBM - 1) / IBM, n_kv_heads, n_requests);
  kern<<<grid, INT, smem, st>>>((const T*)q, q_stride, q_rows, 0, n_heads, n_kv_heads, (const T*)affix_k, k_slot_stride,
                                affix_len, 0, (const TR*)rope_cos, (const TR*)rope_sin, rope_stride,
                                scale * 1.4426950408889634f, partial, err_flag, kBothPasses, partial, req_off, req_shift,
                                rope_rows);
  ACACHE_LAUNCH_CHECK();
  *n_partials = (int)(grid.x * grid.y);
  return ACACHE_OK;
}

}  // namespace tc

// chunks a long affix is cut into (1 = walked by one CTA per row tile and KV head)
int importance_tc_chunks(int affix_len) {
  if (affix_len <= tc::kChunkFrom) return 1;
  const int tiles = (affix_len + tc::IBN - 1) / tc::IBN;
  return (tiles + tc::kChunkTiles - 1) / tc::kChunkTiles;
}
// floats of scratch behind the partial rows for the per-chunk (maximum, denominator) pairs
int64_t importance_tc_ml_floats(int n_q_rows, int n_heads, int affix_len) {
  const int chunks = importance_tc_chunks(affix_len);
  if (chunks <= 1) return 0;
  // row tiles x KV heads <= (n_q_rows / 128 + 1) x n_heads (a KV head's rows are its group's)
  return ((int64_t)n_q_rows / tc::IBM + 1) * n_heads * tc::IBM * 2 * (int64_t)chunks;
}

// Returns ACACHE_EUNSUPPORTED for what the tensor-core kernel does not cover (fp32, head sizes
// other than 64/128); the caller then uses the general kernel.  On success *n_partials rows of
// `partial` ([n_partials][affix_len]) hold per-CTA column sums.
int importance_tc_dispatch(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q, int n_heads, int n_kv_heads,
                           int head_dim, int dtype, const void* affix_k, int64_t k_slot_stride, int affix_len,
                           int affix_shift, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                           int rope_dtype, float scale, float* partial, int* n_partials, float* ml, int32_t* err_flag,
                           cudaStream_t st) {
  if (dtype == ACACHE_F32 || (head_dim != 64 && head_dim != 128)) return ACACHE_EUNSUPPORTED;
  if (!aligned16(q) || !aligned16(affix_k) || q_stride % 8 != 0 || k_slot_stride % 8 != 0) return ACACHE_EUNSUPPORTED;
#define IMP_TC(T, TR)                                                                                                  \
  return head_dim == 128                                                                                               \
             ? tc::launch_importance_tc<T, TR, 128>(q, q_stride, q_rows, n_q, n_heads, n_kv_heads, affix_k,            \
                                                    k_slot_stride, affix_len, affix_shift, rope_cos, rope_sin,         \
                                                    rope_stride, scale, partial, n_partials, ml, err_flag, st)             \
             : tc::launch_importance_tc<T, TR, 64>(q, q_stride, q_rows, n_q, n_heads, n_kv_heads, affix_k,             \
                                                   k_slot_stride, affix_len, affix_shift, rope_cos, rope_sin,          \
                                                   rope_stride, scale, partial, n_partials, ml, err_flag, st)
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) { IMP_TC(__nv_bfloat16, float); }
    if (rope_dtype == ACACHE_BF16) { IMP_TC(__nv_bfloat16, __nv_bfloat16); }
    IMP_TC(__nv_bfloat16, __half);
  }
  if (rope_dtype == ACACHE_F32) { IMP_TC(__half, float); }
  if (rope_dtype == ACACHE_F16) { IMP_TC(__half, __half); }
  IMP_TC(__half, __nv_bfloat16);
#undef IMP_TC
}

// The batched form: ACACHE_EUNSUPPORTED also for affixes long enough to be chunked (the caller
// then loops over the requests).
int importance_tc_batched_dispatch(const void* q, int64_t q_stride, const int32_t* q_rows, const int32_t* req_off,
                                   int n_requests, int max_q, int n_heads, int n_kv_heads, int head_dim, int dtype,
                                   const void* affix_k, int64_t k_slot_stride, int affix_len, const int32_t* req_shift,
                                   const void* rope_cos, const void* rope_sin, int64_t rope_stride, int rope_rows,
                                   int rope_dtype, float scale, float* partial, int* n_partials, int32_t* err_flag,
                                   cudaStream_t st) {
  if (dtype == ACACHE_F32 || (head_dim != 64 && head_dim != 128) || importance_tc_chunks(affix_len) > 1)
    return ACACHE_EUNSUPPORTED;
  if (!aligned16(q) || !aligned16(affix_k) || q_stride % 8 != 0 || k_slot_stride % 8 != 0) return ACACHE_EUNSUPPORTED;
  if (n_requests > 65535) return ACACHE_EUNSUPPORTED;
#define IMP_TCB(T, TR)                                                                                                 \
  return head_dim == 128                                                                                               \
             ? tc::launch_importance_tc_batched<T, TR, 128>(q, q_stride, q_rows, req_off, n_requests, max_q, n_heads,  \
                                                            n_kv_heads, affix_k, k_slot_stride, affix_len, req_shift,  \
                                                            rope_cos, rope_sin, rope_stride, rope_rows, scale, partial, \
                                                            n_partials, err_flag, st)                                  \
             : tc::launch_importance_tc_batched<T, TR, 64>(q, q_stride, q_rows, req_off, n_requests, max_q, n_heads,   \
                                                           n_kv_heads, affix_k, k_slot_stride, affix_len, req_shift,   \
                                                           rope_cos, rope_sin, rope_stride, rope_rows, scale, partial, \
                                                           n_partials, err_flag, st)
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) { IMP_TCB(__nv_bfloat16, float); }
    if (rope_dtype == ACACHE_BF16) { IMP_TCB(__nv_bfloat16, __nv_bfloat16); }
    IMP_TCB(__nv_bfloat16, __half);
  }
  if (rope_dtype == ACACHE_F32) { IMP_TCB(__half, float); }
  if (rope_dtype == ACACHE_F16) { IMP_TCB(__half, __half); }
  IMP_TCB(__half, __nv_bfloat16);
#undef IMP_TCB
}

}  // namespace acache
