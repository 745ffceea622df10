// Bidirectional varlen attention over the slot-mapped paged cache on the 5th-generation
// tensor cores (tcgen05) with TMEM accumulators, for bf16/fp16 and head_dim 64/128.
//
// One CTA (128 threads) = one (request, KV head, tile of 128 "virtual rows").  A virtual
// row is a (query, head-of-the-GQA-group) pair, so all query heads that share a KV head
// share one pass over its K/V.  Per tile of 64 keys:
//   * K and V rows are gathered through the slot map (or block table) with 16-byte
//     cp.async into shared memory in the 128-byte-swizzled layout the MMA descriptors
//     expect (double buffered, the next tile is in flight during the current one),
//   * S = Q K^T      : tcgen05.mma, A = Q (K-major), B = K rows (K-major), fp32 in TMEM,
//   * thread t owns row t (TMEM lane t): tcgen05.ld of its 64 scores, online softmax
//     in the exp2 domain, P written back to shared memory as the A operand,
//   * O += P V       : tcgen05.mma, B = V rows (MN-major), accumulated in TMEM.
// O is only rescaled when a row's running maximum grows by more than 2^8 (otherwise the
// stale reference maximum is kept; the final division by the row sum makes it exact).
// Query-side relocation: the first shared_kv_lens[b] keys are scored against queries
// rotated by the inverse shift, then the query tile is swapped for the plain one.
// Key-side relocation: keys of the shared span are rotated while they are staged.
// Every mbarrier wait is bounded; on expiry the kernel raises the error flag, frees its
// TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {

namespace tc {

constexpr int BM = 128;      // virtual rows per CTA
constexpr int BN = 64;       // keys per tile
constexpr int NT = 128;      // threads
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128;

template <typename T, typename TR, typename TC, int D, bool KEYSIDE>
__global__ void __launch_bounds__(NT, 2) attention_tc_kernel(
    const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t o_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, int64_t num_slots, int n_heads, int n_kv_heads, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ cu_k, const int32_t* __restrict__ slot_map, const int32_t* __restrict__ block_tables,
    int table_stride, int block_size, float scale_log2, int shared_prefix_len,
    const int32_t* __restrict__ shared_kv_lens,
    const int32_t* __restrict__ affix_shifts, const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin,
    int64_t rope_stride, int rope_rows, int32_t* err_flag) {
  constexpr int CH = D * (int)sizeof(T) / 16;     // 16-byte chunks per row
  constexpr int Q_BYTES = BM * D * (int)sizeof(T);
  constexpr int KV_BYTES = BN * D * (int)sizeof(T);
  constexpr int P_BYTES = BM * BN * (int)sizeof(T);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand layout needs 1024-byte aligned atoms
    if (threadIdx.x == 0 && err_flag) atomicExch(err_flag, 6);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;       // 2 stages
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);  // [0] = S done, [1] = O done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int b = blockIdx.y, kvh = blockIdx.z;
  const int g = n_heads / n_kv_heads;
  const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
  const int m0 = blockIdx.x * BM;
  const int vrows = q_len * g;
  if (m0 >= vrows) return;
  const int kv0 = cu_k[b], kv_len = max(cu_k[b + 1] - kv0, 0);
  const int kv_row = n_kv_heads * D;

  const bool query_side = shared_kv_lens != nullptr && affix_shifts != nullptr;
  int n_shared = 0, shift = 0;
  if (query_side) {
    n_shared = min(max(shared_kv_lens[b], 0), kv_len);
    shift = affix_shifts[b];
    if (shift < 0 || shift >= rope_rows) {
      if (tid == 0 && err_flag) atomicExch(err_flag, 4);
      n_shared = 0;
    }
  }
  const int nt0 = (n_shared + BN - 1) / BN;
  const int nt1 = (kv_len - n_shared + BN - 1) / BN;
  const int n_tiles = nt0 + nt1;

  // this thread's virtual row
  const int vr = m0 + tid;
  const bool row_ok = vr < vrows;
  const int qi = row_ok ? vr / g : 0;
  const int head = kvh * g + (row_ok ? vr % g : 0);
  T* out_row = out + (int64_t)(q0 + qi) * o_stride + (int64_t)head * D;

  if (n_tiles == 0) {  // no keys: zeros
    if (row_ok) {
      for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(out_row + c * (16 / sizeof(T))) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  const uint32_t bar_s = smem_u32(&bars[0]), bar_o = smem_u32(&bars[1]);
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

  // ---- loaders -----------------------------------------------------------------------
  auto load_q = [&](bool rotated) {
    // chunk id = it*NT + tid: 16 consecutive threads cover one row
    for (int id = tid; id < BM * CH; id += NT) {
      const int r = id / CH, c = id % CH;
      const int v = m0 + r;
      const bool ok = v < vrows;
      const int rq = ok ? v / g : 0, rh = kvh * g + (ok ? v % g : 0);
      const T* src = q + (int64_t)(q0 + rq) * q_stride + (int64_t)rh * D + c * (16 / sizeof(T));
      const uint32_t dst = smem_u32(sQ) + swz<D>(BM, r, c);
      if (!rotated) {
        cp_async16(dst, src, ok);
      } else if (c < CH / 2) {
        // q*cos - rotate_half(q)*sin for the chunk pair (d, d + D/2), rounded to T
        constexpr int E = 16 / sizeof(T);
        Vec16<T> a, bb, o1, o2;
        a.u = make_uint4(0, 0, 0, 0);
        bb.u = a.u;
        if (ok) {
          a.u = *reinterpret_cast<const uint4*>(src);
          bb.u = *reinterpret_cast<const uint4*>(src + D / 2);
        }
        const TR* cr = rope_cos + (int64_t)shift * rope_stride;
        const TR* sr = rope_sin + (int64_t)shift * rope_stride;
        const int d = c * E;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
          o1.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), -to_f32<TR>(sr[d + e])));
          o2.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), -to_f32<TR>(sr[d + D / 2 + e])));
        }
        *reinterpret_cast<uint4*>(sQ + swz<D>(BM, r, c)) = o1.u;
        *reinterpret_cast<uint4*>(sQ + swz<D>(BM, r, c + CH / 2)) = o2.u;
      }
    }
  };
  auto tile_span = [&](int i, int& j0, int& j_end) {
    if (i < nt0) { j0 = i * BN; j_end = n_shared; }
    else { j0 = n_shared + (i - nt0) * BN; j_end = kv_len; }
  };
  // Slots of a tile are looked up one tile before its copies are issued, so the dependent
  // global load (slot -> row address) is never on the critical path.
  constexpr int ITER = BN * CH / NT;   // rows handled per thread and tile
  constexpr int RPI = NT / CH;         // rows covered per iteration
  const int my_c = tid % CH, my_r = tid / CH;
  auto fetch_slots = [&](int i, int32_t* slots) {
    int j0, j_end;
    tile_span(i, j0, j_end);
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int j = j0 + my_r + it * RPI;
      int64_t slot = -1;  // fits 32 bits: the dispatcher refuses larger caches
      if (j < j_end) {
        if (slot_map) slot = slot_map[kv0 + j];
        else {
          const int blk = block_tables[(int64_t)b * table_stride + j / block_size];
          slot = blk < 0 ? -2 : (int64_t)blk * block_size + j % block_size;
        }
        if (slot < 0 || slot >= num_slots) slot = -2;  // reported when the copy is issued
      }
      slots[it] = (int32_t)slot;
    }
  };
  auto load_kv = [&](int i, const int32_t* slots) {
    int j0, j_end;
    tile_span(i, j0, j_end);
    const uint32_t kb = smem_u32(sK) + (i & 1) * KV_BYTES, vb = smem_u32(sV) + (i & 1) * KV_BYTES;
    const int c = my_c;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int r = my_r + it * RPI;
      const int j = j0 + r;
      int64_t slot = slots[it];
      if (slot == -2 && err_flag) atomicExch(err_flag, 3);
      const bool ok = slot >= 0;
      if (!ok) slot = 0;
      const int64_t off = slot * kv_row + (int64_t)kvh * D + c * (16 / sizeof(T));
      const uint32_t so = swz<D>(BN, r, c);
      cp_async16(vb + so, v_cache + off, ok);
      if (!KEYSIDE) {
        cp_async16(kb + so, k_cache + off, ok);
      } else if (c < CH / 2) {
        // key-side relocation: a key that lives in the shared span is rotated by the table row
        // |j - slot| (sine negated when j < slot), rounded to T, before it is staged
        constexpr int E = 16 / sizeof(T);
        Vec16<T> a, bb;
        a.u = make_uint4(0, 0, 0, 0);
        bb.u = a.u;
        if (ok) {
          a.u = *reinterpret_cast<const uint4*>(k_cache + off);
          bb.u = *reinterpret_cast<const uint4*>(k_cache + off + D / 2);
          if (slot < shared_prefix_len) {
            const int64_t delta = (int64_t)j - slot;
            const bool neg = delta < 0;
            const int64_t row = neg ? -delta : delta;
            if (row >= rope_rows) {
              if (err_flag) atomicExch(err_flag, 4);
            } else {
              const TR* cr = rope_cos + row * rope_stride;
              const TR* sr = rope_sin + row * rope_stride;
              const int d = c * E;
#pragma unroll
              for (int e = 0; e < E; ++e) {
                const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(bb.e[e]);
                float s1 = to_f32<TR>(sr[d + e]), s2 = to_f32<TR>(sr[d + D / 2 + e]);
                if (neg) { s1 = -s1; s2 = -s2; }
                a.e[e] = from_f32<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), s1));
                bb.e[e] = from_f32<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2 + e]), s2));
              }
            }
          }
        }
        *reinterpret_cast<uint4*>(sK + (i & 1) * KV_BYTES + so) = a.u;
        *reinterpret_cast<uint4*>(sK + (i & 1) * KV_BYTES + swz<D>(BN, r, c + CH / 2)) = bb.u;
      }
    }
  };

  const uint32_t idesc_s = make_idesc(Fmt<T>::id, 0, BN, BM);
  const uint32_t idesc_o = make_idesc(Fmt<T>::id, 1, D, BM);

  // ---- prologue ------------------------------------------------------------------------
  const bool start_rotated = nt0 > 0;
  int32_t slots[ITER];
  fetch_slots(0, slots);
  load_q(start_rotated);
  load_kv(0, slots);
  cp_async_commit();
  if (n_tiles > 1) fetch_slots(1, slots);

  // a warp is live when at least one of its 32 rows is a real (query, head) pair
  const bool warp_live = m0 + warp * 32 < vrows;
  if (!warp_live) {  // its rows of P are never written: keep them zero so the MMA reads no junk
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(sP + tid * 128 + (c << 4)) = make_uint4(0, 0, 0, 0);
  }
  float m_ref = -INFINITY, l_sum = 0.f;
  bool failed = false;
  uint32_t s[64];

  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) load_kv(i + 1, slots);
    cp_async_commit();
    if (i + 2 < n_tiles) fetch_slots(i + 2, slots);
    cp_async_wait<1>();          // tile i (and the query tile) have landed for this thread
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    int j0, j_end;
    tile_span(i, j0, j_end);
    const uint32_t kb = smem_u32(sK) + (i & 1) * KV_BYTES, vb = smem_u32(sV) + (i & 1) * KV_BYTES;

    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t a_off = (ks / 4) * (BM * 128) + (ks % 4) * 32;
        const uint32_t b_off = (ks / 4) * (BN * 128) + (ks % 4) * 32;
        mma_ss(tmem_base + kColS, make_desc(smem_u32(sQ) + a_off, 16, 1024), make_desc(kb + b_off, 16, 1024), idesc_s,
               ks > 0 ? 1u : 0u);
      }
      mma_commit(bar_s);
    }
    bool ok = mbar_wait(bar_s, (uint32_t)(i & 1));
    tc_fence_after();
    // the previous P V product must be done before O is rescaled or P overwritten
    if (i > 0) ok = mbar_wait(bar_o, (uint32_t)((i - 1) & 1)) && ok;
    tc_fence_after();
    if (warp_live) {  // warps whose 32 rows are all padding skip the softmax (their P rows stay zero)
      tmem_ld32(t_lane + kColS, s);
      tmem_ld32(t_lane + kColS + 32, s + 32);
      tmem_wait_ld();
      // online softmax of this thread's row, exp2 domain; raw scores are scaled inside the fma
      const int valid = j_end - j0;  // >= 1
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < BN; ++c) {
        const float v = (c < valid) ? __uint_as_float(s[c]) : -INFINITY;
        s[c] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      mx *= scale_log2;
      const bool grow = mx > m_ref + 8.0f;  // also true on the first tile (m_ref = -inf)
      if (__any_sync(0xFFFFFFFFu, grow) && i > 0) {
        const float f = grow ? ex2(m_ref - mx) : 1.0f;
        l_sum *= f;
        uint32_t o[32];
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          tmem_ld32(t_lane + kColO + c0, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * f);
          tmem_st32(t_lane + kColO + c0, o);
        }
        tmem_wait_st();
      }
      if (grow) m_ref = mx;
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < BN; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(s[c + e]), scale_log2, -m_ref));
          const float p1 = ex2(fmaf(__uint_as_float(s[c + e + 1]), scale_log2, -m_ref));
          rs += p0 + p1;
          w[e / 2] = pack2<T>(p0, p1);
        }
        *reinterpret_cast<uint4*>(sP + tid * 128 + (((c / 8) ^ (tid & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l_sum += rs;
    }

    // query tile swap at the partition boundary: every S product against the rotated
    // queries has completed (bar_s of this tile was awaited)
    const bool swap_q = start_rotated && i == nt0 - 1 && nt1 > 0;
    if (swap_q) {
      load_q(false);
      cp_async_commit();
      cp_async_wait<0>();
    }
    fence_proxy_async();
    tc_fence_before();
    if (__syncthreads_or(!ok)) { failed = true; break; }
    tc_fence_after();

    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
        mma_ss(tmem_base + kColO, make_desc(smem_u32(sP) + ks * 32, 16, 1024),
               make_desc(vb + ks * 2048, BN * 128, 1024), idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
      }
      mma_commit(bar_o);
    }
  }

  if (!failed) {
    bool ok = mbar_wait(bar_o, (uint32_t)((n_tiles - 1) & 1));
    tc_fence_after();
    if (__syncthreads_or(!ok)) failed = true;
  }
  if (!failed) {
    const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
    uint32_t o[32];
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      tmem_ld32(t_lane + kColO + c0, o);
      tmem_wait_ld();
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 w;
          w.x = pack2<T>(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
          w.y = pack2<T>(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
          w.z = pack2<T>(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
          w.w = pack2<T>(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
          *reinterpret_cast<uint4*>(out_row + c0 + c) = w;
        }
      }
    }
  } else if (tid == 0 && err_flag) {
    atomicExch(err_flag, 5);
  }
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename T, typename TR> struct PromoteT { using type = float; };
template <> struct PromoteT<__half, __half> { using type = __half; };
template <> struct PromoteT<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR, int D>
static int launch(const AttnArgs& a) {
  using TC = typename PromoteT<T, TR>::type;
  constexpr size_t smem = BM * D * sizeof(T) + 4 * BN * D * sizeof(T) + BM * BN * sizeof(T) + 64;
  const int g = a.n_heads / a.n_kv_heads;
  dim3 grid((a.max_q * g + BM - 1) / BM, a.batch, a.n_kv_heads);
  const bool relocate = a.shared_prefix_len > 0 && a.affix_shifts != nullptr;
  const bool query_side = relocate && a.shared_kv_lens != nullptr;
  const bool key_side = relocate && !query_side;
#define ACACHE_TC_LAUNCH(KS)                                                                                          \
  do {                                                                                                                \
    auto kern = attention_tc_kernel<T, TR, TC, D, KS>;                                                                \
    ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));            \
    kern<<<grid, NT, smem, a.st>>>((const T*)a.q, a.q_stride, (T*)a.out, a.o_stride, (const T*)a.k_cache,             \
                                   (const T*)a.v_cache, a.num_slots, a.n_heads, a.n_kv_heads, a.cu_q, a.cu_k,         \
                                   a.slot_map, a.block_tables, a.table_stride, a.block_size,                          \
                                   a.scale * 1.4426950408889634f, a.shared_prefix_len,                                \
                                   query_side ? a.shared_kv_lens : nullptr, query_side ? a.affix_shifts : nullptr,    \
                                   (const TR*)a.rope_cos, (const TR*)a.rope_sin, a.rope_stride, a.rope_rows,          \
                                   a.err_flag);                                                                       \
  } while (0)
  if (key_side) ACACHE_TC_LAUNCH(true);
  else ACACHE_TC_LAUNCH(false);
#undef ACACHE_TC_LAUNCH
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR>
static int by_dim(const AttnArgs& a) {
  if (a.head_dim == 128) return launch<T, TR, 128>(a);
  if (a.head_dim == 64) return launch<T, TR, 64>(a);
  return ACACHE_EUNSUPPORTED;
}

}  // namespace tc

// Declines (ACACHE_EUNSUPPORTED) what this kernel does not cover: fp32 caches, head sizes
// other than 64/128, unaligned tensors.
int attention_tc_dispatch(const AttnArgs& a, int dtype, int rope_dtype) {
  if (dtype == ACACHE_F32 || a.num_slots >= (1ll << 31)) return ACACHE_EUNSUPPORTED;
  if (a.head_dim != 64 && a.head_dim != 128) return ACACHE_EUNSUPPORTED;
  if (!aligned16(a.q) || !aligned16(a.out) || !aligned16(a.k_cache) || !aligned16(a.v_cache)) return ACACHE_EUNSUPPORTED;
  if (a.q_stride % 8 != 0 || a.o_stride % 8 != 0) return ACACHE_EUNSUPPORTED;
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) return tc::by_dim<__nv_bfloat16, float>(a);
    if (rope_dtype == ACACHE_BF16) return tc::by_dim<__nv_bfloat16, __nv_bfloat16>(a);
    return tc::by_dim<__nv_bfloat16, __half>(a);
  }
  if (rope_dtype == ACACHE_F32) return tc::by_dim<__half, float>(a);
  if (rope_dtype == ACACHE_F16) return tc::by_dim<__half, __half>(a);
  return tc::by_dim<__half, __nv_bfloat16>(a);
}

}  // namespace acache
