// Fused QKV projection for the rows of a forward: one tcgen05 GEMM whose epilogue applies
// the bias, rotates the q and k heads (RoPE at the row's position) and writes q to its output
// buffer and k / v straight into the paged cache at the row's slot.  The rotated K and V never
// exist as separate tensors and pass through HBM once.
//
//   acc[M, N] = X[M, K] . W[N, K]^T           N = (n_heads + 2 n_kv_heads) * 128, one head per N tile
//
// Persistent CTAs (one per SM) walk the (m tile, n tile) grid, n-major so that CTAs running at
// the same time share the weight tile in L2.  Per CTA (192 threads):
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//               128 x 64 X tile and W tile of every k block into a 6-stage ring (mbarrier tx);
//   warp 1      one thread issues tcgen05.mma (M = N = 128, K = 16 x 4 per stage) into one of two
//               128-column TMEM accumulators; tcgen05.commit frees the stage / publishes the tile;
//   warps 2-5   epilogue: thread = row (TMEM lane); both halves (d, d + 64) of a head are in the
//               same thread, so the rotation needs no exchange; overlaps with the next tile's MMAs.
// All waits are bounded and watch a CTA-wide abort flag.
#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {
namespace qkv {

using namespace tc;

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 6, NT = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t kTmemCols = 256;

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort) {
  const long long t0 = clock64();
  for (uint32_t it = 0;; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 63) == 63) {
      if (*abort) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort = 1;
        return false;
      }
      __nanosleep(32);
    }
  }
}

template <typename T, typename TR, typename TC>
__global__ void __launch_bounds__(NT, 1) qkv_rope_scatter_kernel(
    const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, int M, int K, int n_heads,
    int n_kv_heads, const T* __restrict__ bias, const int64_t* __restrict__ positions, const TR* __restrict__ rope_cos,
    const TR* __restrict__ rope_sin, int64_t rope_stride, int rope_rows, T* __restrict__ out_q, int64_t q_stride,
    T* __restrict__ k_cache, T* __restrict__ v_cache, const int32_t* __restrict__ slots, int64_t num_slots,
    int32_t* err_flag) {
  constexpr int D = 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);
  // [0..S) full, [S..2S) empty, [2S, 2S+2) tmem_full, [2S+2, 2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (tid == 0 && err_flag) atomicExch(err_flag, 6);
    return;
  }
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = n_heads + 2 * n_kv_heads;
  const int total = m_tiles * n_tiles;
  const int k_blocks = K / BK;

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(bar(i), 1);
      mbar_init(bar(STAGES + i), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar(2 * STAGES + a), 1);
      mbar_init(bar(2 * STAGES + 2 + a), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int mt = t % m_tiles, nt = t / m_tiles;
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES) ok = wait_or_abort(bar(STAGES + s), (uint32_t)(((it / STAGES) - 1) & 1), abort_flag);
          if (!ok) break;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar(s)), "r"((uint32_t)STAGE_BYTES) : "memory");
          const uint32_t dst = smem_u32(ring) + s * STAGE_BYTES;
          tma_load_2d(dst, &tmap_x, bar(s), kb * BK, mt * BM);
          tma_load_2d(dst + A_BYTES, &tmap_w, bar(s), kb * BK, nt * BN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(Fmt<T>::id, 0, BN, BM);
      int it = 0, n = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++n) {
        const int acc = n & 1;
        if (n >= 2) ok = wait_or_abort(bar(2 * STAGES + 2 + acc), (uint32_t)(((n >> 1) - 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          ok = wait_or_abort(bar(s), (uint32_t)((it / STAGES) & 1), abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a = smem_u32(ring) + s * STAGE_BYTES, b = a + A_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {
            mma_ss(tmem_base + acc * 128, make_desc(a + ks * 32, 16, 1024), make_desc(b + ks * 32, 16, 1024), idesc,
                   (kb > 0 || ks > 0) ? 1u : 0u);
          }
          mma_commit(bar(STAGES + s));            // stage free once these products have read it
        }
        if (ok) mma_commit(bar(2 * STAGES + acc));  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int kv_row = n_kv_heads * D;
    int n = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++n) {
      const int mt = t % m_tiles, nt = t / m_tiles;
      const int acc = n & 1;
      ok = wait_or_abort(bar(2 * STAGES + acc), (uint32_t)((n >> 1) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int m = mt * BM + row;
      const bool live = m < M;
      const int kind = nt < n_heads ? 0 : (nt < n_heads + n_kv_heads ? 1 : 2);   // q / k / v head
      T* dst = nullptr;
      bool store = live;
      if (kind == 0) {
        dst = out_q + (int64_t)(live ? m : 0) * q_stride + (int64_t)nt * D;
      } else {
        const int slot = live ? slots[m] : -1;
        if (slot < 0 || slot >= num_slots) {
          if (slot != -1 && live && err_flag) atomicExch(err_flag, 1);
          store = false;
        }
        const int h = kind == 1 ? nt - n_heads : nt - n_heads - n_kv_heads;
        dst = (kind == 1 ? k_cache : v_cache) + (int64_t)(store ? slot : 0) * kv_row + (int64_t)h * D;
      }
      const TR* cr = rope_cos;
      const TR* sr = rope_sin;
      if (kind < 2 && live) {
        const int64_t pos = positions[m];
        if (pos < 0 || pos >= rope_rows) {
          if (err_flag) atomicExch(err_flag, 2);
          store = false;
        } else {
          cr += pos * rope_stride;
          sr += pos * rope_stride;
        }
      }
      const T* bp = bias ? bias + (int64_t)nt * D : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t lo[32], hi[32];
        tmem_ld32(t_lane + acc * 128 + c0, lo);
        tmem_ld32(t_lane + acc * 128 + 64 + c0, hi);
        tmem_wait_ld();
        if (store) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint32_t wl[4], wh[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              float o1[2], o2[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int d = c0 + c + e + u;
                float x1 = __uint_as_float(lo[c + e + u]), x2 = __uint_as_float(hi[c + e + u]);
                if (bp) {
                  x1 += to_f32<T>(bp[d]);
                  x2 += to_f32<T>(bp[d + 64]);
                }
                x1 = round_to<T>(x1);   // the projection's output in T, as an unfused GEMM leaves it
                x2 = round_to<T>(x2);
                if (kind < 2) {
                  o1[u] = rot_lo<TC>(x1, x2, to_f32<TR>(cr[d]), to_f32<TR>(sr[d]));
                  o2[u] = rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + 64]), to_f32<TR>(sr[d + 64]));
                } else {
                  o1[u] = x1;
                  o2[u] = x2;
                }
              }
              wl[e / 2] = pack2<T>(o1[0], o1[1]);
              wh[e / 2] = pack2<T>(o2[0], o2[1]);
            }
            *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            *reinterpret_cast<uint4*>(dst + 64 + c0 + c) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
          }
        }
      }
      tc_fence_before();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar(2 * STAGES + 2 + acc)) : "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && err_flag) atomicExch(err_flag, 5);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t row_stride_elems,
                     int dtype) {
  return make_tensor_map_2d(map, base, rows, cols, row_stride_elems, 128, dtype);
}

template <typename T, typename TR> struct PromoteQ { using type = float; };
template <> struct PromoteQ<__half, __half> { using type = __half; };
template <> struct PromoteQ<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR>
static int launch(const CUtensorMap& mx, const CUtensorMap& mw, int M, int K, int n_heads, int n_kv_heads,
                  const void* bias, const int64_t* positions, const void* cos, const void* sin, int64_t rope_stride,
                  int rope_rows, void* out_q, int64_t q_stride, void* k_cache, void* v_cache, const int32_t* slots,
                  int64_t num_slots, int32_t* err_flag, cudaStream_t st) {
  using TC = typename PromoteQ<T, TR>::type;
  constexpr size_t smem = STAGES * STAGE_BYTES + 256;
  auto kern = qkv_rope_scatter_kernel<T, TR, TC>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int total = ((M + BM - 1) / BM) * (n_heads + 2 * n_kv_heads);
  const int grid = total < kNumSMs ? total : kNumSMs;
  kern<<<grid, NT, smem, st>>>(mx, mw, M, K, n_heads, n_kv_heads, (const T*)bias, positions, (const TR*)cos,
                               (const TR*)sin, rope_stride, rope_rows, (T*)out_q, q_stride, (T*)k_cache, (T*)v_cache,
                               slots, num_slots, err_flag);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

}  // namespace qkv
}  // namespace acache

using namespace acache;

extern "C" int acache_qkv_rope_scatter(const void* x, int64_t x_stride, int n_rows, int hidden, const void* w_qkv,
                                       const void* bias, int n_heads, int n_kv_heads, int head_dim, int dtype,
                                       const int64_t* positions, const void* rope_cos, const void* rope_sin,
                                       int64_t rope_row_stride, int rope_rows, int rope_dtype, void* out_q,
                                       int64_t q_stride, void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                       int64_t num_slots, int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype) || n_rows < 0 || hidden <= 0 || n_heads <= 0 || n_kv_heads <= 0)
    return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !w_qkv || !positions || !rope_cos || !rope_sin || !out_q || !k_cache || !v_cache || !slot_mapping)
    return ACACHE_EINVAL;
  if (dtype == ACACHE_F32 || head_dim != 128 || hidden % qkv::BK != 0) return ACACHE_EUNSUPPORTED;
  if (!aligned16(x) || !aligned16(w_qkv) || x_stride % 8 != 0 || !aligned16(out_q) || q_stride % 8 != 0 ||
      !aligned16(k_cache) || !aligned16(v_cache) || (bias && !aligned16(bias)))
    return ACACHE_EUNSUPPORTED;
  CUtensorMap mx, mw;
  const int64_t N = (int64_t)(n_heads + 2 * n_kv_heads) * head_dim;
  if (!qkv::make_map(&mx, x, n_rows, hidden, x_stride, dtype) || !qkv::make_map(&mw, w_qkv, N, hidden, hidden, dtype))
    return ACACHE_EUNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
#define QKV(T, TR)                                                                                                  \
  return qkv::launch<T, TR>(mx, mw, n_rows, hidden, n_heads, n_kv_heads, bias, positions, rope_cos, rope_sin,       \
                            rope_row_stride, rope_rows, out_q, q_stride, k_cache, v_cache, slot_mapping, num_slots, \
                            err_flag, st)
  if (dtype == ACACHE_BF16) {
    if (rope_dtype == ACACHE_F32) { QKV(__nv_bfloat16, float); }
    if (rope_dtype == ACACHE_BF16) { QKV(__nv_bfloat16, __nv_bfloat16); }
    QKV(__nv_bfloat16, __half);
  }
  if (rope_dtype == ACACHE_F32) { QKV(__half, float); }
  if (rope_dtype == ACACHE_F16) { QKV(__half, __half); }
  QKV(__half, __nv_bfloat16);
#undef QKV
}
