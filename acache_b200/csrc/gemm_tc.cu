// Dense projections of the served models as tcgen05 GEMMs on CTA pairs, with the work that
// follows each projection in the reference model fused into the epilogue:
//
//   acc[M, N] = X[M, K] . W[N, K]^T        (bf16 / fp16 in, fp32 accumulation in TMEM)
//
//   plain    out = acc (+ bias)                               output / down projections
//   swiglu   out[:, j] = act(gate_j) * up_j                   gate and up projections in one GEMM
//   qkv      bias, RoPE at the row's position, q to its buffer, k / v into the paged cache
//   argmax   per row: arg-max, maximum and sum of exponentials over the N columns (output
//            head + greedy unmasking statistics; the logits never reach global memory)
//   partial  the K range cut into S slices, slice s of every tile is a tile of its own and leaves
//            its fp32 sums in partial[s]; for projections with so few output tiles that whole
//            tiles would leave most of the 74 pairs idle.  The normalisation kernel that consumes
//            the projection adds the slices (`acache_add_rmsnorm_partials`).
//
// Two CTAs of a cluster work as one: `tcgen05.mma.cta_group::2` multiplies a 256-row block of X
// (128 rows staged by each CTA) with a BN-column block of W (BN/2 rows staged by each CTA), so a
// W tile crosses L2 -> shared memory once per 256 rows, or once per 512 rows when a pair keeps
// two row blocks (MB = 2).  Every CTA loads its own halves with plain TMA tile loads whose
// completion is counted on the leader's mbarrier; nothing is multicast.  Per CTA (320 threads):
//   warp 0      one thread issues the TMA loads of every k block into a ring of stages;
//   warp 1      (leader CTA only) one thread issues the products of the pair into TMEM and
//               commits them to the `stage free` barriers of both CTAs / the `accumulator ready`
//               barriers of both CTAs;
//   warps 2-9   epilogue: thread = accumulator row, two warps per 32 rows taking alternate
//               32-column groups; reads TMEM 16 columns at a time.
// The pair walks the tile list (row block fastest, so pairs that run together share W tiles in
// L2); BN is chosen per launch so that the tiles fill whole waves of the 74 pairs, and with two
// accumulator stages (when they fit the 512 TMEM columns) the epilogue of a tile overlaps the
// products of the next.  All waits are bounded; a wait that runs out raises error code 5.
#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {
namespace gemm {

using namespace tc;

constexpr int BK = 64, NT = 320;          // 2 single-thread roles + 8 epilogue warps
constexpr int A_SUB = 128 * BK * 2;      // one 128-row block of X for one k block: 16 KB
constexpr int kPairs = kNumSMs / 2;
constexpr int kMaxStages = 8;
constexpr uint32_t kTmemCols = 512;

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_QKV = 2, EPI_ARGMAX = 3, EPI_PARTIAL = 4 };

struct Params {
  int M, N, K, MB, BN, stages, acc_stages, group;
  int ksplit;           // slices of the K range (1 except for EPI_PARTIAL)
  float* partial;       // EPI_PARTIAL: [ksplit][M][N] fp32
  // plain / swiglu
  void* out; int64_t ldo; const void* bias; int act;
  // qkv
  int n_heads, n_kv_heads; const int64_t* positions; const void* rope_cos; const void* rope_sin; int64_t rope_stride;
  int rope_rows; void* out_q; int64_t q_stride; void* k_cache; void* v_cache; const int32_t* slots; int64_t num_slots;
  // argmax: per (column tile, row) partial maximum, its column and the sum of exp(x - maximum)
  float* part_max; int32_t* part_arg; float* part_sum;
  int32_t* err_flag;
};

// TMA tile load of this CTA's half of a pair's operand; the bytes are counted on `bar`, which
// may be the mbarrier of the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// All products of one k block of the pair (4 k steps of 16 x MB row blocks) from ONE statement, so
// that the issuing thread spends a few integer operations per product: the operand descriptors
// differ only in their 14-bit start address, which advances by 2 (32 bytes) per k step and by 1024
// (16 KB) per row block.  `hi` is the descriptors' common upper word, `a_lo` / `b_lo` the lower
// words for k step 0; `first` = 0 starts the accumulators over with the first k step.
#define ACACHE_MMA2 "tcgen05.mma.cta_group::2.kind::f16 "
template <int MB>
__device__ __forceinline__ void issue_kblock(uint32_t d0, uint32_t d1, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                             uint32_t idesc, uint32_t first);
template <>
__device__ __forceinline__ void issue_kblock<1>(uint32_t d0, uint32_t d1, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                uint32_t idesc, uint32_t first) {
  (void)d1;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t.reg .b32 ta, tb;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 q, %5, %5;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      ACACHE_MMA2 "[%0], da, db, %4, p;\n\t"
      "add.u32 ta, %1, 2;\n\tadd.u32 tb, %2, 2;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      ACACHE_MMA2 "[%0], da, db, %4, q;\n\t"
      "add.u32 ta, %1, 4;\n\tadd.u32 tb, %2, 4;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      ACACHE_MMA2 "[%0], da, db, %4, q;\n\t"
      "add.u32 ta, %1, 6;\n\tadd.u32 tb, %2, 6;\n\tmov.b64 da, {ta, %3};\n\tmov.b64 db, {tb, %3};\n\t"
      ACACHE_MMA2 "[%0], da, db, %4, q;\n\t}"
      ::"r"(d0), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(first) : "memory");
}
template <>
__device__ __forceinline__ void issue_kblock<2>(uint32_t d0, uint32_t d1, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                uint32_t idesc, uint32_t first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, dc, db;\n\t.reg .b32 ta, tc, tb;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 q, %6, %6;\n\t"
      "add.u32 tc, %2, 1024;\n\tmov.b64 da, {%2, %4};\n\tmov.b64 dc, {tc, %4};\n\tmov.b64 db, {%3, %4};\n\t"
      ACACHE_MMA2 "[%0], da, db, %5, p;\n\t"
      ACACHE_MMA2 "[%1], dc, db, %5, p;\n\t"
      "add.u32 ta, %2, 2;\n\tadd.u32 tc, %2, 1026;\n\tadd.u32 tb, %3, 2;\n\t"
      "mov.b64 da, {ta, %4};\n\tmov.b64 dc, {tc, %4};\n\tmov.b64 db, {tb, %4};\n\t"
      ACACHE_MMA2 "[%0], da, db, %5, q;\n\t"
      ACACHE_MMA2 "[%1], dc, db, %5, q;\n\t"
      "add.u32 ta, %2, 4;\n\tadd.u32 tc, %2, 1028;\n\tadd.u32 tb, %3, 4;\n\t"
      "mov.b64 da, {ta, %4};\n\tmov.b64 dc, {tc, %4};\n\tmov.b64 db, {tb, %4};\n\t"
      ACACHE_MMA2 "[%0], da, db, %5, q;\n\t"
      ACACHE_MMA2 "[%1], dc, db, %5, q;\n\t"
      "add.u32 ta, %2, 6;\n\tadd.u32 tc, %2, 1030;\n\tadd.u32 tb, %3, 6;\n\t"
      "mov.b64 da, {ta, %4};\n\tmov.b64 dc, {tc, %4};\n\tmov.b64 db, {tb, %4};\n\t"
      ACACHE_MMA2 "[%0], da, db, %5, q;\n\t"
      ACACHE_MMA2 "[%1], dc, db, %5, q;\n\t}"
      ::"r"(d0), "r"(d1), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(first) : "memory");
}
#undef ACACHE_MMA2

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

__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == 0) return x / (1.0f + __expf(-x));                 // silu
  if (act == 1) return x > 0.f ? x : 0.f;                       // relu
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));    // gelu (erf form)
}

template <typename TR> __device__ __forceinline__ void load8(const TR* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float* o) {
  Vec16<__half> v;
  v.u = *reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = __half2float(v.e[i]);
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
  Vec16<__nv_bfloat16> v;
  v.u = *reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = __bfloat162float(v.e[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float* o) {
  return make_uint4(pack2<T>(o[0], o[1]), pack2<T>(o[2], o[3]), pack2<T>(o[4], o[5]), pack2<T>(o[6], o[7]));
}

// ---- epilogues: one accumulator row (global row m, live = inside the matrix), 16 columns
// starting at global column n, values v[0..15] --------------------------------------------
template <typename T>
__device__ __forceinline__ void epi_plain(const Params& p, int m, int n, const float* v) {
  float o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = v[i];
  if (p.bias) {
    float b[16];
    load8<T>((const T*)p.bias + n, b);
    load8<T>((const T*)p.bias + n + 8, b + 8);
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] += b[i];
  }
  T* dst = (T*)p.out + (int64_t)m * p.ldo + n;
  *reinterpret_cast<uint4*>(dst) = pack8<T>(o);
  *reinterpret_cast<uint4*>(dst + 8) = pack8<T>(o + 8);
}

__device__ __forceinline__ void epi_partial(const Params& p, int ks, int m, int n, const float* v) {
  float4* dst = reinterpret_cast<float4*>(p.partial + ((int64_t)ks * p.M + m) * p.N + n);
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// W rows are interleaved in groups of 8: columns n..n+7 are gate features n/2..n/2+7 and columns
// n+8..n+15 the up features of the same indices; both projections are rounded to T first, the
// activation is rounded to T, then the product, as the separate kernels do
template <typename T>
__device__ __forceinline__ void epi_swiglu(const Params& p, int m, int n, const float* v) {
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float g = round_to<T>(v[i]), u = round_to<T>(v[8 + i]);
    o[i] = round_to<T>(act_fn(g, p.act)) * u;
  }
  *reinterpret_cast<uint4*>((T*)p.out + (int64_t)m * p.ldo + (n >> 1)) = pack8<T>(o);
}

// W rows are interleaved inside every head in groups of 8: columns n..n+7 are features
// d..d+7 and columns n+8..n+15 features d+64..d+71 of head n/128, d = (n % 128) / 2, so both
// halves of a rotation pair sit in one thread
template <typename T, typename TR, typename TC>
__device__ __forceinline__ void epi_qkv(const Params& p, int m, int n, const float* v, int64_t pos, int slot) {
  constexpr int D = 128;
  const int head = n / D, d = (n % D) >> 1;
  const int kind = head < p.n_heads ? 0 : (head < p.n_heads + p.n_kv_heads ? 1 : 2);
  float x1[8], x2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x1[i] = v[i];
    x2[i] = v[8 + i];
  }
  if (p.bias) {
    float b[16];
    load8<T>((const T*)p.bias + n, b);
    load8<T>((const T*)p.bias + n + 8, b + 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x1[i] += b[i];
      x2[i] += b[8 + i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {   // the projection's output in T, as an unfused GEMM leaves it
    x1[i] = round_to<T>(x1[i]);
    x2[i] = round_to<T>(x2[i]);
  }
  T* dst;
  if (kind == 0) {
    dst = (T*)p.out_q + (int64_t)m * p.q_stride + (int64_t)head * D + d;
  } else {
    if (slot < 0) return;
    const int h = kind == 1 ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
    dst = (T*)(kind == 1 ? p.k_cache : p.v_cache) + (int64_t)slot * p.n_kv_heads * D + (int64_t)h * D + d;
  }
  if (kind < 2) {
    if (pos < 0) return;
    const TR* cr = (const TR*)p.rope_cos + pos * p.rope_stride;
    const TR* sr = (const TR*)p.rope_sin + pos * p.rope_stride;
    float c1[8], s1[8], c2[8], s2[8], o1[8], o2[8];
    load8<TR>(cr + d, c1);
    load8<TR>(sr + d, s1);
    load8<TR>(cr + d + 64, c2);
    load8<TR>(sr + d + 64, s2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o1[i] = rot_lo<TC>(x1[i], x2[i], c1[i], s1[i]);
      o2[i] = rot_hi<TC>(x1[i], x2[i], c2[i], s2[i]);
    }
    *reinterpret_cast<uint4*>(dst) = pack8<T>(o1);
    *reinterpret_cast<uint4*>(dst + 64) = pack8<T>(o2);
  } else {
    *reinterpret_cast<uint4*>(dst) = pack8<T>(x1);
    *reinterpret_cast<uint4*>(dst + 64) = pack8<T>(x2);
  }
}

template <typename T, typename TR, typename TC, int EPI, int MB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NT, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  chain_release();
  const int BN = p.BN, S = p.stages, AS = p.acc_stages;
  const int G = p.group;                       // stages released together (1 or 2; S is a multiple)
  const int b_bytes = (BN / 2) * BK * 2;
  const int stage_bytes = MB * A_SUB + b_bytes;
  uint8_t* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)S * stage_bytes);
  // [0, S) full (leader's are used), [S, 2S) empty, [2S, 2S+2) accumulator full, [2S+2, 2S+4) accumulator empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };
  const int FULL = 0, EMPTY = kMaxStages, ACC_FULL = 2 * kMaxStages, ACC_EMPTY = 2 * kMaxStages + 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const bool misplaced = (smem_u32(smem_raw) & 1023u) != 0;

  const int rows_per_tile = 256 * MB;
  const int m_tiles = (p.M + rows_per_tile - 1) / rows_per_tile;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int mn_tiles = m_tiles * n_tiles;
  const int total = mn_tiles * p.ksplit;       // slice-major: the slices of a tile run on different pairs
  const int k_blocks = (p.K + BK - 1) / BK;
  const int k_per = (k_blocks + p.ksplit - 1) / p.ksplit;   // the host made sure no slice is empty
  const int acc_cols = (BN + 31) & ~31;       // TMEM columns reserved per accumulator

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar(FULL + i), 1);
      mbar_init(bar(EMPTY + i), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar(ACC_FULL + a), 1);
      mbar_init(bar(ACC_EMPTY + a), 16);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = misplaced ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0 && (tmem_base & 0xFFFFu) != 0) *abort_flag = 1;   // the pair needs the same columns in both CTAs
  __syncthreads();
  chain_wait();                // everything above is on-chip set-up; X may still be being written until here

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && !*abort_flag) {
      int s = 0;
      uint32_t round = 0;                      // times the ring has wrapped
      bool ok = true;
      for (int t = pair; t < total && ok; t += n_pairs) {
        const int tt = t % mn_tiles, ks = t / mn_tiles;
        const int mt = tt % m_tiles, nt = tt / m_tiles;
        const int m0 = mt * rows_per_tile + (int)rank * 128, n0 = nt * BN + (int)rank * (BN / 2);
        const int kb_end = min(k_blocks, (ks + 1) * k_per);
        for (int kb = ks * k_per; kb < kb_end && ok; ++kb, s = (s + 1 == S) ? 0 : s + 1, round += (s == 0)) {
          // a group of G stages is handed back by one commit after its last stage was read
          if (round > 0 && (s & (G - 1)) == 0) ok = wait_or_abort(bar(EMPTY + s / G), (round - 1) & 1, abort_flag);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(bar(FULL + s), (uint32_t)(2 * stage_bytes));   // both CTAs' bytes
          const uint32_t full = map_to_cta(bar(FULL + s), 0);
          const uint32_t dst = smem_u32(ring) + s * stage_bytes;
          for (int r = 0; r < MB; ++r) tma_load_2d_pair(dst + r * A_SUB, &tmap_x, full, kb * BK, m0 + r * 256);
          tma_load_2d_pair(dst + MB * A_SUB, &tmap_w, full, kb * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ product issuer (leader CTA)
    if (lane == 0 && rank == 0 && !*abort_flag) {
      const uint32_t idesc = make_idesc(Fmt<T>::id, 0, (uint32_t)BN, 256);
      // descriptor words: start address in 16-byte units | leading offset 16 B; stride 1024 B between
      // 8-row groups, descriptor version, 128-byte swizzle
      const uint32_t desc_hi = 64u | (1u << 14) | (2u << 29);
      const uint32_t ring_lo = (smem_u32(ring) >> 4) | (1u << 16);
      const uint32_t stage_units = (uint32_t)stage_bytes >> 4, b_units = (uint32_t)(MB * A_SUB) >> 4;
      int s = 0, n = 0;
      uint32_t full_parity = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += n_pairs, ++n) {
        const int acc = n % AS;
        if (n >= AS) ok = wait_or_abort(bar(ACC_EMPTY + acc), (uint32_t)(((n / AS) - 1) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(acc * MB * acc_cols), d1 = d0 + (uint32_t)acc_cols;
        const int ks = t / mn_tiles, kb_begin = ks * k_per, kb_end = min(k_blocks, (ks + 1) * k_per);
        for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
          ok = wait_or_abort(bar(FULL + s), full_parity, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = ring_lo + (uint32_t)s * stage_units;
          issue_kblock<MB>(d0, d1, a_lo, a_lo + b_units, desc_hi, idesc, kb > kb_begin ? 1u : 0u);
          // the group of stages is free in both CTAs once these products have read it
          if ((s & (G - 1)) == G - 1) mma_commit_pair(bar(EMPTY + s / G));
          if (++s == S) {
            s = 0;
            full_parity ^= 1u;
          }
        }
        if (ok) mma_commit_pair(bar(ACC_FULL + acc));   // accumulator complete, in both CTAs
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    // eight warps: warps w and w + 4 share the TMEM lane quadrant w % 4 (the only lanes either may
    // access) and take alternate 32-column groups of the accumulator
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t acc_empty0 = map_to_cta(bar(ACC_EMPTY), 0);
    int n = 0;
    bool ok = !*abort_flag;
    for (int t = pair; t < total && ok; t += n_pairs, ++n) {
      const int tt = t % mn_tiles, ks = t / mn_tiles;
      const int mt = tt % m_tiles, nt = tt / m_tiles;
      const int acc = n % AS;
      ok = wait_or_abort(bar(ACC_FULL + acc), (uint32_t)((n / AS) & 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int n0 = nt * BN;
      const int cols = min(BN, p.N - n0);          // a multiple of 16
      for (int r = 0; r < MB; ++r) {
        const int m = mt * rows_per_tile + r * 256 + (int)rank * 128 + row;
        const bool live = m < p.M;
        const uint32_t t_acc = t_lane + (uint32_t)((acc * MB + r) * acc_cols);
        int64_t pos = -1;
        int slot = -1;
        if (EPI == EPI_QKV && live) {
          pos = p.positions[m];
          if (pos < 0 || pos >= p.rope_rows) {
            if (p.err_flag) atomicExch(p.err_flag, 2);
            pos = -1;
          }
          slot = p.slots[m];
          if (slot < -1 || slot >= p.num_slots) {
            if (p.err_flag) atomicExch(p.err_flag, 1);
            slot = -1;
          }
        }
        float run_max = -INFINITY, run_sum = 0.f;
        int run_arg = 0;
#pragma unroll 1
        for (int c = chalf * 32; c < cols; c += 64) {
          uint32_t v0[16], v1[16];
          const bool two = c + 16 < cols;
          tmem_ld16(t_acc + c, v0);
          if (two) tmem_ld16(t_acc + c + 16, v1);
          tmem_wait_ld();
          if (!live) continue;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (half == 1 && !two) break;
            const float* v = reinterpret_cast<const float*>(half == 0 ? v0 : v1);
            const int nn = n0 + c + half * 16;
            if (EPI == EPI_PLAIN) epi_plain<T>(p, m, nn, v);
            if (EPI == EPI_PARTIAL) epi_partial(p, ks, m, nn, v);
            if (EPI == EPI_SWIGLU) epi_swiglu<T>(p, m, nn, v);
            if (EPI == EPI_QKV) epi_qkv<T, TR, TC>(p, m, nn, v, pos, slot);
            if (EPI == EPI_ARGMAX) {
              // logits as the unfused projection leaves them (rounded to T); first maximum wins
              float x[16], mx = -INFINITY;
              int am = 0;
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                x[i] = round_to<T>(v[i]);
                if (x[i] > mx) {
                  mx = x[i];
                  am = i;
                }
              }
              if (mx > run_max) {
                run_sum *= __expf(run_max - mx);
                run_max = mx;
                run_arg = nn + am;
              }
#pragma unroll
              for (int i = 0; i < 16; ++i) run_sum += __expf(x[i] - run_max);
            }
          }
        }
        if (EPI == EPI_ARGMAX && live) {
          const int64_t idx = (int64_t)(nt * 2 + chalf) * p.M + m;
          p.part_max[idx] = run_max;
          p.part_arg[idx] = run_arg;
          p.part_sum[idx] = run_sum;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + (uint32_t)acc * 8u);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the other CTA no longer reads this CTA's shared memory or barriers
  if (tid == 0 && *abort_flag && p.err_flag) atomicExch(p.err_flag, misplaced ? 6 : 5);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- the second step of the fused output head: fold the per-tile statistics of every row into
// its arg-max and its confidence exp(max - logsumexp) ---------------------------------------------
__global__ void __launch_bounds__(128) argmax_fold_kernel(const float* __restrict__ part_max,
                                                          const int32_t* __restrict__ part_arg,
                                                          const float* __restrict__ part_sum, int n_parts, int M,
                                                          int64_t* __restrict__ x0, float* __restrict__ conf) {
  // one warp per row; the lanes stride over the row's partial results, then fold by shuffles.
  // Among equal maxima the lowest column wins, whatever order the parts are met in.
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  float mx = -INFINITY, sum = 0.f;
  int arg = 0x7FFFFFFF;
  auto fold = [&](float pm, int pa, float ps) {
    if (pm > mx || (pm == mx && pa < arg)) {
      sum = (mx == -INFINITY ? 0.f : sum * __expf(mx - pm)) + ps;
      mx = pm;
      arg = pa;
    } else if (pm != -INFINITY) {
      sum += ps * __expf(pm - mx);
    }
  };
  for (int t = lane; t < n_parts; t += 32)
    fold(part_max[(int64_t)t * M + m], part_arg[(int64_t)t * M + m], part_sum[(int64_t)t * M + m]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float pm = __shfl_xor_sync(0xFFFFFFFFu, mx, o);
    const int pa = __shfl_xor_sync(0xFFFFFFFFu, arg, o);
    const float ps = __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    fold(pm, pa, ps);
  }
  if (lane == 0) {
    x0[m] = arg;
    conf[m] = 1.0f / sum;      // exp(max - logsumexp) = 1 / sum exp(x - max)
  }
}

// ---------------------------------------------------------------------------------------- host
struct Tile { int mb, bn, stages, acc_stages; size_t smem; };

// Time of a launch ~ waves of the 74 pairs x k blocks x time of one k block of one pair.  Measured
// on B200 (bf16, operands streaming from L2): a k block is bound by the operand bytes a CTA pulls
// from L2 -- about 68 GB/s per SM with one row block per CTA (32 KB stages, 6 of them), 57 GB/s with
// two (48 KB stages, 4 of them) -- and not faster than 0.47 us (one row block) / 0.6 us (two) whatever
// the tile's width (product issue, commits, the tensor pipe at about 94 ns per 256-row product).
// A tile whose epilogue cannot overlap the next tile's products (one accumulator stage) pays for it
// by `exposed` (1.03 for a plain store ... 1.25 for the QKV epilogue).
static Tile pick_tile(int M, int N, int want_mb, int want_bn, int bn_multiple, double exposed) {
  double best = 1e30;
  Tile out{1, 128, 4, 2, 0};
  for (int mb = 1; mb <= 2; ++mb) {
    if (want_mb && mb != want_mb) continue;
    if (!want_mb && mb == 2 && M <= 256) continue;
    const int m_tiles = (M + 256 * mb - 1) / (256 * mb);
    for (int bn = 256; bn >= 64; bn -= 16) {
      if (want_bn && bn != want_bn) continue;
      if (bn % bn_multiple != 0) continue;
      const int acc_cols = (bn + 31) & ~31;
      if (mb * acc_cols > 512) continue;
      const int n_tiles = (N + bn - 1) / bn;
      const long tiles = (long)m_tiles * n_tiles;
      const long waves = (tiles + kPairs - 1) / kPairs;
      const int acc_stages = 2 * mb * acc_cols <= 512 ? 2 : 1;
      const int stage_bytes = mb * A_SUB + (bn / 2) * BK * 2;
      const double load_ns = stage_bytes / (mb == 1 ? 68.0 : 57.0), floor_ns = mb == 1 ? 470.0 : 600.0;
      const double cost = (double)waves * (load_ns > floor_ns ? load_ns : floor_ns) * (acc_stages == 1 ? exposed : 1.0);
      if (cost < best - 1e-9) {      // candidates run from wide to narrow: among equals the widest stays
        best = cost;
        int stages = (int)((200 * 1024) / stage_bytes);
        if (stages > kMaxStages) stages = kMaxStages;
        out = Tile{mb, bn, stages, acc_stages, (size_t)stages * stage_bytes + 512};
      }
    }
  }
  return out;
}

template <typename T, typename TR, typename TC, int EPI, int MB>
static int launch_mb(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, const Tile& tile, cudaStream_t st) {
  auto kern = linear_tc_kernel<T, TR, TC, EPI, MB>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile.smem));
  const int m_tiles = (p.M + 256 * p.MB - 1) / (256 * p.MB), n_tiles = (p.N + p.BN - 1) / p.BN;
  const long total = (long)m_tiles * n_tiles * p.ksplit;
  const int pairs = total < kPairs ? (int)total : kPairs;
  ACACHE_CUDA_CHECK(launch_chained(kern, dim3(2 * pairs), dim3(NT), tile.smem, st, mx, mw, p));
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR, typename TC, int EPI>
static int launch(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, const Tile& tile, cudaStream_t st) {
  if (p.MB == 2) return launch_mb<T, TR, TC, EPI, 2>(mx, mw, p, tile, st);
  return launch_mb<T, TR, TC, EPI, 1>(mx, mw, p, tile, st);
}

template <typename T, typename TR> struct PromoteG { using type = float; };
template <> struct PromoteG<__half, __half> { using type = __half; };
template <> struct PromoteG<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

static int prepare(const void* x, int64_t ldx, const void* w, int M, int N, int K, int dtype, int tile_mb, int tile_bn,
                   double exposed, Params* p, Tile* tile, CUtensorMap* mx, CUtensorMap* mw) {
  if (dtype != ACACHE_BF16 && dtype != ACACHE_F16) return ACACHE_EUNSUPPORTED;
  if (M <= 0 || N <= 0 || K <= 0 || N % 16 != 0 || K % 8 != 0 || ldx % 8 != 0) return ACACHE_EUNSUPPORTED;
  if (!aligned16(x) || !aligned16(w)) return ACACHE_EUNSUPPORTED;
  if ((tile_mb != 0 && tile_mb != 1 && tile_mb != 2) || (tile_bn != 0 && (tile_bn % 16 != 0 || tile_bn < 32 || tile_bn > 256)))
    return ACACHE_EINVAL;
  *tile = pick_tile(M, N, tile_mb, tile_bn, 16, exposed);
  if (tile->smem == 0) return ACACHE_EUNSUPPORTED;
  p->M = M; p->N = N; p->K = K; p->MB = tile->mb; p->BN = tile->bn; p->stages = tile->stages;
  p->acc_stages = tile->acc_stages;
  p->ksplit = 1;
  // `tcgen05.commit` costs the issuing thread a few hundred cycles: with one row block per CTA (6
  // or more stages) two stages are handed back per commit; with two row blocks there are only 4
  // stages and handing them back one by one keeps the loads further ahead
  p->group = tile->mb == 1 ? 2 : 1;
  if (p->group == 2 && (p->stages & 1)) p->stages -= 1;
  if (!make_tensor_map_2d(mx, x, M, K, ldx, 128, dtype) || !make_tensor_map_2d(mw, w, N, K, K, tile->bn / 2, dtype))
    return ACACHE_EUNSUPPORTED;
  return ACACHE_OK;
}

// Slices of the K range for a projection whose whole tiles (256 rows x 256 columns per pair) would
// occupy at most half of the 74 pairs: as many as still run in one wave, at most 4.  Measured on
// B200 (bf16, 4096 output columns): 512 rows, K = 4096: 22 us with 2 slices against 31 us whole;
// K = 12288: 46 against 73 us; 256 rows, K = 12288: 31 us with 4 slices against 72 us; more slices
// only add fp32 traffic.  Pipeline fill, the fp32 epilogue and the slices' extra traffic in the
// consumer cost a sliced launch 6-9 us whatever K, so a slice gets at least 48 k blocks; shorter
// K ranges are not sliced (return 1) and the caller takes a whole-tile GEMM.
static int plan_splits(int M, int N, int K) {
  const long tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
  const int k_blocks = (K + BK - 1) / BK;
  long s = kPairs / tiles;
  if (s > 4) s = 4;
  while (s > 1 && (k_blocks / s < 48 || (s - 1) * ((k_blocks + s - 1) / s) >= k_blocks)) --s;
  return s < 2 ? 1 : (int)s;
}

}  // namespace gemm
}  // namespace acache

using namespace acache;

extern "C" int acache_linear_partials_splits(int n_rows, int in_features, int out_features) {
  if (n_rows <= 0 || in_features <= 0 || out_features <= 0) return 1;
  return gemm::plan_splits(n_rows, out_features, in_features);
}

extern "C" int acache_linear_partials(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                                      int out_features, int dtype, float* partials, int n_splits, int tile_mb,
                                      int tile_bn, int32_t* err_flag, void* stream) {
  if (n_splits < 0 || n_splits > 16) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !weight || !partials) return ACACHE_EINVAL;
  if (n_splits == 0) n_splits = gemm::plan_splits(n_rows, out_features, in_features);
  const int k_blocks = (in_features + gemm::BK - 1) / gemm::BK;
  if ((n_splits - 1) * ((k_blocks + n_splits - 1) / n_splits) >= k_blocks) return ACACHE_EINVAL;   // an empty slice
  gemm::Params p{};
  gemm::Tile tile;
  CUtensorMap mx, mw;
  const int rc = gemm::prepare(x, x_stride, weight, n_rows, out_features, in_features, dtype, tile_mb ? tile_mb : 1,
                               tile_bn ? tile_bn : 256, 1.0, &p, &tile, &mx, &mw);
  if (rc != ACACHE_OK) return rc;
  if (!aligned16(partials)) return ACACHE_EUNSUPPORTED;
  p.partial = partials; p.ksplit = n_splits; p.err_flag = err_flag;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ACACHE_BF16) return gemm::launch<__nv_bfloat16, float, float, gemm::EPI_PARTIAL>(mx, mw, p, tile, st);
  return gemm::launch<__half, float, float, gemm::EPI_PARTIAL>(mx, mw, p, tile, st);
}

extern "C" int acache_linear(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                             int out_features, const void* bias, int dtype, void* out, int64_t out_stride,
                             int tile_mb, int tile_bn, int32_t* err_flag, void* stream) {
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !weight || !out) return ACACHE_EINVAL;
  gemm::Params p{};
  gemm::Tile tile;
  CUtensorMap mx, mw;
  const int rc = gemm::prepare(x, x_stride, weight, n_rows, out_features, in_features, dtype, tile_mb, tile_bn, 1.03, &p,
                               &tile, &mx, &mw);
  if (rc != ACACHE_OK) return rc;
  if (!aligned16(out) || out_stride % 8 != 0 || (bias && !aligned16(bias))) return ACACHE_EUNSUPPORTED;
  p.out = out; p.ldo = out_stride; p.bias = bias; p.err_flag = err_flag;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ACACHE_BF16) return gemm::launch<__nv_bfloat16, float, float, gemm::EPI_PLAIN>(mx, mw, p, tile, st);
  return gemm::launch<__half, float, float, gemm::EPI_PLAIN>(mx, mw, p, tile, st);
}

extern "C" int acache_linear_swiglu(const void* x, int64_t x_stride, int n_rows, int in_features,
                                    const void* weight_gate_up, int ffn_features, int act, int dtype, void* out,
                                    int64_t out_stride, int tile_mb, int tile_bn, int32_t* err_flag, void* stream) {
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !weight_gate_up || !out || act < 0 || act > 2) return ACACHE_EINVAL;
  if (ffn_features % 8 != 0) return ACACHE_EUNSUPPORTED;
  gemm::Params p{};
  gemm::Tile tile;
  CUtensorMap mx, mw;
  const int rc = gemm::prepare(x, x_stride, weight_gate_up, n_rows, 2 * ffn_features, in_features, dtype, tile_mb,
                               tile_bn, 1.08, &p, &tile, &mx, &mw);
  if (rc != ACACHE_OK) return rc;
  if (!aligned16(out) || out_stride % 8 != 0) return ACACHE_EUNSUPPORTED;
  p.out = out; p.ldo = out_stride; p.act = act; p.err_flag = err_flag;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ACACHE_BF16) return gemm::launch<__nv_bfloat16, float, float, gemm::EPI_SWIGLU>(mx, mw, p, tile, st);
  return gemm::launch<__half, float, float, gemm::EPI_SWIGLU>(mx, mw, p, tile, st);
}

extern "C" int acache_linear_qkv_rope_scatter(const void* x, int64_t x_stride, int n_rows, int hidden,
                                              const void* w_qkv_interleaved, const void* bias_interleaved, int n_heads,
                                              int n_kv_heads, int head_dim, int dtype, const int64_t* positions,
                                              const void* rope_cos, const void* rope_sin, int64_t rope_row_stride,
                                              int rope_rows, int rope_dtype, void* out_q, int64_t q_stride,
                                              void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                              int64_t num_slots, int tile_mb, int tile_bn, int32_t* err_flag,
                                              void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype) || n_rows < 0 || hidden <= 0 || n_heads <= 0 || n_kv_heads <= 0)
    return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !w_qkv_interleaved || !positions || !rope_cos || !rope_sin || !out_q || !k_cache || !v_cache ||
      !slot_mapping)
    return ACACHE_EINVAL;
  if (head_dim != 128) return ACACHE_EUNSUPPORTED;
  gemm::Params p{};
  gemm::Tile tile;
  CUtensorMap mx, mw;
  const int N = (n_heads + 2 * n_kv_heads) * head_dim;
  const int rc = gemm::prepare(x, x_stride, w_qkv_interleaved, n_rows, N, hidden, dtype, tile_mb, tile_bn, 1.25, &p,
                               &tile, &mx, &mw);
  if (rc != ACACHE_OK) return rc;
  const int re = dtype_bytes(rope_dtype);
  if (!aligned16(out_q) || q_stride % 8 != 0 || !aligned16(k_cache) || !aligned16(v_cache) ||
      (bias_interleaved && !aligned16(bias_interleaved)) || !aligned16(rope_cos) || !aligned16(rope_sin) ||
      (rope_row_stride * re) % 16 != 0)
    return ACACHE_EUNSUPPORTED;
  p.bias = bias_interleaved; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.positions = positions;
  p.rope_cos = rope_cos; p.rope_sin = rope_sin; p.rope_stride = rope_row_stride; p.rope_rows = rope_rows;
  p.out_q = out_q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.slots = slot_mapping;
  p.num_slots = num_slots; p.err_flag = err_flag;
  cudaStream_t st = (cudaStream_t)stream;
#define QKV(T, TR) \
  return gemm::launch<T, TR, typename gemm::PromoteG<T, TR>::type, gemm::EPI_QKV>(mx, mw, p, tile, st)
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

extern "C" int64_t acache_linear_argmax_scratch_bytes(int n_rows, int out_features) {
  if (n_rows <= 0 || out_features <= 0) return 0;
  const int64_t parts = 2 * ((out_features + 63) / 64);      // two per column tile; the smallest tile bounds the count
  return parts * n_rows * 12;
}

extern "C" int acache_linear_argmax(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                                    int out_features, int dtype, int64_t* x0, float* confidence, void* scratch,
                                    int64_t scratch_bytes, int tile_mb, int tile_bn, int32_t* err_flag, void* stream) {
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !weight || !x0 || !confidence || !scratch) return ACACHE_EINVAL;
  gemm::Params p{};
  gemm::Tile tile;
  CUtensorMap mx, mw;
  const int rc = gemm::prepare(x, x_stride, weight, n_rows, out_features, in_features, dtype, tile_mb, tile_bn, 1.1, &p,
                               &tile, &mx, &mw);
  if (rc != ACACHE_OK) return rc;
  const int64_t n_parts = 2 * ((out_features + tile.bn - 1) / tile.bn);
  if (scratch_bytes < n_parts * n_rows * 12) return ACACHE_EINVAL;
  p.part_max = (float*)scratch;
  p.part_arg = (int32_t*)((float*)scratch + n_parts * n_rows);
  p.part_sum = (float*)scratch + 2 * n_parts * n_rows;
  p.err_flag = err_flag;
  cudaStream_t st = (cudaStream_t)stream;
  int lrc;
  if (dtype == ACACHE_BF16) lrc = gemm::launch<__nv_bfloat16, float, float, gemm::EPI_ARGMAX>(mx, mw, p, tile, st);
  else lrc = gemm::launch<__half, float, float, gemm::EPI_ARGMAX>(mx, mw, p, tile, st);
  if (lrc != ACACHE_OK) return lrc;
  gemm::argmax_fold_kernel<<<(n_rows + 3) / 4, 128, 0, st>>>(p.part_max, p.part_arg, p.part_sum, (int)n_parts, n_rows,
                                                             x0, confidence);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}
