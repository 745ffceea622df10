// General (any dtype, any head_dim up to 256) varlen attention over a slot-mapped or
// block-table paged cache, fp32 CUDA-core arithmetic.  This is the path for fp32 caches
// and unusual head sizes; bf16/fp16 with head_dim 64/128 is served by the tensor-core
// kernel and only falls through to here when that kernel declines a shape.
//
// CTA = 128 threads = one (request, head, 32-query tile).  K/V tiles of 32 keys are
// gathered through the slot map with 16-byte loads, optionally re-rotated (key-side
// relocation) while being staged in shared memory as fp32.  Thread (i, g) with
// i = tid/4, g = tid%4 owns score columns g*8..g*8+7 of query row i and output
// dimensions g, g+4, g+8, ...
#include <atomic>

#include "common.cuh"

namespace acache {

constexpr int kBM = 32, kBN = 32, kThreads = 128;

struct KvAddr {
  const int32_t* slot_map;      // flat slots (slot-map mode) or nullptr
  const int32_t* block_table;   // row of this request (block-table mode)
  int block_size;
  __device__ __forceinline__ int64_t slot(int j) const {
    if (slot_map) return slot_map[j];
    const int b = block_table[j / block_size];
    return b < 0 ? -2 : (int64_t)b * block_size + j % block_size;
  }
};

// Stage rows [j0, j0 + kBN) of K (optionally rotated) and V into shared memory as fp32.
// A slot of -1 marks a key that takes no part (its row is zeroed and dead[row] is set);
// any other slot outside the cache is an error (flagged, treated the same way).
template <typename T, typename TR, typename TC, bool WITH_V>
__device__ __forceinline__ void stage_kv_tile(float* Ks, float* Vs, int ldk, int ldv, const T* __restrict__ k_cache,
                                              const T* __restrict__ v_cache, int64_t num_slots, int kv_row,
                                              int head_off, int D, const KvAddr& addr, int j0, int j_end,
                                              int rot_mode /*0 none, 1 key-side by (j - slot), 2 fixed row*/,
                                              int shared_prefix_len, int fixed_row, const TR* __restrict__ rope_cos,
                                              const TR* __restrict__ rope_sin, int64_t rope_stride, int rope_rows,
                                              int32_t* err_flag, int* dead = nullptr) {
  constexpr int E = 16 / sizeof(T);
  const int half = D / 2;
  const int cph = half / E;
  for (int it = threadIdx.x; it < kBN * cph; it += kThreads) {
    const int jj = it / cph;
    const int d = (it - jj * cph) * E;
    const int j = j0 + jj;
    float k1[E], k2[E], v1[E], v2[E];
    bool ok = j < j_end;
    int64_t slot = 0;
    if (ok) {
      slot = addr.slot(j);
      if (slot < 0 || slot >= num_slots) {
        if (slot != -1 && err_flag) atomicExch(err_flag, 3);
        ok = false;
      }
    }
    if (dead && d == 0) dead[jj] = ok ? 0 : 1;
    if (ok) {
      const T* kp = k_cache + slot * kv_row + head_off + d;
      Vec16<T> a, b;
      a.u = *reinterpret_cast<const uint4*>(kp);
      b.u = *reinterpret_cast<const uint4*>(kp + half);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        k1[e] = to_f32<T>(a.e[e]);
        k2[e] = to_f32<T>(b.e[e]);
      }
      int row = -1;
      bool neg = false;
      if (rot_mode == 1 && slot < shared_prefix_len) {
        const int64_t delta = (int64_t)j - slot;
        neg = delta < 0;
        row = (int)(neg ? -delta : delta);
      } else if (rot_mode == 2) {
        row = fixed_row;
      }
      if (row >= 0) {
        if (row >= rope_rows) {
          if (err_flag) atomicExch(err_flag, 4);
        } else {
          const TR* cr = rope_cos + (int64_t)row * rope_stride;
          const TR* sr = rope_sin + (int64_t)row * rope_stride;
#pragma unroll
          for (int e = 0; e < E; ++e) {
            float s1 = to_f32<TR>(sr[d + e]), s2 = to_f32<TR>(sr[d + half + e]);
            if (neg) { s1 = -s1; s2 = -s2; }
            const float o1 = rot_lo<TC>(k1[e], k2[e], to_f32<TR>(cr[d + e]), s1);
            const float o2 = rot_hi<TC>(k1[e], k2[e], to_f32<TR>(cr[d + half + e]), s2);
            k1[e] = round_to<T>(o1);
            k2[e] = round_to<T>(o2);
          }
        }
      }
      if (WITH_V) {
        const T* vp = v_cache + slot * kv_row + head_off + d;
        a.u = *reinterpret_cast<const uint4*>(vp);
        b.u = *reinterpret_cast<const uint4*>(vp + half);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          v1[e] = to_f32<T>(a.e[e]);
          v2[e] = to_f32<T>(b.e[e]);
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) k1[e] = k2[e] = v1[e] = v2[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      Ks[jj * ldk + d + e] = k1[e];
      Ks[jj * ldk + d + half + e] = k2[e];
      if (WITH_V) {
        Vs[jj * ldv + d + e] = v1[e];
        Vs[jj * ldv + d + half + e] = v2[e];
      }
    }
  }
}

// scores of query row i against the 8 keys g*8..g*8+7 of the staged tile
__device__ __forceinline__ void score_row(const float* Qs, const float* Ks, int ld, int D, int i, int g, float* s) {
#pragma unroll
  for (int c = 0; c < 8; ++c) s[c] = 0.f;
  const float* qr = Qs + i * ld;
  const float* kr = Ks + (g * 8) * ld;
  for (int d = 0; d < D; ++d) {
    const float qv = qr[d];
#pragma unroll
    for (int c = 0; c < 8; ++c) s[c] = fmaf(qv, kr[c * ld + d], s[c]);
  }
}

template <typename T, typename TR, typename TC, int DMAX>
__global__ void __launch_bounds__(kThreads) attention_simt_kernel(
    const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t o_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, int64_t num_slots, int n_heads, int n_kv_heads, int D,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ slot_map,
    const int32_t* __restrict__ block_tables, int table_stride, int block_size, float scale, int shared_prefix_len,
    const int32_t* __restrict__ shared_kv_lens, const int32_t* __restrict__ affix_shifts,
    const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin, int64_t rope_stride, int rope_rows,
    int32_t* err_flag) {
  constexpr int DPT = DMAX / 4;
  extern __shared__ float smem[];
  const int ld = D + 1;
  float* Qs = smem;                 // [kBM][ld]
  float* Qr = Qs + kBM * ld;        // [kBM][ld] inverse-rotated queries (query-side mode)
  float* Ks = Qr + kBM * ld;        // [kBN][ld]
  float* Vs = Ks + kBN * ld;        // [kBN][D]
  float* Ps = Vs + kBN * D;         // [kBM][kBN+1]
  int* dead = reinterpret_cast<int*>(Ps + kBM * (kBN + 1));  // [kBN] keys of the tile that take no part

  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
  const int m0 = blockIdx.x * kBM;
  if (m0 >= q_len) return;
  const int kv0 = cu_k[b], kv_len = cu_k[b + 1] - kv0;
  const int tid = threadIdx.x, i = tid >> 2, g = tid & 3;
  const int kvh = h / (n_heads / n_kv_heads);
  const int kv_row = n_kv_heads * D;
  const bool relocate = shared_prefix_len > 0 && affix_shifts != nullptr;
  const bool query_side = relocate && shared_kv_lens != nullptr;

  // stage queries (and their inverse rotation for query-side relocation)
  const int shift = query_side ? affix_shifts[b] : 0;
  if (query_side && (shift < 0 || shift >= rope_rows)) {
    if (err_flag && tid == 0) atomicExch(err_flag, 4);
    return;
  }
  for (int it = tid; it < kBM * (D / 2); it += kThreads) {
    const int r = it / (D / 2), d = it - r * (D / 2);
    float x1 = 0.f, x2 = 0.f;
    if (m0 + r < q_len) {
      const T* qp = q + (int64_t)(q0 + m0 + r) * q_stride + (int64_t)h * D;
      x1 = to_f32<T>(qp[d]);
      x2 = to_f32<T>(qp[d + D / 2]);
    }
    Qs[r * ld + d] = x1;
    Qs[r * ld + d + D / 2] = x2;
    if (query_side) {
      const TR* cr = rope_cos + (int64_t)shift * rope_stride;
      const TR* sr = rope_sin + (int64_t)shift * rope_stride;
      // q*cos - rotate_half(q)*sin
      const float o1 = rot_lo<TC>(x1, x2, to_f32<TR>(cr[d]), -to_f32<TR>(sr[d]));
      const float o2 = rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + D / 2]), -to_f32<TR>(sr[d + D / 2]));
      Qr[r * ld + d] = round_to<T>(o1);
      Qr[r * ld + d + D / 2] = round_to<T>(o2);
    }
  }

  KvAddr addr;
  addr.slot_map = slot_map ? slot_map + kv0 : nullptr;
  addr.block_table = block_tables ? block_tables + (int64_t)b * table_stride : nullptr;
  addr.block_size = block_size;

  float acc[DPT];
#pragma unroll
  for (int c = 0; c < DPT; ++c) acc[c] = 0.f;
  float m_i = -INFINITY, l_i = 0.f;

  const int n_shared = query_side ? min(max(shared_kv_lens[b], 0), kv_len) : 0;
  // two key ranges: [0, n_shared) scored with the rotated queries, [n_shared, kv_len) with the plain ones
  for (int part = 0; part < 2; ++part) {
    const int j_begin = part == 0 ? 0 : n_shared;
    const int j_end = part == 0 ? n_shared : kv_len;
    const float* Qp = part == 0 ? Qr : Qs;
    for (int j0 = j_begin; j0 < j_end; j0 += kBN) {
      __syncthreads();
      stage_kv_tile<T, TR, TC, true>(Ks, Vs, ld, D, k_cache, v_cache, num_slots, kv_row, kvh * D, D, addr, j0, j_end,
                                     (relocate && !query_side) ? 1 : 0, shared_prefix_len, 0, rope_cos, rope_sin,
                                     rope_stride, rope_rows, err_flag, dead);
      __syncthreads();
      float s[8];
      score_row(Qp, Ks, ld, D, i, g, s);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        s[c] = dead[g * 8 + c] ? -INFINITY : s[c] * scale;
        mx = fmaxf(mx, s[c]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const float m_new = fmaxf(m_i, mx);
      const float alpha = (m_i == -INFINITY) ? 0.f : __expf(m_i - m_new);
      float rs = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float p = (s[c] == -INFINITY) ? 0.f : __expf(s[c] - m_new);
        Ps[i * (kBN + 1) + g * 8 + c] = p;
        rs += p;
      }
      rs += __shfl_xor_sync(0xFFFFFFFFu, rs, 1);
      rs += __shfl_xor_sync(0xFFFFFFFFu, rs, 2);
      l_i = l_i * alpha + rs;
      m_i = m_new;
      __syncwarp();  // the 4 threads of a row sit in one warp; Ps row i is written and read by them only
#pragma unroll
      for (int c = 0; c < DPT; ++c) acc[c] *= alpha;
      for (int jj = 0; jj < kBN; ++jj) {
        const float p = Ps[i * (kBN + 1) + jj];
        const float* vr = Vs + jj * D;
#pragma unroll
        for (int c = 0; c < DPT; ++c) {
          const int d = g + 4 * c;
          if (d < D) acc[c] = fmaf(p, vr[d], acc[c]);
        }
      }
    }
  }
  if (m0 + i < q_len) {
    const float inv = l_i > 0.f ? 1.f / l_i : 0.f;
    T* op = out + (int64_t)(q0 + m0 + i) * o_stride + (int64_t)h * D;
#pragma unroll
    for (int c = 0; c < DPT; ++c) {
      const int d = g + 4 * c;
      if (d < D) op[d] = from_f32<T>(acc[c] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------
// Anchor influence score, one layer, one request.  CTA = (32-row tile of mask queries,
// head).  Pass 1 finds each row's softmax max and denominator over the whole affix,
// pass 2 recomputes the scores and writes the column sums of exp(s - m)/l of this CTA to
// its own row of `partial`; importance_reduce_kernel adds the rows in a fixed order.
template <typename T, typename TR, typename TC>
__global__ void __launch_bounds__(kThreads) importance_partial_kernel(
    const T* __restrict__ q, int64_t q_stride, const int32_t* __restrict__ q_rows, int n_q, int n_heads, int n_kv_heads,
    int D, const T* __restrict__ affix_k, int64_t k_slot_stride, int affix_len, int affix_shift,
    const TR* __restrict__ rope_cos, const TR* __restrict__ rope_sin, int64_t rope_stride, int rope_rows, float scale,
    float* __restrict__ partial) {
  extern __shared__ float smem[];
  const int ld = D + 1;
  float* Qs = smem;            // [kBM][ld]
  float* Ks = Qs + kBM * ld;   // [kBN][ld]
  float* Ps = Ks + kBN * ld;   // [kBM][kBN+1]
  const int h = blockIdx.y;
  const int m0 = blockIdx.x * kBM;
  const int tid = threadIdx.x, i = tid >> 2, g = tid & 3;
  const int kvh = h / (n_heads / n_kv_heads);
  for (int it = tid; it < kBM * D; it += kThreads) {
    const int r = it / D, d = it - r * D;
    float x = 0.f;
    if (m0 + r < n_q) x = to_f32<T>(q[(int64_t)q_rows[m0 + r] * q_stride + (int64_t)h * D + d]);
    Qs[r * ld + d] = x;
  }
  KvAddr addr;  // affix keys are the consecutive slots 0..A-1: identity block table of size A
  addr.slot_map = nullptr;
  addr.block_table = nullptr;
  addr.block_size = 1;
  const bool row_ok = m0 + i < n_q;
  float m_i = -INFINITY, l_i = 0.f;
  float* my_partial = partial + ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * affix_len;
  for (int pass = 0; pass < 2; ++pass) {
    const float inv_l = (pass == 1 && l_i > 0.f) ? 1.f / l_i : 0.f;
    for (int j0 = 0; j0 < affix_len; j0 += kBN) {
      __syncthreads();
      // stage keys j0.. of kv head kvh, rotated by the fixed table row affix_shift
      {
        constexpr int E = 16 / sizeof(T);
        const int half = D / 2, cph = half / E;
        for (int it = tid; it < kBN * cph; it += kThreads) {
          const int jj = it / cph, d = (it - jj * cph) * E;
          const int j = j0 + jj;
          float k1[E], k2[E];
          if (j < affix_len) {
            const T* kp = affix_k + (int64_t)j * k_slot_stride + (int64_t)kvh * D + d;
            Vec16<T> a, b;
            a.u = *reinterpret_cast<const uint4*>(kp);
            b.u = *reinterpret_cast<const uint4*>(kp + half);
            const TR* cr = rope_cos + (int64_t)affix_shift * rope_stride;
            const TR* sr = rope_sin + (int64_t)affix_shift * rope_stride;
#pragma unroll
            for (int e = 0; e < E; ++e) {
              const float x1 = to_f32<T>(a.e[e]), x2 = to_f32<T>(b.e[e]);
              if (affix_shift != 0) {
                k1[e] = round_to<T>(rot_lo<TC>(x1, x2, to_f32<TR>(cr[d + e]), to_f32<TR>(sr[d + e])));
                k2[e] = round_to<T>(rot_hi<TC>(x1, x2, to_f32<TR>(cr[d + half + e]), to_f32<TR>(sr[d + half + e])));
              } else {
                k1[e] = x1;
                k2[e] = x2;
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < E; ++e) k1[e] = k2[e] = 0.f;
          }
#pragma unroll
          for (int e = 0; e < E; ++e) {
            Ks[jj * ld + d + e] = k1[e];
            Ks[jj * ld + d + half + e] = k2[e];
          }
        }
      }
      __syncthreads();
      float s[8];
      score_row(Qs, Ks, ld, D, i, g, s);
#pragma unroll
      for (int c = 0; c < 8; ++c) s[c] = (j0 + g * 8 + c < affix_len) ? s[c] * scale : -INFINITY;
      if (pass == 0) {
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; ++c) mx = fmaxf(mx, s[c]);
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float m_new = fmaxf(m_i, mx);
        float rs = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) rs += (s[c] == -INFINITY) ? 0.f : __expf(s[c] - m_new);
        rs += __shfl_xor_sync(0xFFFFFFFFu, rs, 1);
        rs += __shfl_xor_sync(0xFFFFFFFFu, rs, 2);
        l_i = l_i * ((m_i == -INFINITY) ? 0.f : __expf(m_i - m_new)) + rs;
        m_i = m_new;
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          Ps[i * (kBN + 1) + g * 8 + c] = (row_ok && s[c] != -INFINITY) ? __expf(s[c] - m_i) * inv_l : 0.f;
        __syncthreads();
        if (tid < kBN && j0 + tid < affix_len) {
          float cs = 0.f;
          for (int r = 0; r < kBM; ++r) cs += Ps[r * (kBN + 1) + tid];
          my_partial[j0 + tid] = cs;
        }
      }
    }
  }
}

// blockIdx.y = request of a batched launch: its partial rows follow those of the requests before
// it, its scores are `importance_stride` floats further on
__global__ void importance_reduce_kernel(const float* __restrict__ partial, int n_partials, int affix_len,
                                         float* __restrict__ importance, int64_t importance_stride = 0) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= affix_len) return;
  partial += (int64_t)blockIdx.y * n_partials * affix_len;
  float s = 0.f;
  for (int p = 0; p < n_partials; ++p) s += partial[(int64_t)p * affix_len + a];
  importance[(int64_t)blockIdx.y * importance_stride + a] += s;
}

template <typename T, typename TR> struct PromoteA { using type = float; };
template <> struct PromoteA<__half, __half> { using type = __half; };
template <> struct PromoteA<__nv_bfloat16, __nv_bfloat16> { using type = __nv_bfloat16; };

template <typename T, typename TR, int DMAX>
static int launch_attention_simt(const AttnArgs& a) {
  using TC = typename PromoteA<T, TR>::type;
  const int D = a.head_dim, ld = D + 1;
  const size_t smem = sizeof(float) * ((size_t)2 * kBM * ld + (size_t)kBN * ld + (size_t)kBN * D + (size_t)kBM * (kBN + 1) + kBN);
  auto kern = attention_simt_kernel<T, TR, TC, DMAX>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((a.max_q + kBM - 1) / kBM, a.batch, a.n_heads);
  kern<<<grid, kThreads, smem, a.st>>>((const T*)a.q, a.q_stride, (T*)a.out, a.o_stride, (const T*)a.k_cache,
                                       (const T*)a.v_cache, a.num_slots, a.n_heads, a.n_kv_heads, D, a.cu_q, a.cu_k,
                                       a.slot_map, a.block_tables, a.table_stride, a.block_size, a.scale,
                                       a.shared_prefix_len, a.shared_kv_lens, a.affix_shifts, (const TR*)a.rope_cos,
                                       (const TR*)a.rope_sin, a.rope_stride, a.rope_rows, a.err_flag);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

template <typename T, typename TR>
static int dispatch_dmax(const AttnArgs& a) {
  if (a.head_dim <= 64) return launch_attention_simt<T, TR, 64>(a);
  if (a.head_dim <= 128) return launch_attention_simt<T, TR, 128>(a);
  if (a.head_dim <= 256) return launch_attention_simt<T, TR, 256>(a);
  return ACACHE_EUNSUPPORTED;
}

int attention_simt_dispatch(const AttnArgs& a, int dtype, int rope_dtype) {
  const int E = 16 / dtype_bytes(dtype);
  if (a.head_dim % (2 * E) != 0 || !aligned16(a.k_cache) || !aligned16(a.v_cache)) return ACACHE_EUNSUPPORTED;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (rope_dtype == ACACHE_F32) return dispatch_dmax<T, float>(a);
    if (rope_dtype == ACACHE_F16) return dispatch_dmax<T, __half>(a);
    return dispatch_dmax<T, __nv_bfloat16>(a);
  });
  return ACACHE_EINVAL;
}

// implemented in importance_tc.cu
int importance_tc_dispatch(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q, int n_heads, int n_kv_heads,
                           int head_dim, int dtype, const void* affix_k, int64_t k_slot_stride, int affix_len,
                           int affix_shift, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                           int rope_dtype, float scale, float* partial, int* n_partials, float* ml, int32_t* err_flag,
                           cudaStream_t st);
int64_t importance_tc_ml_floats(int n_q_rows, int n_heads, int affix_len);
int importance_tc_batched_dispatch(const void* q, int64_t q_stride, const int32_t* q_rows, const int32_t* req_off,
                                   int n_requests, int max_q, int n_heads, int n_kv_heads, int head_dim, int dtype,
                                   const void* affix_k, int64_t k_slot_stride, int affix_len, const int32_t* req_shift,
                                   const void* rope_cos, const void* rope_sin, int64_t rope_stride, int rope_rows,
                                   int rope_dtype, float scale, float* partial, int* n_partials, int32_t* err_flag,
                                   cudaStream_t st);

// implemented in attention_tc.cu: returns ACACHE_EUNSUPPORTED when it declines the shape
int attention_tc_dispatch(const AttnArgs& a, int dtype, int rope_dtype);
int attention_split_dispatch(const AttnArgs& a, int dtype, int rope_dtype, int total_q, void* scratch,
                             int64_t scratch_bytes);
int64_t attention_split_scratch_bytes(int total_q, int n_heads, int head_dim, int batch, int n_kv_heads);

}  // namespace acache

using namespace acache;

static int attention_common(AttnArgs& a, int dtype, int rope_dtype) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (a.batch < 0 || a.n_heads <= 0 || a.n_kv_heads <= 0 || a.head_dim <= 0 || a.n_heads % a.n_kv_heads != 0)
    return ACACHE_EINVAL;
  if (a.batch == 0 || a.max_q <= 0) return ACACHE_OK;
  if (!a.q || !a.out || !a.k_cache || !a.v_cache || !a.cu_q || !a.cu_k) return ACACHE_EINVAL;
  const bool relocate = a.shared_prefix_len > 0 && a.affix_shifts != nullptr;
  if (relocate && (!a.rope_cos || !a.rope_sin || a.rope_rows <= 0)) return ACACHE_EINVAL;
  int rc = attention_tc_dispatch(a, dtype, rope_dtype);
  if (rc != ACACHE_EUNSUPPORTED) return rc;
  return attention_simt_dispatch(a, dtype, rope_dtype);
}

extern "C" int acache_attention(const void* q, int64_t q_stride, void* out, int64_t o_stride, const void* k_cache,
                                const void* v_cache, int64_t num_slots, int n_heads, int n_kv_heads, int head_dim,
                                int dtype, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                                int max_seqlen_q, int max_seqlen_k, const int32_t* read_slot_mapping,
                                float softmax_scale, int shared_prefix_len, const int32_t* shared_kv_lens,
                                const int32_t* affix_shifts, const void* rope_cos, const void* rope_sin,
                                int64_t rope_row_stride, int rope_rows, int rope_dtype, int32_t* err_flag,
                                void* stream) {
  (void)max_seqlen_k;
  if (!read_slot_mapping && batch > 0 && max_seqlen_q > 0) return ACACHE_EINVAL;
  AttnArgs a{q, q_stride, out, o_stride, k_cache, v_cache, num_slots, n_heads, n_kv_heads, head_dim, cu_seqlens_q,
             cu_seqlens_k, batch, max_seqlen_q, read_slot_mapping, nullptr, 0, 1, softmax_scale, shared_prefix_len,
             shared_kv_lens, affix_shifts, rope_cos, rope_sin, rope_row_stride, rope_rows, err_flag,
             (cudaStream_t)stream};
  return attention_common(a, dtype, rope_dtype);
}

extern "C" int64_t acache_attention_grouped_scratch_bytes(int total_q, int n_heads, int head_dim, int batch,
                                                          int n_kv_heads) {
  return attention_split_scratch_bytes(total_q, n_heads, head_dim, batch, n_kv_heads);
}

extern "C" int acache_attention_grouped(const void* q, int64_t q_stride, void* out, int64_t o_stride,
                                        const void* k_cache, const void* v_cache, int64_t num_slots, int n_heads,
                                        int n_kv_heads, int head_dim, int dtype, const int32_t* cu_seqlens_q,
                                        const int32_t* cu_seqlens_k, int batch, int total_q, int max_seqlen_q,
                                        const int32_t* read_slot_mapping, float softmax_scale, int shared_prefix_len,
                                        const int32_t* shared_kv_lens, const int32_t* affix_shifts,
                                        const void* rope_cos, const void* rope_sin, int64_t rope_row_stride,
                                        int rope_rows, int rope_dtype, void* scratch, int64_t scratch_bytes,
                                        int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (batch < 0 || total_q < 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_heads % n_kv_heads != 0)
    return ACACHE_EINVAL;
  if (batch == 0 || max_seqlen_q <= 0 || total_q == 0) return ACACHE_OK;
  if (!q || !out || !k_cache || !v_cache || !cu_seqlens_q || !cu_seqlens_k || !read_slot_mapping) return ACACHE_EINVAL;
  const bool relocate = shared_prefix_len > 0 && affix_shifts != nullptr;
  if (relocate && (!rope_cos || !rope_sin || rope_rows <= 0)) return ACACHE_EINVAL;
  AttnArgs a{q, q_stride, out, o_stride, k_cache, v_cache, num_slots, n_heads, n_kv_heads, head_dim, cu_seqlens_q,
             cu_seqlens_k, batch, max_seqlen_q, read_slot_mapping, nullptr, 0, 1, softmax_scale, shared_prefix_len,
             shared_kv_lens, affix_shifts, rope_cos, rope_sin, rope_row_stride, rope_rows, err_flag,
             (cudaStream_t)stream};
  return attention_split_dispatch(a, dtype, rope_dtype, total_q, scratch, scratch_bytes);
}

extern "C" int acache_paged_attention(const void* q, int64_t q_stride, void* out, int64_t o_stride,
                                      const void* k_cache, const void* v_cache, int64_t num_slots, int n_heads,
                                      int n_kv_heads, int head_dim, int dtype, const int32_t* cu_seqlens_q,
                                      const int32_t* cu_seqlens_k, int batch, int max_seqlen_q, int max_seqlen_k,
                                      const int32_t* block_tables, int table_stride, int block_size,
                                      float softmax_scale, int32_t* err_flag, void* stream) {
  (void)max_seqlen_k;
  if ((!block_tables || block_size <= 0 || table_stride <= 0) && batch > 0 && max_seqlen_q > 0) return ACACHE_EINVAL;
  AttnArgs a{q, q_stride, out, o_stride, k_cache, v_cache, num_slots, n_heads, n_kv_heads, head_dim, cu_seqlens_q,
             cu_seqlens_k, batch, max_seqlen_q, nullptr, block_tables, table_stride, block_size, softmax_scale, 0,
             nullptr, nullptr, nullptr, nullptr, 0, 0, err_flag, (cudaStream_t)stream};
  return attention_common(a, dtype, ACACHE_F32);
}

// per-CTA partial column sums: one row of affix_len floats per (32-row tile, head)
static int64_t importance_partial_floats(int n_q_rows, int n_heads, int affix_len) {
  const int64_t tiles = (n_q_rows + kBM - 1) / kBM;
  return tiles * n_heads * (int64_t)affix_len;
}

extern "C" int64_t acache_anchor_importance_scratch_bytes(int n_q_rows, int n_heads, int affix_len) {
  if (n_q_rows <= 0 || n_heads <= 0 || affix_len <= 0) return 0;
  return (importance_partial_floats(n_q_rows, n_heads, affix_len) +
          importance_tc_ml_floats(n_q_rows, n_heads, affix_len)) * (int64_t)sizeof(float);
}

template <typename T, typename TR>
static int launch_importance(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q, int n_heads,
                             int n_kv_heads, int D, const void* affix_k, int64_t k_slot_stride, int affix_len,
                             int affix_shift, const void* rope_cos, const void* rope_sin, int64_t rope_stride,
                             int rope_rows, float scale, float* importance, float* partial, cudaStream_t st) {
  using TC = typename PromoteA<T, TR>::type;
  const int ld = D + 1;
  const size_t smem = sizeof(float) * ((size_t)kBM * ld + (size_t)kBN * ld + (size_t)kBM * (kBN + 1));
  auto kern = importance_partial_kernel<T, TR, TC>;
  ACACHE_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((n_q + kBM - 1) / kBM, n_heads);
  kern<<<grid, kThreads, smem, st>>>((const T*)q, q_stride, q_rows, n_q, n_heads, n_kv_heads, D, (const T*)affix_k,
                                     k_slot_stride, affix_len, affix_shift, (const TR*)rope_cos, (const TR*)rope_sin,
                                     rope_stride, rope_rows, scale, partial);
  ACACHE_LAUNCH_CHECK();
  importance_reduce_kernel<<<(affix_len + 255) / 256, 256, 0, st>>>(partial, grid.x * grid.y, affix_len, importance);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_anchor_importance(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q_rows,
                                        int n_heads, int n_kv_heads, int head_dim, int dtype, const void* affix_k,
                                        int64_t k_slot_stride, int affix_len, int affix_shift, const void* rope_cos,
                                        const void* rope_sin, int64_t rope_row_stride, int rope_rows, int rope_dtype,
                                        float scale, float* importance, void* scratch, int64_t scratch_bytes,
                                        int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (n_q_rows < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || head_dim <= 0 || affix_len < 0)
    return ACACHE_EINVAL;
  if (n_q_rows == 0 || affix_len == 0) return ACACHE_OK;
  if (!q || !q_rows || !affix_k || !importance || !scratch) return ACACHE_EINVAL;
  if (affix_shift != 0 && (!rope_cos || !rope_sin || affix_shift < 0 || affix_shift >= rope_rows)) return ACACHE_EINVAL;
  if (scratch_bytes < acache_anchor_importance_scratch_bytes(n_q_rows, n_heads, affix_len)) return ACACHE_EINVAL;
  const int E = 16 / dtype_bytes(dtype);
  if (head_dim % (2 * E) != 0 || head_dim > 256 || k_slot_stride % E != 0 || !aligned16(affix_k))
    return ACACHE_EUNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  {
    // tensor-core path for bf16/fp16 with head_dim 64/128; it needs no more partial rows than
    // acache_anchor_importance_scratch_bytes() provides
    int n_partials = 0;
    const int rc = importance_tc_dispatch(q, q_stride, q_rows, n_q_rows, n_heads, n_kv_heads, head_dim, dtype, affix_k,
                                          k_slot_stride, affix_len, affix_shift, rope_cos, rope_sin, rope_row_stride,
                                          rope_dtype, scale, (float*)scratch, &n_partials,
                                          (float*)scratch + importance_partial_floats(n_q_rows, n_heads, affix_len), err_flag,
                                          st);
    if (rc == ACACHE_OK) {
      importance_reduce_kernel<<<(affix_len + 255) / 256, 256, 0, st>>>((const float*)scratch, n_partials, affix_len,
                                                                        importance);
      ACACHE_LAUNCH_CHECK();
      return ACACHE_OK;
    }
    if (rc != ACACHE_EUNSUPPORTED) return rc;
  }
#define IMP(T, TR)                                                                                                  \
  return launch_importance<T, TR>(q, q_stride, q_rows, n_q_rows, n_heads, n_kv_heads, head_dim, affix_k,            \
                                  k_slot_stride, affix_len, affix_shift, rope_cos, rope_sin, rope_row_stride,       \
                                  rope_rows, scale, importance, (float*)scratch, st)
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (rope_dtype == ACACHE_F32) { IMP(T, float); }
    if (rope_dtype == ACACHE_F16) { IMP(T, __half); }
    IMP(T, __nv_bfloat16);
  });
#undef IMP
  return ACACHE_EINVAL;
}

extern "C" int64_t acache_anchor_importance_batched_scratch_bytes(int n_requests, int max_q_rows, int n_heads,
                                                                  int affix_len) {
  if (n_requests <= 0 || max_q_rows <= 0 || n_heads <= 0 || affix_len <= 0) return 0;
  return (int64_t)n_requests * importance_partial_floats(max_q_rows, n_heads, affix_len) * (int64_t)sizeof(float);
}

extern "C" int acache_anchor_importance_batched(const void* q, int64_t q_stride, const int32_t* q_rows,
                                                const int32_t* q_row_offsets, int n_requests, int max_q_rows,
                                                int n_heads, int n_kv_heads, int head_dim, int dtype,
                                                const void* affix_k, int64_t k_slot_stride, int affix_len,
                                                const int32_t* affix_shifts, const void* rope_cos,
                                                const void* rope_sin, int64_t rope_row_stride, int rope_rows,
                                                int rope_dtype, float scale, float* importance,
                                                int64_t importance_stride, void* scratch, int64_t scratch_bytes,
                                                int32_t* err_flag, void* stream) {
  if (!dtype_ok(dtype) || !dtype_ok(rope_dtype)) return ACACHE_EINVAL;
  if (n_requests < 0 || max_q_rows < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 ||
      head_dim <= 0 || affix_len < 0 || importance_stride < affix_len)
    return ACACHE_EINVAL;
  if (n_requests == 0 || max_q_rows == 0 || affix_len == 0) return ACACHE_OK;
  if (!q || !q_rows || !q_row_offsets || !affix_k || !importance || !scratch) return ACACHE_EINVAL;
  if (affix_shifts != nullptr && (!rope_cos || !rope_sin || rope_rows <= 0)) return ACACHE_EINVAL;
  if (scratch_bytes < acache_anchor_importance_batched_scratch_bytes(n_requests, max_q_rows, n_heads, affix_len))
    return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  int n_partials = 0;
  const int rc = importance_tc_batched_dispatch(q, q_stride, q_rows, q_row_offsets, n_requests, max_q_rows, n_heads,
                                                n_kv_heads, head_dim, dtype, affix_k, k_slot_stride, affix_len,
                                                affix_shifts, rope_cos, rope_sin, rope_row_stride, rope_rows, rope_dtype,
                                                scale, (float*)scratch, &n_partials, err_flag, st);
  if (rc != ACACHE_OK) return rc;
  importance_reduce_kernel<<<dim3((affix_len + 255) / 256, n_requests), 256, 0, st>>>(
      (const float*)scratch, n_partials, affix_len, importance, importance_stride);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

// ------------------------------------------------------------------------------------
// Anchor influence score without any allocation by anybody.
//
// Some hosts of this library may not allocate device memory at the moment they need a
// score: a serving loop that has handed the whole GPU to its own arena (so cudaMalloc
// fails or blocks), a plugin that is only ever given its input and output buffers, or a
// latency-critical path where the implicit device synchronisation of cudaMalloc/cudaFree
// is not acceptable.  For them the per-CTA partial sums live in this fixed array that is
// part of the library image; every GPU that loads the library carries it until the
// process exits.
namespace acache {
constexpr int64_t kStaticScratchFloats = 2 * 1024 * 1024;  // 8 MiB
static __device__ __align__(256) float g_importance_scratch[kStaticScratchFloats];

// In host code `g_importance_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up once per device, with that device
// current, and kept here.
// The cache assumes that the device's primary context lives as long as the process (after a
// cudaDeviceReset the array has a new address and this entry would be stale).
constexpr int kMaxDevices = 64;
static std::atomic<float*> g_scratch_addr[kMaxDevices];
}  // namespace acache

extern "C" int64_t acache_anchor_importance_static_scratch_bytes(void) {
  return acache::kStaticScratchFloats * (int64_t)sizeof(float);
}

extern "C" int acache_anchor_importance_static(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q_rows,
                                               int n_heads, int n_kv_heads, int head_dim, int dtype,
                                               const void* affix_k, int64_t k_slot_stride, int affix_len,
                                               int affix_shift, const void* rope_cos, const void* rope_sin,
                                               int64_t rope_row_stride, int rope_rows, int rope_dtype, float scale,
                                               float* importance, int32_t* err_flag, void* stream) {
  // sizes first: a request that needs more partial-sum space than the fixed array holds is
  // refused here, before anything touches the device
  const int64_t need = acache_anchor_importance_scratch_bytes(n_q_rows, n_heads, affix_len);
  if (need > acache_anchor_importance_static_scratch_bytes()) return ACACHE_ELIMIT;
  int dev = -1;
  ACACHE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ACACHE_ELIMIT;
  float* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    // first call on this device: resolve the array's device address (no allocation happens).
    // The look-up is not a stream operation, so it is refused while the stream is capturing
    // instead of invalidating the capture: make the first call on a device before capturing.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    ACACHE_CUDA_CHECK(cudaStreamIsCapturing((cudaStream_t)stream, &capturing));
    if (capturing != cudaStreamCaptureStatusNone) return ACACHE_EUNSUPPORTED;
    float* p = nullptr;
    ACACHE_CUDA_CHECK(cudaGetSymbolAddress((void**)&p, g_importance_scratch));
    if (p == nullptr) return ACACHE_ECUDA;
    g_scratch_addr[dev].store(p, std::memory_order_release);   // every thread resolves the same address
    addr = p;
  }
  return acache_anchor_importance(q, q_stride, q_rows, n_q_rows, n_heads, n_kv_heads, head_dim, dtype, affix_k,
                                  k_slot_stride, affix_len, affix_shift, rope_cos, rope_sin, rope_row_stride,
                                  rope_rows, rope_dtype, scale, importance, addr, need, err_flag, stream);
}
