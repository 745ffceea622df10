// Anchor top-k: radix select on order-preserving integer keys, ties broken by lowest
// index, selected indices emitted in ascending order.
//   * rows of up to 1024 scores: one warp per row, keys in registers, bit-serial select
//     with warp reductions, ordered compaction with ballots;
//   * longer rows: one CTA per row, keys staged in shared memory, 4 passes of 8-bit
//     histograms, ordered compaction with a block scan.
#include "common.cuh"

namespace acache {

// float -> uint32 whose unsigned order equals the float order (NaN above +inf);
// for "smallest" selection the key is complemented so that the same code selects the
// largest keys.
__device__ __forceinline__ uint32_t order_key(float f, bool largest) {
  uint32_t u = __float_as_uint(f);
  uint32_t k;
  if (f != f) k = 0xFFFFFFFFu;
  else k = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  if (!largest) k = (f != f) ? 0xFFFFFFFFu : ~k;
  return k;
}

template <int KPL>  // keys per lane
__global__ void __launch_bounds__(128) topk_warp_kernel(const float* __restrict__ scores, int n_rows, int n_cols,
                                                        int64_t row_stride, int k, int largest,
                                                        const int32_t* __restrict__ offsets, int64_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float* s = scores + (int64_t)row * row_stride;
  uint32_t key[KPL];
  uint32_t valid = 0;
#pragma unroll
  for (int j = 0; j < KPL; ++j) {
    const int c = j * 32 + lane;
    if (c < n_cols) {
      key[j] = order_key(s[c], largest != 0);
      valid |= 1u << j;
    } else {
      key[j] = 0;
    }
  }
  // bit-serial radix select of the k-th largest key
  uint32_t cand = valid, thr = 0;
  int kr = k;
  for (int bit = 31; bit >= 0; --bit) {
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < KPL; ++j) cnt += ((cand >> j) & 1u) & (key[j] >> bit);
    cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
    uint32_t with_bit = 0;
#pragma unroll
    for (int j = 0; j < KPL; ++j) with_bit |= ((key[j] >> bit) & 1u) << j;
    if (cnt >= kr) {
      cand &= with_bit;
      thr |= 1u << bit;
    } else {
      kr -= cnt;
      cand &= ~with_bit;
    }
  }
  // kr = how many of the keys equal to thr are taken (lowest indices first)
  const uint32_t lt = (1u << lane) - 1u;
  int base_e = 0, base_s = 0;
  const int64_t off = offsets ? (int64_t)offsets[row] : 0;
  int64_t* o = out + (int64_t)row * k;
#pragma unroll
  for (int j = 0; j < KPL; ++j) {
    const bool ok = (valid >> j) & 1u;
    const bool g = ok && key[j] > thr;
    const bool e = ok && key[j] == thr;
    const uint32_t be = __ballot_sync(0xFFFFFFFFu, e);
    const bool sel = g || (e && (base_e + __popc(be & lt)) < kr);
    const uint32_t bs = __ballot_sync(0xFFFFFFFFu, sel);
    if (sel) o[base_s + __popc(bs & lt)] = (int64_t)(j * 32 + lane) + off;
    base_e += __popc(be);
    base_s += __popc(bs);
  }
}

constexpr int kTopkBlock = 512;

__global__ void __launch_bounds__(kTopkBlock) topk_block_kernel(const float* __restrict__ scores, int n_cols,
                                                                int64_t row_stride, int k, int largest,
                                                                const int32_t* __restrict__ offsets,
                                                                int64_t* __restrict__ out, int keys_in_smem) {
  extern __shared__ uint32_t smem_keys[];
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_kr;
  __shared__ int warp_e[kTopkBlock / 32], warp_s[kTopkBlock / 32];
  __shared__ int s_base_e, s_base_s;

  const int row = blockIdx.x;
  const float* s = scores + (int64_t)row * row_stride;
  const int tid = threadIdx.x;
  const bool lg = largest != 0;
  if (keys_in_smem)
    for (int c = tid; c < n_cols; c += kTopkBlock) smem_keys[c] = order_key(s[c], lg);
  if (tid == 0) {
    s_prefix = 0;
    s_kr = k;
    s_base_e = 0;
    s_base_s = 0;
  }
  __syncthreads();
  auto key_at = [&](int c) -> uint32_t { return keys_in_smem ? smem_keys[c] : order_key(s[c], lg); };

  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int c = tid; c < n_cols; c += kTopkBlock) {
      const uint32_t key = key_at(c);
      if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid < 32) {
      // suffix scan over 256 buckets, 8 per lane (lane 31 owns the highest buckets)
      int loc[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        loc[j] = hist[tid * 8 + j];
        sum += loc[j];
      }
      // inclusive suffix sum over lanes: incl = keys in this lane's buckets and above
      int incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int t = __shfl_down_sync(0xFFFFFFFFu, incl, d);
        if (tid + d < 32) incl += t;
      }
      const int above = incl - sum;  // keys in buckets of higher lanes
      const int kr = s_kr;
      // the bucket where the running count from the top first reaches kr
      if (above < kr && incl >= kr) {
        int run = above;
        for (int j = 7; j >= 0; --j) {
          if (run + loc[j] >= kr) {
            s_prefix = prefix | ((uint32_t)(tid * 8 + j) << shift);
            s_kr = kr - run;
            break;
          }
          run += loc[j];
        }
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need = s_kr;
  const int64_t off = offsets ? (int64_t)offsets[row] : 0;
  int64_t* o = out + (int64_t)row * k;
  const int lane = tid & 31, wid = tid >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  for (int c0 = 0; c0 < n_cols; c0 += kTopkBlock) {
    const int c = c0 + tid;
    const bool ok = c < n_cols;
    const uint32_t key = ok ? key_at(c) : 0u;
    const bool g = ok && key > thr;
    const bool e = ok && key == thr;
    const uint32_t be = __ballot_sync(0xFFFFFFFFu, e);
    if (lane == 0) warp_e[wid] = __popc(be);
    __syncthreads();
    int pe = s_base_e;
    for (int w = 0; w < wid; ++w) pe += warp_e[w];
    const bool sel = g || (e && (pe + __popc(be & lt)) < need);
    const uint32_t bs = __ballot_sync(0xFFFFFFFFu, sel);
    if (lane == 0) warp_s[wid] = __popc(bs);
    __syncthreads();
    int ps = s_base_s;
    for (int w = 0; w < wid; ++w) ps += warp_s[w];
    if (sel) o[ps + __popc(bs & lt)] = (int64_t)c + off;
    __syncthreads();
    if (tid == 0) {
      int te = 0, ts = 0;
      for (int w = 0; w < kTopkBlock / 32; ++w) {
        te += warp_e[w];
        ts += warp_s[w];
      }
      s_base_e += te;
      s_base_s += ts;
    }
    __syncthreads();
  }
}

}  // namespace acache

using namespace acache;

extern "C" int acache_anchor_topk(const float* scores, int n_rows, int n_cols, int64_t row_stride, int k,
                                  int largest, const int32_t* offsets, int64_t* out, void* stream) {
  if (n_rows < 0 || n_cols < 0 || k < 0 || row_stride < n_cols) return ACACHE_EINVAL;
  if (k > n_cols) k = n_cols;
  if (n_rows == 0 || k == 0) return ACACHE_OK;
  if (!scores || !out) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_cols <= 1024) {
    const int grid = (n_rows + 3) / 4;
#define TOPK_WARP(KPL) \
  topk_warp_kernel<KPL><<<grid, 128, 0, st>>>(scores, n_rows, n_cols, row_stride, k, largest, offsets, out)
    if (n_cols <= 128) TOPK_WARP(4);
    else if (n_cols <= 256) TOPK_WARP(8);
    else if (n_cols <= 512) TOPK_WARP(16);
    else TOPK_WARP(32);
#undef TOPK_WARP
  } else {
    const size_t bytes = (size_t)n_cols * 4;
    const int in_smem = bytes <= 200 * 1024;
    ACACHE_CUDA_CHECK(cudaFuncSetAttribute(topk_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    topk_block_kernel<<<n_rows, kTopkBlock, in_smem ? bytes : 0, st>>>(scores, n_cols, row_stride, k, largest,
                                                                       offsets, out, in_smem);
  }
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}
