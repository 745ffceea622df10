// Confidence-threshold unmasking: fused argmax + logsumexp over the vocabulary (one pass
// over the logits, HBM-bound), then the per-row commit rule applied in place.
#include "common.cuh"

namespace acache {

struct ArgStat {
  float m;   // running max
  int idx;   // its (lowest) index
  float s;   // sum of exp(x - m)
};

__device__ __forceinline__ ArgStat combine(const ArgStat& a, const ArgStat& b) {
  ArgStat r;
  if (a.m > b.m || (a.m == b.m && a.idx < b.idx)) { r.m = a.m; r.idx = a.idx; }
  else { r.m = b.m; r.idx = b.idx; }
  const float sa = (a.m == -INFINITY) ? 0.f : a.s * __expf(a.m - r.m);
  const float sb = (b.m == -INFINITY) ? 0.f : b.s * __expf(b.m - r.m);
  r.s = sa + sb;
  return r;
}

template <typename T>
__global__ void __launch_bounds__(512) argmax_conf_kernel(const T* __restrict__ logits, int64_t stride, int vocab,
                                                          int64_t* __restrict__ x0, float* __restrict__ conf) {
  constexpr int E = 16 / sizeof(T);
  const T* row = logits + (int64_t)blockIdx.x * stride;
  ArgStat st{-INFINITY, 0x7FFFFFFF, 0.f};
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const int nvec = vec ? vocab / E : 0;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    Vec16<T> v;
    v.u = ld_global_nc(row + (int64_t)c * E);
    float f[E];
    float lm = -INFINITY;
    int li = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      f[e] = to_f32<T>(v.e[e]);
      if (f[e] > lm) { lm = f[e]; li = e; }
    }
    if (lm > st.m) {
      st.s = (st.m == -INFINITY) ? 0.f : st.s * __expf(st.m - lm);
      st.m = lm;
      st.idx = c * E + li;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) st.s += __expf(f[e] - st.m);
  }
  for (int c = nvec * E + threadIdx.x; c < vocab; c += blockDim.x) {
    const float f = to_f32<T>(row[c]);
    if (f > st.m) {
      st.s = (st.m == -INFINITY) ? 0.f : st.s * __expf(st.m - f);
      st.m = f;
      st.idx = c;
    }
    st.s += __expf(f - st.m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgStat other;
    other.m = __shfl_xor_sync(0xFFFFFFFFu, st.m, o);
    other.idx = __shfl_xor_sync(0xFFFFFFFFu, st.idx, o);
    other.s = __shfl_xor_sync(0xFFFFFFFFu, st.s, o);
    st = combine(st, other);
  }
  __shared__ ArgStat red[16];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = st;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgStat t = red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) t = combine(t, red[i]);
    x0[blockIdx.x] = t.idx;
    conf[blockIdx.x] = 1.f / t.s;  // exp(max - logsumexp)
  }
}

// one warp per block row
__global__ void apply_transfer_kernel(int64_t* __restrict__ blocks, const int64_t* __restrict__ x0,
                                      const float* __restrict__ conf, int n_rows, int block_len, int64_t mask_id,
                                      float threshold) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  int64_t* b = blocks + (int64_t)row * block_len;
  const int64_t* xr = x0 + (int64_t)row * block_len;
  const float* cr = conf + (int64_t)row * block_len;
  bool any_mask = false, any_commit = false;
  float best = -INFINITY;
  int best_pos = 0x7FFFFFFF;
  for (int p = lane; p < block_len; p += 32) {
    if (b[p] == mask_id) {
      any_mask = true;
      const float c = cr[p];
      if (c >= threshold) any_commit = true;
      if (c > best || (c == best && p < best_pos)) { best = c; best_pos = p; }
    }
  }
  any_mask = __any_sync(0xFFFFFFFFu, any_mask);
  any_commit = __any_sync(0xFFFFFFFFu, any_commit);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    const int op = __shfl_xor_sync(0xFFFFFFFFu, best_pos, o);
    if (ob > best || (ob == best && op < best_pos)) { best = ob; best_pos = op; }
  }
  if (!any_mask) return;
  if (any_commit) {
    for (int p = lane; p < block_len; p += 32)
      if (b[p] == mask_id && cr[p] >= threshold) b[p] = xr[p];
  } else if (lane == 0 && best_pos < block_len) {
    b[best_pos] = xr[best_pos];
  }
}

}  // namespace acache

using namespace acache;

extern "C" int acache_transfer_tokens(const void* logits, int64_t logits_stride, int vocab, int dtype,
                                      int64_t* blocks, int n_rows, int block_len, int64_t mask_id, float threshold,
                                      int64_t* x0_out, float* conf_out, void* stream) {
  if (!dtype_ok(dtype) || vocab <= 0 || n_rows < 0 || block_len <= 0 || logits_stride < vocab) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!logits || !blocks || !x0_out || !conf_out) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int rows = n_rows * block_len;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    argmax_conf_kernel<T><<<rows, 512, 0, st>>>((const T*)logits, logits_stride, vocab, x0_out, conf_out);
  });
  ACACHE_LAUNCH_CHECK();
  apply_transfer_kernel<<<(n_rows + 3) / 4, 128, 0, st>>>(blocks, x0_out, conf_out, n_rows, block_len, mask_id, threshold);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_apply_transfer(int64_t* blocks, const int64_t* x0, const float* confidence, int n_rows,
                                     int block_len, int64_t mask_id, float threshold, void* stream) {
  if (n_rows < 0 || block_len <= 0) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!blocks || !x0 || !confidence) return ACACHE_EINVAL;
  apply_transfer_kernel<<<(n_rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(blocks, x0, confidence, n_rows, block_len,
                                                                             mask_id, threshold);
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}
