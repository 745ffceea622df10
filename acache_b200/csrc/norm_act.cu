// RMSNorm and gated activation of the transformer block: single-pass, HBM-bound.
#include "common.cuh"

namespace acache {

// one CTA per row; the row is kept in registers between the reduction and the write
template <typename T, int VPT /*16-byte vectors per thread*/>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, int64_t x_stride,
                                                      const T* __restrict__ w, T* __restrict__ y, int64_t y_stride,
                                                      int n_cols, float eps) {
  constexpr int E = 16 / sizeof(T);
  chain_release();
  chain_wait();
  const int row = blockIdx.x;
  const T* xr = x + (int64_t)row * x_stride;
  T* yr = y + (int64_t)row * y_stride;
  const int nvec = n_cols / E;
  Vec16<T> v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      v[i].u = *reinterpret_cast<const uint4*>(xr + (int64_t)c * E);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float f = to_f32<T>(v[i].e[e]);
        ss = fmaf(f, f, ss);
      }
    }
  }
  __shared__ float red[8];
  __shared__ float s_scale;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    s_scale = rsqrtf(t / (float)n_cols + eps);
  }
  __syncthreads();
  const float sc = s_scale;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      Vec16<T> wv, o;
      wv.u = *reinterpret_cast<const uint4*>(w + (int64_t)c * E);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float n = round_to<T>(to_f32<T>(v[i].e[e]) * sc);      // normalised value cast back to T
        o.e[e] = from_f32<T>(to_f32<T>(wv.e[e]) * n);                 // weight * x in T
      }
      *reinterpret_cast<uint4*>(yr + (int64_t)c * E) = o.u;
    }
  }
}

// x_new = x + delta (rounded to T, written back in place of x), y = rmsnorm(x_new): the residual
// add of the previous sub-layer fused into the normalisation that follows it
// With PART the update arrives as `n_splits` fp32 slices of a projection's K range
// (`partials[s][row][col]`, rows `d_stride` floats apart, slices `split_stride` floats apart): they
// are summed in slice order and rounded to T, which is the projection's output as a GEMM in T
// leaves it, before the add.
template <typename T, int VPT, bool PART>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(T* __restrict__ x, int64_t x_stride, const T* __restrict__ delta,
                                                          int64_t d_stride, const T* __restrict__ w, T* __restrict__ y,
                                                          int64_t y_stride, int n_cols, float eps,
                                                          const float* __restrict__ partials, int n_splits,
                                                          int64_t split_stride) {
  constexpr int E = 16 / sizeof(T);
  chain_release();
  chain_wait();
  const int row = blockIdx.x;
  T* xr = x + (int64_t)row * x_stride;
  const T* dr = PART ? nullptr : delta + (int64_t)row * d_stride;
  const float* pr = PART ? partials + (int64_t)row * d_stride : nullptr;
  T* yr = y + (int64_t)row * y_stride;
  const int nvec = n_cols / E;
  Vec16<T> v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      Vec16<T> a, b;
      a.u = *reinterpret_cast<const uint4*>(xr + (int64_t)c * E);
      if (PART) {
        float acc[E];
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
          const float* src = pr + sp * split_stride + (int64_t)c * E;
#pragma unroll
          for (int q = 0; q < E / 4; ++q) {
            const uint4 u = ld_global_nc(src + 4 * q);
            acc[4 * q] += __uint_as_float(u.x);
            acc[4 * q + 1] += __uint_as_float(u.y);
            acc[4 * q + 2] += __uint_as_float(u.z);
            acc[4 * q + 3] += __uint_as_float(u.w);
          }
        }
#pragma unroll
        for (int e = 0; e < E; ++e) b.e[e] = from_f32<T>(acc[e]);
      } else {
        b.u = ld_global_nc(dr + (int64_t)c * E);
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        v[i].e[e] = from_f32<T>(to_f32<T>(a.e[e]) + to_f32<T>(b.e[e]));
        const float f = to_f32<T>(v[i].e[e]);
        ss = fmaf(f, f, ss);
      }
      *reinterpret_cast<uint4*>(xr + (int64_t)c * E) = v[i].u;
    }
  }
  __shared__ float red[8];
  __shared__ float s_scale;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    s_scale = rsqrtf(t / (float)n_cols + eps);
  }
  __syncthreads();
  const float sc = s_scale;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      Vec16<T> wv, o;
      wv.u = *reinterpret_cast<const uint4*>(w + (int64_t)c * E);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float n = round_to<T>(to_f32<T>(v[i].e[e]) * sc);
        o.e[e] = from_f32<T>(to_f32<T>(wv.e[e]) * n);
      }
      *reinterpret_cast<uint4*>(yr + (int64_t)c * E) = o.u;
    }
  }
}

// generic row kernel for widths the register kernel does not cover
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_generic_kernel(const T* __restrict__ x, int64_t x_stride,
                                                              const T* __restrict__ w, T* __restrict__ y,
                                                              int64_t y_stride, int n_cols, float eps) {
  const int row = blockIdx.x;
  const T* xr = x + (int64_t)row * x_stride;
  T* yr = y + (int64_t)row * y_stride;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n_cols; c += 256) {
    const float f = to_f32<T>(xr[c]);
    ss = fmaf(f, f, ss);
  }
  __shared__ float red[8];
  __shared__ float s_scale;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    s_scale = rsqrtf(t / (float)n_cols + eps);
  }
  __syncthreads();
  const float sc = s_scale;
  for (int c = threadIdx.x; c < n_cols; c += 256) {
    const float n = round_to<T>(to_f32<T>(xr[c]) * sc);
    yr[c] = from_f32<T>(to_f32<T>(w[c]) * n);
  }
}

__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == 0) return x / (1.f + expf(-x));
  if (act == 1) return fmaxf(x, 0.f);
  return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
}

template <typename T>
__global__ void __launch_bounds__(256) act_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                      T* __restrict__ y, int64_t n_vec, int64_t n, int act) {
  constexpr int E = 16 / sizeof(T);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    Vec16<T> g, u, o;
    g.u = ld_global_nc(gate + i * E);
    u.u = ld_global_nc(up + i * E);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float a = round_to<T>(act_fn(to_f32<T>(g.e[e]), act));
      o.e[e] = from_f32<T>(a * to_f32<T>(u.e[e]));
    }
    *reinterpret_cast<uint4*>(y + i * E) = o.u;
  }
  // tail (n not a multiple of the vector width)
  if (blockIdx.x == 0) {
    for (int64_t i = n_vec * E + threadIdx.x; i < n; i += blockDim.x) {
      const float a = round_to<T>(act_fn(to_f32<T>(gate[i]), act));
      y[i] = from_f32<T>(a * to_f32<T>(up[i]));
    }
  }
}

// gate and up as the two halves of one projection output: x[rows, 2 * ffn] = [gate | up]
template <typename T>
__global__ void __launch_bounds__(256) act_mul_halves_kernel(const T* __restrict__ x, int64_t x_stride,
                                                             T* __restrict__ y, int64_t y_stride, int rows, int ffn,
                                                             int act) {
  constexpr int E = 16 / sizeof(T);
  const int vec_per_row = ffn / E;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * E;
    Vec16<T> g, u, o;
    g.u = ld_global_nc(x + r * x_stride + c);
    u.u = ld_global_nc(x + r * x_stride + ffn + c);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float a = round_to<T>(act_fn(to_f32<T>(g.e[e]), act));
      o.e[e] = from_f32<T>(a * to_f32<T>(u.e[e]));
    }
    *reinterpret_cast<uint4*>(y + r * y_stride + c) = o.u;
  }
}

}  // namespace acache

using namespace acache;

extern "C" int acache_act_mul_halves(const void* x, int64_t x_stride, void* y, int64_t y_stride, int n_rows, int ffn,
                                     int act, int dtype, void* stream) {
  if (!dtype_ok(dtype) || n_rows < 0 || ffn <= 0 || act < 0 || act > 2) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !y) return ACACHE_EINVAL;
  const int E = 16 / dtype_bytes(dtype);
  if (ffn % E != 0 || x_stride % E != 0 || y_stride % E != 0 || !aligned16(x) || !aligned16(y)) return ACACHE_EUNSUPPORTED;
  const int64_t total = (int64_t)n_rows * (ffn / E);
  int64_t blocks = (total + 255) / 256;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    act_mul_halves_kernel<T><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const T*)x, x_stride, (T*)y, y_stride,
                                                                             n_rows, ffn, act);
  });
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_rmsnorm(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride,
                              int n_rows, int n_cols, float eps, int dtype, void* stream) {
  if (!dtype_ok(dtype) || n_rows < 0 || n_cols <= 0) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !weight || !y) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int E = 16 / dtype_bytes(dtype);
  const bool vec = n_cols % E == 0 && x_stride % E == 0 && y_stride % E == 0 && aligned16(x) && aligned16(y) &&
                   aligned16(weight);
  const int nvec = n_cols / E;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (vec && nvec <= 256) {
      ACACHE_CUDA_CHECK(launch_chained(rmsnorm_kernel<T, 1>, dim3(n_rows), dim3(256), 0, st, (const T*)x, x_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps));
    } else if (vec && nvec <= 512) {
      ACACHE_CUDA_CHECK(launch_chained(rmsnorm_kernel<T, 2>, dim3(n_rows), dim3(256), 0, st, (const T*)x, x_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps));
    } else if (vec && nvec <= 1024) {
      ACACHE_CUDA_CHECK(launch_chained(rmsnorm_kernel<T, 4>, dim3(n_rows), dim3(256), 0, st, (const T*)x, x_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps));
    } else {
      rmsnorm_generic_kernel<T><<<n_rows, 256, 0, st>>>((const T*)x, x_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps);
    }
  });
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_act_mul(const void* gate, const void* up, void* y, int64_t n, int act, int dtype,
                              void* stream) {
  if (!dtype_ok(dtype) || n < 0 || act < 0 || act > 2) return ACACHE_EINVAL;
  if (n == 0) return ACACHE_OK;
  if (!gate || !up || !y) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int E = 16 / dtype_bytes(dtype);
  const bool vec = aligned16(gate) && aligned16(up) && aligned16(y);
  const int64_t n_vec = vec ? n / E : 0;
  int64_t blocks = (n_vec + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    act_mul_kernel<T><<<(int)blocks, 256, 0, st>>>((const T*)gate, (const T*)up, (T*)y, n_vec, n, act);
  });
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_add_rmsnorm(void* x, int64_t x_stride, const void* delta, int64_t d_stride, const void* weight,
                                  void* y, int64_t y_stride, int n_rows, int n_cols, float eps, int dtype,
                                  void* stream) {
  if (!dtype_ok(dtype) || n_rows < 0 || n_cols <= 0) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !delta || !weight || !y) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int E = 16 / dtype_bytes(dtype);
  const bool vec = n_cols % E == 0 && x_stride % E == 0 && y_stride % E == 0 && d_stride % E == 0 && aligned16(x) &&
                   aligned16(y) && aligned16(weight) && aligned16(delta);
  const int nvec = n_cols / E;
  if (!vec || nvec > 1024) return ACACHE_EUNSUPPORTED;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (nvec <= 256) {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 1, false>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, (const T*)delta, d_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, nullptr, 0, 0));
    } else if (nvec <= 512) {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 2, false>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, (const T*)delta, d_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, nullptr, 0, 0));
    } else {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 4, false>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, (const T*)delta, d_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, nullptr, 0, 0));
    }
  });
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}

extern "C" int acache_add_rmsnorm_partials(void* x, int64_t x_stride, const float* partials, int n_splits,
                                           int64_t split_stride, int64_t p_stride, const void* weight, void* y,
                                           int64_t y_stride, int n_rows, int n_cols, float eps, int dtype,
                                           void* stream) {
  if (!dtype_ok(dtype) || n_rows < 0 || n_cols <= 0 || n_splits <= 0) return ACACHE_EINVAL;
  if (n_rows == 0) return ACACHE_OK;
  if (!x || !partials || !weight || !y) return ACACHE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int E = 16 / dtype_bytes(dtype);
  const bool vec = n_cols % E == 0 && x_stride % E == 0 && y_stride % E == 0 && p_stride % 4 == 0 &&
                   split_stride % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(weight) && aligned16(partials);
  const int nvec = n_cols / E;
  if (!vec || nvec > 1024) return ACACHE_EUNSUPPORTED;
  ACACHE_DISPATCH_DTYPE(dtype, T, {
    if (nvec <= 256) {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 1, true>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, nullptr, p_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, partials, n_splits, split_stride));
    } else if (nvec <= 512) {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 2, true>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, nullptr, p_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, partials, n_splits, split_stride));
    } else {
      ACACHE_CUDA_CHECK(launch_chained(add_rmsnorm_kernel<T, 4, true>, dim3(n_rows), dim3(256), 0, st, (T*)x, x_stride, nullptr, p_stride, (const T*)weight, (T*)y, y_stride, n_cols, eps, partials, n_splits, split_stride));
    }
  });
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}
