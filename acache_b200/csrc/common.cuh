// Shared helpers of the acache_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/acache_b200.h"

namespace acache {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

void set_last_cuda_error(cudaError_t e);

#define ACACHE_CUDA_CHECK(expr)                      \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) {                         \
      ::acache::set_last_cuda_error(_e);             \
      return ACACHE_ECUDA;                           \
    }                                                \
  } while (0)

#define ACACHE_LAUNCH_CHECK() ACACHE_CUDA_CHECK(cudaGetLastError())

inline int dtype_bytes(int dtype) { return dtype == ACACHE_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == ACACHE_F32 || dtype == ACACHE_F16 || dtype == ACACHE_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- programmatic dependent launch ------------------------------------------------
// A kernel launched with `launch_chained` may become resident while the kernel before it in the
// stream is still running (as SMs free up), once every CTA of that kernel has executed
// `chain_release()`; it must not touch global memory before `chain_wait()`, which returns when
// the kernel before it has completed and its writes are visible.  Kernels of a decode step
// release at their first instruction and wait after their on-chip set-up (barriers, TMEM), so
// launch latency and set-up overlap the tail of the previous kernel; the order of all global
// memory accesses stays that of plain stream order.  Both are no-ops in a kernel launched the
// ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif
bool chained_launches();     // false when ACACHE_CHAINED_LAUNCHES=0 is set in the environment

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args... args) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.dynamicSmemBytes = smem;
  lc.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = chained_launches() ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kern, static_cast<KArgs>(args)...);
}

// ---- element conversion ---------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// round-trip through T: the rounding an eager op producing dtype T applies
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

// 16-byte vector of elements
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 u; T e[N]; };
};

__device__ __forceinline__ uint4 ld_global_nc(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_global_cs(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Arithmetic dtype of a rotation: promote(element dtype, table dtype).  When it is
// fp32 the three operations (mul, mul, add) each round once in fp32 and the result is
// cast once; when it is a 16-bit type every operation result is rounded to it, which
// is what an eager framework op chain in that dtype produces.
template <typename TC>
__device__ __forceinline__ float rot_lo(float x1, float x2, float c, float s) {
  // out = x1*c + (-x2)*s
  float a = round_to<TC>(__fmul_rn(x1, c));
  float b = round_to<TC>(__fmul_rn(-x2, s));
  return round_to<TC>(__fadd_rn(a, b));
}
template <typename TC>
__device__ __forceinline__ float rot_hi(float x1, float x2, float c, float s) {
  // out = x2*c + x1*s
  float a = round_to<TC>(__fmul_rn(x2, c));
  float b = round_to<TC>(__fmul_rn(x1, s));
  return round_to<TC>(__fadd_rn(a, b));
}

// arguments of one varlen attention launch (shared by the tensor-core and the general kernel)
struct AttnArgs {
  const void* q; int64_t q_stride; void* out; int64_t o_stride; const void* k_cache; const void* v_cache;
  int64_t num_slots; int n_heads, n_kv_heads, head_dim; const int32_t* cu_q; const int32_t* cu_k; int batch;
  int max_q; const int32_t* slot_map; const int32_t* block_tables; int table_stride, block_size; float scale;
  int shared_prefix_len; const int32_t* shared_kv_lens; const int32_t* affix_shifts; const void* rope_cos;
  const void* rope_sin; int64_t rope_stride; int rope_rows; int32_t* err_flag; cudaStream_t st;
};

// dispatch helpers ---------------------------------------------------------------
#define ACACHE_DISPATCH_DTYPE(dtype, T, ...)                    \
  switch (dtype) {                                              \
    case ACACHE_F32: { using T = float; __VA_ARGS__; break; }   \
    case ACACHE_F16: { using T = __half; __VA_ARGS__; break; }  \
    case ACACHE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: return ACACHE_EINVAL;                              \
  }

}  // namespace acache
