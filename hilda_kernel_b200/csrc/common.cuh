// Shared device helpers for the hilda B200 kernels: 128-bit vector access,
// dtype traits, warp/block reductions, and the C-ABI status codes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#ifdef HILDA_DEBUG
#include <cstdio>
#endif

// ---- status codes returned by every extern "C" entry point -----------------
#define HILDA_OK 0
#define HILDA_ERR_DTYPE (-1)      // unsupported dtype enum
#define HILDA_ERR_ALIGN (-2)      // pointer or stride not 16-byte aligned where required
#define HILDA_ERR_SIZE (-3)       // size not supported by this entry point
#define HILDA_ERR_CUDA (-4)       // a CUDA runtime call or launch failed
#define HILDA_ERR_NULL (-5)       // required pointer is null
#define HILDA_ERR_DEVICE (-6)     // device status word reported a bounded wait ran out
#define HILDA_ERR_ARG (-7)        // inconsistent arguments

// dtype enum shared with the Python side
#define HILDA_F32 0
#define HILDA_BF16 1
#define HILDA_F16 2

namespace hilda {

static inline int dtype_size(int dt) { return dt == HILDA_F32 ? 4 : (dt == HILDA_BF16 || dt == HILDA_F16) ? 2 : 0; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

#ifdef HILDA_DEBUG
// Debug build: wait for the launch and report a fault from the entry point that caused it (a
// release build would see it at some later call). Not usable while a stream is being captured.
#define HILDA_LAUNCH_CHECK()                                                                  \
  do {                                                                                        \
    cudaError_t e__ = cudaGetLastError();                                                     \
    if (e__ == cudaSuccess) e__ = cudaDeviceSynchronize();                                    \
    if (e__ != cudaSuccess) {                                                                 \
      fprintf(stderr, "hilda_b200: %s at %s:%d\n", cudaGetErrorString(e__), __FILE__, __LINE__); \
      return HILDA_ERR_CUDA;                                                                  \
    }                                                                                         \
  } while (0)
#else
#define HILDA_LAUNCH_CHECK()                                   \
  do {                                                         \
    cudaError_t e__ = cudaGetLastError();                      \
    if (e__ != cudaSuccess) return HILDA_ERR_CUDA;             \
  } while (0)
#endif

// ---- dtype traits: VEC elements per 16-byte vector --------------------------
template <typename T> struct VT;

template <> struct VT<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float round(float x) { return x; }
  static __device__ __forceinline__ float load1(const float* p) { return *p; }
  static __device__ __forceinline__ void store1(float* p, float x) { *p = x; }
};

template <> struct VT<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store1(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
};

template <> struct VT<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ float load1(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void store1(__half* p, float x) { *p = __float2half_rn(x); }
};

// ---- 16-byte global access ---------------------------------------------------
__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
// read-only, streamed once: bypass L1 allocation
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }
// streaming store (evict-first): outputs that are not re-read by this kernel
__device__ __forceinline__ void st16_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Load one element of a tensor whose dtype is only known at run time (weights, tables).
__device__ __forceinline__ float load_any(const void* p, int dt, int64_t i) {
  if (dt == HILDA_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == HILDA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_any(void* p, int dt, int64_t i, float x) {
  if (dt == HILDA_F32) reinterpret_cast<float*>(p)[i] = x;
  else if (dt == HILDA_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
}
__device__ __forceinline__ float round_any(float x, int dt) {
  if (dt == HILDA_F32) return x;
  if (dt == HILDA_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return __half2float(__float2half_rn(x));
}

// ---- reductions --------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result. `red` holds >= 33 floats of shared memory.
// Deterministic: fixed shuffle tree, then a fixed-order sum over warps.
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  constexpr int NW = THREADS / 32;
  v = warp_sum(v);
  if constexpr (NW == 1) return v;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();  // protect `red` from the previous use
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < NW) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  constexpr int NW = THREADS / 32;
  v = warp_max(v);
  if constexpr (NW == 1) return v;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < NW) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

}  // namespace hilda
