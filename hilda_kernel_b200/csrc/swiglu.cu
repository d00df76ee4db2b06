// SwiGLU and GeGLU forward and backward: HBM-bound streaming kernels for sm_100a.
//
// GeGLU follows kernels/geglu.py:54-72 and :92-124 with gelu_tanh(a) =
// 0.5*a*(1 + tanh(sqrt(2/pi)*(a + 0.044715*a^3))) in place of silu (same rounding points).
//
// Semantics follow kernels/swiglu.py:38-57 and :77-105 of hilda-kernel:
//   forward : c = round_T(silu(a) in fp32) * b   (the product is taken in T)
//   backward: db = dc*silu(a); da = dc*b*(sig + a*sig*(1-sig)), all in fp32, rounded once.
// da/db may alias a/b (the reference overwrites the saved inputs): every thread reads its own
// elements before it writes them.
#include "common.cuh"

namespace hilda {

template <typename T> __device__ __forceinline__ float sigmoidf_t(float a) {
  if constexpr (sizeof(T) == 4) return 1.0f / (1.0f + expf(-a));
  else return __fdividef(1.0f, 1.0f + __expf(-a));
}

constexpr int ACT_SILU = 0, ACT_GELU_TANH = 1;
constexpr float GELU_C0 = 0.7978845608028654f;  // sqrt(2/pi)
constexpr float GELU_C1 = 0.044715f;

template <typename T> __device__ __forceinline__ float tanhf_t(float x) {
  if constexpr (sizeof(T) == 4) return tanhf(x);
  else return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x));
}
// act(a)
template <typename T, int ACT> __device__ __forceinline__ float act_fwd(float a) {
  if constexpr (ACT == ACT_SILU) return a * sigmoidf_t<T>(a);
  else return 0.5f * a * (1.0f + tanhf_t<T>(GELU_C0 * (a + GELU_C1 * a * a * a)));
}
// act(a) and d act / d a
template <typename T, int ACT> __device__ __forceinline__ void act_fwd_grad(float a, float& f, float& df) {
  if constexpr (ACT == ACT_SILU) {
    const float sg = sigmoidf_t<T>(a);
    f = a * sg;
    df = sg + f * (1.0f - sg);
  } else {
    const float th = tanhf_t<T>(GELU_C0 * (a + GELU_C1 * a * a * a));
    f = 0.5f * a * (1.0f + th);
    df = 0.5f * (1.0f + th) + 0.5f * a * (1.0f - th * th) * GELU_C0 * (1.0f + 3.0f * GELU_C1 * a * a);
  }
}

constexpr int SW_UNROLL = 2;  // 16-byte vectors per thread per tensor kept in flight

template <typename T, int ACT>
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int64_t n_vec, int64_t n) {
  constexpr int VEC = VT<T>::N;
  const int64_t stride = (int64_t)gridDim.x * 256;
  int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x;
  for (; v + (SW_UNROLL - 1) * stride < n_vec; v += SW_UNROLL * stride) {
    uint4 av[SW_UNROLL], bv[SW_UNROLL];
#pragma unroll
    for (int u = 0; u < SW_UNROLL; ++u) {
      av[u] = ld16_stream(A + (v + u * stride) * VEC);
      bv[u] = ld16_stream(B + (v + u * stride) * VEC);
    }
#pragma unroll
    for (int u = 0; u < SW_UNROLL; ++u) {
      float a[VEC], b[VEC];
      VT<T>::unpack(av[u], a);
      VT<T>::unpack(bv[u], b);
#pragma unroll
      for (int j = 0; j < VEC; ++j) a[j] = VT<T>::round(act_fwd<T, ACT>(a[j])) * b[j];
      st16_stream(C + (v + u * stride) * VEC, VT<T>::pack(a));
    }
  }
  for (; v < n_vec; v += stride) {
    float a[VEC], b[VEC];
    VT<T>::unpack(ld16_stream(A + v * VEC), a);
    VT<T>::unpack(ld16_stream(B + v * VEC), b);
#pragma unroll
    for (int j = 0; j < VEC; ++j) a[j] = VT<T>::round(act_fwd<T, ACT>(a[j])) * b[j];
    st16_stream(C + v * VEC, VT<T>::pack(a));
  }
  // ragged tail (n not a multiple of VEC, or unaligned tensors when n_vec == 0)
  for (int64_t e = n_vec * VEC + (int64_t)blockIdx.x * 256 + threadIdx.x; e < n; e += stride) {
    const float a = VT<T>::load1(A + e);
    VT<T>::store1(C + e, VT<T>::round(act_fwd<T, ACT>(a)) * VT<T>::load1(B + e));
  }
}

template <typename T, int ACT>
__device__ __forceinline__ void swiglu_bwd_elem(float a, float b, float dc, float& da, float& db) {
  float f, df;
  act_fwd_grad<T, ACT>(a, f, df);
  db = dc * f;
  da = dc * b * df;
}

template <typename T, int ACT>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const T* A, const T* B, const T* __restrict__ DC, T* DA, T* DB, int64_t n_vec, int64_t n) {
  constexpr int VEC = VT<T>::N;
  const int64_t stride = (int64_t)gridDim.x * 256;
  int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x;
  for (; v + (SW_UNROLL - 1) * stride < n_vec; v += SW_UNROLL * stride) {
    uint4 av[SW_UNROLL], bv[SW_UNROLL], cv[SW_UNROLL];
#pragma unroll
    for (int u = 0; u < SW_UNROLL; ++u) {
      av[u] = ld16(A + (v + u * stride) * VEC);
      bv[u] = ld16(B + (v + u * stride) * VEC);
      cv[u] = ld16_stream(DC + (v + u * stride) * VEC);
    }
#pragma unroll
    for (int u = 0; u < SW_UNROLL; ++u) {
      float a[VEC], b[VEC], dc[VEC];
      VT<T>::unpack(av[u], a);
      VT<T>::unpack(bv[u], b);
      VT<T>::unpack(cv[u], dc);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        float da, db;
        swiglu_bwd_elem<T, ACT>(a[j], b[j], dc[j], da, db);
        a[j] = da; b[j] = db;
      }
      st16_stream(DA + (v + u * stride) * VEC, VT<T>::pack(a));
      st16_stream(DB + (v + u * stride) * VEC, VT<T>::pack(b));
    }
  }
  for (; v < n_vec; v += stride) {
    float a[VEC], b[VEC], dc[VEC];
    VT<T>::unpack(ld16(A + v * VEC), a);
    VT<T>::unpack(ld16(B + v * VEC), b);
    VT<T>::unpack(ld16_stream(DC + v * VEC), dc);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float da, db;
      swiglu_bwd_elem<T, ACT>(a[j], b[j], dc[j], da, db);
      a[j] = da; b[j] = db;
    }
    st16_stream(DA + v * VEC, VT<T>::pack(a));
    st16_stream(DB + v * VEC, VT<T>::pack(b));
  }
  for (int64_t e = n_vec * VEC + (int64_t)blockIdx.x * 256 + threadIdx.x; e < n; e += stride) {
    float da, db;
    swiglu_bwd_elem<T, ACT>(VT<T>::load1(A + e), VT<T>::load1(B + e), VT<T>::load1(DC + e), da, db);
    VT<T>::store1(DA + e, da);
    VT<T>::store1(DB + e, db);
  }
}

static inline unsigned stream_grid(int64_t n_vec, int64_t n) {
  int64_t work = n_vec > 0 ? (n_vec + SW_UNROLL - 1) / SW_UNROLL : n;
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

template <typename T, int ACT>
static int swiglu_fwd_t(const void* a, const void* b, void* c, int64_t n, cudaStream_t st) {
  const bool al = aligned16(a) && aligned16(b) && aligned16(c);
  const int64_t n_vec = al ? n / VT<T>::N : 0;
  swiglu_fwd_kernel<T, ACT><<<stream_grid(n_vec, n), 256, 0, st>>>((const T*)a, (const T*)b, (T*)c, n_vec, n);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
template <typename T, int ACT>
static int swiglu_bwd_t(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, cudaStream_t st) {
  const bool al = aligned16(a) && aligned16(b) && aligned16(dc) && aligned16(da) && aligned16(db);
  const int64_t n_vec = al ? n / VT<T>::N : 0;
  swiglu_bwd_kernel<T, ACT><<<stream_grid(n_vec, n), 256, 0, st>>>((const T*)a, (const T*)b, (const T*)dc, (T*)da, (T*)db,
                                                              n_vec, n);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // namespace hilda

using namespace hilda;

template <int ACT>
static int glu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype, void* stream) {
  if (!a || !b || !c) return HILDA_ERR_NULL;
  if (n < 0) return HILDA_ERR_SIZE;
  if (n == 0) return HILDA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return swiglu_fwd_t<float, ACT>(a, b, c, n, st);
    case HILDA_BF16: return swiglu_fwd_t<__nv_bfloat16, ACT>(a, b, c, n, st);
    case HILDA_F16: return swiglu_fwd_t<__half, ACT>(a, b, c, n, st);
  }
  return HILDA_ERR_DTYPE;
}
template <int ACT>
static int glu_bwd(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, int dtype, void* stream) {
  if (!a || !b || !dc || !da || !db) return HILDA_ERR_NULL;
  if (n < 0) return HILDA_ERR_SIZE;
  if (n == 0) return HILDA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return swiglu_bwd_t<float, ACT>(a, b, dc, da, db, n, st);
    case HILDA_BF16: return swiglu_bwd_t<__nv_bfloat16, ACT>(a, b, dc, da, db, n, st);
    case HILDA_F16: return swiglu_bwd_t<__half, ACT>(a, b, dc, da, db, n, st);
  }
  return HILDA_ERR_DTYPE;
}

extern "C" {

int hilda_swiglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype, void* stream) {
  return glu_fwd<ACT_SILU>(a, b, c, n, dtype, stream);
}
int hilda_swiglu_bwd(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, int dtype,
                     void* stream) {
  return glu_bwd<ACT_SILU>(a, b, dc, da, db, n, dtype, stream);
}
int hilda_geglu_fwd(const void* a, const void* b, void* c, int64_t n, int dtype, void* stream) {
  return glu_fwd<ACT_GELU_TANH>(a, b, c, n, dtype, stream);
}
int hilda_geglu_bwd(const void* a, const void* b, const void* dc, void* da, void* db, int64_t n, int dtype,
                    void* stream) {
  return glu_bwd<ACT_GELU_TANH>(a, b, dc, da, db, n, dtype, stream);
}

}  // extern "C"
