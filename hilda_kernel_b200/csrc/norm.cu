// RMSNorm and FusedAddRMSNorm, forward and backward, for sm_100a.
//
// Behaviour follows the reference kernels (kernels/rms_norm.py:78-142, :200-254 and
// kernels/fused_add_rms_norm.py:40-77, :122-165 of hilda-kernel):
//   forward : s = x (+ r, rounded to the input dtype); rstd = 1/sqrt(mean(s^2)+eps) in fp32;
//             y = round_T(s * rstd) * w; only rstd is saved.
//   backward: m = dy*w; dx = rstd*m - rstd^3 * (sum(m*s)/H) * s (+ ds); dW = sum_rows dy*(s*rstd).
// Design: one CTA owns one row at a time and keeps it in registers as 128-bit vectors, so each
// tensor is read once and written once. dW is accumulated per CTA in registers over the rows it
// owns, written as one fp32 partial row per CTA, and reduced by a second small kernel (fixed
// order, no atomics, bit-reproducible).
#include <cstdlib>
#include <type_traits>
#include "common.cuh"

namespace hilda {

// W (dtype only known at run time) -> VEC floats starting at element e0 (e0 % VEC == 0).
template <int VEC>
__device__ __forceinline__ void load_w_vec(const void* W, int w_dt, int e0, float* out) {
  if (w_dt == HILDA_F32) {
    const float* p = reinterpret_cast<const float*>(W) + e0;
#pragma unroll
    for (int j = 0; j < VEC; j += 4) VT<float>::unpack(ld16(p + j), out + j);
  } else if (w_dt == HILDA_BF16) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(W) + e0;
    if constexpr (VEC == 8) {
      VT<__nv_bfloat16>::unpack(ld16(p), out);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[j] = __bfloat162float(p[j]);
    }
  } else {
    const __half* p = reinterpret_cast<const __half*>(W) + e0;
    if constexpr (VEC == 8) {
      VT<__half>::unpack(ld16(p), out);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[j] = __half2float(p[j]);
    }
  }
}

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
norm_fwd_kernel(const T* __restrict__ X, const T* __restrict__ R, const void* __restrict__ W, int w_dt,
                T* __restrict__ Y, T* __restrict__ S, float* __restrict__ RSTD,
                int64_t n_rows, int n_cols, float eps) {
  constexpr int VEC = VT<T>::N;
  const int n_vec = n_cols / VEC;
  __shared__ float red[33];
  const int tid = threadIdx.x;

  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const T* xr = X + row * n_cols;
    uint4 xv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      xv[i] = (v < n_vec) ? ld16_stream(xr + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
    }
    if (R != nullptr) {
      const T* rr = R + row * n_cols;
      T* sr = S + row * n_cols;
      uint4 rv[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * THREADS;
        rv[i] = (v < n_vec) ? ld16_stream(rr + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * THREADS;
        float a[VEC], b[VEC];
        VT<T>::unpack(xv[i], a);
        VT<T>::unpack(rv[i], b);
#pragma unroll
        for (int j = 0; j < VEC; ++j) a[j] = a[j] + b[j];  // rounded to T by pack()
        xv[i] = VT<T>::pack(a);
        if (v < n_vec) st16(sr + (int64_t)v * VEC, xv[i]);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float a[VEC];
      VT<T>::unpack(xv[i], a);
#pragma unroll
      for (int j = 0; j < VEC; ++j) ss = fmaf(a[j], a[j], ss);
    }
    ss = block_sum<THREADS>(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)n_cols + eps);
    if (tid == 0) RSTD[row] = rstd;
    T* yr = Y + row * n_cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      if (v < n_vec) {
        float a[VEC], w[VEC];
        VT<T>::unpack(xv[i], a);
        load_w_vec<VEC>(W, w_dt, v * VEC, w);
#pragma unroll
        for (int j = 0; j < VEC; ++j) a[j] = VT<T>::round(a[j] * rstd) * w[j];
        st16(yr + (int64_t)v * VEC, VT<T>::pack(a));
      }
    }
  }
}

// 16-bit rows without the residual stream, w in the data's dtype: the next row's loads are issued before
// the current row is reduced (one row per CTA is in flight the whole time, not only while it loads), w
// is held packed in registers, and the second rounding is the packed multiply itself:
// round_T(round_T(x * rstd) * w) == hmul2(pack(x * rstd), w), the exact product rounded once.
template <typename T, int THREADS, int VPT, bool FULL>
__global__ void __launch_bounds__(THREADS)
norm_fwd16_kernel(const T* __restrict__ X, const T* __restrict__ W, T* __restrict__ Y, float* __restrict__ RSTD,
                  int64_t n_rows, int n_cols_rt, float eps) {
  using P2 = typename std::conditional<std::is_same<T, __nv_bfloat16>::value, __nv_bfloat162, __half2>::type;
  constexpr int VEC = 8;
  const int n_cols = FULL ? VEC * THREADS * VPT : n_cols_rt;
  const int n_vec = n_cols / VEC;
  __shared__ float red[33];
  const int tid = threadIdx.x;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  bool ok[VPT];
  uint4 wv[VPT], cur[VPT], nxt[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    ok[i] = FULL || (tid + i * THREADS < n_vec);
    wv[i] = ok[i] ? ld16(W + (tid + i * THREADS) * VEC) : zero4;
  }
  const int64_t step = (int64_t)gridDim.x * n_cols;
  int64_t off = (int64_t)blockIdx.x * n_cols + (int64_t)tid * VEC;
  if ((int64_t)blockIdx.x < n_rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) cur[i] = ok[i] ? ld16_stream(X + off + i * (THREADS * VEC)) : zero4;
  }
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x, off += step) {
    const bool more = row + gridDim.x < n_rows;
#pragma unroll
    for (int i = 0; i < VPT; ++i) nxt[i] = (more && ok[i]) ? ld16_stream(X + off + step + i * (THREADS * VEC)) : zero4;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float a[VEC];
      VT<T>::unpack(cur[i], a);
#pragma unroll
      for (int j = 0; j < VEC; ++j) ss = fmaf(a[j], a[j], ss);
    }
    ss = block_sum<THREADS>(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)n_cols + eps);
    if (tid == 0) RSTD[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (ok[i]) {
        float a[VEC];
        VT<T>::unpack(cur[i], a);
#pragma unroll
        for (int j = 0; j < VEC; ++j) a[j] *= rstd;
        uint4 n4 = VT<T>::pack(a);
        P2* n2 = reinterpret_cast<P2*>(&n4);
        const P2* w2 = reinterpret_cast<const P2*>(&wv[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) n2[j] = __hmul2(n2[j], w2[j]);
        st16(Y + off + i * (THREADS * VEC), n4);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) cur[i] = nxt[i];
  }
}

// Any n_cols (no alignment requirement): scalar access, row re-read from L1/L2.
template <typename T>
__global__ void __launch_bounds__(256)
norm_fwd_generic_kernel(const T* __restrict__ X, const T* __restrict__ R, const void* __restrict__ W, int w_dt,
                        T* __restrict__ Y, T* __restrict__ S, float* __restrict__ RSTD,
                        int64_t n_rows, int64_t n_cols, float eps) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const T* xr = X + row * n_cols;
    const T* rr = R ? R + row * n_cols : nullptr;
    T* sr = S ? S + row * n_cols : nullptr;
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < n_cols; c += 256) {
      float s = VT<T>::load1(xr + c);
      if (rr) {
        s = VT<T>::round(s + VT<T>::load1(rr + c));
        VT<T>::store1(sr + c, s);
      }
      ss = fmaf(s, s, ss);
    }
    ss = block_sum<256>(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)n_cols + eps);
    if (threadIdx.x == 0) RSTD[row] = rstd;
    T* yr = Y + row * n_cols;
    for (int64_t c = threadIdx.x; c < n_cols; c += 256) {
      // each thread re-reads exactly the elements it wrote above
      float s = rr ? VT<T>::load1(sr + c) : VT<T>::load1(xr + c);
      VT<T>::store1(yr + c, VT<T>::round(s * rstd) * load_any(W, w_dt, c));
    }
  }
}

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS, (sizeof(T) == 2 && VPT <= 2) ? (1024 / THREADS) : 1)
norm_bwd_kernel(const T* __restrict__ dY, const T* __restrict__ dS, const T* __restrict__ X,
                const void* __restrict__ W, int w_dt, const float* __restrict__ RSTD,
                T* __restrict__ dX, float* __restrict__ partial, int64_t n_rows, int n_cols, int prefetch_rows) {
  constexpr int VEC = VT<T>::N;
  const int n_vec = n_cols / VEC;
  __shared__ float red[33];
  const int tid = threadIdx.x;
  const float inv_n = 1.0f / (float)n_cols;

  // w is re-read per row (an L1 hit after the first row) rather than held in registers.
  float dw[VPT][VEC];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < VEC; ++j) dw[i][j] = 0.f;

  const uint32_t row_bytes = (uint32_t)n_cols * (uint32_t)sizeof(T);
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    // Optional: one thread asks the L2 for the rows this CTA reaches `prefetch_rows` iterations from now
    // (bulk prefetch, one instruction per tensor row), so that their loads find them on chip.
    if (prefetch_rows > 0 && threadIdx.x == 0) {
      const int64_t ahead = row + (int64_t)prefetch_rows * gridDim.x;
      if (ahead < n_rows) {
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(X + ahead * n_cols), "r"(row_bytes) : "memory");
        if (dY) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(dY + ahead * n_cols), "r"(row_bytes) : "memory");
        if (dS) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(dS + ahead * n_cols), "r"(row_bytes) : "memory");
      }
    }
    // all of the row's loads (dS too) are issued before the reduction: one DRAM round trip per row
    uint4 dyv[VPT], xv[VPT], dsv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      const bool ok = v < n_vec;
      dyv[i] = (ok && dY) ? ld16_stream(dY + row * n_cols + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
      xv[i] = ok ? ld16_stream(X + row * n_cols + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
      dsv[i] = (ok && dS) ? ld16_stream(dS + row * n_cols + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
    }
    const float rstd = RSTD[row];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      float dy[VEC], x[VEC], w[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (v < n_vec) {
        load_w_vec<VEC>(W, w_dt, v * VEC, w);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc = fmaf(dy[j] * w[j], x[j], acc);
      }
    }
    acc = block_sum<THREADS>(acc, red);
    const float coef = rstd * rstd * rstd * (acc * inv_n);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      float dy[VEC], x[VEC], dx[VEC], w[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (v < n_vec) {
        load_w_vec<VEC>(W, w_dt, v * VEC, w);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          dx[j] = rstd * (dy[j] * w[j]) - coef * x[j];
          dw[i][j] = fmaf(dy[j], x[j] * rstd, dw[i][j]);
        }
        if (dS != nullptr) {
          float ds[VEC];
          VT<T>::unpack(dsv[i], ds);
#pragma unroll
          for (int j = 0; j < VEC; ++j) dx[j] += ds[j];
        }
        st16(dX + row * n_cols + (int64_t)v * VEC, VT<T>::pack(dx));
      }
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the second pass may start launching
  float* pr = partial + (int64_t)blockIdx.x * n_cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * THREADS;
    if (v < n_vec) {
#pragma unroll
      for (int j = 0; j < VEC; j += 4)
        st16(pr + (int64_t)v * VEC + j, VT<float>::pack(&dw[i][j]));
    }
  }
}

// ---- 16-bit backward for rows that fill the plan exactly -----------------------------------------
// The general kernel above spends about as many instructions on bounds tests, 64-bit row offsets and the
// per-vector fetch of w as on the arithmetic, and for 16-bit rows it is instruction issue, not HBM,
// that bounds it (28 instructions per element, 60 % of the issue slots busy at 0.89 of HBM). This
// kernel serves the common case only: 16-bit rows of up to 8192 elements, w in the data's own dtype, dY
// present. w is unpacked once into registers, the row pointers advance by a constant, and the bounds
// tests are per-thread flags set once (none at all when the row fills the plan exactly).
// Same arithmetic as norm_bwd_kernel; the sums are grouped by this kernel's own thread plan and its own,
// smaller grid (three or two CTAs per SM), so dX and dW agree with the other kernels' within rounding, not
// bit for bit. Measured on B200, bf16 (TB/s of dY, x and dX): [16384,4096] 5.77 against 4.85 (with dS 88.7 us
// against 91.9), [32768,2048] 5.86 against 4.99, H = 3072 5.12 against 4.33, 5120 4.94 against 3.90, 7168 5.56
// against 4.58, 8192 5.02 against 4.71.
template <typename T, int THREADS, int VPT, bool HAS_DS, bool FULL>
__global__ void __launch_bounds__(THREADS, (VPT <= 2 ? 768 : 512) / THREADS)
norm_bwd16_kernel(const T* __restrict__ dY, const T* __restrict__ dS, const T* __restrict__ X,
                  const T* __restrict__ W, const float* __restrict__ RSTD, T* __restrict__ dX,
                  float* __restrict__ partial, int64_t n_rows, int n_cols_rt, int prefetch_rows) {
  constexpr int VEC = 8;
  // FULL: the row fills the plan exactly (n_cols == 8 * THREADS * VPT), nothing is predicated
  const int n_cols = FULL ? VEC * THREADS * VPT : n_cols_rt;
  const int n_vec = n_cols / VEC;
  __shared__ float red[33];
  const int tid = threadIdx.x;
  const float inv_n = 1.0f / (float)n_cols;
  bool ok[VPT];
  float w[VPT][VEC], dw[VPT][VEC];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    ok[i] = FULL || (tid + i * THREADS < n_vec);
#pragma unroll
    for (int j = 0; j < VEC; ++j) { w[i][j] = 0.f; dw[i][j] = 0.f; }
    if (ok[i]) VT<T>::unpack(ld16(W + (tid + i * THREADS) * VEC), w[i]);
  }
  const int64_t step = (int64_t)gridDim.x * n_cols;
  int64_t off = (int64_t)blockIdx.x * n_cols + (int64_t)tid * VEC;
  const uint32_t row_bytes = (uint32_t)n_cols * (uint32_t)sizeof(T);
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x, off += step) {
    if (prefetch_rows > 0 && tid == 0) {
      const int64_t ahead = row + (int64_t)prefetch_rows * gridDim.x;
      if (ahead < n_rows) {
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(X + ahead * n_cols), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(dY + ahead * n_cols), "r"(row_bytes) : "memory");
        if (HAS_DS) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(dS + ahead * n_cols), "r"(row_bytes) : "memory");
      }
    }
    uint4 dyv[VPT], xv[VPT], dsv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      dyv[i] = ok[i] ? ld16_stream(dY + off + i * (THREADS * VEC)) : zero4;
      xv[i] = ok[i] ? ld16_stream(X + off + i * (THREADS * VEC)) : zero4;
      if (HAS_DS) dsv[i] = ok[i] ? ld16_stream(dS + off + i * (THREADS * VEC)) : zero4;
    }
    const float rstd = RSTD[row];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float dy[VEC], x[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (ok[i]) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc = fmaf(dy[j] * w[i][j], x[j], acc);
      }
    }
    acc = block_sum<THREADS>(acc, red);
    const float coef = rstd * rstd * rstd * (acc * inv_n);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float dy[VEC], x[VEC], dx[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (ok[i]) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          dx[j] = rstd * (dy[j] * w[i][j]) - coef * x[j];
          dw[i][j] = fmaf(dy[j], x[j] * rstd, dw[i][j]);
        }
        if (HAS_DS) {
          float ds[VEC];
          VT<T>::unpack(dsv[i], ds);
#pragma unroll
          for (int j = 0; j < VEC; ++j) dx[j] += ds[j];
        }
        st16(dX + off + i * (THREADS * VEC), VT<T>::pack(dx));
      }
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the second pass may start launching
  float* pr = partial + (int64_t)blockIdx.x * n_cols + (int64_t)tid * VEC;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (ok[i]) {
#pragma unroll
      for (int j = 0; j < VEC; j += 4) st16(pr + i * (THREADS * VEC) + j, VT<float>::pack(&dw[i][j]));
    }
  }
}

// ---- backward with the row loads decoupled from the arithmetic --------------------------------
// norm_bwd_kernel above keeps ONE row per CTA in flight and goes load -> block reduction -> store, so
// every row exposes a DRAM round trip (2 CTAs of 122 registers per SM for fp32: about 64 KB in
// flight per SM, and only during the load phase). Here a CTA owns a ring of `stages` shared-memory
// slots; one thread fills a slot with the row's dY, X (and dS) by bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier) and refills it as soon as the CTA has taken the
// row into registers, so `stages` rows per CTA are in flight the whole time while the CTA reduces
// and stores the current one. Same arithmetic, same order, same results as norm_bwd_kernel.
__device__ __forceinline__ uint32_t nb_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void nb_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool nb_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
constexpr uint32_t NB_WAIT_CAP = 1u << 24;  // try_wait attempts (each suspends for a while) before giving up
constexpr int NB_MAX_STAGES = 6;

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS, (sizeof(T) == 2 && VPT <= 2) ? (1024 / THREADS) : 1)
norm_bwd_ring_kernel(const T* __restrict__ dY, const T* __restrict__ dS, const T* __restrict__ X,
                     const void* __restrict__ W, int w_dt, const float* __restrict__ RSTD,
                     T* __restrict__ dX, float* __restrict__ partial, int64_t n_rows, int n_cols, int stages) {
  constexpr int VEC = VT<T>::N;
  // dynamic shared memory: W as fp32 [n_cols] (the ring takes most of the SM's L1 away, so W would
  // otherwise come from L2 twice per row), then the ring slots
  extern __shared__ __align__(128) uint8_t ring_raw[];
  float* w_s = reinterpret_cast<float*>(ring_raw);
  uint8_t* ring = ring_raw + (size_t)n_cols * 4;
  __shared__ __align__(8) uint64_t full_bar[NB_MAX_STAGES];
  __shared__ float red[33];
  __shared__ int gave_up;
  const int n_vec = n_cols / VEC;
  const int tid = threadIdx.x;
  const float inv_n = 1.0f / (float)n_cols;
  const uint32_t row_bytes = (uint32_t)n_cols * (uint32_t)sizeof(T);
  const int n_tensors = 1 + (dY ? 1 : 0) + (dS ? 1 : 0);
  const uint32_t stage_bytes = row_bytes * n_tensors;
  // slot layout: X, then dY (if any), then dS (if any)
  const uint32_t off_dy = row_bytes, off_ds = row_bytes * (dY ? 2u : 1u);
  const uint32_t ring0 = nb_smem_u32(ring), bar0 = nb_smem_u32(full_bar);
  const int64_t n_mine = (n_rows > (int64_t)blockIdx.x) ? (n_rows - 1 - blockIdx.x) / gridDim.x + 1 : 0;

  auto issue = [&](int64_t it) {  // thread 0 only: fill slot it % stages with this CTA's it-th row
    const int s = (int)(it % stages);
    const int64_t row = (int64_t)blockIdx.x + it * gridDim.x;
    const uint32_t dst = ring0 + (uint32_t)s * stage_bytes, bar = bar0 + 8u * s;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_bytes) : "memory");
    nb_bulk_load(dst, X + row * n_cols, row_bytes, bar);
    if (dY) nb_bulk_load(dst + off_dy, dY + row * n_cols, row_bytes, bar);
    if (dS) nb_bulk_load(dst + off_ds, dS + row * n_cols, row_bytes, bar);
  };

  if (tid == 0) {
    for (int s = 0; s < stages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8u * s) : "memory");
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int64_t it = 0; it < n_mine && it < stages; ++it) issue(it);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * THREADS;
    if (v < n_vec) {
      float w[VEC];
      load_w_vec<VEC>(W, w_dt, v * VEC, w);
#pragma unroll
      for (int j = 0; j < VEC; ++j) w_s[v * VEC + j] = w[j];
    }
  }
  __syncthreads();

  float dw[VPT][VEC];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < VEC; ++j) dw[i][j] = 0.f;

  int64_t it = 0;
  for (; it < n_mine; ++it) {
    const int s = (int)(it % stages);
    const uint32_t parity = (uint32_t)((it / stages) & 1);
    const int64_t row = (int64_t)blockIdx.x + it * gridDim.x;
    const float rstd = RSTD[row];
    bool ok = false;
    for (uint32_t t = 0; t < NB_WAIT_CAP; ++t)
      if (nb_try_wait(bar0 + 8u * s, parity)) { ok = true; break; }
    if (!ok) gave_up = 1;  // reported below; every thread sees the same barrier, so all or none get here
    const uint8_t* slot = ring + (size_t)s * stage_bytes;
    uint4 dyv[VPT], xv[VPT], dsv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      const bool in = v < n_vec;
      xv[i] = in ? *reinterpret_cast<const uint4*>(slot + (size_t)v * 16) : make_uint4(0, 0, 0, 0);
      dyv[i] = (in && dY) ? *reinterpret_cast<const uint4*>(slot + off_dy + (size_t)v * 16) : make_uint4(0, 0, 0, 0);
      dsv[i] = (in && dS) ? *reinterpret_cast<const uint4*>(slot + off_ds + (size_t)v * 16) : make_uint4(0, 0, 0, 0);
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      float dy[VEC], x[VEC], w[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (v < n_vec) {
#pragma unroll
        for (int j = 0; j < VEC; j += 4) {
          const float4 t4 = *reinterpret_cast<const float4*>(w_s + v * VEC + j);
          w[j] = t4.x; w[j + 1] = t4.y; w[j + 2] = t4.z; w[j + 3] = t4.w;
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc = fmaf(dy[j] * w[j], x[j], acc);
      }
    }
    // the block sum's barriers also mean: every thread has taken its part of the slot into registers
    acc = block_sum<THREADS>(acc, red);
    if (gave_up) break;
    if (tid == 0 && it + stages < n_mine) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the reads above before the refill below
      issue(it + stages);
    }
    const float coef = rstd * rstd * rstd * (acc * inv_n);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * THREADS;
      float dy[VEC], x[VEC], dx[VEC], w[VEC];
      VT<T>::unpack(dyv[i], dy);
      VT<T>::unpack(xv[i], x);
      if (v < n_vec) {
#pragma unroll
        for (int j = 0; j < VEC; j += 4) {
          const float4 t4 = *reinterpret_cast<const float4*>(w_s + v * VEC + j);
          w[j] = t4.x; w[j + 1] = t4.y; w[j + 2] = t4.z; w[j + 3] = t4.w;
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          dx[j] = rstd * (dy[j] * w[j]) - coef * x[j];
          dw[i][j] = fmaf(dy[j], x[j] * rstd, dw[i][j]);
        }
        if (dS != nullptr) {
          float ds[VEC];
          VT<T>::unpack(dsv[i], ds);
#pragma unroll
          for (int j = 0; j < VEC; ++j) dx[j] += ds[j];
        }
        st16(dX + row * n_cols + (int64_t)v * VEC, VT<T>::pack(dx));
      }
    }
  }
  if (gave_up) {
    // A wait ran out (it never should: the copies are this CTA's own). Say so loudly, NaN in this CTA's
    // partial sums and therefore in dW, and before leaving wait, again bounded, for the copies still
    // in flight into this CTA's shared memory.
    for (int64_t j = it; j < n_mine && j < it + stages; ++j)
      for (uint32_t t = 0; t < NB_WAIT_CAP; ++t)
        if (nb_try_wait(bar0 + 8u * (int)(j % stages), (uint32_t)((j / stages) & 1))) break;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < VEC; ++j) dw[i][j] = __int_as_float(0x7fc00000);
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the second pass may start launching
  float* pr = partial + (int64_t)blockIdx.x * n_cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * THREADS;
    if (v < n_vec) {
#pragma unroll
      for (int j = 0; j < VEC; j += 4)
        st16(pr + (int64_t)v * VEC + j, VT<float>::pack(&dw[i][j]));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
norm_bwd_generic_kernel(const T* __restrict__ dY, const T* __restrict__ dS, const T* __restrict__ X,
                        const void* __restrict__ W, int w_dt, const float* __restrict__ RSTD,
                        T* __restrict__ dX, float* __restrict__ partial, int64_t n_rows, int64_t n_cols) {
  __shared__ float red[33];
  float* pr = partial + (int64_t)blockIdx.x * n_cols;
  for (int64_t c = threadIdx.x; c < n_cols; c += 256) pr[c] = 0.f;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const T* dyr = dY ? dY + row * n_cols : nullptr;
    const T* xr = X + row * n_cols;
    const float rstd = RSTD[row];
    float acc = 0.f;
    for (int64_t c = threadIdx.x; c < n_cols; c += 256) {
      const float dy = dyr ? VT<T>::load1(dyr + c) : 0.f;
      acc = fmaf(dy * load_any(W, w_dt, c), VT<T>::load1(xr + c), acc);
    }
    acc = block_sum<256>(acc, red);
    const float coef = rstd * rstd * rstd * (acc / (float)n_cols);
    for (int64_t c = threadIdx.x; c < n_cols; c += 256) {
      const float dy = dyr ? VT<T>::load1(dyr + c) : 0.f;
      const float x = VT<T>::load1(xr + c);
      float dx = rstd * (dy * load_any(W, w_dt, c)) - coef * x;
      if (dS) dx += VT<T>::load1(dS + row * n_cols + c);
      VT<T>::store1(dX + row * n_cols + c, dx);
      pr[c] = fmaf(dy, x * rstd, pr[c]);  // same thread owns column c for every row
    }
  }
}

// partial [P, n_cols] fp32 -> dW [n_cols] in W's dtype. 32 columns x 32 row-groups per CTA.
__global__ void __launch_bounds__(1024)
dw_reduce_kernel(const float* __restrict__ partial, int P, int64_t n_cols, void* __restrict__ dW, int w_dt) {
  __shared__ float tile[32][33];
  // launched with programmatic stream serialisation: its CTAs may become resident while the backward
  // kernel drains; nothing is read before that kernel has completed and its writes are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int cx = threadIdx.x & 31, gy = threadIdx.x >> 5;
  const int64_t col = (int64_t)blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (col < n_cols) {
    // four loads in flight per thread; the order of the additions stays fixed
    int p = gy;
    for (; p + 96 < P; p += 128) {
      const float a0 = partial[(int64_t)p * n_cols + col], a1 = partial[(int64_t)(p + 32) * n_cols + col];
      const float a2 = partial[(int64_t)(p + 64) * n_cols + col], a3 = partial[(int64_t)(p + 96) * n_cols + col];
      acc += a0; acc += a1; acc += a2; acc += a3;
    }
    for (; p < P; p += 32) acc += partial[(int64_t)p * n_cols + col];
  }
  tile[gy][cx] = acc;
  __syncthreads();
  if (gy == 0 && col < n_cols) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) t += tile[g][cx];
    store_any(dW, w_dt, col, t);
  }
}

// ---- host-side dispatch --------------------------------------------------------
struct NormPlan { int threads; int vpt; bool generic; };

static NormPlan plan_norm(int64_t n_cols, int vec, int pref_vpt, bool all_aligned) {
  NormPlan p{256, 1, true};
  if (!all_aligned || n_cols % vec != 0) return p;
  const int64_t n_vec = n_cols / vec;
  int vpt = pref_vpt;
  while (vpt > 1 && n_vec <= 128 * (vpt / 2)) vpt >>= 1;  // fewer vectors per thread only if 128 threads still cover the row
  while (vpt < 8 && n_vec > (int64_t)vpt * 1024) vpt <<= 1;
  if (n_vec > (int64_t)vpt * 1024) return p;
  int threads = 128;
  while ((int64_t)threads * vpt < n_vec) threads <<= 1;
  p.threads = threads; p.vpt = vpt; p.generic = false;
  return p;
}

#define NORM_DISPATCH_TV(T, CALL)                                                     \
  switch (plan.threads * 16 + plan.vpt) {                                             \
    case 128 * 16 + 1: CALL(T, 128, 1); break;  case 128 * 16 + 2: CALL(T, 128, 2); break;   \
    case 128 * 16 + 4: CALL(T, 128, 4); break;  case 128 * 16 + 8: CALL(T, 128, 8); break;   \
    case 256 * 16 + 1: CALL(T, 256, 1); break;  case 256 * 16 + 2: CALL(T, 256, 2); break;   \
    case 256 * 16 + 4: CALL(T, 256, 4); break;  case 256 * 16 + 8: CALL(T, 256, 8); break;   \
    case 512 * 16 + 1: CALL(T, 512, 1); break;  case 512 * 16 + 2: CALL(T, 512, 2); break;   \
    case 512 * 16 + 4: CALL(T, 512, 4); break;  case 512 * 16 + 8: CALL(T, 512, 8); break;   \
    case 1024 * 16 + 1: CALL(T, 1024, 1); break; case 1024 * 16 + 2: CALL(T, 1024, 2); break; \
    case 1024 * 16 + 4: CALL(T, 1024, 4); break; case 1024 * 16 + 8: CALL(T, 1024, 8); break; \
    default: return HILDA_ERR_SIZE;                                                   \
  }

// HILDA_NORM_FWD16=0 keeps the general forward kernel for every shape (comparisons). Measured on B200, bf16,
// TB/s of x and y, lean against general: H = 3072 5.91 / 5.33, 4096 6.14 / 5.94, 5120 5.42 / 4.49, 7168 6.03 / 5.18,
// 8192 6.13 / 5.42.
static bool norm_fwd16_enabled() {
  static const bool v = []() { const char* e = getenv("HILDA_NORM_FWD16"); return e ? atoi(e) != 0 : true; }();
  return v;
}

template <typename T>
static int norm_fwd_t(const void* x, const void* r, const void* w, int w_dt, void* y, void* s, float* rstd,
                      int64_t n_rows, int64_t n_cols, float eps, cudaStream_t st) {
  const bool al = aligned16(x) && aligned16(y) && aligned16(w) && (!r || (aligned16(r) && aligned16(s)));
  // 16-bit rows without the residual stream keep four vectors per thread in flight (half as many threads
  // per row, twice as many rows per SM): bf16 [16384,4096] 5.90 against 4.98 TB/s, [8192,8192] 5.43 against
  // 3.89, [13107,5120] 4.49 against 2.94; with the residual stream two per thread measured best
  const int pref = (sizeof(T) == 4) ? 4 : ((r && n_cols <= 4096) ? 2 : 4);
  NormPlan plan = plan_norm(n_cols, VT<T>::N, pref, al);
  const int64_t max_grid = (int64_t)sm_count() * 64;
  if (plan.generic) {
    int grid = (int)(n_rows < max_grid ? n_rows : max_grid);
    norm_fwd_generic_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (const T*)r, w, w_dt, (T*)y, (T*)s, rstd,
                                                       n_rows, n_cols, eps);
    HILDA_LAUNCH_CHECK();
    return HILDA_OK;
  }
  int grid = (int)(n_rows < max_grid ? n_rows : max_grid);
  if constexpr (sizeof(T) == 2) {
    const int64_t nv16 = n_cols / 8;
    if (!r && w_dt == (std::is_same<T, __nv_bfloat16>::value ? HILDA_BF16 : HILDA_F16) && nv16 > 128 && nv16 <= 1024 &&
        ((plan.vpt == 4 && (plan.threads == 128 || plan.threads == 256)) || (plan.vpt == 2 && plan.threads == 128)) &&
        norm_fwd16_enabled()) {
#define F16_CALL(TH, VP, FU)                                                                                \
  do {                                                                                                      \
    int occ = 0;  /* rows are walked with a grid stride and prefetched: a grid of resident CTAs */           \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, norm_fwd16_kernel<T, TH, VP, FU>, TH, 0) == cudaSuccess && \
        occ > 0 && grid > occ * sm_count())                                                                 \
      grid = occ * sm_count();                                                                              \
    norm_fwd16_kernel<T, TH, VP, FU><<<grid, TH, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, n_rows, (int)n_cols, eps); \
  } while (0)
      const bool fu = nv16 == (int64_t)plan.threads * plan.vpt;
      if (plan.vpt == 2) { if (fu) F16_CALL(128, 2, true); else F16_CALL(128, 2, false); }
      else if (plan.threads == 128) { if (fu) F16_CALL(128, 4, true); else F16_CALL(128, 4, false); }
      else { if (fu) F16_CALL(256, 4, true); else F16_CALL(256, 4, false); }
#undef F16_CALL
      HILDA_LAUNCH_CHECK();
      return HILDA_OK;
    }
  }
#define FWD_CALL(TT, TH, VP)                                                                            \
  norm_fwd_kernel<TT, TH, VP><<<grid, TH, 0, st>>>((const TT*)x, (const TT*)r, w, w_dt, (TT*)y, (TT*)s, rstd, \
                                                    n_rows, (int)n_cols, eps)
  NORM_DISPATCH_TV(T, FWD_CALL)
#undef FWD_CALL
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// Number of CTAs (= rows of the fp32 partial buffer) the backward uses.
template <typename T>
static int norm_bwd_ctas(int64_t n_rows, int64_t n_cols, bool al) {
  const int pref = (sizeof(T) == 4) ? 4 : 2;
  NormPlan plan = plan_norm(n_cols, VT<T>::N, pref, al);
  int per_sm = 4;
  if (!plan.generic) {
#define OCC_CALL(TT, TH, VP) \
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, norm_bwd_kernel<TT, TH, VP>, TH, 0)
    NORM_DISPATCH_TV(T, OCC_CALL)
#undef OCC_CALL
    if (per_sm < 1) per_sm = 1;
  }
  int64_t ctas = (int64_t)sm_count() * per_sm;
  if (ctas > n_rows) ctas = n_rows;
  if (ctas < 1) ctas = 1;
  return (int)ctas;
}

// The second pass, launched so that it may be scheduled while the backward kernel is still draining
// (programmatic dependent launch; the kernel itself waits for the backward's completion).
static int launch_dw_reduce(const float* partial, int P, int64_t n_cols, void* dw, int w_dt, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((n_cols + 31) / 32), 1, 1);
  cfg.blockDim = dim3(1024, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, dw_reduce_kernel, partial, P, n_cols, dw, w_dt) == cudaSuccess ? HILDA_OK : HILDA_ERR_CUDA;
}

// Kernel choice of the backward for vectorisable shapes (per host thread; HILDA_NORM_RING presets it):
//   1 (default) automatic: for 32-bit rows the shared-memory ring (norm_bwd_ring_kernel) when three or more
//     row slots fit beside the SM's other CTAs; else, and for 16-bit rows always, the register kernel with
//     an L2 bulk prefetch one row ahead (16-bit rows that fill the plan exactly: its lean form,
//     norm_bwd16_kernel).
//     Measured on B200: fp32 [4096,4096] (3 slots, 2 CTAs per SM) ring 37.6 us, register kernel 42.0,
//     with prefetch 38.8; bf16 [16384,4096] with dS (2 slots, 4 CTAs per SM) ring 101.7 us, register
//     kernel 100.5, with prefetch one row ahead 93.5, two rows ahead 96.7.
//   0 register kernel, no prefetch; 2 / 3 register kernel with prefetch 1 / 2 rows ahead; 4 ring whenever
//     two slots fit.
static int norm_ring_default() {
  static const int v = []() { const char* e = getenv("HILDA_NORM_RING"); return e ? atoi(e) : 1; }();
  return v;
}
static thread_local int g_norm_ring = norm_ring_default();

template <typename T>
static int norm_bwd_t(const void* dy, const void* ds, const void* x, const void* w, int w_dt, const float* rstd,
                      void* dx, void* dw, float* workspace, int64_t n_rows, int64_t n_cols, cudaStream_t st,
                      int64_t max_ctas = 0) {
  const bool al = aligned16(x) && aligned16(dx) && aligned16(w) && aligned16(workspace) &&
                  (!dy || aligned16(dy)) && (!ds || aligned16(ds));
  const int pref = (sizeof(T) == 4) ? 4 : 2;
  NormPlan plan = plan_norm(n_cols, VT<T>::N, pref, al);
  // The workspace is sized for the aligned plan; a misaligned call uses no more CTAs than that.
  int grid = norm_bwd_ctas<T>(n_rows, n_cols, true);
  if (max_ctas > 0 && grid > max_ctas) grid = (int)max_ctas;  // the rows are walked with a grid stride: any grid is correct
  if (plan.generic) {
    int g2 = norm_bwd_ctas<T>(n_rows, n_cols, false);
    if (g2 < grid) grid = g2;
    norm_bwd_generic_kernel<T><<<grid, 256, 0, st>>>((const T*)dy, (const T*)ds, (const T*)x, w, w_dt, rstd,
                                                       (T*)dx, workspace, n_rows, n_cols);
  } else {
    // 16-bit rows of 129 to 1024 vectors, w in the data's dtype: the lean kernel (automatic choice only)
    if constexpr (sizeof(T) == 2) {
      const int64_t n_vec16 = n_cols / 8;
      if (g_norm_ring == 1 && dy && w_dt == (std::is_same<T, __nv_bfloat16>::value ? HILDA_BF16 : HILDA_F16) &&
          n_vec16 > 128 && n_vec16 <= 1024) {
#define B16_CALL(TH, VP, DS, FU)                                                                              \
  do {                                                                                                        \
    int occ = 0;  /* a persistent grid: no more CTAs than are resident at once */                             \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, norm_bwd16_kernel<T, TH, VP, DS, FU>, TH, 0) == cudaSuccess && \
        occ > 0 && grid > occ * sm_count())                                                                   \
      grid = occ * sm_count();                                                                                \
    norm_bwd16_kernel<T, TH, VP, DS, FU><<<grid, TH, 0, st>>>((const T*)dy, (const T*)ds, (const T*)x, (const T*)w, rstd, \
                                                              (T*)dx, workspace, n_rows, (int)n_cols, 1);      \
  } while (0)
        // The form without bounds flags only where it measured faster: two vectors per thread, no dS (bf16
        // [16384,4096] 69.8 against 71.8 us). With dS, and with four vectors per thread, the compiler spills
        // in that form and the flagged one is faster ([16384,4096] with dS 85.5 against 88.4 us, [8192,8192]
        // 70.0 against 80.4, with dS 87.5 against 105.8).
#define B16_PICK2(TH)                                                                                         \
  do {                                                                                                        \
    if (ds) B16_CALL(TH, 2, true, false);                                                                     \
    else if (n_vec16 == (int64_t)(TH) * 2) B16_CALL(TH, 2, false, true);                                      \
    else B16_CALL(TH, 2, false, false);                                                                       \
  } while (0)
        if (n_vec16 <= 256) B16_PICK2(128);
        else if (n_vec16 <= 512) B16_PICK2(256);
        else if (ds) B16_CALL(256, 4, true, false);
        else B16_CALL(256, 4, false, false);
#undef B16_PICK2
#undef B16_CALL
        HILDA_LAUNCH_CHECK();
        return launch_dw_reduce(workspace, grid, n_cols, dw, w_dt, st);
      }
    }
    // ring of row slots in shared memory: as many as fit beside the other CTAs of the SM, at most NB_MAX_STAGES
    const int per_sm = (grid + sm_count() - 1) / sm_count();
    const int64_t stage_bytes = n_cols * (int64_t)sizeof(T) * (1 + (dy ? 1 : 0) + (ds ? 1 : 0));
    // 228 KB of shared memory per SM, 1 KB of it reserved per resident CTA, a few hundred bytes static
    int64_t stages = ((int64_t)228 * 1024 / per_sm - 1024 - 512 - n_cols * 4) / stage_bytes;
    if (stages > NB_MAX_STAGES) stages = NB_MAX_STAGES;
    const int64_t min_stages = g_norm_ring == 4 ? 2 : 3;
    // automatic choice: the ring for 32-bit rows only. For 16-bit rows the register kernel with the L2
    // prefetch measured faster wherever the ring fits (bf16, dY and x: H = 3072 4.35 against 3.76 TB/s,
    // 5120 3.90 against 3.35, 7168 4.60 against 4.15)
    const bool ring_auto = g_norm_ring == 1 && sizeof(T) == 4;
    if ((ring_auto || g_norm_ring == 4) && stages >= min_stages) {
      int smem = 0;
      cudaError_t e = cudaSuccess;
      int occ = 0;
#define RING_PREP(TT, TH, VP)                                                                                  \
  do {                                                                                                         \
    e = cudaFuncSetAttribute(norm_bwd_ring_kernel<TT, TH, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, norm_bwd_ring_kernel<TT, TH, VP>, TH, smem); \
  } while (0)
      // one slot fewer while the planned number of CTAs per SM does not fit with this many
      for (; stages >= min_stages; --stages) {
        smem = (int)(stages * stage_bytes + n_cols * 4);
        NORM_DISPATCH_TV(T, RING_PREP)
        if (e != cudaSuccess || occ >= per_sm) break;
      }
#undef RING_PREP
      if (stages < min_stages) { occ = 0; e = cudaSuccess; }
      if (e != cudaSuccess) return HILDA_ERR_CUDA;
      if (occ >= per_sm) {
#define RING_CALL(TT, TH, VP)                                                                                  \
  norm_bwd_ring_kernel<TT, TH, VP><<<grid, TH, smem, st>>>((const TT*)dy, (const TT*)ds, (const TT*)x, w, w_dt, rstd, \
                                                           (TT*)dx, workspace, n_rows, (int)n_cols, (int)stages)
        NORM_DISPATCH_TV(T, RING_CALL)
#undef RING_CALL
        HILDA_LAUNCH_CHECK();
        return launch_dw_reduce(workspace, grid, n_cols, dw, w_dt, st);
      }
    }
#define BWD_CALL(TT, TH, VP)                                                                               \
  norm_bwd_kernel<TT, TH, VP><<<grid, TH, 0, st>>>((const TT*)dy, (const TT*)ds, (const TT*)x, w, w_dt, rstd, \
                                                    (TT*)dx, workspace, n_rows, (int)n_cols, \
                                                    (g_norm_ring == 1 || g_norm_ring == 4) ? 1 : (g_norm_ring >= 2 ? g_norm_ring - 1 : 0))
    NORM_DISPATCH_TV(T, BWD_CALL)
#undef BWD_CALL
  }
  HILDA_LAUNCH_CHECK();
  return launch_dw_reduce(workspace, grid, n_cols, dw, w_dt, st);
}

// ---- scratch for the entry point that allocates nothing ------------------------------------
// One fixed array per GPU that loads the library (it stays resident until the process exits).
// 4 Mi floats = 16 MiB: room for e.g. 444 partial rows of 8192 columns or 592 rows of 4096.
constexpr int64_t NOALLOC_SCRATCH_FLOATS = 4ll * 1024 * 1024;
static __device__ __align__(256) float g_norm_bwd_scratch[NOALLOC_SCRATCH_FLOATS];

// In host code `g_norm_bwd_scratch` is only a handle; the device address has to be asked for,
// once per device, while that device is current.
static float* noalloc_scratch_ptr(int* rc) {
  static float* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *rc = HILDA_ERR_CUDA; return nullptr; }
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_norm_bwd_scratch) != cudaSuccess || p == nullptr) { *rc = HILDA_ERR_CUDA; return nullptr; }
    cached[dev] = reinterpret_cast<float*>(p);
  }
  *rc = HILDA_OK;
  return cached[dev];
}

}  // namespace hilda

using namespace hilda;

extern "C" {

int hilda_rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t n_rows, int64_t n_cols,
                       float eps, int dtype, int w_dtype, void* stream) {
  if (n_rows == 0) return HILDA_OK;
  if (!x || !w || !y || !rstd) return HILDA_ERR_NULL;
  if (n_rows < 0 || n_cols <= 0 || n_cols > 0x7fffffff) return HILDA_ERR_SIZE;
  if (dtype_size(w_dtype) == 0) return HILDA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return norm_fwd_t<float>(x, nullptr, w, w_dtype, y, nullptr, rstd, n_rows, n_cols, eps, st);
    case HILDA_BF16: return norm_fwd_t<__nv_bfloat16>(x, nullptr, w, w_dtype, y, nullptr, rstd, n_rows, n_cols, eps, st);
    case HILDA_F16: return norm_fwd_t<__half>(x, nullptr, w, w_dtype, y, nullptr, rstd, n_rows, n_cols, eps, st);
  }
  return HILDA_ERR_DTYPE;
}

int hilda_fused_add_rms_norm_fwd(const void* x, const void* r, const void* w, void* y, void* s, float* rstd,
                                 int64_t n_rows, int64_t n_cols, float eps, int dtype, int w_dtype, void* stream) {
  if (n_rows == 0) return HILDA_OK;
  if (!x || !r || !w || !y || !s || !rstd) return HILDA_ERR_NULL;
  if (n_rows < 0 || n_cols <= 0 || n_cols > 0x7fffffff) return HILDA_ERR_SIZE;
  if (dtype_size(w_dtype) == 0) return HILDA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return norm_fwd_t<float>(x, r, w, w_dtype, y, s, rstd, n_rows, n_cols, eps, st);
    case HILDA_BF16: return norm_fwd_t<__nv_bfloat16>(x, r, w, w_dtype, y, s, rstd, n_rows, n_cols, eps, st);
    case HILDA_F16: return norm_fwd_t<__half>(x, r, w, w_dtype, y, s, rstd, n_rows, n_cols, eps, st);
  }
  return HILDA_ERR_DTYPE;
}

int64_t hilda_norm_bwd_workspace_bytes(int64_t n_rows, int64_t n_cols, int dtype) {
  if (n_rows <= 0 || n_cols <= 0) return 16;
  int ctas;
  switch (dtype) {
    case HILDA_F32: ctas = norm_bwd_ctas<float>(n_rows, n_cols, true); break;
    case HILDA_BF16: ctas = norm_bwd_ctas<__nv_bfloat16>(n_rows, n_cols, true); break;
    case HILDA_F16: ctas = norm_bwd_ctas<__half>(n_rows, n_cols, true); break;
    default: return HILDA_ERR_DTYPE;
  }
  return (int64_t)ctas * n_cols * 4;
}

static int norm_bwd_any(const void* dy, const void* ds, const void* x, const void* w, const float* rstd, void* dx,
                        void* dw, float* workspace, int64_t n_rows, int64_t n_cols, int dtype, int w_dtype,
                        void* stream, int64_t max_ctas) {
  if (!w || !dw) return HILDA_ERR_NULL;
  if (n_rows > 0 && (!x || !rstd || !dx || !workspace)) return HILDA_ERR_NULL;
  if (n_rows < 0 || n_cols <= 0 || n_cols > 0x7fffffff) return HILDA_ERR_SIZE;
  if (dtype_size(w_dtype) == 0) return HILDA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_rows == 0) {
    if (cudaMemsetAsync(dw, 0, (size_t)n_cols * dtype_size(w_dtype), st) != cudaSuccess) return HILDA_ERR_CUDA;
    return HILDA_OK;
  }
  switch (dtype) {
    case HILDA_F32: return norm_bwd_t<float>(dy, ds, x, w, w_dtype, rstd, dx, dw, workspace, n_rows, n_cols, st, max_ctas);
    case HILDA_BF16: return norm_bwd_t<__nv_bfloat16>(dy, ds, x, w, w_dtype, rstd, dx, dw, workspace, n_rows, n_cols, st, max_ctas);
    case HILDA_F16: return norm_bwd_t<__half>(dy, ds, x, w, w_dtype, rstd, dx, dw, workspace, n_rows, n_cols, st, max_ctas);
  }
  return HILDA_ERR_DTYPE;
}

// dy and ds may each be null (treated as zero); x is the saved input (RMSNorm) or saved sum S
// (FusedAddRMSNorm).
int hilda_norm_bwd(const void* dy, const void* ds, const void* x, const void* w, const float* rstd, void* dx,
                   void* dw, float* workspace, int64_t n_rows, int64_t n_cols, int dtype, int w_dtype,
                   void* stream) {
  return norm_bwd_any(dy, ds, x, w, rstd, dx, dw, workspace, n_rows, n_cols, dtype, w_dtype, stream, 0);
}

// Kernel behind hilda_norm_bwd for vectorisable shapes: 1 (default) = rows staged through a
// shared-memory ring by bulk asynchronous copies, 0 = register-only kernel; anything else only
// queries. Returns the previous choice. Per host thread.
int hilda_norm_bwd_set_path(int path) {
  const int prev = g_norm_ring;
  if (path >= 0 && path <= 4) g_norm_ring = path;
  return prev;
}

int64_t hilda_norm_bwd_noalloc_max_bytes(void) { return NOALLOC_SCRATCH_FLOATS * 4; }

// hilda_norm_bwd for hosts that cannot hand over a workspace: same arguments minus `workspace`, same
// kernels. The per-CTA dW partial sums go to a 16 MiB array that lives inside the library (one copy
// on every GPU that loads it). Meant for callers that have no allocator to ask: a C/FFI host
// without torch's caching allocator, or a server that gave all device memory to its own pool at
// start-up and must not call cudaMalloc afterwards.
//  * The array holds hilda_norm_bwd_noalloc_max_bytes() / (4 * n_cols) partial rows. When the default
//    launch would use more CTAs than that, fewer CTAs are launched (the kernel walks the rows with a
//    grid stride, so any grid is correct): dX is then bit-identical to hilda_norm_bwd's and dW equal
//    within the rounding of a different summation grouping. Only a row longer than the whole array
//    (n_cols > 4 Mi) is refused with HILDA_ERR_SIZE.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress);
//    make that first call during set-up, before any stream capture begins. (The look-up fills a
//    per-device table without a lock; two threads racing on it store the same value.)
//  * Nothing in the array has to start at zero (each CTA overwrites its whole partial row before
//    the reduce pass reads it), so the contents left by an earlier call are harmless. But every
//    call uses the SAME array: two calls that can overlap on the GPU (different streams, or the
//    same stream from two host threads without ordering) race on it. Keep them ordered.
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
int hilda_norm_bwd_noalloc(const void* dy, const void* ds, const void* x, const void* w, const float* rstd, void* dx,
                           void* dw, int64_t n_rows, int64_t n_cols, int dtype, int w_dtype, void* stream) {
  if (n_cols <= 0) return HILDA_ERR_SIZE;
  const int64_t fit = NOALLOC_SCRATCH_FLOATS / n_cols;
  if (fit < 1) return HILDA_ERR_SIZE;
  int rc = HILDA_OK;
  float* scratch = noalloc_scratch_ptr(&rc);
  if (rc != HILDA_OK) return rc;
  return norm_bwd_any(dy, ds, x, w, rstd, dx, dw, scratch, n_rows, n_cols, dtype, w_dtype, stream, fit);
}

}  // extern "C"
