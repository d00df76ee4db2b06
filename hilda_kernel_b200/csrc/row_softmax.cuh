// One-pass row softmax engine shared by CrossEntropy, the GRPO loss and selective log-softmax.
//
// A vocabulary row (128K-152K logits, 256-304 KB in bf16) does not fit one SM's registers or
// shared memory, so a row is owned by a thread-block CLUSTER: each of the CLUSTER CTAs (on
// different SMs) loads a contiguous slice of the row with 128-bit loads, part of it into registers
// and part into thread-private slots of shared memory, reduces its own (max, sum-exp) pair, and the
// pairs are exchanged through distributed shared memory with a single cluster barrier. Every CTA
// then knows the row's logsumexp and writes the gradient of its slice straight from where it holds
// it. HBM traffic is therefore exactly one read of the row and one write of the gradient row.
//
// The per-row "Op" supplies: which rows are active, the target column, 1/temperature, and how
// the per-row scalars (loss, kl, ...) and the gradient coefficients follow from (lse, x_target):
//     grad[j] = alpha * softmax(x/T)[j] + (j == target ? beta : 0).
#pragma once
#include "common.cuh"

namespace hilda {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void row_cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void row_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void row_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <typename T> __device__ __forceinline__ uint4 neg_inf_vec();
template <> __device__ __forceinline__ uint4 neg_inf_vec<float>() {
  return make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u);
}
template <> __device__ __forceinline__ uint4 neg_inf_vec<__nv_bfloat16>() {
  return make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
}
template <> __device__ __forceinline__ uint4 neg_inf_vec<__half>() {
  return make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);
}

struct RowCoef { float alpha, beta; };

// Compiler barrier on a packed vector: stops the unpacked fp32 copy of the row from being kept
// live across passes (which would triple the register footprint).
__device__ __forceinline__ void opaque(uint4& v) {
  asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}


// ---- per-vector math, specialised per dtype to keep the instruction count per element low ------
// vmax : running maximum over a packed vector (packed 16-bit max for bf16/fp16, no unpacking)
// scale: v * coef in place. For 16-bit types coef is split into hi + lo parts in T so that the
//        packed fused multiply-add e*hi + (e*lo) rounds like one fp32 multiply followed by a
//        rounding to T.
template <typename T> struct RowMath;

template <> struct RowMath<float> {
  struct MaxAcc { float m; };
  struct Coef { float c; };
  static __device__ __forceinline__ MaxAcc max_init() { return MaxAcc{-INFINITY}; }
  static __device__ __forceinline__ void vmax(MaxAcc& a, const uint4& v) {
    a.m = fmaxf(fmaxf(a.m, __uint_as_float(v.x)), fmaxf(__uint_as_float(v.y), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w))));
  }
  static __device__ __forceinline__ float max_final(const MaxAcc& a) { return a.m; }
  static __device__ __forceinline__ Coef make_coef(float c) { return Coef{c}; }
  static __device__ __forceinline__ void scale(uint4& v, const Coef& c) {
    v.x = __float_as_uint(__uint_as_float(v.x) * c.c); v.y = __float_as_uint(__uint_as_float(v.y) * c.c);
    v.z = __float_as_uint(__uint_as_float(v.z) * c.c); v.w = __float_as_uint(__uint_as_float(v.w) * c.c);
  }
};

template <typename P2, typename T> struct RowMath16 {
  struct MaxAcc { P2 m; };
  struct Coef { P2 hi, lo; };
  static __device__ __forceinline__ MaxAcc max_init() {
    const uint4 n = neg_inf_vec<T>();
    return MaxAcc{*reinterpret_cast<const P2*>(&n.x)};
  }
  static __device__ __forceinline__ void vmax(MaxAcc& a, const uint4& v) {
    const P2* p = reinterpret_cast<const P2*>(&v);
    a.m = __hmax2(__hmax2(a.m, p[0]), __hmax2(p[1], __hmax2(p[2], p[3])));
  }
  static __device__ __forceinline__ float max_final(const MaxAcc& a) {
    return fmaxf(VT<T>::load1(reinterpret_cast<const T*>(&a.m)), VT<T>::load1(reinterpret_cast<const T*>(&a.m) + 1));
  }
  static __device__ __forceinline__ Coef make_coef(float c) {
    T hi, lo;
    VT<T>::store1(&hi, c);
    VT<T>::store1(&lo, c - VT<T>::load1(&hi));
    Coef r;
    T* ph = reinterpret_cast<T*>(&r.hi);
    T* pl = reinterpret_cast<T*>(&r.lo);
    ph[0] = hi; ph[1] = hi; pl[0] = lo; pl[1] = lo;
    return r;
  }
  static __device__ __forceinline__ void scale(uint4& v, const Coef& c) {
    P2* p = reinterpret_cast<P2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) p[j] = __hfma2(p[j], c.hi, __hmul2(p[j], c.lo));
  }
};
template <> struct RowMath<__nv_bfloat16> : RowMath16<__nv_bfloat162, __nv_bfloat16> {};
template <> struct RowMath<__half> : RowMath16<__half2, __half> {};

// v <- 2^(v*k - m) (rounded to T), returns the fp32 sum of the eight/four exponentials
template <typename T>
__device__ __forceinline__ float vec_exp_inplace(uint4& v, float k, float m) {
  constexpr int VEC = VT<T>::N;
  float f[VEC];
  VT<T>::unpack(v, f);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    f[j] = ex2_approx(fmaf(f[j], k, -m));
    s += f[j];
  }
  v = VT<T>::pack(f);
  return s;
}

// Build-time variants, measured on B200 at the benchmark shapes (CrossEntropy [8192,128256] / GRPO
// [16,1024,151936] bf16, us): warp-local maxima 699.5 / 1373, block maximum first 707.5 / 1372; loading
// the vectors every thread holds without a bounds test made both slower (718.6 / 1402: more code, spills).
#ifndef ROW_WARP_LOCAL
#define ROW_WARP_LOCAL 1   // 1: warps work relative to their own maximum (one block barrier per row); 0: block maximum first
#endif
#ifndef ROW_FULL_FAST
#define ROW_FULL_FAST 0    // 1: vectors every thread holds are loaded / stored without a bounds test
#endif
#ifndef ROW_ARRIVE_SPLIT
#define ROW_ARRIVE_SPLIT 1  // 1: only the warp that wrote to the peers arrives with release (651 / 774 us against 673 / 800)
#endif
constexpr int ROW_THREADS_DEFAULT = 256;
constexpr int ROW_STATUS_TARGET_RANGE = 31;  // status word: a target / token id outside [0, V)

// Register-resident, cluster-per-row kernel. Requires 16-byte aligned tensors; any V of four vectors or more.
// CTAs per SM the register budget is held to (the row slice itself takes 4*NV registers).
constexpr int row_min_blocks(int threads, int nv) {
  return nv <= 10 ? (threads <= 256 ? 4 : (threads <= 320 ? 3 : 2)) : 2;
}

// NS > 0: besides its NV register vectors a thread owns NS more vectors of the row in dynamic shared
// memory (slot [j][tid], private to the thread, filled by 16-byte cp.async): the register file limits
// a CTA to NV vectors per thread at four CTAs per SM, the idle shared memory holds the rest, so a row
// needs a smaller cluster, more bytes are in flight per SM, and the per-row fixed work (reductions,
// cluster exchange, loss terms) is spread over more elements per thread.
template <typename T, int ROW_THREADS, int NV, int CLUSTER, class Op, int NS = 0>
__global__ void __launch_bounds__(ROW_THREADS, row_min_blocks(ROW_THREADS, NV))
row_softmax_kernel(const T* __restrict__ logits, T* __restrict__ grad, int64_t V, Op op, int* __restrict__ status) {
  constexpr int VEC = VT<T>::N;
  extern __shared__ __align__(16) unsigned char row_stage_raw[];
  uint4* const stage = reinterpret_cast<uint4*>(row_stage_raw) + threadIdx.x;  // slot j at stage[j * ROW_THREADS]
#if ROW_WARP_LOCAL
  __shared__ float wpair[2 * (ROW_THREADS / 32)];  // per warp: (max in the log2 domain, sum of 2^(x - max))
#else
  __shared__ float red[33];
#endif
  __shared__ float xchg[2 * CLUSTER];
  const int tid = threadIdx.x;
  const uint32_t rank = (CLUSTER > 1) ? cluster_ctarank() : 0u;
  const int64_t row = blockIdx.x / CLUSTER;
  const int64_t roff = op.row_offset(row, V);
  // A row need not start or end on a 16-byte boundary (V = 50257, say): the vectors are the aligned
  // body of the row, and the up to VEC - 1 elements before and after it are held one each, as scalars,
  // by the first threads of the cluster's first CTA. The tensors' base addresses are 16-byte aligned.
  const int head = (int)((VEC - (roff & (VEC - 1))) & (VEC - 1));
  const int n_vec = (int)((V - head) / VEC);
  const int n_extra = (int)(V - (int64_t)n_vec * VEC);  // head + tail elements, < 2 * VEC
  const int slice = (n_vec + CLUSTER - 1) / CLUSTER;
  const int v0 = (int)rank * slice;
  const int v1 = min(n_vec, v0 + slice);
  const T* xr = logits + roff;
  T* gr = grad ? grad + roff : nullptr;
  const bool writer = (rank == 0 && tid == 0);
  const bool has_x = (rank == 0 && tid < n_extra);
  const int64_t xi = tid < head ? (int64_t)tid : (int64_t)n_vec * VEC + tid;  // head + n_vec * VEC + (tid - head)

  int64_t target = -1;
  const bool active = op.begin(row, target);  // identical in every CTA of the cluster
  if (!active) {
    if (gr) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = v0 + tid; v < v1; v += ROW_THREADS) st16_stream(gr + head + (int64_t)v * VEC, z);
      if (has_x) VT<T>::store1(gr + xi, 0.f);
    }
    if (writer) op.inactive(row);
    return;
  }
  // "I have started": a peer may write into this CTA's shared memory only once it knows that, so
  // every CTA of an active row arrives here and waits for the others right before its remote
  // stores; the wait has the whole row load and two reductions to hide under.
  if constexpr (CLUSTER > 1) cluster_arrive_relaxed();
  // A target outside [0, V) is not "ignored": the row takes part with no target logit and no
  // one-hot term, and the status word tells the host (the reference reads out of bounds there).
  if (writer && status && (target < 0 || target >= V)) atomicCAS(status, 0, ROW_STATUS_TARGET_RANGE);

  // per-thread base pointers: vector i of this thread sits at a compile-time offset from them
  const int my_vec = v1 - v0;  // vectors in this CTA's slice
  const int full = ROW_FULL_FAST ? my_vec / ROW_THREADS : 0;  // vectors every thread of the CTA holds: no bounds test for those
  const uint4* src = reinterpret_cast<const uint4*>(xr + head) + v0 + tid;
  const float xe = has_x ? VT<T>::load1(xr + xi) : -INFINITY;
  uint4 xv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (i < full) xv[i] = ld16_stream(src + i * ROW_THREADS);
    else xv[i] = (tid + i * ROW_THREADS < my_vec) ? ld16_stream(src + i * ROW_THREADS) : neg_inf_vec<T>();
  }
  if constexpr (NS > 0) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      if (tid + (NV + j) * ROW_THREADS < my_vec) row_cp_async16(stage + j * ROW_THREADS, src + (NV + j) * ROW_THREADS);
      else stage[j * ROW_THREADS] = neg_inf_vec<T>();
    }
    row_cp_async_commit();
  }
  const float inv_t = op.inv_temperature();
  const float k = inv_t * LOG2E;  // logits -> log2 domain
  float x_t = 0.f;
  if (target >= 0 && target < V) x_t = VT<T>::load1(xr + target) * inv_t;
  // the per-row scalars finish() needs are fetched now, under the row loads, not after the reduction
  const typename Op::Pre pre = op.prefetch(row);

#if ROW_WARP_LOCAL
  // pass 1: max of the raw logits over the WARP only (k > 0, so the scale is applied once to the
  // maximum). Each warp works relative to its own maximum: it goes on to the exponentials as soon as
  // its own loads have landed, and the block needs one barrier per row instead of four.
  typename RowMath<T>::MaxAcc macc = RowMath<T>::max_init();
#pragma unroll
  for (int i = 0; i < NV; ++i) RowMath<T>::vmax(macc, xv[i]);
  if constexpr (NS > 0) {
    row_cp_async_wait_all();  // the thread reads only the slots it filled itself
#pragma unroll
    for (int j = 0; j < NS; ++j) RowMath<T>::vmax(macc, stage[j * ROW_THREADS]);
  }
  const float m_w = warp_max(fmaxf(RowMath<T>::max_final(macc), xe)) * k;
  const float m_safe = (m_w == -INFINITY) ? 0.f : m_w;
  // pass 2: e = 2^(x*k - m_w) summed in fp32, and kept IN PLACE of x (rounded to T): the gradient
  // pass then needs one multiply per element instead of a second exponential (the SFU would
  // otherwise be the bottleneck at HBM speed).
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    opaque(xv[i]);
    s += vec_exp_inplace<T>(xv[i], k, m_safe);
    opaque(xv[i]);  // orders the iterations: at most one vector is unpacked to fp32 at a time
  }
  if constexpr (NS > 0) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      uint4 v = stage[j * ROW_THREADS];
      s += vec_exp_inplace<T>(v, k, m_safe);
      stage[j * ROW_THREADS] = v;
    }
  }
  const float ee = ex2_approx(fmaf(xe, k, -m_safe));  // 0 for a thread without a scalar element
  s += ee;
  s = warp_sum(s);
  // the warps' (max, sum) pairs -> the CTA's pair, computed by every thread (fixed order)
  constexpr int NW = ROW_THREADS / 32;
  if ((tid & 31) == 0) { wpair[2 * (tid >> 5)] = m_w; wpair[2 * (tid >> 5) + 1] = s; }
  __syncthreads();
  float m = -INFINITY;
#pragma unroll
  for (int w = 0; w < NW; ++w) m = fmaxf(m, wpair[2 * w]);
  s = 0.f;
#pragma unroll
  for (int w = 0; w < NW; ++w) s = fmaf(wpair[2 * w + 1], ex2_approx(wpair[2 * w] - m), s);  // empty warp: 0 * 2^-inf
  if (m == -INFINITY) s = 0.f;

#else
  static_assert(NS == 0, "shared-memory vectors need the warp-local variant");
  // pass 1: max of the raw logits (k > 0, so the scale is applied once to the maximum)
  typename RowMath<T>::MaxAcc macc = RowMath<T>::max_init();
#pragma unroll
  for (int i = 0; i < NV; ++i) RowMath<T>::vmax(macc, xv[i]);
  float m = block_max<ROW_THREADS>(fmaxf(RowMath<T>::max_final(macc), xe), red) * k;
  const float m_w = m;
  const float m_safe = (m == -INFINITY) ? 0.f : m;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    opaque(xv[i]);
    s += vec_exp_inplace<T>(xv[i], k, m_safe);
    opaque(xv[i]);
  }
  const float ee = ex2_approx(fmaf(xe, k, -m_safe));
  s += ee;
  s = block_sum<ROW_THREADS>(s, red);

#endif
  float M = m, S = s;
  if constexpr (CLUSTER > 1) {
    cluster_wait();  // every CTA of the cluster is running: its shared memory may be written
    if (tid < CLUSTER) {
      const uint32_t base = (uint32_t)__cvta_generic_to_shared(xchg);
      const uint32_t remote = map_to_cta(base, (uint32_t)tid);
      st_cluster_f32(remote + 8u * rank, m);
      st_cluster_f32(remote + 8u * rank + 4u, s);
    }
    // only warp 0 stored anything a peer must see: the other warps arrive without the release fence
#if ROW_ARRIVE_SPLIT
    if (tid < 32) cluster_arrive_release(); else cluster_arrive_relaxed();
#else
    cluster_arrive_release();
#endif
    cluster_wait_acquire();
    M = -INFINITY;
#pragma unroll
    for (int c = 0; c < CLUSTER; ++c) M = fmaxf(M, xchg[2 * c]);
    S = 0.f;
#pragma unroll
    for (int c = 0; c < CLUSTER; ++c) S = fmaf(xchg[2 * c + 1], ex2_approx(xchg[2 * c] - M), S);  // empty slice: 0 * 2^-inf
  }
  const float lse2 = M + log2f(S);
  const float lse = lse2 * LN2;  // natural-log logsumexp of logits/T

  const RowCoef co = op.finish(row, lse, x_t, writer, pre);
  if (!gr) return;

  // softmax_j = e_j * 2^(m_warp - lse2)
  const float coef = (m_w == -INFINITY) ? 0.f : co.alpha * ex2_approx(m_w - lse2);
  const typename RowMath<T>::Coef pc = RowMath<T>::make_coef(coef);
  uint4* dst = reinterpret_cast<uint4*>(gr + head) + v0 + tid;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    RowMath<T>::scale(xv[i], pc);
    if (i < full || tid + i * ROW_THREADS < my_vec) st16_stream(dst + i * ROW_THREADS, xv[i]);
  }
  if constexpr (NS > 0) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      uint4 v = stage[j * ROW_THREADS];
      RowMath<T>::scale(v, pc);
      if (tid + (NV + j) * ROW_THREADS < my_vec) st16_stream(dst + (NV + j) * ROW_THREADS, v);
    }
  }
  // The target column gets alpha*softmax + beta: the thread that stored its vector overwrites that
  // one element afterwards (same thread, same address: program order holds).
  const bool t_ok = target >= 0 && target < V;
  const bool t_body = t_ok && target >= head && target < head + (int64_t)n_vec * VEC;
  if (t_body) {
    const int tv = (int)((target - head) / VEC) - v0;
    if (tv >= 0 && tv < my_vec && (tv % ROW_THREADS) == tid)
      VT<T>::store1(gr + target, co.alpha * ex2_approx((x_t - lse) * LOG2E) + co.beta);
  }
  // the scalar head / tail elements: gradient straight from fp32
  if (has_x) VT<T>::store1(gr + xi, coef * ee + ((t_ok && xi == target) ? co.beta : 0.f));
}

// Any V / alignment: one CTA per row, scalar access, row read twice (second read from L2).
template <typename T, class Op>
__global__ void __launch_bounds__(512)
row_softmax_generic_kernel(const T* __restrict__ logits, T* __restrict__ grad, int64_t V, Op op, int* __restrict__ status) {
  __shared__ float red[33];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int64_t roff = op.row_offset(row, V);
  const T* xr = logits + roff;
  T* gr = grad ? grad + roff : nullptr;
  const bool writer = (tid == 0);
  int64_t target = -1;
  const bool active = op.begin(row, target);
  if (!active) {
    if (gr)
      for (int64_t c = tid; c < V; c += 512) VT<T>::store1(gr + c, 0.f);
    if (writer) op.inactive(row);
    return;
  }
  if (writer && status && (target < 0 || target >= V)) atomicCAS(status, 0, ROW_STATUS_TARGET_RANGE);
  const float inv_t = op.inv_temperature();
  const float k = inv_t * LOG2E;
  float x_t = 0.f;
  if (target >= 0 && target < V) x_t = VT<T>::load1(xr + target) * inv_t;
  float m = -INFINITY;
  for (int64_t c = tid; c < V; c += 512) m = fmaxf(m, VT<T>::load1(xr + c) * k);
  m = block_max<512>(m, red);
  const float m_safe = (m == -INFINITY) ? 0.f : m;
  float s = 0.f;
  for (int64_t c = tid; c < V; c += 512) s += ex2_approx(fmaf(VT<T>::load1(xr + c), k, -m_safe));
  s = block_sum<512>(s, red);
  const float lse2 = m + log2f(s);
  const float lse = lse2 * LN2;
  const RowCoef co = op.finish(row, lse, x_t, writer, op.prefetch(row));
  if (!gr) return;
  for (int64_t c = tid; c < V; c += 512) {
    float g = co.alpha * ex2_approx(fmaf(VT<T>::load1(xr + c), k, -lse2));
    if (c == target) g += co.beta;
    VT<T>::store1(gr + c, g);
  }
}

struct RowPlan { int threads; int nv; int cluster; bool generic; int ns; };

// Pick (threads, register vectors and shared-memory vectors per thread, cluster size). Rows of up to
// 2048 vectors stay in the registers of one CTA. Longer rows take the smallest cluster of 1, 2, 4 or 8
// CTAs whose threads then hold at most 19 vectors each, 8 or 10 of them in registers and the rest in
// shared memory. Measured on B200 (CrossEntropy, bf16, every row active, TB/s of read + write) against
// the register-only plans with twice the cluster size: V = 32000: 6.59 against 5.90; 65536: 6.27 against
// 5.74; 128256: 6.30 against 5.67; 151936: 6.27 against 5.76. More than 9 shared-memory vectors (36 KB per
// CTA, four CTAs per SM) was slower than none: the carve-out then leaves the L1 too small for the register
// loads in flight (11 vectors 5.56, 12 vectors 5.50 at V = 151936; 8 vectors with the largest carve-out
// forced 5.63 at V = 128256 against 6.30 with the default one).
// force_nv may carry the thread count as threads*100 + nv.
static inline RowPlan plan_row(int64_t V, int vec, bool aligned, int force_nv, int force_cluster, int force_ns) {
  RowPlan p{ROW_THREADS_DEFAULT, 0, 1, true, 0};
  if (!aligned || V / vec > 0x7fffffff || V < 4 * vec) return p;
  const int64_t n_vec = V / vec;  // a row that does not start on a 16-byte boundary has one vector fewer
  if (force_nv > 0 && force_cluster > 0) {
    const int th = force_nv >= 100 ? force_nv / 100 : ROW_THREADS_DEFAULT;
    const int nv = force_nv % 100;
    if ((int64_t)(nv + force_ns) * force_cluster * th >= n_vec) {
      p.threads = th; p.nv = nv; p.cluster = force_cluster; p.ns = force_ns; p.generic = false;
    }
    return p;
  }
  const int64_t per = ROW_THREADS_DEFAULT;
  if (n_vec <= per * 8) {
    p.nv = n_vec <= per ? 1 : (n_vec <= per * 2 ? 2 : (n_vec <= per * 4 ? 4 : 8));
    p.generic = false;
    return p;
  }
  for (int th = ROW_THREADS_DEFAULT; th <= 512; th *= 2) {
    for (int c = (th == ROW_THREADS_DEFAULT ? 1 : 8); c <= 8; c *= 2) {
      const int64_t slots = (n_vec + (int64_t)th * c - 1) / ((int64_t)th * c);
      if (slots > 19) continue;
      p.threads = th; p.cluster = c; p.generic = false;
      if (th == 512 || slots > 16) { p.nv = 10; p.ns = 9; }
      else if (slots > 14) { p.nv = 8; p.ns = 8; }
      else if (slots > 12) { p.nv = 8; p.ns = 6; }
      else { p.nv = 8; p.ns = 4; }
      return p;
    }
  }
  return p;
}

// Cluster scheduling preference: 0 the driver's default, 1 spread, 2 load balancing (the default here; HILDA_ROW_POLICY
// presets it). Measured on B200, CrossEntropy bf16 [8192,128256] / [8192,151936], every row active: 644.9 / 770.7 us
// with load balancing, 651 / 774 with the default or spread.
extern thread_local int g_row_cluster_policy;

template <typename T, int THREADS, int NV, int CLUSTER, class Op, int NS = 0>
static int launch_row_cfg(const T* logits, T* grad, int64_t n_rows, int64_t V, const Op& op, int* status, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_rows * CLUSTER), 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = (size_t)NS * THREADS * sizeof(uint4);
  cfg.stream = st;
  if (NS * THREADS * sizeof(uint4) + 1024 > 48 * 1024) {  // static shared memory counts toward the 48 KB default
    if (cudaFuncSetAttribute(row_softmax_kernel<T, THREADS, NV, CLUSTER, Op, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(NS * THREADS * sizeof(uint4))) != cudaSuccess)
      return HILDA_ERR_CUDA;
  }
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (g_row_cluster_policy > 0 && CLUSTER > 1) {
    attr[1].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
    attr[1].val.clusterSchedulingPolicyPreference =
        g_row_cluster_policy == 1 ? cudaClusterSchedulingPolicySpread : cudaClusterSchedulingPolicyLoadBalancing;
    cfg.numAttrs = 2;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, row_softmax_kernel<T, THREADS, NV, CLUSTER, Op, NS>, logits, grad, V, op, status);
  return e == cudaSuccess ? HILDA_OK : HILDA_ERR_CUDA;
}

// Every (threads, register vectors, cluster, shared-memory vectors) the kernel is instantiated for: what
// plan_row may return, plus the register-only cluster plans the shared-memory ones replaced, kept for
// comparisons through the override. One list for the dispatch and for hilda_row_engine_has_kernel.
#define ROW_CFG_LIST(X)                                                          \
  X(256, 1, 1, 0) X(256, 2, 1, 0) X(256, 4, 1, 0) X(256, 8, 1, 0)                 \
  X(256, 8, 1, 4) X(256, 8, 1, 6) X(256, 8, 1, 8) X(256, 10, 1, 9)                \
  X(256, 8, 2, 4) X(256, 8, 2, 6) X(256, 8, 2, 8) X(256, 10, 2, 9)                \
  X(256, 8, 4, 4) X(256, 8, 4, 6) X(256, 8, 4, 8) X(256, 10, 4, 9)                \
  X(256, 8, 8, 4) X(256, 8, 8, 6) X(256, 8, 8, 8) X(256, 10, 8, 9)                \
  X(512, 10, 8, 9)                                                               \
  X(256, 8, 8, 0) X(256, 10, 8, 0)

// Override of the plan on the calling host thread, for tuning runs (0 = automatic).
extern thread_local int g_row_force_nv, g_row_force_cluster, g_row_force_ns;

template <typename T, class Op>
static int launch_rows(const void* logits_v, void* grad_v, int64_t n_rows, int64_t V, const Op& op, int* status,
                       cudaStream_t st) {
  const T* logits = (const T*)logits_v;
  T* grad = (T*)grad_v;
  if (n_rows == 0) return HILDA_OK;
  if (n_rows * 8 > 0x7fffffffLL) return HILDA_ERR_SIZE;
  const bool al = aligned16(logits) && (!grad || aligned16(grad)) && op.rows_aligned(V, VT<T>::N);
  const RowPlan p = plan_row(V, VT<T>::N, al, g_row_force_nv, g_row_force_cluster, g_row_force_ns);
  if (p.generic) {
    row_softmax_generic_kernel<T, Op><<<(unsigned)n_rows, 512, 0, st>>>(logits, grad, V, op, status);
    HILDA_LAUNCH_CHECK();
    return HILDA_OK;
  }
#define ROW_CFG(TH_, NV_, CL_, NS_) \
  if (p.threads == TH_ && p.nv == NV_ && p.cluster == CL_ && p.ns == NS_)  \
    return launch_row_cfg<T, TH_, NV_, CL_, Op, NS_>(logits, grad, n_rows, V, op, status, st);
  ROW_CFG_LIST(ROW_CFG)
#undef ROW_CFG
  return HILDA_ERR_SIZE;
}

}  // namespace hilda
