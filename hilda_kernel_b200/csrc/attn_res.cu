// AttnRes (attention residuals): softmax attention over the depth of a stack of N residual blocks.
// Replaces the Triton kernels of hilda-kernel's kernels/attn_res.py (_attn_res_fwd_kernel :32-103,
// _attn_res_bwd_kernel :110-190):
//   k_i = RMSNorm(v_i) * w_norm,  score_i = <w_query, k_i>,  alpha = softmax_i(score),  h = sum_i alpha_i v_i
// per token, V = [N, tokens, D].
//
// HBM-bound: the forward reads every block row ONCE (the reference reads them twice): blocks are
// folded into the output with an online softmax (running max, running sum, rescaled accumulator
// in registers), the next block's row is in flight while the current one is reduced. The backward
// reads the rows once from HBM and once more from L2, and accumulates dW_query / dW_norm in
// registers across the tokens of a persistent CTA (fixed-order second pass; the reference uses
// float atomics).
#include <type_traits>

#include <cstdlib>

#include "common.cuh"
#include "hilda_b200.h"

namespace hilda {

constexpr int AR_MAX_BLOCKS = 32;

// Block-wide sums of two values at once; every thread gets both. red: >= 66 floats.
template <int THREADS>
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  constexpr int NW = THREADS / 32;
  a = warp_sum(a);
  b = warp_sum(b);
  if constexpr (NW == 1) return make_float2(a, b);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { red[wid] = a; red[33 + wid] = b; }
  __syncthreads();
  float ta = (lane < NW) ? red[lane] : 0.f;
  float tb = (lane < NW) ? red[33 + lane] : 0.f;
  return make_float2(warp_sum(ta), warp_sum(tb));
}

// k = (v * rstd) rounded to w_norm's dtype, times w_norm in that dtype (attn_res.py:72), as fp32.
__device__ __forceinline__ float ar_key(float v, float rstd, float wn, int wn_dt) {
  return round_any(round_any(v * rstd, wn_dt) * wn, wn_dt);
}

// acc += a.lo * b.lo + a.hi * b.hi for packed 16-bit pairs with an fp32 accumulator (mixed-precision
// FMA: the product of two 16-bit floats is exact in fp32, so this equals converting first).
template <typename T>
__device__ __forceinline__ float fma2_mixed(uint32_t a, uint32_t b, float acc) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm("{\n.reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n fma.rn.f32.bf16 %0, ah, bh, %0;\n}" : "+f"(acc) : "r"(a), "r"(b));
  } else {
    asm("{\n.reg .b16 al, ah, bl, bh;\n mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n"
        "fma.rn.f32.f16 %0, al, bl, %0;\n fma.rn.f32.f16 %0, ah, bh, %0;\n}" : "+f"(acc) : "r"(a), "r"(b));
  }
  return acc;
}
// sum of squares of the 8 values of a 16-byte vector of 16-bit floats, no unpacking
template <typename T>
__device__ __forceinline__ float sumsq16(const uint4& v, float acc) {
  acc = fma2_mixed<T>(v.x, v.x, acc); acc = fma2_mixed<T>(v.y, v.y, acc);
  acc = fma2_mixed<T>(v.z, v.z, acc); acc = fma2_mixed<T>(v.w, v.w, acc);
  return acc;
}
// dot product of two 16-byte vectors of 16-bit floats, fp32 accumulation
template <typename T>
__device__ __forceinline__ float dot16(const uint4& a, const uint4& b, float acc) {
  acc = fma2_mixed<T>(a.x, b.x, acc); acc = fma2_mixed<T>(a.y, b.y, acc);
  acc = fma2_mixed<T>(a.z, b.z, acc); acc = fma2_mixed<T>(a.w, b.w, acc);
  return acc;
}

// sum_e wq[e] * k(v[e]) over one 16-byte vector, with k as ar_key. The dtype test is hoisted out of
// the element loop; when the keys round to the data's own 16-bit type the two roundings are one
// packed convert and one packed multiply per pair.
template <typename T>
__device__ __forceinline__ float ar_key_dot(const float* vf, float rstd, const float* wq, const float* wn, int wn_dt) {
  constexpr int VEC = VT<T>::N;
  float dot = 0.f;
  if (wn_dt == HILDA_F32) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) dot += wq[e] * (vf[e] * rstd * wn[e]);
  } else if (sizeof(T) == 2 && wn_dt == (std::is_same<T, __nv_bfloat16>::value ? HILDA_BF16 : HILDA_F16)) {
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const __nv_bfloat162 k2 = __hmul2(__floats2bfloat162_rn(vf[e] * rstd, vf[e + 1] * rstd),
                                          __floats2bfloat162_rn(wn[e], wn[e + 1]));
        dot += wq[e] * __low2float(k2) + wq[e + 1] * __high2float(k2);
      } else {
        const __half2 k2 = __hmul2(__floats2half2_rn(vf[e] * rstd, vf[e + 1] * rstd), __floats2half2_rn(wn[e], wn[e + 1]));
        dot += wq[e] * __low2float(k2) + wq[e + 1] * __high2float(k2);
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < VEC; ++e) dot += wq[e] * ar_key(vf[e], rstd, wn[e], wn_dt);
  }
  return dot;
}

// ---------------------------------------------------------------------------------- forward
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
attn_res_fwd_kernel(const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt, const void* __restrict__ w_norm,
                    int wn_dt, T* __restrict__ out, float* __restrict__ alpha, float* __restrict__ rstd_out, int n_blocks,
                    int64_t n_tokens, int D, float eps) {
  constexpr int VEC = VT<T>::N;
  __shared__ float red[66];
  __shared__ float scores[AR_MAX_BLOCKS];
  const int n_vec = D / VEC;
  const float inv_d = 1.0f / (float)D;
  float wq[VPT][VEC], wn[VPT][VEC];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wq[j][e] = v < n_vec ? load_any(w_query, wq_dt, (int64_t)v * VEC + e) : 0.f;
      wn[j][e] = v < n_vec ? load_any(w_norm, wn_dt, (int64_t)v * VEC + e) : 0.f;
    }
  }
  const int64_t blk_stride = n_tokens * (int64_t)D;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    const T* v0 = V + tok * D;
    float acc[VPT][VEC];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[j][e] = 0.f;
    float m = -INFINITY, l = 0.f;
    uint4 cur[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      cur[j] = v < n_vec ? ld16_stream(v0 + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0);
    }
    for (int i = 0; i < n_blocks; ++i) {
      uint4 nxt[VPT];
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * THREADS;
        nxt[j] = (i + 1 < n_blocks && v < n_vec) ? ld16_stream(v0 + (int64_t)(i + 1) * blk_stride + (int64_t)v * VEC)
                                                 : make_uint4(0, 0, 0, 0);
      }
      float vf[VPT][VEC];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        VT<T>::unpack(cur[j], vf[j]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += vf[j][e] * vf[j][e];
      }
      ss = block_sum<THREADS>(ss, red);
      const float rstd = rsqrtf(ss * inv_d + eps);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) dot += ar_key_dot<T>(vf[j], rstd, wq[j], wn[j], wn_dt);
      const float sc = block_sum<THREADS>(dot, red);
      if (threadIdx.x == 0) {
        scores[i] = sc;
        rstd_out[(int64_t)i * n_tokens + tok] = rstd;
      }
      const float m_new = fmaxf(m, sc);
      const float corr = __expf(m - m_new), p = __expf(sc - m_new);
#pragma unroll
      for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[j][e] = acc[j][e] * corr + p * vf[j][e];
      l = l * corr + p;
      m = m_new;
#pragma unroll
      for (int j = 0; j < VPT; ++j) cur[j] = nxt[j];
    }
    const float inv_l = 1.0f / l;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[j][e] *= inv_l;
      if (v < n_vec) st16_stream(out + tok * D + (int64_t)v * VEC, VT<T>::pack(acc[j]));
    }
    __syncthreads();  // scores[] complete
    if (threadIdx.x < n_blocks) alpha[(int64_t)threadIdx.x * n_tokens + tok] = __expf(scores[threadIdx.x] - m) * inv_l;
    __syncthreads();  // before the next token overwrites scores[]
  }
}

// Any D, any alignment: element loops, the block rows re-read from L1/L2 for the weighted sum.
template <typename T>
__global__ void __launch_bounds__(256)
attn_res_fwd_generic_kernel(const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                            const void* __restrict__ w_norm, int wn_dt, T* __restrict__ out, float* __restrict__ alpha,
                            float* __restrict__ rstd_out, int n_blocks, int64_t n_tokens, int D, float eps) {
  __shared__ float red[66];
  __shared__ float scores[AR_MAX_BLOCKS];
  const int64_t blk_stride = n_tokens * (int64_t)D;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    for (int i = 0; i < n_blocks; ++i) {
      const T* v = V + (int64_t)i * blk_stride + tok * D;
      float ss = 0.f;
      for (int c = threadIdx.x; c < D; c += 256) { const float x = VT<T>::load1(v + c); ss += x * x; }
      ss = block_sum<256>(ss, red);
      const float rstd = rsqrtf(ss / (float)D + eps);
      float dot = 0.f;
      for (int c = threadIdx.x; c < D; c += 256)
        dot += load_any(w_query, wq_dt, c) * ar_key(VT<T>::load1(v + c), rstd, load_any(w_norm, wn_dt, c), wn_dt);
      dot = block_sum<256>(dot, red);
      if (threadIdx.x == 0) { scores[i] = dot; rstd_out[(int64_t)i * n_tokens + tok] = rstd; }
    }
    __syncthreads();
    float m = -INFINITY, l = 0.f;
    for (int i = 0; i < n_blocks; ++i) m = fmaxf(m, scores[i]);
    for (int i = 0; i < n_blocks; ++i) l += __expf(scores[i] - m);
    const float inv_l = 1.0f / l;
    for (int c = threadIdx.x; c < D; c += 256) {
      float h = 0.f;
      for (int i = 0; i < n_blocks; ++i)
        h += __expf(scores[i] - m) * inv_l * VT<T>::load1(V + (int64_t)i * blk_stride + tok * D + c);
      VT<T>::store1(out + tok * D + c, h);
    }
    if (threadIdx.x < n_blocks) alpha[(int64_t)threadIdx.x * n_tokens + tok] = __expf(scores[threadIdx.x] - m) * inv_l;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------- backward
// Per token (attn_res.py:124-190), with g = w_query * w_norm:
//   d_alpha_i = <dh, v_i>,  c_i = <g, v_i>,  d_score_i = alpha_i (d_alpha_i - sum_j alpha_j d_alpha_j)
//   dV_i = alpha_i dh + rstd_i d_score_i g - rstd_i^3 (d_score_i c_i / D) v_i
//   dW_query += d_score_i (v_i rstd_i) w_norm,   dW_norm += d_score_i w_query (v_i rstd_i)
// Pass 1 reduces all 2N dot products with one pair of barriers; pass 2 re-reads the rows (L2).
// partial: [gridDim.x][2 * D] fp32, this CTA's dW_query then dW_norm sums over its tokens.
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
attn_res_bwd_kernel(const T* __restrict__ dOut, const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                    const void* __restrict__ w_norm, int wn_dt, const float* __restrict__ alpha,
                    const float* __restrict__ rstd_in, T* __restrict__ dV, float* __restrict__ partial, int n_blocks,
                    int64_t n_tokens, int D) {
  constexpr int VEC = VT<T>::N;
  constexpr int NW = THREADS / 32;
  __shared__ float part[NW][2 * AR_MAX_BLOCKS];
  __shared__ float tot[2 * AR_MAX_BLOCKS];
  __shared__ float ds_sh[AR_MAX_BLOCKS];
  const int n_vec = D / VEC;
  const float inv_d = 1.0f / (float)D;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float wq[VPT][VEC], wn[VPT][VEC], dwq[VPT][VEC], dwn[VPT][VEC];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wq[j][e] = v < n_vec ? load_any(w_query, wq_dt, (int64_t)v * VEC + e) : 0.f;
      wn[j][e] = v < n_vec ? load_any(w_norm, wn_dt, (int64_t)v * VEC + e) : 0.f;
      dwq[j][e] = 0.f; dwn[j][e] = 0.f;
    }
  }
  const int64_t blk_stride = n_tokens * (int64_t)D;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    float dh[VPT][VEC];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      VT<T>::unpack(v < n_vec ? ld16_stream(dOut + tok * D + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0), dh[j]);
    }
    // pass 1: the 2N dot products, warp-reduced into shared memory
    for (int i = 0; i < n_blocks; ++i) {
      float da = 0.f, c = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * THREADS;
        float vf[VEC];
        VT<T>::unpack(v < n_vec ? ld16(V + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC) : make_uint4(0, 0, 0, 0), vf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) { da += dh[j][e] * vf[e]; c += wq[j][e] * wn[j][e] * vf[e]; }
      }
      da = warp_sum(da);
      c = warp_sum(c);
      if (lane == 0) { part[wid][2 * i] = da; part[wid][2 * i + 1] = c; }
    }
    __syncthreads();
    if (threadIdx.x < 2 * n_blocks) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += part[w][threadIdx.x];
      tot[threadIdx.x] = s;
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // softmax backward over the blocks, one warp
      const float a = lane < n_blocks ? alpha[(int64_t)lane * n_tokens + tok] : 0.f;
      const float da = lane < n_blocks ? tot[2 * lane] : 0.f;
      const float sum_a_da = warp_sum(a * da);
      if (lane < n_blocks) ds_sh[lane] = a * (da - sum_a_da);
    }
    __syncthreads();
    // pass 2: gradients
    for (int i = 0; i < n_blocks; ++i) {
      const float a = alpha[(int64_t)i * n_tokens + tok];
      const float rstd = rstd_in[(int64_t)i * n_tokens + tok];
      const float ds = ds_sh[i];
      const float coef_v = rstd * rstd * rstd * (ds * tot[2 * i + 1] * inv_d);
      const float coef_g = rstd * ds;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * THREADS;
        if (v >= n_vec) continue;
        float vf[VEC], o[VEC];
        VT<T>::unpack(ld16(V + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC), vf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          o[e] = a * dh[j][e] + coef_g * wq[j][e] * wn[j][e] - coef_v * vf[e];
          const float vn = vf[e] * rstd;
          dwq[j][e] += ds * vn * wn[j][e];
          dwn[j][e] += ds * wq[j][e] * vn;
        }
        st16_stream(dV + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC, VT<T>::pack(o));
      }
    }
    __syncthreads();  // part / tot / ds_sh are reused by the next token
  }
  float* prow = partial + (int64_t)blockIdx.x * 2 * D;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
    if (v >= n_vec) continue;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      prow[(int64_t)v * VEC + e] = dwq[j][e];
      prow[D + (int64_t)v * VEC + e] = dwn[j][e];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
attn_res_bwd_generic_kernel(const T* __restrict__ dOut, const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                            const void* __restrict__ w_norm, int wn_dt, const float* __restrict__ alpha,
                            const float* __restrict__ rstd_in, T* __restrict__ dV, float* __restrict__ partial,
                            int n_blocks, int64_t n_tokens, int D) {
  __shared__ float red[66];
  __shared__ float da_sh[AR_MAX_BLOCKS], c_sh[AR_MAX_BLOCKS], ds_sh[AR_MAX_BLOCKS];
  const int64_t blk_stride = n_tokens * (int64_t)D;
  float* prow = partial + (int64_t)blockIdx.x * 2 * D;
  for (int c = threadIdx.x; c < 2 * D; c += 256) prow[c] = 0.f;  // column c is only ever touched by this thread
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    for (int i = 0; i < n_blocks; ++i) {
      const T* v = V + (int64_t)i * blk_stride + tok * D;
      float da = 0.f, cc = 0.f;
      for (int c = threadIdx.x; c < D; c += 256) {
        const float x = VT<T>::load1(v + c);
        da += VT<T>::load1(dOut + tok * D + c) * x;
        cc += load_any(w_query, wq_dt, c) * load_any(w_norm, wn_dt, c) * x;
      }
      const float2 r = block_sum2<256>(da, cc, red);
      if (threadIdx.x == 0) { da_sh[i] = r.x; c_sh[i] = r.y; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int i = 0; i < n_blocks; ++i) s += alpha[(int64_t)i * n_tokens + tok] * da_sh[i];
      for (int i = 0; i < n_blocks; ++i) ds_sh[i] = alpha[(int64_t)i * n_tokens + tok] * (da_sh[i] - s);
    }
    __syncthreads();
    for (int i = 0; i < n_blocks; ++i) {
      const float a = alpha[(int64_t)i * n_tokens + tok], rstd = rstd_in[(int64_t)i * n_tokens + tok], ds = ds_sh[i];
      const float coef_v = rstd * rstd * rstd * (ds * c_sh[i] / (float)D), coef_g = rstd * ds;
      for (int c = threadIdx.x; c < D; c += 256) {
        const float x = VT<T>::load1(V + (int64_t)i * blk_stride + tok * D + c);
        const float q = load_any(w_query, wq_dt, c), n = load_any(w_norm, wn_dt, c);
        VT<T>::store1(dV + (int64_t)i * blk_stride + tok * D + c,
                      a * VT<T>::load1(dOut + tok * D + c) + coef_g * q * n - coef_v * x);
        const float vn = x * rstd;
        prow[c] += ds * vn * n;
        prow[D + c] += ds * q * vn;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------- staged kernels
// The kernels above keep one block row in flight per CTA, which leaves them bound by DRAM latency
// (N serial round trips per token). The staged variants copy ALL N rows of a token (and dh in the
// backward) into a shared-memory stage with 16-byte cp.async, the next token's stage filling while
// the current one is reduced. Every thread only ever reads back the 16-byte pieces it copied
// itself, so the row data needs no barrier, only cp.async.wait_group; the per-token reductions
// over blocks are batched (all N sums of squares in one barrier pair, then all N dot products).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Sum over the warps of a [NW][cols] shared array into tot[cols]; part is free for reuse after it.
template <int NW>
__device__ __forceinline__ void reduce_parts(const float (*part)[2 * AR_MAX_BLOCKS], float* tot, int cols) {
  __syncthreads();
  if ((int)threadIdx.x < cols) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += part[w][threadIdx.x];
    tot[threadIdx.x] = s;
  }
  __syncthreads();
}

template <typename T, int THREADS, int VPT, int STAGES>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
attn_res_fwd_staged_kernel(const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                           const void* __restrict__ w_norm, int wn_dt, T* __restrict__ out, float* __restrict__ alpha,
                           float* __restrict__ rstd_out, int n_blocks, int64_t n_tokens, int D, float eps) {
  constexpr int VEC = VT<T>::N;
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) uint8_t ar_smem[];
  __shared__ float part[NW][2 * AR_MAX_BLOCKS];
  __shared__ float tot[2 * AR_MAX_BLOCKS];
  T* stage0 = reinterpret_cast<T*>(ar_smem);
  const int64_t stage_elems = (int64_t)n_blocks * D;
  const int n_vec = D / VEC;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float inv_d = 1.0f / (float)D;
  float wq[VPT][VEC], wn[VPT][VEC];  // this thread's slices of the two weight vectors
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wq[j][e] = v < n_vec ? load_any(w_query, wq_dt, (int64_t)v * VEC + e) : 0.f;
      wn[j][e] = v < n_vec ? load_any(w_norm, wn_dt, (int64_t)v * VEC + e) : 0.f;
    }
  }
  const int64_t blk_stride = n_tokens * (int64_t)D;
  auto issue = [&](int64_t tok, int st) {
    if (tok < n_tokens) {
      T* dst = stage0 + st * stage_elems;
      for (int i = 0; i < n_blocks; ++i)
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
          const int v = threadIdx.x + j * THREADS;
          if (v < n_vec) cp_async16(dst + (int64_t)i * D + (int64_t)v * VEC, V + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC);
        }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue((int64_t)blockIdx.x + (int64_t)s * gridDim.x, s);
  int st = 0;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    issue(tok + (int64_t)(STAGES - 1) * gridDim.x, (st + STAGES - 1) % STAGES);
    cp_async_wait<STAGES - 1>();
    const T* rows = stage0 + st * stage_elems + (int64_t)threadIdx.x * VEC;  // this thread's first piece of row 0
    // all N sums of squares
#pragma unroll 4
    for (int i = 0; i < n_blocks; ++i) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (threadIdx.x + j * THREADS < n_vec) {
          const uint4 raw = *reinterpret_cast<const uint4*>(rows + i * D + j * THREADS * VEC);
          if constexpr (sizeof(T) == 2) {
            ss = sumsq16<T>(raw, ss);
          } else {
            float vf[VEC];
            VT<T>::unpack(raw, vf);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss += vf[e] * vf[e];
          }
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) part[wid][i] = ss;
    }
    __syncthreads();
    if ((int)threadIdx.x < n_blocks) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += part[w][threadIdx.x];
      tot[threadIdx.x] = rsqrtf(s * inv_d + eps);  // rstd of block threadIdx.x
    }
    __syncthreads();
    // all N scores
#pragma unroll 4
    for (int i = 0; i < n_blocks; ++i) {
      const float rstd = tot[i];
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (threadIdx.x + j * THREADS < n_vec) {
          float vf[VEC];
          VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + i * D + j * THREADS * VEC), vf);
          dot += ar_key_dot<T>(vf, rstd, wq[j], wn[j], wn_dt);
        }
      }
      dot = warp_sum(dot);
      if (lane == 0) part[wid][AR_MAX_BLOCKS + i] = dot;
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // softmax over the blocks by one warp: alpha replaces the scores
      float sc = -INFINITY;
      if (lane < n_blocks) {
        sc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) sc += part[w][AR_MAX_BLOCKS + lane];
      }
      const float mx = warp_max(sc);
      const float ex = lane < n_blocks ? __expf(sc - mx) : 0.f;
      const float a = ex / warp_sum(ex);
      if (lane < n_blocks) {
        tot[AR_MAX_BLOCKS + lane] = a;
        alpha[(int64_t)lane * n_tokens + tok] = a;
        rstd_out[(int64_t)lane * n_tokens + tok] = tot[lane];
      }
    }
    __syncthreads();
    float acc[VPT][VEC];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[j][e] = 0.f;
#pragma unroll 4
    for (int i = 0; i < n_blocks; ++i) {
      const float a = tot[AR_MAX_BLOCKS + i];
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (threadIdx.x + j * THREADS < n_vec) {
          float vf[VEC];
          VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + i * D + j * THREADS * VEC), vf);
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[j][e] += a * vf[e];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      if (v < n_vec) st16_stream(out + tok * D + (int64_t)v * VEC, VT<T>::pack(acc[j]));
    }
    __syncthreads();  // part / tot are rewritten by the next token
    st = (st + 1) % STAGES;
  }
  cp_async_wait<0>();
}

// ---- forward with the two reductions over D on the tensor cores (16-bit data and weights)
// The staged kernel above spends most of its issue slots on the per-element work of the two
// reductions over D (sum of squares; w_query . key) and on their warp reductions. Both are
// contractions over D with the blocks as rows, so here they are mma.sync m16n8k16 (16-bit inputs,
// fp32 accumulators; products of two 16-bit values are exact in fp32):
//   Gram diagonal:  C[i][i] = sum_d v_i[d] v_i[d]     with A = B^T = the block rows,
//   scores:         C[i][i] = sum_d wq[d] key_i[d]     with w_query in every row of A and the keys
//                                                      of block i as column i of B.
// Lane (g, j) (g = lane / 4, j = lane % 4) reads row g (block g) of the staged token, 16 bytes at
// a time; an MMA's contraction index may be any permutation of the dims, and because only the
// diagonal C[g][g] is used (column g of B comes from the same lanes (g, .) as row g of A) the
// permutation may even differ between rows: odd rows take the two 64-byte halves of a 128-byte
// chunk in the opposite order, which keeps the eight lanes of a quarter warp on different banks.
// The four registers of a 16-byte piece go into the A operand as they are (no register moves):
// its words 0 and 2 are then row g of A, words 1 and 3 row g + 8, so a piece takes two MMAs, one
// whose B holds the partners of words (0, 2) and whose rows 0-7 are kept, one with the partners of
// words (1, 3) whose rows 8-15 are kept; the other half of each result is discarded.
// The diagonal element of row g (and of row g + 8) sits in lane (g, g / 2). The weighted sum over the blocks stays on
// the CUDA cores, one 16-byte piece of every row per thread as above. Needs n_blocks <= 8,
// D % 64 == 0, w_query and w_norm in the data's own 16-bit type (staged in shared memory).
template <typename T> struct ArMma;
template <> struct ArMma<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
  }
  // bf16(bf16(v * rstd) * wn) for a pair, the reference's two roundings
  static __device__ __forceinline__ uint32_t key_pair(uint32_t v, float rstd, uint32_t wn) {
    const __nv_bfloat162 n = __floats2bfloat162_rn(__uint_as_float(v << 16) * rstd, __uint_as_float(v & 0xffff0000u) * rstd);
    const __nv_bfloat162 k = __hmul2(n, *reinterpret_cast<const __nv_bfloat162*>(&wn));
    return *reinterpret_cast<const uint32_t*>(&k);
  }
};
template <> struct ArMma<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t key_pair(uint32_t v, float rstd, uint32_t wn) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    const __half2 k = __hmul2(__floats2half2_rn(f.x * rstd, f.y * rstd), *reinterpret_cast<const __half2*>(&wn));
    return *reinterpret_cast<const uint32_t*>(&k);
  }
};

// FULL8: n_blocks == 8 (every row of the MMA's A operand is a block: no predicated loads, constant
// trip counts) and D == 8 * THREADS * VPT (every thread has a piece: no bounds checks).
template <typename T, int THREADS, int VPT, int STAGES, bool FULL8>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
attn_res_fwd_mma_kernel(const T* __restrict__ V, const T* __restrict__ w_query, const T* __restrict__ w_norm,
                        T* __restrict__ out, float* __restrict__ alpha, float* __restrict__ rstd_out, int n_blocks,
                        int64_t n_tokens, int D, float eps) {
  constexpr int VEC = VT<T>::N;  // 8
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) uint8_t ar_smem[];
  __shared__ float part[NW][2 * AR_MAX_BLOCKS];
  __shared__ float tot[2 * AR_MAX_BLOCKS];
  T* stage0 = reinterpret_cast<T*>(ar_smem);
  const int64_t stage_elems = (int64_t)n_blocks * D;
  T* wq_s = stage0 + STAGES * stage_elems;  // the two weight vectors, after the stages
  T* wn_s = wq_s + D;
  const int n_vec = D / VEC;
  const int n_chunks = D / 64;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  const bool row_ok = FULL8 || g < n_blocks;
  const int nb = FULL8 ? 8 : n_blocks;  // a constant trip count unrolls the loops over the blocks
  const int my_chunks = n_chunks > wid ? (n_chunks - wid + NW - 1) / NW : 0;  // chunks wid, wid + NW, ... of this warp
  const int piece0 = wid * 64 + 8 * (j + 4 * (g & 1)), piece1 = wid * 64 + 8 * (j + 4 * ((g & 1) ^ 1));  // the two halves of a chunk
  const float inv_d = 1.0f / (float)D;
  for (int v = threadIdx.x; v < n_vec; v += THREADS) {
    *reinterpret_cast<uint4*>(wq_s + (int64_t)v * VEC) = *reinterpret_cast<const uint4*>(w_query + (int64_t)v * VEC);
    *reinterpret_cast<uint4*>(wn_s + (int64_t)v * VEC) = *reinterpret_cast<const uint4*>(w_norm + (int64_t)v * VEC);
  }
  const int64_t blk_stride = n_tokens * (int64_t)D;
  auto issue = [&](int64_t tok, int st) {  // pointers advance row by row: no 64-bit multiply per piece
    if (tok < n_tokens) {
      uint32_t dst = (uint32_t)__cvta_generic_to_shared(stage0 + st * stage_elems) + threadIdx.x * 16u;
      const T* src = V + tok * D + (int64_t)threadIdx.x * VEC;
#pragma unroll 8
      for (int i = 0; i < nb; ++i) {
#pragma unroll
        for (int jj = 0; jj < VPT; ++jj)
          if (FULL8 || threadIdx.x + jj * THREADS < n_vec)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + jj * THREADS * 16u), "l"(src + jj * THREADS * VEC) : "memory");
        dst += (uint32_t)D * (uint32_t)sizeof(T);
        src += blk_stride;
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue((int64_t)blockIdx.x + (int64_t)s * gridDim.x, s);
  int st = 0;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    issue(tok + (int64_t)(STAGES - 1) * gridDim.x, (st + STAGES - 1) % STAGES);
    cp_async_wait<STAGES - 1>();
    __syncthreads();  // the reductions read pieces that other threads copied (and the weights, the first time)
    const T* stage = stage0 + st * stage_elems;
    const T* my_row = stage + (int64_t)(row_ok ? g : 0) * D;
    // ---- all N sums of squares: the diagonal of the Gram matrix of this warp's chunks
    {
      float c02[4] = {0.f, 0.f, 0.f, 0.f}, c13[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int it = 0; it < my_chunks; ++it) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint4 r = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok) r = *reinterpret_cast<const uint4*>(my_row + (c ? piece1 : piece0) + it * (NW * 64));
          ArMma<T>::mma(c02, r, r.x, r.z);
          ArMma<T>::mma(c13, r, r.y, r.w);
        }
      }
      if (row_ok && j == (g >> 1)) part[wid][g] = (g & 1) ? c02[1] + c13[3] : c02[0] + c13[2];
    }
    __syncthreads();
    if ((int)threadIdx.x < n_blocks) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += part[w][threadIdx.x];
      tot[threadIdx.x] = rsqrtf(s * inv_d + eps);  // rstd of block threadIdx.x
    }
    __syncthreads();
    // ---- all N scores: keys (two 16-bit roundings) against w_query
    {
      const float rstd = row_ok ? tot[g] : 0.f;
      float c02[4] = {0.f, 0.f, 0.f, 0.f}, c13[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int it = 0; it < my_chunks; ++it) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int off = (c ? piece1 : piece0) + it * (NW * 64);
          uint4 r = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok) r = *reinterpret_cast<const uint4*>(my_row + off);
          const uint4 n4 = *reinterpret_cast<const uint4*>(wn_s + off);
          const uint4 q4 = *reinterpret_cast<const uint4*>(wq_s + off);  // A operand as loaded; the keys are B
          ArMma<T>::mma(c02, q4, ArMma<T>::key_pair(r.x, rstd, n4.x), ArMma<T>::key_pair(r.z, rstd, n4.z));
          ArMma<T>::mma(c13, q4, ArMma<T>::key_pair(r.y, rstd, n4.y), ArMma<T>::key_pair(r.w, rstd, n4.w));
        }
      }
      if (row_ok && j == (g >> 1)) part[wid][AR_MAX_BLOCKS + g] = (g & 1) ? c02[1] + c13[3] : c02[0] + c13[2];
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // softmax over the blocks by one warp: alpha replaces the scores
      float sc = -INFINITY;
      if (lane < n_blocks) {
        sc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) sc += part[w][AR_MAX_BLOCKS + lane];
      }
      const float mx = warp_max(sc);
      const float ex = lane < n_blocks ? __expf(sc - mx) : 0.f;
      const float a = ex / warp_sum(ex);
      if (lane < n_blocks) {
        tot[AR_MAX_BLOCKS + lane] = a;
        alpha[(int64_t)lane * n_tokens + tok] = a;
        rstd_out[(int64_t)lane * n_tokens + tok] = tot[lane];
      }
    }
    __syncthreads();
    // ---- weighted sum over the blocks: this thread's 16-byte piece of every row
    const T* rows = stage + (int64_t)threadIdx.x * VEC;
    float acc[VPT][VEC];
#pragma unroll
    for (int jj = 0; jj < VPT; ++jj)
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[jj][e] = 0.f;
#pragma unroll 8
    for (int i = 0; i < nb; ++i, rows += D) {
      const float a = tot[AR_MAX_BLOCKS + i];
#pragma unroll
      for (int jj = 0; jj < VPT; ++jj) {
        if (FULL8 || threadIdx.x + jj * THREADS < n_vec) {
          float vf[VEC];
          VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + jj * THREADS * VEC), vf);
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[jj][e] += a * vf[e];
        }
      }
    }
#pragma unroll
    for (int jj = 0; jj < VPT; ++jj) {
      const int v = threadIdx.x + jj * THREADS;
      if (FULL8 || v < n_vec) st16_stream(out + tok * D + (int64_t)v * VEC, VT<T>::pack(acc[jj]));
    }
    __syncthreads();  // part / tot are rewritten by the next token
    st = (st + 1) % STAGES;
  }
  cp_async_wait<0>();
}

// ---- backward with its two dot products over D on the tensor cores (16-bit data)
// Per block i the backward needs da_i = <dh, v_i> and c_i = <w_query * w_norm, v_i>. Here both come
// from one pair of MMAs per 16-byte piece: A = the block rows (row g of A = block g, the piece's
// four registers as loaded), B's columns 0, 1, 2 = dh and the high and low 16-bit halves of
// w_query * w_norm (split so that the product keeps fp32 accuracy), supplied by lane groups 0, 1, 2.
// The elementwise pass needs only S[d] = sum over tokens and blocks of (ds_i rstd_i) v_i[d] for the
// weight gradients (d w_query = w_norm * S, d w_norm = w_query * S), one FMA per element instead
// of two products and two accumulators.
template <typename T>
__device__ __forceinline__ void ar_split16(float x, T& hi, T& lo) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
  } else {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
  }
}

template <typename T, int THREADS, int VPT, int STAGES, bool FULL8>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
attn_res_bwd_mma_kernel(const T* __restrict__ dOut, const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                        const void* __restrict__ w_norm, int wn_dt, const float* __restrict__ alpha,
                        const float* __restrict__ rstd_in, T* __restrict__ dV, float* __restrict__ partial, int n_blocks,
                        int64_t n_tokens, int D) {
  constexpr int VEC = VT<T>::N;  // 8
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) uint8_t ar_smem[];
  __shared__ float part[NW][2 * AR_MAX_BLOCKS];
  __shared__ float tot[2 * AR_MAX_BLOCKS];
  __shared__ float ds_sh[AR_MAX_BLOCKS], a_sh[AR_MAX_BLOCKS], r_sh[AR_MAX_BLOCKS];
  T* stage0 = reinterpret_cast<T*>(ar_smem);
  const int64_t stage_elems = (int64_t)(n_blocks + 1) * D;  // N rows, then dh
  // halves of w_query * w_norm; the first starts 64 bytes off a 128-byte boundary so that lane
  // groups 0 (dh) and 1 (high halves) of a quarter warp read different banks
  T* g_hi = stage0 + STAGES * stage_elems + 32;
  T* g_lo = g_hi + D + 32;
  const int n_vec = D / VEC;
  const int n_chunks = D / 64;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  const bool row_ok = FULL8 || g < n_blocks;
  const int nb = FULL8 ? 8 : n_blocks;  // a constant trip count unrolls the loops over the blocks
  const int my_chunks = n_chunks > wid ? (n_chunks - wid + NW - 1) / NW : 0;  // chunks wid, wid + NW, ... of this warp
  const float inv_d = 1.0f / (float)D;
  float g_w[VPT][VEC], S[VPT][VEC];
#pragma unroll
  for (int jj = 0; jj < VPT; ++jj) {
    const int v = threadIdx.x + jj * THREADS;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      g_w[jj][e] = FULL8 || v < n_vec ? load_any(w_query, wq_dt, (int64_t)v * VEC + e) * load_any(w_norm, wn_dt, (int64_t)v * VEC + e) : 0.f;
      S[jj][e] = 0.f;
      if (FULL8 || v < n_vec) ar_split16<T>(g_w[jj][e], g_hi[(int64_t)v * VEC + e], g_lo[(int64_t)v * VEC + e]);
    }
  }
  const int64_t blk_stride = n_tokens * (int64_t)D;
  auto issue = [&](int64_t tok, int st) {
    if (tok < n_tokens) {
      T* dst = stage0 + st * stage_elems;
#pragma unroll 9
      for (int i = 0; i <= nb; ++i) {
        const T* src = i < nb ? V + (int64_t)i * blk_stride + tok * D : dOut + tok * D;
#pragma unroll
        for (int jj = 0; jj < VPT; ++jj) {
          const int v = threadIdx.x + jj * THREADS;
          if (FULL8 || v < n_vec) cp_async16(dst + (int64_t)i * D + (int64_t)v * VEC, src + (int64_t)v * VEC);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue((int64_t)blockIdx.x + (int64_t)s * gridDim.x, s);
  int st = 0;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    issue(tok + (int64_t)(STAGES - 1) * gridDim.x, (st + STAGES - 1) % STAGES);
    if ((int)threadIdx.x < n_blocks) {
      a_sh[threadIdx.x] = alpha[(int64_t)threadIdx.x * n_tokens + tok];
      r_sh[threadIdx.x] = rstd_in[(int64_t)threadIdx.x * n_tokens + tok];
    }
    cp_async_wait<STAGES - 1>();
    __syncthreads();  // the dot products read pieces that other threads copied (and g_hi / g_lo, the first time)
    const T* rows = stage0 + st * stage_elems;
    // ---- da_i and c_i for all blocks
    {
      const T* a_row = rows + (int64_t)(row_ok ? g : 0) * D;
      const T* b_vec = g == 0 ? rows + (int64_t)n_blocks * D : (g == 1 ? g_hi : g_lo);  // this lane group's column of B
      float c02[4] = {0.f, 0.f, 0.f, 0.f}, c13[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int it = 0; it < my_chunks; ++it) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int off = wid * 64 + 8 * (j + 4 * c) + it * (NW * 64);
          uint4 r = make_uint4(0u, 0u, 0u, 0u), bv = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok) r = *reinterpret_cast<const uint4*>(a_row + off);
          if (g < 3) bv = *reinterpret_cast<const uint4*>(b_vec + off);
          ArMma<T>::mma(c02, r, bv.x, bv.z);  // rows 0-7: words 0 and 2 of the piece
          ArMma<T>::mma(c13, r, bv.y, bv.w);  // rows 8-15: words 1 and 3
        }
      }
      // lane (g, 0): columns 0 (da) and 1 (high half); lane (g, 1): column 2 (low half)
      const float col_even = c02[0] + c13[2], col_odd = c02[1] + c13[3];
      const float low = __shfl_down_sync(0xffffffffu, col_even, 1);
      if (row_ok && j == 0) { part[wid][2 * g] = col_even; part[wid][2 * g + 1] = col_odd + low; }
    }
    reduce_parts<NW>(part, tot, 2 * n_blocks);
    if (threadIdx.x < 32) {
      const float a = lane < n_blocks ? a_sh[lane] : 0.f;
      const float da = lane < n_blocks ? tot[2 * lane] : 0.f;
      const float sum_a_da = warp_sum(a * da);
      if (lane < n_blocks) ds_sh[lane] = a * (da - sum_a_da);
    }
    __syncthreads();
    // ---- dV and the running sum for the weight gradients: this thread's piece of every row
    float dh[VPT][VEC];
#pragma unroll
    for (int jj = 0; jj < VPT; ++jj) {
      const int v = threadIdx.x + jj * THREADS;
      VT<T>::unpack(FULL8 || v < n_vec ? *reinterpret_cast<const uint4*>(rows + (int64_t)n_blocks * D + (int64_t)v * VEC)
                              : make_uint4(0, 0, 0, 0), dh[jj]);
    }
#pragma unroll 8
    for (int i = 0; i < nb; ++i) {
      const float a = a_sh[i], rstd = r_sh[i], ds = ds_sh[i];
      const float coef_v = rstd * rstd * rstd * (ds * tot[2 * i + 1] * inv_d);
      const float coef_g = rstd * ds;
#pragma unroll
      for (int jj = 0; jj < VPT; ++jj) {
        const int v = threadIdx.x + jj * THREADS;
        if (!FULL8 && v >= n_vec) continue;
        float vf[VEC], o[VEC];
        VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + (int64_t)i * D + (int64_t)v * VEC), vf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          o[e] = a * dh[jj][e] + coef_g * g_w[jj][e] - coef_v * vf[e];
          S[jj][e] += coef_g * vf[e];
        }
        st16_stream(dV + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC, VT<T>::pack(o));
      }
    }
    __syncthreads();  // part / tot / ds_sh / a_sh / r_sh and (one stage) the rows are rewritten for the next token
    st = (st + 1) % STAGES;
  }
  cp_async_wait<0>();
  float* prow = partial + (int64_t)blockIdx.x * 2 * D;
#pragma unroll
  for (int jj = 0; jj < VPT; ++jj) {
    const int v = threadIdx.x + jj * THREADS;
    if (!FULL8 && v >= n_vec) continue;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      prow[(int64_t)v * VEC + e] = load_any(w_norm, wn_dt, (int64_t)v * VEC + e) * S[jj][e];
      prow[D + (int64_t)v * VEC + e] = load_any(w_query, wq_dt, (int64_t)v * VEC + e) * S[jj][e];
    }
  }
}

template <typename T, int THREADS, int VPT, int STAGES>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
attn_res_bwd_staged_kernel(const T* __restrict__ dOut, const T* __restrict__ V, const void* __restrict__ w_query, int wq_dt,
                           const void* __restrict__ w_norm, int wn_dt, const float* __restrict__ alpha,
                           const float* __restrict__ rstd_in, T* __restrict__ dV, float* __restrict__ partial, int n_blocks,
                           int64_t n_tokens, int D) {
  constexpr int VEC = VT<T>::N;
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) uint8_t ar_smem[];
  __shared__ float part[NW][2 * AR_MAX_BLOCKS];
  __shared__ float tot[2 * AR_MAX_BLOCKS];
  __shared__ float ds_sh[AR_MAX_BLOCKS], a_sh[AR_MAX_BLOCKS], r_sh[AR_MAX_BLOCKS];
  T* stage0 = reinterpret_cast<T*>(ar_smem);
  const int64_t stage_elems = (int64_t)(n_blocks + 1) * D;  // N rows, then dh
  const int n_vec = D / VEC;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const float inv_d = 1.0f / (float)D;
  float wq[VPT][VEC], wn[VPT][VEC], dwq[VPT][VEC], dwn[VPT][VEC];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      wq[j][e] = v < n_vec ? load_any(w_query, wq_dt, (int64_t)v * VEC + e) : 0.f;
      wn[j][e] = v < n_vec ? load_any(w_norm, wn_dt, (int64_t)v * VEC + e) : 0.f;
      dwq[j][e] = 0.f; dwn[j][e] = 0.f;
    }
  }
  float g_w[VPT][VEC];  // w_query * w_norm, the gradient direction of a score through the key
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int e = 0; e < VEC; ++e) g_w[j][e] = wq[j][e] * wn[j][e];
  const int64_t blk_stride = n_tokens * (int64_t)D;
  auto issue = [&](int64_t tok, int st) {
    if (tok < n_tokens) {
      T* dst = stage0 + st * stage_elems;
      for (int i = 0; i <= n_blocks; ++i) {
        const T* src = i < n_blocks ? V + (int64_t)i * blk_stride + tok * D : dOut + tok * D;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
          const int v = threadIdx.x + j * THREADS;
          if (v < n_vec) cp_async16(dst + (int64_t)i * D + (int64_t)v * VEC, src + (int64_t)v * VEC);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue((int64_t)blockIdx.x + (int64_t)s * gridDim.x, s);
  int st = 0;
  for (int64_t tok = blockIdx.x; tok < n_tokens; tok += gridDim.x) {
    issue(tok + (int64_t)(STAGES - 1) * gridDim.x, (st + STAGES - 1) % STAGES);
    if ((int)threadIdx.x < n_blocks) {
      a_sh[threadIdx.x] = alpha[(int64_t)threadIdx.x * n_tokens + tok];
      r_sh[threadIdx.x] = rstd_in[(int64_t)threadIdx.x * n_tokens + tok];
    }
    cp_async_wait<STAGES - 1>();
    const T* rows = stage0 + st * stage_elems;
    float dh[VPT][VEC];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = threadIdx.x + j * THREADS;
      VT<T>::unpack(v < n_vec ? *reinterpret_cast<const uint4*>(rows + (int64_t)n_blocks * D + (int64_t)v * VEC)
                              : make_uint4(0, 0, 0, 0), dh[j]);
    }
    for (int i = 0; i < n_blocks; ++i) {
      float da = 0.f, c = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * THREADS;
        if (v < n_vec) {
          float vf[VEC];
          VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + (int64_t)i * D + (int64_t)v * VEC), vf);
#pragma unroll
          for (int e = 0; e < VEC; ++e) { da += dh[j][e] * vf[e]; c += g_w[j][e] * vf[e]; }
        }
      }
      da = warp_sum(da);
      c = warp_sum(c);
      if (lane == 0) { part[wid][2 * i] = da; part[wid][2 * i + 1] = c; }
    }
    reduce_parts<NW>(part, tot, 2 * n_blocks);
    if (threadIdx.x < 32) {
      const float a = lane < n_blocks ? a_sh[lane] : 0.f;
      const float da = lane < n_blocks ? tot[2 * lane] : 0.f;
      const float sum_a_da = warp_sum(a * da);
      if (lane < n_blocks) ds_sh[lane] = a * (da - sum_a_da);
    }
    __syncthreads();
    for (int i = 0; i < n_blocks; ++i) {
      const float a = a_sh[i], rstd = r_sh[i], ds = ds_sh[i];
      const float coef_v = rstd * rstd * rstd * (ds * tot[2 * i + 1] * inv_d);
      const float coef_g = rstd * ds;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * THREADS;
        if (v >= n_vec) continue;
        float vf[VEC], o[VEC];
        VT<T>::unpack(*reinterpret_cast<const uint4*>(rows + (int64_t)i * D + (int64_t)v * VEC), vf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float q = wq[j][e], n = wn[j][e];
          o[e] = a * dh[j][e] + coef_g * g_w[j][e] - coef_v * vf[e];
          const float vn = vf[e] * rstd;
          dwq[j][e] += ds * vn * n;
          dwn[j][e] += ds * q * vn;
        }
        st16_stream(dV + (int64_t)i * blk_stride + tok * D + (int64_t)v * VEC, VT<T>::pack(o));
      }
    }
    __syncthreads();  // part / tot / ds_sh / a_sh / r_sh are rewritten by the next token
    st = (st + 1) % STAGES;
  }
  cp_async_wait<0>();
  float* prow = partial + (int64_t)blockIdx.x * 2 * D;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int v = threadIdx.x + j * THREADS;
    if (v >= n_vec) continue;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      prow[(int64_t)v * VEC + e] = dwq[j][e];
      prow[D + (int64_t)v * VEC + e] = dwn[j][e];
    }
  }
}

// dW_query[c] = sum over CTAs of partial[cta][c], dW_norm[c] = ... partial[cta][D + c]; fixed order.
__global__ void __launch_bounds__(256)
attn_res_dw_reduce_kernel(const float* __restrict__ partial, int n_ctas, int D, void* __restrict__ dwq, int wq_dt,
                          void* __restrict__ dwn, int wn_dt) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= 2 * D) return;
  float s = 0.f;
  for (int r = 0; r < n_ctas; ++r) s += partial[(int64_t)r * 2 * D + c];
  if (c < D) store_any(dwq, wq_dt, c, s);
  else store_any(dwn, wn_dt, c - D, s);
}

struct ArPlan { int threads, vpt; bool generic; };
static ArPlan ar_plan(int D, int vec, bool aligned) {
  ArPlan p{256, 1, true};
  if (!aligned || D % vec != 0) return p;
  const int n_vec = D / vec;
  int threads = n_vec >= 512 ? 512 : (n_vec >= 256 ? 256 : 128);
  int vpt = 1;
  while (vpt < 4 && threads * vpt < n_vec) vpt <<= 1;
  if (threads * vpt < n_vec) return p;
  p.threads = threads; p.vpt = vpt; p.generic = false;
  return p;
}

#define AR_DISPATCH(T, CALL)                                                                   \
  switch (plan.threads * 8 + plan.vpt) {                                                       \
    case 128 * 8 + 1: CALL(T, 128, 1); break; case 128 * 8 + 2: CALL(T, 128, 2); break;       \
    case 128 * 8 + 4: CALL(T, 128, 4); break; case 256 * 8 + 1: CALL(T, 256, 1); break;       \
    case 256 * 8 + 2: CALL(T, 256, 2); break; case 256 * 8 + 4: CALL(T, 256, 4); break;       \
    case 512 * 8 + 1: CALL(T, 512, 1); break; case 512 * 8 + 2: CALL(T, 512, 2); break;       \
    case 512 * 8 + 4: CALL(T, 512, 4); break;                                                 \
    default: return HILDA_ERR_SIZE;                                                            \
  }

// Shared-memory plan of the staged kernels: `stages` stages of `rows` rows of D elements. Two CTAs per SM with two stages each when that fits,
// otherwise one CTA with as many stages (at most 2) as fit; stages == 0: does not fit at all.
struct ArStagePlan { int stages, ctas_per_sm; size_t smem; };
static ArStagePlan ar_stage_plan(int rows, int D, int elem, size_t extra = 0) {  // extra: bytes beside the stages
  const size_t cap = 227 * 1024 - 16 * 1024;  // leave room for the static shared memory and the per-CTA reserve
  const size_t stage = (size_t)rows * D * elem;
  ArStagePlan p{0, 1, 0};
  if (2 * stage + extra <= cap / 2) { p.stages = 2; p.ctas_per_sm = 2; }       // two CTAs per SM, double-buffered
  else if (stage + extra <= cap / 2) { p.stages = 1; p.ctas_per_sm = 2; }      // two CTAs per SM overlap each other
  else if (2 * stage + extra <= cap) { p.stages = 2; }
  else if (stage + extra <= cap) { p.stages = 1; }
  p.smem = (size_t)p.stages * stage + extra;
  return p;
}

// 0: forward reductions on the CUDA cores, 1 (default): on the tensor cores where the shapes and dtypes allow
// (HILDA_AR_PATH, hilda_attn_res_set_path)
static int g_ar_path = []() { const char* e = getenv("HILDA_AR_PATH"); return e ? atoi(e) : 1; }();

#define AR_DISPATCH_STAGED(T, CALL)                                                            \
  switch (plan.threads * 8 + plan.vpt) {                                                       \
    case 256 * 8 + 1: CALL(T, 256, 1); break; case 256 * 8 + 2: CALL(T, 256, 2); break;       \
    case 256 * 8 + 4: CALL(T, 256, 4); break; case 512 * 8 + 1: CALL(T, 512, 1); break;       \
    case 512 * 8 + 2: CALL(T, 512, 2); break; case 512 * 8 + 4: CALL(T, 512, 4); break;       \
    default: staged = false; break;                                                            \
  }

static int ar_bwd_ctas(int64_t n_tokens) {
  int64_t c = (int64_t)sm_count() * 2;
  if (c > n_tokens) c = n_tokens;
  return (int)(c < 1 ? 1 : c);
}

template <typename T>
static int ar_fwd_t(const void* V, const void* wq, int wq_dt, const void* wn, int wn_dt, void* out, float* alpha, float* rstd,
                    int n_blocks, int64_t n_tokens, int D, float eps, cudaStream_t st) {
  const ArPlan plan = ar_plan(D, VT<T>::N, aligned16(V) && aligned16(out));
  const int64_t cap = (int64_t)sm_count() * 8;
  const int grid = (int)(n_tokens < cap ? n_tokens : cap);
  if (plan.generic) {
    attn_res_fwd_generic_kernel<T><<<grid, 256, 0, st>>>((const T*)V, wq, wq_dt, wn, wn_dt, (T*)out, alpha, rstd, n_blocks,
                                                         n_tokens, D, eps);
    HILDA_LAUNCH_CHECK();
    return HILDA_OK;
  }
  if constexpr (sizeof(T) == 2) {
    const int dt = std::is_same<T, __nv_bfloat16>::value ? HILDA_BF16 : HILDA_F16;
    const ArStagePlan sp = ar_stage_plan(n_blocks, D, (int)sizeof(T), (size_t)2 * D * sizeof(T));
    bool staged = g_ar_path == 1 && wq_dt == dt && wn_dt == dt && n_blocks <= 8 && D % 64 == 0 && aligned16(wq) &&
                  aligned16(wn) && sp.stages > 0 && plan.threads >= 256;
    if (staged) {
      int64_t g = (int64_t)sm_count() * sp.ctas_per_sm;
      if (g > n_tokens) g = n_tokens;
#define AR_FWD_MMA(TT, TH, VP)                                                                                       \
  do {                                                                                                                \
    const bool full8 = n_blocks == 8 && D == 8 * TH * VP;                                                             \
    auto kern = sp.stages == 2 ? (full8 ? attn_res_fwd_mma_kernel<TT, TH, VP, 2, true>                        \
                                                : attn_res_fwd_mma_kernel<TT, TH, VP, 2, false>)                      \
                               : (full8 ? attn_res_fwd_mma_kernel<TT, TH, VP, 1, true>                        \
                                                : attn_res_fwd_mma_kernel<TT, TH, VP, 1, false>);                     \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sp.smem) != cudaSuccess)         \
      return HILDA_ERR_CUDA;                                                                                          \
    kern<<<(unsigned)g, TH, sp.smem, st>>>((const TT*)V, (const TT*)wq, (const TT*)wn, (TT*)out, alpha, rstd, n_blocks, \
                                           n_tokens, D, eps);                                                         \
  } while (0)
      AR_DISPATCH_STAGED(T, AR_FWD_MMA)
#undef AR_FWD_MMA
      if (staged) {
        HILDA_LAUNCH_CHECK();
        return HILDA_OK;
      }
    }
  }
  const ArStagePlan sp = ar_stage_plan(n_blocks, D, (int)sizeof(T));
  bool staged = sp.stages > 0 && plan.threads >= 256;
  if (staged) {
    int64_t g = (int64_t)sm_count() * sp.ctas_per_sm;
    if (g > n_tokens) g = n_tokens;
#define AR_FWD_ST(TT, TH, VP)                                                                                        \
  do {                                                                                                                \
    auto k1 = attn_res_fwd_staged_kernel<TT, TH, VP, 1>;                                                              \
    auto k2 = attn_res_fwd_staged_kernel<TT, TH, VP, 2>;                                                              \
    auto kern = sp.stages == 2 ? k2 : k1;                                                                             \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sp.smem) != cudaSuccess)         \
      return HILDA_ERR_CUDA;                                                                                          \
    kern<<<(unsigned)g, TH, sp.smem, st>>>((const TT*)V, wq, wq_dt, wn, wn_dt, (TT*)out, alpha, rstd, n_blocks, n_tokens, D, \
                                           eps);                                                                      \
  } while (0)
    AR_DISPATCH_STAGED(T, AR_FWD_ST)
#undef AR_FWD_ST
    if (staged) {
      HILDA_LAUNCH_CHECK();
      return HILDA_OK;
    }
  }
#define AR_FWD(TT, TH, VP)                                                                                          \
  attn_res_fwd_kernel<TT, TH, VP><<<grid, TH, 0, st>>>((const TT*)V, wq, wq_dt, wn, wn_dt, (TT*)out, alpha, rstd, n_blocks, \
                                                       n_tokens, D, eps)
  AR_DISPATCH(T, AR_FWD)
#undef AR_FWD
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

template <typename T>
static int ar_bwd_t(const void* dOut, const void* V, const void* wq, int wq_dt, const void* wn, int wn_dt, const float* alpha,
                    const float* rstd, void* dV, void* dwq, void* dwn, float* workspace, int n_blocks, int64_t n_tokens, int D,
                    cudaStream_t st) {
  const ArPlan plan = ar_plan(D, VT<T>::N, aligned16(V) && aligned16(dV) && aligned16(dOut));
  int grid = ar_bwd_ctas(n_tokens);
  bool done = false;
  if (plan.generic) {
    attn_res_bwd_generic_kernel<T><<<grid, 256, 0, st>>>((const T*)dOut, (const T*)V, wq, wq_dt, wn, wn_dt, alpha, rstd,
                                                         (T*)dV, workspace, n_blocks, n_tokens, D);
    done = true;
  }
  if constexpr (sizeof(T) == 2) {
    const ArStagePlan sp = ar_stage_plan(n_blocks + 1, D, (int)sizeof(T), (size_t)(2 * D + 64) * sizeof(T));
    bool staged = !done && g_ar_path == 1 && n_blocks <= 8 && D % 64 == 0 && sp.stages > 0 && plan.threads >= 256;
    if (staged) {
      int64_t g = (int64_t)sm_count() * sp.ctas_per_sm;  // never more than the workspace rows (2 per SM)
      if (g > grid) g = grid;
#define AR_BWD_MMA(TT, TH, VP)                                                                                        \
  do {                                                                                                                \
    const bool full8 = n_blocks == 8 && D == 8 * TH * VP;                                                             \
    auto kern = sp.stages == 2 ? (full8 ? attn_res_bwd_mma_kernel<TT, TH, VP, 2, true>                        \
                                                : attn_res_bwd_mma_kernel<TT, TH, VP, 2, false>)                      \
                               : (full8 ? attn_res_bwd_mma_kernel<TT, TH, VP, 1, true>                        \
                                                : attn_res_bwd_mma_kernel<TT, TH, VP, 1, false>);                     \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sp.smem) != cudaSuccess)         \
      return HILDA_ERR_CUDA;                                                                                          \
    kern<<<(unsigned)g, TH, sp.smem, st>>>((const TT*)dOut, (const TT*)V, wq, wq_dt, wn, wn_dt, alpha, rstd, (TT*)dV,   \
                                           workspace, n_blocks, n_tokens, D);                                         \
  } while (0)
      AR_DISPATCH_STAGED(T, AR_BWD_MMA)
#undef AR_BWD_MMA
      if (staged) { grid = (int)g; done = true; }
    }
  }
  const ArStagePlan sp = ar_stage_plan(n_blocks + 1, D, (int)sizeof(T));
  bool staged = !done && sp.stages > 0 && plan.threads >= 256;
  if (staged) {
    int64_t g = (int64_t)sm_count() * sp.ctas_per_sm;  // never more than the workspace rows (2 per SM)
    if (g > grid) g = grid;
#define AR_BWD_ST(TT, TH, VP)                                                                                         \
  do {                                                                                                                \
    auto k1 = attn_res_bwd_staged_kernel<TT, TH, VP, 1>;                                                              \
    auto k2 = attn_res_bwd_staged_kernel<TT, TH, VP, 2>;                                                              \
    auto kern = sp.stages == 2 ? k2 : k1;                                                                             \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sp.smem) != cudaSuccess)         \
      return HILDA_ERR_CUDA;                                                                                          \
    kern<<<(unsigned)g, TH, sp.smem, st>>>((const TT*)dOut, (const TT*)V, wq, wq_dt, wn, wn_dt, alpha, rstd, (TT*)dV,   \
                                           workspace, n_blocks, n_tokens, D);                                         \
  } while (0)
    AR_DISPATCH_STAGED(T, AR_BWD_ST)
#undef AR_BWD_ST
    if (staged) { grid = (int)g; done = true; }
  }
  if (!done) {
#define AR_BWD(TT, TH, VP)                                                                                           \
  attn_res_bwd_kernel<TT, TH, VP><<<grid, TH, 0, st>>>((const TT*)dOut, (const TT*)V, wq, wq_dt, wn, wn_dt, alpha, rstd, \
                                                       (TT*)dV, workspace, n_blocks, n_tokens, D)
    AR_DISPATCH(T, AR_BWD)
#undef AR_BWD
  }
  HILDA_LAUNCH_CHECK();
  attn_res_dw_reduce_kernel<<<(2 * D + 255) / 256, 256, 0, st>>>(workspace, grid, D, dwq, wq_dt, dwn, wn_dt);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // namespace hilda

using namespace hilda;

extern "C" {

// V [n_blocks, n_tokens, D] in dtype; w_query, w_norm [D] in their own dtypes; out [n_tokens, D];
// alpha, rstd [n_blocks, n_tokens] fp32 (saved for the backward). n_blocks <= 32.
int hilda_attn_res_fwd(const void* V, const void* w_query, const void* w_norm, void* out, float* alpha, float* rstd,
                       int64_t n_blocks, int64_t n_tokens, int64_t D, float eps, int dtype, int wq_dtype, int wn_dtype,
                       void* stream) {
  if (n_blocks < 1 || n_blocks > AR_MAX_BLOCKS || D < 1 || D > (1 << 24) || n_tokens < 0) return HILDA_ERR_SIZE;
  if (n_tokens == 0) return HILDA_OK;
  if (!V || !w_query || !w_norm || !out || !alpha || !rstd) return HILDA_ERR_NULL;
  if (!dtype_size(wq_dtype) || !dtype_size(wn_dtype)) return HILDA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return ar_fwd_t<float>(V, w_query, wq_dtype, w_norm, wn_dtype, out, alpha, rstd, (int)n_blocks, n_tokens, (int)D, eps, st);
    case HILDA_BF16: return ar_fwd_t<__nv_bfloat16>(V, w_query, wq_dtype, w_norm, wn_dtype, out, alpha, rstd, (int)n_blocks, n_tokens, (int)D, eps, st);
    case HILDA_F16: return ar_fwd_t<__half>(V, w_query, wq_dtype, w_norm, wn_dtype, out, alpha, rstd, (int)n_blocks, n_tokens, (int)D, eps, st);
    default: return HILDA_ERR_DTYPE;
  }
}

int64_t hilda_attn_res_bwd_workspace_bytes(int64_t n_tokens, int64_t D) {
  if (n_tokens <= 0 || D <= 0) return 256;
  return (int64_t)ar_bwd_ctas(n_tokens) * 2 * D * 4;
}

// dV [n_blocks, n_tokens, D] in dtype; dw_query / dw_norm [D] in the weights' dtypes; workspace of
// hilda_attn_res_bwd_workspace_bytes(n_tokens, D) bytes.
int hilda_attn_res_bwd(const void* d_out, const void* V, const void* w_query, const void* w_norm, const float* alpha,
                       const float* rstd, void* dV, void* dw_query, void* dw_norm, void* workspace, int64_t n_blocks,
                       int64_t n_tokens, int64_t D, int dtype, int wq_dtype, int wn_dtype, void* stream) {
  if (n_blocks < 1 || n_blocks > AR_MAX_BLOCKS || D < 1 || D > (1 << 24) || n_tokens < 0) return HILDA_ERR_SIZE;
  if (!dw_query || !dw_norm) return HILDA_ERR_NULL;
  if (!dtype_size(wq_dtype) || !dtype_size(wn_dtype)) return HILDA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_tokens == 0) {
    if (cudaMemsetAsync(dw_query, 0, (size_t)D * dtype_size(wq_dtype), st) != cudaSuccess) return HILDA_ERR_CUDA;
    if (cudaMemsetAsync(dw_norm, 0, (size_t)D * dtype_size(wn_dtype), st) != cudaSuccess) return HILDA_ERR_CUDA;
    return HILDA_OK;
  }
  if (!d_out || !V || !w_query || !w_norm || !alpha || !rstd || !dV || !workspace) return HILDA_ERR_NULL;
  float* ws = reinterpret_cast<float*>(workspace);
  switch (dtype) {
    case HILDA_F32: return ar_bwd_t<float>(d_out, V, w_query, wq_dtype, w_norm, wn_dtype, alpha, rstd, dV, dw_query, dw_norm, ws, (int)n_blocks, n_tokens, (int)D, st);
    case HILDA_BF16: return ar_bwd_t<__nv_bfloat16>(d_out, V, w_query, wq_dtype, w_norm, wn_dtype, alpha, rstd, dV, dw_query, dw_norm, ws, (int)n_blocks, n_tokens, (int)D, st);
    case HILDA_F16: return ar_bwd_t<__half>(d_out, V, w_query, wq_dtype, w_norm, wn_dtype, alpha, rstd, dV, dw_query, dw_norm, ws, (int)n_blocks, n_tokens, (int)D, st);
    default: return HILDA_ERR_DTYPE;
  }
}

// Kernel choice: 0 = reductions over D on the CUDA cores, 1 = on the tensor cores (16-bit data, at
// most 8 blocks, D a multiple of 64, for the forward weights of the data's type; other cases take
// 0). Returns the previous choice.
int hilda_attn_res_set_path(int path) {
  const int old = g_ar_path;
  if (path == 0 || path == 1) g_ar_path = path;
  return old;
}

}  // extern "C"
