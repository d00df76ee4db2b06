// Rotate-half RoPE on q and k in one launch, optionally in place, for sm_100a.
//
// Semantics follow kernels/rope.py:28-83 of hilda-kernel: for every (batch, head, position) row of
// head_dim elements, with half-width cos/sin tables indexed by position,
//     y1 = x1*cos - x2*sin,  y2 = x2*cos + x1*sin      (x1 = first half, x2 = second half)
// and the backward pass is the same map with -sin (rope.py:139-172). Arithmetic is carried out in
// the dtype of the cos table (x is cast to it first, rope.py:76-77) with a rounding after every
// multiply and add, which is also what the PyTorch reference (benchmarks/bench_rope.py:40-58)
// does, and the result is cast to x's dtype on store.
//
// Layout: q/k are addressed as (batch, head, seq, head_dim) with arbitrary element strides on the
// first three dims and a contiguous last dim, so both (B,H,S,D) and transposed views of (B,S,H,D)
// memory work without a copy. One thread handles one 16-byte vector of x1 and the matching vector
// of x2; q and k items are folded into one flat index space so a single launch covers both.
#include <cstdlib>
#include "common.cuh"

namespace hilda {

struct RopeTensor {
  const void* in;
  void* out;
  int64_t stride_b, stride_h, stride_s;     // element strides of `in`
  int64_t ostride_b, ostride_h, ostride_s;  // element strides of `out`
  int n_heads;
};

struct RopeArgs {
  RopeTensor t[2];
  const void* cos;
  const void* sin;
  int64_t cos_stride_b;  // 0 when the table has batch size 1
  int64_t cos_stride_s;
  int cs_dtype;
  float sin_sign;  // +1 forward, -1 backward
  int bsz, seq, half;  // half = head_dim / 2
  int s_inner;         // 1: iterate seq faster than heads (memory order B,H,S,D)
};

template <int VEC>
__device__ __forceinline__ void load_vec_any(const void* base, int dt, int64_t e0, float* out) {
  if (dt == HILDA_F32) {
    const float* p = reinterpret_cast<const float*>(base) + e0;
    if constexpr (VEC % 4 == 0) {
#pragma unroll
      for (int j = 0; j < VEC; j += 4) VT<float>::unpack(ld16(p + j), out + j);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[j] = p[j];
    }
  } else if (dt == HILDA_BF16) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(base) + e0;
    if constexpr (VEC == 8) VT<__nv_bfloat16>::unpack(ld16(p), out);
    else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[j] = __bfloat162float(p[j]);
    }
  } else {
    const __half* p = reinterpret_cast<const __half*>(base) + e0;
    if constexpr (VEC == 8) VT<__half>::unpack(ld16(p), out);
    else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) out[j] = __half2float(p[j]);
    }
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void load_x(const T* p, float* out) {
  if constexpr (VEC == VT<T>::N) VT<T>::unpack(ld16(p), out);
  else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) out[j] = VT<T>::load1(p + j);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_x(T* p, const float* v) {
  if constexpr (VEC == VT<T>::N) st16(p, VT<T>::pack(v));
  else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) VT<T>::store1(p + j, v[j]);
  }
}

// Packed 16-bit arithmetic with one rounding per multiply/add: bit-identical to computing in fp32 and
// rounding after every operation (products of two 16-bit values are exact in fp32; a sum of two
// needs more than 24 bits only when the smaller term is below the result's rounding granularity),
// at a fraction of the instruction count.
template <typename T> struct Pk;
template <> struct Pk<__nv_bfloat16> { using P2 = __nv_bfloat162; static constexpr int DT = HILDA_BF16; };
template <> struct Pk<__half> { using P2 = __half2; static constexpr int DT = HILDA_F16; };

template <typename P2>
__device__ __forceinline__ void rope_packed(const uint4& X1, const uint4& X2, const uint4& C, const uint4& S, bool neg,
                                            uint4& Y1, uint4& Y2) {
  const P2* x1 = reinterpret_cast<const P2*>(&X1);
  const P2* x2 = reinterpret_cast<const P2*>(&X2);
  const P2* c = reinterpret_cast<const P2*>(&C);
  const P2* s = reinterpret_cast<const P2*>(&S);
  P2* y1 = reinterpret_cast<P2*>(&Y1);
  P2* y2 = reinterpret_cast<P2*>(&Y2);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const P2 sj = neg ? __hneg2(s[j]) : s[j];
    y1[j] = __hsub2_rn(__hmul2_rn(x1[j], c[j]), __hmul2_rn(x2[j], sj));
    y2[j] = __hadd2_rn(__hmul2_rn(x2[j], c[j]), __hmul2_rn(x1[j], sj));
  }
}

// grid.x = outer index (token b*S+s, or b*H+h when seq is the faster dim), grid.y = chunk of the
// inner (head|position, vector) items. Only 32-bit divisions per item.
template <typename T, int VEC>
__global__ void __launch_bounds__(512) rope_kernel(const RopeArgs a, int inner_items, int chunk_items) {
  const unsigned vph = a.half / VEC;  // vectors per half head
  const int h_total = a.t[0].n_heads + a.t[1].n_heads;
  const unsigned outer = blockIdx.x;
  const unsigned odiv = a.s_inner ? (unsigned)h_total : (unsigned)a.seq;
  const int b = (int)(outer / odiv);
  const int orem = (int)(outer - (unsigned)b * odiv);
  const int i0 = blockIdx.y * chunk_items;
  const int i1 = min(inner_items, i0 + chunk_items);
  const int cd = a.cs_dtype;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    const unsigned mid = (unsigned)i / vph;
    const int v = (int)((unsigned)i - mid * vph);
    const int h = a.s_inner ? orem : (int)mid;
    const int s = a.s_inner ? (int)mid : orem;
    const int ti = (h >= a.t[0].n_heads) ? 1 : 0;
    const RopeTensor& t = a.t[ti];
    const int hh = ti ? h - a.t[0].n_heads : h;
    const int64_t off = b * t.stride_b + hh * t.stride_h + s * t.stride_s + (int64_t)v * VEC;
    const T* xin = reinterpret_cast<const T*>(t.in) + off;
    T* xout = reinterpret_cast<T*>(t.out) + b * t.ostride_b + hh * t.ostride_h + s * t.ostride_s + (int64_t)v * VEC;
    const int64_t coff = b * a.cos_stride_b + s * a.cos_stride_s + (int64_t)v * VEC;

    if constexpr (sizeof(T) == 2 && VEC == 8) {
      if (cd == Pk<T>::DT) {  // x and the tables share a 16-bit dtype: packed path
        const uint4 X1 = ld16(xin), X2 = ld16(xin + a.half);
        const uint4 C = ld16(reinterpret_cast<const T*>(a.cos) + coff);
        const uint4 S = ld16(reinterpret_cast<const T*>(a.sin) + coff);
        uint4 Y1, Y2;
        rope_packed<typename Pk<T>::P2>(X1, X2, C, S, a.sin_sign < 0.f, Y1, Y2);
        st16(xout, Y1);
        st16(xout + a.half, Y2);
        continue;
      }
    }
    float x1[VEC], x2[VEC], c[VEC], sn[VEC], y1[VEC], y2[VEC];
    load_x<T, VEC>(xin, x1);
    load_x<T, VEC>(xin + a.half, x2);
    load_vec_any<VEC>(a.cos, cd, coff, c);
    load_vec_any<VEC>(a.sin, cd, coff, sn);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float sj = sn[j] * a.sin_sign;
      const float a1 = round_any(x1[j], cd), a2 = round_any(x2[j], cd);
      const float p1 = round_any(__fmul_rn(a1, c[j]), cd), p2 = round_any(__fmul_rn(a2, sj), cd);
      const float p3 = round_any(__fmul_rn(a2, c[j]), cd), p4 = round_any(__fmul_rn(a1, sj), cd);
      y1[j] = round_any(__fsub_rn(p1, p2), cd);
      y2[j] = round_any(__fadd_rn(p3, p4), cd);
    }
    store_x<T, VEC>(xout, y1);
    store_x<T, VEC>(xout + a.half, y2);
  }
}

// Fast path for the common training layout: 16-bit q/k whose tables share their dtype (packed
// arithmetic), positions slower than heads in memory ((B,S,H,D) order), head_dim/2 a multiple of 8.
// A CTA owns TOK consecutive tokens; thread i owns the same (head, vector) item of each of them, so
// its index arithmetic is done once and all TOK tokens' loads (two 16-byte vectors of q or k and the
// token's cos / sin vectors, which hit L1 after the first head) are in flight together before the
// first result is stored. TOK x 2 x 16 bytes per thread in flight is what hides the DRAM latency that
// the one-token-per-CTA form above exposes once per CTA.
__device__ __forceinline__ uint4 ld16_once(const void* p) {  // read once, do not keep in L1; not .nc: may be in place
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename T, int TOK>
__global__ void __launch_bounds__(512) rope_tokens_kernel(const RopeArgs a, int items, int64_t n_tokens) {
  using P2 = typename Pk<T>::P2;
  const int i = threadIdx.x;
  if (i >= items) return;
  const unsigned vph = a.half / 8;
  const unsigned mid = (unsigned)i / vph;
  const int v = (int)((unsigned)i - mid * vph);
  const int ti = ((int)mid >= a.t[0].n_heads) ? 1 : 0;
  const RopeTensor& t = a.t[ti];
  const int hh = ti ? (int)mid - a.t[0].n_heads : (int)mid;
  const T* in = reinterpret_cast<const T*>(t.in) + hh * t.stride_h + (int64_t)v * 8;
  T* out = reinterpret_cast<T*>(t.out) + hh * t.ostride_h + (int64_t)v * 8;
  const T* cosp = reinterpret_cast<const T*>(a.cos) + (int64_t)v * 8;
  const T* sinp = reinterpret_cast<const T*>(a.sin) + (int64_t)v * 8;
  const bool neg = a.sin_sign < 0.f;
  const int64_t tok0 = (int64_t)blockIdx.x * TOK;
  uint4 X1[TOK], X2[TOK], C[TOK], S[TOK];
  int64_t oo[TOK];
#pragma unroll
  for (int k = 0; k < TOK; ++k) {
    const int64_t tok = tok0 + k;
    if (tok < n_tokens) {
      const int64_t b = tok / a.seq, s_ = tok - b * a.seq;
      const T* p = in + b * t.stride_b + s_ * t.stride_s;
      oo[k] = b * t.ostride_b + s_ * t.ostride_s;
      X1[k] = ld16_once(p);
      X2[k] = ld16_once(p + a.half);
      const int64_t coff = b * a.cos_stride_b + s_ * a.cos_stride_s;
      C[k] = ld16(cosp + coff);
      S[k] = ld16(sinp + coff);
    }
  }
#pragma unroll
  for (int k = 0; k < TOK; ++k) {
    if (tok0 + k < n_tokens) {
      uint4 Y1, Y2;
      rope_packed<P2>(X1[k], X2[k], C[k], S[k], neg, Y1, Y2);
      st16(out + oo[k], Y1);
      st16(out + oo[k] + a.half, Y2);
    }
  }
}

// The same token structure for 16-bit q / k with fp32 tables (what the reference's RotaryEmbedding module
// hands out: its cos / sin caches are fp32): arithmetic in fp32 with one rounding per operation, as the
// reference does after casting x to the tables' dtype, result rounded to q's dtype.
template <typename T, int TOK>
__global__ void __launch_bounds__(512) rope_tokens_f32cs_kernel(const RopeArgs a, int items, int64_t n_tokens) {
  const int i = threadIdx.x;
  if (i >= items) return;
  const unsigned vph = a.half / 8;
  const unsigned mid = (unsigned)i / vph;
  const int v = (int)((unsigned)i - mid * vph);
  const int ti = ((int)mid >= a.t[0].n_heads) ? 1 : 0;
  const RopeTensor& t = a.t[ti];
  const int hh = ti ? (int)mid - a.t[0].n_heads : (int)mid;
  const T* in = reinterpret_cast<const T*>(t.in) + hh * t.stride_h + (int64_t)v * 8;
  T* out = reinterpret_cast<T*>(t.out) + hh * t.ostride_h + (int64_t)v * 8;
  const float* cosp = reinterpret_cast<const float*>(a.cos) + (int64_t)v * 8;
  const float* sinp = reinterpret_cast<const float*>(a.sin) + (int64_t)v * 8;
  const float sign = a.sin_sign;
  const int64_t tok0 = (int64_t)blockIdx.x * TOK;
  uint4 X1[TOK], X2[TOK], C0[TOK], C1[TOK], S0[TOK], S1[TOK];
  int64_t oo[TOK];
#pragma unroll
  for (int k = 0; k < TOK; ++k) {
    const int64_t tok = tok0 + k;
    if (tok < n_tokens) {
      const int64_t b = tok / a.seq, s_ = tok - b * a.seq;
      const T* p = in + b * t.stride_b + s_ * t.stride_s;
      oo[k] = b * t.ostride_b + s_ * t.ostride_s;
      X1[k] = ld16_once(p);
      X2[k] = ld16_once(p + a.half);
      const int64_t coff = b * a.cos_stride_b + s_ * a.cos_stride_s;
      C0[k] = ld16(cosp + coff); C1[k] = ld16(cosp + coff + 4);
      S0[k] = ld16(sinp + coff); S1[k] = ld16(sinp + coff + 4);
    }
  }
#pragma unroll
  for (int k = 0; k < TOK; ++k) {
    if (tok0 + k < n_tokens) {
      float x1[8], x2[8], c[8], sn[8], y1[8], y2[8];
      VT<T>::unpack(X1[k], x1);
      VT<T>::unpack(X2[k], x2);
      VT<float>::unpack(C0[k], c); VT<float>::unpack(C1[k], c + 4);
      VT<float>::unpack(S0[k], sn); VT<float>::unpack(S1[k], sn + 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sj = sn[j] * sign;
        y1[j] = __fsub_rn(__fmul_rn(x1[j], c[j]), __fmul_rn(x2[j], sj));
        y2[j] = __fadd_rn(__fmul_rn(x2[j], c[j]), __fmul_rn(x1[j], sj));
      }
      st16(out + oo[k], VT<T>::pack(y1));
      st16(out + oo[k] + a.half, VT<T>::pack(y2));
    }
  }
}

// tokens per CTA of the fast path: 0 = the general kernel; HILDA_ROPE_TOK presets it
static int rope_tok_default() {
  static const int v = []() { const char* e = getenv("HILDA_ROPE_TOK"); return e ? atoi(e) : 4; }();
  return v;
}

template <typename T>
static int rope_launch(const RopeArgs& a, bool vec_ok, cudaStream_t st) {
  const int h_total = a.t[0].n_heads + a.t[1].n_heads;
  const int vec = vec_ok ? VT<T>::N : 1;
  const int64_t vph = a.half / vec;
  const int64_t outer = (int64_t)a.bsz * (a.s_inner ? h_total : a.seq);
  const int64_t inner = (int64_t)(a.s_inner ? a.seq : h_total) * vph;
  if (outer == 0 || inner == 0) return HILDA_OK;
  if (outer > 0x7fffffffLL || inner > 0x7fffffffLL) return HILDA_ERR_SIZE;
  if constexpr (sizeof(T) == 2) {
    const int tok = rope_tok_default();
    if (vec_ok && tok > 0 && !a.s_inner && a.cs_dtype == Pk<T>::DT && inner <= 512) {
      const int threads = (int)((inner + 31) / 32 * 32);
      const int64_t n_tokens = outer;
      // four tokens per CTA take 92 registers per thread: above 341 threads only one such CTA fits an SM,
      // and two tokens per CTA (50 registers, three CTAs) keep more loads in flight
      const int per = (tok >= 4 && threads * 96 * 2 <= 65536) ? 4 : (tok >= 2 ? 2 : 1);
      const int64_t ctas = (n_tokens + per - 1) / per;
      if (per == 4) rope_tokens_kernel<T, 4><<<(unsigned)ctas, threads, 0, st>>>(a, (int)inner, n_tokens);
      else if (per == 2) rope_tokens_kernel<T, 2><<<(unsigned)ctas, threads, 0, st>>>(a, (int)inner, n_tokens);
      else rope_tokens_kernel<T, 1><<<(unsigned)ctas, threads, 0, st>>>(a, (int)inner, n_tokens);
      HILDA_LAUNCH_CHECK();
      return HILDA_OK;
    }
    if (vec_ok && tok > 0 && !a.s_inner && a.cs_dtype == HILDA_F32 && inner <= 512) {
      const int threads = (int)((inner + 31) / 32 * 32);
      const int64_t ctas = (outer + 1) / 2;
      rope_tokens_f32cs_kernel<T, 2><<<(unsigned)ctas, threads, 0, st>>>(a, (int)inner, outer);
      HILDA_LAUNCH_CHECK();
      return HILDA_OK;
    }
  }
  int threads, chunk;
  if (inner <= 512) { threads = (int)((inner + 31) / 32 * 32); chunk = threads; }
  else { threads = 256; chunk = 1024; }
  const int64_t chunks = (inner + chunk - 1) / chunk;
  if (chunks > 65535) return HILDA_ERR_SIZE;
  dim3 grid((unsigned)outer, (unsigned)chunks);
  if (vec_ok) rope_kernel<T, VT<T>::N><<<grid, threads, 0, st>>>(a, (int)inner, chunk);
  else rope_kernel<T, 1><<<grid, threads, 0, st>>>(a, (int)inner, chunk);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // namespace hilda

using namespace hilda;

extern "C" int hilda_rope(const void* q_in, void* q_out, const int64_t* q_strides, int n_q_heads,
                          const void* k_in, void* k_out, const int64_t* k_strides, int n_k_heads,
                          const void* cos, const void* sin, int64_t cos_stride_b, int64_t cos_stride_s,
                          int bsz, int seq, int head_dim, int dtype, int cs_dtype, int backward, void* stream) {
  if (!cos || !sin) return HILDA_ERR_NULL;
  if ((n_q_heads > 0 && (!q_in || !q_out || !q_strides)) || (n_k_heads > 0 && (!k_in || !k_out || !k_strides)))
    return HILDA_ERR_NULL;
  if (head_dim <= 0 || (head_dim & 1) || bsz < 0 || seq < 0 || n_q_heads < 0 || n_k_heads < 0) return HILDA_ERR_SIZE;
  if (dtype_size(dtype) == 0 || dtype_size(cs_dtype) == 0) return HILDA_ERR_DTYPE;
  RopeArgs a;
  // q_strides / k_strides: six element strides each, (b, h, s) of the input then of the output
  const int64_t zero6[6] = {0, 0, 0, 0, 0, 0};
  const int64_t* qs = q_strides ? q_strides : zero6;
  const int64_t* ks = k_strides ? k_strides : zero6;
  a.t[0] = RopeTensor{q_in, q_out, qs[0], qs[1], qs[2], qs[3], qs[4], qs[5], n_q_heads};
  a.t[1] = RopeTensor{k_in, k_out, ks[0], ks[1], ks[2], ks[3], ks[4], ks[5], n_k_heads};
  a.cos = cos; a.sin = sin; a.cos_stride_b = cos_stride_b; a.cos_stride_s = cos_stride_s;
  a.cs_dtype = cs_dtype; a.sin_sign = backward ? -1.f : 1.f;
  a.bsz = bsz; a.seq = seq; a.half = head_dim / 2;
  const RopeTensor& ref = n_q_heads > 0 ? a.t[0] : a.t[1];
  a.s_inner = (ref.stride_s < ref.stride_h) ? 1 : 0;

  const int vec = 16 / dtype_size(dtype);
  bool vec_ok = (a.half % vec == 0) && aligned16(cos) && aligned16(sin) && (cos_stride_b % 8 == 0) &&
                (cos_stride_s % 8 == 0);
  for (int i = 0; i < 2 && vec_ok; ++i) {
    const RopeTensor& t = a.t[i];
    if (t.n_heads == 0) continue;
    vec_ok = aligned16(t.in) && aligned16(t.out) && t.stride_b % vec == 0 && t.stride_h % vec == 0 &&
             t.stride_s % vec == 0 && t.ostride_b % vec == 0 && t.ostride_h % vec == 0 && t.ostride_s % vec == 0;
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return rope_launch<float>(a, vec_ok, st);
    case HILDA_BF16: return rope_launch<__nv_bfloat16>(a, vec_ok, st);
    case HILDA_F16: return rope_launch<__half>(a, vec_ok, st);
  }
  return HILDA_ERR_DTYPE;
}
