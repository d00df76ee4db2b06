// Decode attention over a paged FP8 (e4m3) KV cache. Replaces the Triton kernel of hilda-kernel's
// kernels/paged_attention_fp8.py (_paged_attention_fp8_decode_kernel :7-92): one query token per
// sequence, q [batch, heads, 128] bf16, K / V cache [blocks, block_size, kv_heads, 128] fp8, a block
// table and a context length per sequence, output bf16.
//
// HBM-bound on the KV cache, which is read ONCE per kv head: a CTA serves all query heads of one
// (sequence, kv head) (the reference launches one program per query head and re-reads K / V for
// every head of a GQA group) over a slice of the context (split-KV: slices are merged by a second
// small kernel when there is more than one). Eight lanes share a token: each loads 16 bytes
// (16 fp8) of its K row and its V row, so a warp touches four whole 128-byte rows per load; the
// dot product is reduced over the eight lanes with three shuffles; every lane group keeps its own
// online-softmax state (max, sum, 16 output dims per head), merged at the end.
#include <cuda_fp8.h>

#include "common.cuh"
#include "hilda_b200.h"

namespace hilda {

constexpr int PA_HEAD_DIM = 128;
constexpr int PA_THREADS = 128;          // 4 warps x 4 tokens per step
constexpr int PA_TOKENS_PER_STEP = 16;
constexpr int PA_UNROLL = 2;             // steps whose loads are in flight together (4 measured slower)
constexpr int PA_PARTIAL = PA_HEAD_DIM + 2;  // per (sequence, head, split): m, l, 128 unnormalised sums

struct PaParams {
  const __nv_bfloat16* q; int64_t q_sb, q_sh;
  const uint8_t* k; const uint8_t* v;
  int64_t k_sblk, k_stok, k_sh, v_sblk, v_stok, v_sh;
  __nv_bfloat16* out; int64_t o_sb, o_sh;
  const int32_t* block_tables; int64_t bt_sb;
  const int32_t* context_lens;
  float* partial;  // [batch, heads, splits, PA_PARTIAL] when splits > 1
  float scale;
  int n_heads, n_kv_heads, group, block_size, max_blocks, splits, tokens_per_split;
};

// 16 fp8 (e4m3) values in a uint4 -> 8 packed half2 (exact: e4m3 is a subset of fp16).
__device__ __forceinline__ void fp8x16_to_half2(const uint4& raw, uint32_t* h) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
    h[2 * i] = *reinterpret_cast<const uint32_t*>(&lo);
    h[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hi);
  }
}
// acc += a.lo * b.lo + a.hi * b.hi with fp16 inputs and an fp32 accumulator (mixed-precision FMA:
// the products of two fp16 values are exact in fp32, so nothing is lost against converting first).
__device__ __forceinline__ float fma2_f32_f16(uint32_t a, uint32_t b, float acc) {
  asm("{\n.reg .b16 al, ah, bl, bh;\n"
      "mov.b32 {al, ah}, %1;\n mov.b32 {bl, bh}, %2;\n"
      "fma.rn.f32.f16 %0, al, bl, %0;\n"
      "fma.rn.f32.f16 %0, ah, bh, %0;\n}"
      : "+f"(acc) : "r"(a), "r"(b));
  return acc;
}
// acc0 += v.lo * p, acc1 += v.hi * p (p an fp16 scalar replicated in both halves of pp).
__device__ __forceinline__ void fma_pv(uint32_t v, uint32_t pp, float& acc0, float& acc1) {
  asm("{\n.reg .b16 vl, vh, pl, ph;\n"
      "mov.b32 {vl, vh}, %2;\n mov.b32 {pl, ph}, %3;\n"
      "fma.rn.f32.f16 %0, vl, pl, %0;\n"
      "fma.rn.f32.f16 %1, vh, ph, %1;\n}"
      : "+f"(acc0), "+f"(acc1) : "r"(v), "r"(pp));
}

// G query heads of one kv head per pass; grid (kv_heads * passes, batch, splits).
template <int G>
__global__ void __launch_bounds__(PA_THREADS, G <= 2 ? 4 : 2)
paged_attention_fp8_kernel(const PaParams p) {
  const int passes = p.group / G;
  const int kv_head = blockIdx.x / passes, pass = blockIdx.x % passes;
  const int b = blockIdx.y, split = blockIdx.z;
  const int head0 = kv_head * p.group + pass * G;  // first query head of this CTA
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane >> 3, part = lane & 7;      // token within the warp's step, 16-dim slice
  int ctx = p.context_lens[b];
  if (ctx > p.max_blocks * p.block_size) ctx = p.max_blocks * p.block_size;  // never index past the block table
  const int t_begin = split * p.tokens_per_split;
  int t_end = t_begin + p.tokens_per_split;
  if (t_end > ctx) t_end = ctx;

  // q * scale as fp16 pairs: bf16 -> fp16 is exact except below fp16's normal range (|q| < 6e-5,
  // where the product with a key no longer matters) and the scale is folded in before rounding
  uint32_t q[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = p.q + (int64_t)b * p.q_sb + (int64_t)(head0 + g) * p.q_sh + part * 16;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      const __half2 h = __floats2half2_rn(__bfloat162float(qp[2 * d]) * p.scale, __bfloat162float(qp[2 * d + 1]) * p.scale);
      q[g][d] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  float m[G], l[G], acc[G][16];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) acc[g][d] = 0.f;
  }
  const int32_t* table = p.block_tables + (int64_t)b * p.bt_sb;
  // PA_UNROLL steps of loads are issued before any of them is used: the kernel is bound by how many
  // bytes it keeps in flight, not by arithmetic
  for (int t0 = t_begin + warp * 4; t0 < t_end; t0 += PA_TOKENS_PER_STEP * PA_UNROLL) {
    uint4 kraw[PA_UNROLL], vraw[PA_UNROLL];
#pragma unroll
    for (int u = 0; u < PA_UNROLL; ++u) {
      const int t = t0 + u * PA_TOKENS_PER_STEP + sub;
      kraw[u] = make_uint4(0, 0, 0, 0); vraw[u] = make_uint4(0, 0, 0, 0);
      if (t < t_end) {
        const int64_t blk = table[t / p.block_size];
        const int64_t tok = t % p.block_size;
        kraw[u] = ld16_stream(p.k + blk * p.k_sblk + tok * p.k_stok + (int64_t)kv_head * p.k_sh + part * 16);
        vraw[u] = ld16_stream(p.v + blk * p.v_sblk + tok * p.v_stok + (int64_t)kv_head * p.v_sh + part * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < PA_UNROLL; ++u) {
      const bool valid = t0 + u * PA_TOKENS_PER_STEP + sub < t_end;
      uint32_t kh[8], vh[8];
      fp8x16_to_half2(kraw[u], kh);
      fp8x16_to_half2(vraw[u], vh);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < 8; ++d) s = fma2_f32_f16(q[g][d], kh[d], s);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (valid) {  // uniform over the eight lanes of a token
          if (s > m[g]) {  // a new maximum (rare after the first tokens): rescale what is there
            const float corr = __expf(m[g] - s);
            l[g] *= corr;
#pragma unroll
            for (int d = 0; d < 16; ++d) acc[g][d] *= corr;
            m[g] = s;
          }
          const float pw = __expf(s - m[g]);
          l[g] += pw;
          const __half2 ph = __float2half2_rn(pw);
          const uint32_t pp = *reinterpret_cast<const uint32_t*>(&ph);
#pragma unroll
          for (int d = 0; d < 8; ++d) fma_pv(vh[d], pp, acc[g][2 * d], acc[g][2 * d + 1]);
        }
      }
    }
  }
  // merge the four lane groups of the warp (lanes with the same 16-dim slice)
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float m_new = fmaxf(m[g], m_o);
      const float c_s = m_new == -INFINITY ? 0.f : __expf(m[g] - m_new);
      const float c_o = m_new == -INFINITY ? 0.f : __expf(m_o - m_new);
      l[g] = l[g] * c_s + l_o * c_o;
#pragma unroll
      for (int d = 0; d < 16; ++d) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[g][d], o);
        acc[g][d] = acc[g][d] * c_s + a_o * c_o;
      }
      m[g] = m_new;
    }
  }
  // merge the warps through shared memory; warp 0 finishes
  __shared__ float sm_acc[PA_THREADS / 32][G][PA_HEAD_DIM];
  __shared__ float sm_ml[PA_THREADS / 32][G][2];
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int d = 0; d < 16; ++d) sm_acc[warp][g][part * 16 + d] = acc[g][d];
      if (part == 0) { sm_ml[warp][g][0] = m[g]; sm_ml[warp][g][1] = l[g]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * PA_HEAD_DIM; idx += PA_THREADS) {
    const int g = idx / PA_HEAD_DIM, d = idx % PA_HEAD_DIM;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < PA_THREADS / 32; ++w) mt = fmaxf(mt, sm_ml[w][g][0]);
    float lt = 0.f, at = 0.f;
#pragma unroll
    for (int w = 0; w < PA_THREADS / 32; ++w) {
      const float c = mt == -INFINITY ? 0.f : __expf(sm_ml[w][g][0] - mt);
      lt += sm_ml[w][g][1] * c;
      at += sm_acc[w][g][d] * c;
    }
    const int head = head0 + g;
    if (p.splits == 1) {
      p.out[(int64_t)b * p.o_sb + (int64_t)head * p.o_sh + d] = __float2bfloat16_rn(lt > 0.f ? at / lt : 0.f);
    } else {
      float* dst = p.partial + (((int64_t)b * p.n_heads + head) * p.splits + split) * PA_PARTIAL;
      dst[2 + d] = at;
      if (d == 0) { dst[0] = mt; dst[1] = lt; }
    }
  }
}

// out[b, head, :] from the splits' (m, l, unnormalised sums); one CTA of 128 threads per (b, head).
__global__ void __launch_bounds__(PA_HEAD_DIM)
paged_attention_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int64_t o_sb, int64_t o_sh,
                             int n_heads, int splits) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* src = partial + ((int64_t)b * n_heads + head) * splits * PA_PARTIAL;
  float mt = -INFINITY;
  for (int s = 0; s < splits; ++s) mt = fmaxf(mt, src[(int64_t)s * PA_PARTIAL]);
  float lt = 0.f, at = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float c = mt == -INFINITY ? 0.f : __expf(src[(int64_t)s * PA_PARTIAL] - mt);
    lt += src[(int64_t)s * PA_PARTIAL + 1] * c;
    at += src[(int64_t)s * PA_PARTIAL + 2 + d] * c;
  }
  out[(int64_t)b * o_sb + (int64_t)head * o_sh + d] = __float2bfloat16_rn(lt > 0.f ? at / lt : 0.f);
}

// Split-KV plan: about eight CTAs per SM (two to four waves of resident CTAs, so that a partly
// filled last wave costs little), slices of at least 256 tokens and a multiple of the tokens a CTA
// takes per loop iteration.
static void pa_plan(int64_t batch, int64_t n_kv_heads, int64_t passes, int64_t max_ctx, int* splits, int* tokens_per_split) {
  const int64_t base = batch * n_kv_heads * passes;
  int64_t want = (8 * (int64_t)sm_count() + base - 1) / (base > 0 ? base : 1);
  const int64_t max_splits = (max_ctx + 255) / 256;
  if (want > max_splits) want = max_splits;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  int64_t tps = (max_ctx + want - 1) / want;
  constexpr int64_t quantum = PA_TOKENS_PER_STEP * PA_UNROLL;
  tps = (tps + quantum - 1) / quantum * quantum;
  if (tps < quantum) tps = quantum;
  *splits = (int)((max_ctx + tps - 1) / tps);
  if (*splits < 1) *splits = 1;
  *tokens_per_split = (int)tps;
}

static int pa_group_unit(int group) { return group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1); }

}  // namespace hilda

using namespace hilda;

extern "C" {

int64_t hilda_paged_attention_fp8_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int64_t max_blocks,
                                                  int64_t block_size) {
  if (batch <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_blocks <= 0 || block_size <= 0 || n_heads % n_kv_heads) return 256;
  const int group = (int)(n_heads / n_kv_heads);
  int splits, tps;
  pa_plan(batch, n_kv_heads, group / pa_group_unit(group), max_blocks * block_size, &splits, &tps);
  return splits > 1 ? batch * n_heads * splits * PA_PARTIAL * 4 + 256 : 256;
}

// q [batch, n_heads, 128] bf16 with element strides q_sb, q_sh (last dim contiguous); k_cache,
// v_cache fp8 e4m3 with element (= byte) strides per block, token and kv head (last dim
// contiguous, 16-byte aligned rows); block_tables int32 [batch, max_blocks] with row stride bt_sb;
// context_lens int32 [batch]; out [batch, n_heads, 128] bf16.
int hilda_paged_attention_fp8_decode(const void* q, int64_t q_sb, int64_t q_sh, const void* k_cache, int64_t k_sblk,
                                     int64_t k_stok, int64_t k_sh, const void* v_cache, int64_t v_sblk, int64_t v_stok,
                                     int64_t v_sh, void* out, int64_t o_sb, int64_t o_sh, const int32_t* block_tables,
                                     int64_t bt_sb, const int32_t* context_lens, void* workspace, float scale, int64_t batch,
                                     int64_t n_heads, int64_t n_kv_heads, int64_t head_dim, int64_t block_size,
                                     int64_t max_blocks, void* stream) {
  if (head_dim != PA_HEAD_DIM) return HILDA_ERR_SIZE;
  if (batch < 0 || n_heads <= 0 || n_kv_heads <= 0 || block_size <= 0 || max_blocks < 0) return HILDA_ERR_SIZE;
  if (n_heads % n_kv_heads != 0) return HILDA_ERR_ARG;
  if (batch == 0) return HILDA_OK;
  if (!q || !k_cache || !v_cache || !out || !block_tables || !context_lens) return HILDA_ERR_NULL;
  if (batch > 65535) return HILDA_ERR_SIZE;
  if (!aligned16(k_cache) || !aligned16(v_cache) || (k_sblk | k_stok | k_sh | v_sblk | v_stok | v_sh) % 16 != 0) return HILDA_ERR_ALIGN;
  PaParams p;
  p.q = (const __nv_bfloat16*)q; p.q_sb = q_sb; p.q_sh = q_sh;
  p.k = (const uint8_t*)k_cache; p.v = (const uint8_t*)v_cache;
  p.k_sblk = k_sblk; p.k_stok = k_stok; p.k_sh = k_sh; p.v_sblk = v_sblk; p.v_stok = v_stok; p.v_sh = v_sh;
  p.out = (__nv_bfloat16*)out; p.o_sb = o_sb; p.o_sh = o_sh;
  p.block_tables = block_tables; p.bt_sb = bt_sb; p.context_lens = context_lens;
  p.scale = scale; p.n_heads = (int)n_heads; p.n_kv_heads = (int)n_kv_heads; p.group = (int)(n_heads / n_kv_heads);
  p.block_size = (int)block_size; p.max_blocks = (int)max_blocks;
  const int G = pa_group_unit(p.group);
  const int passes = p.group / G;
  pa_plan(batch, n_kv_heads, passes, max_blocks * block_size, &p.splits, &p.tokens_per_split);
  if (max_blocks == 0) { p.splits = 1; p.tokens_per_split = PA_TOKENS_PER_STEP; }
  p.partial = nullptr;
  if (p.splits > 1) {
    if (!workspace) return HILDA_ERR_NULL;
    p.partial = reinterpret_cast<float*>(workspace);
  }
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((unsigned)(n_kv_heads * passes), (unsigned)batch, (unsigned)p.splits);
  if (G == 4) paged_attention_fp8_kernel<4><<<grid, PA_THREADS, 0, st>>>(p);
  else if (G == 2) paged_attention_fp8_kernel<2><<<grid, PA_THREADS, 0, st>>>(p);
  else paged_attention_fp8_kernel<1><<<grid, PA_THREADS, 0, st>>>(p);
  HILDA_LAUNCH_CHECK();
  if (p.splits > 1) {
    paged_attention_merge_kernel<<<dim3((unsigned)n_heads, (unsigned)batch), PA_HEAD_DIM, 0, st>>>(p.partial, p.out, o_sb, o_sh,
                                                                                                   p.n_heads, p.splits);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

}  // extern "C"
