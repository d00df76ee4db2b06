// Decode attention over a paged FP8 (e4m3) KV cache. Replaces the Triton kernel of hilda-kernel's
// kernels/paged_attention_fp8.py (_paged_attention_fp8_decode_kernel :7-92): one query token per
// sequence, q [batch, heads, 128] bf16, K / V cache [blocks, block_size, kv_heads, 128] fp8, a block
// table and a context length per sequence, output bf16.
//
// HBM-bound on the KV cache, which is read ONCE per kv head: a CTA serves all query heads of one
// (sequence, kv head) (the reference launches one program per query head and re-reads K / V for
// every head of a GQA group) over a slice of the context (split-KV: slices are merged by a second
// small kernel when there is more than one). One warp per kv head; eight lanes share a token: each loads 16 bytes
// (16 fp8) of its K row and its V row, so a warp touches four whole 128-byte rows per load; the
// dot product is reduced over the eight lanes with three shuffles; every lane group keeps its own
// online-softmax state (max, sum, 16 output dims per head), merged at the end.
#include <cuda_fp8.h>

#include "common.cuh"
#include "hilda_b200.h"

namespace hilda {

constexpr int PA_HEAD_DIM = 128;
constexpr int PA_MAX_WARPS = 8;          // head groups (kv head x pass) per CTA, one warp each
constexpr int PA_TOKENS_PER_STEP = 4;    // tokens a warp takes per step (eight lanes each)
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

// G query heads of one kv head per pass. Grid (CTAs of head groups, batch, context splits); one
// WARP per head group (kv head x pass), no cross-warp merge, and all the head groups of a sequence
// side by side in a CTA, so that the 128-byte rows of the different kv heads of a token (adjacent
// in the cache) are requested at about the same time. Measured against one CTA of four warps per
// kv head with a shared-memory merge: 87 instead of 105 us at batch 32 x 4096 tokens; letting one
// warp cover four adjacent kv heads of a single token (512 contiguous bytes per load) was slower.
template <int G>
__global__ void __launch_bounds__(PA_MAX_WARPS * 32, G <= 2 ? 2 : 1)
paged_attention_fp8_kernel(const PaParams p) {
  const int passes = p.group / G;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hg = blockIdx.x * (blockDim.x >> 5) + warp;     // head group of this warp
  if (hg >= p.n_kv_heads * passes) return;                   // no block-wide barrier below
  const int kv_head = hg / passes, pass = hg % passes;
  const int b = blockIdx.y, split = blockIdx.z;
  const int head0 = kv_head * p.group + pass * G;  // first query head of this warp
  const int sub = lane >> 3, part = lane & 7;      // token within the step, 16-dim slice
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
  // Software pipeline: the loads of the NEXT iteration (PA_UNROLL steps) are issued before this
  // iteration's values are used, so that every warp always has loads in flight; the kernel is
  // bound by the bytes it keeps in flight, not by arithmetic.
  auto load_steps = [&](int t0, uint4* kr, uint4* vr) {
#pragma unroll
    for (int u = 0; u < PA_UNROLL; ++u) {
      const int t = t0 + u * PA_TOKENS_PER_STEP + sub;
      kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0);
      if (t < t_end) {
        const int64_t blk = table[t / p.block_size];
        const int64_t tok = t % p.block_size;
        kr[u] = ld16_stream(p.k + blk * p.k_sblk + tok * p.k_stok + (int64_t)kv_head * p.k_sh + part * 16);
        vr[u] = ld16_stream(p.v + blk * p.v_sblk + tok * p.v_stok + (int64_t)kv_head * p.v_sh + part * 16);
      }
    }
  };
  constexpr int PA_ITER = PA_TOKENS_PER_STEP * PA_UNROLL;
  uint4 kraw[PA_UNROLL], vraw[PA_UNROLL], knext[PA_UNROLL], vnext[PA_UNROLL];
  load_steps(t_begin, kraw, vraw);
  for (int t0 = t_begin; t0 < t_end; t0 += PA_ITER) {
    load_steps(t0 + PA_ITER, knext, vnext);  // past t_end: nothing is loaded
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
#pragma unroll
    for (int u = 0; u < PA_UNROLL; ++u) { kraw[u] = knext[u]; vraw[u] = vnext[u]; }
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
  // lanes 0-7 hold the warp's result for their 16 dims
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int head = head0 + g;
      if (p.splits == 1) {
        const float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
        __nv_bfloat16* dst = p.out + (int64_t)b * p.o_sb + (int64_t)head * p.o_sh + part * 16;
#pragma unroll
        for (int d = 0; d < 16; ++d) dst[d] = __float2bfloat16_rn(acc[g][d] * inv);
      } else {
        float* dst = p.partial + (((int64_t)b * p.n_heads + head) * p.splits + split) * PA_PARTIAL;
#pragma unroll
        for (int d = 0; d < 16; ++d) dst[2 + part * 16 + d] = acc[g][d];
        if (part == 0) { dst[0] = m[g]; dst[1] = l[g]; }
      }
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

// Split-KV plan: the number of context slices is the one (up to 64, slices of at least 256 tokens)
// that best fills whole waves of resident CTAs (ctas_per_sm per SM, what the kernel's launch bounds
// allow); more slices win ties above two waves, fewer below. tokens_per_split is a multiple of the
// tokens a CTA takes per loop iteration.
static void pa_plan(int64_t batch, int64_t n_kv_heads, int64_t passes, int64_t max_ctx, int ctas_per_sm, int* splits,
                    int* tokens_per_split) {
  constexpr int64_t quantum = PA_TOKENS_PER_STEP * PA_UNROLL;
  const int64_t hg_ctas = (n_kv_heads * passes + PA_MAX_WARPS - 1) / PA_MAX_WARPS;
  const int64_t base = batch * hg_ctas > 0 ? batch * hg_ctas : 1;
  const int64_t slots = (int64_t)sm_count() * ctas_per_sm;
  int64_t max_splits = max_ctx / 256;
  if (max_splits > 64) max_splits = 64;
  if (max_splits < 1) max_splits = 1;
  int64_t best = 1;
  double best_score = -1.0;
  for (int64_t s = 1; s <= max_splits; ++s) {
    const int64_t ctas = base * s;
    const int64_t waves = (ctas + slots - 1) / slots;
    // efficiency of the wave fill, with a small preference for fewer slices (less merge work)
    const double score = (double)ctas / (double)(waves * slots) - 0.002 * (double)s;
    if (score > best_score) { best_score = score; best = s; }
  }
  int64_t tps = (max_ctx + best - 1) / best;
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
  const int unit = pa_group_unit(group);
  pa_plan(batch, n_kv_heads, group / unit, max_blocks * block_size, unit <= 2 ? 2 : 1, &splits, &tps);
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
  pa_plan(batch, n_kv_heads, passes, max_blocks * block_size, G <= 2 ? 2 : 1, &p.splits, &p.tokens_per_split);
  if (max_blocks == 0) { p.splits = 1; p.tokens_per_split = PA_TOKENS_PER_STEP; }
  p.partial = nullptr;
  if (p.splits > 1) {
    if (!workspace) return HILDA_ERR_NULL;
    p.partial = reinterpret_cast<float*>(workspace);
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int head_groups = (int)n_kv_heads * passes;
  const int warps = head_groups < PA_MAX_WARPS ? head_groups : PA_MAX_WARPS;
  const dim3 grid((unsigned)((head_groups + warps - 1) / warps), (unsigned)batch, (unsigned)p.splits);
  if (G == 4) paged_attention_fp8_kernel<4><<<grid, warps * 32, 0, st>>>(p);
  else if (G == 2) paged_attention_fp8_kernel<2><<<grid, warps * 32, 0, st>>>(p);
  else paged_attention_fp8_kernel<1><<<grid, warps * 32, 0, st>>>(p);
  HILDA_LAUNCH_CHECK();
  if (p.splits > 1) {
    paged_attention_merge_kernel<<<dim3((unsigned)n_heads, (unsigned)batch), PA_HEAD_DIM, 0, st>>>(p.partial, p.out, o_sb, o_sh,
                                                                                                   p.n_heads, p.splits);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

}  // extern "C"
