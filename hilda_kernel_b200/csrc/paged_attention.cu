// Decode attention over a paged FP8 (e4m3) KV cache. Replaces the Triton kernel of hilda-kernel's
// kernels/paged_attention_fp8.py (_paged_attention_fp8_decode_kernel :7-92): one query token per
// sequence, q [batch, heads, 128] bf16, K / V cache [blocks, block_size, kv_heads, 128] fp8, a block
// table and a context length per sequence, output bf16.
//
// HBM-bound on the KV cache, which is read ONCE per kv head: a warp serves all query heads of one
// (sequence, kv head) (the reference launches one program per query head and re-reads K / V for
// every head of a GQA group) over a slice of the context (split-KV: slices are merged by a second
// small kernel when there is more than one). q.k and p.v run as mma.sync over 16 tokens x up to 8
// query heads, K / V staged through shared memory with cp.async. (A CUDA-core formulation, one FMA
// per query head and element with eight lanes sharing a token, took 87 us where this takes 58 and
// was removed: it covered no shape this kernel does not.)
#include <cuda_fp8.h>

#include <cstdlib>

#include "common.cuh"
#include "hilda_b200.h"

namespace hilda {

constexpr int PA_HEAD_DIM = 128;
constexpr int PA_MAX_WARPS = 8;          // head groups (kv head x pass) per CTA, one warp each
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
  int passes;  // tensor-core kernel: passes of up to eight query heads per kv head
};

// ------------------------------------------------------------------------- the kernel
// Both contractions go to mma.sync (m16n8k16, fp16 inputs, fp32
// accumulators) with the KV TOKENS in the M dimension and the query heads of the kv head (up to
// eight per pass) in N, so that a GQA group of any size up to eight costs the same instructions:
//   S^T [16 tokens x 8 heads] = K [16 tokens x 128] . Q^T          (8 MMAs over 128 dims)
//   O^T [128 dims x 8 heads] += V^T [128 x 16 tokens] . P^T        (8 MMAs of 16 dims)
// A warp owns one (kv head, pass) and walks its context slice 16 tokens at a time. Per step every
// lane copies eight 16-byte pieces of the K and V rows (exactly the bytes its own MMA fragments
// are built from) into its own shared-memory slots with cp.async, PM_STAGES steps ahead; a lane
// reads back only what it copied, so there is no barrier, only cp.async.wait_group.
//
// Fragment bookkeeping (g = lane / 4, j = lane % 4). The contraction index of an MMA may be any
// permutation of the real index as long as both operands use the same one:
//  * q.k: lane (g, j) holds bytes [16j, 16j+16) and [64+16j, 64+16j+16) of the K rows of tokens g
//    and g+8. k-step s (0..7) takes word s%4 of the first (s < 4) or second piece: its low half
//    (two fp8 -> one half2) is the A fragment's columns 2j, 2j+1, its high half columns 2j+8, 2j+9.
//    The B fragment is q[head g] at the same four dims.
//  * S^T arrives as (token g | g+8; heads 2j, 2j+1) per lane. The online softmax runs there in
//    fp32 (max over tokens = over g: three shuffles); p is rounded to fp16, and movmatrix turns
//    (token g; heads 2j, 2j+1) into (head g; tokens 2j, 2j+1) = the B fragment of the second MMA.
//  * p.v: lane (g, j) holds bytes [16g, 16g+16) of the V rows of tokens 2j, 2j+1, 2j+8, 2j+9.
//    MMA i (0..7) has row g = dim 16g+i and row g+8 = dim 16g+8+i; its A registers pair the same
//    byte of two tokens (one prmt per two bytes, then fp8x2 -> half2).
//  * O^T accumulators: acc[i][0..3] = (dim 16g+i, heads 2j, 2j+1), (dim 16g+8+i, heads 2j, 2j+1):
//    lane (g, j) ends with dims [16g, 16g+16) of heads 2j and 2j+1.
constexpr int PM_STEP = 16;                          // tokens per step (the M of the first MMA)
constexpr int PM_STAGES = 3;                         // steps in flight per warp
constexpr int PM_STAGE_BYTES = 8 * 32 * 16;          // eight 16-byte pieces per lane
constexpr int PM_WARP_SMEM = PM_STAGES * PM_STAGE_BYTES;

// .ca, not .cg: with .cg (L1 bypassed) every lane's 16 bytes went to L2 as a sector request of its
// own, two per 32-byte sector (measured: 16.8 M sectors for 8.4 M sectors of cache, 67 instead of
// 58 us); through L1 the two halves of a sector are one request. Staging whole 128-byte rows with
// one cp.async.bulk per lane on an mbarrier per (warp, stage) instead was measured at 79 us: the
// copy engine's rate of 128-byte requests, not the memory system, then sets the pace.
__device__ __forceinline__ void pm_cp_async16(uint32_t smem_dst, const void* gsrc, bool valid) {
  const int n = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled and nothing is read
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void pm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xffffu), __NV_E4M3);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float warp_max_over_g(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float warp_sum_over_g(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  return v + __shfl_xor_sync(0xffffffffu, v, 16);
}

// Grid (CTAs of head groups, batch, context splits) as above; a head group is (kv head, pass of up
// to eight query heads). Dynamic shared memory: PM_WARP_SMEM bytes per warp.
__global__ void __launch_bounds__(PA_MAX_WARPS * 32, 2)
paged_attention_fp8_mma_kernel(const PaParams p) {
  extern __shared__ __align__(16) uint8_t pm_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hg = blockIdx.x * (blockDim.x >> 5) + warp;
  if (hg >= p.n_kv_heads * p.passes) return;  // no block-wide barrier below
  const int kv_head = hg / p.passes, pass = hg % p.passes;
  const int b = blockIdx.y, split = blockIdx.z;
  const int head0 = kv_head * p.group + pass * 8;
  const int G = p.group - pass * 8 < 8 ? p.group - pass * 8 : 8;  // query heads of this pass
  const int g = lane >> 2, j = lane & 3;
  int ctx = p.context_lens[b];
  if (ctx > p.max_blocks * p.block_size) ctx = p.max_blocks * p.block_size;  // never index past the block table
  const int t_begin = split * p.tokens_per_split;  // a multiple of PM_STEP
  int t_end = t_begin + p.tokens_per_split;
  if (t_end > ctx) t_end = ctx;
  const int n_steps = t_end > t_begin ? (t_end - t_begin + PM_STEP - 1) / PM_STEP : 0;

  // B fragments of the first MMA: q[head g] * scale as fp16 at this lane's dims (zero for g >= G)
  uint32_t qf[8][2];
#pragma unroll
  for (int s = 0; s < 8; ++s) { qf[s][0] = 0u; qf[s][1] = 0u; }
  if (g < G) {
    const __nv_bfloat16* qp = p.q + (int64_t)b * p.q_sb + (int64_t)(head0 + g) * p.q_sh;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const __nv_bfloat16* qs = qp + (s < 4 ? 16 * j + 4 * s : 64 + 16 * j + 4 * (s - 4));
      qf[s][0] = pack_f16x2(__bfloat162float(qs[0]) * p.scale, __bfloat162float(qs[1]) * p.scale);
      qf[s][1] = pack_f16x2(__bfloat162float(qs[2]) * p.scale, __bfloat162float(qs[3]) * p.scale);
    }
  }
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;  // heads 2j (A) and 2j+1 (B)
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }

  const int32_t* table = p.block_tables + (int64_t)b * p.bt_sb;
  uint8_t* my_smem = pm_smem + warp * PM_WARP_SMEM + lane * 16;
  const uint32_t my_smem_u32 = (uint32_t)__cvta_generic_to_shared(my_smem);
  const uint8_t* k_lane = p.k + (int64_t)kv_head * p.k_sh + 16 * j;
  const uint8_t* v_lane = p.v + (int64_t)kv_head * p.v_sh + 16 * g;
  const bool block16 = p.block_size % PM_STEP == 0;  // a step never straddles two cache blocks

  // Copies of step n into stage n % PM_STAGES (nothing past the slice's end: the caller still
  // commits a group so that the group count stays in step with n). Steps are issued in order, so
  // the cache block of the next step is tracked incrementally (no division per step) and its
  // block-table entry is loaded one step early: the load is not on the path of the copies.
  int is_blk = t_begin / p.block_size, is_tok = t_begin % p.block_size;  // position of the next step to issue
  int64_t blk_ahead = t_begin < t_end ? table[is_blk] : 0;
  auto issue = [&](int n) {
    const int t0 = t_begin + n * PM_STEP;
    if (t0 >= t_end) return;
    const uint32_t dst = my_smem_u32 + (uint32_t)(n % PM_STAGES) * PM_STAGE_BYTES;
    const int tk[2] = {t0 + g, t0 + g + 8};
    const int tv[4] = {t0 + 2 * j, t0 + 2 * j + 1, t0 + 2 * j + 8, t0 + 2 * j + 9};
    if (block16) {
      const int64_t blk = blk_ahead;
      const int tok0 = is_tok;
      is_tok += PM_STEP;
      if (is_tok >= p.block_size) { is_tok = 0; ++is_blk; }
      if (t0 + PM_STEP < t_end) blk_ahead = table[is_blk];  // for the next call
      const uint8_t* kb = k_lane + blk * p.k_sblk + (int64_t)tok0 * p.k_stok;
      const uint8_t* vb = v_lane + blk * p.v_sblk + (int64_t)tok0 * p.v_stok;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint8_t* row = kb + (int64_t)(tk[c] - t0) * p.k_stok;
        pm_cp_async16(dst + (2 * c) * 512, row, tk[c] < t_end);
        pm_cp_async16(dst + (2 * c + 1) * 512, row + 64, tk[c] < t_end);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        pm_cp_async16(dst + (4 + c) * 512, vb + (int64_t)(tv[c] - t0) * p.v_stok, tv[c] < t_end);
    } else {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const bool ok = tk[c] < t_end;
        const int t = ok ? tk[c] : t0;  // any valid row: nothing is read from it
        const uint8_t* row = k_lane + (int64_t)table[t / p.block_size] * p.k_sblk + (int64_t)(t % p.block_size) * p.k_stok;
        pm_cp_async16(dst + (2 * c) * 512, row, ok);
        pm_cp_async16(dst + (2 * c + 1) * 512, row + 64, ok);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const bool ok = tv[c] < t_end;
        const int t = ok ? tv[c] : t0;
        const uint8_t* row = v_lane + (int64_t)table[t / p.block_size] * p.v_sblk + (int64_t)(t % p.block_size) * p.v_stok;
        pm_cp_async16(dst + (4 + c) * 512, row, ok);
      }
    }
  };

#pragma unroll
  for (int n = 0; n < PM_STAGES; ++n) { issue(n); pm_commit(); }
  for (int n = 0; n < n_steps; ++n) {
    pm_wait<PM_STAGES - 1>();  // step n's pieces have landed
    const uint8_t* sp = my_smem + (n % PM_STAGES) * PM_STAGE_BYTES;
    const int t0 = t_begin + n * PM_STEP;
    // ---- S^T = K . Q^T
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
    float s4b[4] = {0.f, 0.f, 0.f, 0.f};  // second accumulator: two chains of four dependent MMAs instead of one of eight
    {
      const uint4 k0a = *reinterpret_cast<const uint4*>(sp), k0b = *reinterpret_cast<const uint4*>(sp + 512);
      const uint4 k1a = *reinterpret_cast<const uint4*>(sp + 1024), k1b = *reinterpret_cast<const uint4*>(sp + 1536);
      const uint32_t w0[8] = {k0a.x, k0a.y, k0a.z, k0a.w, k0b.x, k0b.y, k0b.z, k0b.w};  // token g
      const uint32_t w1[8] = {k1a.x, k1a.y, k1a.z, k1a.w, k1b.x, k1b.y, k1b.z, k1b.w};  // token g + 8
#pragma unroll
      for (int s = 0; s < 8; ++s)
        mma_16816(s & 1 ? s4b : s4, e4m3x2_to_f16x2(w0[s]), e4m3x2_to_f16x2(w1[s]), e4m3x2_to_f16x2(w0[s] >> 16),
                  e4m3x2_to_f16x2(w1[s] >> 16), qf[s][0], qf[s][1]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) s4[c] += s4b[c];
    // ---- online softmax per head over this step's tokens (fp32)
    const bool ok0 = t0 + g < t_end, ok1 = t0 + g + 8 < t_end;
    const float sA0 = ok0 ? s4[0] : -INFINITY, sB0 = ok0 ? s4[1] : -INFINITY;
    const float sA1 = ok1 ? s4[2] : -INFINITY, sB1 = ok1 ? s4[3] : -INFINITY;
    const float mA_new = fmaxf(mA, warp_max_over_g(fmaxf(sA0, sA1)));  // finite: token t0 is valid
    const float mB_new = fmaxf(mB, warp_max_over_g(fmaxf(sB0, sB1)));
    if (__any_sync(0xffffffffu, mA_new > mA || mB_new > mB)) {  // rare after the first steps
      const float cA = __expf(mA - mA_new), cB = __expf(mB - mB_new);
      lA *= cA; lB *= cB;
#pragma unroll
      for (int i = 0; i < 8; ++i) { acc[i][0] *= cA; acc[i][2] *= cA; acc[i][1] *= cB; acc[i][3] *= cB; }
      mA = mA_new; mB = mB_new;
    }
    const float pA0 = __expf(sA0 - mA), pB0 = __expf(sB0 - mB), pA1 = __expf(sA1 - mA), pB1 = __expf(sB1 - mB);
    lA += pA0 + pA1; lB += pB0 + pB1;
    const uint32_t pb0 = movmatrix_trans(pack_f16x2(pA0, pB0));  // (head g; tokens 2j, 2j+1)
    const uint32_t pb1 = movmatrix_trans(pack_f16x2(pA1, pB1));  // (head g; tokens 2j+8, 2j+9)
    // ---- O^T += V^T . P^T
    {
      const uint4 r0 = *reinterpret_cast<const uint4*>(sp + 4 * 512), r1 = *reinterpret_cast<const uint4*>(sp + 5 * 512);
      const uint4 r2 = *reinterpret_cast<const uint4*>(sp + 6 * 512), r3 = *reinterpret_cast<const uint4*>(sp + 7 * 512);
      issue(n + PM_STAGES);  // this stage's pieces are all in registers now
      pm_commit();
      const uint32_t v0[4] = {r0.x, r0.y, r0.z, r0.w}, v1[4] = {r1.x, r1.y, r1.z, r1.w};  // tokens 2j, 2j+1
      const uint32_t v2[4] = {r2.x, r2.y, r2.z, r2.w}, v3[4] = {r3.x, r3.y, r3.z, r3.w};  // tokens 2j+8, 2j+9
#pragma unroll
      for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (int hsel = 0; hsel < 2; ++hsel) {
          const uint32_t sel = hsel == 0 ? 0x5140u : 0x7362u;  // bytes 0, 1 or 2, 3 of both words, interleaved
          const uint32_t a0p = __byte_perm(v0[w], v1[w], sel), a1p = __byte_perm(v0[w + 2], v1[w + 2], sel);
          const uint32_t a2p = __byte_perm(v2[w], v3[w], sel), a3p = __byte_perm(v2[w + 2], v3[w + 2], sel);
          const int i = 4 * w + 2 * hsel;
          mma_16816(acc[i], e4m3x2_to_f16x2(a0p), e4m3x2_to_f16x2(a1p), e4m3x2_to_f16x2(a2p), e4m3x2_to_f16x2(a3p), pb0, pb1);
          mma_16816(acc[i + 1], e4m3x2_to_f16x2(a0p >> 16), e4m3x2_to_f16x2(a1p >> 16), e4m3x2_to_f16x2(a2p >> 16),
                    e4m3x2_to_f16x2(a3p >> 16), pb0, pb1);
        }
      }
    }
  }
  pm_wait<0>();
  lA = warp_sum_over_g(lA);
  lB = warp_sum_over_g(lB);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (2 * j + h >= G) continue;
    const int head = head0 + 2 * j + h;
    const float m = h == 0 ? mA : mB, l = h == 0 ? lA : lB;
    if (p.splits == 1) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + (int64_t)b * p.o_sb + (int64_t)head * p.o_sh + 16 * g;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dst[i] = __float2bfloat16_rn(acc[i][h] * inv);
        dst[8 + i] = __float2bfloat16_rn(acc[i][2 + h] * inv);
      }
    } else {
      float* dst = p.partial + (((int64_t)b * p.n_heads + head) * p.splits + split) * PA_PARTIAL;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dst[2 + 16 * g + i] = acc[i][h];
        dst[2 + 16 * g + 8 + i] = acc[i][2 + h];
      }
      if (g == 0) { dst[0] = m; dst[1] = l; }
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
// allow); more slices win ties above two waves, fewer below. tokens_per_split is a multiple of
// quantum, the tokens a warp takes per loop iteration.
static void pa_plan(int64_t batch, int64_t n_kv_heads, int64_t passes, int64_t max_ctx, int ctas_per_sm, int64_t quantum,
                    int* splits, int* tokens_per_split) {
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

// Warps per CTA and CTAs per SM (shared memory and the 128-register bound of
// its launch bounds both allow sixteen warps per SM).
static void pm_shape(int64_t head_groups, int* warps, int* ctas_per_sm) {
  *warps = (int)(head_groups < PA_MAX_WARPS ? head_groups : PA_MAX_WARPS);
  int c = 16 / *warps;
  const int by_smem = (220 * 1024) / (*warps * PM_WARP_SMEM + 1024);
  if (c > by_smem) c = by_smem;
  *ctas_per_sm = c < 1 ? 1 : c;
}
static void pm_plan(int64_t batch, int64_t n_kv_heads, int group, int64_t max_ctx, int* passes, int* splits, int* tps) {
  *passes = (group + 7) / 8;
  int warps, ctas;
  pm_shape(n_kv_heads * *passes, &warps, &ctas);
  pa_plan(batch, n_kv_heads, *passes, max_ctx, ctas, PM_STEP, splits, tps);
}

}  // namespace hilda

using namespace hilda;

extern "C" {

int64_t hilda_paged_attention_fp8_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int64_t max_blocks,
                                                  int64_t block_size) {
  if (batch <= 0 || n_heads <= 0 || n_kv_heads <= 0 || max_blocks <= 0 || block_size <= 0 || n_heads % n_kv_heads) return 256;
  const int group = (int)(n_heads / n_kv_heads);
  int splits, tps, passes;
  pm_plan(batch, n_kv_heads, group, max_blocks * block_size, &passes, &splits, &tps);
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
  cudaStream_t st = (cudaStream_t)stream;
  pm_plan(batch, n_kv_heads, p.group, max_blocks * block_size, &p.passes, &p.splits, &p.tokens_per_split);
  if (max_blocks == 0) { p.splits = 1; p.tokens_per_split = PM_STEP; }
  p.partial = nullptr;
  if (p.splits > 1) {
    if (!workspace) return HILDA_ERR_NULL;
    p.partial = reinterpret_cast<float*>(workspace);
  }
  const int head_groups = (int)n_kv_heads * p.passes;
  int warps, ctas;
  pm_shape(head_groups, &warps, &ctas);
  const int smem = warps * PM_WARP_SMEM;
  void (*kern)(const PaParams) = paged_attention_fp8_mma_kernel;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return HILDA_ERR_CUDA;
  const dim3 grid((unsigned)((head_groups + warps - 1) / warps), (unsigned)batch, (unsigned)p.splits);
  kern<<<grid, warps * 32, smem, st>>>(p);
  HILDA_LAUNCH_CHECK();
  if (p.splits > 1) {
    paged_attention_merge_kernel<<<dim3((unsigned)n_heads, (unsigned)batch), PA_HEAD_DIM, 0, st>>>(p.partial, p.out, o_sb, o_sh,
                                                                                                   p.n_heads, p.splits);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

}  // extern "C"
