// Persistent, warp-specialised bf16/fp16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// the fp32 accumulator in tensor memory (TMEM), double-buffered so the epilogue of one tile runs
// under the main loop of the next. Used three times by FusedLinearCrossEntropy:
//   logits  = hidden  x W^T   (A K-major, B K-major)  epilogue: round to 16 bit, store, online LSE stats
//   dHidden = dlogits x W     (A K-major, B MN-major) epilogue: store 16 bit / fp32
//   dW     += dlogits^T x hidden (A MN-major, B MN-major) epilogue: fp32 accumulate / final 16-bit store
//
// This file holds the single-CTA kernel and what it shares with the CTA-pair kernel
// (tcgen05_gemm2.cuh, the default): PTX wrappers, descriptors, tensor maps and the epilogues.
// CTA = 224 threads: lane 0 of warps 0 and 6 issue the TMA loads of operands A and B, warp 1 lane 0
// issues the MMAs (warp 1 also owns the TMEM allocation), warps 2-5 are the epilogue (one TMEM lane
// quadrant each). Tile 128 x 256, K block 64 (one 128-byte swizzle span), 4 stages of 48 KB. Every
// mbarrier wait is bounded: if one runs out, the CTA records a code in the status word, stops,
// frees its TMEM and returns.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace hilda {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int GEMM_STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_SMEM_BYTES = GEMM_STAGES * STAGE_BYTES + 1024;  // + slack for 1024-byte alignment
constexpr int GEMM_THREADS = 224;  // warp 0: TMA of A, warp 1: MMA, warps 2-5: epilogue, warp 6: TMA of B
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t WAIT_CAP = 1u << 22;  // bounded spin: default number of try_wait attempts before giving up

enum GemmEpilogue {
  EPI_STORE16 = 0,      // C16 = acc
  EPI_LOGITS_STATS = 1, // C16 = acc (padded scratch, unmasked) + per (row, n-tile) (max2, sumexp2) of the rounded values
  EPI_STORE32 = 2,      // C32 = acc
  EPI_ACCUM32 = 3,      // C32 += acc
  EPI_ACCUM_FINAL16 = 4 // C16 = C32 + acc
};

struct GemmParams {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int m_fast;        // 1: consecutive tiles walk M first (B tile shared), 0: walk N first
  uint32_t idesc;    // tcgen05 instruction descriptor
  int is_bf16;
  void* C16; int64_t ldc16;
  float* C32; int64_t ldc32;
  float2* stats; int64_t stats_ld;
  float stat_scale;  // EPI_LOGITS_STATS: factor on the rounded logits before the base-2 (max, sum-exp)
  int* status;       // device word; non-zero = a bounded wait ran out
  uint32_t mn_lbo, mn_sbo;  // descriptor byte offsets for MN-major operands (8192, 1024)
  int sm_limit;      // use at most this many SMs (0 = all): leaves room for a concurrent collective
  long long* probe;  // optional [gridDim.x][8] cycle counters of the role loops (null = off)
  int dry;           // 1, measurement only: the producer signals "full" without loading (results are garbage);
                     // 2, test of the bounded waits: the producer loads nothing and signals nothing
  uint32_t wait_cap; // try_wait attempts before a wait gives up
  // Row count known only on the device (ignored tokens compacted away without a host round trip):
  // rows = clamp(*dyn_rows - dyn_off, 0, extent) replaces M (dyn_dim 1: tiles beyond it are skipped)
  // or K (dyn_dim 2: k-blocks beyond it are skipped; rows between it and the next multiple of 64
  // must hold zeros). dyn_dim 0: off.
  const int* dyn_rows; int dyn_off; int dyn_dim;
};

// (m_tiles, k_blocks) after the device-side row count; TILE_M = rows per output tile.
template <int TILE_M>
__device__ __forceinline__ void gemm_dynamic_extent(const GemmParams& p, int& m_tiles, int& k_blocks) {
  m_tiles = p.m_tiles; k_blocks = p.k_blocks;
  if (p.dyn_dim == 0) return;
  int r = *p.dyn_rows - p.dyn_off;
  if (p.dyn_dim == 1) {
    r = r < 0 ? 0 : (r > p.M ? p.M : r);
    m_tiles = (r + TILE_M - 1) / TILE_M;
  } else {
    r = r < 0 ? 0 : (r > p.K ? p.K : r);
    k_blocks = (r + BK - 1) / BK;
  }
}

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// Bounded wait. Returns false if the wait ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          uint32_t cap) {
  for (uint32_t it = 0; it < cap; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Halves of the 64-bit shared-memory matrix descriptor, 128-byte swizzle: the low word carries the
// start address (16-byte units, bits 0-13) and LBO (bits 16-29); the high word SBO (bits 32-45),
// the sm_100 descriptor version (bit 46) and the swizzle mode (bits 61-63 = 2). K-major operand:
// rows of 128 bytes, SBO = 1024 (8 rows), LBO unused. MN-major operand: 64-element (128-byte) runs
// along M/N, LBO = byte distance between consecutive 64-element groups, SBO = byte distance between
// groups of 8 K rows. The issuing thread keeps the halves in registers and only adds a constant to
// the low word between MMAs.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint32_t smem_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
// One k-block of the issuer, as a single instruction sequence: peek at the NEXT slot's "full"
// barrier first (its latency then hides under the MMA issue instead of sitting between two
// k-blocks), the four K = 16 MMAs of this slot, the commit that frees it, and only then the
// peek's result. Returns 1 when the next slot was already full. peek_bar == 0 skips the peek.
template <uint32_t A_KSTEP, uint32_t B_KSTEP>
__device__ __forceinline__ uint32_t umma_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t accumulate, uint32_t empty_bar_addr,
                                                uint32_t peek_bar, uint32_t peek_parity) {
  uint32_t ready;
  asm volatile(
      "{\n.reg .pred p, q, t;\n.reg .b64 da, db;\n.reg .b32 al, bl;\n"
      "setp.ne.b32 t, %9, 0;\n"
      "mov.pred q, 0;\n"
      "@t mbarrier.try_wait.parity.shared::cta.b64 q, [%9], %10;\n"
      "setp.ne.b32 p, %7, 0;\n"
      "mov.b64 da, {%2, %3};\n"
      "mov.b64 db, {%4, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %6, p;\n"
      "setp.ne.b32 p, 1, 0;\n"
      "add.u32 al, %2, %11;\n add.u32 bl, %4, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %6, p;\n"
      "add.u32 al, al, %11;\n add.u32 bl, bl, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %6, p;\n"
      "add.u32 al, al, %11;\n add.u32 bl, bl, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %6, p;\n"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%8];\n"
      "selp.u32 %0, 1, 0, q;\n}"
      : "=r"(ready)
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(empty_bar_addr),
        "r"(peek_bar), "r"(peek_parity), "n"(A_KSTEP), "n"(B_KSTEP)
      : "memory");
  return ready;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane = row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack16(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float unpack16_lo(uint32_t u, int is_bf16) {
  if (is_bf16) return __uint_as_float(u << 16);
  return __half2float(__ushort_as_half((unsigned short)(u & 0xffffu)));
}
__device__ __forceinline__ float unpack16_hi(uint32_t u, int is_bf16) {
  if (is_bf16) return __uint_as_float(u & 0xffff0000u);
  return __half2float(__ushort_as_half((unsigned short)(u >> 16)));
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Epilogue of one 128 x 256 accumulator tile for the calling thread (thread = TMEM lane = row).
// taddr0: TMEM address of column 0 of the accumulator in this warp's lane quadrant.
template <int EPI>
__device__ __forceinline__ void gemm_epilogue_tile(const GemmParams& p, uint32_t taddr0, int64_t row, int col0, int nt,
                                                   bool zero_acc = false) {
  if constexpr (EPI == EPI_ACCUM32 || EPI == EPI_ACCUM_FINAL16) {
    // C (+)= acc: the fp32 values of column chunk c + 1 are requested before chunk c is added and
    // stored, so that a tile's 8 round trips to memory overlap instead of following one another (the
    // tile has to be through here before the next one's main loop ends).
    const bool in_m = row < p.M;
    float* crow = p.C32 + row * p.ldc32 + col0;
    float4 nxt[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      nxt[j] = (in_m && col0 + 4 * j + 4 <= p.N) ? *reinterpret_cast<const float4*>(crow + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      float4 cur[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
      tmem_ld32(taddr0 + c * 32, r);
      const int cbase = col0 + c * 32;
      if (c + 1 < BN / 32) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          nxt[j] = (in_m && cbase + 32 + 4 * j + 4 <= p.N) ? *reinterpret_cast<const float4*>(crow + (c + 1) * 32 + 4 * j)
                                                            : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      tmem_ld_wait();
      if (zero_acc) {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (in_m) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[4 * j] = cur[j].x + __uint_as_float(r[4 * j]);
          v[4 * j + 1] = cur[j].y + __uint_as_float(r[4 * j + 1]);
          v[4 * j + 2] = cur[j].z + __uint_as_float(r[4 * j + 2]);
          v[4 * j + 3] = cur[j].w + __uint_as_float(r[4 * j + 3]);
        }
        if constexpr (EPI == EPI_ACCUM32) {
          float* c32 = crow + c * 32;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (cbase + 4 * j + 4 <= p.N)
              *reinterpret_cast<float4*>(c32 + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
          uint16_t* dst = reinterpret_cast<uint16_t*>(p.C16) + row * p.ldc16 + cbase;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (cbase + 8 * j + 8 <= p.N)
              *reinterpret_cast<uint4*>(dst + 8 * j) =
                  make_uint4(pack16(v[8 * j], v[8 * j + 1], p.is_bf16), pack16(v[8 * j + 2], v[8 * j + 3], p.is_bf16),
                             pack16(v[8 * j + 4], v[8 * j + 5], p.is_bf16), pack16(v[8 * j + 6], v[8 * j + 7], p.is_bf16));
        }
      }
    }
    return;
  }
  float run_m = -INFINITY, run_s = 0.f;
  const float stat_scale = p.stat_scale;  // log2(e) / temperature: the statistics are of logits / temperature
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr0 + c * 32, r);
    tmem_ld_wait();
    if (zero_acc) {  // no k-block ran (a device-side row count of zero): the product is zero
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    const int cbase = col0 + c * 32;
    if constexpr (EPI == EPI_STORE16 || EPI == EPI_LOGITS_STATS) {
      uint32_t h[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) h[j] = pack16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), p.is_bf16);
      if constexpr (EPI == EPI_LOGITS_STATS) {
        // scratch is padded to whole tiles: unmasked stores
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C16) + row * p.ldc16 + cbase);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
        // online (max, sum-exp) in the log2 domain over the ROUNDED values, columns >= N masked
        float y[32];
        float cm = -INFINITY;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float lo = unpack16_lo(h[j], p.is_bf16) * stat_scale;
          const float hi = unpack16_hi(h[j], p.is_bf16) * stat_scale;
          y[2 * j] = (cbase + 2 * j < p.N) ? lo : -INFINITY;
          y[2 * j + 1] = (cbase + 2 * j + 1 < p.N) ? hi : -INFINITY;
          cm = fmaxf(cm, fmaxf(y[2 * j], y[2 * j + 1]));
        }
        const float m_new = fmaxf(run_m, cm);
        if (m_new != -INFINITY) {
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) s += ex2_fast(y[j] - m_new);
          run_s = run_s * ex2_fast(run_m - m_new) + s;
          run_m = m_new;
        }
      } else {
        if (row < p.M) {
          uint16_t* dst = reinterpret_cast<uint16_t*>(p.C16) + row * p.ldc16 + cbase;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (cbase + 8 * j + 8 <= p.N)
              *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
        }
      }
    } else {
      if (row < p.M) {
        float* c32 = p.C32 + row * p.ldc32 + cbase;
        if constexpr (EPI == EPI_STORE32) {  // (the accumulate epilogues returned above)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (cbase + 4 * j + 4 <= p.N)
              *reinterpret_cast<uint4*>(c32 + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
      }
    }
  }
  if constexpr (EPI == EPI_LOGITS_STATS) {
    if (row < p.M) p.stats[row * p.stats_ld + nt] = make_float2(run_m, run_s);
  }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
tcgen05_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[GEMM_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GEMM_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 4); }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  int m_tiles_d, k_blocks_d;
  gemm_dynamic_extent<BM>(p, m_tiles_d, k_blocks_d);
  const int total_tiles = m_tiles_d * p.n_tiles;
  const uint32_t wait_cap = p.wait_cap;

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers
    // Warp 0 copies operand A and posts the expect-tx arrive, warp 6 copies operand B: two
    // threads issue a slot's copies side by side. The ring is latency-bound (slot freed -> copy
    // issued -> data landed -> MMA), so nothing sits between the wait for a free slot and the
    // copies but the copies themselves: addresses and coordinates are ready before the wait, and
    // the expect-tx arrive follows the copies (the transaction count may run negative until then).
    if (lane == 0) {
      const bool is_a = warp == 0;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      long long w_empty = 0;
      const long long t_begin = clock64();
      const bool probing = p.probe != nullptr;
      const int dry = p.dry;
      const int k_blocks = k_blocks_d;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mt = p.m_fast ? tile % m_tiles_d : tile / p.n_tiles;
        const int nt = p.m_fast ? tile / m_tiles_d : tile % p.n_tiles;
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0, kc = 0; kb < k_blocks; ++kb, kc += BK) {
          const uint32_t fb = full0 + stage * 8u, eb = empty0 + stage * 8u;
          const uint32_t sA = stage_base + stage * STAGE_BYTES;
          const uint32_t sB = sA + A_STAGE_BYTES;
          const uint32_t want = phase ^ 1u;
          if (++stage == GEMM_STAGES) { stage = 0; phase ^= 1u; }
          const long long t0 = probing ? clock64() : 0;
          if (!mbar_wait(eb, want, abortp, p.status, 1, wait_cap)) { ok = false; break; }
          if (probing) w_empty += clock64() - t0;
          if (dry == 2) continue;  // test hook: nothing is loaded or signalled, so the issuer's wait runs out
          if (is_a) {
            if (dry) { mbar_arrive(fb); continue; }
            if constexpr (!A_MN) {
              tma_load_2d(sA, &tmA, fb, kc, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sA + j * 8192, &tmA, fb, m0 + j * 64, kc);
            }
            mbar_expect_tx(fb, STAGE_BYTES);
          } else {
            if (dry) continue;
            if constexpr (!B_MN) {
              tma_load_2d(sB, &tmB, fb, kc, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &tmB, fb, n0 + j * 64, kc);
            }
          }
        }
      }
      if (probing && is_a) { p.probe[blockIdx.x * 8 + 0] = w_empty; p.probe[blockIdx.x * 8 + 1] = clock64() - t_begin; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      long long w_full = 0, w_tempty = 0;
      const long long t_begin = clock64();
      // everything the loop needs, in registers: this thread's instruction latency per k-block
      // has to stay under the 4 x 128 cycles the tensor pipe takes for it
      const bool probing = p.probe != nullptr;
      const int k_blocks = k_blocks_d;
      const uint32_t idesc = p.idesc;
      const uint32_t a_hi = smem_desc_hi(A_MN ? p.mn_sbo : 1024u), b_hi = smem_desc_hi(B_MN ? p.mn_sbo : 1024u);
      const uint32_t a_lo0 = smem_desc_lo(stage_base, A_MN ? p.mn_lbo : 0u);
      const uint32_t b_lo0 = smem_desc_lo(stage_base + A_STAGE_BYTES, B_MN ? p.mn_lbo : 0u);
      constexpr uint32_t A_KSTEP = (A_MN ? 2048u : 32u) >> 4, B_KSTEP = (B_MN ? 2048u : 32u) >> 4;  // per UMMA_K, 16-byte units
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      uint32_t ready = 0;  // set when the peek of the previous k-block already saw this slot full
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const long long t1 = probing ? clock64() : 0;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1u, abortp, p.status, 2, wait_cap)) break;
        if (probing) w_tempty += clock64() - t1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0;
        const bool more_tiles = tile + (int)gridDim.x < total_tiles;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready) {
            const long long t0 = probing ? clock64() : 0;
            if (!mbar_wait(full0 + stage * 8u, phase, abortp, p.status, 3, wait_cap)) { ok = false; break; }
            if (probing) w_full += clock64() - t0;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (uint32_t)(STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (uint32_t)(STAGE_BYTES >> 4);
          const uint32_t empty_addr = empty0 + stage * 8u;
          if (++stage == GEMM_STAGES) { stage = 0; phase ^= 1u; }
          // the next slot of the ring is this CTA's next k-block, in this tile or its next one
          const uint32_t peek = (kb + 1 < k_blocks || more_tiles) ? full0 + stage * 8u : 0u;
          ready = umma_kblock<A_KSTEP, B_KSTEP>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accum, empty_addr, peek, phase);
          accum = 1u;
        }
        if (!ok) break;
        umma_commit(smem_u32(&tfull_bar[acc]));  // accumulator complete
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (p.probe) {
        p.probe[blockIdx.x * 8 + 2] = w_full; p.probe[blockIdx.x * 8 + 3] = w_tempty;
        p.probe[blockIdx.x * 8 + 4] = clock64() - t_begin;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    const int row_in_tile = q * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    long long w_tfull = 0, t_epi = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int mt = p.m_fast ? tile % m_tiles_d : tile / p.n_tiles;
      const int nt = p.m_fast ? tile / m_tiles_d : tile % p.n_tiles;
      const long long t0 = p.probe ? clock64() : 0;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abortp, p.status, 4, wait_cap)) break;
      const long long t1 = p.probe ? clock64() : 0;
      w_tfull += t1 - t0;
      tc_fence_after();
      const int64_t row = (int64_t)mt * BM + row_in_tile;
      const int col0 = nt * BN;
      const uint32_t taddr0 = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      gemm_epilogue_tile<EPI>(p, taddr0, row, col0, nt, k_blocks_d == 0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if (p.probe) t_epi += clock64() - t1;
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.probe && warp == 2 && lane == 0) { p.probe[blockIdx.x * 8 + 5] = w_tfull; p.probe[blockIdx.x * 8 + 6] = t_epi; }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major 16-bit tensor [outer, inner] with row pitch `pitch_elems`; box [box_outer, box_inner];
// 128-byte swizzle; out-of-range elements read as zero.
static inline int make_tmap_2d(CUtensorMap* tm, const void* base, int is_bf16, uint64_t inner, uint64_t outer,
                               uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return HILDA_ERR_CUDA;
  if (!aligned16(base) || (pitch_elems * 2) % 16 != 0) return HILDA_ERR_ALIGN;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HILDA_OK : HILDA_ERR_CUDA;
}

static inline uint32_t make_idesc(int is_bf16, bool a_mn, bool b_mn) {
  const uint32_t fmt = is_bf16 ? 1u : 0u;  // kind::f16: 0 = f16, 1 = bf16
  return (1u << 4)                          // D format f32
         | (fmt << 7) | (fmt << 10)         // A, B formats
         | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16)
         | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// C[M,N] = A x B with A given as [M,K] (K-major, a_mn=false) or stored [K,M] (MN-major, a_mn=true),
// B given as [N,K] (K-major) or stored [K,N] (MN-major). lda/ldb are row pitches in elements of the
// STORED matrices.
template <bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, GemmParams p, cudaStream_t st) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return HILDA_ERR_SIZE;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, p.is_bf16, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda, BK, BM);
  else rc = make_tmap_2d(&tmA, A, p.is_bf16, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda, 64, BK);
  if (rc != HILDA_OK) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, p.is_bf16, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb, BK, BN);
  else rc = make_tmap_2d(&tmB, B, p.is_bf16, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb, 64, BK);
  if (rc != HILDA_OK) return rc;
  p.m_tiles = (p.M + BM - 1) / BM;
  p.n_tiles = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + BK - 1) / BK;
  p.idesc = make_idesc(p.is_bf16, A_MN, B_MN);
  if (p.mn_lbo == 0) { p.mn_lbo = 8192; p.mn_sbo = 1024; }
  auto kern = tcgen05_gemm_kernel<A_MN, B_MN, EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess)
    return HILDA_ERR_CUDA;
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  if (tiles > 0x7fffffffLL) return HILDA_ERR_SIZE;
  int grid = sm_count();
  if (p.sm_limit > 0 && p.sm_limit < grid) grid = p.sm_limit;
  if (tiles < grid) grid = (int)tiles;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(tmA, tmB, p);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // namespace hilda
