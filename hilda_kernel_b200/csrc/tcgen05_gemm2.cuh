// CTA-pair variant of the tcgen05 GEMM: two CTAs of a cluster (two SMs) work on one 256 x 256 tile
// with `tcgen05.mma.cta_group::2`. Each CTA stages its own 128 rows of A and 128 of the 256 columns
// of B (32 KB per stage instead of 48 KB, so 7 stages fit and the shared-memory operand traffic
// per SM drops by a third); the leader CTA (cluster rank 0) issues the MMAs, which read both CTAs'
// shared memory and write each CTA's half of the accumulator into that CTA's TMEM.
//
// Barriers (all mbarriers; every wait bounded):
//   full[s]    in the leader only: 1 arrival (leader's expect_tx of both CTAs' bytes) + the bytes of
//              both CTAs' TMA loads (the peer's loads signal the leader's barrier);
//   empty[s]   in each CTA: released by the leader's commit, delivered to both CTAs of the pair;
//   tfull[a]   in each CTA: accumulator a complete (same commit mechanism);
//   tempty[a]  in the leader only: 8 arrivals = 4 epilogue warps of each CTA (the peer arrives remotely).
// No TMA load here is a cluster broadcast: every CTA fetches its own operand tiles.
#pragma once
#include "tcgen05_gemm.cuh"

namespace hilda {

constexpr int G2_STAGES = 7;
constexpr int G2_B_ROWS = BN / 2;                      // B columns staged per CTA
constexpr int G2_A_BYTES = BM * BK * 2;                // 16 KB
constexpr int G2_B_BYTES = G2_B_ROWS * BK * 2;         // 16 KB
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + 1024;

__device__ __forceinline__ uint32_t g2_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t g2_map_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void g2_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes are credited to a barrier that may live in the peer CTA.
__device__ __forceinline__ void g2_tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void g2_mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void g2_tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void g2_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void g2_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive (once all prior MMAs of this thread retired) on the barrier at this shared-memory offset in
// BOTH CTAs of the pair.
__device__ __forceinline__ void g2_umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}

// One k-block of the pair's issuer as a single instruction sequence (see umma_kblock): peek at
// the next slot's "full" barrier, four cta_group::2 MMAs, the commit that frees the slot in both
// CTAs, then the peek's result.
template <uint32_t A_KSTEP, uint32_t B_KSTEP>
__device__ __forceinline__ uint32_t g2_umma_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                   uint32_t b_hi, uint32_t idesc, uint32_t accumulate,
                                                   uint32_t empty_bar_addr, uint32_t peek_bar, uint32_t peek_parity) {
  uint32_t ready;
  const uint16_t mask = 0x3;
  asm volatile(
      "{\n.reg .pred p, q, t;\n.reg .b64 da, db;\n.reg .b32 al, bl;\n"
      "setp.ne.b32 t, %9, 0;\n"
      "mov.pred q, 0;\n"
      "@t mbarrier.try_wait.parity.shared::cta.b64 q, [%9], %10;\n"
      "setp.ne.b32 p, %7, 0;\n"
      "mov.b64 da, {%2, %3};\n"
      "mov.b64 db, {%4, %5};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], da, db, %6, p;\n"
      "setp.ne.b32 p, 1, 0;\n"
      "add.u32 al, %2, %11;\n add.u32 bl, %4, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], da, db, %6, p;\n"
      "add.u32 al, al, %11;\n add.u32 bl, bl, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], da, db, %6, p;\n"
      "add.u32 al, al, %11;\n add.u32 bl, bl, %12;\n"
      "mov.b64 da, {al, %3};\n mov.b64 db, {bl, %5};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], da, db, %6, p;\n"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%8], %13;\n"
      "selp.u32 %0, 1, 0, q;\n}"
      : "=r"(ready)
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(empty_bar_addr),
        "r"(peek_bar), "r"(peek_parity), "n"(A_KSTEP), "n"(B_KSTEP), "h"(mask)
      : "memory");
  return ready;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
tcgen05_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[G2_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[G2_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = g2_cta_rank();
  const bool leader = (rank == 0);
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abortp = &abort_flag;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 8); }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    g2_tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    g2_tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  g2_cluster_sync();  // both CTAs' barriers are initialised and their TMEM allocated before any cross-CTA traffic
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  int m_tiles_d, k_blocks_d;  // m_tiles counts 256-row tiles here
  gemm_dynamic_extent<2 * BM>(p, m_tiles_d, k_blocks_d);
  const int total_tiles = m_tiles_d * p.n_tiles;
  const uint32_t wait_cap = p.wait_cap;

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ TMA producers (both CTAs)
    // as in the single-CTA kernel: warp 0 copies this CTA's half of A (and, in the leader, posts
    // the expect-tx arrive for both CTAs' bytes), warp 6 copies its half of B; nothing sits
    // between the wait for a free slot and the copies
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
      const uint32_t full0_leader = g2_map_rank(full0, 0);  // the leader's barriers, 8 bytes apart like ours
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
        const int mt = p.m_fast ? tile % m_tiles_d : tile / p.n_tiles;
        const int nt = p.m_fast ? tile / m_tiles_d : tile % p.n_tiles;
        const int m0 = mt * (2 * BM) + (int)rank * BM;        // this CTA's 128 rows of A
        const int n0 = nt * BN + (int)rank * G2_B_ROWS;        // this CTA's 128 columns of B
        for (int kb = 0, kc = 0; kb < k_blocks; ++kb, kc += BK) {
          const uint32_t fb_local = full0 + stage * 8u, fb = full0_leader + stage * 8u, eb = empty0 + stage * 8u;
          const uint32_t sA = stage_base + stage * G2_STAGE_BYTES;
          const uint32_t sB = sA + G2_A_BYTES;
          const uint32_t want = phase ^ 1u;
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1u; }
          const long long t0 = probing ? clock64() : 0;
          if (!mbar_wait(eb, want, abortp, p.status, 21, wait_cap)) { ok = false; break; }
          if (probing) w_empty += clock64() - t0;
          if (dry == 2) continue;  // test hook: nothing is loaded or signalled, so the issuer's wait runs out
          if (is_a) {
            if (dry) {
              if (leader) mbar_arrive(fb_local);
              continue;
            }
            if constexpr (!A_MN) {
              g2_tma_load_2d(sA, &tmA, fb, kc, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) g2_tma_load_2d(sA + j * 8192, &tmA, fb, m0 + j * 64, kc);
            }
            if (leader) mbar_expect_tx(fb_local, 2 * G2_STAGE_BYTES);
          } else {
            if (dry) continue;
            if constexpr (!B_MN) {
              g2_tma_load_2d(sB, &tmB, fb, kc, n0);
            } else {
#pragma unroll
              for (int j = 0; j < G2_B_ROWS / 64; ++j) g2_tma_load_2d(sB + j * 8192, &tmB, fb, n0 + j * 64, kc);
            }
          }
        }
      }
      if (probing && leader && is_a) { p.probe[pair * 8 + 0] = w_empty; p.probe[pair * 8 + 1] = clock64() - t_begin; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      long long w_full = 0, w_tempty = 0;
      const long long t_begin = clock64();
      const bool probing = p.probe != nullptr;
      const int k_blocks = k_blocks_d;
      const uint32_t idesc = p.idesc;
      const uint32_t a_hi = smem_desc_hi(A_MN ? p.mn_sbo : 1024u), b_hi = smem_desc_hi(B_MN ? p.mn_sbo : 1024u);
      const uint32_t a_lo0 = smem_desc_lo(stage_base, A_MN ? p.mn_lbo : 0u);
      const uint32_t b_lo0 = smem_desc_lo(stage_base + G2_A_BYTES, B_MN ? p.mn_lbo : 0u);
      constexpr uint32_t A_KSTEP = (A_MN ? 2048u : 32u) >> 4, B_KSTEP = (B_MN ? 2048u : 32u) >> 4;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      uint32_t ready = 0;  // set when the peek of the previous k-block already saw this slot full
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
        const long long t1 = probing ? clock64() : 0;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1u, abortp, p.status, 22, wait_cap)) break;
        if (probing) w_tempty += clock64() - t1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accum = 0;
        const bool more_tiles = tile + n_pairs < total_tiles;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ready) {
            const long long t0 = probing ? clock64() : 0;
            if (!mbar_wait(full0 + stage * 8u, phase, abortp, p.status, 23, wait_cap)) { ok = false; break; }
            if (probing) w_full += clock64() - t0;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (uint32_t)(G2_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (uint32_t)(G2_STAGE_BYTES >> 4);
          const uint32_t empty_addr = empty0 + stage * 8u;
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1u; }
          const uint32_t peek = (kb + 1 < k_blocks || more_tiles) ? full0 + stage * 8u : 0u;
          ready = g2_umma_kblock<A_KSTEP, B_KSTEP>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accum, empty_addr, peek, phase);
          accum = 1u;
        }
        if (!ok) break;
        g2_umma_commit_pair(smem_u32(&tfull_bar[acc]));  // accumulator halves complete in both CTAs
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (p.probe) {
        p.probe[pair * 8 + 2] = w_full; p.probe[pair * 8 + 3] = w_tempty; p.probe[pair * 8 + 4] = clock64() - t_begin;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    uint32_t acc = 0, acc_phase = 0;
    long long w_tfull = 0, t_epi = 0;
    for (int tile = pair; tile < total_tiles; tile += n_pairs) {
      const int mt = p.m_fast ? tile % m_tiles_d : tile / p.n_tiles;
      const int nt = p.m_fast ? tile / m_tiles_d : tile % p.n_tiles;
      const long long t0 = p.probe ? clock64() : 0;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abortp, p.status, 24, wait_cap)) break;
      const long long t1 = p.probe ? clock64() : 0;
      w_tfull += t1 - t0;
      tc_fence_after();
      const int64_t row = (int64_t)mt * (2 * BM) + (int64_t)rank * BM + row_in_tile;
      const uint32_t taddr0 = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      gemm_epilogue_tile<EPI>(p, taddr0, row, nt * BN, nt, k_blocks_d == 0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) g2_mbar_arrive_remote(g2_map_rank(smem_u32(&tempty_bar[acc]), 0));
      if (p.probe) t_epi += clock64() - t1;
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.probe && leader && warp == 2 && lane == 0) { p.probe[pair * 8 + 5] = w_tfull; p.probe[pair * 8 + 6] = t_epi; }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  __syncwarp();       // lanes of the producer / MMA warps rejoin before the warp-aligned cluster barrier
  g2_cluster_sync();  // neither CTA frees TMEM or exits while its peer may still touch it
  if (warp == 1) {
    tc_fence_after();
    g2_tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_gemm2(const void* A, int64_t lda, const void* B, int64_t ldb, GemmParams p, cudaStream_t st) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return HILDA_ERR_SIZE;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_2d(&tmA, A, p.is_bf16, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda, BK, BM);
  else rc = make_tmap_2d(&tmA, A, p.is_bf16, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda, 64, BK);
  if (rc != HILDA_OK) return rc;
  if (!B_MN) rc = make_tmap_2d(&tmB, B, p.is_bf16, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb, BK, G2_B_ROWS);
  else rc = make_tmap_2d(&tmB, B, p.is_bf16, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb, 64, BK);
  if (rc != HILDA_OK) return rc;
  p.m_tiles = (p.M + 2 * BM - 1) / (2 * BM);
  p.n_tiles = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + BK - 1) / BK;
  // instruction descriptor for the pair: M = 256
  const uint32_t fmt = p.is_bf16 ? 1u : 0u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
            ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
  if (p.mn_lbo == 0) { p.mn_lbo = 8192; p.mn_sbo = 1024; }
  auto kern = tcgen05_gemm2_kernel<A_MN, B_MN, EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_BYTES) != cudaSuccess)
    return HILDA_ERR_CUDA;
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  if (tiles > 0x7fffffffLL) return HILDA_ERR_SIZE;
  int pairs = sm_count() / 2;
  if (p.sm_limit > 0 && p.sm_limit / 2 < pairs) pairs = p.sm_limit / 2 > 0 ? p.sm_limit / 2 : 1;
  if (tiles < pairs) pairs = (int)tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(pairs * 2), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = G2_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
  return e == cudaSuccess ? HILDA_OK : HILDA_ERR_CUDA;
}

}  // namespace hilda
