// FusedLinearCrossEntropy for sm_100a: loss, d(hidden) and d(W) of CE(hidden @ W^T, targets) without
// ever holding the full [BT, V] logits.
//
// What it replaces: fused_linear_cross_entropy_forward (kernels/fused_linear_cross_entropy.py:103-171
// of hilda-kernel), a host loop over row chunks of {cuBLAS GEMM, Triton CE kernel, two more cuBLAS
// GEMMs, grad_weight += ...}. Here the tokens are processed in row chunks too, but
//   1. the lm_head GEMM runs on tcgen05/TMEM fed by TMA and its epilogue rounds the logits to the
//      compute dtype (as the reference's cuBLAS call does), stores them to a [chunk, V] scratch and
//      produces the online (max, sum-exp) statistics per (row, 256-column tile) in the same pass;
//   2. a small kernel merges the tile statistics per row (this is the only data a vocab-parallel
//      run has to exchange: max, sum-exp and the target logit per row);
//   3. one streaming pass turns the scratch into dlogits = (softmax - onehot) * scale in place;
//   4. dHidden = dlogits @ W and dW += dlogits^T @ hidden run on the same tcgen05 kernel with
//      MN-major operands (no transposed copies); dW is accumulated across chunks in fp32 and
//      rounded once at the end (the reference accumulates in the 16-bit dtype).
#include <cstdio>
#include <cstdlib>
#include "tcgen05_gemm2.cuh"
#include "reduce_kernels.cuh"

namespace hilda {

constexpr float FL_LOG2E = 1.4426950408889634f;
constexpr float FL_LN2 = 0.6931471805599453f;

// One warp per row: merge the per-tile (max2, sum2) pairs; fetch the target logit from the scratch.
// rowstat layout [3][rows]: natural-log max, sum of exp(x - max), target logit (0 if not in this shard).
__global__ void __launch_bounds__(256)
flce_row_stats_kernel(const float2* __restrict__ stats, int64_t stats_ld, int n_tiles, const uint16_t* __restrict__ logits,
                      int64_t pitch, const int64_t* __restrict__ targets, float* __restrict__ rowstat, int64_t rows,
                      int64_t V, int64_t vocab_start, int is_bf16, const int* __restrict__ dyn_rows, int64_t dyn_off) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  if (dyn_rows && row + dyn_off >= *dyn_rows) return;  // beyond the device-side row count: nothing was computed
  float m = -INFINITY;
  for (int t = lane; t < n_tiles; t += 32) m = fmaxf(m, stats[row * stats_ld + t].x);
  m = warp_max(m);
  float s = 0.f;
  for (int t = lane; t < n_tiles; t += 32) {
    const float2 v = stats[row * stats_ld + t];
    if (v.x != -INFINITY) s += v.y * exp2f(v.x - m);
  }
  s = warp_sum(s);
  if (lane == 0) {
    const int64_t t = targets ? targets[row] - vocab_start : -1;
    float xt = 0.f;
    if (t >= 0 && t < V) {
      const uint16_t raw = logits[row * pitch + t];
      xt = is_bf16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
    }
    rowstat[row] = m * FL_LN2;
    rowstat[rows + row] = s;
    rowstat[2 * rows + row] = xt;
  }
}

// lse = m + log(s); loss = lse - x_t on valid rows, 0 on ignored rows.
// With n_shards > 1, rowstat is [n_shards, 3, rows] (every vocabulary shard's triple, as gathered from
// the ranks) and the shards are merged first: M = max m_g, S = sum s_g exp(m_g - M), x_t = sum x_t,g
// (exactly one shard holds the target; the others contribute 0).
__global__ void __launch_bounds__(256)
flce_finalize_kernel(const float* __restrict__ rowstat, int n_shards, const int64_t* __restrict__ targets,
                     int64_t ignore_index, float* __restrict__ lse, float* __restrict__ loss_rows, int64_t rows,
                     const int* __restrict__ dyn_rows, int64_t dyn_off) {
  const int64_t row = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (row >= rows) return;
  if (dyn_rows && row + dyn_off >= *dyn_rows) { loss_rows[row] = 0.f; return; }
  float m = rowstat[row], sum = rowstat[rows + row], xt = rowstat[2 * rows + row];
  if (n_shards > 1) {
    for (int g = 1; g < n_shards; ++g) m = fmaxf(m, rowstat[(int64_t)g * 3 * rows + row]);
    sum = 0.f; xt = 0.f;
    for (int g = 0; g < n_shards; ++g) {
      const float* rs = rowstat + (int64_t)g * 3 * rows;
      const float mg = rs[row];
      if (mg != -INFINITY) sum += rs[rows + row] * expf(mg - m);
      xt += rs[2 * rows + row];
    }
  }
  const float l = m + logf(sum);
  lse[row] = l;
  loss_rows[row] = (targets[row] != ignore_index) ? (l - xt) : 0.f;
}

// In place on the scratch: x -> (exp(x - lse) - [col == target]) * scale; ignored rows -> 0.
template <typename T>
__global__ void __launch_bounds__(256)
flce_dlogits_kernel(T* __restrict__ logits, int64_t pitch, const float* __restrict__ lse,
                    const int64_t* __restrict__ targets, int64_t ignore_index, const int* __restrict__ n_valid,
                    int64_t V, int64_t vocab_start, const int* __restrict__ dyn_rows, int64_t dyn_off) {
  constexpr int VEC = VT<T>::N;
  const int64_t row = blockIdx.y;
  if (dyn_rows) {
    // Rows at or beyond the device-side row count carry the ignore index: up to the next multiple of 256
    // (what the GEMMs' last tile and k-block still touch) they are cleared below; the rest is never read.
    const int64_t live = ((int64_t)(*dyn_rows) - dyn_off + 255) / 256 * 256;
    if (row >= live) return;
  }
  T* xr = logits + row * pitch;
  const int64_t tgt = targets[row];
  const int64_t n_vec = (V + VEC - 1) / VEC;  // pitch is a multiple of 256: a ragged last vector stays in the row
  const int64_t v_begin = (int64_t)blockIdx.x * 256 * 4;
  if (tgt == ignore_index) {
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t v = v_begin + u * 256 + threadIdx.x;
      if (v < n_vec) st16(xr + v * VEC, z);
    }
    return;
  }
  const float scale = n_valid ? 1.0f / fmaxf((float)(*n_valid), 1.0f) : 1.0f;
  const float l2 = lse[row] * FL_LOG2E;
  const int64_t t = tgt - vocab_start;
  const int64_t tvec = (t >= 0 && t < V) ? t / VEC : -1;
  const int tsub = (int)(t - tvec * VEC);
  uint4 xv[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t v = v_begin + u * 256 + threadIdx.x;
    xv[u] = (v < n_vec) ? ld16(xr + v * VEC) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t v = v_begin + u * 256 + threadIdx.x;
    float f[VEC];
    VT<T>::unpack(xv[u], f);
#pragma unroll
    for (int j = 0; j < VEC; ++j) f[j] = scale * ex2_fast(fmaf(f[j], FL_LOG2E, -l2));
    if (v == tvec) {
#pragma unroll
      for (int j = 0; j < VEC; ++j)
        if (j == tsub) f[j] -= scale;
    }
    if (v < n_vec) st16(xr + v * VEC, VT<T>::pack(f));
  }
}

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// Index lists of the non-ignored rows, built on the device so that no host round trip is needed:
// idx[j] = source row of compacted row j (-1 for j >= n_valid), inv[i] = compacted position of source
// row i (-1 if ignored), t_c[j] = targets[idx[j]] (ignore_index for j >= n_valid), *n_valid = count.
// One CTA of 32 warps; warp w owns the contiguous range [w * per_warp, (w + 1) * per_warp) and walks it
// 32 elements at a time (coalesced), positions from ballot + popcount, so the order is kept.
__global__ void __launch_bounds__(1024)
flce_compact_kernel(const int64_t* __restrict__ targets, int64_t n, int64_t ignore_index, int64_t* __restrict__ idx,
                    int* __restrict__ inv, int64_t* __restrict__ t_c, int* __restrict__ n_valid) {
  __shared__ int warp_base[33];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int64_t per_warp = ((n + 31) / 32 + 31) / 32 * 32;
  const int64_t w0 = (int64_t)wid * per_warp;
  const int64_t w1 = (w0 + per_warp < n) ? w0 + per_warp : n;
  int cnt = 0;
  for (int64_t base = w0; base < w1; base += 32) {
    const int64_t e = base + lane;
    const bool valid = e < w1 && targets[e] != ignore_index;
    cnt += __popc(__ballot_sync(0xffffffffu, valid));
  }
  if (lane == 0) warp_base[wid] = cnt;
  __syncthreads();
  if (wid == 0) {
    const int c = warp_base[lane];
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    warp_base[lane] = incl - c;  // exclusive
    if (lane == 31) { warp_base[32] = incl; *n_valid = incl; }
  }
  __syncthreads();
  int pos = warp_base[wid];
  for (int64_t base = w0; base < w1; base += 32) {
    const int64_t e = base + lane;
    const int64_t t = e < w1 ? targets[e] : ignore_index;
    const bool valid = e < w1 && t != ignore_index;
    const unsigned mask = __ballot_sync(0xffffffffu, valid);
    const int mine = pos + __popc(mask & ((1u << lane) - 1u));
    if (valid) { idx[mine] = e; t_c[mine] = t; inv[e] = mine; }
    else if (e < w1) inv[e] = -1;
    pos += __popc(mask);
  }
  for (int64_t j = (int64_t)warp_base[32] + tid; j < n; j += 1024) { idx[j] = -1; t_c[j] = ignore_index; }
}

// dst[j, :] = src[idx[j], :] for idx[j] >= 0; rows j in [n_valid, round_up(n_valid, 256)) are cleared (the
// GEMMs' last tile reads them), rows beyond are left alone (never read).
__global__ void __launch_bounds__(256)
gather_valid_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int64_t* __restrict__ idx,
                         const int* __restrict__ n_valid, int64_t n, int64_t vecs) {
  const int64_t live = ((int64_t)(*n_valid) + 255) / 256 * 256;
  const int64_t end = live < n ? live : n;
  for (int64_t j = blockIdx.x; j < end; j += gridDim.x) {
    const int64_t r = idx[j];
    uint4* d = dst + j * vecs;
    if (r >= 0) {
      const uint4* s_ = src + r * vecs;
      for (int64_t v = threadIdx.x; v < vecs; v += 256) d[v] = s_[v];
    } else {
      for (int64_t v = threadIdx.x; v < vecs; v += 256) d[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// dst[i, :] = inv[i] >= 0 ? src[inv[i], :] : 0 over all n destination rows (no separate clearing pass).
__global__ void __launch_bounds__(256)
scatter_valid_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int* __restrict__ inv, int64_t n,
                          int64_t vecs) {
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    const int j = inv[i];
    uint4* d = dst + i * vecs;
    if (j >= 0) {
      const uint4* s_ = src + (int64_t)j * vecs;
      for (int64_t v = threadIdx.x; v < vecs; v += 256) d[v] = s_[v];
    } else {
      for (int64_t v = threadIdx.x; v < vecs; v += 256) d[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// out[i] = inv[i] >= 0 ? in[inv[i]] : 0 (per-row losses back to the caller's row order)
__global__ void __launch_bounds__(256)
scatter_valid_f32_kernel(const float* __restrict__ in, float* __restrict__ out, const int* __restrict__ inv, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = inv[i] >= 0 ? in[inv[i]] : 0.f;
}

// dst[i, :] = src[idx[i], :] (gather) or dst[idx[i], :] = src[i, :] (scatter); rows of `vecs` 16-byte vectors.
__global__ void __launch_bounds__(256)
move_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int64_t* __restrict__ idx, int64_t n_idx,
                 int64_t vecs, int scatter) {
  for (int64_t i = blockIdx.x; i < n_idx; i += gridDim.x) {
    const int64_t r = idx[i];
    const uint4* s = src + (scatter ? i : r) * vecs;
    uint4* d = dst + (scatter ? r : i) * vecs;
    for (int64_t v = threadIdx.x; v < vecs; v += 256) d[v] = s[v];
  }
}

// Switches of the GEMM launchers. They are per host thread (thread_local), so that two threads
// driving two GPUs do not see each other's settings; a setter affects the launches the SAME thread
// makes afterwards. HILDA_GEMM_PAIR in the environment presets the pair mask of every thread.
// pair mask: bit 0 logits, 1 d(hidden), 2 d(W) GEMM run as CTA pairs (256 x 256 tiles, cta_group::2);
// a clear bit = one CTA per 128 x 256 tile.
static int gemm_pair_default() {
  static const int v = []() { const char* e = getenv("HILDA_GEMM_PAIR"); return e ? (atoi(e) & 7) : 7; }();
  return v;
}
static thread_local int g_debug_mfast = 1;
static thread_local long long* g_gemm_probe = nullptr;
static thread_local int g_gemm_dry = 0;
static thread_local int g_gemm_sm_limit = 0;
static thread_local uint32_t g_gemm_wait_cap = WAIT_CAP;
static thread_local int g_gemm_pair = gemm_pair_default();

struct DynRows { const int* count; int64_t offset; };

template <bool A_MN, bool B_MN, int EPI>
static int run_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, GemmParams p, cudaStream_t st,
                    int kind_bit = 7) {
  p.probe = g_gemm_probe; p.dry = g_gemm_dry; p.sm_limit = g_gemm_sm_limit; p.wait_cap = g_gemm_wait_cap;
  if (g_gemm_pair & kind_bit) return launch_gemm2<A_MN, B_MN, EPI>(A, lda, B, ldb, p, st);
  return launch_gemm<A_MN, B_MN, EPI>(A, lda, B, ldb, p, st);
}

// Optional timing of the GEMM launches with CUDA events on the launching stream (off by default;
// per host thread like the switches above). kind 0 = logits GEMM, 1 = d(hidden) GEMM, 2 = d(W) GEMM.
constexpr int PROF_MAX = 1024;
static thread_local bool g_prof_on = false;
static thread_local int g_prof_n = 0;
static thread_local cudaEvent_t g_prof_ev[PROF_MAX][2];
static thread_local int g_prof_kind[PROF_MAX];
static thread_local int g_prof_created = 0;

struct ProfScope {
  int idx;
  cudaStream_t st;
  ProfScope(int kind, cudaStream_t s) : idx(-1), st(s) {
    if (!g_prof_on || g_prof_n >= PROF_MAX) return;
    idx = g_prof_n++;
    if (idx >= g_prof_created) {
      cudaEventCreate(&g_prof_ev[idx][0]);
      cudaEventCreate(&g_prof_ev[idx][1]);
      g_prof_created = idx + 1;
    }
    g_prof_kind[idx] = kind;
    cudaEventRecord(g_prof_ev[idx][0], st);
  }
  ~ProfScope() {
    if (idx >= 0) cudaEventRecord(g_prof_ev[idx][1], st);
  }
};

static inline void set_dyn(GemmParams& p, const DynRows& d, int dim) {
  if (d.count) { p.dyn_rows = d.count; p.dyn_off = (int)d.offset; p.dyn_dim = dim; }
}

static int flce_logits(const void* hidden, const void* W, void* logits, float* stats, int64_t rows, int64_t H,
                       int64_t V, int is_bf16, int* status, cudaStream_t st, float inv_temperature, DynRows dyn) {
  GemmParams p = {};
  p.stat_scale = FL_LOG2E * inv_temperature;
  p.M = (int)rows; p.N = (int)V; p.K = (int)H; p.m_fast = 1; p.is_bf16 = is_bf16;
  p.C16 = logits; p.ldc16 = round_up(V, BN);
  p.stats = reinterpret_cast<float2*>(stats); p.stats_ld = (V + BN - 1) / BN;
  p.status = status;
  set_dyn(p, dyn, 1);
  ProfScope prof(0, st);
  return run_gemm<false, false, EPI_LOGITS_STATS>(hidden, H, W, H, p, st, 1);
}

static int flce_grad_hidden(const void* dlogits, const void* W, void* dh16, float* dh32, int64_t rows, int64_t H,
                            int64_t V, int is_bf16, int* status, cudaStream_t st, DynRows dyn) {
  GemmParams p = {};
  static const int mfast = []() { const char* e = getenv("HILDA_GEMM2_MFAST"); return e ? atoi(e) : 1; }();
  p.M = (int)rows; p.N = (int)H; p.K = (int)V; p.m_fast = mfast; p.is_bf16 = is_bf16; p.status = status;
  set_dyn(p, dyn, 1);
  const int64_t pitch = round_up(V, BN);
  ProfScope prof(1, st);
  if (dh16) {
    p.C16 = dh16; p.ldc16 = H;
    return run_gemm<false, true, EPI_STORE16>(dlogits, pitch, W, H, p, st, 2);
  }
  p.C32 = dh32; p.ldc32 = H;
  return run_gemm<false, true, EPI_STORE32>(dlogits, pitch, W, H, p, st, 2);
}

// mode 0: dw32 = D^T h; 1: dw32 += D^T h; 2: dw16 = dw32 + D^T h; 3: dw16 = D^T h
static int flce_grad_weight(const void* dlogits, const void* hidden, float* dw32, void* dw16, int mode, int64_t rows,
                            int64_t H, int64_t V, int is_bf16, int* status, cudaStream_t st, DynRows dyn) {
  GemmParams p = {};
  p.M = (int)V; p.N = (int)H; p.K = (int)rows; p.m_fast = 0; p.is_bf16 = is_bf16; p.status = status;
  p.C32 = dw32; p.ldc32 = H; p.C16 = dw16; p.ldc16 = H;
  set_dyn(p, dyn, 2);
  const int64_t pitch = round_up(V, BN);
  ProfScope prof(2, st);
  switch (mode) {
    case 0: return run_gemm<true, true, EPI_STORE32>(dlogits, pitch, hidden, H, p, st, 4);
    case 1: return run_gemm<true, true, EPI_ACCUM32>(dlogits, pitch, hidden, H, p, st, 4);
    case 2: return run_gemm<true, true, EPI_ACCUM_FINAL16>(dlogits, pitch, hidden, H, p, st, 4);
    case 3: return run_gemm<true, true, EPI_STORE16>(dlogits, pitch, hidden, H, p, st, 4);
  }
  return HILDA_ERR_ARG;
}

static int flce_check(int64_t rows, int64_t H, int64_t V, int dtype) {
  if (dtype != HILDA_BF16 && dtype != HILDA_F16) return HILDA_ERR_DTYPE;
  if (rows <= 0 || H <= 0 || V <= 0 || rows > 0x7fffff00LL || V > 0x7fffff00LL || H > 0x7fffff00LL) return HILDA_ERR_SIZE;
  if (H % 8 != 0) return HILDA_ERR_SIZE;  // TMA needs 16-byte row pitches
  return HILDA_OK;
}

// *out = sum(rows) / (divide ? max(*n_valid, 1) : 1); NaN when the status word says that a bounded
// wait inside a GEMM ran out (the sums are then meaningless and must not pass for a loss).
__global__ void __launch_bounds__(1024)
flce_sum_loss_kernel(const float* __restrict__ rows, int64_t n, const int* __restrict__ n_valid, int divide,
                     const int* __restrict__ status, float* __restrict__ out) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) acc += rows[i];
  acc = block_sum<1024>(acc, red);
  if (threadIdx.x == 0) {
    if (divide) acc /= fmaxf((float)(*n_valid), 1.0f);
    if (status && *status != 0) acc = __int_as_float(0x7fc00000);
    *out = acc;
  }
}

}  // namespace hilda

using namespace hilda;

extern "C" {

int64_t hilda_flce_logits_pitch(int64_t V) { return round_up(V, BN); }
int64_t hilda_flce_padded_rows(int64_t rows) { return round_up(rows, 2 * BM); }
int64_t hilda_flce_stat_tiles(int64_t V) { return (V + BN - 1) / BN; }

int hilda_count_valid(const int64_t* targets, int64_t n, int64_t ignore_index, int* out, void* stream) {
  if (!targets || !out) return HILDA_ERR_NULL;
  count_valid_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(targets, n, ignore_index, out);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

int hilda_flce_logits(const void* hidden, const void* W, void* logits, float* stats, int64_t rows, int64_t H,
                      int64_t V, int dtype, int* status, const int* dyn_rows, int64_t dyn_off, void* stream) {
  if (!hidden || !W || !logits || !stats) return HILDA_ERR_NULL;
  int rc = flce_check(rows, H, V, dtype);
  if (rc) return rc;
  return flce_logits(hidden, W, logits, stats, rows, H, V, dtype == HILDA_BF16, status, (cudaStream_t)stream, 1.0f,
                     DynRows{dyn_rows, dyn_off});
}

// The same GEMM with the epilogue statistics taken of logits * inv_temperature (the stored logits are
// unscaled): the log-softmax at a temperature of the fused linear + JSD loss
// (kernels/fused_linear_jsd.py:46-62).
int hilda_flce_logits_scaled(const void* hidden, const void* W, void* logits, float* stats, int64_t rows, int64_t H,
                             int64_t V, float inv_temperature, int dtype, int* status, void* stream) {
  if (!hidden || !W || !logits || !stats) return HILDA_ERR_NULL;
  if (!(inv_temperature > 0.f)) return HILDA_ERR_ARG;
  int rc = flce_check(rows, H, V, dtype);
  if (rc) return rc;
  return flce_logits(hidden, W, logits, stats, rows, H, V, dtype == HILDA_BF16, status, (cudaStream_t)stream,
                     inv_temperature, DynRows{nullptr, 0});
}

int hilda_flce_row_stats(const float* stats, const void* logits, const int64_t* targets, float* rowstat, int64_t rows,
                         int64_t V, int64_t vocab_start, int dtype, const int* dyn_rows, int64_t dyn_off,
                         void* stream) {
  if (!stats || !logits || !rowstat) return HILDA_ERR_NULL;  // targets == null: no target logit (rowstat[2] = 0)
  if (rows <= 0) return HILDA_OK;
  const int n_tiles = (int)((V + BN - 1) / BN);
  flce_row_stats_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const float2*>(stats), n_tiles, n_tiles, reinterpret_cast<const uint16_t*>(logits),
      round_up(V, BN), targets, rowstat, rows, V, vocab_start, dtype == HILDA_BF16, dyn_rows, dyn_off);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// rowstat: [n_shards, 3, rows]; n_shards <= 1 is the single-shard layout [3, rows].
int hilda_flce_finalize(const float* rowstat, int n_shards, const int64_t* targets, int64_t ignore_index, float* lse,
                        float* loss_rows, int64_t rows, const int* dyn_rows, int64_t dyn_off, void* stream) {
  if (!rowstat || !targets || !lse || !loss_rows) return HILDA_ERR_NULL;
  if (rows <= 0) return HILDA_OK;
  flce_finalize_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      rowstat, n_shards, targets, ignore_index, lse, loss_rows, rows, dyn_rows, dyn_off);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

int hilda_flce_dlogits(void* logits, const float* lse, const int64_t* targets, int64_t ignore_index,
                       const int* n_valid, int64_t rows, int64_t V, int64_t vocab_start, int dtype,
                       const int* dyn_rows, int64_t dyn_off, void* stream) {
  if (!logits || !lse || !targets) return HILDA_ERR_NULL;
  if (rows <= 0) return HILDA_OK;
  if (rows > 65535LL * 65535LL) return HILDA_ERR_SIZE;
  const int64_t pitch = round_up(V, BN);
  const int64_t n_vec = (V + 7) / 8;
  cudaStream_t st = (cudaStream_t)stream;
  // grid.y is limited to 65535 rows per launch
  for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
    const int64_t nr = (rows - r0 < 65535) ? rows - r0 : 65535;
    dim3 grid((unsigned)((n_vec + 1023) / 1024), (unsigned)nr);
    if (dtype == HILDA_BF16)
      flce_dlogits_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(logits) + r0 * pitch, pitch,
                                                             lse + r0, targets + r0, ignore_index, n_valid, V, vocab_start,
                                                             dyn_rows, dyn_off + r0);
    else if (dtype == HILDA_F16)
      flce_dlogits_kernel<__half><<<grid, 256, 0, st>>>(reinterpret_cast<__half*>(logits) + r0 * pitch, pitch, lse + r0,
                                                      targets + r0, ignore_index, n_valid, V, vocab_start, dyn_rows,
                                                      dyn_off + r0);
    else return HILDA_ERR_DTYPE;
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

int hilda_flce_grad_hidden(const void* dlogits, const void* W, void* dh16, float* dh32, int64_t rows, int64_t H,
                           int64_t V, int dtype, int* status, const int* dyn_rows, int64_t dyn_off, void* stream) {
  if (!dlogits || !W || (!dh16 && !dh32)) return HILDA_ERR_NULL;
  int rc = flce_check(rows, H, V, dtype);
  if (rc) return rc;
  return flce_grad_hidden(dlogits, W, dh16, dh32, rows, H, V, dtype == HILDA_BF16, status, (cudaStream_t)stream,
                          DynRows{dyn_rows, dyn_off});
}

int hilda_flce_grad_weight(const void* dlogits, const void* hidden, float* dw32, void* dw16, int mode, int64_t rows,
                           int64_t H, int64_t V, int dtype, int* status, const int* dyn_rows, int64_t dyn_off,
                           void* stream) {
  if (!dlogits || !hidden) return HILDA_ERR_NULL;
  if ((mode != 3 && !dw32) || (mode >= 2 && !dw16)) return HILDA_ERR_NULL;
  int rc = flce_check(rows, H, V, dtype);
  if (rc) return rc;
  return flce_grad_weight(dlogits, hidden, dw32, dw16, mode, rows, H, V, dtype == HILDA_BF16, status,
                          (cudaStream_t)stream, DynRows{dyn_rows, dyn_off});
}

// Default rows per chunk. The scratch [chunk, pitch(V)] is kept at or below 1.25 GiB (about a
// quarter of the full logits at the 16384 x 128256 benchmark shape). Within [half of that, that]
// the chunk is chosen so that the d(hidden) GEMM, the one with few output tiles
// (chunk/256 x H/256 on CTA pairs, chunk/128 x H/256 on single CTAs), fills whole waves: e.g.
// 4608 rows = 18 x 16 = 288 pair tiles, just under 4 x 74.
int64_t hilda_flce_default_chunk_rows(int64_t BT, int64_t H, int64_t V) {
  // the d(hidden) GEMM's tile height and the number of units that run tiles at a time
  const bool pair = (g_gemm_pair & 2) != 0;
  const int64_t tile_rows = pair ? 2 * BM : BM;
  const int64_t units = pair ? 148 / 2 : 148;
  const int64_t pitch = round_up(V > 0 ? V : 1, BN);
  int64_t cap = (((int64_t)5 << 28)) / (pitch * 2);
  cap = cap / tile_rows * tile_rows;
  if (cap < tile_rows) cap = tile_rows;
  if (BT <= cap) return BT > 0 ? BT : 1;
  const int64_t n_tiles = (H + BN - 1) / BN;
  int64_t best = cap;
  double best_eff = -1.0;
  for (int64_t c = cap; c >= cap / 2 && c >= tile_rows; c -= tile_rows) {
    int64_t waves = 0, tiles = 0;
    for (int64_t r0 = 0; r0 < BT; r0 += c) {
      const int64_t rows = (BT - r0 < c) ? BT - r0 : c;
      const int64_t t = ((rows + tile_rows - 1) / tile_rows) * n_tiles;
      tiles += t;
      waves += (t + units - 1) / units;
    }
    const double eff = (double)tiles / (double)(waves * units);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = c; }
  }
  return best;
}

// Workspace layout (all offsets 256-byte aligned), for chunk_rows rows per chunk:
//   [0]      int status, int n_valid
//   scratch  16-bit [padded(chunk_rows), pitch(V)]
//   stats    float2 [chunk_rows, tiles(V)]
//   rowstat  float [3, chunk_rows]
//   lse      float [chunk_rows]
//   loss     float [BT]            per-row loss in the order the rows are computed in
//   dw32     float [V, H]          (only when BT > chunk_rows and gradients are requested)
//   with HILDA_FLCE_COMPACT: idx int64 [BT], t_c int64 [BT], inv int [BT], h_c 16-bit [BT, H],
//   and with gradients dh_c 16-bit [BT, H]
static int64_t flce_ws_layout(int64_t BT, int64_t H, int64_t V, int64_t chunk, int with_grad, int flags, int64_t* off) {
  int64_t o = 256;
  off[0] = o; o = round_up(o + round_up(chunk, 2 * BM) * round_up(V, BN) * 2, 256);
  off[1] = o; o = round_up(o + chunk * ((V + BN - 1) / BN) * 8, 256);
  off[2] = o; o = round_up(o + 3 * chunk * 4, 256);
  off[3] = o; o = round_up(o + chunk * 4, 256);
  off[4] = o; o = round_up(o + BT * 4, 256);
  off[5] = o;
  if (with_grad && BT > chunk) o = round_up(o + V * H * 4, 256);
  off[6] = off[7] = off[8] = off[9] = off[10] = o;
  if (flags & 1) {
    off[6] = o; o = round_up(o + BT * 8, 256);
    off[7] = o; o = round_up(o + BT * 8, 256);
    off[8] = o; o = round_up(o + BT * 4, 256);
    off[9] = o; o = round_up(o + BT * H * 2, 256);
    off[10] = o;
    if (with_grad) o = round_up(o + BT * H * 2, 256);
  }
  return o;
}

int64_t hilda_flce_workspace_bytes(int64_t BT, int64_t H, int64_t V, int64_t chunk_rows, int with_grad, int flags) {
  if (BT <= 0 || H <= 0 || V <= 0) return 256;
  if (chunk_rows <= 0) chunk_rows = hilda_flce_default_chunk_rows(BT, H, V);
  if (chunk_rows > BT) chunk_rows = BT;
  int64_t off[11];
  return flce_ws_layout(BT, H, V, chunk_rows, with_grad, flags, off);
}

// The whole operator on one device. reduction: 0 none (loss_rows gets the per-row loss), 1 mean,
// 2 sum (loss_out scalar). dh / dw null => loss only. flags bit 0 (HILDA_FLCE_COMPACT): the rows whose
// target is ignore_index are compacted away on the device before the GEMMs run (index lists, gather,
// GEMM extents and the scatter of d(hidden) all follow a device-side count: no host round trip).
// Returns after enqueueing; the int at workspace[0] is non-zero afterwards if a bounded wait inside
// a GEMM ran out, and a mean / sum loss is then NaN.
int hilda_fused_linear_cross_entropy_fwd(const void* hidden, const void* W, const int64_t* targets, float* loss_out,
                                         float* loss_rows, void* dh, void* dw, void* workspace, int64_t BT, int64_t H,
                                         int64_t V, int64_t ignore_index, int reduction, int64_t chunk_rows, int dtype,
                                         int flags, void* stream) {
  if (!hidden || !W || !targets || !workspace) return HILDA_ERR_NULL;
  if (reduction < 0 || reduction > 2) return HILDA_ERR_ARG;
  if (reduction == 0 ? !loss_rows : !loss_out) return HILDA_ERR_NULL;
  if ((dh == nullptr) != (dw == nullptr)) return HILDA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (BT == 0) {
    if (loss_out && cudaMemsetAsync(loss_out, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
    if (dw && cudaMemsetAsync(dw, 0, (size_t)V * H * 2, st) != cudaSuccess) return HILDA_ERR_CUDA;
    return HILDA_OK;
  }
  int rc = flce_check(BT, H, V, dtype);
  if (rc) return rc;
  if (!aligned16(hidden) || !aligned16(W) || (dh && (!aligned16(dh) || !aligned16(dw)))) return HILDA_ERR_ALIGN;
  const int with_grad = dh != nullptr;
  const bool compact = (flags & 1) != 0;
  if (chunk_rows <= 0) chunk_rows = hilda_flce_default_chunk_rows(BT, H, V);
  if (chunk_rows > BT) chunk_rows = BT;
  int64_t off[11];
  flce_ws_layout(BT, H, V, chunk_rows, with_grad, flags, off);
  char* ws = reinterpret_cast<char*>(workspace);
  int* status = reinterpret_cast<int*>(ws);
  int* n_valid = status + 1;
  void* scratch = ws + off[0];
  float* stats = reinterpret_cast<float*>(ws + off[1]);
  float* rowstat = reinterpret_cast<float*>(ws + off[2]);
  float* lse = reinterpret_cast<float*>(ws + off[3]);
  float* ws_loss = reinterpret_cast<float*>(ws + off[4]);
  // per-row losses in computed order: straight into the caller's array unless the rows are compacted
  float* rows_loss = (loss_rows && !compact) ? loss_rows : ws_loss;
  float* dw32 = reinterpret_cast<float*>(ws + off[5]);
  const int is_bf16 = dtype == HILDA_BF16;
  const int64_t esz = 2;
  const int64_t vecs = H * esz / 16;
  const int64_t move_grid = BT < (int64_t)sm_count() * 16 ? BT : (int64_t)sm_count() * 16;

  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
  const void* h_use = hidden;
  const int64_t* t_use = targets;
  void* dh_use = dh;
  DynRows dyn{nullptr, 0};
  int* inv = nullptr;
  if (compact) {
    int64_t* idx = reinterpret_cast<int64_t*>(ws + off[6]);
    int64_t* t_c = reinterpret_cast<int64_t*>(ws + off[7]);
    inv = reinterpret_cast<int*>(ws + off[8]);
    void* h_c = ws + off[9];
    flce_compact_kernel<<<1, 1024, 0, st>>>(targets, BT, ignore_index, idx, inv, t_c, n_valid);
    HILDA_LAUNCH_CHECK();
    gather_valid_rows_kernel<<<(unsigned)move_grid, 256, 0, st>>>((const uint4*)hidden, (uint4*)h_c, idx, n_valid, BT, vecs);
    HILDA_LAUNCH_CHECK();
    h_use = h_c; t_use = t_c; dh_use = with_grad ? (void*)(ws + off[10]) : nullptr;
    dyn.count = n_valid;
  } else {
    count_valid_kernel<<<1, 1024, 0, st>>>(targets, BT, ignore_index, n_valid);
    HILDA_LAUNCH_CHECK();
  }
  const int64_t n_chunks = (BT + chunk_rows - 1) / chunk_rows;
  for (int64_t c = 0; c < n_chunks; ++c) {
    const int64_t r0 = c * chunk_rows;
    const int64_t rows = (BT - r0 < chunk_rows) ? BT - r0 : chunk_rows;
    const char* hc = reinterpret_cast<const char*>(h_use) + r0 * H * esz;
    const DynRows d{dyn.count, r0};
    rc = flce_logits(hc, W, scratch, stats, rows, H, V, is_bf16, status, st, 1.0f, d);
    if (rc) return rc;
    rc = hilda_flce_row_stats(stats, scratch, t_use + r0, rowstat, rows, V, 0, dtype, d.count, r0, stream);
    if (rc) return rc;
    rc = hilda_flce_finalize(rowstat, 1, t_use + r0, ignore_index, lse, rows_loss + r0, rows, d.count, r0, stream);
    if (rc) return rc;
    if (!with_grad) continue;
    rc = hilda_flce_dlogits(scratch, lse, t_use + r0, ignore_index, reduction == 1 ? n_valid : nullptr, rows, V, 0,
                            dtype, d.count, r0, stream);
    if (rc) return rc;
    rc = flce_grad_hidden(scratch, W, reinterpret_cast<char*>(dh_use) + r0 * H * esz, nullptr, rows, H, V, is_bf16, status,
                          st, d);
    if (rc) return rc;
    int mode;
    if (n_chunks == 1) mode = 3;
    else if (c == 0) mode = 0;
    else if (c == n_chunks - 1) mode = 2;
    else mode = 1;
    rc = flce_grad_weight(scratch, hc, dw32, dw, mode, rows, H, V, is_bf16, status, st, d);
    if (rc) return rc;
  }
  if (compact) {
    if (with_grad) {
      scatter_valid_rows_kernel<<<(unsigned)move_grid, 256, 0, st>>>((const uint4*)dh_use, (uint4*)dh, inv, BT, vecs);
      HILDA_LAUNCH_CHECK();
    }
    if (loss_rows) {
      scatter_valid_f32_kernel<<<(unsigned)((BT + 255) / 256), 256, 0, st>>>(rows_loss, loss_rows, inv, BT);
      HILDA_LAUNCH_CHECK();
    }
  }
  if (reduction != 0) {
    flce_sum_loss_kernel<<<1, 1024, 0, st>>>(rows_loss, BT, n_valid, reduction == 1 ? 1 : 0, status, loss_out);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

// Device-side index lists of the non-ignored rows for callers that drive the step entry points
// themselves (the vocab-parallel form): idx int64 [n] (source row of compacted row j, -1 beyond the
// count), inv int32 [n] (compacted position of row i, -1 if ignored), t_c int64 [n] (targets in
// compacted order, ignore_index beyond the count), *n_valid the count. No host synchronisation.
int hilda_flce_compact(const int64_t* targets, int64_t n, int64_t ignore_index, int64_t* idx, int* inv, int64_t* t_c,
                       int* n_valid, void* stream) {
  if (!targets || !idx || !inv || !t_c || !n_valid) return HILDA_ERR_NULL;
  if (n < 0 || n > 0x7fffff00LL) return HILDA_ERR_SIZE;
  flce_compact_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(targets, n, ignore_index, idx, inv, t_c, n_valid);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
// dst[j,:] = src[idx[j],:] for the *n_valid leading rows, zero rows up to the next multiple of 256 (read by
// the GEMMs' last tile), the rest untouched; n = rows of dst and entries of idx.
int hilda_gather_valid_rows(const void* src, const int64_t* idx, const int* n_valid, void* dst, int64_t n,
                            int64_t row_bytes, void* stream) {
  if (n == 0) return HILDA_OK;
  if (!src || !idx || !n_valid || !dst) return HILDA_ERR_NULL;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(src) || !aligned16(dst)) return HILDA_ERR_ALIGN;
  const int64_t grid = n < (int64_t)sm_count() * 16 ? n : (int64_t)sm_count() * 16;
  gather_valid_rows_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, idx, n_valid, n,
                                                                             row_bytes / 16);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
// dst[i,:] = inv[i] >= 0 ? src[inv[i],:] : 0 over all n rows of dst.
int hilda_scatter_valid_rows(const void* src, const int* inv, void* dst, int64_t n, int64_t row_bytes, void* stream) {
  if (n == 0) return HILDA_OK;
  if (!src || !inv || !dst) return HILDA_ERR_NULL;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(src) || !aligned16(dst)) return HILDA_ERR_ALIGN;
  const int64_t grid = n < (int64_t)sm_count() * 16 ? n : (int64_t)sm_count() * 16;
  scatter_valid_rows_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, inv, n,
                                                                              row_bytes / 16);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
// out[i] = inv[i] >= 0 ? in[inv[i]] : 0 (fp32 per-row values back to the caller's row order).
int hilda_scatter_valid_f32(const float* in, const int* inv, float* out, int64_t n, void* stream) {
  if (n == 0) return HILDA_OK;
  if (!in || !inv || !out) return HILDA_ERR_NULL;
  scatter_valid_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(in, out, inv, n);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
// *out = sum(rows) (/ max(*n_valid, 1) when divide), NaN if *status != 0 (status may be null).
int hilda_flce_sum_loss(const float* rows, int64_t n, const int* n_valid, int divide, const int* status, float* out,
                        void* stream) {
  if (!rows || !out || (divide && !n_valid)) return HILDA_ERR_NULL;
  flce_sum_loss_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(rows, n, n_valid, divide, status, out);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// Time every GEMM launch of the FLCE entry points with CUDA events (enable != 0 also resets the
// record). hilda_flce_profile_collect waits for the recorded events and returns, per kind
// (0 logits, 1 d hidden, 2 d W), the summed device time in ms and the launch count.
void hilda_flce_profile(int enable) {
  g_prof_on = enable != 0;
  g_prof_n = 0;
}
int hilda_flce_profile_collect(float* ms_per_kind, int* launches_per_kind) {
  if (!ms_per_kind || !launches_per_kind) return HILDA_ERR_NULL;
  for (int k = 0; k < 3; ++k) { ms_per_kind[k] = 0.f; launches_per_kind[k] = 0; }
  for (int i = 0; i < g_prof_n; ++i) {
    if (cudaEventSynchronize(g_prof_ev[i][1]) != cudaSuccess) return HILDA_ERR_CUDA;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, g_prof_ev[i][0], g_prof_ev[i][1]) != cudaSuccess) return HILDA_ERR_CUDA;
    ms_per_kind[g_prof_kind[i]] += ms;
    launches_per_kind[g_prof_kind[i]] += 1;
  }
  return HILDA_OK;
}

// The i-th recorded launch since profiling was switched on: its kind and device time in ms
// (HILDA_ERR_ARG once i is past the last one). Call after hilda_flce_profile_collect.
int hilda_flce_profile_entry(int i, int* kind, float* ms) {
  if (!kind || !ms) return HILDA_ERR_NULL;
  if (i < 0 || i >= g_prof_n) return HILDA_ERR_ARG;
  if (cudaEventSynchronize(g_prof_ev[i][1]) != cudaSuccess) return HILDA_ERR_CUDA;
  if (cudaEventElapsedTime(ms, g_prof_ev[i][0], g_prof_ev[i][1]) != cudaSuccess) return HILDA_ERR_CUDA;
  *kind = g_prof_kind[i];
  return HILDA_OK;
}

// Row moves with a host-known index list: gather dst[i] = src[idx[i]] and scatter dst[idx[i]] = src[i]
// over rows of row_bytes (a multiple of 16) bytes; idx is int64 on the device. The scatter first
// clears dst (n_dst_rows rows), so rows not named by idx come out as zeros.
int hilda_gather_rows(const void* src, const int64_t* idx, void* dst, int64_t n_idx, int64_t row_bytes, void* stream) {
  if (n_idx == 0) return HILDA_OK;
  if (!src || !idx || !dst) return HILDA_ERR_NULL;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(src) || !aligned16(dst)) return HILDA_ERR_ALIGN;
  int64_t grid = n_idx < (int64_t)sm_count() * 16 ? n_idx : (int64_t)sm_count() * 16;
  move_rows_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, idx, n_idx,
                                                                     row_bytes / 16, 0);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}
int hilda_scatter_rows(const void* src, const int64_t* idx, void* dst, int64_t n_idx, int64_t n_dst_rows,
                       int64_t row_bytes, void* stream) {
  if (!dst) return HILDA_ERR_NULL;
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(dst)) return HILDA_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_dst_rows > 0 && cudaMemsetAsync(dst, 0, (size_t)(n_dst_rows * row_bytes), st) != cudaSuccess) return HILDA_ERR_CUDA;
  if (n_idx == 0) return HILDA_OK;
  if (!src || !idx) return HILDA_ERR_NULL;
  if (!aligned16(src)) return HILDA_ERR_ALIGN;
  int64_t grid = n_idx < (int64_t)sm_count() * 16 ? n_idx : (int64_t)sm_count() * 16;
  move_rows_kernel<<<(unsigned)grid, 256, 0, st>>>((const uint4*)src, (uint4*)dst, idx, n_idx, row_bytes / 16, 1);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// The setters below act on the calling host thread's launches only (see the switches at the top).
// Select the GEMM variant per use: bit 0 = logits, bit 1 = d(hidden), bit 2 = d(W) run on CTA pairs
// (cta_group::2, 256 x 256 tiles); a clear bit = single CTAs. hilda_debug_gemm uses pairs if any bit is set.
void hilda_gemm_set_pair(int mask) { g_gemm_pair = mask & 7; }
// The FLCE GEMMs launch on at most `sms` SMs (0 = all of them) until set back: a caller that runs a
// collective on another stream beside a GEMM leaves it a few SMs this way.
void hilda_gemm_set_sm_limit(int sms) { g_gemm_sm_limit = sms > 0 ? sms : 0; }
// Attempts a bounded mbarrier wait makes before it gives up (0 restores the default of 2^22).
void hilda_gemm_set_wait_cap(unsigned attempts) { g_gemm_wait_cap = attempts > 0 ? attempts : WAIT_CAP; }
// Tile walk order used by hilda_debug_gemm (1 = M first, 0 = N first).
void hilda_debug_gemm_set_order(int m_fast) { g_debug_mfast = m_fast ? 1 : 0; }
// Cycle counters of the single-CTA GEMM's role loops: device buffer of [sm_count][8] int64
// {producer wait-for-slot, producer total, issuer wait-for-data, issuer wait-for-accumulator,
//  issuer total, epilogue wait-for-accumulator, epilogue busy, 0}; null switches it off.
// dry = 1 (measurement only, results are garbage): the producer signals its slots full without
// loading anything, which shows the rate of the MMA / barrier loop with the memory system out of it.
// dry = 2 (test of the failure path): the producer neither loads nor signals, so the issuer's bounded
// wait runs out, the status word is set and every role leaves; nothing is left in flight.
void hilda_gemm_set_probe(void* buf, int dry) { g_gemm_probe = (long long*)buf; g_gemm_dry = dry; }
int hilda_gemm_get_pair(void) { return g_gemm_pair; }

// Plain GEMM through the same kernel, for validating operand layouts against a library matmul.
// A is [M,K] (a_mn=0) or stored [K,M] (a_mn=1); B is [N,K] (b_mn=0) or stored [K,N] (b_mn=1);
// exactly one of c16 / c32 is written. mn_lbo/mn_sbo = 0 selects the defaults.
int hilda_debug_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* c16, float* c32, int64_t ldc, int M,
                     int N, int K, int a_mn, int b_mn, int dtype, int mn_lbo, int mn_sbo, int* status, void* stream) {
  if (!A || !B || (!c16 && !c32)) return HILDA_ERR_NULL;
  if (dtype != HILDA_BF16 && dtype != HILDA_F16) return HILDA_ERR_DTYPE;
  // the epilogue stores 16-byte vectors: rows of C must start on 16-byte boundaries
  if (ldc % 8 != 0 || N % 8 != 0 || !aligned16(c16) || !aligned16(c32)) return HILDA_ERR_ALIGN;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.m_fast = g_debug_mfast; p.is_bf16 = dtype == HILDA_BF16; p.status = status;
  p.C16 = c16; p.ldc16 = ldc; p.C32 = c32; p.ldc32 = ldc;
  p.mn_lbo = (uint32_t)mn_lbo; p.mn_sbo = (uint32_t)mn_sbo;
  cudaStream_t st = (cudaStream_t)stream;
  const int key = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (c16) {
    switch (key) {
      case 0: return run_gemm<false, false, EPI_STORE16>(A, lda, B, ldb, p, st);
      case 1: return run_gemm<false, true, EPI_STORE16>(A, lda, B, ldb, p, st);
      case 2: return run_gemm<true, false, EPI_STORE16>(A, lda, B, ldb, p, st);
      default: return run_gemm<true, true, EPI_STORE16>(A, lda, B, ldb, p, st);
    }
  }
  switch (key) {
    case 0: return run_gemm<false, false, EPI_STORE32>(A, lda, B, ldb, p, st);
    case 1: return run_gemm<false, true, EPI_STORE32>(A, lda, B, ldb, p, st);
    case 2: return run_gemm<true, false, EPI_STORE32>(A, lda, B, ldb, p, st);
    default: return run_gemm<true, true, EPI_STORE32>(A, lda, B, ldb, p, st);
  }
}

}  // extern "C"
