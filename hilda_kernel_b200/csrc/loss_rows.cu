// CrossEntropy, GRPO PPO-clip loss and selective log-softmax on top of the one-pass row engine.
//
// CrossEntropy follows kernels/cross_entropy.py:114-166 (training kernel: loss and dlogits in one
// kernel, ignored rows -> loss 0 and zero gradient, 'mean' divides by the count of non-ignored
// rows clamped to >= 1 read from a device scalar) and :32-65 (inference path: loss and lse only).
// GRPO follows kernels/grpo_loss.py:87-159 (forward), :166-234 (backward) and :290-295, :309-310
// (reductions and the per-token upstream scale); here forward and backward are one kernel that
// writes dlogits for a unit upstream gradient, so the logits are read once.
#include <cstdio>
#include <cstdlib>
#include "row_softmax.cuh"
#include "reduce_kernels.cuh"

namespace hilda {

// Plan override and cluster scheduling preference of the row engine: per host thread, so that threads
// driving different GPUs do not disturb each other. Tuning runs may preset them through the environment
// (read once): HILDA_ROW_ENGINE="nv,cluster[,ns]", HILDA_ROW_POLICY=0|1|2.
struct RowEnv { int nv = 0, cluster = 0, ns = 0, policy = 2; };
static const RowEnv& row_env() {
  static const RowEnv env = []() {
    RowEnv r;
    if (const char* e = getenv("HILDA_ROW_ENGINE")) {
      int a = 0, b = 0, c = 0;
      if (sscanf(e, "%d,%d,%d", &a, &b, &c) >= 2) { r.nv = a; r.cluster = b; r.ns = c; }
    }
    if (const char* pol = getenv("HILDA_ROW_POLICY")) r.policy = atoi(pol);
    return r;
  }();
  return env;
}
thread_local int g_row_force_nv = row_env().nv, g_row_force_cluster = row_env().cluster, g_row_force_ns = row_env().ns;
thread_local int g_row_cluster_policy = row_env().policy;

// ---------------------------------------------------------------- CrossEntropy
struct CEOp {
  const int64_t* targets;
  int64_t ignore_index;
  const int* n_valid;   // device scalar, used when mean != 0
  int mean;             // 1: scale loss and grad by 1/max(n_valid,1)
  float* loss_rows;     // [n_rows] per-row loss (already scaled when mean)
  float* lse_rows;      // optional [n_rows]
  int scale_loss;       // 0: leave the per-row loss unscaled (inference 'mean' divides afterwards)

  __device__ __forceinline__ int64_t row_offset(int64_t row, int64_t V) const { return row * V; }
  __host__ bool rows_aligned(int64_t, int) const { return true; }  // rows start at row * V: any V
  __device__ __forceinline__ float inv_temperature() const { return 1.0f; }
  __device__ __forceinline__ bool begin(int64_t row, int64_t& target) const {
    target = targets[row];
    return target != ignore_index;
  }
  __device__ __forceinline__ void inactive(int64_t row) const {
    loss_rows[row] = 0.f;
    if (lse_rows) lse_rows[row] = 0.f;
  }
  struct Pre { float scale; };
  __device__ __forceinline__ Pre prefetch(int64_t) const {
    return Pre{mean ? 1.0f / fmaxf((float)(*n_valid), 1.0f) : 1.0f};
  }
  __device__ __forceinline__ RowCoef finish(int64_t row, float lse, float x_t, bool writer, const Pre& pre) const {
    const float scale = pre.scale;
    if (writer) {
      loss_rows[row] = (lse - x_t) * (scale_loss ? scale : 1.0f);
      if (lse_rows) lse_rows[row] = lse;
    }
    return RowCoef{scale, -scale};
  }
};

// out[r, :] = in[r, :] * (per_row ? scale[r] : scale[0]); in and out may alias.
template <typename T>
__global__ void __launch_bounds__(256)
scale_rows_kernel(const T* in, T* out, const float* __restrict__ scale, int per_row, int64_t n_rows, int64_t n_cols,
                  int vec_ok) {
  constexpr int VEC = VT<T>::N;
  for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
    const float sc = per_row ? scale[row] : scale[0];
    const T* ir = in + row * n_cols;
    T* orow = out + row * n_cols;
    if (vec_ok) {
      const int64_t n_vec = n_cols / VEC;
      for (int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * 256) {
        float f[VEC];
        VT<T>::unpack(ld16(ir + v * VEC), f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] *= sc;
        st16(orow + v * VEC, VT<T>::pack(f));
      }
    } else {
      for (int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x; c < n_cols; c += (int64_t)gridDim.x * 256)
        VT<T>::store1(orow + c, VT<T>::load1(ir + c) * sc);
    }
  }
}

// ---------------------------------------------------------------- GRPO
struct GRPOOp {
  const int64_t* ids;        // [B, L]
  const float* mask;         // [B, L] or null: weight of the token; 0 = inactive
  const float* advantages;   // [B]
  const float* old_logp;     // [B, L] or null
  const float* ref_logp;     // [B, L] or null (required when beta != 0)
  const float* seq_len;      // [B] clamp(sum(mask), 1)
  float* loss; float* kl; float* clipped; float* lse_out; float* logp_out;  // [B, L] each; kl/logp_out optional
  int64_t B, L;
  float b_norm;              // sequences the loss is averaged over (all shards' when row-sharded)
  float inv_t, beta, eps_low, eps_high;
  int logp_only;             // selective log-softmax: write logp_out only

  __device__ __forceinline__ int64_t row_offset(int64_t row, int64_t V) const { return row * V; }
  __host__ bool rows_aligned(int64_t, int) const { return true; }  // rows start at row * V: any V
  __device__ __forceinline__ float inv_temperature() const { return inv_t; }
  __device__ __forceinline__ bool begin(int64_t row, int64_t& target) const {
    const int64_t b = row / (L + 1), l = row - b * (L + 1);
    if (l == L) return false;
    const int64_t i = b * L + l;
    if (mask && mask[i] == 0.f) return false;
    target = ids[i];
    return true;
  }
  __device__ __forceinline__ void inactive(int64_t row) const {
    const int64_t b = row / (L + 1), l = row - b * (L + 1);
    if (l == L) return;
    const int64_t i = b * L + l;
    if (logp_out) logp_out[i] = 0.f;
    if (logp_only) return;
    loss[i] = 0.f; clipped[i] = 0.f; lse_out[i] = 0.f;
    if (kl) kl[i] = 0.f;
  }
  struct Pre { float old, ref, adv, gscale; int has_old; };
  __device__ __forceinline__ Pre prefetch(int64_t row) const {
    Pre p{0.f, 0.f, 0.f, 0.f, 0};
    if (logp_only) return p;
    const int64_t b = row / (L + 1), l = row - b * (L + 1);
    const int64_t i = b * L + l;
    if (old_logp) { p.old = old_logp[i]; p.has_old = 1; }
    if (beta != 0.f) p.ref = ref_logp[i];
    p.adv = advantages[b];
    // upstream scale for a unit loss gradient: mask / (seq_len_b * B), then 1/T
    const float mval = mask ? mask[i] : 1.0f;
    p.gscale = (mval / (seq_len[b] * b_norm)) * inv_t;
    return p;
  }
  __device__ __forceinline__ RowCoef finish(int64_t row, float lse, float x_t, bool writer, const Pre& pre) const {
    const int64_t b = row / (L + 1), l = row - b * (L + 1);
    const int64_t i = b * L + l;
    const float logp = x_t - lse;
    if (logp_only) {
      if (writer) logp_out[i] = logp;
      return RowCoef{0.f, 0.f};
    }
    const float old = pre.has_old ? pre.old : logp;
    const float coef1 = expf(logp - old);
    const float adv = pre.adv;
    const float lo = 1.0f - eps_low, hi = 1.0f + eps_high;
    const float coef2 = fminf(fmaxf(coef1, lo), hi);
    const bool is_clipped = ((coef1 < lo) && (adv < 0.f)) || ((coef1 > hi) && (adv > 0.f));
    const float l1 = coef1 * adv, l2 = coef2 * adv;
    float ptl = -fminf(l1, l2);
    float dlogp = (l2 >= l1) ? -coef1 * adv : 0.f;
    float klv = 0.f;
    if (beta != 0.f) {
      const float d = pre.ref - logp;
      const float e = expf(d);
      klv = e - d - 1.0f;
      ptl += beta * klv;
      dlogp += beta * (1.0f - e);
    }
    if (writer) {
      loss[i] = ptl; clipped[i] = is_clipped ? 1.f : 0.f; lse_out[i] = lse;
      if (kl) kl[i] = klv;
      if (logp_out) logp_out[i] = logp;
    }
    const float g = dlogp * pre.gscale;
    return RowCoef{-g, g};
  }
};

// seq_len[b] = max(sum_l mask[b,l], 1)  (L when there is no mask)
__global__ void __launch_bounds__(256)
grpo_seq_len_kernel(const float* __restrict__ mask, int64_t L, float* __restrict__ seq_len) {
  __shared__ float red[33];
  const int64_t b = blockIdx.x;
  float acc = 0.f;
  if (mask) for (int64_t l = threadIdx.x; l < L; l += 256) acc += mask[b * L + l];
  else acc = (threadIdx.x == 0) ? (float)L : 0.f;
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) seq_len[b] = fmaxf(acc, 1.0f);
}

// out[0] = sum_b( sum_l loss*mask / seq_len_b ) / b_norm; out[3] = sum mask; out[1] = sum(kl*mask)/max(sum mask,1);
// out[2] = sum(clipped*mask)/max(sum mask,1). One CTA, one warp per sequence at a time.
__global__ void __launch_bounds__(1024)
grpo_reduce_kernel(const float* __restrict__ loss, const float* __restrict__ kl, const float* __restrict__ clipped,
                   const float* __restrict__ mask, const float* __restrict__ seq_len, int64_t B, int64_t L,
                   float b_norm, float* __restrict__ out) {
  __shared__ float red[4][33];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float a_loss = 0.f, a_kl = 0.f, a_clip = 0.f, a_mask = 0.f;
  for (int64_t b = wid; b < B; b += 32) {
    float sl = 0.f, sk = 0.f, sc = 0.f, sm = 0.f;
    // eight positions of the lane at a time: their loads are all issued before the first sum (one CTA
    // walks every sequence, so the chain of dependent round trips is what this kernel's time is made of);
    // the sums stay in ascending position order
    for (int64_t l0 = lane; l0 < L; l0 += 32 * 8) {
      float vl[8], vk[8], vc[8], vm[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int64_t l = l0 + 32 * u;
        const bool in = l < L;
        const int64_t i = b * L + (in ? l : 0);
        vm[u] = in ? (mask ? mask[i] : 1.0f) : 0.f;
        vl[u] = in ? loss[i] : 0.f;
        vc[u] = in ? clipped[i] : 0.f;
        vk[u] = (in && kl) ? kl[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (l0 + 32 * u < L) {
          sl += vl[u] * vm[u]; sc += vc[u] * vm[u]; sm += vm[u];
          if (kl) sk += vk[u] * vm[u];
        }
      }
    }
    sl = warp_sum(sl); sk = warp_sum(sk); sc = warp_sum(sc); sm = warp_sum(sm);
    a_loss += sl / seq_len[b]; a_kl += sk; a_clip += sc; a_mask += sm;
  }
  if (lane == 0) { red[0][wid] = a_loss; red[1][wid] = a_kl; red[2][wid] = a_clip; red[3][wid] = a_mask; }
  __syncthreads();
  if (wid == 0) {
    float v0 = warp_sum(red[0][lane]), v1 = warp_sum(red[1][lane]), v2 = warp_sum(red[2][lane]), v3 = warp_sum(red[3][lane]);
    if (lane == 0) {
      const float msum = fmaxf(v3, 1.0f);
      out[0] = v0 / b_norm; out[1] = v1 / msum; out[2] = v2 / msum; out[3] = v3;
    }
  }
}

template <typename T>
static int scale_rows_t(const void* in, void* out, const float* scale, int per_row, int64_t n_rows, int64_t n_cols,
                        cudaStream_t st) {
  const int vec_ok = aligned16(in) && aligned16(out) && (n_cols % VT<T>::N == 0);
  int64_t bx = (n_cols / (vec_ok ? VT<T>::N : 1) + 255) / 256;
  if (bx > 1024) bx = 1024;
  if (bx < 1) bx = 1;
  int64_t by = n_rows < 65535 ? n_rows : 65535;
  scale_rows_kernel<T><<<dim3((unsigned)bx, (unsigned)by), 256, 0, st>>>((const T*)in, (T*)out, scale, per_row, n_rows,
                                                                        n_cols, vec_ok);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // namespace hilda

using namespace hilda;

extern "C" {

// Tuning hook: force (register vectors per thread, cluster size, shared-memory vectors per thread) of the
// row engine; (0,0,0) restores automatic.
void hilda_row_engine_force(int nv, int cluster, int ns) {
  g_row_force_nv = nv; g_row_force_cluster = cluster; g_row_force_ns = ns;
}
// The plan the row engine takes for a vocabulary of V elements of `dtype` on aligned tensors (host only, no
// GPU needed): out = {threads, register vectors, cluster, shared-memory vectors}. Returns 1, or 0 when
// the scalar kernel serves the shape. hilda_row_engine_has_kernel says whether a plan is instantiated.
int hilda_row_engine_plan(int64_t V, int dtype, int* out) {
  const int vec = dtype == HILDA_F32 ? 4 : 8;
  const RowPlan p = plan_row(V, vec, true, 0, 0, 0);
  if (out) { out[0] = p.threads; out[1] = p.nv; out[2] = p.cluster; out[3] = p.ns; }
  return p.generic ? 0 : 1;
}
int hilda_row_engine_has_kernel(int threads, int nv, int cluster, int ns) {
#define ROW_HAS(TH_, NV_, CL_, NS_) if (threads == TH_ && nv == NV_ && cluster == CL_ && ns == NS_) return 1;
  ROW_CFG_LIST(ROW_HAS)
#undef ROW_HAS
  return 0;
}

int64_t hilda_cross_entropy_workspace_bytes(int64_t n_rows) { return 16 + (n_rows > 0 ? n_rows : 0) * 4; }

// workspace layout: int n_valid at byte 0, int status at byte 8, float loss_rows[n_rows] at byte 16 (only used when the
// caller passes loss_rows == null).
// reduction: 0 none, 1 mean, 2 sum. grad may be null (inference path: loss only).
// loss_out: scalar for mean/sum; unused for none (per-row loss is in loss_rows).
int hilda_cross_entropy_fwd(const void* logits, const int64_t* targets, void* grad, float* loss_rows, float* lse_rows,
                            float* loss_out, void* workspace, const int* n_valid_in, int64_t n_rows, int64_t V,
                            int64_t ignore_index, int reduction, int dtype, void* stream) {
  if (!logits || !targets || !workspace) return HILDA_ERR_NULL;
  if (n_rows < 0 || V <= 0) return HILDA_ERR_SIZE;
  if (reduction < 0 || reduction > 2) return HILDA_ERR_ARG;
  if (reduction != 0 && !loss_out) return HILDA_ERR_NULL;
  cudaStream_t st = (cudaStream_t)stream;
  int* n_valid = reinterpret_cast<int*>(workspace);
  int* status = n_valid + 2;  // byte 8 of the workspace: non-zero if a bounded device-side wait ran out
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
  float* rows = loss_rows ? loss_rows : reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 16);
  count_valid_kernel<<<1, 1024, 0, st>>>(targets, n_rows, ignore_index, n_valid);
  HILDA_LAUNCH_CHECK();
  // row-sharded callers pass the count of valid rows over ALL shards, so that 'mean' is the global mean
  const int* nv = n_valid_in ? n_valid_in : n_valid;
  CEOp op;
  op.targets = targets; op.ignore_index = ignore_index; op.n_valid = nv;
  // training path: loss rows and grad pre-scaled by 1/n_valid; inference path: divide afterwards
  op.mean = (reduction == 1) ? 1 : 0;
  op.scale_loss = (grad != nullptr) ? 1 : 0;
  op.loss_rows = rows; op.lse_rows = lse_rows;
  int rc;
  switch (dtype) {
    case HILDA_F32: rc = launch_rows<float, CEOp>(logits, grad, n_rows, V, op, status, st); break;
    case HILDA_BF16: rc = launch_rows<__nv_bfloat16, CEOp>(logits, grad, n_rows, V, op, status, st); break;
    case HILDA_F16: rc = launch_rows<__half, CEOp>(logits, grad, n_rows, V, op, status, st); break;
    default: return HILDA_ERR_DTYPE;
  }
  if (rc != HILDA_OK) return rc;
  if (reduction != 0) {
    const int divide = (reduction == 1 && grad == nullptr) ? 1 : 0;
    sum_rows_kernel<<<1, 1024, 0, st>>>(rows, n_rows, nv, divide, loss_out);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

int hilda_scale_rows(const void* in, void* out, const float* scale, int per_row, int64_t n_rows, int64_t n_cols,
                     int dtype, void* stream) {
  if (!in || !out || !scale) return HILDA_ERR_NULL;
  if (n_rows < 0 || n_cols < 0) return HILDA_ERR_SIZE;
  if (n_rows == 0 || n_cols == 0) return HILDA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HILDA_F32: return scale_rows_t<float>(in, out, scale, per_row, n_rows, n_cols, st);
    case HILDA_BF16: return scale_rows_t<__nv_bfloat16>(in, out, scale, per_row, n_rows, n_cols, st);
    case HILDA_F16: return scale_rows_t<__half>(in, out, scale, per_row, n_rows, n_cols, st);
  }
  return HILDA_ERR_DTYPE;
}

int64_t hilda_grpo_workspace_bytes(int64_t B) { return 16 + (B > 0 ? B : 0) * 4; }

// logits [B, L+1, V] contiguous; ids [B, L] int64; mask [B, L] fp32 or null (0 = token skipped, any other
// value = its weight in the reductions, as the reference's completion_mask.float()); advantages [B] fp32;
// old_logp / ref_logp [B, L] fp32 or null. Per-token outputs loss/kl/clipped/lse [B, L] fp32
// (kl may be null when beta == 0). scalars_out[4] = {loss, kl_mean, clip_ratio, sum(mask)}. B_total > 0: the
// loss and the gradient are normalised by B_total sequences instead of B (sequences sharded over ranks).
// grad: [B, L+1, V] in the logits dtype (gradient for a unit upstream loss gradient) or null.
// workspace: hilda_grpo_workspace_bytes(B); seq_len[b] lives at byte 16.
int hilda_grpo_loss_fwd(const void* logits, const int64_t* ids, const float* advantages, const float* old_logp,
                        const float* ref_logp, const float* mask, void* grad, float* loss, float* kl, float* clipped,
                        float* lse, float* scalars_out, void* workspace, int64_t B, int64_t L, int64_t V,
                        int64_t B_total, float temperature, float beta, float eps_low, float eps_high, int dtype,
                        void* stream) {
  if (!logits || !ids || !advantages || !loss || !clipped || !lse || !scalars_out || !workspace) return HILDA_ERR_NULL;
  if (beta != 0.f && (!ref_logp || !kl)) return HILDA_ERR_NULL;
  if (B < 0 || L < 0 || V <= 0 || !(temperature > 0.f)) return HILDA_ERR_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  float* seq_len = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 16);
  int* status = reinterpret_cast<int*>(workspace);  // byte 0: non-zero if a bounded device-side wait ran out
  if (cudaMemsetAsync(status, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
  if (B > 0) {
    grpo_seq_len_kernel<<<(unsigned)B, 256, 0, st>>>(mask, L, seq_len);
    HILDA_LAUNCH_CHECK();
  }
  GRPOOp op;
  op.ids = ids; op.mask = mask; op.advantages = advantages; op.old_logp = old_logp; op.ref_logp = ref_logp;
  op.seq_len = seq_len; op.loss = loss; op.kl = (beta != 0.f) ? kl : nullptr; op.clipped = clipped; op.lse_out = lse;
  op.logp_out = nullptr; op.B = B; op.L = L; op.b_norm = (float)(B_total > 0 ? B_total : B); op.inv_t = 1.0f / temperature; op.beta = beta; op.eps_low = eps_low;
  op.eps_high = eps_high; op.logp_only = 0;
  const int64_t n_rows = B * (L + 1);
  int rc;
  switch (dtype) {
    case HILDA_F32: rc = launch_rows<float, GRPOOp>(logits, grad, n_rows, V, op, status, st); break;
    case HILDA_BF16: rc = launch_rows<__nv_bfloat16, GRPOOp>(logits, grad, n_rows, V, op, status, st); break;
    case HILDA_F16: rc = launch_rows<__half, GRPOOp>(logits, grad, n_rows, V, op, status, st); break;
    default: return HILDA_ERR_DTYPE;
  }
  if (rc != HILDA_OK) return rc;
  grpo_reduce_kernel<<<1, 1024, 0, st>>>(loss, op.kl, clipped, mask, seq_len, B, L, op.b_norm, scalars_out);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// logp[b,l] = logits[b,l,ids[b,l]]/T - logsumexp(logits[b,l,:]/T); masked positions give 0.
int hilda_selective_log_softmax(const void* logits, const int64_t* ids, const float* mask, float* logp, int64_t B,
                                int64_t L, int64_t V, float temperature, int dtype, void* stream) {
  if (!logits || !ids || !logp) return HILDA_ERR_NULL;
  if (B < 0 || L < 0 || V <= 0 || !(temperature > 0.f)) return HILDA_ERR_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  GRPOOp op = {};
  op.ids = ids; op.mask = mask; op.logp_out = logp; op.B = B; op.L = L; op.inv_t = 1.0f / temperature;
  op.logp_only = 1;
  const int64_t n_rows = B * (L + 1);
  switch (dtype) {
    case HILDA_F32: return launch_rows<float, GRPOOp>(logits, nullptr, n_rows, V, op, nullptr, st);
    case HILDA_BF16: return launch_rows<__nv_bfloat16, GRPOOp>(logits, nullptr, n_rows, V, op, nullptr, st);
    case HILDA_F16: return launch_rows<__half, GRPOOp>(logits, nullptr, n_rows, V, op, nullptr, st);
  }
  return HILDA_ERR_DTYPE;
}

}  // extern "C"
