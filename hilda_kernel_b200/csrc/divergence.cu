// KL divergence, Jensen-Shannon divergence and the row pass of the fused linear + JSD loss.
// Replaces the Triton kernels of hilda-kernel's kernels/kl_div.py (_kl_div_fwd_kernel :40-69,
// _kl_div_bwd_kernel :87-107), kernels/jsd.py (_jsd_kernel :30-90) and, for the fused operator,
// kernels/fused_linear_jsd.py (_log_softmax_kernel :46-76, _jsd_kernel, _softmax_grad_kernel :84-112
// as ONE kernel that goes from the two heads' logits to the student's dlogits).
//
// All three are HBM-bound row kernels: one CTA per row iteration, 16-byte vectors, fp32 math,
// a deterministic block reduction per row, no float atomics.
#include "common.cuh"
#include "reduce_kernels.cuh"
#include "hilda_b200.h"

namespace hilda {

constexpr float DV_LOG2E = 1.4426950408889634f;
constexpr float DV_LN2 = 0.6931471805599453f;
constexpr int DV_THREADS = 512;

__device__ __forceinline__ float dv_exp(float x) {  // e^x through ex2.approx
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * DV_LOG2E));
  return y;
}
__device__ __forceinline__ float dv_log(float x) {  // ln x through lg2.approx
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y * DV_LN2;
}

// fp32 data: library expf / logf (the sums cancel to a small KL value, keep the margin); 16-bit
// data: the approximate units.
template <typename T> __device__ __forceinline__ float kl_exp(float x) { return sizeof(T) == 4 ? expf(x) : dv_exp(x); }
template <typename T> __device__ __forceinline__ float kl_log(float x) { return sizeof(T) == 4 ? logf(x) : dv_log(x); }

// ---------------------------------------------------------------------------------- KL divergence
// loss_rows[row] = sum_j t * (log(max(t, eps)) - y)        (log_target == 0, kl_div.py:61-64)
//                = sum_j exp(t) * (t - y)                   (log_target != 0, kl_div.py:57-59)
template <typename T>
__global__ void __launch_bounds__(DV_THREADS)
kl_div_fwd_kernel(const T* __restrict__ y_pred, const T* __restrict__ y_true, float* __restrict__ loss_rows,
                  int64_t n_rows, int64_t n_cols, float eps, int log_target, int aligned) {
  constexpr int VEC = VT<T>::N;
  __shared__ float red[33];
  const bool vec_ok = aligned != 0;  // misaligned views take the element-wise path
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const T* yp = y_pred + row * n_cols;
    const T* yt = y_true + row * n_cols;
    float acc = 0.f;
    if (vec_ok) {
      // a row whose length is no multiple of the vector width starts and ends between 16-byte
      // boundaries: vectors over its aligned body, the few elements before and after one by one
      const int64_t head = min((int64_t)((VEC - ((row * n_cols) & (VEC - 1))) & (VEC - 1)), n_cols);
      const int64_t n_vec = (n_cols - head) / VEC;
      const int64_t rest = head + n_vec * VEC;
      for (int64_t v = threadIdx.x; v < n_vec; v += DV_THREADS) {
        float y[VEC], t[VEC];
        VT<T>::unpack(ld16_stream(yp + head + v * VEC), y);
        VT<T>::unpack(ld16_stream(yt + head + v * VEC), t);
#pragma unroll
        for (int j = 0; j < VEC; ++j)
          acc += log_target ? kl_exp<T>(t[j]) * (t[j] - y[j]) : t[j] * (kl_log<T>(fmaxf(t[j], eps)) - y[j]);
      }
      const int64_t n_edge = head + (n_cols - rest);
      if ((int64_t)threadIdx.x < n_edge) {
        const int64_t c = (int64_t)threadIdx.x < head ? (int64_t)threadIdx.x : rest + ((int64_t)threadIdx.x - head);
        const float y = VT<T>::load1(yp + c), t = VT<T>::load1(yt + c);
        acc += log_target ? kl_exp<T>(t) * (t - y) : t * (kl_log<T>(fmaxf(t, eps)) - y);
      }
    } else {
      for (int64_t c = threadIdx.x; c < n_cols; c += DV_THREADS) {
        const float y = VT<T>::load1(yp + c), t = VT<T>::load1(yt + c);
        acc += log_target ? kl_exp<T>(t) * (t - y) : t * (kl_log<T>(fmaxf(t, eps)) - y);
      }
    }
    acc = block_sum<DV_THREADS>(acc, red);
    if (threadIdx.x == 0) loss_rows[row] = acc;
  }
}

// dy_pred = -y_true * scale (or -exp(y_true) * scale), kl_div.py:98-105. scale = factor * grad_out[0]
// (grad_out null: factor alone).
template <typename T>
__global__ void __launch_bounds__(256)
kl_div_bwd_kernel(const T* __restrict__ y_true, T* __restrict__ dy, const float* __restrict__ grad_out, float factor,
                  int64_t n, int log_target, int aligned) {
  constexpr int VEC = VT<T>::N;
  const float scale = grad_out ? factor * grad_out[0] : factor;
  const int64_t n_vec = aligned ? n / VEC : 0;  // misaligned views: everything goes through the element-wise tail
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x; v < n_vec; v += stride) {
    float t[VEC];
    VT<T>::unpack(ld16_stream(y_true + v * VEC), t);
#pragma unroll
    for (int j = 0; j < VEC; ++j) t[j] = -(log_target ? kl_exp<T>(t[j]) : t[j]) * scale;
    st16_stream(dy + v * VEC, VT<T>::pack(t));
  }
  // ragged tail (n not a multiple of the vector width)
  for (int64_t i = n_vec * VEC + (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const float t = VT<T>::load1(y_true + i);
    VT<T>::store1(dy + i, -(log_target ? kl_exp<T>(t) : t) * scale);
  }
}

// out[0] = sum(rows) * factor, one CTA, fixed order.
__global__ void __launch_bounds__(1024)
dv_sum_scale_kernel(const float* __restrict__ rows, int64_t n, float factor, float* __restrict__ out) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) acc += rows[i];
  acc = block_sum<1024>(acc, red);
  if (threadIdx.x == 0) out[0] = acc * factor;
}

// ---------------------------------------------------------------------------------- JSD
// Per element, with x = student log-prob (log Q), y = teacher log-prob (log P) (jsd.py:66-84):
//   beta == 0: loss = p (y - x),                   dx = -p
//   beta == 1: loss = q (x - y),                   dx = q (x - y + 1)
//   else     : m = beta p + (1 - beta) q;  loss = beta p (y - log m) + (1 - beta) q (x - log m),
//              dx = (1 - beta) q (x - log m)
// (dx here is before the division by the number of non-ignored rows.)
// PRECISE (fp32 data): library expf / logf, so that the fp32 tolerance of 1e-5 has margin where
// x - log m nearly cancels; 16-bit data uses the approximate ex2 / lg2 units.
struct JsdTerm { float loss, dx; };
template <bool PRECISE>
__device__ __forceinline__ JsdTerm jsd_term(float x, float y, float beta, int mode) {
  auto ex = [](float v) { return PRECISE ? expf(v) : dv_exp(v); };
  auto lg = [](float v) { return PRECISE ? logf(v) : dv_log(v); };
  JsdTerm r;
  if (mode == 0) {
    const float p = ex(y);
    r.loss = p * (y - x);
    r.dx = -p;
  } else if (mode == 1) {
    const float q = ex(x);
    r.loss = q * (x - y);
    r.dx = q * (x - y + 1.0f);
  } else {
    const float q = ex(x), p = ex(y);
    const float m = beta * p + (1.0f - beta) * q;
    const float log_m = m > 0.f ? lg(m) : 0.f;  // both probabilities underflowed: the terms are 0, not 0 * inf
    const float qs = (1.0f - beta) * q * (x - log_m);
    r.loss = beta * p * (y - log_m) + qs;
    r.dx = qs;
  }
  return r;
}

__device__ __forceinline__ int jsd_mode(float beta) { return beta == 0.0f ? 0 : (beta == 1.0f ? 1 : 2); }

// The general-beta term of 16-bit data in the log2 domain, with the constants taken out of the element:
// with x2 = x log2(e), y2 = y log2(e), q = 2^x2, p = 2^y2, l = log2(beta p + (1 - beta) q),
//   t = q (x2 - l), u = p (y2 - l):  loss = ln2 (beta u + (1 - beta) t),  dx = ln2 (1 - beta) t.
// The kernel sums t and u and applies the constants once per row: 15 instructions per element instead of 18.
// m is clamped to the smallest normal number instead of tested against 0: where both probabilities
// underflow, t and u are 0 x finite = 0 as before.
struct JsdFast { float t, u; };
__device__ __forceinline__ JsdFast jsd_fast(float x, float y, float bp, float bq) {
  const float x2 = x * DV_LOG2E, y2 = y * DV_LOG2E;
  float q, p, l;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(q) : "f"(x2));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(y2));
  const float m = fmaxf(fmaf(bp, p, bq * q), 1.17549435e-38f);
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(m));
  return JsdFast{q * (x2 - l), p * (y2 - l)};
}

// Stand-alone JSD (jsd.py:30-90): X, Y log-probs [n_rows, V]; one sweep writes dX = dx / n and the
// row's loss / n, n = number of rows whose label is not ignore_index (all rows without labels).
template <typename T>
__global__ void __launch_bounds__(DV_THREADS)
jsd_rows_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ dX, float* __restrict__ loss_rows,
                const int64_t* __restrict__ labels, int64_t ignore_index, const int* __restrict__ n_valid,
                int64_t n_rows, int64_t V, float beta, int aligned) {
  constexpr int VEC = VT<T>::N;
  __shared__ float red[33];
  const int mode = jsd_mode(beta);
  const float inv_n = 1.0f / (n_valid ? fmaxf((float)(*n_valid), 1.0f) : (float)n_rows);
  const bool vec_ok = aligned != 0;
  for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
    const bool ignored = labels && labels[row] == ignore_index;
    float acc = 0.f, acc_t = 0.f, acc_u = 0.f;
    const bool fast = sizeof(T) == 2 && mode == 2;
    const float dx_c = DV_LN2 * (1.0f - beta) * inv_n;
    if (vec_ok) {
      // vectors over the aligned body of the row; the elements before and after it one by one
      const int64_t head = min((int64_t)((VEC - ((row * V) & (VEC - 1))) & (VEC - 1)), V);
      const int64_t n_vec = (V - head) / VEC;
      const int64_t rest = head + n_vec * VEC;
      const int64_t n_edge = head + (V - rest);
      if ((int64_t)threadIdx.x < n_edge) {
        const int64_t c = (int64_t)threadIdx.x < head ? (int64_t)threadIdx.x : rest + ((int64_t)threadIdx.x - head);
        const int64_t at = row * V + c;
        if (ignored) {
          VT<T>::store1(dX + at, 0.f);
        } else {
          const JsdTerm t = jsd_term<sizeof(T) == 4>(VT<T>::load1(X + at), VT<T>::load1(Y + at), beta, mode);
          acc += t.loss;
          VT<T>::store1(dX + at, t.dx * inv_n);
        }
      }
      const T* x = X + row * V + head;
      const T* y = Y + row * V + head;
      T* d = dX + row * V + head;
      if (ignored) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int64_t v = threadIdx.x; v < n_vec; v += DV_THREADS) st16_stream(d + v * VEC, z);
      } else {
        // two vectors of each operand in flight per thread and iteration
        for (int64_t v = threadIdx.x; v < n_vec; v += 2 * DV_THREADS) {
          const int64_t v2 = v + DV_THREADS;
          const bool has2 = v2 < n_vec;
          const uint4 xa = ld16_stream(x + v * VEC), ya = ld16_stream(y + v * VEC);
          const uint4 xb = has2 ? ld16_stream(x + v2 * VEC) : make_uint4(0, 0, 0, 0);
          const uint4 yb = has2 ? ld16_stream(y + v2 * VEC) : make_uint4(0, 0, 0, 0);
          float xf[VEC], yf[VEC];
          VT<T>::unpack(xa, xf);
          VT<T>::unpack(ya, yf);
          if (fast) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
              const JsdFast f = jsd_fast(xf[j], yf[j], beta, 1.0f - beta);
              acc_t += f.t; acc_u += f.u;
              xf[j] = f.t * dx_c;
            }
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
              const JsdTerm t = jsd_term<sizeof(T) == 4>(xf[j], yf[j], beta, mode);
              acc += t.loss;
              xf[j] = t.dx * inv_n;
            }
          }
          st16_stream(d + v * VEC, VT<T>::pack(xf));
          if (has2) {
            VT<T>::unpack(xb, xf);
            VT<T>::unpack(yb, yf);
            if (fast) {
#pragma unroll
              for (int j = 0; j < VEC; ++j) {
                const JsdFast f = jsd_fast(xf[j], yf[j], beta, 1.0f - beta);
                acc_t += f.t; acc_u += f.u;
                xf[j] = f.t * dx_c;
              }
            } else {
#pragma unroll
              for (int j = 0; j < VEC; ++j) {
                const JsdTerm t = jsd_term<sizeof(T) == 4>(xf[j], yf[j], beta, mode);
                acc += t.loss;
                xf[j] = t.dx * inv_n;
              }
            }
            st16_stream(d + v2 * VEC, VT<T>::pack(xf));
          }
        }
      }
    } else {
      const T* x = X + row * V;
      const T* y = Y + row * V;
      T* d = dX + row * V;
      for (int64_t c = threadIdx.x; c < V; c += DV_THREADS) {
        if (ignored) { VT<T>::store1(d + c, 0.f); continue; }
        const JsdTerm t = jsd_term<sizeof(T) == 4>(VT<T>::load1(x + c), VT<T>::load1(y + c), beta, mode);
        acc += t.loss;
        VT<T>::store1(d + c, t.dx * inv_n);
      }
    }
    acc += DV_LN2 * (beta * acc_u + (1.0f - beta) * acc_t);
    acc = block_sum<DV_THREADS>(acc, red);
    if (threadIdx.x == 0) loss_rows[row] = ignored ? 0.f : acc * inv_n;
  }
}

// Row pass of the fused linear + JSD loss (fused_linear_jsd.py:168-205 between the two lm_head GEMMs
// and the two gradient GEMMs). In: the student's and the teacher's logits of one row chunk as the
// logits GEMM left them (16-bit, row pitch `pitch`), and per row the natural-log (max, sum-exp) of
// logits / temperature from that GEMM's epilogue statistics. Sweep 1: x = s / T - lse_s,
// y = t / T - lse_t, the row's loss and sum_j dx_j. Sweep 2 (the row is still in L2): the student's
//   dlogits_j = (dx_j - exp(x_j) * sum dx) / (T * n)
// over its logits, in place. Ignored rows: loss 0, zero row.
template <typename T>
__global__ void __launch_bounds__(DV_THREADS)
fljsd_rows_kernel(T* __restrict__ S, const T* __restrict__ Tt, int64_t pitch, const float* __restrict__ rowstat_s,
                  const float* __restrict__ rowstat_t, const int64_t* __restrict__ labels, int64_t ignore_index,
                  const int* __restrict__ n_valid, int64_t n_norm, float* __restrict__ loss_rows, int64_t rows, int64_t V,
                  float beta, float inv_temp) {
  constexpr int VEC = VT<T>::N;
  __shared__ float red[33];
  const int mode = jsd_mode(beta);
  const float inv_n = 1.0f / (n_valid ? fmaxf((float)(*n_valid), 1.0f) : (float)n_norm);
  const int64_t n_vec = (V + VEC - 1) / VEC;  // the pitch is a multiple of 256: a ragged last vector stays in the row
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    T* s = S + row * pitch;
    const T* t = Tt + row * pitch;
    if (labels && labels[row] == ignore_index) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int64_t v = threadIdx.x; v < n_vec; v += DV_THREADS) st16(s + v * VEC, z);
      if (threadIdx.x == 0) loss_rows[row] = 0.f;
      continue;
    }
    const float lse_s = rowstat_s[row] + logf(rowstat_s[rows + row]);
    const float lse_t = rowstat_t[row] + logf(rowstat_t[rows + row]);
    float acc_loss = 0.f, acc_dx = 0.f;
    for (int64_t v = threadIdx.x; v < n_vec; v += DV_THREADS) {
      float sf[VEC], tf[VEC];
      VT<T>::unpack(ld16(s + v * VEC), sf);
      VT<T>::unpack(ld16(t + v * VEC), tf);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        if (v * VEC + j < V) {
          const JsdTerm e = jsd_term<sizeof(T) == 4>(fmaf(sf[j], inv_temp, -lse_s), fmaf(tf[j], inv_temp, -lse_t), beta, mode);
          acc_loss += e.loss;
          acc_dx += e.dx;
        }
      }
    }
    acc_loss = block_sum<DV_THREADS>(acc_loss, red);
    acc_dx = block_sum<DV_THREADS>(acc_dx, red);
    const float g = inv_temp * inv_n;
    for (int64_t v = threadIdx.x; v < n_vec; v += DV_THREADS) {
      float sf[VEC], tf[VEC];
      VT<T>::unpack(ld16(s + v * VEC), sf);
      VT<T>::unpack(ld16(t + v * VEC), tf);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float x = fmaf(sf[j], inv_temp, -lse_s);
        const JsdTerm e = jsd_term<sizeof(T) == 4>(x, fmaf(tf[j], inv_temp, -lse_t), beta, mode);
        sf[j] = (v * VEC + j < V) ? (e.dx - dv_exp(x) * acc_dx) * g : 0.f;
      }
      st16(s + v * VEC, VT<T>::pack(sf));
    }
    if (threadIdx.x == 0) loss_rows[row] = acc_loss * inv_n;
  }
}

static inline int dv_grid(int64_t n_rows) {
  const int64_t cap = (int64_t)sm_count() * 4;  // 4 CTAs of 512 threads per SM
  return (int)(n_rows < cap ? (n_rows > 0 ? n_rows : 1) : cap);
}

}  // namespace hilda

using namespace hilda;

extern "C" {

// reduction: 0 none (loss_rows only), 1 sum, 2 mean (/ (n_rows * n_cols)), 3 batchmean (/ n_rows)
int hilda_kl_div_fwd(const void* y_pred, const void* y_true, float* loss_rows, float* loss_out, int64_t n_rows,
                     int64_t n_cols, int reduction, int log_target, float eps, int dtype, void* stream) {
  if (reduction < 0 || reduction > 3) return HILDA_ERR_ARG;
  if (n_rows < 0 || n_cols <= 0) return HILDA_ERR_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_rows == 0) {
    if (reduction != 0 && loss_out && cudaMemsetAsync(loss_out, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
    return HILDA_OK;
  }
  if (!y_pred || !y_true || !loss_rows || (reduction != 0 && !loss_out)) return HILDA_ERR_NULL;
  const int al = aligned16(y_pred) && aligned16(y_true);
  const int grid = dv_grid(n_rows);
  switch (dtype) {
    case HILDA_F32:
      kl_div_fwd_kernel<float><<<grid, DV_THREADS, 0, st>>>((const float*)y_pred, (const float*)y_true, loss_rows, n_rows,
                                                           n_cols, eps, log_target, al);
      break;
    case HILDA_BF16:
      kl_div_fwd_kernel<__nv_bfloat16><<<grid, DV_THREADS, 0, st>>>((const __nv_bfloat16*)y_pred, (const __nv_bfloat16*)y_true,
                                                                   loss_rows, n_rows, n_cols, eps, log_target, al);
      break;
    case HILDA_F16:
      kl_div_fwd_kernel<__half><<<grid, DV_THREADS, 0, st>>>((const __half*)y_pred, (const __half*)y_true, loss_rows, n_rows,
                                                            n_cols, eps, log_target, al);
      break;
    default: return HILDA_ERR_DTYPE;
  }
  HILDA_LAUNCH_CHECK();
  if (reduction != 0) {
    const float factor = reduction == 1 ? 1.0f : (reduction == 2 ? 1.0f / ((float)n_rows * (float)n_cols) : 1.0f / (float)n_rows);
    dv_sum_scale_kernel<<<1, 1024, 0, st>>>(loss_rows, n_rows, factor, loss_out);
    HILDA_LAUNCH_CHECK();
  }
  return HILDA_OK;
}

// dy_pred = -y_true (or -exp(y_true)) * grad_out[0] * (reduction factor); reduction 0 ignores grad_out
// (scale 1, as kl_div.py:146-153 does).
int hilda_kl_div_bwd(const void* y_true, void* dy_pred, const float* grad_out, int64_t n_rows, int64_t n_cols,
                     int reduction, int log_target, int dtype, void* stream) {
  if (reduction < 0 || reduction > 3) return HILDA_ERR_ARG;
  if (n_rows < 0 || n_cols <= 0) return HILDA_ERR_SIZE;
  if (n_rows == 0) return HILDA_OK;
  if (!y_true || !dy_pred || (reduction != 0 && !grad_out)) return HILDA_ERR_NULL;
  const int al = aligned16(y_true) && aligned16(dy_pred);
  cudaStream_t st = (cudaStream_t)stream;
  const float factor = reduction == 2 ? 1.0f / ((float)n_rows * (float)n_cols) : (reduction == 3 ? 1.0f / (float)n_rows : 1.0f);
  const float* g = reduction == 0 ? nullptr : grad_out;
  const int64_t n = n_rows * n_cols;
  const int es = dtype_size(dtype);
  if (!es) return HILDA_ERR_DTYPE;
  int64_t blocks = (n / (16 / es) + 256 * 4 - 1) / (256 * 4);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  switch (dtype) {
    case HILDA_F32:
      kl_div_bwd_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)y_true, (float*)dy_pred, g, factor, n, log_target, al);
      break;
    case HILDA_BF16:
      kl_div_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)y_true, (__nv_bfloat16*)dy_pred, g,
                                                                       factor, n, log_target, al);
      break;
    default:
      kl_div_bwd_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half*)y_true, (__half*)dy_pred, g, factor, n, log_target, al);
      break;
  }
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// Stand-alone JSD: loss_out = sum over rows of loss_rows; dX already divided by the number of
// non-ignored rows. workspace: one int (the count), needed only with labels.
int hilda_jsd_fwd(const void* X, const void* Y, void* dX, float* loss_rows, float* loss_out, const int64_t* labels,
                  int64_t ignore_index, void* workspace, int64_t n_rows, int64_t V, float beta, int dtype, void* stream) {
  if (n_rows < 0 || V <= 0) return HILDA_ERR_SIZE;
  cudaStream_t st = (cudaStream_t)stream;
  if (n_rows == 0) {
    if (loss_out && cudaMemsetAsync(loss_out, 0, 4, st) != cudaSuccess) return HILDA_ERR_CUDA;
    return HILDA_OK;
  }
  if (!X || !Y || !dX || !loss_rows || !loss_out || (labels && !workspace)) return HILDA_ERR_NULL;
  const int al = aligned16(X) && aligned16(Y) && aligned16(dX);
  int* n_valid = nullptr;
  if (labels) {
    n_valid = reinterpret_cast<int*>(workspace);
    count_valid_kernel<<<1, 1024, 0, st>>>(labels, n_rows, ignore_index, n_valid);
    HILDA_LAUNCH_CHECK();
  }
  const int grid = dv_grid(n_rows);
  switch (dtype) {
    case HILDA_F32:
      jsd_rows_kernel<float><<<grid, DV_THREADS, 0, st>>>((const float*)X, (const float*)Y, (float*)dX, loss_rows, labels,
                                                         ignore_index, n_valid, n_rows, V, beta, al);
      break;
    case HILDA_BF16:
      jsd_rows_kernel<__nv_bfloat16><<<grid, DV_THREADS, 0, st>>>((const __nv_bfloat16*)X, (const __nv_bfloat16*)Y,
                                                                 (__nv_bfloat16*)dX, loss_rows, labels, ignore_index, n_valid,
                                                                 n_rows, V, beta, al);
      break;
    case HILDA_F16:
      jsd_rows_kernel<__half><<<grid, DV_THREADS, 0, st>>>((const __half*)X, (const __half*)Y, (__half*)dX, loss_rows, labels,
                                                          ignore_index, n_valid, n_rows, V, beta, al);
      break;
    default: return HILDA_ERR_DTYPE;
  }
  HILDA_LAUNCH_CHECK();
  dv_sum_scale_kernel<<<1, 1024, 0, st>>>(loss_rows, n_rows, 1.0f, loss_out);
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

// Row pass of the fused linear + JSD loss over one row chunk: s_logits (in: the student's logits,
// out: its dlogits) and t_logits are [padded rows, hilda_flce_logits_pitch(V)] 16-bit scratch as
// hilda_flce_logits_scaled leaves them; rowstat_s / rowstat_t are [3, rows] from
// hilda_flce_row_stats. The divisor is *n_valid (clamped to 1) when given, else n_norm.
int hilda_fljsd_dlogits(void* s_logits, const void* t_logits, const float* rowstat_s, const float* rowstat_t,
                        const int64_t* labels, int64_t ignore_index, const int* n_valid, int64_t n_norm, float* loss_rows,
                        int64_t rows, int64_t V, float beta, float inv_temperature, int dtype, void* stream) {
  if (rows < 0 || V <= 0) return HILDA_ERR_SIZE;
  if (rows == 0) return HILDA_OK;
  if (!s_logits || !t_logits || !rowstat_s || !rowstat_t || !loss_rows) return HILDA_ERR_NULL;
  if (!n_valid && n_norm <= 0) return HILDA_ERR_ARG;
  if (!aligned16(s_logits) || !aligned16(t_logits)) return HILDA_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t pitch = hilda_flce_logits_pitch(V);
  // 2 CTAs of 512 threads per SM: both sweeps of the rows in flight (148 x 2 x 2 x 256 KB at
  // V = 128256) stay within L2
  int64_t grid = (int64_t)sm_count() * 2;
  if (grid > rows) grid = rows;
  if (dtype == HILDA_BF16)
    fljsd_rows_kernel<__nv_bfloat16><<<(unsigned)grid, DV_THREADS, 0, st>>>((__nv_bfloat16*)s_logits, (const __nv_bfloat16*)t_logits,
                                                                          pitch, rowstat_s, rowstat_t, labels, ignore_index,
                                                                          n_valid, n_norm, loss_rows, rows, V, beta,
                                                                          inv_temperature);
  else if (dtype == HILDA_F16)
    fljsd_rows_kernel<__half><<<(unsigned)grid, DV_THREADS, 0, st>>>((__half*)s_logits, (const __half*)t_logits, pitch, rowstat_s,
                                                                   rowstat_t, labels, ignore_index, n_valid, n_norm, loss_rows,
                                                                   rows, V, beta, inv_temperature);
  else
    return HILDA_ERR_DTYPE;
  HILDA_LAUNCH_CHECK();
  return HILDA_OK;
}

}  // extern "C"
