// A residual stream kept in fp32 whatever the activation dtype: scaled embedding rows, the
// "norm on the sublayer's output" update with a one-number RMSNorm gain, the weighted sum over
// the outputs of all earlier layers (depth-weighted average), and the gated-linear-unit
// activation with clamped pre-activations that the feed-forward layers of such models use.
//
// Every kernel takes the activation dtype as a template parameter (the GEMMs between these ops
// read and write that dtype) and does its arithmetic in fp32.
#include "common.cuh"

namespace llb {

// Block-wide sum of one float per thread (any blockDim.x that is a multiple of 32, up to 1024).
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// x[m][:] = wte[idx[m]][:] * scale  (fp32), and the same rounded to the activation dtype.
template <typename TW, typename TA>
__global__ void embed_scaled_kernel(const TW* __restrict__ wte, const int64_t* __restrict__ idx, float scale,
                                    float* __restrict__ x, TA* __restrict__ x_act, int dim) {
  const int m = blockIdx.x;
  const TW* row = wte + (size_t)idx[m] * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = dt<TW>::ld(row, i) * scale;
    x[(size_t)m * dim + i] = v;
    if (x_act) dt<TA>::st(x_act, (size_t)m * dim + i, v);
  }
}

// r = x + gain * y / sqrt(mean(y^2) + eps)                      -> out      (fp32; may be a slot of `stack`)
// n_mix > 0:  v = mix_w[n_mix-1] * r + sum_{j < n_mix-1} mix_w[j] * stack[j]   else v = r
// v -> next (fp32, optional) and next_act (activation dtype, optional)
// x == nullptr means a plain norm (r = gain * y / rms).
template <typename TY, typename TA>
__global__ void gain_norm_add_mix_kernel(const float* x, const TY* __restrict__ y,
                                         const float* __restrict__ gain, float eps, float* out,
                                         const float* stack, size_t stack_stride,
                                         const float* __restrict__ mix_w, int n_mix, float* next,
                                         TA* __restrict__ next_act, int dim) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = dt<TY>::ld(y, base + i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float k = gain[0] / sqrtf(ss / (float)dim + eps);
  const float w_last = n_mix > 0 ? mix_w[n_mix - 1] : 1.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float r = dt<TY>::ld(y, base + i) * k;
    if (x) r += x[base + i];
    if (out) out[base + i] = r;
    float v = r * w_last;
    for (int j = 0; j < n_mix - 1; ++j) v += mix_w[j] * stack[(size_t)j * stack_stride + base + i];
    if (next) next[base + i] = v;
    if (next_act) dt<TA>::st(next_act, base + i, v);
  }
}

// Gated linear unit with clamped pre-activations, on the output of one GEMM over the stacked
// [gate; up] weight:  g = min(gu[m][c], limit), u = clamp(gu[m][ff + c], -limit, limit),
// h[m][c] = g * sigmoid(alpha * g) * (u + 1).
template <typename T>
__global__ void glu_clamp_kernel(const T* __restrict__ gu, int gu_stride, int ff, float limit, float alpha,
                                 T* __restrict__ h, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t m = i / ff;
  const int c = (int)(i - m * ff);
  const float g = fminf(dt<T>::ld(gu, m * gu_stride + c), limit);
  const float u = fminf(fmaxf(dt<T>::ld(gu, m * gu_stride + ff + c), -limit), limit);
  dt<T>::st(h, i, g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_embed_scaled(const void* wte, int wte_dtype, const int64_t* idx, float scale, float* x, void* x_act,
                    int act_dtype, int M, int dim, ll_stream stream) {
  LL_CHECK_ARG(wte && idx && x && M >= 0 && dim > 0, "bad embed_scaled arguments");
  if (M == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 1024 ? 256 : 128;
  if (wte_dtype == LL_F32 && act_dtype == LL_F32)
    embed_scaled_kernel<float, float><<<M, threads, 0, st>>>((const float*)wte, idx, scale, x, (float*)x_act, dim);
  else if (wte_dtype == LL_BF16 && act_dtype == LL_BF16)
    embed_scaled_kernel<__nv_bfloat16, __nv_bfloat16><<<M, threads, 0, st>>>((const __nv_bfloat16*)wte, idx, scale, x,
                                                                            (__nv_bfloat16*)x_act, dim);
  else if (wte_dtype == LL_BF16 && act_dtype == LL_F32)
    embed_scaled_kernel<__nv_bfloat16, float><<<M, threads, 0, st>>>((const __nv_bfloat16*)wte, idx, scale, x, (float*)x_act, dim);
  else {
    set_error("embed_scaled: unsupported dtypes %d / %d", wte_dtype, act_dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("embed_scaled_kernel");
  return LL_OK;
}

int ll_gain_norm_add_mix(const float* x, const void* y, int y_dtype, const float* gain, float eps, float* out,
                         const float* stack, size_t stack_stride, const float* mix_w, int n_mix, float* next,
                         void* next_act, int act_dtype, int rows, int dim, ll_stream stream) {
  LL_CHECK_ARG(y && gain && rows >= 0 && dim > 0 && n_mix >= 0, "bad gain_norm_add_mix arguments");
  LL_CHECK_ARG(n_mix <= 1 || (stack && mix_w), "gain_norm_add_mix: a mix needs the stack and its weights");
  LL_CHECK_ARG(n_mix == 0 || mix_w, "gain_norm_add_mix: a mix needs its weights");
  if (rows == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 2048 ? 512 : dim >= 512 ? 256 : 128;
  if (y_dtype == LL_F32 && act_dtype == LL_F32)
    gain_norm_add_mix_kernel<float, float><<<rows, threads, 0, st>>>(x, (const float*)y, gain, eps, out, stack, stack_stride,
                                                                     mix_w, n_mix, next, (float*)next_act, dim);
  else if (y_dtype == LL_BF16 && act_dtype == LL_BF16)
    gain_norm_add_mix_kernel<__nv_bfloat16, __nv_bfloat16><<<rows, threads, 0, st>>>(
        x, (const __nv_bfloat16*)y, gain, eps, out, stack, stack_stride, mix_w, n_mix, next, (__nv_bfloat16*)next_act, dim);
  else if (y_dtype == LL_F32 && act_dtype == LL_BF16)
    gain_norm_add_mix_kernel<float, __nv_bfloat16><<<rows, threads, 0, st>>>(x, (const float*)y, gain, eps, out, stack, stack_stride,
                                                                             mix_w, n_mix, next, (__nv_bfloat16*)next_act, dim);
  else {
    set_error("gain_norm_add_mix: unsupported dtypes %d / %d", y_dtype, act_dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("gain_norm_add_mix_kernel");
  return LL_OK;
}

int ll_glu_clamp(const void* gu, int gu_stride, int ff, float limit, float alpha, void* h, int dtype, int rows,
                 ll_stream stream) {
  LL_CHECK_ARG(gu && h && ff > 0 && gu_stride >= 2 * ff && rows >= 0, "bad glu_clamp arguments");
  const size_t n = (size_t)rows * ff;
  if (n == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == LL_F32) glu_clamp_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, gu_stride, ff, limit, alpha, (float*)h, n);
  else if (dtype == LL_BF16)
    glu_clamp_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu, gu_stride, ff, limit, alpha, (__nv_bfloat16*)h, n);
  else {
    set_error("glu_clamp: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("glu_clamp_kernel");
  return LL_OK;
}

}  // extern "C"

// ---- two-branch layers on an fp32 stream: x += sum of branch outputs, then two norms of the same x -----------------
namespace llb {

// x[m][:] += s0 * a0 + s1 * a1 + s2 * a2 (each optional, activation dtype TA), in place, fp32.  Then, with
// n = x / sqrt(mean(x^2) + eps):  out1 = n * w1 (fp32 or TA, see out1_f32; optional), out2 = n * w2 (TA; optional).
template <typename TA>
__global__ void add_norm_pair_kernel(float* __restrict__ x, const TA* __restrict__ a0, float s0, const TA* __restrict__ a1,
                                     float s1, const TA* __restrict__ a2, float s2, const float* __restrict__ w1,
                                     const float* __restrict__ w2, float eps, void* __restrict__ out1, int out1_f32,
                                     TA* __restrict__ out2, int dim) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = x[base + i];
    if (a0 || a1 || a2) {
      float add = 0.f;
      if (a0) add += s0 * dt<TA>::ld(a0, base + i);
      if (a1) add += s1 * dt<TA>::ld(a1, base + i);
      if (a2) add += s2 * dt<TA>::ld(a2, base + i);
      v += add;
      x[base + i] = v;
    }
    ss += v * v;
  }
  if (!out1 && !out2) return;
  ss = block_sum(ss, red);
  const float k = 1.f / sqrtf(ss / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float n = x[base + i] * k;
    if (out1) {
      if (out1_f32) ((float*)out1)[base + i] = n * w1[i];
      else dt<TA>::st((TA*)out1, base + i, n * w1[i]);
    }
    if (out2) dt<TA>::st(out2, base + i, n * w2[i]);
  }
}

// RMS norm of an fp32 row in `groups` equal parts (each by its own root mean square), a weight, and a gate (silu, or a
// sigmoid when gate_sigmoid):
//   gate_first: t = y * gate(g);  out = t / rms_part(t) * w          (the gate enters the norm)
//   otherwise : out = y / rms_part(y) * w * gate(g)                  (the gate follows the norm)
// w has C entries, or C / groups entries shared by the parts (w_shared).  One block per row.
// A part of y spans y_gs >= C / groups numbers (the rest is skipped), except with `stab`: then number C / groups of every
// part is a normaliser's product nq and stab[m][part] a stabiliser mx, and the part is first divided by
// max(|nq|, exp(-mx)) + 1e-6 (the read-out of a matrix memory with exponential gates).
template <typename TA>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int y_gs, const float* __restrict__ stab,
                                        const TA* __restrict__ gate, int gate_stride, const float* __restrict__ w, int w_shared,
                                        float eps, int groups, int gate_first, int gate_sigmoid, TA* __restrict__ out, int C) {
  const int m = blockIdx.x;
  const int gs = C / groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nw) {
    const float* yr = y + ((size_t)m * groups + g) * y_gs;
    const TA* gr = gate + (size_t)m * gate_stride + (size_t)g * gs;
    const float pre = stab ? 1.f / (fmaxf(fabsf(yr[gs]), expf(-stab[(size_t)m * groups + g])) + 1e-6f) : 1.f;
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) {
      float v = yr[i] * pre;
      if (gate_first) {
        const float z = dt<TA>::ld(gr, i);
        v *= (gate_sigmoid ? 1.f : z) / (1.f + expf(-z));
      }
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float k = 1.f / sqrtf(ss / (float)gs + eps);
    for (int i = lane; i < gs; i += 32) {
      const float z = dt<TA>::ld(gr, i);
      const float sg = (gate_sigmoid ? 1.f : z) / (1.f + expf(-z));
      const float wv = w[w_shared ? i : g * gs + i];
      const float yv = yr[i] * pre;
      const float v = gate_first ? (yv * sg) * k * wv : yv * k * wv * sg;
      dt<TA>::st(out, (size_t)m * C + (size_t)g * gs + i, v);
    }
  }
}

// in place: relu(v)^2
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ h, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = fmaxf(dt<T>::ld(h, i), 0.f);
  dt<T>::st(h, i, v * v);
}

// in place: gelu(v), the erf form 0.5 v (1 + erf(v / sqrt 2)) or (tanh_form) 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))
template <typename T>
__global__ void gelu_kernel(T* __restrict__ h, int tanh_form, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = dt<T>::ld(h, i);
  const float r = tanh_form ? 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)))
                            : 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  dt<T>::st(h, i, r);
}

// Several copies of the residual stream ("hyper-connections"): X [rows][S][dim] fp32.  One launch closes a sublayer and opens
// the next:
//   write   X'[t] = sum_s mix[s][t] X[s] + out[t] * r * ls * y      all S copies at once from the old ones (mix [S][S] indexed
//           [from][to], NULL: every copy keeps itself; y the sublayer's result in the activation dtype, NULL: nothing is added;
//           ls a per-channel scale of y, NULL: none)
//   read    u = sum_t in[t] X'[t] (in NULL: the plain sum);  h = u / sqrt(mean(u^2) + eps) * w      (h NULL: no read)
//   total   (optional) the plain sum of the new copies, fp32 [rows][dim]
// The old copies are read at src + m * src_row + s * src_copy (src_copy 0: every copy starts as the same row, the embedding
// output); when src is X itself and nothing is added or mixed, nothing is written.
template <typename TA, int SMAX>
__global__ void hyper_mix_norm_kernel(const float* src, long long src_row, long long src_copy, float* X, const TA* __restrict__ y,
                                      const float* __restrict__ ls, float r, const float* __restrict__ mix,
                                      const float* __restrict__ w_out, const float* __restrict__ w_in, const float* __restrict__ w,
                                      float eps, void* __restrict__ h, int h_f32, float* __restrict__ total, int S, int dim) {
  extern __shared__ float hyper_us[];            // the row of u
  __shared__ float red[32];
  __shared__ float cm[SMAX * SMAX], co[SMAX], ci[SMAX];
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) cm[i] = mix ? mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) co[i] = w_out ? w_out[i] : 1.f, ci[i] = w_in ? w_in[i] : 1.f;
  __syncthreads();
  const size_t m = blockIdx.x;
  const bool write = y || mix || src != X || src_row != (long long)S * dim || src_copy != dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float xs[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) xs[s] = s < S ? src[m * src_row + s * src_copy + i] : 0.f;
    float yv = 0.f;
    if (y) {
      yv = dt<TA>::ld(y, m * dim + i);
      if (ls) yv *= ls[i];
      yv *= r;
    }
    float u = 0.f, tot = 0.f;
#pragma unroll
    for (int t = 0; t < SMAX; ++t) {
      if (t >= S) break;
      float xt = xs[t];
      if (mix) {
        xt = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) xt = fmaf(cm[s * S + t], xs[s], xt);
      }
      if (y) xt = fmaf(co[t], yv, xt);
      if (write) X[(m * S + t) * dim + i] = xt;
      u = fmaf(ci[t], xt, u);
      tot += xt;
    }
    if (total) total[m * dim + i] = tot;
    hyper_us[i] = u;
    ss += u * u;
  }
  if (!h) return;
  ss = block_sum(ss, red);
  const float k = 1.f / sqrtf(ss / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float n = hyper_us[i] * k * w[i];
    if (h_f32) ((float*)h)[m * dim + i] = n;
    else dt<TA>::st((TA*)h, m * dim + i, n);
  }
}

// out[m][:] = x[m][:] / sqrt(mean(x[m][:]^2) + eps) * w      (rows of x_stride / out_stride elements; w fp32 or NULL)
template <typename T>
__global__ void row_norm_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w, float eps, T* __restrict__ out,
                                int out_stride, int dim) {
  __shared__ float red[32];
  const T* xr = x + (size_t)blockIdx.x * x_stride;
  T* orow = out + (size_t)blockIdx.x * out_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = dt<T>::ld(xr, i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float k = 1.f / sqrtf(ss / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dt<T>::st(orow, i, dt<T>::ld(xr, i) * k * (w ? w[i] : 1.f));
}

// out[m][c] = a[m][c] * sigmoid(gate[m][c])     (each with its own row stride; out may be a)
template <typename T>
__global__ void sigmoid_gate_mul_kernel(const T* a, int a_stride, const T* __restrict__ gate, int gate_stride, T* out, int out_stride,
                                        int C, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t m = i / C, c = i - m * C;
  const float g = dt<T>::ld(gate, m * gate_stride + c);
  dt<T>::st(out, m * out_stride + c, dt<T>::ld(a, m * a_stride + c) / (1.f + expf(-g)));
}

// in place: cap * tanh(v / cap)
__global__ void tanh_cap_kernel(float* __restrict__ x, float cap, float inv_cap, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}

}  // namespace llb

extern "C" {

int ll_hyper_mix_norm(const float* src, long long src_row, long long src_copy, float* X, const void* y, const float* ls, float r,
                      const float* mix, const float* w_out, const float* w_in, const float* w, float eps, void* h, int h_f32,
                      float* total, int act_dtype, int rows, int S, int dim, ll_stream stream) {
  LL_CHECK_ARG(src && X && rows >= 0 && S >= 1 && dim > 0 && (!h || w) && (!y || w_out), "bad hyper_mix_norm arguments");
  if (S > 8) {
    set_error("hyper_mix_norm: %d copies of the stream (up to 8)", S);
    return LL_ERR_UNSUPPORTED;
  }
  if (rows == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 2048 ? 512 : dim >= 512 ? 256 : 128;
  const size_t smem = (size_t)dim * sizeof(float);
  if (smem > 200 * 1024) {
    set_error("hyper_mix_norm: rows of %d numbers", dim);
    return LL_ERR_UNSUPPORTED;
  }
#define LL_HYPER(TA, SM)                                                                                                            \
  {                                                                                                                                 \
    static bool sized = false;                                                                                                      \
    if (!sized && smem > 48 * 1024) {                                                                                               \
      LL_CUDA(cudaFuncSetAttribute(hyper_mix_norm_kernel<TA, SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));        \
      sized = true;                                                                                                                 \
    }                                                                                                                               \
    hyper_mix_norm_kernel<TA, SM><<<rows, threads, smem, st>>>(src, src_row, src_copy, X, (const TA*)y, ls, r, mix, w_out, w_in, w, eps, \
                                                              h, h_f32, total, S, dim);                                             \
  }
#define LL_HYPER_S(TA)                                                                                                              \
  if (S == 1) LL_HYPER(TA, 1) else if (S == 2) LL_HYPER(TA, 2) else if (S <= 4) LL_HYPER(TA, 4) else LL_HYPER(TA, 8)
  if (act_dtype == LL_F32) {
    LL_HYPER_S(float)
  } else if (act_dtype == LL_BF16) {
    LL_HYPER_S(__nv_bfloat16)
  } else {
    set_error("hyper_mix_norm: unsupported dtype %d", act_dtype);
    return LL_ERR_UNSUPPORTED;
  }
#undef LL_HYPER_S
#undef LL_HYPER
  LL_LAUNCH_OK("hyper_mix_norm_kernel");
  return LL_OK;
}

int ll_row_norm(const void* x, int x_stride, const float* w, float eps, void* out, int out_stride, int dtype, int rows, int dim,
                ll_stream stream) {
  LL_CHECK_ARG(x && out && rows >= 0 && dim > 0 && x_stride >= dim && out_stride >= dim, "bad row_norm arguments");
  if (rows == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 1024 ? 256 : dim >= 256 ? 128 : 64;
  if (dtype == LL_F32) row_norm_kernel<float><<<rows, threads, 0, st>>>((const float*)x, x_stride, w, eps, (float*)out, out_stride, dim);
  else if (dtype == LL_BF16)
    row_norm_kernel<__nv_bfloat16><<<rows, threads, 0, st>>>((const __nv_bfloat16*)x, x_stride, w, eps, (__nv_bfloat16*)out, out_stride,
                                                            dim);
  else {
    set_error("row_norm: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("row_norm_kernel");
  return LL_OK;
}

int ll_sigmoid_gate_mul(const void* a, int a_stride, const void* gate, int gate_stride, void* out, int out_stride, int dtype, int rows,
                        int C, ll_stream stream) {
  LL_CHECK_ARG(a && gate && out && rows >= 0 && C > 0, "bad sigmoid_gate_mul arguments");
  const size_t n = (size_t)rows * C;
  if (n == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == LL_F32)
    sigmoid_gate_mul_kernel<float><<<blocks, 256, 0, st>>>((const float*)a, a_stride, (const float*)gate, gate_stride, (float*)out,
                                                          out_stride, C, n);
  else if (dtype == LL_BF16)
    sigmoid_gate_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)a, a_stride, (const __nv_bfloat16*)gate,
                                                                  gate_stride, (__nv_bfloat16*)out, out_stride, C, n);
  else {
    set_error("sigmoid_gate_mul: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("sigmoid_gate_mul_kernel");
  return LL_OK;
}

int ll_tanh_cap(float* x, float cap, size_t n, ll_stream stream) {
  LL_CHECK_ARG(x && cap > 0.f, "bad tanh_cap arguments");
  if (n == 0) return LL_OK;
  tanh_cap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, cap, 1.f / cap, n);
  LL_LAUNCH_OK("tanh_cap_kernel");
  return LL_OK;
}

int ll_add_norm_pair(float* x, const void* a0, float s0, const void* a1, float s1, const void* a2, float s2, const float* w1,
                     const float* w2, float eps, void* out1, int out1_f32, void* out2, int act_dtype, int rows, int dim,
                     ll_stream stream) {
  LL_CHECK_ARG(x && rows >= 0 && dim > 0 && (!out1 || w1) && (!out2 || w2), "bad add_norm_pair arguments");
  if (rows == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = dim >= 2048 ? 512 : dim >= 512 ? 256 : 128;
  if (act_dtype == LL_F32)
    add_norm_pair_kernel<float><<<rows, threads, 0, st>>>(x, (const float*)a0, s0, (const float*)a1, s1, (const float*)a2, s2, w1, w2,
                                                         eps, out1, out1_f32, (float*)out2, dim);
  else if (act_dtype == LL_BF16)
    add_norm_pair_kernel<__nv_bfloat16><<<rows, threads, 0, st>>>(x, (const __nv_bfloat16*)a0, s0, (const __nv_bfloat16*)a1, s1,
                                                                 (const __nv_bfloat16*)a2, s2, w1, w2, eps, out1, out1_f32,
                                                                 (__nv_bfloat16*)out2, dim);
  else {
    set_error("add_norm_pair: unsupported dtype %d", act_dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("add_norm_pair_kernel");
  return LL_OK;
}

int ll_gated_group_norm(const float* y, int y_gs, const float* stab, const void* gate, int gate_stride, const float* w, int w_shared,
                        float eps, int groups, int gate_first, int gate_sigmoid, void* out, int act_dtype, int rows, int C,
                        ll_stream stream) {
  LL_CHECK_ARG(y && gate && w && out && rows >= 0 && C > 0 && groups > 0 && C % groups == 0 && gate_stride >= C,
               "bad gated_group_norm arguments");
  if (y_gs == 0) y_gs = C / groups;
  LL_CHECK_ARG(y_gs >= C / groups + (stab ? 1 : 0), "gated_group_norm: a part of y is shorter than the part it norms");
  if (rows == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = groups >= 8 ? 256 : groups >= 4 ? 128 : 32 * groups;
  if (act_dtype == LL_F32)
    gated_group_norm_kernel<float><<<rows, threads, 0, st>>>(y, y_gs, stab, (const float*)gate, gate_stride, w, w_shared, eps, groups,
                                                            gate_first, gate_sigmoid, (float*)out, C);
  else if (act_dtype == LL_BF16)
    gated_group_norm_kernel<__nv_bfloat16><<<rows, threads, 0, st>>>(y, y_gs, stab, (const __nv_bfloat16*)gate, gate_stride, w, w_shared,
                                                                    eps, groups, gate_first, gate_sigmoid, (__nv_bfloat16*)out, C);
  else {
    set_error("gated_group_norm: unsupported dtype %d", act_dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("gated_group_norm_kernel");
  return LL_OK;
}

int ll_relu_squared(void* h, int dtype, size_t n, ll_stream stream) {
  LL_CHECK_ARG(h, "relu_squared: null pointer");
  if (n == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == LL_F32) relu_squared_kernel<float><<<blocks, 256, 0, st>>>((float*)h, n);
  else if (dtype == LL_BF16) relu_squared_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)h, n);
  else {
    set_error("relu_squared: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("relu_squared_kernel");
  return LL_OK;
}

int ll_gelu(void* h, int dtype, int tanh_form, size_t n, ll_stream stream) {
  LL_CHECK_ARG(h, "gelu: null pointer");
  if (n == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == LL_F32) gelu_kernel<float><<<blocks, 256, 0, st>>>((float*)h, tanh_form, n);
  else if (dtype == LL_BF16) gelu_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)h, tanh_form, n);
  else {
    set_error("gelu: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("gelu_kernel");
  return LL_OK;
}

}  // extern "C"
