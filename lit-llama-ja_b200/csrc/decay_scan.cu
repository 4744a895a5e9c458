// Linear recurrence with a diagonal decay: the state of selective state-space layers (one decay per head and token) and
// of gated linear attention (one decay per key channel and token).  Per sequence b and head h, with S an n x p matrix:
//
//   S_t[i][c] = a_t[i] * S_(t-1)[i][c] + (ks_t * k_t[i]) * v_t[c]
//   y_t[c]    = qs * sum_i q_t[i] * S_t[i][c]  +  skip[h] * v_t[c]
//
// q, k (n per head; `qk_heads` heads shared by consecutive groups of heads) and v (p per head) are column slices of
// projection outputs in the activation dtype; a (the decay itself, in (0, 1]), ks and skip are fp32; S and y are fp32 and
// every product and sum is fp32.  The state is carried in `state[B][H][n][p]`; a sequence at position 0 starts from zero
// whatever the state holds.
//
// unit_col: the LAST of the p columns of every head is not in memory but the constant 1 (v then holds p - 1 columns per
// head).  That column of S is the running sum of the keys alone and that column of y its product with the query: the
// normaliser of a matrix memory, carried by the same walk.
#include "common.cuh"

namespace llb {

constexpr int DS_THREADS = 128;
// tokens staged per round (fewer when a head's state rows are many, so that the staging stays small)
__host__ __device__ constexpr int ds_tc(int npad) { return npad <= 64 ? 16 : npad <= 128 ? 8 : npad <= 256 ? 4 : 2; }

// grid (p tiles, H, B).  NP threads (consecutive lanes) share one column c and split the n rows; PT = DS_THREADS / NP
// columns per block.  A thread's rows are interleaved in quads, row(k, e) = (k * NP + part) * 4 + e, so that the NP lanes of
// a column read consecutive 16-byte units of the staged token (no bank conflicts).
// DS_NL: state rows a thread keeps in registers (8: more threads per head, the usual case; 16: heads of more than 256 rows).
// PERCH: a decay per state row (gated linear attention); otherwise one per head and token, read once per token.
template <typename T, int NP, int DS_NL, bool PERCH>
__global__ void __launch_bounds__(DS_THREADS) decay_scan_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride, const T* __restrict__ v, int v_stride,
    const float* __restrict__ a, int a_per_channel, const float* __restrict__ ks, const float* __restrict__ skip, float qs,
    float* __restrict__ state, const int32_t* __restrict__ pos_ids, float* __restrict__ y, int Tn, int H, int qk_heads, int n,
    int p, int vw) {
  constexpr int PT = DS_THREADS / NP;
  constexpr int NPAD = NP * DS_NL;
  constexpr int DS_TC = ds_tc(NPAD);
  __shared__ __align__(16) float s_a[DS_TC][NPAD], s_k[DS_TC][NPAD], s_q[DS_TC][NPAD];
  __shared__ float s_v[DS_TC][PT];
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (H / qk_heads);
  const int part = threadIdx.x % NP, pl = threadIdx.x / NP;
  const int c = blockIdx.x * PT + pl;
  const bool live = c < p;
  float S[DS_NL];
#define DS_ROW(i) ((((i) >> 2) * NP + part) * 4 + ((i) & 3))
  float* sp = state + (((size_t)b * H + h) * n) * p;
  const bool fresh = pos_ids[0] == 0;
#pragma unroll
  for (int i = 0; i < DS_NL; ++i) S[i] = (!fresh && live && DS_ROW(i) < n) ? sp[(size_t)DS_ROW(i) * p + c] : 0.f;
  const float sk = skip ? skip[h] : 0.f;
  // The next round's tokens are fetched into registers while this round's are consumed from shared memory.
  constexpr int IT = DS_TC * NPAD / DS_THREADS, VIT = (DS_TC * PT + DS_THREADS - 1) / DS_THREADS;
  // (raw values only: nothing may depend on a load before the round that consumes it, or the fetch would wait for it)
  float ra[IT], rs[IT];
  T rk[IT], rq[IT], rv[VIT];
  auto fetch = [&](int t0) {
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int idx = it * DS_THREADS + threadIdx.x;
      const int tt = idx / NPAD, i = idx - tt * NPAD;
      const size_t m = (size_t)b * Tn + t0 + tt;
      const bool ok = t0 + tt < Tn && i < n;
      ra[it] = ok ? (a_per_channel ? a[(m * H + h) * n + i] : a[m * H + h]) : 1.f;
      rs[it] = (ok && ks) ? ks[m * H + h] : 1.f;
      rk[it] = k[ok ? m * k_stride + (size_t)g * n + i : 0];
      rq[it] = q[ok ? m * q_stride + (size_t)g * n + i : 0];
    }
#pragma unroll
    for (int it = 0; it < VIT; ++it) {
      const int idx = it * DS_THREADS + threadIdx.x;
      const int tt = idx / PT, cc = idx - tt * PT;
      const int col = blockIdx.x * PT + cc;
      const bool ok = tt < DS_TC && t0 + tt < Tn && col < vw;
      rv[it] = v[ok ? ((size_t)b * Tn + t0 + tt) * v_stride + (size_t)h * vw + col : 0];
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < Tn; t0 += DS_TC) {
    const int nt = min(DS_TC, Tn - t0);
    __syncthreads();
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int idx = it * DS_THREADS + threadIdx.x;
      const int tt = idx / NPAD, i = idx - tt * NPAD;
      const bool ok = t0 + tt < Tn && i < n;
      s_a[tt][i] = ra[it];
      s_k[tt][i] = ok ? dt<T>::ld(&rk[it], 0) * rs[it] : 0.f;
      s_q[tt][i] = ok ? dt<T>::ld(&rq[it], 0) * qs : 0.f;
    }
#pragma unroll
    for (int it = 0; it < VIT; ++it) {
      const int idx = it * DS_THREADS + threadIdx.x;
      const int tt = idx / PT, cc = idx - tt * PT;
      if (tt < DS_TC) {
        const int col = blockIdx.x * PT + cc;
        s_v[tt][cc] = (t0 + tt < Tn && col < p) ? (col < vw ? dt<T>::ld(&rv[it], 0) : 1.f) : 0.f;
      }
    }
    __syncthreads();
    if (t0 + DS_TC < Tn) fetch(t0 + DS_TC);
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = s_v[tt][pl];
      float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
      const float a1 = s_a[tt][0];
#pragma unroll
      for (int i4 = 0; i4 < DS_NL; i4 += 4) {
        const int at = ((i4 >> 2) * NP + part) * 4;
        const float4 a4 = PERCH ? *(const float4*)&s_a[tt][at] : make_float4(a1, a1, a1, a1);
        const float4 k4 = *(const float4*)&s_k[tt][at];
        const float4 q4 = *(const float4*)&s_q[tt][at];
        S[i4 + 0] = a4.x * S[i4 + 0] + k4.x * vv;
        S[i4 + 1] = a4.y * S[i4 + 1] + k4.y * vv;
        S[i4 + 2] = a4.z * S[i4 + 2] + k4.z * vv;
        S[i4 + 3] = a4.w * S[i4 + 3] + k4.w * vv;
        c0 += q4.x * S[i4 + 0];
        c1 += q4.y * S[i4 + 1];
        c2 += q4.z * S[i4 + 2];
        c3 += q4.w * S[i4 + 3];
      }
      float acc = (c0 + c1) + (c2 + c3);
#pragma unroll
      for (int o = NP / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (part == 0 && live) y[((size_t)b * Tn + t0 + tt) * ((size_t)H * p) + (size_t)h * p + c] = acc + sk * vv;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DS_NL; ++i)
      if (DS_ROW(i) < n) sp[(size_t)DS_ROW(i) * p + c] = S[i];
  }
#undef DS_ROW
}

template <typename T, int NP, int NL>
static int decay_scan_launch(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, const float* a,
                             int a_per_channel, const float* ks, const float* skip, float qs, float* state, const int32_t* pos_ids,
                             float* y, int B, int Tn, int H, int qk_heads, int n, int p, int vw, cudaStream_t st) {
  constexpr int PT = DS_THREADS / NP;
  const dim3 grid((p + PT - 1) / PT, H, B);
  if (a_per_channel)
    decay_scan_kernel<T, NP, NL, true><<<grid, DS_THREADS, 0, st>>>((const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, a, 1,
                                                                    ks, skip, qs, state, pos_ids, y, Tn, H, qk_heads, n, p, vw);
  else
    decay_scan_kernel<T, NP, NL, false><<<grid, DS_THREADS, 0, st>>>((const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, a, 0,
                                                                     ks, skip, qs, state, pos_ids, y, Tn, H, qk_heads, n, p, vw);
  LL_LAUNCH_OK("decay_scan_kernel");
  return LL_OK;
}

// Step sizes and decays of a selective state-space layer: dt = softplus(raw + dt_bias[h]) (no clamp),
// decay = exp(-exp(a_log[h]) * dt); raw is a column slice of the input projection's output.
template <typename T>
__global__ void ssm_gates_kernel(const T* __restrict__ raw, int stride, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ dt_out, float* __restrict__ decay, int H,
                                 size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / H;
  const int h = (int)(i - m * H);
  const float z = dt<T>::ld(raw, m * stride + h) + dt_bias[h];
  const float d = z > 20.f ? z : log1pf(expf(z));
  dt_out[i] = d;
  decay[i] = expf(-expf(a_log[h]) * d);
}

// Decay per key channel of gated linear attention: sigmoid(z + bias)^(1/tau) = exp(-softplus(-(z + bias)) / tau).
template <typename T>
__global__ void channel_decay_kernel(const T* __restrict__ z, int stride, const float* __restrict__ bias, float inv_tau,
                                     float* __restrict__ out, int C, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / C;
  const int c = (int)(i - m * C);
  const float u = -(dt<T>::ld(z, m * stride + c) + (bias ? bias[c] : 0.f));
  const float sp = u > 20.f ? u : log1pf(expf(u));
  out[i] = expf(-sp * inv_tau);
}

// Exponential gates of a matrix memory with a running stabiliser.  Per (sequence, head), with raw_i / raw_f column slices
// of the input projection's output, li = cap(raw_i + bi), lf = logsigmoid(cap(raw_f + bf)), cap(z) = c tanh(z / c) (c <= 0:
// no cap), and mx carried from token to token (0 at a sequence's start, not minus infinity):
//   mx_t = max(lf_t + mx_(t-1), li_t);   keep_t = exp(lf_t + mx_(t-1) - mx_t);   take_t = exp(li_t - mx_t)
// A block owns one (sequence, head) and takes MG_THREADS tokens a round, one per thread.  Token t acts on the stabiliser as
// the map mx -> max(mx + lf_t, li_t); two such maps compose to one of the same form, (F, M) then (F', M') = (F + F',
// max(M + F', M')), so a warp composes its 32 maps by a shuffle scan (five steps), the warps' totals meet in shared memory,
// and every thread applies what lies before it to the round's incoming mx.  Every token's keep uses as mx_(t-1) exactly the
// value its left neighbour reports as mx_t: the recurrence the walk then runs is consistent, and what it computes does not
// depend on the stabiliser's rounding.  The transcendental part (cap, log sigmoid, exponentials) of a round's tokens runs
// in parallel; only the few compositions per round are sequential.
constexpr int MG_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(MG_THREADS) matrix_memory_gates_kernel(
    const T* __restrict__ raw_i, const T* __restrict__ raw_f, int stride, const float* __restrict__ bias_i,
    const float* __restrict__ bias_f, float cap, float* __restrict__ mstate, const int32_t* __restrict__ pos_ids,
    float* __restrict__ keep, float* __restrict__ take, float* __restrict__ stab, int Tn, int H) {
  constexpr int NW = MG_THREADS / 32;
  __shared__ float wF[2][NW], wM[2][NW];
  const int w = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = w / H, h = w - b * H;
  float mx = pos_ids[0] == 0 ? 0.f : mstate[w];
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv = cap > 0.f ? 1.f / cap : 0.f;
  auto fetch = [&](int t, float& zi, float& zf) {
    const bool ok = t < Tn;
    const size_t m = (size_t)b * Tn + (ok ? t : 0);
    zi = ok ? dt<T>::ld(raw_i, m * stride + h) : 0.f;
    zf = ok ? dt<T>::ld(raw_f, m * stride + h) : 0.f;
  };
  float ni, nf;
  fetch(threadIdx.x, ni, nf);
  int buf = 0;
  for (int t0 = 0; t0 < Tn; t0 += MG_THREADS, buf ^= 1) {
    const int t = t0 + threadIdx.x;
    float zi = ni + bi, zf = nf + bf;
    if (t0 + MG_THREADS < Tn) fetch(t + MG_THREADS, ni, nf);   // the next round's loads fly under this round's scan
    if (cap > 0.f) zi = cap * tanhf(zi * inv), zf = cap * tanhf(zf * inv);
    const float li = t < Tn ? zi : -INFINITY;                  // tokens past the end are the identity map (F = 0, M = -inf)
    const float lf = t < Tn ? fminf(zf, 0.f) - log1pf(expf(-fabsf(zf))) : 0.f;       // log sigmoid
    float F = lf, M = li;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float pF = __shfl_up_sync(0xffffffffu, F, d), pM = __shfl_up_sync(0xffffffffu, M, d);
      if (lane >= d) {
        M = fmaxf(pM + F, M);
        F = pF + F;
      }
    }
    if (lane == 31) wF[buf][warp] = F, wM[buf][warp] = M;
    __syncthreads();                                           // (the other buffer is free again: its readers passed this barrier a round ago)
    float m_in = mx, m_out = mx;
#pragma unroll
    for (int ww = 0; ww < NW; ++ww) {
      m_out = fmaxf(m_out + wF[buf][ww], wM[buf][ww]);
      if (ww + 1 == warp) m_in = m_out;
    }
    const float my_new = fmaxf(m_in + F, M);
    float my_prev = __shfl_up_sync(0xffffffffu, my_new, 1);
    if (lane == 0) my_prev = m_in;
    if (t < Tn) {
      const size_t o = ((size_t)b * Tn + t) * H + h;
      keep[o] = expf(lf + my_prev - my_new);
      take[o] = expf(li - my_new);
      stab[o] = my_new;
    }
    mx = m_out;
  }
  if (threadIdx.x == 0) mstate[w] = mx;
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_decay_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype, const float* a,
                  int a_per_channel, const float* ks, const float* skip, float qs, float* state, const int32_t* pos_ids, float* y,
                  int B, int T, int H, int qk_heads, int n, int p, int unit_col, ll_stream stream) {
  LL_CHECK_ARG(q && k && v && a && state && pos_ids && y, "decay_scan: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && H > 0 && qk_heads > 0 && H % qk_heads == 0 && n > 0 && p > (unit_col ? 1 : 0),
               "bad decay_scan arguments");
  const int vw = unit_col ? p - 1 : p;
  if (n > 32 * 16) {
    set_error("decay_scan: %d state rows per head (up to %d)", n, 32 * 16);
    return LL_ERR_UNSUPPORTED;
  }
  if (B == 0 || T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // 16 rows per thread when that already gives half of the SMs a block (each block stages its head's tokens: fewer blocks,
  // less staging); 8 rows when the heads are few, so that twice as many warps share the latency of the sequential walk
  int np16 = 1;
  while (np16 * 16 < n) np16 *= 2;
  const long long blocks16 = (long long)B * H * ((p + DS_THREADS / np16 - 1) / (DS_THREADS / np16));
  const int nl = (n > 256 || 2 * blocks16 >= sm_count()) ? 16 : 8;
  int np = 1;
  while (np * nl < n) np *= 2;
#define LL_DS(TT, NP)                                                                                                                 \
  return nl == 8 ? decay_scan_launch<TT, NP, 8>(q, q_stride, k, k_stride, v, v_stride, a, a_per_channel, ks, skip, qs, state, pos_ids, \
                                                y, B, T, H, qk_heads, n, p, vw, st)                                                        \
                 : decay_scan_launch<TT, NP, 16>(q, q_stride, k, k_stride, v, v_stride, a, a_per_channel, ks, skip, qs, state, pos_ids, \
                                                 y, B, T, H, qk_heads, n, p, vw, st)
#define LL_DS_T(TT)                 \
  switch (np) {                     \
    case 1: LL_DS(TT, 1);           \
    case 2: LL_DS(TT, 2);           \
    case 4: LL_DS(TT, 4);           \
    case 8: LL_DS(TT, 8);           \
    case 16: LL_DS(TT, 16);         \
    default: LL_DS(TT, 32);         \
  }
  if (dtype == LL_F32) { LL_DS_T(float) }
  if (dtype == LL_BF16) { LL_DS_T(__nv_bfloat16) }
#undef LL_DS_T
#undef LL_DS
  set_error("decay_scan: unsupported dtype %d", dtype);
  return LL_ERR_UNSUPPORTED;
}

int ll_ssm_gates(const void* raw, int dtype, int stride, const float* dt_bias, const float* a_log, float* dt_out, float* decay,
                 int M, int H, ll_stream stream) {
  LL_CHECK_ARG(raw && dt_bias && a_log && dt_out && decay && M >= 0 && H > 0 && stride >= H, "bad ssm_gates arguments");
  const size_t total = (size_t)M * H;
  if (total == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == LL_F32) ssm_gates_kernel<float><<<blocks, 256, 0, st>>>((const float*)raw, stride, dt_bias, a_log, dt_out, decay, H, total);
  else if (dtype == LL_BF16)
    ssm_gates_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)raw, stride, dt_bias, a_log, dt_out, decay, H, total);
  else {
    set_error("ssm_gates: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("ssm_gates_kernel");
  return LL_OK;
}

int ll_channel_decay(const void* z, int dtype, int stride, const float* bias, float tau, float* out, int M, int C,
                     ll_stream stream) {
  LL_CHECK_ARG(z && out && M >= 0 && C > 0 && stride >= C && tau > 0.f, "bad channel_decay arguments");
  const size_t total = (size_t)M * C;
  if (total == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == LL_F32) channel_decay_kernel<float><<<blocks, 256, 0, st>>>((const float*)z, stride, bias, 1.f / tau, out, C, total);
  else if (dtype == LL_BF16)
    channel_decay_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)z, stride, bias, 1.f / tau, out, C, total);
  else {
    set_error("channel_decay: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("channel_decay_kernel");
  return LL_OK;
}

int ll_matrix_memory_gates(const void* raw_i, const void* raw_f, int dtype, int stride, const float* bias_i, const float* bias_f,
                           float cap, float* mstate, const int32_t* pos_ids, float* keep, float* take, float* stab, int B, int T, int H,
                           ll_stream stream) {
  LL_CHECK_ARG(raw_i && raw_f && mstate && pos_ids && keep && take && stab && B >= 0 && T >= 0 && H > 0 && stride >= H,
               "bad matrix_memory_gates arguments");
  if (B == 0 || T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)(B * H);
  if (dtype == LL_F32)
    matrix_memory_gates_kernel<float><<<blocks, MG_THREADS, 0, st>>>((const float*)raw_i, (const float*)raw_f, stride, bias_i, bias_f, cap,
                                                                    mstate, pos_ids, keep, take, stab, T, H);
  else if (dtype == LL_BF16)
    matrix_memory_gates_kernel<__nv_bfloat16><<<blocks, MG_THREADS, 0, st>>>((const __nv_bfloat16*)raw_i, (const __nv_bfloat16*)raw_f,
                                                                            stride, bias_i, bias_f, cap, mstate, pos_ids, keep, take,
                                                                            stab, T, H);
  else {
    set_error("matrix_memory_gates: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("matrix_memory_gates_kernel");
  return LL_OK;
}

}  // extern "C"
