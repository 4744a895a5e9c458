// Softmax attention with rotary positions over a ring of key / value rows, with the variations as parameters:
//
//   prepare   q, k <- [rmsnorm over the WHOLE projection row * w]  ->  rotation of the first `rot_dims` dimensions of every head
//             (dimension i paired with i + rot_dims/2, angle = position * freq[i], all fp32)  ->  q rows out, k rows into the
//             ring at slot position % ring; the value rows are a projection of their own or the keys BEFORE rotation.
//   attend    s_h(i, j) = scale * q_h(i).k_g(j),  optionally cap * tanh(s / cap);
//             key j visible to query i when j <= i, (window == 0 or i - j < window), (chunk == 0 or j / chunk == i / chunk);
//             softmax over the visible keys, optionally with exp(sink_h) added to the denominator (a key without a value);
//             o_h(i) = sum_j w(i, j) v_g(j), optionally times sigmoid(gate) element by element.
//
// Query head h reads key / value head g = h / (H / G).  Scores, softmax and the weighted sums are fp32 in every form; the
// tensor-core form (prompts in bf16) rounds the softmax weights to bf16 as the operand of P.V, which is the only place.
//
//   maps      a head may carry `maps` score maps (1 or 2): its query row is [map 0 | map 1] (dim each), the key row of head g
//             likewise, and every map is a softmax attention of its own over the SAME value row of head g.  Two maps are
//             combined as a difference, o = a_0 - lambda * a_1, then divided by the root mean square of o over the head's
//             values (eps inside the root) and multiplied by `post`; the gate, if any, follows.
#include "common.cuh"

namespace llb {

// ---------------------------------------------------------------------------------------------------------------- prepare
constexpr int QP_THREADS = 256;

__device__ __forceinline__ float qp_block_sum(float v, float* red) {
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

// One row of `heads` heads of `dim`: optional whole-row norm, rotation, store to `out` (row of heads * dim); `plain`
// (optional) gets the row as it is before the rotation (after the norm).
template <typename T>
__device__ __forceinline__ void qp_row(const T* __restrict__ x, const float* __restrict__ nw, float eps, const float* __restrict__ freq,
                                       int rot_dims, float pos, int heads, int dim, T* __restrict__ out, T* __restrict__ plain,
                                       float* red) {
  const int n = heads * dim, half = rot_dims >> 1;
  float kn = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = dt<T>::ld(x, i);
      ss += v * v;
    }
    ss = qp_block_sum(ss, red);
    kn = 1.f / sqrtf(ss / (float)n + eps);
  }
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int i = idx % dim;
    float a = dt<T>::ld(x, idx) * kn;
    if (nw) a *= nw[idx];
    if (plain) dt<T>::st(plain, idx, a);
    if (i < rot_dims) {
      const bool lower = i < half;
      const int mate = lower ? idx + half : idx - half;
      float b = dt<T>::ld(x, mate) * kn;
      if (nw) b *= nw[mate];
      float sn, cs;
      sincosf(pos * freq[lower ? i : i - half], &sn, &cs);
      a = lower ? a * cs - b * sn : a * cs + b * sn;
    }
    dt<T>::st(out, idx, a);
  }
}

template <typename T>
__global__ void __launch_bounds__(QP_THREADS) qk_rotary_append_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride, const T* __restrict__ v, int v_stride,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, const float* __restrict__ freq, int rot_dims,
    const int32_t* __restrict__ pos_ids, T* __restrict__ q_out, T* __restrict__ kc, T* __restrict__ vc, int Tn, int H, int G, int dim,
    int vdim, int ring, int maps) {
  __shared__ float red[32];
  const int m = blockIdx.x, b = m / Tn, t = m - b * Tn;
  const int p = pos_ids[t];
  const float pos = (float)p;
  const int HM = H * maps, GM = G * maps;      // head rows of the q and k projections; the values have G
  if (q) qp_row<T>(q + (size_t)m * q_stride, q_norm, eps, freq, rot_dims, pos, HM, dim, q_out + (size_t)m * HM * dim, nullptr, red);
  if (!k) return;
  const size_t slot = (size_t)b * ring + (size_t)(p % ring);
  T* vrow = vc + slot * (size_t)G * vdim;
  qp_row<T>(k + (size_t)m * k_stride, k_norm, eps, freq, rot_dims, pos, GM, dim, kc + slot * (size_t)GM * dim, v ? nullptr : vrow, red);
  if (v)
    for (int i = threadIdx.x; i < G * vdim; i += blockDim.x) vrow[i] = v[(size_t)m * v_stride + i];
}

// ---------------------------------------------------------------------------------------------------------------- attend, fp32 form
// A warp owns one (query, head); its four groups of eight lanes take every fourth visible key, the eight lanes of a group
// split the head's dimensions in runs of eight (one 16-byte load in bf16).  Every group keeps a running (max, sum, weighted
// sum); the groups are merged at the end.  With splits > 1 a query's keys are cut into that many ranges (blockIdx.y), each
// leaving its (max, sum, weighted sum) in scratch for the merge kernel: decoding one token over a long cache then fills the
// device.
constexpr int SA_WARPS = 4;

// score maps per head and how two of them meet: o = a_0 - lambda * a_1, o / sqrt(mean(o^2) + eps) * post
struct DiffMaps {
  int maps;
  float lambda, post, eps;
};

template <typename T>
__device__ __forceinline__ void sa_load8(const T* __restrict__ row, int e0, int n, bool vec, float (&o)[8]);
template <>
__device__ __forceinline__ void sa_load8<float>(const float* __restrict__ row, int e0, int n, bool vec, float (&o)[8]) {
  if (vec && e0 + 8 <= n) {
    const float4 a = *(const float4*)(row + e0), b = *(const float4*)(row + e0 + 4);
    o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = e0 + i < n ? row[e0 + i] : 0.f;
  }
}
template <>
__device__ __forceinline__ void sa_load8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ row, int e0, int n, bool vec, float (&o)[8]) {
  if (vec && e0 + 8 <= n) {
    const uint4 u = *(const uint4*)(row + e0);
    o[0] = bf16_bits_to_f32(u.x & 0xffffu), o[1] = bf16_bits_to_f32(u.x >> 16);
    o[2] = bf16_bits_to_f32(u.y & 0xffffu), o[3] = bf16_bits_to_f32(u.y >> 16);
    o[4] = bf16_bits_to_f32(u.z & 0xffffu), o[5] = bf16_bits_to_f32(u.z >> 16);
    o[6] = bf16_bits_to_f32(u.w & 0xffffu), o[7] = bf16_bits_to_f32(u.w >> 16);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = e0 + i < n ? __bfloat162float(row[e0 + i]) : 0.f;
  }
}

__device__ __forceinline__ int sa_first_visible(int i, int window, int chunk) {
  int lo = 0;
  if (window > 0) lo = max(lo, i - window + 1);
  if (chunk > 0) lo = max(lo, (i / chunk) * chunk);
  return lo;
}

// R / RV: runs of 64 dimensions a head's keys / values span (dim <= 64 R, vdim <= 64 RV).
template <typename T, int R, int RV>
__global__ void __launch_bounds__(SA_WARPS * 32) softmax_attn_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ gate, int gate_stride, const T* __restrict__ kc, const T* __restrict__ vc,
    const int32_t* __restrict__ pos_ids, const float* __restrict__ sink, float scale, float softcap, int Tn, int H, int G, int dim,
    int vdim, int window, int chunk, int ring, int splits, int maps, int pairs, float* __restrict__ part_ml,
    float* __restrict__ part_acc, T* __restrict__ y) {
  // a warp owns one (query, head, map); with one map per head, h below is the head itself
  const int pair = blockIdx.x * SA_WARPS + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;
  const int HM = H * maps;
  const int m = pair / HM, h = pair - m * HM, head = h / maps, g = head / (H / G);
  const int GK = G * maps, gk = g * maps + (h - head * maps);
  const int b = m / Tn, t = m - b * Tn;
  const int i = pos_ids[t];
  const int lo = sa_first_visible(i, window, chunk);
  const int nvis = i - lo + 1;
  const int per = (nvis + splits - 1) / splits;
  const int j0 = lo + blockIdx.y * per, j1 = min(i + 1, j0 + per);
  const bool kvec = (dim & 7) == 0, vvec = (vdim & 7) == 0;
  float qr[R][8];
  const T* qrow = q + (size_t)m * q_stride + (size_t)h * dim;
#pragma unroll
  for (int r = 0; r < R; ++r) sa_load8<T>(qrow, r * 64 + sub * 8, dim, kvec && ((q_stride | (h * dim)) & 7) == 0, qr[r]);
  float acc[RV][8];
#pragma unroll
  for (int r = 0; r < RV; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
  float mx = -INFINITY, l = 0.f;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const T* kbase = kc + ((size_t)b * ring * GK + gk) * dim;
  const T* vbase = vc + ((size_t)b * ring * G + g) * vdim;
  const unsigned gmask = 0xffu << (grp * 8);
  for (int j = j0 + grp; j < j1; j += 4) {
    const size_t slot = (size_t)(j % ring);
    const T* krow = kbase + slot * GK * dim;
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float kk[8];
      sa_load8<T>(krow, r * 64 + sub * 8, dim, kvec, kk);
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(qr[r][e], kk[e], s);
    }
    s += __shfl_xor_sync(gmask, s, 1);          // the groups' trip counts differ: only the group's own lanes meet here
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    s *= scale;
    if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
    const float mn = fmaxf(mx, s);
    const float corr = expf(mx - mn), p = expf(s - mn);
    mx = mn;
    l = l * corr + p;
    const T* vrow = vbase + slot * G * vdim;
#pragma unroll
    for (int r = 0; r < RV; ++r) {
      float vv[8];
      sa_load8<T>(vrow, r * 64 + sub * 8, vdim, vvec, vv);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(p, vv[e], acc[r][e] * corr);
    }
  }
  // the four groups of the warp hold disjoint keys: merge them (lanes 8 and 16 apart hold the same dimensions).  The
  // trip counts differ between groups, so the shuffles wait until the whole warp is here.
  __syncwarp();
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, mx, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mn = fmaxf(mx, m2);
    const float c1 = mx == -INFINITY ? 0.f : expf(mx - mn), c2 = m2 == -INFINITY ? 0.f : expf(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int r = 0; r < RV; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a2 = __shfl_xor_sync(0xffffffffu, acc[r][e], o);
        acc[r][e] = acc[r][e] * c1 + a2 * c2;
      }
    mx = mn;
  }
  if (splits > 1 || maps > 1) {                  // several maps meet in the merge kernel, also when the keys are not split
    const size_t at = (size_t)pair * splits + blockIdx.y;
    if (lane == 0) part_ml[at * 2] = mx, part_ml[at * 2 + 1] = l;
    if (grp == 0) {
#pragma unroll
      for (int r = 0; r < RV; ++r)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = r * 64 + sub * 8 + e;
          if (c < vdim) part_acc[at * vdim + c] = acc[r][e];
        }
    }
    return;
  }
  if (grp != 0) return;
  float den = l;
  if (sink) {
    const float sk = sink[h];
    const float mn = fmaxf(mx, sk);
    const float c1 = expf(mx - mn);
    den = l * c1 + expf(sk - mn);
#pragma unroll
    for (int r = 0; r < RV; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[r][e] *= c1;
  }
  const float inv = 1.f / den;
#pragma unroll
  for (int r = 0; r < RV; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = r * 64 + sub * 8 + e;
      if (c < vdim) {
        float o = acc[r][e] * inv;
        if (gate) o *= 1.f / (1.f + expf(-dt<T>::ld(gate, (size_t)m * gate_stride + (size_t)h * vdim + c)));
        dt<T>::st(y, (size_t)m * H * vdim + (size_t)h * vdim + c, o);
      }
    }
}

// Merge of the key ranges of one (query, head), in order; a warp per pair, a lane per value dimension.  The weight of every
// range (e^(m_s - m) / denominator) is formed once, a lane per range, and kept in shared memory, so that the sums over the
// ranges are loads that do not wait for one another.  With two maps per head the warp merges both and combines them:
// o = a_0 - lambda * a_1, o / sqrt(mean(o^2) + eps) * post.
constexpr int SA_MAX_SPLITS = 64;
template <typename T>
__global__ void softmax_attn_merge_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_acc,
                                          const T* __restrict__ gate, int gate_stride, const float* __restrict__ sink, int H, int vdim,
                                          int splits, int maps, float lambda, float post, float eps, int pairs, T* __restrict__ y) {
  __shared__ float wsp[4][2][SA_MAX_SPLITS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (blockDim.x >> 5) + warp;      // (query, head)
  if (pair >= pairs) return;
  const int m = pair / H, h = pair - m * H;
  for (int mp = 0; mp < maps; ++mp) {
    const size_t sp = (size_t)pair * maps + mp;  // the (query, head, map) the attention kernel numbered
    const float snk = sink ? sink[(size_t)h * maps + mp] : -INFINITY;
    float ms[SA_MAX_SPLITS / 32], ls[SA_MAX_SPLITS / 32];
    float mx = snk;
#pragma unroll
    for (int e = 0; e < SA_MAX_SPLITS / 32; ++e) {
      const int sidx = lane + e * 32;
      ms[e] = sidx < splits ? part_ml[(sp * splits + sidx) * 2] : -INFINITY;
      ls[e] = sidx < splits ? part_ml[(sp * splits + sidx) * 2 + 1] : 0.f;
      mx = fmaxf(mx, ms[e]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float den = 0.f;
#pragma unroll
    for (int e = 0; e < SA_MAX_SPLITS / 32; ++e) {
      ms[e] = ms[e] == -INFINITY ? 0.f : expf(ms[e] - mx);
      den += ls[e] * ms[e];
    }
    den = warp_sum(den);
    if (sink) den += expf(snk - mx);
    const float wgt = (mp == 0 ? 1.f : -lambda) / den;
#pragma unroll
    for (int e = 0; e < SA_MAX_SPLITS / 32; ++e)
      if (lane + e * 32 < splits) wsp[warp][mp][lane + e * 32] = ms[e] * wgt;
  }
  __syncwarp();
  float ov[8];                                   // vdim <= 256: up to eight values per lane
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int c = lane + e * 32;
    float o = 0.f;
    if (c < vdim)
      for (int mp = 0; mp < maps; ++mp) {
        const float* acc = part_acc + ((size_t)pair * maps + mp) * splits * vdim + c;
        for (int s2 = 0; s2 < splits; ++s2) o = fmaf(acc[(size_t)s2 * vdim], wsp[warp][mp][s2], o);
      }
    ov[e] = o;
  }
  float k = 1.f;
  if (maps > 1) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += ov[e] * ov[e];
    ss = warp_sum(ss);
    k = post / sqrtf(ss / (float)vdim + eps);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int c = lane + e * 32;
    if (c >= vdim) continue;
    float o = ov[e] * k;
    if (gate) o *= 1.f / (1.f + expf(-dt<T>::ld(gate, (size_t)m * gate_stride + (size_t)h * vdim + c)));
    dt<T>::st(y, (size_t)m * H * vdim + (size_t)h * vdim + c, o);
  }
}

template <typename T, int R, int RV>
static int sa_launch(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc,
                     const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int Tn, int H, int G, int dim,
                     int vdim, int window, int chunk, int ring, int splits, const DiffMaps& dm, float* scratch, void* y,
                     cudaStream_t st) {
  const int pairs = B * Tn * H * dm.maps;
  float* part_ml = scratch;
  float* part_acc = scratch ? scratch + (size_t)pairs * splits * 2 : nullptr;
  const dim3 grid((pairs + SA_WARPS - 1) / SA_WARPS, splits);
  softmax_attn_kernel<T, R, RV><<<grid, SA_WARPS * 32, 0, st>>>((const T*)q, q_stride, (const T*)gate, gate_stride, (const T*)kc,
                                                               (const T*)vc, pos_ids, sink, scale, softcap, Tn, H, G, dim, vdim, window,
                                                               chunk, ring, splits, dm.maps, pairs, part_ml, part_acc, (T*)y);
  LL_LAUNCH_OK("softmax_attn_kernel");
  if (splits > 1 || dm.maps > 1) {
    const int heads = B * Tn * H;
    softmax_attn_merge_kernel<T><<<(heads + 3) / 4, 128, 0, st>>>(part_ml, part_acc, (const T*)gate, gate_stride, sink, H, vdim, splits,
                                                                 dm.maps, dm.lambda, dm.post, dm.eps, heads, (T*)y);
    LL_LAUNCH_OK("softmax_attn_merge_kernel");
  }
  return LL_OK;
}

template <typename T>
static int sa_dispatch(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc,
                       const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int Tn, int H, int G, int dim,
                       int vdim, int window, int chunk, int ring, int splits, const DiffMaps& dm, float* scratch, void* y,
                       cudaStream_t st) {
  const int r = dim <= 64 ? 1 : dim <= 128 ? 2 : 4, rv = vdim <= 64 ? 1 : vdim <= 128 ? 2 : 4;
#define LL_SA(RR, RRV)                                                                                                              \
  if (r == RR && rv == RRV)                                                                                                         \
    return sa_launch<T, RR, RRV>(q, q_stride, gate, gate_stride, kc, vc, pos_ids, sink, scale, softcap, B, Tn, H, G, dim, vdim, window, \
                                 chunk, ring, splits, dm, scratch, y, st);
  LL_SA(1, 1) LL_SA(1, 2) LL_SA(1, 4) LL_SA(2, 1) LL_SA(2, 2) LL_SA(2, 4) LL_SA(4, 1) LL_SA(4, 2) LL_SA(4, 4)
#undef LL_SA
  return LL_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------------- attend, tensor-core form
// Prompts in bf16 (mma.sync m16n8k16, fp32 accumulation).  A block of four warps owns 64 consecutive queries of one head,
// 16 per warp, whose fragments stay in registers; the keys the tile can see are walked 64 at a time through shared memory
// (cp.async into two stages, the next tile under the current one's math; rows found by position % ring, dimensions beyond
// the rows' sizes zero-filled up to DK / DV).  S = Q K^T, then scale,
// cap and mask on the accumulator fragments, an online softmax per row in fp32, and O += P V with the weights split into
// two bf16 terms p = hi + lo (two products), so that what meets the values carries 16 bits of the fp32 weight and not 8.
// The sink joins the denominator and the gate multiplies the output in the epilogue.
constexpr int TM_Q = 64, TM_K = 64, TM_THREADS = 128;

__device__ __forceinline__ void tm_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void tm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void tm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
// (hi, lo) bf16 pairs of two fp32 numbers: hi = bf16(x), lo = bf16(x - hi)
__device__ __forceinline__ void tm_split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
  const __nv_bfloat16 l0 = __float2bfloat16_rn(x0 - __bfloat162float(h0)), l1 = __float2bfloat16_rn(x1 - __bfloat162float(h1));
  hi = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
}

// tanh from one fast exponential and one fast division (relative error about 1e-6 of the result for arguments of order one,
// 1e-4 for arguments of 1e-3: far below the 2^-9 of the bf16 operands this form works on)
__device__ __forceinline__ float tm_tanh(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }

// MAPS = 2: the block walks its keys once per map (queries and keys of the map, the same values) and keeps the first map's
// normalised output in registers until the second is there; the difference, its unit norm and `post` are the epilogue.
// DK / DV: the padded sizes of a key row and of a value row (a map's keys may be half as wide as the values).
template <int DK, int DV, int MAPS>
__global__ void __launch_bounds__(TM_THREADS, MAPS == 1 ? 3 : 2) softmax_attn_mma_kernel(
    const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ gate, int gate_stride,
    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc, const int32_t* __restrict__ pos_ids,
    const float* __restrict__ sink, float scale, float softcap, int Tn, int H, int G, int dim, int vdim, int window, int chunk, int ring,
    float lambda, float post, float eps, __nv_bfloat16* __restrict__ y) {
  constexpr int LD = DK + 8, CH = DK / 8, LV = DV + 8, CV = DV / 8, STAGE = TM_K * (LD + LV);      // a stage: 64 key rows, then 64 value rows
  extern __shared__ __align__(16) unsigned char tm_smem[];
  __nv_bfloat16* const stages = (__nv_bfloat16*)tm_smem;
  __nv_bfloat16* Ks = stages;                                       // (the queries pass through stage 0 first)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // late query tiles walk the most keys: they are launched first, so that the long blocks do not end up as the tail
  const int t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * TM_Q, h = blockIdx.y, b = blockIdx.z, g = h / (H / G);
  const int nq = min(TM_Q, Tn - t0);
  const int p0 = pos_ids[t0];                    // a step's positions are consecutive
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  const int qp[2] = {p0 + warp * 16 + (lane >> 2), p0 + warp * 16 + (lane >> 2) + 8};
  const int qlo[2] = {sa_first_visible(qp[0], window, chunk), sa_first_visible(qp[1], window, chunk)};
  const int wlo = sa_first_visible(p0 + warp * 16, window, chunk), whi = p0 + warp * 16 + 15;     // what the warp's rows can see
  const int khi = p0 + nq - 1;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int wlo_last = sa_first_visible(whi, window, chunk);
  const int kt0 = sa_first_visible(p0, window, chunk);
  const __nv_bfloat16* vbase = vc + ((size_t)b * ring * G + g) * vdim;
  float first[MAPS == 1 ? 1 : DV / 8][4];         // the first map's output, rows and columns as in o
#pragma unroll 1
  for (int mp = 0; mp < MAPS; ++mp) {
  const int hq = h * MAPS + mp, GK = G * MAPS;
  Ks = stages;
  for (int c = tid; c < TM_Q * CH; c += TM_THREADS) {
    const int r = c / CH, ch = c - r * CH;
    uint4 val = zero4;
    if (r < nq && ch * 8 < dim) val = *(const uint4*)(q + ((size_t)b * Tn + t0 + r) * q_stride + (size_t)hq * dim + ch * 8);
    *(uint4*)&Ks[r * LD + ch * 8] = val;
  }
  __syncthreads();
  uint32_t qf[DK / 16][4];
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk) tm_ldmatrix_x4(qf[kk], &Ks[(warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8]);
  __syncthreads();
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const __nv_bfloat16* kbase = kc + ((size_t)b * ring * GK + (g * MAPS + mp)) * dim;
  // the next tile's rows are copied under the current tile's math: two stages, one cp.async group per tile
  auto load_tile = [&](int kt, int st) {
    __nv_bfloat16* Kd = stages + st * STAGE;
    __nv_bfloat16* Vd = Kd + TM_K * LD;
    for (int c = tid; c < TM_K * CH; c += TM_THREADS) {
      const int r = c / CH, ch = c - r * CH;
      const int j = kt + r;
      const size_t slot = (size_t)(j % ring);
      if (j <= khi && ch * 8 < dim) tm_cp_async16(&Kd[r * LD + ch * 8], kbase + slot * GK * dim + ch * 8);
      else *(uint4*)&Kd[r * LD + ch * 8] = zero4;
    }
    for (int c = tid; c < TM_K * CV; c += TM_THREADS) {
      const int r = c / CV, ch = c - r * CV;
      const int j = kt + r;
      const size_t slot = (size_t)(j % ring);
      if (j <= khi && ch * 8 < vdim) tm_cp_async16(&Vd[r * LV + ch * 8], vbase + slot * G * vdim + ch * 8);
      else *(uint4*)&Vd[r * LV + ch * 8] = zero4;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_tile(kt0, 0);
  int st = 0;
  for (int kt = kt0; kt <= khi; kt += TM_K, st ^= 1) {
    if (kt + TM_K <= khi) {
      load_tile(kt + TM_K, st ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    Ks = stages + st * STAGE;
    const __nv_bfloat16* Vs = Ks + TM_K * LD;
    // every key of the tile is visible to every row of the warp: no mask to apply
    const bool full = kt >= wlo_last && kt + TM_K - 1 <= p0 + warp * 16;
    if (kt <= whi && kt + TM_K - 1 >= wlo) {       // else: nothing in this tile that a row of this warp sees
      float sc[TM_K / 8][4];
#pragma unroll
      for (int n = 0; n < TM_K / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < TM_K / 16; ++np) {
          uint32_t bf[4];
          tm_ldmatrix_x4(bf, &Ks[(np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8]);
          mma_bf16_16816(sc[2 * np], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bf[0], bf[1]);
          mma_bf16_16816(sc[2 * np + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], bf[2], bf[3]);
        }
      }
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < TM_K / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rr = e >> 1;
          const int kp = kt + n * 8 + (lane & 3) * 2 + (e & 1);
          float v = sc[n][e] * scale;
          if (softcap > 0.f) v = softcap * tm_tanh(v * inv_cap);
          if (!full) v = (kp <= qp[rr] && kp >= qlo[rr]) ? v : -INFINITY;
          sc[n][e] = v;
          tmax[rr] = fmaxf(tmax[rr], v);
        }
      float corr[2], msafe[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
        const float mn = fmaxf(mrow[rr], tmax[rr]);
        msafe[rr] = mn == -INFINITY ? 0.f : mn;
        corr[rr] = __expf(mrow[rr] - msafe[rr]);
        mrow[rr] = mn;
        lrow[rr] *= corr[rr];
      }
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) o[n][0] *= corr[0], o[n][1] *= corr[0], o[n][2] *= corr[1], o[n][3] *= corr[1];
#pragma unroll
      for (int n = 0; n < TM_K / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pw = __expf(sc[n][e] - msafe[e >> 1]);
          sc[n][e] = pw;
          lrow[e >> 1] += pw;
        }
#pragma unroll
      for (int ks = 0; ks < TM_K / 16; ++ks) {
        uint32_t ah[4], al[4];
        tm_split2(sc[2 * ks][0], sc[2 * ks][1], ah[0], al[0]);
        tm_split2(sc[2 * ks][2], sc[2 * ks][3], ah[1], al[1]);
        tm_split2(sc[2 * ks + 1][0], sc[2 * ks + 1][1], ah[2], al[2]);
        tm_split2(sc[2 * ks + 1][2], sc[2 * ks + 1][3], ah[3], al[3]);
#pragma unroll
        for (int dp = 0; dp < DV / 16; ++dp) {
          uint32_t bf[4];
          tm_ldmatrix_x4_trans(bf, &Vs[(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LV + dp * 16 + (lane >> 4) * 8]);
          mma_bf16_16816(o[2 * dp], ah[0], ah[1], ah[2], ah[3], bf[0], bf[1]);
          mma_bf16_16816(o[2 * dp + 1], ah[0], ah[1], ah[2], ah[3], bf[2], bf[3]);
          mma_bf16_16816(o[2 * dp], al[0], al[1], al[2], al[3], bf[0], bf[1]);
          mma_bf16_16816(o[2 * dp + 1], al[0], al[1], al[2], al[3], bf[2], bf[3]);
        }
      }
    }
    __syncthreads();
  }
  float fin[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    lrow[rr] += __shfl_xor_sync(0xffffffffu, lrow[rr], 1);
    lrow[rr] += __shfl_xor_sync(0xffffffffu, lrow[rr], 2);
    float den = lrow[rr], c1 = 1.f;
    if (sink) {
      const float sk = sink[hq];
      const float mn = fmaxf(mrow[rr], sk);
      c1 = expf(mrow[rr] - mn);
      den = lrow[rr] * c1 + expf(sk - mn);
    }
    fin[rr] = den > 0.f ? c1 / den : 0.f;
  }
  if (MAPS == 2) {
    if (mp == 0) {
#pragma unroll
      for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) first[MAPS == 1 ? 0 : n][e] = o[n][e] * fin[e >> 1];
      continue;                                  // (the loop's last barrier has passed: stage 0 is free for the next queries)
    }
    float ss[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d = first[MAPS == 1 ? 0 : n][e] - lambda * (o[n][e] * fin[e >> 1]);
        o[n][e] = d;                             // columns from vdim on hold zeros: the value rows are zero-filled there
        ss[e >> 1] += d * d;
      }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      ss[rr] += __shfl_xor_sync(0xffffffffu, ss[rr], 1);
      ss[rr] += __shfl_xor_sync(0xffffffffu, ss[rr], 2);
      fin[rr] = post / sqrtf(ss[rr] / (float)vdim + eps);
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = warp * 16 + (lane >> 2) + rr * 8;
    if (r >= nq) continue;
    const float f = fin[rr];
    const size_t m = (size_t)b * Tn + t0 + r;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      const int c = n * 8 + (lane & 3) * 2;
      if (c < vdim) {                            // vdim is a multiple of 8: the pair is inside together
        float v0 = o[n][rr * 2] * f, v1 = o[n][rr * 2 + 1] * f;
        if (gate) {
          const __nv_bfloat162 gg = *(const __nv_bfloat162*)(gate + m * gate_stride + (size_t)h * vdim + c);
          v0 *= 1.f / (1.f + expf(-__bfloat162float(gg.x)));
          v1 *= 1.f / (1.f + expf(-__bfloat162float(gg.y)));
        }
        *(__nv_bfloat162*)(y + m * H * vdim + (size_t)h * vdim + c) = __floats2bfloat162_rn(v0, v1);
      }
    }
  }
  }  // maps
}

template <int DK, int DV, int MAPS>
static int tm_launch(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, const int32_t* pos_ids,
                     const float* sink, float scale, float softcap, int B, int Tn, int H, int G, int dim, int vdim, int window, int chunk,
                     int ring, const DiffMaps& dm, void* y, cudaStream_t st) {
  const dim3 grid((Tn + TM_Q - 1) / TM_Q, H, B);
  constexpr int smem = 2 * TM_K * (DK + 8 + DV + 8) * (int)sizeof(__nv_bfloat16);
  static bool sized = false;
  if (!sized) {
    LL_CUDA(cudaFuncSetAttribute(softmax_attn_mma_kernel<DK, DV, MAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    sized = true;
  }
  softmax_attn_mma_kernel<DK, DV, MAPS><<<grid, TM_THREADS, smem, st>>>(
      (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)gate, gate_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
      pos_ids, sink, scale, softcap, Tn, H, G, dim, vdim, window, chunk, ring, dm.lambda, dm.post, dm.eps, (__nv_bfloat16*)y);
  LL_LAUNCH_OK("softmax_attn_mma_kernel");
  return LL_OK;
}

// The tensor-core form takes bf16 heads of up to 128 dimensions in multiples of 8 (16-byte rows), gates and queries on
// 4-byte / 16-byte boundaries.
static bool tm_supported(int dtype, int T, int dim, int vdim, int q_stride, int gate_stride, int splits) {
  return dtype == LL_BF16 && splits == 1 && T >= 16 && dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && vdim <= 128 && q_stride % 8 == 0 &&
         gate_stride % 2 == 0;
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_qk_rotary_append_maps(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                             const float* q_norm, const float* k_norm, float eps, const float* freq, int rot_dims,
                             const int32_t* pos_ids, void* q_out, void* kc, void* vc, int B, int T, int H, int G, int dim, int vdim,
                             int ring, int maps, ll_stream stream) {
  LL_CHECK_ARG((q || k) && (!q || q_out) && pos_ids && B >= 0 && T >= 0 && H > 0 && dim > 0 && maps >= 1,
               "bad qk_rotary_append arguments");
  LL_CHECK_ARG(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq), "qk_rotary_append: bad rotation");
  LL_CHECK_ARG(!k || (kc && vc && G > 0 && vdim > 0 && ring > 0), "qk_rotary_append: keys need their ring");
  LL_CHECK_ARG(!k || v || (vdim == dim && maps == 1), "qk_rotary_append: values taken from the keys have the keys' size");
  if (B == 0 || T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LL_F32)
    qk_rotary_append_kernel<float><<<B * T, QP_THREADS, 0, st>>>((const float*)q, q_stride, (const float*)k, k_stride, (const float*)v,
                                                                v_stride, q_norm, k_norm, eps, freq, rot_dims, pos_ids, (float*)q_out,
                                                                (float*)kc, (float*)vc, T, H, G, dim, vdim, ring, maps);
  else if (dtype == LL_BF16)
    qk_rotary_append_kernel<__nv_bfloat16><<<B * T, QP_THREADS, 0, st>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, q_norm, k_norm, eps,
        freq, rot_dims, pos_ids, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, T, H, G, dim, vdim, ring, maps);
  else {
    set_error("qk_rotary_append: unsupported dtype %d", dtype);
    return LL_ERR_UNSUPPORTED;
  }
  LL_LAUNCH_OK("qk_rotary_append_kernel");
  return LL_OK;
}

int ll_qk_rotary_append(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                        const float* q_norm, const float* k_norm, float eps, const float* freq, int rot_dims,
                        const int32_t* pos_ids, void* q_out, void* kc, void* vc, int B, int T, int H, int G, int dim, int vdim, int ring,
                        ll_stream stream) {
  LL_CHECK_ARG(q, "bad qk_rotary_append arguments");
  return ll_qk_rotary_append_maps(q, q_stride, k, k_stride, v, v_stride, dtype, q_norm, k_norm, eps, freq, rot_dims, pos_ids, q_out, kc,
                                  vc, B, T, H, G, dim, vdim, ring, 1, stream);
}

int ll_softmax_attn_tensor_form(int dtype, int T, int dim, int vdim, int q_stride, int gate_stride, int splits) {
  return tm_supported(dtype, T, dim, vdim, q_stride, gate_stride, splits) ? 1 : 0;
}

size_t ll_softmax_attn_scratch_bytes(int M, int H, int vdim, int splits) {
  if (splits < 1) return 16;
  return (size_t)M * H * splits * (2 + (size_t)vdim) * sizeof(float);
}

int ll_softmax_attn_maps(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                         const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int T, int H, int G, int dim,
                         int vdim, int window, int chunk, int ring, int splits, int form, int maps, float diff_lambda, float diff_post,
                         float eps, float* scratch, void* y, ll_stream stream) {
  LL_CHECK_ARG(q && kc && vc && pos_ids && y, "softmax_attn: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && ring > 0 && window >= 0 && chunk >= 0 &&
                   splits >= 1 && splits <= SA_MAX_SPLITS && (maps == 1 || maps == 2),
               "bad softmax_attn arguments");
  if (dim > 256 || vdim > 256) {
    set_error("softmax_attn: heads of %d / %d dimensions (up to 256)", dim, vdim);
    return LL_ERR_UNSUPPORTED;
  }
  if (B == 0 || T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const DiffMaps dm{maps, diff_lambda, diff_post, eps};
  if (form == 0 && tm_supported(dtype, T, dim, vdim, q_stride, gate ? gate_stride : 0, splits)) {
    const int d = dim > vdim ? dim : vdim;
    if (maps == 1) {           // one map: key and value rows padded alike
#define LL_TM(DD)                                                                                                                   \
  if (d <= DD)                                                                                                                      \
    return tm_launch<DD, DD, 1>(q, q_stride, gate, gate_stride, kc, vc, pos_ids, sink, scale, softcap, B, T, H, G, dim, vdim, window, \
                                chunk, ring, dm, y, st);
      LL_TM(32) LL_TM(64) LL_TM(96) LL_TM(128)
#undef LL_TM
    }
#define LL_TM2(KK, VV)                                                                                                              \
  if (dim <= KK && vdim <= VV)                                                                                                      \
    return tm_launch<KK, VV, 2>(q, q_stride, gate, gate_stride, kc, vc, pos_ids, sink, scale, softcap, B, T, H, G, dim, vdim, window, \
                                chunk, ring, dm, y, st);
#define LL_TM2_ROW(KK) LL_TM2(KK, 32) LL_TM2(KK, 64) LL_TM2(KK, 96) LL_TM2(KK, 128)
    LL_TM2_ROW(32) LL_TM2_ROW(64) LL_TM2_ROW(96) LL_TM2_ROW(128)
#undef LL_TM2_ROW
#undef LL_TM2
  }
  LL_CHECK_ARG(scratch || (splits == 1 && maps == 1), "softmax_attn: split key ranges and several maps meet in scratch memory");
  if (dtype == LL_F32)
    return sa_dispatch<float>(q, q_stride, gate, gate_stride, kc, vc, pos_ids, sink, scale, softcap, B, T, H, G, dim, vdim, window, chunk,
                              ring, splits, dm, scratch, y, st);
  if (dtype == LL_BF16)
    return sa_dispatch<__nv_bfloat16>(q, q_stride, gate, gate_stride, kc, vc, pos_ids, sink, scale, softcap, B, T, H, G, dim, vdim, window,
                                      chunk, ring, splits, dm, scratch, y, st);
  set_error("softmax_attn: unsupported dtype %d", dtype);
  return LL_ERR_UNSUPPORTED;
}

int ll_softmax_attn(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                    const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int T, int H, int G, int dim,
                    int vdim, int window, int chunk, int ring, int splits, int form, float* scratch, void* y, ll_stream stream) {
  return ll_softmax_attn_maps(q, q_stride, gate, gate_stride, kc, vc, dtype, pos_ids, sink, scale, softcap, B, T, H, G, dim, vdim,
                              window, chunk, ring, splits, form, 1, 0.f, 1.f, 0.f, scratch, y, stream);
}

}  // extern "C"
