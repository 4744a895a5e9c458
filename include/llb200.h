/*
 * llb200 - B200-native (sm_100a) kernels for lit-llama-ja's quantized-inference hot path.
 *
 * Drop-in boundary: a C-ABI shared library (plain pointers and sizes, no torch types).
 * Every pointer is a DEVICE pointer unless it says "host".  Every call enqueues work on
 * `stream` (a cudaStream_t passed as void*) and returns immediately; nothing synchronises.
 * Return value: LL_OK or a negative LL_ERR_* code; ll_last_error() then holds a message
 * (thread-local).  Nothing throws across this boundary.
 *
 * "ref:" citations are into /root/reference (if001/lit-llama-ja); each entry point names
 * the reference interface it replaces.  The reference has no native code on this path: its
 * FFI-equivalent is the Triton launcher + the PyTorch fallback inside
 * lit_llama/quantization.py, bitsandbytes for llm.int8, and ATen ops in lit_llama/model.py.
 */
#ifndef LLB200_H
#define LLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LL_ABI_VERSION 15

#define LL_OK 0
#define LL_ERR_ARG (-1)         /* bad shape / dtype / null pointer */
#define LL_ERR_CUDA (-2)        /* a CUDA runtime/driver call failed */
#define LL_ERR_UNSUPPORTED (-3) /* valid request this build has no kernel for */

/* element types of activation / parameter buffers */
#define LL_F32 0
#define LL_BF16 1
#define LL_F16 2

typedef void* ll_stream; /* cudaStream_t */

#if defined(__GNUC__)
#define LL_API __attribute__((visibility("default")))
#else
#define LL_API
#endif

LL_API const char* ll_last_error(void);
LL_API int ll_abi_version(void);
/* number of SMs of the current device (host query; <0 on error) */
LL_API int ll_sm_count(void);

/* ---------------------------------------------------------------------------------------
 * GPTQ column-block storage (ref: lit_llama/quantization.py:339-372).
 *   qw      uint8, logical [N][K/epb], MEMORY [K/epb][N] (N fastest) - the reference's
 *           column-major buffer, used in place.  epb = 8/bits; entry nr of a byte sits at
 *           bit nr*bits (bits=4: even k = low nibble).
 *   scales, zeros  [N][G] row-major, G = ceil(K/tile); tile_cols = -1 means tile = K.
 * ------------------------------------------------------------------------------------- */

/* ref: ColBlockQuantizedLinear.pack_weight, quantization.py:374-388.  Bit-exact: per group,
 * in the weight dtype, `/= scale` then `+= zero`, clamp [0, 2^bits-1], TRUNCATE to uint8. */
LL_API int ll_pack_weight(const void* weight /*[N][K]*/, int weight_dtype, const void* scales, const void* zeros,
                   int param_dtype, uint8_t* qw, int N, int K, int bits, int tile_cols, ll_stream stream);

/* ref: ColBlockQuantizedLinear.get_weight, quantization.py:390-409.  Bit-exact: code as float,
 * `-= zero`, `*= scale`, each rounded to out_dtype.  out is [N][K] row-major. */
LL_API int ll_get_weight(const uint8_t* qw, const void* scales, const void* zeros, int param_dtype, void* out,
                  int out_dtype, int N, int K, int bits, int tile_cols, ll_stream stream);

/* ref: ColBlockQuantizedLinear.forward, quantization.py:411-421 (both branches), any M, bits in
 * {4,8}, any tile, fp32 or bf16 activations: y[M][N] = x[M][K] . W^T (+ bias), W as get_weight
 * would produce it in the activation dtype, fp32 accumulation, one rounding on store.
 * SIMT kernel: the always-correct path for shapes/dtypes the tensor-core kernels do not take. */
LL_API int ll_qlinear_simt(const void* x, int act_dtype, int M, const uint8_t* qw, const void* scales, const void* zeros,
                    int param_dtype, const void* bias, void* y, int N, int K, int bits, int tile_cols,
                    ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * int4 decode GEMV (M <= 8), bf16 activations.  Replaces the Triton launcher
 * qlinear_4bit_weight (quantization.py:282-331: pads M to 256, per-row scales only) and the
 * dequantise-then-F.linear fallback (quantization.py:420-421) for grouped scales.
 *
 * The kernel streams a one-time REPACK of the checkpoint bytes ("stream"): blocks of
 * 16 output columns x KB input features (KB = 128, 64 or 32 = gcd-style divisor of the group
 * size), each block = the 32 lanes' mma.m16n8k16 A-fragments in issue order followed by the
 * block's 16 (scale, -(16+zero)) bf16 pairs.  Blocks are ordered (tile, k-block), k fastest,
 * so any contiguous range of work items is one contiguous byte range (1-D bulk TMA).
 * Arithmetic: y = sum_blocks scale * (sum_k (16+q) x_k - (16+zero) sum_k x_k), products exact,
 * fp32 accumulation: the exact (q - zero) * scale of the reference's Triton kernel
 * (quantization.py:247-251) without its TF32 rounding or the fallback's bf16 weight rounding.
 * ------------------------------------------------------------------------------------- */

/* bytes of the repacked stream for an [N][K] int4 matrix with scale groups of `group` columns
 * (group = K for per-row); 0 if the shape is not supported by the GEMV (use ll_qlinear_simt). */
LL_API size_t ll_int4_stream_bytes(int N, int K, int group);

/* One-time repack: qw (checkpoint layout) + scales/zeros [N][K/group] -> stream.  status[0]
 * (device int32) is set to 1 unless every scale and every (16 + zero) is exactly representable
 * in bf16 (then the caller must use ll_qlinear_simt). */
LL_API int ll_int4_prepare(const uint8_t* qw, const void* scales, const void* zeros, int param_dtype, uint8_t* stream_out,
                    int N, int K, int group, int kind, int32_t* status, ll_stream stream);

/* Stream kinds (same size, same tile / block order; they differ in how a block's nibbles are arranged):
 *   LL_STREAM_BF16: words are mma.m16n8k16 bf16 A fragments (nibble i at bit 3 + 4 i); tail (scale, -(16 + zero)); M = 1..8.
 *   LL_STREAM_U8:   words are mma.m16n8k32 u8 A fragment pairs (column g in the low nibbles, g + 8 in the high nibbles);
 *                   tail (scale, -zero); the batch-1 decode kernel (activations as four exact base-256 digit planes).
 * ll_int4_stream_kind() names the kind the GEMV wants for a shape and batch: prepare that one and pass it in
 * ll_gemv_args.stream_kind. */
#define LL_STREAM_BF16 0
#define LL_STREAM_U8 1
LL_API int ll_int4_stream_kind(int N, int K, int group, int M);

/* GPTQ 8-bit weights (`gptq.int8`: ColBlockQuantizedLinear(bits=8), ref utils.py:182-184, quantization.py:343-347; the
 * reference serves it only through get_weight + F.linear, quantization.py:420-421).  Stream kind LL_STREAM_W8 of the same
 * batch-1 GEMV (ll_int4_gemv with stream_kind = LL_STREAM_W8, M = 1, group % 128 == 0): a block is 16 columns x 128 k
 * bytes laid out as the lanes' u8 mma.m16n8k32 A-fragment registers + the (scale, -zero) tail, so the main loop is loads and
 * MMAs only; activations as the four exact base-256 digit planes.  qw: the checkpoint buffer, logical [N][K], memory [K][N].
 * status as in ll_int4_prepare. */
#define LL_STREAM_W8 2
LL_API size_t ll_q8_stream_bytes(int N, int K, int group);
LL_API int ll_q8_gemv_supported(int N, int K, int group, int nmat, int M); /* 1 / 0 */
LL_API int ll_q8_prepare(const uint8_t* qw, const void* scales, const void* zeros, int param_dtype, uint8_t* stream_out, int N,
                  int K, int group, int32_t* status, ll_stream stream);

#define LL_EPI_STORE 0    /* y = bf16(acc (+bias)) */
#define LL_EPI_RESIDUAL 1 /* y (residual stream, in place) = bf16(y + bf16(acc)) */
#define LL_EPI_ROPE_KV 2  /* c_attn: RoPE on q,k; q -> y, k,v -> KV cache at pos[1] */
#define LL_EPI_SWIGLU 3   /* y = bf16(bf16(silu(bf16(accA))) * bf16(accB)), accB from w2 */
#define LL_EPI_PUSH 4     /* y_r[M][N] = x . W^T on every rank r (peer stores) + arrival counters, see push_dst */

#define LL_GEMV_PDL 1 /* launch with programmatic stream serialization (prologue overlap) */
/* Footprint parity of a batch-1 launch inside a PDL chain (stream kind 1 only).  Consecutive GEMVs of a chain alternate
 * EVEN / ODD: an EVEN launch asks for 116 KB of shared memory (two EVEN CTAs cannot share an SM), an ODD launch carries
 * two idle warps (two ODD CTAs exceed the register file), an EVEN + ODD pair fits - so the block scheduler can never put
 * two CTAs of the SAME GEMV on one SM, whatever else is resident (profiles/r02_gemv_experiments.md section 6). */
#define LL_GEMV_EVEN 4
#define LL_GEMV_ODD 2

typedef struct ll_gemv_args {
  const uint8_t* w;    /* repacked stream from ll_int4_prepare */
  const uint8_t* w2;   /* second matrix (LL_EPI_SWIGLU: c_fc2), same shape; else NULL */
  int32_t N, K, group; /* group = k per scale group (K when per-row) */
  int32_t M;           /* rows of x, 1..8 */
  const void* x;       /* [M][K] bf16 */
  /* optional fused RMSNorm on x (ref: model.py:276-283): x_used = bf16(w * bf16(x * r)),
   * r = bf16(rsqrt(bf16(bf16(sum(bf16(x*x)) / K) + eps))), computed by every CTA from its staged row */
  const void* norm_weight; /* [K] bf16 or NULL */
  float eps;
  int32_t epilogue;
  int32_t flags;
  void* y;          /* see LL_EPI_* ; [M][N] bf16 (ROPE_KV: q [M][N/3]) */
  const void* bias; /* [N] bf16 or NULL (LL_EPI_STORE) */
  /* LL_EPI_ROPE_KV (ref: model.py:204-228, 312-329) */
  const float* rope;  /* [block_size][head_size/2][2] fp32 (cos, sin) */
  const int32_t* pos; /* device int32[3]: rope position, cache slot, #valid slots */
  void* k_cache;      /* [M][n_head][cache_len][head_size] bf16 */
  void* v_cache;
  int32_t n_head, head_size, cache_len;
  int32_t grid; /* 0 = one CTA per SM; >0 forces the CTA count (tests).  CTAs own whole 16-column tiles. */
  /* LL_EPI_PUSH (tensor parallel, row-parallel layer): the bf16 result [M][N] is stored into push_dst[r] for every
   * rank r < push_world (peer-mapped receive buffers, the local one included; y is not used), then every CTA adds 1 to
   * *push_cnt[r] with release semantics at system scope: compute and the first half of the all-reduce in one kernel. */
  uint64_t push_dst[8];
  uint64_t push_cnt[8];
  int32_t push_world;
  int32_t stream_kind; /* LL_STREAM_* of w / w2 (what ll_int4_prepare was asked for) */
  /* Stream kinds 1 / 2 without the fused norm (optional): x already converted by its producer (ll_decode_attn_digits) into the
   * kernel's own staging format - four signed base-256 digit planes [4][K + 16] bytes and [K / 128][4] float records
   * (2^-sh, sum x, 2^(16 - sh), 0) - so that the prologue is two bulk copies.  x is then not read. */
  const uint8_t* x_planes;
  const float* x_rec;
} ll_gemv_args;

/* Host query: LL_OK if the GEMV takes (N, K, group, nmat, M) (LL_ERR_UNSUPPORTED otherwise, e.g. M*K too
 * large for shared memory); *smem_bytes / *ctas (optional) report the launch it would use. */
LL_API int ll_int4_gemv_plan(int N, int K, int group, int nmat, int M, int grid, size_t* smem_bytes, int32_t* ctas);
LL_API int ll_int4_gemv(const ll_gemv_args* args /* host */, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Large-M path (prefill, batched decode): tcgen05 / TMEM / TMA tensor-core GEMM.
 * y[M][N] = x[M][K] . w[N][K]^T (+ bias), all bf16 row-major, fp32 accumulation in TMEM.  With
 * w = ll_get_weight(..., LL_BF16) this is the reference's F.linear(inp, get_weight(inp.dtype), bias)
 * (quantization.py:420-421) and what its Triton kernel (quantization.py:185-331) computes for large M.
 * K % 8 == 0; any M, N (tails are zero-filled by TMA and masked on store).
 * ------------------------------------------------------------------------------------- */
LL_API int ll_gemm_bf16_tc(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, ll_stream stream);

/* Fused int4 de-quantise + GEMM on tcgen05 for 1 <= M <= 128 rows (batched decode, short prefill; the HBM-bound regime):
 * y[M][N] (bf16) = x[M][K] (bf16) . W^T (+ bias), W de-quantised INSIDE the main loop from the packed stream
 * (w_stream = ll_int4_prepare(..., LL_STREAM_U8, ...), the batch-1 GEMV's stream) with the reference's bf16 rounding steps
 * bf16(bf16(q - zero) * scale) (get_weight, ref quantization.py:390-409), fp32 accumulation in tensor memory - the
 * arithmetic of F.linear(inp, get_weight(bf16)) (ref quantization.py:420-421) and the structure of the reference's
 * Triton kernel (de-quantise in the K loop, ref quantization.py:259-267).  N % 128 == 0, group % 128 == 0, K % group == 0.
 * K is split over CTAs to fill the SMs; `scratch` (ll_int4_gemm_tc_scratch_bytes(), may be 0 -> NULL allowed) holds the
 * partial sums, added in a fixed order by a second kernel. */
LL_API size_t ll_int4_gemm_tc_scratch_bytes(int M, int N, int K);
LL_API int ll_int4_gemm_tc(const uint8_t* w_stream, const void* x, const void* bias, void* y, float* scratch, int M, int N,
                           int K, int group, ll_stream stream);

/* No counterpart in the reference: added at the request of the run's operators for callers that cannot call cudaMalloc
 * (code under CUDA-graph capture, tight serving loops, harnesses that forbid it).  Same arithmetic, arguments and result
 * as ll_int4_gemm_tc, but the split-K partial sums go to an array built into the library
 * (LL_INT4_GEMM_TC_STATIC_SCRATCH_BYTES per GPU, held until exit); the call allocates nothing.  Shapes whose
 * ll_int4_gemm_tc_scratch_bytes() exceeds that maximum return LL_ERR_UNSUPPORTED (every 7B layer up to M = 128 fits
 * except the 32000-column head above M = 64).  All calls on a device share the array: calls that overlap on the GPU
 * race; calls ordered on one stream do not (nothing in the array has to start at zero). */
#define LL_INT4_GEMM_TC_STATIC_SCRATCH_BYTES (32u << 20)
LL_API int ll_int4_gemm_tc_static(const uint8_t* w_stream, const void* x, const void* bias, void* y, int M, int N, int K,
                                  int group, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * llm.int8 (ref: Linear8bitLt, quantization.py:36-75; arithmetic = bitsandbytes double_quant / MatMul8bitLt,
 * un-vendored in the reference, restated from arXiv:2208.07339 - see oracle/quant.py).
 * ------------------------------------------------------------------------------------- */

/* ref: Linear8bitLt._quantize_weight, quantization.py:67-75: W.half(), SCB[n] = absmax of row n,
 * CB = rint(127 * W / SCB) int8 [N][K] row-major. */
LL_API int ll_int8_quantize_weight(const void* w /*[N][K]*/, int w_dtype, int8_t* cb, float* scb, int N, int K, ll_stream stream);

/* ref: bnb MatMul8bitLt forward (has_fp16_weights=False, threshold) as reached through quantization.py:36-45:
 * y[M][N] = int8 matmul of the row-quantised non-outlier part + fp16 outlier-column part (+ bias), in the
 * activation dtype.  K % 128 == 0.  workspace: ll_int8_workspace_bytes(min(M, 64), N, K) bytes, 256-byte aligned. */
LL_API size_t ll_int8_workspace_bytes(int M, int N, int K);
/* cbt: CB transposed, int8 [K][N] (optional, NULL = none): with it an outlier column of the weights is one contiguous row
 * read coalesced (the outlier part then costs count * N bytes instead of one 32-byte sector per (row, outlier column)). */
LL_API int ll_int8_linear(const void* x, int act_dtype, const int8_t* cb, const int8_t* cbt, const float* scb, const void* bias,
                   void* y, int M, int N, int K, float threshold, void* workspace, size_t workspace_bytes, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * GPTQ solver, one block of <= 128 columns (ref GPTQQuantizer.quantize, quantization.py:559-590; fp32).
 * W [N][ldw] working weights (columns i1 .. i1+count-1 are read), Hinv [K][ldh] upper Cholesky factor of the inverse
 * Hessian, scales/zeros [N][G] (read for groupsize == -1; written at group starts otherwise - the reference's grouped
 * branch raises at 573-577, its evident intent is implemented), Q [N][ldq] receives the on-grid weights of the block's
 * columns, Err [N][count] the scaled errors for the caller's cross-block update W[:, i2:] -= Err @ Hinv[i1:i2, i2:],
 * loss[N] += sum_i (w - q)^2 / d^2.  Same fp32 operation order as the reference: identical codes for identical Hinv.
 * ------------------------------------------------------------------------------------- */
LL_API int ll_gptq_block(float* W, int ldw, const float* Hinv, int ldh, float* scales, float* zeros, int G, float* Q, int ldq,
                  float* Err, float* loss, int N, int i1, int count, int groupsize, int maxq, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Sampling tail of generate() (ref generate.py:62-75: logits / temperature, top-k mask, softmax, multinomial) as one
 * single-CTA kernel, bf16 logits [V].  l = bf16(logit / temperature); entries below the top_k-th largest l are dropped
 * (ties kept; top_k <= 0 keeps all); p = bf16(softmax(l)); the token is drawn by inverse CDF in index order from the
 * uniform number u[*step]; *step is then incremented.  The token is written to tok[0] (int64: the next step's
 * embedding index) and, when out_tokens is not NULL, to out_tokens[pos[0] + 1].  Same distribution as the reference's
 * torch.multinomial; a different random stream.
 * ------------------------------------------------------------------------------------- */
LL_API int ll_sample_topk(const void* logits, int V, float temperature, int top_k, const float* u, int32_t* step, const int32_t* pos,
                   int64_t* out_tokens, int64_t* tok, ll_stream stream);
/* The same draw followed, in the same kernel, by what ll_advance_pos and ll_embed_ssq do (the engine's sampled step: one
 * launch instead of three before the first GEMV of the next token): pos (int32[3]) is advanced by one position after the
 * token was written to out_tokens[pos[0] + 1] (a position >= max_pos traps, as ll_advance_pos), and the chosen token's row
 * of wte [V][dim] bf16 is copied to x [dim] (ref model.py:110). */
LL_API int ll_sample_advance_embed(const void* logits, int V, float temperature, int top_k, const float* u, int32_t* step,
                            int32_t* pos, int64_t* out_tokens, int64_t* tok, int cache_len, int max_pos, const void* wte,
                            void* x, int dim, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Tensor-parallel exchange (new: the reference is single-device, generate.py:122).  One-shot all-reduce over
 * NVLink peer memory fused with the residual add: x = bf16(x + bf16(sum over ranks of part_r)), summed in rank
 * order on every rank.  peer_parts / peer_flags: HOST arrays of `world` device pointers (symmetric-memory mappings
 * of every rank's partial-sum buffer and int32[world] flag array, zeroed once).  The caller alternates between two
 * partial-sum buffers from call to call.  epoch_counter: local device int32[LL_TP_MAX_CTAS], zero before first use.
 * flags: LL_GEMV_PDL = launch as a link of a programmatic-dependent-launch chain (the next kernel of the stream may start
 * its prologue while the exchange runs; needs the EVEN / ODD GEMV footprints around it), 0 = plain launch. */
#define LL_TP_MAX_CTAS 8
LL_API int ll_tp_allreduce_add(void* x, const uint64_t* peer_parts, const uint64_t* peer_flags, int32_t* epoch_counter, int rank,
                        int world, int n, int flags, ll_stream stream);
/* The same exchange in ONE NVLink traversal: every rank pushes its partial sums `part` ([n] bf16, local) into every peer's
 * receive buffer as 16-byte {word, epoch, word, epoch} units (data and flag in one store, NCCL-LL style) and reads the
 * peers' units from its own memory.  peer_recv: HOST array of `world` device pointers - the symmetric-memory mappings of
 * every rank's receive buffer of ll_tp_ll_recv_bytes(world, n) bytes, zeroed once.  epoch_counter, flags: as above.
 * Same result bits as ll_tp_allreduce_add (rank-order fp32 sum, one bf16 rounding, residual add). */
LL_API size_t ll_tp_ll_recv_bytes(int world, int n);
LL_API int ll_tp_ll_allreduce_add(void* x, const void* part, const uint64_t* peer_recv, int32_t* epoch_counter, int rank, int world,
                           int n, int flags, ll_stream stream);
/* Second half of the pushed exchange (LL_EPI_PUSH): wait until `arrivals` more CTAs have signalled the counter of the
 * current buffer (cnt[j], j alternating 0, 1 from call to call), then x = bf16(x + bf16(sum_r recv[j][r])) from LOCAL
 * memory, rank order.  recv: [2][world][n] bf16 in this rank's symmetric memory; cnt: uint32[2], zero before first use. */
LL_API int ll_tp_reduce_add(void* x, const void* recv, uint32_t* cnt, int32_t* epoch_counter, int world, int n, int arrivals,
                     ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * model.py kernels
 * ------------------------------------------------------------------------------------- */

/* ref: RMSNorm.forward, model.py:276-283 - every intermediate rounded to the activation dtype. */
LL_API int ll_rmsnorm(const void* x, const void* weight, void* y, int dtype, int rows, int dim, float eps, ll_stream stream);

/* ref: wte lookup, model.py:110, fused with the sum-of-squares partials the first fused RMSNorm
 * consumes: x[m][:] = wte[idx[m]][:]; ssq (optional, may be NULL): ssq[m][p] = sum over 16-column tile p of
 * bf16(x*x). */
LL_API int ll_embed_ssq(const void* wte, const int64_t* idx, void* x, float* ssq, int M, int dim, ll_stream stream);

/* ref: apply_rope (model.py:312-329) on q and k of a fused qkv row + KV-cache write (model.py:218-228,
 * in place - the ring slot replaces the reference's roll).  qkv [B][T][3E]; q_out [B][nh][T][hs];
 * caches [B][nh][S][hs]; pos_ids[T] rope rows, slots[T] cache slots (device int32). */
LL_API int ll_rope_kv_append(const void* qkv, const float* rope, const int32_t* pos_ids, const int32_t* slots, void* q_out,
                      void* k_cache, void* v_cache, int dtype, int B, int T, int n_head, int head_size, int cache_len,
                      ll_stream stream);

/* ref: apply_rope, model.py:312-329 (standalone form): x, y [B][T][nh][hs]; rope [T][hs/2][2] fp32 rows
 * already selected for the T positions.  fp32 rotation of interleaved pairs, rounded to dtype. */
LL_API int ll_apply_rope(const void* x, const float* rope, void* y, int dtype, int B, int T, int n_head, int head_size,
                  ll_stream stream);

/* ref: the prefix cross-attention of LLaMA-Adapter, lit_llama/adapter.py:145-165 - the second
 * scaled_dot_product_attention (queries against the adaption prompt's keys/values, all-true mask), the product with
 * the per-head gating factor and the sum with the self-attention output, in one launch:
 *   y[b][t][h][:] = dtype(y[b][t][h][:] + dtype(gate[h] * dtype(softmax(q[b][h][t] . K[h]^T / sqrt(hs)) . V[h])))
 * q [B][nh][T][hs] (rotated, as ll_rope_kv_append leaves it); prefix_k / prefix_v [nh][prompt_len][hs] (one prompt for
 * every batch row, prefix_batched = 0) or [B][nh][prompt_len][hs] (prefix_batched = 1, the reference's repeated
 * layout); gate [nh]; y [B][T][nh*hs] updated in place.  head_size: multiples of 32 up to 256. */
LL_API int ll_adapter_attn_add(const void* q, const void* prefix_k, const void* prefix_v, const void* gate, void* y,
                               int dtype, int B, int n_head, int T, int head_size, int prompt_len, int prefix_batched,
                               ll_stream stream);

/* ref: adapter_v2_new_forward, lit_llama/adapter_v2.py:29-32, applied to a Linear's output y [rows][n]:
 *   out = dtype(scale[c] * dtype(y[r][c] + bias[c]));  out may alias y. */
LL_API int ll_bias_scale(const void* y, const void* bias, const void* scale, void* out, int dtype, size_t rows, int n,
                         ll_stream stream);

/* ref: F.scaled_dot_product_attention over the KV cache for ONE query token per sequence
 * (model.py:237 with T=1): attends slots [0, pos[2]).  q [B][nh][hs]; y [B][nh*hs].
 * Split along the cache (flash-decoding) with a deterministic last-arriver combine.
 * scratch: float [B*nh*splits*(hs+2)], counters int32 [B*nh] (zero; left zero). */
LL_API int ll_decode_attn(const void* q, const void* k_cache, const void* v_cache, const int32_t* pos, void* y, int dtype,
                   int B, int n_head, int head_size, int cache_len, int max_splits, float* scratch,
                   int32_t* counters, int flags, ll_stream stream);
LL_API size_t ll_decode_attn_scratch_bytes(int B, int n_head, int head_size, int max_splits);
/* The same attention (bf16, batch 1, head size 128, a split that fits the K/V-staging kernel: ..._supported() says so) whose
 * per-head leader also writes y in the batch-1 GEMV's staging format: planes [4][plane_stride] bytes (plane_stride =
 * n_head * 128 + 16), rec [n_head][4] floats - one head is one 128-element k-block of attn.c_proj's input
 * (ll_gemv_args.x_planes / x_rec).  Same arithmetic and order as the GEMV's own conversion: identical bits downstream. */
LL_API int ll_decode_attn_digits_supported(int dtype, int B, int head_size, int cache_len, int max_splits);
LL_API int ll_decode_attn_digits(const void* q, const void* k_cache, const void* v_cache, const int32_t* pos, void* y, int B,
                          int n_head, int head_size, int cache_len, int max_splits, int flags, uint8_t* planes, float* rec,
                          int plane_stride, ll_stream stream);

/* ref: MLP.forward's silu(a) * b, model.py:258, rounded like torch (silu -> dtype, product -> dtype). */
LL_API int ll_silu_mul(const void* a, const void* b, void* y, int dtype, size_t n, ll_stream stream);
/* y = dtype(a + b) : the residual adds of Block.forward, model.py:172-173 */
LL_API int ll_add(const void* a, const void* b, void* y, int dtype, size_t n, ll_stream stream);
/* pos[0] += 1; pos[1] = pos[0] % cache_len; pos[2] = min(pos[0] + 1, cache_len): one decode step
 * (ref: generate.py:77 input_pos advance + model.py:221-225 sliding window).  A position outside [0, max_pos)
 * (max_pos = rows of the RoPE table = block_size) traps on the device: the reference's
 * rope_cache.index_select(0, input_pos) raises there (model.py:101). */
LL_API int ll_advance_pos(int32_t* pos, int cache_len, int max_pos, ll_stream stream);
/* pos[0] = input_pos[0] (device int64, the caller's position tensor); pos[1], pos[2] as above.
 * Lets LLaMA.forward(idx, max_seq_length, input_pos) honour an arbitrary input_pos without a
 * host sync (ref: model.py:101-104 index_select by input_pos). */
LL_API int ll_set_pos(int32_t* pos, const int64_t* input_pos, int cache_len, int max_pos, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * A residual stream kept in fp32 whatever the activation dtype (csrc/residual_ops.cu).
 * ------------------------------------------------------------------------------------- */

/* x[m][:] = wte[idx[m]][:] * scale in fp32; x_act (optional) the same in the activation dtype. */
LL_API int ll_embed_scaled(const void* wte, int wte_dtype, const int64_t* idx, float scale, float* x, void* x_act,
                           int act_dtype, int M, int dim, ll_stream stream);

/* Norm on the sublayer's OUTPUT, with a one-number gain (a device scalar), then the residual sum:
 *   r = x + gain * y / sqrt(mean(y^2) + eps)      (x == NULL: r is the normed y alone)
 * r -> out (fp32, optional; may alias x, or be a slot of `stack`).  Then, optionally, the weighted sum over the outputs
 * of all earlier layers:  v = mix_w[n_mix-1] * r + sum_{j < n_mix-1} mix_w[j] * stack[j * stack_stride + ...]
 * (n_mix == 0: v = r).  v -> next (fp32, optional) and next_act (act_dtype, optional).  (y_dtype, act_dtype): both fp32,
 * both bf16, or fp32 y with bf16 activations (the norm of the stream itself). */
LL_API int ll_gain_norm_add_mix(const float* x, const void* y, int y_dtype, const float* gain, float eps, float* out,
                                const float* stack, size_t stack_stride, const float* mix_w, int n_mix, float* next,
                                void* next_act, int act_dtype, int rows, int dim, ll_stream stream);

/* Clamped gated linear unit on the output gu [rows][gu_stride] of a GEMM over a stacked [gate; up] weight:
 *   g = min(gu[c], limit), u = clamp(gu[ff + c], -limit, limit), h[c] = g * sigmoid(alpha * g) * (u + 1). */
LL_API int ll_glu_clamp(const void* gu, int gu_stride, int ff, float limit, float alpha, void* h, int dtype, int rows,
                        ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Latent attention over a ring cache of latent rows (csrc/latent_attn.cu).  A cache row is
 * [c (kv_rank) | k_rot (rot_dim)]; caches are [B][cache_len][kv_rank + rot_dim] in the activation dtype; the slot of
 * position p is p % cache_len.  rope is [positions][rot_dims / 2][2] fp32 (cos, sin); rotation pairs dimension 2i with
 * 2i + 1 on the first rot_dims (even, <= rot_dim) dimensions of the rotated part.  pos_ids [T] device int32: the
 * positions of the step's tokens, the same for every sequence of the batch.
 * ------------------------------------------------------------------------------------- */

/* Row m = b * T + t of proj [B*T][proj_stride] holds at col0 the down-projection [kv_rank | rot_dim]:
 * c = first part / sqrt(mean(first part^2) + eps) * norm_w (fp32 weights), k_rot = rotated second part -> cache row. */
LL_API int ll_latent_kv_append(const void* proj, int dtype, int proj_stride, int col0, const float* norm_w, float eps,
                               const float* rope, const int32_t* pos_ids, void* cache, int B, int T, int kv_rank,
                               int rot_dim, int rot_dims, int cache_len, ll_stream stream);

/* Attention in latent space.  q_lat (h, m, i) at q_lat[h * qs_h + m * qs_m + i]: the query with the key up-projection
 * absorbed.  Head h's rotary query part (not yet rotated) is at proj[m][q_rot_col0 + h * q_head_stride ...], its gate
 * logit at proj[m][gate_col0 + h] (gate_col0 < 0: none).  A query at position p sees p - window + 1 .. p (window <= 0: all).
 *   out(h, m, :) = sigmoid(gate) * sum_j softmax_j((q_lat . c_j + rot(q_rot) . k_rot_j) * scale) c_j
 * at out[h * os_h + m * os_m + i].  splits > 1 shares one query's keys among that many blocks (scratch of
 * ll_latent_attn_scratch_bytes) and merges them in split order. */
LL_API int ll_latent_attn(const void* q_lat, long long qs_h, long long qs_m, const void* proj, int proj_stride,
                          int q_rot_col0, int q_head_stride, int gate_col0, const float* rope, const int32_t* pos_ids,
                          const void* cache, void* out, long long os_h, long long os_m, int dtype, int B, int T, int n_head,
                          int kv_rank, int rot_dim, int rot_dims, int cache_len, int window, float scale, int splits,
                          float* scratch, ll_stream stream);
LL_API size_t ll_latent_attn_scratch_bytes(int M, int n_head, int kv_rank, int splits);

/* ---------------------------------------------------------------------------------------
 * Mixture of experts (csrc/moe_ops.cu).  Nothing here synchronises with the host: counts, offsets and the
 * permutation stay on the device.
 * ------------------------------------------------------------------------------------- */

/* Router: z = w_router [X][dim] (fp32) . x[m] + bias (fp32, optional); the `top` largest logits (ties: lowest index);
 * expert_w = softmax over the chosen logits.  Also sorts the M * top (token, choice) pairs by expert:
 * offsets [X + 1], perm [M * top] with perm[offsets[e] + r] = m * top + k.  counts [X], rank [M * top]: scratch. */
LL_API int ll_moe_route(const void* x, int dtype, const float* w_router, const float* bias, int M, int dim, int n_experts,
                        int top, int32_t* expert_idx, float* expert_w, int32_t* counts, int32_t* rank, int32_t* offsets,
                        int32_t* perm, ll_stream stream);
/* The same with the scoring as a parameter.  score_all 0: as above.  score_all 1: scores = softmax over ALL experts,
 * expert_w = chosen scores / (their sum + 1e-20).  n_groups > 1: the experts form n_groups equal groups of neighbours, a
 * group's score is its largest, and only experts of the keep_groups best groups (ties: lowest index) can be chosen. */
LL_API int ll_moe_route_scored(const void* x, int dtype, const float* w_router, const float* bias, int M, int dim, int n_experts,
                               int top, int score_all, int n_groups, int keep_groups, int32_t* expert_idx, float* expert_w,
                               int32_t* counts, int32_t* rank, int32_t* offsets, int32_t* perm, ll_stream stream);

/* Grouped GEMM over the sorted rows, one expert's weight per row segment; w is the experts' stack.
 * mode 1: w [X][2N][K] = [gate; up]; a [M][lda] read at token perm[r] / top;
 *         c[r][:] = glu(a . gate^T, a . up^T) with ll_glu_clamp's formula, rows in sorted order.
 * mode 2: as mode 1 with the up branch entering as it is: g * sigmoid(alpha g) * u (limit +inf: no clamp; alpha 1: silu).
 * mode 0: w [X][N][K]; a [n_rows][lda] in sorted order; c[perm[r]][:] = a[r] . w[e]^T. */
LL_API int ll_moe_grouped_gemm(const void* a, int lda, const void* w, const int32_t* offsets, const int32_t* perm, int mode,
                               int dtype, int n_rows, int top, int n_experts, int N, int K, float limit, float alpha,
                               void* c, int ldc, ll_stream stream);

/* The same grouped GEMM on the tcgen05 tensor cores (bf16, TMA-tiled operands, accumulators in TMEM), for steps with
 * many rows per expert.  a [n_rows][K] holds the rows ALREADY in sorted order (mode 1: gather them with
 * ll_moe_gather_rows: out[r] = x[perm[r] / top]); w, offsets, perm, mode, c as in ll_moe_grouped_gemm.  K a multiple of 8,
 * operands 16-byte aligned.  ll_moe_tc_error(): 0, or the code of the first bounded wait that ran out inside these
 * kernels since the library was loaded (synchronises the device). */
LL_API int ll_moe_gather_rows(const void* x, int ldx, const int32_t* perm, int top, int n_rows, int K, void* out, ll_stream stream);
LL_API int ll_moe_grouped_gemm_tc(const void* a, const void* w, const int32_t* offsets, const int32_t* perm, int mode, int n_rows,
                                  int n_experts, int N, int K, float limit, float alpha, void* c, int ldc, ll_stream stream);
LL_API int ll_moe_tc_error(void);

/* out[m] = sum_k expert_w[m][k] * y[m * top + k]  (+ sigmoid(shared_gate[m * gate_ld]) * shared_y[m], when shared_y is
 * given; shared_gate NULL: the shared expert is added as it is). */
LL_API int ll_moe_combine(const void* y, const float* expert_w, int top, const void* shared_y, int shared_ld,
                          const void* shared_gate, int gate_ld, void* out, int dtype, int M, int dim, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Two-branch layers on an fp32 stream (csrc/residual_ops.cu)
 * ------------------------------------------------------------------------------------- */

/* x[m][:] += s0 * a0 + s1 * a1 + s2 * a2 (each optional, activation dtype), in place; then with n = x / sqrt(mean(x^2) + eps):
 * out1 = n * w1 (fp32 when out1_f32, else the activation dtype; optional), out2 = n * w2 (activation dtype; optional). */
LL_API int ll_add_norm_pair(float* x, const void* a0, float s0, const void* a1, float s1, const void* a2, float s2, const float* w1,
                            const float* w2, float eps, void* out1, int out1_f32, void* out2, int act_dtype, int rows, int dim,
                            ll_stream stream);
/* RMS norm of fp32 rows y in `groups` equal parts with a gate (activation dtype, row stride gate_stride; silu, or a sigmoid
 * when gate_sigmoid):  gate_first 1: (y * gate(g)) / rms_part(.) * w;  0: y / rms_part(y) * w * gate(g).  w: C entries, or
 * C / groups shared by the parts (w_shared).  A part of y spans y_gs numbers (0: C / groups), of which the first C / groups are
 * normed.  stab (fp32 [rows][groups], optional): number C / groups of every part is a normaliser's product nq and stab the
 * stabiliser mx; the part is divided by max(|nq|, exp(-mx)) + 1e-6 before the norm. */
LL_API int ll_gated_group_norm(const float* y, int y_gs, const float* stab, const void* gate, int gate_stride, const float* w,
                               int w_shared, float eps, int groups, int gate_first, int gate_sigmoid, void* out, int act_dtype,
                               int rows, int C, ll_stream stream);
/* h <- relu(h)^2, in place */
LL_API int ll_relu_squared(void* h, int dtype, size_t n, ll_stream stream);
/* h <- gelu(h), in place: 0.5 h (1 + erf(h / sqrt 2)), or with tanh_form 0.5 h (1 + tanh(sqrt(2/pi) (h + 0.044715 h^3))) */
LL_API int ll_gelu(void* h, int dtype, int tanh_form, size_t n, ll_stream stream);

/* Several copies of the residual stream X [rows][S][dim] fp32 (S <= 8).  write: X'[t] = sum_s mix[s][t] X[s] + out[t] * r * ls * y,
 * all copies at once from the old ones (mix [S][S] indexed [from][to], NULL: every copy keeps itself; y [rows][dim] in the
 * activation dtype, NULL: nothing is added; ls fp32 [dim], NULL: none).  read: u = sum_t in[t] X'[t] (in NULL: the plain sum),
 * h = u / sqrt(mean(u^2) + eps) * w (fp32 when h_f32, else the activation dtype; h NULL: no read).  total (optional): the plain
 * sum of the new copies, fp32 [rows][dim].  The old copies are read at src + m * src_row + s * src_copy (src_copy 0: every copy
 * starts as the same row); X may be src. */
LL_API int ll_hyper_mix_norm(const float* src, long long src_row, long long src_copy, float* X, const void* y, const float* ls, float r,
                             const float* mix, const float* w_out, const float* w_in, const float* w, float eps, void* h, int h_f32,
                             float* total, int act_dtype, int rows, int S, int dim, ll_stream stream);
/* out[m][:] = x[m][:] / sqrt(mean(x[m][:]^2) + eps) * w  (w fp32 [dim] or NULL; rows of x_stride / out_stride elements) */
LL_API int ll_row_norm(const void* x, int x_stride, const float* w, float eps, void* out, int out_stride, int dtype, int rows, int dim,
                       ll_stream stream);
/* out[m][c] = a[m][c] * sigmoid(gate[m][c]), c < C; each operand with its own row stride; out may be a */
LL_API int ll_sigmoid_gate_mul(const void* a, int a_stride, const void* gate, int gate_stride, void* out, int out_stride, int dtype,
                               int rows, int C, ll_stream stream);
/* x <- cap * tanh(x / cap), fp32, in place */
LL_API int ll_tanh_cap(float* x, float cap, size_t n, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Short causal convolution with state (csrc/short_conv.cu)
 * ------------------------------------------------------------------------------------- */

/* y[b][t][c] = (flags & 1 ? x[b][t][c] : 0) + bias[c] + sum_j w[c][j] x[b][t - (taps-1) + j][c], then silu when flags & 2.
 * x: column slice (col0, C columns) of rows of x_stride elements; w fp32 [C][taps] (last column: the current token); bias
 * fp32 [C] or NULL; state fp32 [B][taps-1][C]: the last taps-1 inputs, read (unless pos_ids[0] == 0: no past) and replaced. */
LL_API int ll_short_conv(const void* x, int x_dtype, int x_stride, int col0, const float* w, const float* bias, float* state,
                         const int32_t* pos_ids, void* y, int y_dtype, int y_stride, int B, int T, int C, int taps, int flags,
                         ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Linear recurrence with diagonal decay (csrc/decay_scan.cu): state-space layers, gated linear attention
 * ------------------------------------------------------------------------------------- */

/* Per (b, h): S_t[i][c] = a_t[i] S_(t-1)[i][c] + ks_t k_t[i] v_t[c];  y_t[c] = qs sum_i q_t[i] S_t[i][c] + skip[h] v_t[c].
 * q, k: [B*T][stride], head g = h / (H / qk_heads) at columns g*n..; v: head h at columns h*p..; a: fp32 [B*T][H][n]
 * (a_per_channel) or [B*T][H]; ks fp32 [B*T][H] or NULL; skip fp32 [H] or NULL; state fp32 [B][H][n][p] (read unless
 * pos_ids[0] == 0, replaced); y fp32 [B*T][H*p].  unit_col: the last of the p columns of every head is the constant 1 and v
 * holds p - 1 columns per head (that column of S sums the keys alone: a normaliser carried by the same walk). */
LL_API int ll_decay_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                         const float* a, int a_per_channel, const float* ks, const float* skip, float qs, float* state,
                         const int32_t* pos_ids, float* y, int B, int T, int H, int qk_heads, int n, int p, int unit_col,
                         ll_stream stream);
/* Exponential gates with a running stabiliser, per (b, h): li = cap(raw_i + bias_i[h]), lf = logsigmoid(cap(raw_f + bias_f[h])),
 * cap(z) = c tanh(z / c) (c <= 0: none); mx_t = max(lf_t + mx_(t-1), li_t) with mx carried in mstate fp32 [B][H] (0 when
 * pos_ids[0] == 0); keep = exp(lf + mx_(t-1) - mx_t), take = exp(li - mx_t), stab = mx_t   (fp32 [B*T][H] each). */
LL_API int ll_matrix_memory_gates(const void* raw_i, const void* raw_f, int dtype, int stride, const float* bias_i,
                                  const float* bias_f, float cap, float* mstate, const int32_t* pos_ids, float* keep, float* take,
                                  float* stab, int B, int T, int H, ll_stream stream);
/* dt = softplus(raw[m][h] + dt_bias[h]); decay = exp(-exp(a_log[h]) dt)   (fp32 [M][H] each) */
LL_API int ll_ssm_gates(const void* raw, int dtype, int stride, const float* dt_bias, const float* a_log, float* dt_out,
                        float* decay, int M, int H, ll_stream stream);
/* out[m][c] = sigmoid(z[m][c] + bias[c])^(1/tau)   (fp32 [M][C]) */
LL_API int ll_channel_decay(const void* z, int dtype, int stride, const float* bias, float tau, float* out, int M, int C,
                            ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Windowed attention with kept first tokens, soft cap, distance penalty and mixed heads (csrc/window_attn.cu)
 * ------------------------------------------------------------------------------------- */

/* Rows of this step into the cache [B][keep + ring][cols]: position j -> slot j (j < keep) or keep + (j - keep) % ring. */
LL_API int ll_sink_ring_append(const void* k, int k_stride, const void* v, int v_stride, int dtype, const int32_t* pos_ids, void* kc,
                               void* vc, int B, int T, int kcols, int vcols, int keep, int ring, ll_stream stream);
/* s_h(i,j) = cap tanh(scale q_h(i).k_g(j) / cap) - r1_h ln(1 + r2_h (i-j)) (cap 0: none); j visible when j <= i and
 * (i-j < window or j < keep); softmax per head; weights mixed over heads by talk [H][H]; o_h = sigmoid(gate[m][h]) *
 * sum_j mixed_h(i,j) v_g(h)(j) -> y [B*T][H*vdim] (gate NULL: no gate).  scratch: ll_window_attn_scratch_bytes. */
LL_API size_t ll_window_attn_scratch_bytes(int M, int H, int vdim, int splits);
LL_API int ll_window_attn(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                          const int32_t* pos_ids, const float* r1, const float* r2, const float* talk, float scale, float softcap,
                          int B, int T, int H, int G, int dim, int vdim, int window, int keep, int ring, int splits, float* scratch,
                          void* y, ll_stream stream);

/* ---------------------------------------------------------------------------------------
 * Softmax attention with rotary positions over a ring of rows (csrc/rotary_attn.cu)
 * ------------------------------------------------------------------------------------- */

/* Rows of this step: q (H heads of dim) and k (G heads of dim; NULL: queries only) get an optional RMS norm over the whole
 * row times q_norm / k_norm (fp32, NULL: none), then the first rot_dims dimensions of every head turn by position * freq[i]
 * (fp32 [rot_dims / 2]; dimension i pairs with i + rot_dims / 2).  q -> q_out [B*T][H*dim]; k -> kc [B][ring][G*dim] at slot
 * position % ring; vc [B][ring][G*vdim] gets v, or (v NULL, vdim == dim) the keys as they are before the rotation. */
LL_API int ll_qk_rotary_append(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                               const float* q_norm, const float* k_norm, float eps, const float* freq, int rot_dims,
                               const int32_t* pos_ids, void* q_out, void* kc, void* vc, int B, int T, int H, int G, int dim, int vdim,
                               int ring, ll_stream stream);
/* s_h(i,j) = scale q_h(i).k_g(j), then cap tanh(s / cap) (softcap 0: none); j visible when j <= i, (window 0 or i - j < window),
 * (chunk 0 or j / chunk == i / chunk); softmax with exp(sink[h]) added to the denominator (sink NULL: none); o_h = sum_j w v_g(j),
 * times sigmoid(gate[m][h*vdim + c]) (gate NULL: none) -> y [B*T][H*vdim].  form 0: chosen by shape and dtype; 1: the fp32
 * form.  splits > 1 cuts every query's keys into that many ranges (fp32 form; scratch: ll_softmax_attn_scratch_bytes). */
LL_API size_t ll_softmax_attn_scratch_bytes(int M, int H, int vdim, int splits);
LL_API int ll_softmax_attn(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                           const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int T, int H, int G, int dim,
                           int vdim, int window, int chunk, int ring, int splits, int form, float* scratch, void* y,
                           ll_stream stream);

/* The same two calls for heads that carry `maps` score maps (1 or 2): the q row holds H heads of [map 0 | map 1] (dim each), the
 * k row G heads likewise (kc [B][ring][G*maps*dim]), the values stay [G*vdim] and serve every map.  Two maps are combined as
 * o = a_0 - diff_lambda * a_1, o / sqrt(mean_c(o^2) + eps) * diff_post, before the gate.  sink: [H*maps].  In the append q may be
 * NULL (keys and values only); values taken from the keys need maps == 1.  The fp32 form needs scratch
 * (ll_softmax_attn_scratch_bytes(M, H*maps, vdim, splits)) whenever maps > 1; ll_softmax_attn_tensor_form() tells whether a call
 * with form 0 takes the tensor-core form, which needs none. */
LL_API int ll_qk_rotary_append_maps(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                                    const float* q_norm, const float* k_norm, float eps, const float* freq, int rot_dims,
                                    const int32_t* pos_ids, void* q_out, void* kc, void* vc, int B, int T, int H, int G, int dim,
                                    int vdim, int ring, int maps, ll_stream stream);
LL_API int ll_softmax_attn_tensor_form(int dtype, int T, int dim, int vdim, int q_stride, int gate_stride, int splits);
LL_API int ll_softmax_attn_maps(const void* q, int q_stride, const void* gate, int gate_stride, const void* kc, const void* vc, int dtype,
                                const int32_t* pos_ids, const float* sink, float scale, float softcap, int B, int T, int H, int G,
                                int dim, int vdim, int window, int chunk, int ring, int splits, int form, int maps, float diff_lambda,
                                float diff_post, float eps, float* scratch, void* y, ll_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* LLB200_H */
