/*
 * kvmix_b200 -- C ABI of the B200 (sm_100a) KV-cache hot path: group quantizer, dequant GEMV
 * and fused decode attention over a mixed-precision (1/2/3/4-bit + fp16 tail) KV cache.
 *
 * Every entry point takes plain device pointers, sizes and element strides, launches on the
 * stream it is given, never synchronises the host, never allocates, and returns 0 or a negative
 * KVQ_ERR_* code detected on the host before any launch.  Launch errors are returned as
 * KVQ_ERR_CUDA (kvq_last_cuda_error() gives the CUDA text).
 *
 * Formats (identical to the upstream KVmix extension, so buffers are interchangeable):
 *   codes   int32 words, fields LSB first; 32/b fields of b bits for b in {1,2,4}; b = 3 packs 11
 *           fields per word: ten 3-bit fields at bits 0..29 and one 2-bit field at bits 30..31
 *           (upstream quant_cuda/csrc/quantization_cuda.cu:612-626)
 *   scale   (max-min)/(2^b-1) of each group, computed in fp32, stored in the input dtype
 *   mn      min of each group ("zero")
 *   dequantised value = scale * code + mn
 */
#ifndef KVMIX_B200_H
#define KVMIX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *kvq_stream_t; /* a cudaStream_t */

enum {
    KVQ_OK = 0,
    KVQ_ERR_BITS = -1,        /* bits not in {1,2,3,4}                               */
    KVQ_ERR_GROUP3 = -2,      /* 3-bit requires group 11                             */
    KVQ_ERR_DIV11 = -3,       /* 3-bit requires length divisible by 11               */
    KVQ_ERR_DIVGROUP = -4,    /* length not divisible by group                       */
    KVQ_ERR_DIVWORD = -5,     /* length not divisible by 32/bits                     */
    KVQ_ERR_HEADS = -6,       /* query heads not divisible by kv heads               */
    KVQ_ERR_SHAPE = -7,       /* inconsistent sizes                                  */
    KVQ_ERR_GROUPWORD = -8,   /* group not a multiple of 32/bits where one is needed */
    KVQ_ERR_TOKENS = -9,      /* K and V token counts differ                         */
    KVQ_ERR_NULL = -10,       /* null pointer                                        */
    KVQ_ERR_UNSUPPORTED = -11,/* outside what the kernels implement (see each call)  */
    KVQ_ERR_WORKSPACE = -12,  /* workspace missing or too small                      */
    KVQ_ERR_ALIGN = -13,      /* pointer or stride alignment                         */
    KVQ_ERR_STATIC_SCRATCH = -14, /* problem needs more than KVQ_STATIC_SCRATCH_BYTES */
    KVQ_ERR_CUDA = -100       /* a CUDA call or launch failed                        */
};

int kvq_version(void);
const char *kvq_error_string(int code);
const char *kvq_last_cuda_error(void);

/* Fields per 32-bit word: 32/bits, or 11 for bits == 3. */
int kvq_features_per_int(int bits);

/*
 * Group quantizer along the last dimension of a 4-D tensor.
 * Replaces quantize_pack_last_dim_cuda, upstream quant_cuda/csrc/quantization_cuda.cu:631-721
 * (kernels :540-598 and :601-629), and -- through the output strides -- the append forms
 * process_key_quantization_cuda (:298-411) and process_value_quantization_cuda (:413-537):
 * point code/scale/mn at the first free word/group of a preallocated cache and the new
 * groups are written in place.
 *
 * x is logically [B, H, A, S]; element (b,h,a,s) is at x[b*x_sB + h*x_sH + a*x_sA + s*x_sS]
 * (strides in elements), so a [B,H,T,D] key tensor is quantized per channel over token groups
 * by passing A = D, S = T, x_sA = 1, x_sS = D without a transposed copy.
 * Groups of `group` consecutive s.  Outputs:
 *   code  [B,H,A,S/fpi] int32   strides c_sB, c_sH, c_sA (words), last dim contiguous
 *   scale [B,H,A,S/group]       strides z_sB, z_sH, z_sA (elements), last dim contiguous
 *   mn    same shape and strides as scale
 * x_is_f32 = 0: x, scale, mn are fp16;  1: they are fp32.
 * Rules (same as upstream): bits == 3 needs group == 11 and S % 11 == 0; otherwise
 * S % group == 0 and S % (32/bits) == 0.
 * Codes always come from the true fp32 quotient (x-mn)/((max-min)/(2^b-1)).  The *stored* scale is
 *   scale_by_division = 0: (max-min) * fl32(1/(2^b-1)), what quantize_pack_last_dim_cuda returns
 *       (its torch-side "tensor / scalar" at :711 is evaluated as a multiplication by the reciprocal);
 *   scale_by_division = 1: (max-min) / (2^b-1), what the upstream append kernels store (:51-53, :232-234).
 *
 * EXTENSION WITHOUT AN UPSTREAM COUNTERPART (nothing upstream pins it): ragged_tail != 0 with bits == 3 lifts the
 * S % 11 == 0 rule.  code, scale and mn then have ceil(S/11) entries per row: groups of 11 with a last group of
 * S % 11 elements, each group one word, unused fields 0, upstream's 3-bit group rule otherwise (element 10 of a full
 * group keeps its 2-bit field).  It exists for 3-bit *values* at head_dim 128 (12 words per token, the last holding 7
 * codes), which upstream cannot represent (:433-434).  kvq_decode_attn reads that layout when v_bits == 3.
 */
typedef struct {
    const void *x;
    int32_t x_is_f32;
    int64_t B, H, A, S;
    int64_t x_sB, x_sH, x_sA, x_sS;
    int32_t group, bits;
    int32_t scale_by_division;
    int32_t *code;
    int64_t c_sB, c_sH, c_sA;
    void *scale;
    void *mn;
    int64_t z_sB, z_sH, z_sA;
    int32_t ragged_tail;                /* extension, see below; 0 = upstream's rules */
} kvq_quant_args;

int kvq_quant_lastdim(const kvq_quant_args *a, kvq_stream_t stream);

/*
 * The functional append forms: out = previous ++ quantize(x), written into caller-allocated contiguous tensors.
 * Replace process_key_quantization_cuda (upstream quant_cuda/csrc/quantization_cuda.cu:298-411) and
 * process_value_quantization_cuda (:413-537), whose wrappers allocate the outputs and whose kernels copy the
 * previous tensors and quantize the new tokens.  (A preallocated cache does not need them: it points
 * kvq_quant_lastdim at its first free word and moves nothing.)
 *
 * kvq_append_k: x [B,H,D,Tn] (strides x_sB, x_sH, x_sA, x_sS over those four axes), groups over the Tn new tokens;
 *   prev_code [B,H,D,old_words], prev_scale/prev_mn [B,H,D,old_groups] contiguous (NULL when old_* == 0);
 *   code [B,H,D,old_words + Tn/fpi], scale/mn [B,H,D,old_groups + Tn/group] contiguous.
 * kvq_append_v: x [B,H,Tn,D] (same four strides), groups over D; old_tokens previous tokens:
 *   prev_code [B,H,old_tokens,D/fpi], prev_scale/prev_mn [B,H,old_tokens,D/group] contiguous;
 *   code [B,H,old_tokens+Tn,D/fpi], scale/mn [B,H,old_tokens+Tn,D/group] contiguous.
 * The stored scale is the quotient (max-min)/(2^b-1), as the upstream append kernels store it (:51-53, :232-234).
 * Previous 3-bit code words are copied as well (upstream's fused 3-bit key kernel leaves them uninitialised,
 * :131-134).  Same divisibility rules and error codes as kvq_quant_lastdim.
 */
typedef struct {
    const void *x;
    int32_t x_is_f32;
    int64_t B, H, A, S;                 /* x is [B,H,A,S]: keys A = D, S = Tn; values A = Tn, S = D */
    int64_t x_sB, x_sH, x_sA, x_sS;
    int32_t group, bits;
    const int32_t *prev_code;
    const void *prev_scale;
    const void *prev_mn;
    int64_t old_words, old_groups;      /* kvq_append_k: previous words / groups per channel row */
    int64_t old_tokens;                 /* kvq_append_v: previous tokens */
    int32_t *code;
    void *scale;
    void *mn;
} kvq_append_form_args;

int kvq_append_k(const kvq_append_form_args *a, kvq_stream_t stream);
int kvq_append_v(const kvq_append_form_args *a, kvq_stream_t stream);

/*
 * Append one token's keys and values (fp16, after RoPE) to the fp16 tails of the cache, in one launch.
 * Replaces the two torch.cat calls upstream makes per layer and step (models/modeling_llama_KVmix.py:111-112)
 * without moving the old tail: row `k_slot` of kfull and row `v_slot` of vfull are overwritten.
 *   k_new, v_new [B, Hkv, D] fp16, strides kn_sB, kn_sH / vn_sB, vn_sH (D contiguous)
 *   kfull, vfull [B, Hkv, cap, D] fp16, strides *_sB, *_sH, *_sT
 * D must be a multiple of 8 and all rows 16-byte aligned.
 */
typedef struct {
    int32_t B, Hkv, D;
    const void *k_new;
    int64_t kn_sB, kn_sH;
    const void *v_new;
    int64_t vn_sB, vn_sH;
    void *kfull;
    int64_t kf_sB, kf_sH, kf_sT;
    int32_t k_slot;
    void *vfull;
    int64_t vf_sB, vf_sH, vf_sT;
    int32_t v_slot;
} kvq_append_args;

int kvq_append_kv(const kvq_append_args *a, kvq_stream_t stream);

/*
 * Prompt prefill straight from the projections.
 * Replaces the quantization half of upstream's no-cache branch (models/modeling_llama_KVmix.py:213-254) together with
 * what precedes it there: the rotary embedding of the keys (:103, apply_rotary_pos_emb), the slice + .contiguous() +
 * .transpose(2, 3).contiguous() copies of the keys (:225-231) and the slice copies of the tails (:226, :243).
 *   k, v      the k_proj / v_proj outputs of the prompt, fp16, element (b, t, h, d) at k + b*k_sB + t*k_sT + h*k_sH + d
 *             (e.g. [B, L, Hkv*D] as the projection writes it: k_sT = Hkv*D, k_sH = D; [B, Hkv, L, D] works alike)
 *   cos, sin  rotary tables, fp16, element (b, t, d) at cos + b*r_sB + t*r_sT + d (r_sB = 0 for one table shared by
 *             the batch); NULL when the keys arrive rotated.  Rotation is the rotate_half form with fp16 rounding of
 *             each product and of the sum, i.e. bit-identical to (k * cos) + (rotate_half(k) * sin) on fp16 tensors.
 *   nk, nv    tokens to quantize (upstream's split points: multiples of k_group / v_group); keys [0, nk) are rotated
 *             and quantized per channel over groups of k_group tokens into kcode / kscale / kmn, values [0, nv) per
 *             token over groups of v_group channels, exactly as kvq_quant_lastdim (scale_by_division = 0) would;
 *             the remaining tokens go, rotated, to rows 0.. of the fp16 tails kfull / vfull.
 * Three launches (key quantizer, value quantizer, tails), no temporary tensors.  D must be 128.
 */
typedef struct {
    const void *k;
    const void *v;
    int64_t k_sB, k_sT, k_sH, v_sB, v_sT, v_sH;
    const void *cos;
    const void *sin;
    int64_t r_sB, r_sT;
    int32_t B, Hkv, L, D;
    int32_t nk, nv;
    int32_t k_bits, k_group, v_bits, v_group;
    int32_t *kcode;
    int64_t kc_sB, kc_sH, kc_sD;
    void *kscale;
    void *kmn;
    int64_t ks_sB, ks_sH, ks_sD;
    int32_t *vcode;
    int64_t vc_sB, vc_sH, vc_sT;
    void *vscale;
    void *vmn;
    int64_t vs_sB, vs_sH, vs_sT;
    void *kfull;
    int64_t kf_sB, kf_sH, kf_sT;
    void *vfull;
    int64_t vf_sB, vf_sH, vf_sT;
} kvq_prefill_args;

int kvq_prefill(const kvq_prefill_args *a, kvq_stream_t stream);

/*
 * Dequantising mat-vec, M = 1.
 * Replaces quantized_gemm, upstream quant_cuda/csrc/dequantization_gemv_cuda.cu:127-248 (kernel
 * :7-124), reading the caller's layout directly (upstream first transposes codes, scales and
 * zeros on every call, :151-171):
 *   out[b,h,n] = fp16( sum_k fA[b,h,k] * (scale[b,hk,k,n/group] * code[b,hk,k,n] + zero[b,hk,k,n/group]) )
 *   hk = h / (nh / nh_kv), fp32 accumulation.
 *   fA    [B, nh, K] fp16                 strides a_sB, a_sH, K contiguous
 *   qB    [B, nh_kv, K, n_words] int32    strides q_sB, q_sH, q_sK (words)
 *   scale [B, nh_kv, K, n_groups] fp16    strides s_sB, s_sH, s_sK; zeros alike
 *   out   [B, nh, N] fp16, N = n_groups * group, strides o_sB, o_sH
 * group must be a multiple of 32/bits (11 for bits == 3): one scale per packed word, as upstream.
 */
typedef struct {
    const void *fA;
    int64_t a_sB, a_sH;
    const int32_t *qB;
    int64_t q_sB, q_sH, q_sK;
    const void *scale;
    const void *zero;
    int64_t s_sB, s_sH, s_sK;
    void *out;
    int64_t o_sB, o_sH;
    int64_t B, nh, nh_kv, K, n_words, n_groups;
    int32_t group, bits;
} kvq_gemv_args;

int kvq_gemv(const kvq_gemv_args *a, kvq_stream_t stream);

/*
 * Fused decode attention for one query token per sequence over a mixed cache:
 *   scores = [ q.Kq^T (packed keys, tokens 0..Tkq) | q.Kfull^T (fp16 keys, tokens Tkq..T) ] / sqrt(D)
 *   p = softmax(scores);  out = p[:Tvq].Vq (packed values) + p[Tvq:].Vfull (fp16 values)
 * Replaces, in one launch, the cached branch of the upstream attention forward
 * (models/modeling_llama_KVmix.py:170-211, models/modeling_mistral_KVmix.py:207-262): two
 * quantized_gemm calls, repeat_kv_quant copies, two fp16 matmuls, concat, softmax and add.
 * The key and value boundaries Tkq and Tvq are independent (upstream uses different group sizes
 * and residual ratios for K and V).  GQA is native: query head h reads kv head h/(nh/nh_kv).
 *
 *   q      [B, nh, D] fp16              strides q_sB, q_sH
 *   out    [B, nh, D] fp16              strides o_sB, o_sH
 *   kcode  [B, nh_kv, D, Tkq/fpi_k]     strides kc_sB, kc_sH, kc_sD (words)
 *   kscale, kmn [B, nh_kv, D, Tkq/k_group] fp16, strides ks_sB, ks_sH, ks_sD
 *   kfull  [B, nh_kv, kf_cap, D] fp16   strides kf_sB, kf_sH, kf_sT; token Tkq+r lives in row
 *          (kf_start + r) mod kf_cap  (kf_start = 0 and kf_cap >= Rk for a linear tail)
 *   vcode  [B, nh_kv, Tvq, D/fpi_v]     strides vc_sB, vc_sH, vc_sT (words)
 *   vscale, vmn [B, nh_kv, Tvq, D/v_group] fp16, strides vs_sB, vs_sH, vs_sT
 *   vfull  [B, nh_kv, vf_cap, D] fp16   strides vf_sB, vf_sH, vf_sT, ring like kfull
 * Two kernels serve the call.  The tensor-core kernel takes D = 128, k_group in {32, 64, 128} (11 for 3-bit keys),
 * v_group in {32, 64, 128}, Tvq a multiple of 32, nh a multiple of nh_kv, every packed tensor and fp16 tail 16-byte
 * aligned with row strides that keep rows 16-byte aligned (kc_sD % 4, ks_sD % 8, kf_sT % 8, vf_sT % 8 == 0; value
 * rows contiguous: vc_sT == D/fpi_v, vs_sT == D/v_group) -- what a preallocated cache provides.  Anything else runs
 * on a slower CUDA-core kernel with the same results.
 * D must be 128.  k_group and v_group must be multiples of the fields per word (k_group == 11 for
 * 3-bit keys).  3-bit values (v_bits == 3, v_group == 11) are an extension without an upstream counterpart --
 * upstream needs D % 11 == 0 for them (quant_cuda/csrc/quantization_cuda.cu:433-434) -- in the layout
 * kvq_quant_lastdim writes with ragged_tail: vcode [B, nh_kv, Tvq, 12], vscale / vmn [B, nh_kv, Tvq, 12], word j
 * holding channels 11j .. min(11j + 10, 127) as its own group; they run on the CUDA-core kernel.
 * round_scores != 0 narrows each raw score to fp16 before scaling, as upstream's GEMV and fp16
 * matmul do; everything else accumulates in fp32.
 *
 * mask (optional, NULL = none): additive attention mask over the T key positions, as the upstream forward
 * applies it (models/modeling_llama_KVmix.py:188-193: weights + mask, then clamped from below at the most
 * negative finite fp32, then softmax).  mask[b*mask_sB + h*mask_sH + t], fp16 (mask_is_f32 == 0) or fp32;
 * mask_sH = 0 broadcasts one row over the heads (the usual [B,1,1,T] padding mask).  Position t counts the
 * packed prefix first and the fp16 tail after it, i.e. chronological order, so a left-padding mask indexes
 * it directly.
 *
 * workspace: kvq_decode_attn_workspace_bytes(B, nh, T) bytes of device memory (partials of heads held by
 * several CTAs and one counter per query head).  The call zeroes the counters itself unless flags says they are
 * ready; concurrent calls must not share a workspace.
 */
#define KVQ_MAX_PEERS 8
typedef struct {
    int32_t B, nh, nh_kv, D;
    int32_t T, Tkq, Tvq;
    int32_t k_bits, k_group, v_bits, v_group;
    int32_t round_scores;
    float softmax_scale;
    const void *q;
    int64_t q_sB, q_sH;
    void *out;
    int64_t o_sB, o_sH;
    const int32_t *kcode;
    int64_t kc_sB, kc_sH, kc_sD;
    const void *kscale;
    const void *kmn;
    int64_t ks_sB, ks_sH, ks_sD;
    const void *kfull;
    int64_t kf_sB, kf_sH, kf_sT;
    int32_t kf_cap, kf_start;
    const int32_t *vcode;
    int64_t vc_sB, vc_sH, vc_sT;
    const void *vscale;
    const void *vmn;
    int64_t vs_sB, vs_sH, vs_sT;
    const void *vfull;
    int64_t vf_sB, vf_sH, vf_sT;
    int32_t vf_cap, vf_start;
    void *workspace;
    uint64_t workspace_bytes;
    const void *mask;
    int64_t mask_sB, mask_sH;
    int32_t mask_is_f32;
    int32_t flags;                 /* KVQ_ATTN_* bits; 0 for the behaviour described above */
    /* Optional cache update fused into the launch (k_new == NULL: none); see "fused decode step" below. */
    const void *k_new;             /* [B, nh_kv, D] fp16: the step's new key rows, strides kn_sB, kn_sH */
    const void *v_new;
    int64_t kn_sB, kn_sH, vn_sB, vn_sH;
    int32_t k_quant, v_quant;      /* tokens to quantize in this launch: 0, or exactly k_group / v_group */
    int32_t k_quant_slot, v_quant_slot;   /* ring row of the first of them */
    /* Optional device-resident cache state (NULL: none); see "device-resident state" below. */
    int32_t *state;
    int32_t window;                /* fp16 tokens kept (>= 0), or < 0: keep int(ratio * current fp16 length) */
    double k_ratio, v_ratio;
    /* Optional exchange fused into the launch (n_peers == 0: none); see "head-sharded exchange" below. */
    int32_t n_peers, peer_head0;
    void *peer_out[KVQ_MAX_PEERS];         /* [B, nh_total, D] fp16 gather buffer of every rank, strides peer_sB, peer_sH */
    uint32_t *peer_flag[KVQ_MAX_PEERS];    /* one arrival counter per rank */
    int64_t peer_sB, peer_sH;
} kvq_attn_args;

/*
 * Fused decode step.  Upstream updates the cache and attends in one forward call
 * (models/modeling_llama_KVmix.py:111-211: cat the new token onto the fp16 tails, quantize a group of the oldest tail
 * tokens when one is due, then the attention); with k_new / v_new set, kvq_decode_attn does the same in its one
 * launch.  The caller describes the cache as it is AFTER the update -- T counts the new token, Tkq / Tvq count a group
 * that becomes packed in this step, kf_start / vf_start are the ring starts after that group left the tails -- and
 * says what is to be done: the new rows (every reader takes token T-1 from k_new / v_new; one CTA per kv head also
 * stores them into ring row (kf_start + T-1-Tkq) mod kf_cap, likewise for values), and k_quant / v_quant tokens at
 * ring rows k_quant_slot.. / v_quant_slot.. to be quantized into packed positions [Tkq - k_quant, Tkq) /
 * [Tvq - v_quant, Tvq) with the arithmetic of kvq_quant_lastdim (scale_by_division = 0), bit for bit.  kcode, kscale,
 * kmn, vcode, vscale, vmn, kfull and vfull are written although the struct declares them const.
 * Served by the tensor-core kernels when exactly one CTA reads a kv head's tokens: nh == nh_kv, or grouped queries
 * with nh / nh_kv in {2, 4} and group sizes the grouped kernel takes; otherwise KVQ_ERR_UNSUPPORTED is returned before
 * anything is launched and the caller runs kvq_append_kv / kvq_quant_lastdim / kvq_decode_attn separately.
 */

/*
 * Device-resident state.  With `state` set (and a fused decode step: k_new / v_new given) the lengths and ring
 * starts of the cache are not taken from this struct but from device memory: state[0..4] = {T, Tkq, Tvq, kf_start,
 * vf_start} BEFORE the step, state[5] = 0.  The kernel applies upstream's window policy itself
 * (models/modeling_llama_KVmix.py:115-126: keep `window` tokens, or int(ratio * current_fp16_len)), appends,
 * quantizes the group that falls due, attends, and leaves state[] describing the cache after the step.  T in this
 * struct is then only an upper bound used to lay out the grid and the score buffers (any value >= the real length
 * after the step), Tkq / Tvq / kf_start / vf_start / k_quant* / v_quant* are ignored -- so the same argument block
 * serves every step and a decode step can be captured once in a CUDA graph and replayed.  At most one group per
 * step is quantized: use it once the cache is in steady state (a fixed window always is; upstream's ratio policy is
 * after the first few steps that shrink a prompt's tail).
 */

/*
 * Head-sharded exchange.  When the KV heads of a long sequence are split across the GPUs of a node, every rank needs
 * all ranks' attention outputs before the output projection (no upstream counterpart: upstream is single-GPU).  With
 * n_peers > 0 the CTA that finishes a query head stores its row, besides `out`, straight into every rank's gather
 * buffer -- peer_out[p] + b*peer_sB + (peer_head0 + h)*peer_sH, plain stores through peer-mapped pointers (NVLink),
 * no multicast -- and then adds the number of heads it wrote to every rank's arrival counter peer_flag[p] with a
 * system-scope release.  A consumer waits for its counter with kvq_peer_wait.  peer_out / peer_flag include this
 * rank's own buffer and counter.  KVQ_MAX_PEERS ranks at most.
 */

/* flags: the counters at the start of the workspace are known to be zero -- cleared once with
 * kvq_decode_attn_workspace_init and since then touched only by this library, whose kernels leave every counter
 * they use at zero.  The call then skips its own clearing (one memset node less per decode step). */
#define KVQ_ATTN_WORKSPACE_READY 1

/*
 * Waits (on `stream`, on the device) until *counter has reached `expected` arrivals (counters only grow; the
 * comparison is wrap-safe), polling at most max_polls times with a short sleep between polls -- about 1 us each, so
 * 1000000 is roughly a second.  If the count does not arrive, the kernel gives up, stores 1 into status[0] and the
 * value it last saw into status[1], and returns; the context stays usable and the host decides what to do (a peer that
 * died, a shard that was never launched).  status must be device memory holding two int32, zeroed by the caller.
 */
int kvq_peer_wait(const uint32_t *counter, uint32_t expected, uint32_t max_polls, int32_t *status, kvq_stream_t stream);
/*
 * The same bounded wait with the target kept on the device, for steps replayed from a CUDA graph: *generation (device
 * memory, one uint32 per counter, zeroed by the caller together with the counter) is incremented by the kernel, and
 * the wait is for generation * per_use arrivals, per_use being what one use of the counter adds (batch * all ranks'
 * query heads).  No argument changes from step to step.  No upstream counterpart.
 */
int kvq_peer_wait_next(const uint32_t *counter, uint32_t per_use, uint32_t *generation, uint32_t max_polls,
                       int32_t *status, kvq_stream_t stream);

uint64_t kvq_decode_attn_workspace_bytes(int32_t B, int32_t nh, int32_t T);
/* Clears the counters of a workspace for B * nh query heads (asynchronously, on `stream`). */
int kvq_decode_attn_workspace_init(void *workspace, uint64_t bytes, int32_t B, int32_t nh, kvq_stream_t stream);
int kvq_decode_attn(const kvq_attn_args *a, kvq_stream_t stream);

/*
 * How kvq_decode_attn would spread the call described by `a` (shapes, bit widths and group sizes are read; no pointer
 * is dereferenced) over CTAs.  No upstream counterpart: upstream's GEMV never splits a row.
 * tensor_core > 0 asks for the tensor-core kernels' plan, 0 for the generic kernel's, < 0 for whichever
 * kvq_decode_attn would run for `a` (then pointers and strides are inspected for alignment too).
 * The token axis of a head is cut into units of `unit` tokens.  Tensor-core kernels (aligned caches, see
 * kvq_decode_attn): kernel 1 gives every query head its own CTAs, kernel 2 lets the heads_per_cta query heads that
 * share a kv head share CTAs (chosen when nh / nh_kv is 2 or a multiple of 4 and the group sizes allow it).  The
 * first n_whole heads take one CTA each -- a multiple of the GPU's resident-CTA slots, so they fill whole waves -- and
 * each of the remaining n_cut heads is cut into `segments` pieces of segment_units units, launched after them, so
 * that the last wave of the grid consists of short CTAs and fills every slot whatever the batch size.  A head held
 * by several CTAs is merged by the one that finishes last, in token order (results do not depend on timing).
 * Generic kernel (tensor_core == 0): every head is cut into `segments` chunks of `unit` tokens, one CTA each.
 * max_segment_tokens: most tokens one CTA holds.  Host-only; returns KVQ_OK or KVQ_ERR_NULL / KVQ_ERR_BITS /
 * KVQ_ERR_SHAPE / KVQ_ERR_HEADS.
 */
typedef struct {
    int32_t kernel;              /* 0 generic, 1 tensor-core, 2 tensor-core with grouped query heads */
    int32_t heads_per_cta;
    int32_t unit, units_per_head;
    int32_t n_ctas, n_whole, n_cut;
    int32_t segments, segment_units, max_segment_tokens;
} kvq_attn_plan;

int kvq_decode_attn_plan(const kvq_attn_args *a, int32_t tensor_core, kvq_attn_plan *out);

/*
 * kvq_decode_attn for callers that have no device memory to give.  (No counterpart in upstream KVmix:
 * there every call allocates through torch.)
 *
 * Who needs it: a host that reaches this library over a foreign-function boundary (cgo, JNI, ctypes from
 * a process without torch) owns no device allocator at all -- it only holds the cache pointers it was
 * handed; and a serving engine that gives every free byte of HBM to its KV-cache pool at start-up cannot
 * get a further cudaMalloc to succeed later, nor afford the device-wide synchronisation a cudaMalloc
 * implies in the middle of a decode loop.  Neither can supply the split-partials workspace that
 * kvq_decode_attn asks for.
 *
 * This variant takes the same arguments, ignores a->workspace / a->workspace_bytes, and keeps the split
 * partials and per-head counters in a fixed KVQ_STATIC_SCRATCH_BYTES (8 MiB) array that is part of the
 * library image: every GPU on which the library is loaded holds those 8 MiB until the process exits.
 * It calls no cudaMalloc, cudaFree or any allocating routine.
 *
 *  - Limit: kvq_decode_attn_workspace_bytes(B, nh, T) must not exceed KVQ_STATIC_SCRATCH_BYTES, else
 *    KVQ_ERR_STATIC_SCRATCH is returned and nothing is launched (8 MiB covers e.g. 32 heads at 131072
 *    tokens, or 2048 heads at any length that needs one split).
 *  - First call on each device: the device address of the array is looked up once per device, on the
 *    first call made while that device is current (cudaGetSymbolAddress); make that first call before
 *    starting any stream capture.
 *  - The array is shared by every call on the device and keeps the previous call's contents; the call
 *    zeroes the counters it needs itself.  Two calls that overlap on the GPU (different streams, or
 *    different host threads) race on it: serialise them on one stream, or use kvq_decode_attn with a
 *    workspace per stream.
 */
#define KVQ_STATIC_SCRATCH_BYTES (8u << 20)
int kvq_decode_attn_static(const kvq_attn_args *a, kvq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KVMIX_B200_H */
