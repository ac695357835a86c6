/*
 * TEST INFRASTRUCTURE -- not part of the product, never linked into it.
 *
 * CPU restatement, in plain C, of the arithmetic of the upstream KVmix CUDA extension for the
 * KV-cache hot path.  Upstream has no CPU (or PyTorch) implementation of this path; its only
 * statement of the algorithm is the CUDA kernel bodies, which are scalar C once the thread
 * indices are replaced by loops.  Every function below names the upstream lines it follows
 * (paths relative to the upstream project root).
 *
 * Parity status: upstream ships no golden vectors or known-answer tests for this path
 * (quant_cuda/test.py calls functions the module does not export and asserts nothing).  This
 * restatement is therefore pinned against outputs of the upstream extension itself, rebuilt
 * unmodified for sm_100a (oracle/build_ref.py) and run on a B200; the vectors it produced are
 * committed under tests/golden/ with the script that made them.
 *
 * Arithmetic rules restated here:
 *   - all quantizer math in IEEE binary32: fminf/fmaxf reductions, true division, roundf
 *     (half away from zero), compiled with -ffp-contract=off;
 *   - a constant group has scale 0 and (x-mn)/scale = 0/0 = NaN; the CUDA float->int
 *     conversion of NaN yields 0, stated explicitly here instead of relying on a C cast;
 *   - the GEMV uses fused multiply-adds where nvcc contracts them (fmaf), the upstream
 *     per-lane summation order and its 5-step shuffle tree.
 *
 * fp16 values cross this interface as uint16_t bit patterns.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t h16;

static inline float h2f(h16 h) { _Float16 x; memcpy(&x, &h, 2); return (float)x; }
static inline h16 f2h(float f) { _Float16 x = (_Float16)f; h16 h; memcpy(&h, &x, 2); return h; }

int orc_features_per_int(int bits) { return bits == 3 ? 11 : 32 / bits; }

/* Thread control for the timed CPU baseline: launchers such as torchrun export OMP_NUM_THREADS=1, which would
 * silently turn the "all host cores" figure into a one-core one. */
#ifdef _OPENMP
#include <omp.h>
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int orc_max_threads(void) { return omp_get_max_threads(); }
#else
void orc_set_threads(int n) { (void)n; }
int orc_max_threads(void) { return 1; }
#endif

/* Argument rules of quantize_pack_last_dim_cuda, quant_cuda/csrc/quantization_cuda.cu:637-653,687.
 * Returns 0 when legal, a negative code naming the violated TORCH_CHECK otherwise. */
int orc_quant_check(int64_t S, int G, int bits) {
    if (bits < 1 || bits > 4) return -1;
    if (bits == 3) {
        if (G != 11) return -2;            /* :638  group_length must be 11 */
        if (S % 11 != 0) return -3;        /* :649  steps divisible by 11 */
    } else {
        if (G <= 0 || S % G != 0) return -4;            /* :652 */
        if (S % (32 / bits) != 0) return -5;            /* :687 */
    }
    return 0;
}

/*
 * One group: min_max_quantize_kernel, quantization_cuda.cu:553-596, followed by the word
 * packing of pack_data_kernel, :612-626, applied to a row of S fp32 values.
 *   code  [S/fpi] int32, LSB-first fields; 3-bit: ten 3-bit fields then a 2-bit field at bit 30
 *   mn,mx [S/G]   fp32
 */
static void quant_row(const float *x, int64_t S, int G, int bits, int32_t *code, float *mn_out,
                      float *mx_out, int32_t *tmp) {
    const int fpi = orc_features_per_int(bits);
    const float qmax = (float)((1 << bits) - 1);
    const int64_t ng = S / G;
    for (int64_t g = 0; g < ng; ++g) {
        const float *p = x + g * G;
        float mn = FLT_MAX, mx = -FLT_MAX;                                  /* :554-555 */
        for (int i = 0; i < G; ++i) { mn = fminf(mn, p[i]); mx = fmaxf(mx, p[i]); }
        mn_out[g] = mn; mx_out[g] = mx;                                      /* :566-567 */
        const float scale = (mx - mn) / qmax;                                /* :570 */
        for (int i = 0; i < G; ++i) {
            const float normalized = (p[i] - mn) / scale;                    /* :577 / :589 */
            int q = isnan(normalized) ? 0 : (int)roundf(normalized);         /* :578 / :590 */
            int emax = (int)qmax;
            if (bits == 3 && i >= 10) emax = 3;                              /* :579 */
            if (q > emax) q = emax;
            if (q < 0) q = 0;
            tmp[g * G + i] = q;
        }
    }
    const int64_t nw = S / fpi;
    for (int64_t w = 0; w < nw; ++w) {                                       /* :612-626 */
        const int32_t *c = tmp + w * fpi;
        uint32_t v = 0;
        if (bits == 3) {
            for (int i = 0; i < 10; ++i) v |= (uint32_t)c[i] << (i * 3);
            v |= (uint32_t)c[10] << 30;
        } else {
            for (int i = 0; i < fpi; ++i) v |= (uint32_t)c[i] << (i * bits);
        }
        code[w] = (int32_t)v;
    }
}

/*
 * quantize_pack_last_dim_cuda on an fp16 tensor viewed as [rows, S] (quantization_cuda.cu:631-721):
 * the fp16 input is widened to fp32 (:641-642), quantized, and scale = (max-min)/(2^b-1) is
 * recomputed on the torch side in fp32 (:711) and then narrowed to fp16 together with min
 * (:715-718).  torch evaluates "tensor / host scalar" as tensor * (1/scalar) in the tensor's
 * dtype, so the returned scale is (max-min) * fl32(1/(2^b-1)) -- not the true quotient the
 * kernel used for the codes (:570).  The vectors from the real extension pin this (every fp32
 * scale of the fp32-input case differs otherwise).  The append forms below store the in-kernel
 * quotient instead (:51-53, :150-152, :232-234), hence the scale_by_division switch.
 */
static int quant_lastdim_f16(const h16 *x, int64_t rows, int64_t S, int G, int bits, int32_t *code,
                             h16 *scale, h16 *mn, int scale_by_division) {
    int rc = orc_quant_check(S, G, bits);
    if (rc) return rc;
    const int fpi = orc_features_per_int(bits);
    const int64_t ng = S / G, nw = S / fpi;
    const float qmax = (float)((1 << bits) - 1);
#pragma omp parallel
    {
        float *xf = (float *)malloc(sizeof(float) * (size_t)S);
        float *mnf = (float *)malloc(sizeof(float) * (size_t)(2 * ng + 2));
        float *mxf = mnf + ng + 1;
        int32_t *tmp = (int32_t *)malloc(sizeof(int32_t) * (size_t)S);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            for (int64_t i = 0; i < S; ++i) xf[i] = h2f(x[r * S + i]);
            quant_row(xf, S, G, bits, code + r * nw, mnf, mxf, tmp);
            for (int64_t g = 0; g < ng; ++g) {
                scale[r * ng + g] = scale_by_division ? f2h((mxf[g] - mnf[g]) / qmax)
                                                      : f2h((mxf[g] - mnf[g]) * (1.0f / qmax));
                mn[r * ng + g] = f2h(mnf[g]);
            }
        }
        free(xf); free(mnf); free(tmp);
    }
    return 0;
}

int orc_quant_lastdim_f16(const h16 *x, int64_t rows, int64_t S, int G, int bits, int32_t *code,
                          h16 *scale, h16 *mn) {
    return quant_lastdim_f16(x, rows, S, G, bits, code, scale, mn, 0);
}

/* Same for an fp32 tensor: scale and min stay fp32 (quantization_cuda.cu:641,715). */
int orc_quant_lastdim_f32(const float *x, int64_t rows, int64_t S, int G, int bits, int32_t *code,
                          float *scale, float *mn) {
    int rc = orc_quant_check(S, G, bits);
    if (rc) return rc;
    const int fpi = orc_features_per_int(bits);
    const int64_t ng = S / G, nw = S / fpi;
    const float qmax = (float)((1 << bits) - 1);
#pragma omp parallel
    {
        float *mxf = (float *)malloc(sizeof(float) * (size_t)(ng + 1));
        int32_t *tmp = (int32_t *)malloc(sizeof(int32_t) * (size_t)S);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            quant_row(x + r * S, S, G, bits, code + r * nw, mn + r * ng, mxf, tmp);
            for (int64_t g = 0; g < ng; ++g) scale[r * ng + g] = (mxf[g] - mn[r * ng + g]) * (1.0f / qmax);
        }
        free(mxf); free(tmp);
    }
    return 0;
}

/*
 * EXTENSION -- no upstream counterpart, so nothing pins it ("parity unpinned"): 3-bit quantization of rows whose
 * length S is not a multiple of 11.  Upstream rejects such rows (quantization_cuda.cu:649, and :433-434 for the
 * value form), which rules out 3-bit values at head_dim 128.  The rule here is upstream's 3-bit group rule
 * (:553-596, word packing :612-626) applied to groups of 11 with a last group of S % 11 elements: every group is one
 * word; min/max, scale = (max-min)/7 and codes over the elements the group has; element 10 of a full group keeps
 * upstream's 2-bit field (clamped at 3, :579); unused fields of the last word are 0.
 *   code [rows, ceil(S/11)] int32, scale/mn [rows, ceil(S/11)] fp16; stored scale as in quant_lastdim_f16.
 */
int orc_quant_ragged3_f16(const h16 *x, int64_t rows, int64_t S, int32_t *code, h16 *scale, h16 *mn,
                          int scale_by_division) {
    if (S <= 0) return -4;
    const int64_t nw = (S + 10) / 11;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t w = 0; w < nw; ++w) {
            const int n = (int)((S - w * 11) < 11 ? (S - w * 11) : 11);
            float v[11], lo = FLT_MAX, hi = -FLT_MAX;
            for (int i = 0; i < n; ++i) {
                v[i] = h2f(x[r * S + w * 11 + i]);
                lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]);
            }
            const float sc = (hi - lo) / 7.0f;
            uint32_t word = 0;
            for (int i = 0; i < n; ++i) {
                const float nrm = (v[i] - lo) / sc;
                int q = isnan(nrm) ? 0 : (int)roundf(nrm);
                const int emax = i >= 10 ? 3 : 7;
                if (q > emax) q = emax;
                if (q < 0) q = 0;
                word |= (uint32_t)q << (i < 10 ? 3 * i : 30);
            }
            code[r * nw + w] = (int32_t)word;
            scale[r * nw + w] = scale_by_division ? f2h((hi - lo) / 7.0f) : f2h((hi - lo) * (1.0f / 7.0f));
            mn[r * nw + w] = f2h(lo);
        }
    }
    return 0;
}

/*
 * quantized_gemm + execute_quantized_matvec, quant_cuda/csrc/dequantization_gemv_cuda.cu:7-124
 * (kernel) and :127-248 (shape algebra), for M = 1 (the kernel never reads blockIdx.z, so only
 * M = 1 is meaningful).
 *
 * Caller layout (before the transposes upstream performs at :151-171):
 *   fA     [B, nh,    1, K]        fp16
 *   qB     [B, nh_kv, K, N/fpi]    int32
 *   scales [B, nh_kv, K, N/G]      fp16     zeros: same
 *   out    [B, nh,    1, N]        fp16,  N = (N/G) * G   (:184)
 *
 * The upstream kernel works on the transposed operands ([N/fpi, K], [N/G, K]); here the
 * untransposed arrays are indexed directly, which addresses the same elements.  Summation
 * order is upstream's: lane l of 32 takes k = 128*chunk + 4*l + seg (:50-56,75), one scale and
 * zero per packed word taken at group (word*fpi)/G (:24,53), fp32 fma chain per lane, then
 * the shuffle-down tree 16,8,4,2,1 read at lane 0 (:112-121), narrowed with round-to-nearest.
 */
int orc_gemv(int G, const h16 *fA, const int32_t *qB, const h16 *scales, const h16 *zeros, int bits,
             int64_t B, int64_t nh, int64_t nh_kv, int64_t K, int64_t n_words, int64_t n_groups,
             h16 *out) {
    if (bits < 1 || bits > 4) return -1;                        /* :174-176 */
    if (nh_kv <= 0 || nh % nh_kv != 0) return -6;               /* :177-178 */
    if (bits == 3 && G != 11) return -2;                        /* :203 */
    const int fpi = orc_features_per_int(bits);
    const int64_t N = n_groups * G;                             /* :184 */
    const int64_t n_pack = N / fpi;                             /* grid.y*4 covers ceil(N/fpi) */
    if (n_pack > n_words) return -7;
    const int64_t rep = nh / nh_kv;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t s = 0; s < B * nh; ++s) {
        for (int64_t pg = 0; pg < n_pack; ++pg) {
            const int64_t wb = s / rep;                         /* :28-30 */
            const h16 *in = fA + s * K;
            const int32_t *wbase = qB + wb * K * n_words;
            const h16 *sbase = scales + wb * K * n_groups;
            const h16 *zbase = zeros + wb * K * n_groups;
            const int64_t grp = (pg * fpi) / G;                 /* :24 */
            float lane_acc[32][32];
            for (int l = 0; l < 32; ++l)
                for (int e = 0; e < fpi; ++e) lane_acc[l][e] = 0.0f;
            for (int64_t k0 = 0; k0 < K; k0 += 128) {
                for (int l = 0; l < 32; ++l) {
                    for (int seg = 0; seg < 4; ++seg) {
                        const int64_t k = k0 + 4 * l + seg;
                        if (k >= K) continue;                   /* zero input beyond K (:68-71) */
                        uint32_t w = (uint32_t)wbase[k * n_words + pg];
                        const float x = h2f(in[k]);
                        const float sc = h2f(sbase[k * n_groups + grp]);
                        const float ze = h2f(zbase[k * n_groups + grp]);
                        if (bits == 3) {                        /* :81-95 */
                            for (int e = 0; e < 10; ++e) {
                                const float wv = (float)(w & 7u); w >>= 3;
                                lane_acc[l][e] = fmaf(fmaf(sc, wv, ze), x, lane_acc[l][e]);
                            }
                            const float wv = (float)(w & 3u);
                            lane_acc[l][10] = fmaf(fmaf(sc, wv, ze), x, lane_acc[l][10]);
                        } else {                                /* :98-104 */
                            for (int e = 0; e < fpi; ++e) {
                                const float wv = (float)(w & mask); w >>= bits;
                                lane_acc[l][e] = fmaf(fmaf(sc, wv, ze), x, lane_acc[l][e]);
                            }
                        }
                    }
                }
            }
            for (int e = 0; e < fpi; ++e) {                     /* :109-123 */
                float v[64];
                for (int l = 0; l < 32; ++l) { v[l] = lane_acc[l][e]; v[32 + l] = 0.0f; }
                for (int off = 16; off > 0; off >>= 1)
                    for (int l = 0; l < off; ++l) v[l] += v[l + off];
                out[s * N + pg * fpi + e] = f2h(v[0]);
            }
        }
    }
    return 0;
}

/*
 * Append forms: process_key_quantization_cuda (quantization_cuda.cu:298-411, kernels :12-185)
 * and process_value_quantization_cuda (:413-537, kernels :188-296).  Both return
 * concat(previous, quantize(new)) along the token axis; the new part uses exactly the group
 * arithmetic above (scale computed and applied in fp32, narrowed on return).
 *
 * Deliberate deviation: upstream's fused 3-bit key kernel (:108-185) never copies the previous
 * code words into its output (only scale and min, :131-134); this restatement copies them,
 * which is what the function's contract and its non-3-bit twin (:80-82) state.
 *
 * Key form:   new  [rows, Tn] fp16, prev_code [rows, old_w], prev_scale/min [rows, old_g]
 *             out  [rows, old_w + Tn/fpi], [rows, old_g + Tn/G]
 */
int orc_append_k_f16(const h16 *xnew, int64_t rows, int64_t Tn, const int32_t *prev_code, int64_t old_w,
                     const h16 *prev_scale, const h16 *prev_mn, int64_t old_g, int G, int bits,
                     int32_t *code, h16 *scale, h16 *mn) {
    if (bits < 1 || bits > 4) return -1;
    if (bits == 3) { if (G != 11) return -2; if (Tn % 11) return -3; }      /* :317-319 */
    else { if (Tn % G) return -4; if (Tn % (32 / bits)) return -5; if (G % (32 / bits)) return -8; }
    const int fpi = orc_features_per_int(bits);
    const int64_t nw = Tn / fpi, ng = Tn / G;
    int32_t *c_new = (int32_t *)malloc(sizeof(int32_t) * (size_t)(rows * nw + 1));
    h16 *s_new = (h16 *)malloc(sizeof(h16) * (size_t)(rows * ng + 1));
    h16 *m_new = (h16 *)malloc(sizeof(h16) * (size_t)(rows * ng + 1));
    int rc = quant_lastdim_f16(xnew, rows, Tn, G, bits, c_new, s_new, m_new, 1);
    if (rc == 0) {
        for (int64_t r = 0; r < rows; ++r) {
            memcpy(code + r * (old_w + nw), prev_code + r * old_w, sizeof(int32_t) * (size_t)old_w);
            memcpy(code + r * (old_w + nw) + old_w, c_new + r * nw, sizeof(int32_t) * (size_t)nw);
            memcpy(scale + r * (old_g + ng), prev_scale + r * old_g, sizeof(h16) * (size_t)old_g);
            memcpy(scale + r * (old_g + ng) + old_g, s_new + r * ng, sizeof(h16) * (size_t)ng);
            memcpy(mn + r * (old_g + ng), prev_mn + r * old_g, sizeof(h16) * (size_t)old_g);
            memcpy(mn + r * (old_g + ng) + old_g, m_new + r * ng, sizeof(h16) * (size_t)ng);
        }
    }
    free(c_new); free(s_new); free(m_new);
    return rc;
}

/*
 * Value form: new [bh, Tn, D] fp16, prev_code [bh, Told, D/fpi], prev_scale/min [bh, Told, D/G];
 *             out [bh, Told+Tn, D/fpi], [bh, Told+Tn, D/G].  D % G == 0 (:432-437).
 */
int orc_append_v_f16(const h16 *xnew, int64_t bh, int64_t Tn, int64_t D, const int32_t *prev_code,
                     const h16 *prev_scale, const h16 *prev_mn, int64_t Told, int G, int bits,
                     int32_t *code, h16 *scale, h16 *mn) {
    int rc = orc_quant_check(D, G, bits);
    if (rc) return rc;
    const int fpi = orc_features_per_int(bits);
    const int64_t wpt = D / fpi, gpt = D / G;
    for (int64_t r = 0; r < bh; ++r) {
        memcpy(code + r * (Told + Tn) * wpt, prev_code + r * Told * wpt, sizeof(int32_t) * (size_t)(Told * wpt));
        memcpy(scale + r * (Told + Tn) * gpt, prev_scale + r * Told * gpt, sizeof(h16) * (size_t)(Told * gpt));
        memcpy(mn + r * (Told + Tn) * gpt, prev_mn + r * Told * gpt, sizeof(h16) * (size_t)(Told * gpt));
        rc = quant_lastdim_f16(xnew + r * Tn * D, Tn, D, G, bits, code + (r * (Told + Tn) + Told) * wpt,
                               scale + (r * (Told + Tn) + Told) * gpt, mn + (r * (Told + Tn) + Told) * gpt, 1);
        if (rc) return rc;
    }
    return 0;
}

/*
 * Decode attention for one query token, the cached branch of LlamaAttention_KVmix.forward,
 * models/modeling_llama_KVmix.py:170-211 (Mistral twin models/modeling_mistral_KVmix.py:207-262),
 * with upstream's rounding points when ref_rounding != 0:
 *   R1 q.Kq      -> fp16   (dequantization_gemv_cuda.cu:120)
 *   R2 q.Kfull^T -> fp16   (modeling_llama_KVmix.py:185, fp16 matmul)
 *   R3 concat as fp32, divide by sqrt(D) (:68-75)
 *   R4 softmax in fp32, probabilities -> fp16 (:194)
 *   R5 p.Vq -> fp16 (GEMV) and p.Vfull -> fp16 (:205-210)
 *   R6 fp16 sum of the two (:211)
 * ref_rounding is a bit mask: 1 = R1+R2, 2 = R4, 4 = R5+R6 (7 = upstream).  With 0 nothing is
 * narrowed before the final fp16 store (fp32-accumulate mode).
 * GQA: query head h reads kv head h / (nh / nh_kv), which is what repeat_kv_quant
 * (modeling_llama_KVmix.py:19-28) materialises.  The quantized products use plain fp32
 * accumulation here (order differs from the GEMV tree above by rounding noise only).
 *
 *   q       [B, nh, D] fp16
 *   kcode   [B, nh_kv, D, Tkq/fpi_k], kscale/kmn [B, nh_kv, D, Tkq/Gk]
 *   kfull   [B, nh_kv, Rk, D]   fp16, tokens Tkq .. Tkq+Rk-1
 *   vcode   [B, nh_kv, Tvq, D/fpi_v], vscale/vmn [B, nh_kv, Tvq, D/Gv]
 *   vfull   [B, nh_kv, Rv, D]   fp16, tokens Tvq .. Tvq+Rv-1;  Tkq+Rk == Tvq+Rv == T
 *   out     [B, nh, D] fp16
 */
int orc_decode_attn(const h16 *q, const int32_t *kcode, const h16 *kscale, const h16 *kmn, const h16 *kfull,
                    const int32_t *vcode, const h16 *vscale, const h16 *vmn, const h16 *vfull, int64_t B,
                    int64_t nh, int64_t nh_kv, int64_t D, int64_t Tkq, int64_t Rk, int64_t Tvq, int64_t Rv,
                    int kbits, int Gk, int vbits, int Gv, int ref_rounding, const float *mask, int64_t mask_heads,
                    h16 *out) {
    if (Tkq + Rk != Tvq + Rv) return -9;
    if (nh % nh_kv) return -6;
    if (vbits == 3 && Gv != 11) return -2;
    /* vbits == 3 with D % 11 != 0 is the extension format of orc_quant_ragged3_f16 (upstream cannot hold such V,
     * quantization_cuda.cu:433-434): ceil(D/11) words and groups per token, the last one short */
    const int64_t T = Tkq + Rk, rep = nh / nh_kv;
    const int fk = orc_features_per_int(kbits), fv = orc_features_per_int(vbits);
    const int64_t kw = Tkq / fk, kg = Tkq ? Tkq / Gk : 0, vw = (D + fv - 1) / fv, vg = (D + Gv - 1) / Gv;
#pragma omp parallel
    {
        float *sc = (float *)malloc(sizeof(float) * (size_t)(T + 1));
        float *acc_q = (float *)malloc(sizeof(float) * (size_t)D * 2);
        float *acc_f = acc_q + D;
#pragma omp for schedule(static)
        for (int64_t s = 0; s < B * nh; ++s) {
            const int64_t b = s / nh, h = s % nh, hk = h / rep, kv = b * nh_kv + hk;
            const h16 *qv = q + s * D;
            for (int64_t t = 0; t < Tkq; ++t) sc[t] = 0.0f;
            for (int64_t d = 0; d < D; ++d) {
                const float x = h2f(qv[d]);
                const int32_t *cw = kcode + (kv * D + d) * kw;
                const h16 *sp = kscale + (kv * D + d) * kg, *zp = kmn + (kv * D + d) * kg;
                for (int64_t w = 0; w < kw; ++w) {
                    uint32_t v = (uint32_t)cw[w];
                    const int64_t g = (w * fk) / Gk;
                    const float scl = h2f(sp[g]), ze = h2f(zp[g]);
                    for (int e = 0; e < fk; ++e) {
                        int nb = (kbits == 3) ? (e < 10 ? 3 : 2) : kbits;
                        float c = (float)(v & ((1u << nb) - 1u)); v >>= nb;
                        sc[w * fk + e] = fmaf(fmaf(scl, c, ze), x, sc[w * fk + e]);
                    }
                }
            }
            if (ref_rounding & 1) for (int64_t t = 0; t < Tkq; ++t) sc[t] = h2f(f2h(sc[t]));      /* R1 */
            for (int64_t r = 0; r < Rk; ++r) {
                const h16 *kr = kfull + (kv * Rk + r) * D;
                float a = 0.0f;
                for (int64_t d = 0; d < D; ++d) a = fmaf(h2f(qv[d]), h2f(kr[d]), a);
                sc[Tkq + r] = (ref_rounding & 1) ? h2f(f2h(a)) : a;                                /* R2 */
            }
            float mx = -FLT_MAX;
            /* additive mask [B, mask_heads (1 or nh), T], then clamp at finfo(float32).min: modeling_llama_KVmix.py:188-192 */
            const float *mrow = mask ? mask + (b * mask_heads + (mask_heads == 1 ? 0 : h)) * T : 0;
            for (int64_t t = 0; t < T; ++t) {
                sc[t] = sc[t] / sqrtf((float)D);                                                     /* R3 */
                if (mrow) sc[t] = fmaxf(sc[t] + mrow[t], -FLT_MAX);
                mx = fmaxf(mx, sc[t]);
            }
            float sum = 0.0f;
            for (int64_t t = 0; t < T; ++t) { sc[t] = expf(sc[t] - mx); sum += sc[t]; }
            for (int64_t t = 0; t < T; ++t) {
                sc[t] = sc[t] / sum;
                if (ref_rounding & 2) sc[t] = h2f(f2h(sc[t]));                                     /* R4 */
            }
            for (int64_t d = 0; d < D; ++d) { acc_q[d] = 0.0f; acc_f[d] = 0.0f; }
            for (int64_t t = 0; t < Tvq; ++t) {
                const float p = sc[t];
                const int32_t *cw = vcode + (kv * Tvq + t) * vw;
                const h16 *sp = vscale + (kv * Tvq + t) * vg, *zp = vmn + (kv * Tvq + t) * vg;
                for (int64_t w = 0; w < vw; ++w) {
                    uint32_t v = (uint32_t)cw[w];
                    const int64_t g = (w * fv) / Gv;
                    const float scl = h2f(sp[g]), ze = h2f(zp[g]);
                    for (int e = 0; e < fv && w * fv + e < D; ++e) {
                        int nb = (vbits == 3) ? (e < 10 ? 3 : 2) : vbits;
                        float c = (float)(v & ((1u << nb) - 1u)); v >>= nb;
                        acc_q[w * fv + e] = fmaf(fmaf(scl, c, ze), p, acc_q[w * fv + e]);
                    }
                }
            }
            for (int64_t r = 0; r < Rv; ++r) {
                const float p = sc[Tvq + r];
                const h16 *vr = vfull + (kv * Rv + r) * D;
                for (int64_t d = 0; d < D; ++d) acc_f[d] = fmaf(p, h2f(vr[d]), acc_f[d]);
            }
            for (int64_t d = 0; d < D; ++d) {
                if (ref_rounding & 4) {
                    float a = Tvq ? h2f(f2h(acc_q[d])) : 0.0f, f = h2f(f2h(acc_f[d]));            /* R5 */
                    out[s * D + d] = Tvq ? f2h(a + f) : f2h(acc_f[d]);                              /* R6 */
                } else {
                    out[s * D + d] = f2h(acc_q[d] + acc_f[d]);
                }
            }
        }
        free(sc); free(acc_q);
    }
    return 0;
}
