// Fused decode attention over a mixed-precision KV cache (packed prefix + fp16 tail), one query
// token per sequence.  One launch replaces upstream's two GEMV launches, repeat_kv copies, two fp16
// matmuls, concat, softmax and add (models/modeling_llama_KVmix.py:170-211).
//
// Work decomposition: CTA = (split of the token axis, query head).  Each CTA
//   1. scores its token range: packed keys are read word-column-wise (lanes on consecutive words
//      of one channel row, so every warp load is one contiguous run), the per-channel scale is
//      folded into the query once per word and the zero term accumulated once per word;
//      fp16 tail keys are scored one warp per token;
//   2. takes max / exp / sum over its range in shared memory;
//   3. accumulates p.V: packed values with lanes on consecutive words of a token row, fp16 tail
//      values with lanes on channel pairs; partial sums meet in shared memory in a fixed order;
//   4. writes (acc, max, sum) for its split; the last CTA of a head to finish (one counter per
//      head) merges the splits in index order, so results are run-to-run identical.
#include "common.cuh"
#include "attn_plan.cuh"

namespace kvq {

constexpr int kAttnThreads = 256;
constexpr int kMaxChunk = 4224;  // tokens per split held in shared memory (multiple of 128 and of 352)

struct SplitPlan {
    int chunk, n_splits;
};

// Generic kernel: splits start on a packed-word and key-group boundary: multiples of 128 tokens, or of
// 352 = 11*32 for 3-bit keys (11 tokens per word).
static SplitPlan plan_splits_generic(int T, int k_bits, int64_t heads) {
    const int unit = (k_bits == 3) ? 352 : 128;
    const int64_t want_ctas = 148 * 4;
    int64_t n = (T + kMaxChunk - 1) / kMaxChunk;
    const int64_t by_fill = (want_ctas + heads - 1) / heads;
    const int64_t by_len = (T + 4 * unit - 1) / (4 * unit);   // keep splits long
    n = n > (by_fill < by_len ? by_fill : by_len) ? n : (by_fill < by_len ? by_fill : by_len);
    if (n < 1) n = 1;
    int chunk = (int)((T + n - 1) / n);
    chunk = ((chunk + unit - 1) / unit) * unit;
    if (chunk > kMaxChunk) chunk = (kMaxChunk / unit) * unit;
    SplitPlan p;
    p.chunk = chunk;
    p.n_splits = (T + chunk - 1) / chunk;
    return p;
}

struct Smem {
    float q[kHeadDim];
    float scores[kMaxChunk];
    float red[12][kHeadDim];
    float warp_red[8];
    float bcast[2];
    int last;
};

template <int KB>
__device__ __forceinline__ void score_packed(const kvq_attn_args &a, const int32_t *kc, const __half *ks,
                                             const __half *kz, Smem &sm, int t0, int lo, int hi) {
    constexpr int FPI = fields_per_word(KB);
    for (int w = lo / FPI + threadIdx.x; w < hi / FPI; w += kAttnThreads) {
        const int grp = (w * FPI) / a.k_group;
        float acc[FPI];
#pragma unroll
        for (int i = 0; i < FPI; ++i) acc[i] = 0.f;
        float zacc = 0.f;
#pragma unroll 4
        for (int d = 0; d < kHeadDim; ++d) {
            const uint32_t word = (uint32_t)__ldg(kc + d * a.kc_sD + w);
            const float x = sm.q[d];
            const float xs = x * __half2float(__ldg(ks + d * a.ks_sD + grp));
            zacc = fmaf(x, __half2float(__ldg(kz + d * a.ks_sD + grp)), zacc);
#pragma unroll
            for (int i = 0; i < FPI; ++i) acc[i] = fmaf(xs, (float)field<KB>(word, i), acc[i]);
        }
#pragma unroll
        for (int i = 0; i < FPI; ++i) {
            float s = acc[i] + zacc;
            if (a.round_scores) s = __half2float(__float2half_rn(s));
            sm.scores[w * FPI + i - t0] = s * a.softmax_scale;
        }
    }
}

template <int VB>
__device__ __forceinline__ void pv_packed(const kvq_attn_args &a, const int32_t *vc, const __half *vs,
                                          const __half *vz, Smem &sm, int t0, int lo, int hi) {
    constexpr int FPI = fields_per_word(VB);
    constexpr int WPT = kHeadDim / FPI;      // words per token row
    constexpr int TL = kAttnThreads / WPT;   // token lanes
    const int j = threadIdx.x % WPT, tl = threadIdx.x / WPT;
    const int grp = (j * FPI) / a.v_group;
    float acc[FPI];
#pragma unroll
    for (int i = 0; i < FPI; ++i) acc[i] = 0.f;
    float zacc = 0.f;
    for (int t = lo + tl; t < hi; t += TL) {
        const uint32_t word = (uint32_t)__ldg(vc + (int64_t)t * a.vc_sT + j);
        const float p = sm.scores[t - t0];
        const float ps = p * __half2float(__ldg(vs + (int64_t)t * a.vs_sT + grp));
        zacc = fmaf(p, __half2float(__ldg(vz + (int64_t)t * a.vs_sT + grp)), zacc);
#pragma unroll
        for (int i = 0; i < FPI; ++i) acc[i] = fmaf(ps, (float)field<VB>(word, i), acc[i]);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < FPI; ++i) {
        float v = acc[i] + zacc;
#pragma unroll
        for (int o = WPT; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane < WPT) sm.red[warp][j * FPI + i] = v;
    }
}

// 3-bit values, an extension upstream does not have (its 3-bit rule needs head_dim % 11 == 0): 12 words per token
// row, word j holding channels 11j .. min(11j + 10, 127) and being its own group (scale/zero j).  16 lane slots per
// token of which 12 work, 16 tokens per pass.
__device__ __forceinline__ void pv_packed3(const kvq_attn_args &a, const int32_t *vc, const __half *vs,
                                           const __half *vz, Smem &sm, int t0, int lo, int hi) {
    constexpr int WPT = (kHeadDim + 10) / 11;
    const int j = threadIdx.x & 15, tl = threadIdx.x >> 4;
    float acc[11];
#pragma unroll
    for (int i = 0; i < 11; ++i) acc[i] = 0.f;
    float zacc = 0.f;
    if (j < WPT) {
        for (int t = lo + tl; t < hi; t += kAttnThreads / 16) {
            const uint32_t word = (uint32_t)__ldg(vc + (int64_t)t * a.vc_sT + j);
            const float p = sm.scores[t - t0];
            const float ps = p * __half2float(__ldg(vs + (int64_t)t * a.vs_sT + j));
            zacc = fmaf(p, __half2float(__ldg(vz + (int64_t)t * a.vs_sT + j)), zacc);
#pragma unroll
            for (int i = 0; i < 11; ++i) acc[i] = fmaf(ps, (float)field<3>(word, i), acc[i]);
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 11; ++i) {
        float v = acc[i] + zacc;
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane < WPT && j * 11 + i < kHeadDim) sm.red[warp][j * 11 + i] = v;
    }
}

__global__ void __launch_bounds__(kAttnThreads) decode_attn_kernel(kvq_attn_args a, int chunk, int n_splits,
                                                                  float *__restrict__ parts,
                                                                  unsigned int *__restrict__ counters) {
    __shared__ Smem sm;
    const int split = blockIdx.x % n_splits;
    const int s = blockIdx.x / n_splits;  // b * nh + h
    const int b = s / a.nh, h = s % a.nh, hk = h / (a.nh / a.nh_kv);
    const int t0 = split * chunk, t1 = min(a.T, t0 + chunk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const __half *q = static_cast<const __half *>(a.q) + (int64_t)b * a.q_sB + (int64_t)h * a.q_sH;
    if (tid < kHeadDim) sm.q[tid] = __half2float(q[tid]);
    for (int i = tid; i < 12 * kHeadDim; i += kAttnThreads) (&sm.red[0][0])[i] = 0.f;
    __syncthreads();

    // ---- 1. scores --------------------------------------------------------------------------
    {
        const int hi = min(t1, a.Tkq);
        if (t0 < hi) {
            const int32_t *kc = a.kcode + (int64_t)b * a.kc_sB + (int64_t)hk * a.kc_sH;
            const __half *ks = static_cast<const __half *>(a.kscale) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            const __half *kz = static_cast<const __half *>(a.kmn) + (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH;
            switch (a.k_bits) {
                case 1: score_packed<1>(a, kc, ks, kz, sm, t0, t0, hi); break;
                case 2: score_packed<2>(a, kc, ks, kz, sm, t0, t0, hi); break;
                case 3: score_packed<3>(a, kc, ks, kz, sm, t0, t0, hi); break;
                default: score_packed<4>(a, kc, ks, kz, sm, t0, t0, hi); break;
            }
        }
        const int lo = max(t0, a.Tkq);
        if (lo < t1) {
            const __half *kf = static_cast<const __half *>(a.kfull) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH;
            const float4 qv = *reinterpret_cast<const float4 *>(&sm.q[4 * lane]);
            for (int t = lo + warp; t < t1; t += kAttnThreads / 32) {
                int slot = a.kf_start + (t - a.Tkq);
                if (slot >= a.kf_cap) slot -= a.kf_cap;
                const uint2 u = __ldg(reinterpret_cast<const uint2 *>(kf + (int64_t)slot * a.kf_sT) + lane);
                const float2 k01 = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
                const float2 k23 = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
                float v = qv.x * k01.x + qv.y * k01.y + qv.z * k23.x + qv.w * k23.y;
                v = warp_sum(v);
                if (lane == 0) {
                    if (a.round_scores) v = __half2float(__float2half_rn(v));
                    sm.scores[t - t0] = v * a.softmax_scale;
                }
            }
        }
    }
    __syncthreads();

    // ---- 2. softmax numerators over this split ------------------------------------------------
    const int n = t1 - t0;
    float m = kMaskFloor;                                      // a fully masked range then weighs uniformly, as upstream's does
    if (a.mask) {                                              // weights + mask, clamped at the fp32 floor
        for (int i = tid; i < n; i += kAttnThreads) {
            const float v = fmaxf(sm.scores[i] + attn_mask_at(a, b, h, t0 + i), kMaskFloor);
            sm.scores[i] = v;
            m = fmaxf(m, v);
        }
    } else {
        for (int i = tid; i < n; i += kAttnThreads) m = fmaxf(m, sm.scores[i]);
    }
    m = warp_max(m);
    if (lane == 0) sm.warp_red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float v = sm.warp_red[0];
        for (int i = 1; i < 8; ++i) v = fmaxf(v, sm.warp_red[i]);
        sm.bcast[0] = v;
    }
    __syncthreads();
    m = sm.bcast[0];
    float l = 0.f;
    for (int i = tid; i < n; i += kAttnThreads) {
        const float p = __expf(sm.scores[i] - m);
        sm.scores[i] = p;
        l += p;
    }
    l = warp_sum(l);
    __syncthreads();
    if (lane == 0) sm.warp_red[warp] = l;
    __syncthreads();
    if (tid == 0) {
        float v = 0.f;
        for (int i = 0; i < 8; ++i) v += sm.warp_red[i];
        sm.bcast[1] = v;
    }
    __syncthreads();
    l = sm.bcast[1];

    // ---- 3. p.V ---------------------------------------------------------------------------------
    {
        const int hi = min(t1, a.Tvq);
        if (t0 < hi) {
            const int32_t *vc = a.vcode + (int64_t)b * a.vc_sB + (int64_t)hk * a.vc_sH;
            const __half *vs = static_cast<const __half *>(a.vscale) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
            const __half *vz = static_cast<const __half *>(a.vmn) + (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH;
            switch (a.v_bits) {
                case 1: pv_packed<1>(a, vc, vs, vz, sm, t0, t0, hi); break;
                case 2: pv_packed<2>(a, vc, vs, vz, sm, t0, t0, hi); break;
                case 3: pv_packed3(a, vc, vs, vz, sm, t0, t0, hi); break;
                default: pv_packed<4>(a, vc, vs, vz, sm, t0, t0, hi); break;
            }
        }
        const int lo = max(t0, a.Tvq);
        if (lo < t1) {
            const __half *vf = static_cast<const __half *>(a.vfull) + (int64_t)b * a.vf_sB + (int64_t)hk * a.vf_sH;
            const int c = tid & 63, tl = tid >> 6;
            float2 acc = make_float2(0.f, 0.f);
            for (int t = lo + tl; t < t1; t += 4) {
                int slot = a.vf_start + (t - a.Tvq);
                if (slot >= a.vf_cap) slot -= a.vf_cap;
                const __half2 hv = __ldg(reinterpret_cast<const __half2 *>(vf + (int64_t)slot * a.vf_sT) + c);
                const float2 f = __half22float2(hv);
                const float p = sm.scores[t - t0];
                acc.x = fmaf(p, f.x, acc.x);
                acc.y = fmaf(p, f.y, acc.y);
            }
            sm.red[8 + tl][2 * c] = acc.x;
            sm.red[8 + tl][2 * c + 1] = acc.y;
        }
    }
    __syncthreads();

    // ---- 4. finish / merge ---------------------------------------------------------------------
    float o = 0.f;
    if (tid < kHeadDim) {
#pragma unroll
        for (int r = 0; r < 12; ++r) o += sm.red[r][tid];
    }
    __half *out = static_cast<__half *>(a.out) + (int64_t)b * a.o_sB + (int64_t)h * a.o_sH;
    if (n_splits == 1) {
        if (tid < kHeadDim) out[tid] = __float2half_rn(o / l);
        return;
    }
    float *part = parts + ((int64_t)s * n_splits + split) * kPartStride;
    if (tid < kHeadDim) part[tid] = o;
    if (tid == 0) { part[kHeadDim] = m; part[kHeadDim + 1] = l; }
    __threadfence();
    __syncthreads();
    if (tid == 0) sm.last = (atomicAdd(&counters[s], 1u) == (unsigned)(n_splits - 1));
    __syncthreads();
    if (!sm.last) return;
    __threadfence();
    const float *base = parts + (int64_t)s * n_splits * kPartStride;
    float M = kMaskFloor;
    for (int i = 0; i < n_splits; ++i) M = fmaxf(M, __ldcg(base + i * kPartStride + kHeadDim));
    if (tid < kHeadDim) {
        float L = 0.f, acc = 0.f;
        for (int i = 0; i < n_splits; ++i) {
            const float w = __expf(__ldcg(base + i * kPartStride + kHeadDim) - M);
            L = fmaf(__ldcg(base + i * kPartStride + kHeadDim + 1), w, L);
            acc = fmaf(__ldcg(base + i * kPartStride + tid), w, acc);
        }
        out[tid] = __float2half_rn(acc / L);
    }
    if (tid == 0) counters[s] = 0u;                          // ready for the next launch
}

// tensor-core paths (decode_attn_mma.cu: one query head per segment; decode_attn_gqa.cu: the query heads of a kv
// head share a segment)
bool mma_path_eligible(const kvq_attn_args &a);
AttnPlan plan_attn_mma(int T, int k_bits, long long heads);
int launch_decode_attn_mma(const kvq_attn_args &a, const AttnPlan &plan, float *parts, unsigned int *counters,
                           cudaStream_t st);
int gqa_heads_per_cta(const kvq_attn_args &a);
AttnPlan plan_attn_gqa(int T, int k_bits, long long head_groups);
int launch_decode_attn_gqa(const kvq_attn_args &a, const AttnPlan &plan, int qhv, float *parts, unsigned int *counters,
                           cudaStream_t st);

// Upper bound, over every shorter context and every kernel, of the partial results (one per query head and segment)
// a call may hold: the generic kernel's heads x splits; for the tensor-core kernels either what the score buffers
// force (a segment holds at most 8192 tokens, 2048 / 2816 when four query heads share it) or the planner's own cap of
// kMaxCtaRounds waves of CTAs over the cut heads (attn_plan.cuh), whichever is larger.
static int64_t max_partials_bound(int T, int64_t heads) {
    int64_t n = heads;
    for (int kb = 3; kb <= 4; ++kb) {
        const int64_t g = heads * plan_splits_generic(T, kb, heads).n_splits;
        n = g > n ? g : n;
    }
    const int64_t forced = heads * ((T + 1759) / 1760);
    const int64_t capped = (int64_t)kMaxCtaRounds * kSmCount * 3 * 4 + heads;
    n = forced > n ? forced : n;
    return capped > n ? capped : n;
}

struct AttnLaunch {
    bool use_mma;
    int qhv;             // query heads per CTA (grouped kernel), 0 otherwise
    AttnPlan mplan;
    SplitPlan gplan;
    int64_t heads, ctas, partials;
};

static AttnLaunch plan_launch(const kvq_attn_args &a) {
    AttnLaunch L = {};
    L.heads = (int64_t)a.B * a.nh;
    L.use_mma = mma_path_eligible(a);
    L.qhv = L.use_mma ? gqa_heads_per_cta(a) : 0;
    L.gplan = {0, 1};
    if (L.qhv) {
        L.mplan = plan_attn_gqa(a.T, a.k_bits, L.heads / L.qhv);
        L.ctas = (int64_t)L.mplan.n_whole + (int64_t)L.mplan.n_cut * L.mplan.k;
        L.partials = L.mplan.k > 1 ? (int64_t)L.mplan.n_cut * L.mplan.k * L.qhv : 0;
    } else if (L.use_mma) {
        L.mplan = plan_attn_mma(a.T, a.k_bits, L.heads);
        L.ctas = (int64_t)L.mplan.n_whole + (int64_t)L.mplan.n_cut * L.mplan.k;
        L.partials = L.mplan.k > 1 ? (int64_t)L.mplan.n_cut * L.mplan.k : 0;
    } else {
        L.gplan = plan_splits_generic(a.T, a.k_bits, L.heads);
        L.ctas = L.heads * L.gplan.n_splits;
        L.partials = L.gplan.n_splits > 1 ? L.ctas : 0;
    }
    return L;
}

}  // namespace kvq

extern "C" uint64_t kvq_decode_attn_workspace_bytes(int32_t B, int32_t nh, int32_t T) {
    using namespace kvq;
    if (B <= 0 || nh <= 0 || T <= 0) return 256;
    const int64_t heads = (int64_t)B * nh;
    uint64_t bytes = (uint64_t)heads * 4;
    bytes = (bytes + 255) / 256 * 256;
    bytes += (uint64_t)max_partials_bound(T, heads) * kPartStride * 4;
    return (bytes + 255) / 256 * 256;
}

extern "C" int kvq_decode_attn_workspace_init(void *workspace, uint64_t bytes, int32_t B, int32_t nh, kvq_stream_t stream) {
    using namespace kvq;
    if (!workspace) return KVQ_ERR_NULL;
    if (B <= 0 || nh <= 0) return KVQ_OK;
    const uint64_t cbytes = ((uint64_t)B * nh * 4 + 255) / 256 * 256;
    if (bytes < cbytes) return KVQ_ERR_WORKSPACE;
    return record_cuda_error(cudaMemsetAsync(workspace, 0, cbytes, reinterpret_cast<cudaStream_t>(stream)));
}

extern "C" int kvq_decode_attn_plan(const kvq_attn_args *a, int32_t tensor_core, kvq_attn_plan *out) {
    using namespace kvq;
    if (!a || !out) return KVQ_ERR_NULL;
    if (a->k_bits < 1 || a->k_bits > 4 || a->v_bits < 1 || a->v_bits > 4) return KVQ_ERR_BITS;
    if (a->B <= 0 || a->nh <= 0 || a->T <= 0) return KVQ_ERR_SHAPE;
    if (a->nh_kv <= 0 || a->nh % a->nh_kv != 0) return KVQ_ERR_HEADS;
    const int64_t heads = (int64_t)a->B * a->nh;
    if (tensor_core < 0) tensor_core = mma_path_eligible(*a) ? 1 : 0;      // what kvq_decode_attn itself would pick
    if (tensor_core) {
        const int qhv = gqa_heads_per_cta(*a);
        const AttnPlan p = qhv ? plan_attn_gqa(a->T, a->k_bits, heads / qhv) : plan_attn_mma(a->T, a->k_bits, heads);
        out->kernel = qhv ? 2 : 1;
        out->heads_per_cta = qhv ? qhv : 1;
        out->unit = p.unit;
        out->units_per_head = p.uph;
        out->n_whole = p.n_whole;
        out->n_cut = p.n_cut;
        out->segments = p.k;
        out->segment_units = p.seg_units;
        out->n_ctas = p.n_whole + p.n_cut * p.k;
        out->max_segment_tokens = p.n_scores;
    } else {
        const SplitPlan p = plan_splits_generic(a->T, a->k_bits, heads);
        out->kernel = 0;
        out->heads_per_cta = 1;
        out->unit = p.chunk;
        out->units_per_head = p.n_splits;
        out->n_whole = 0;
        out->n_cut = (int32_t)heads;
        out->segments = p.n_splits;
        out->segment_units = 1;
        out->n_ctas = (int32_t)(heads * p.n_splits);
        out->max_segment_tokens = p.chunk;
    }
    return KVQ_OK;
}

extern "C" int kvq_decode_attn(const kvq_attn_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->D != kHeadDim) return KVQ_ERR_UNSUPPORTED;
    if (a->B <= 0 || a->nh <= 0) return KVQ_OK;
    if (a->nh_kv <= 0 || a->nh % a->nh_kv != 0) return KVQ_ERR_HEADS;
    if (a->T <= 0 || a->Tkq < 0 || a->Tvq < 0 || a->Tkq > a->T || a->Tvq > a->T) return KVQ_ERR_TOKENS;
    if (a->k_bits < 1 || a->k_bits > 4 || a->v_bits < 1 || a->v_bits > 4) return KVQ_ERR_BITS;
    const int fk = fields_per_word(a->k_bits), fv = fields_per_word(a->v_bits);
    if (a->k_bits == 3 && a->k_group != 11) return KVQ_ERR_GROUP3;
    if (a->v_bits == 3 && a->v_group != 11) return KVQ_ERR_GROUP3;   // 3-bit values: the short-last-group extension layout
    if (a->k_group <= 0 || a->k_group % fk != 0 || a->v_group <= 0 || a->v_group % fv != 0) return KVQ_ERR_GROUPWORD;
    if (a->Tkq % a->k_group != 0) return KVQ_ERR_DIVGROUP;
    if (a->v_bits != 3 && kHeadDim % a->v_group != 0) return KVQ_ERR_DIVGROUP;
    if (!a->q || !a->out) return KVQ_ERR_NULL;
    if (a->Tkq > 0 && (!a->kcode || !a->kscale || !a->kmn)) return KVQ_ERR_NULL;
    if (a->Tvq > 0 && (!a->vcode || !a->vscale || !a->vmn)) return KVQ_ERR_NULL;
    const bool dev_state = a->state != nullptr;                // lengths live on the device: T here is only an upper bound
    const int Rk = a->T - a->Tkq, Rv = a->T - a->Tvq;
    if (!dev_state && Rk > 0 && (!a->kfull || a->kf_cap < Rk || a->kf_start < 0 || a->kf_start >= a->kf_cap)) return KVQ_ERR_SHAPE;
    if (!dev_state && Rv > 0 && (!a->vfull || a->vf_cap < Rv || a->vf_start < 0 || a->vf_start >= a->vf_cap)) return KVQ_ERR_SHAPE;
    if (dev_state && (!a->k_new || !a->kfull || !a->vfull || !a->kcode || !a->vcode || !a->kscale || !a->vscale || !a->kmn || !a->vmn))
        return KVQ_ERR_NULL;                                   // device-resident state comes with the fused decode step
    if (dev_state && a->window < 0 && !(a->k_ratio >= 0.0 && a->k_ratio < 1.0 && a->v_ratio >= 0.0 && a->v_ratio < 1.0))
        return KVQ_ERR_SHAPE;
    if (Rk > 0 && (reinterpret_cast<uintptr_t>(a->kfull) % 8 || a->kf_sB % 4 || a->kf_sH % 4 || a->kf_sT % 4))
        return KVQ_ERR_ALIGN;
    if (Rv > 0 && (reinterpret_cast<uintptr_t>(a->vfull) % 4 || a->vf_sB % 2 || a->vf_sH % 2 || a->vf_sT % 2))
        return KVQ_ERR_ALIGN;

    const AttnLaunch L = plan_launch(*a);
    if (L.ctas > 2147483647LL) return KVQ_ERR_UNSUPPORTED;
    if (a->n_peers != 0) {                                     // head-sharded exchange (see the header)
        if (a->n_peers < 0 || a->n_peers > KVQ_MAX_PEERS || a->peer_head0 < 0) return KVQ_ERR_SHAPE;
        if (!L.use_mma) return KVQ_ERR_UNSUPPORTED;
        for (int p = 0; p < a->n_peers; ++p)
            if (!a->peer_out[p] || !a->peer_flag[p]) return KVQ_ERR_NULL;
    }
    if (a->k_new || a->v_new) {                                // fused decode step (see the header)
        if (!a->k_new || !a->v_new) return KVQ_ERR_NULL;
        const int n_rep = a->nh / a->nh_kv;
        if (!L.use_mma || (L.qhv ? n_rep != L.qhv : n_rep != 1)) return KVQ_ERR_UNSUPPORTED;   // one CTA per kv head and segment
        if (!dev_state) {
            if (Rk < 1 || Rv < 1) return KVQ_ERR_TOKENS;       // the new token stays in the fp16 tails
            if ((a->k_quant != 0 && a->k_quant != a->k_group) || (a->v_quant != 0 && a->v_quant != a->v_group)) return KVQ_ERR_TOKENS;
            if (a->k_quant > a->Tkq || a->v_quant > a->Tvq) return KVQ_ERR_TOKENS;
            if (a->k_quant && (a->k_quant_slot < 0 || a->k_quant_slot + a->k_quant > a->kf_cap)) return KVQ_ERR_SHAPE;
            if (a->v_quant && (a->v_quant_slot < 0 || a->v_quant_slot + a->v_quant > a->vf_cap)) return KVQ_ERR_SHAPE;
        } else if (a->kf_cap % a->k_group != 0 || a->vf_cap % a->v_group != 0) {
            return KVQ_ERR_SHAPE;                              // a group must not wrap around its ring
        }
        auto bad = [](const void *p, int64_t s0, int64_t s1) { return reinterpret_cast<uintptr_t>(p) % 16 != 0 || s0 % 8 != 0 || s1 % 8 != 0; };
        if (bad(a->k_new, a->kn_sB, a->kn_sH) || bad(a->v_new, a->vn_sB, a->vn_sH)) return KVQ_ERR_ALIGN;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    float *parts = nullptr;
    unsigned int *counters = nullptr;
    if (L.partials > 0) {
        uint64_t cbytes = ((uint64_t)L.heads * 4 + 255) / 256 * 256;
        uint64_t need = cbytes + (uint64_t)L.partials * kPartStride * 4;
        if (!a->workspace || a->workspace_bytes < need) return KVQ_ERR_WORKSPACE;
        counters = static_cast<unsigned int *>(a->workspace);
        parts = reinterpret_cast<float *>(static_cast<char *>(a->workspace) + cbytes);
        // every kernel leaves the counters it used at zero; a workspace not yet vouched for is cleared here
        if (!(a->flags & KVQ_ATTN_WORKSPACE_READY)) {
            int rc = record_cuda_error(cudaMemsetAsync(counters, 0, (size_t)L.heads * 4, st));
            if (rc) return rc;
        }
    }
    if (L.qhv) return launch_decode_attn_gqa(*a, L.mplan, L.qhv, parts, counters, st);
    if (L.use_mma) return launch_decode_attn_mma(*a, L.mplan, parts, counters, st);
    decode_attn_kernel<<<(unsigned)L.ctas, kAttnThreads, 0, st>>>(*a, L.gplan.chunk, L.gplan.n_splits, parts, counters);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in the library image.  The symbol below is a host-side
// handle in host code, not a device address; its address on the current device is fetched once per
// device with cudaGetSymbolAddress and cached.
static __device__ __align__(256) unsigned char g_static_scratch[KVQ_STATIC_SCRATCH_BYTES];

namespace kvq {
constexpr int kMaxDevices = 64;
static void *g_static_scratch_ptr[kMaxDevices];
static int g_static_scratch_state[kMaxDevices];   // 0 = not looked up, 1 = ready

static int static_scratch_for_current_device(void **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= kMaxDevices) return KVQ_ERR_UNSUPPORTED;
    if (__atomic_load_n(&g_static_scratch_state[dev], __ATOMIC_ACQUIRE) != 1) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);    // device `dev` is current here
        if (e != cudaSuccess) return record_cuda_error(e);
        if (!p) return KVQ_ERR_CUDA;
        g_static_scratch_ptr[dev] = p;                     // same value from every thread: benign if raced
        __atomic_store_n(&g_static_scratch_state[dev], 1, __ATOMIC_RELEASE);
    }
    *out = g_static_scratch_ptr[dev];
    return KVQ_OK;
}
}  // namespace kvq

extern "C" int kvq_decode_attn_static(const kvq_attn_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->B > 0 && a->nh > 0 && a->T > 0 &&
        kvq_decode_attn_workspace_bytes(a->B, a->nh, a->T) > (uint64_t)KVQ_STATIC_SCRATCH_BYTES)
        return KVQ_ERR_STATIC_SCRATCH;
    void *scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != KVQ_OK) return rc;
    kvq_attn_args b = *a;
    b.workspace = scratch;
    b.workspace_bytes = KVQ_STATIC_SCRATCH_BYTES;
    b.flags &= ~KVQ_ATTN_WORKSPACE_READY;                     // the shared array is cleared on every call
    return kvq_decode_attn(&b, stream);                    // zeroes the counters it uses on `stream`
}
