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

namespace kvq {

constexpr int kAttnThreads = 256;
constexpr int kMaxChunk = 4224;  // tokens per split held in shared memory (multiple of 128 and of 352)
constexpr int kPartStride = kHeadDim + 2;

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

// Tensor-core kernel: a CTA step is 4 warps x one 256-token key tile (88 tokens for 3-bit keys), so chunks are
// multiples of 1024 (352) tokens, at most 8192 (8096) scores are held, and the last split runs to T, absorbing a
// remainder of up to a quarter step.  The chunk is the candidate with the best estimated throughput under a
// model fitted to measurements on B200 (2-bit keys and values, 256..8192 CTAs of 1024..8192 tokens):
//   rate ~ q / ceil(q) * chunk / (chunk + 670),  q = CTAs / (148 SMs * 3 resident CTAs),
// i.e. whole waves of CTAs and a fitted per-CTA term worth 670 tokens (it absorbs launch ramp, tail and co-residency
// effects: an undisturbed CTA shows no such fixed cost on the phase clock); chunks
// under 4096 tokens measured a further ~10 % below that and more than one split pays for the counter reset and the
// merge.  Ties go to fewer splits.
constexpr int kMmaSlots = 148 * 3;
constexpr double kMmaCtaCost = 670.0;

struct PlanMemo {
    int T, kb;
    int64_t heads;
    SplitPlan plan;
};

static SplitPlan plan_splits_mma(int T, int k_bits, int64_t heads) {
    const int unit = (k_bits == 3) ? 352 : 1024;
    const int max_chunk = (k_bits == 3) ? 8096 : 8192;
    static thread_local PlanMemo memo[4] = {};
    static thread_local int next = 0;
    for (const PlanMemo &m : memo)
        if (m.T == T && m.kb == k_bits && m.heads == heads) return m.plan;

    // no finer than ~16 CTAs per slot in total: bounds the search and the workspace
    const int64_t n_cap = (16 * kMmaSlots + heads - 1) / heads;
    SplitPlan best = {0, 0};
    double best_rate = 0.0;
    for (int chunk = (max_chunk / unit) * unit; chunk >= unit; chunk -= unit) {
        int n = (T + chunk - 1) / chunk;
        int last = T - (n - 1) * chunk;
        if (n > 1 && last <= unit / 4) {
            --n;
            last += chunk;
        }
        if (n > n_cap && best.n_splits > 0) break;
        const double q = (double)(heads * n) / kMmaSlots;
        const double waves = (double)((heads * n + kMmaSlots - 1) / kMmaSlots);
        const double longest = chunk > last ? chunk : last;
        double rate = q / waves * ((double)T / n) / (longest + kMmaCtaCost);
        if (longest < 4096) rate *= 0.9;
        if (n > 1) rate *= 0.92;
        if (rate > best_rate * 1.0001) {
            best = {chunk, n};
            best_rate = rate;
        }
    }
    memo[next] = {T, k_bits, heads, best};
    next = (next + 1) & 3;
    return best;
}

// Upper bound of plan_splits_mma's split count for every T' <= T (the workspace is sized once for a cache).
static int64_t max_splits_mma(int T, int k_bits, int64_t heads) {
    const int unit = (k_bits == 3) ? 352 : 1024;
    const int max_chunk = (k_bits == 3) ? 8096 : 8192;
    const int64_t n_cap = (16 * kMmaSlots + heads - 1) / heads;
    const int64_t by_unit = (T + unit - 1) / unit, by_max = (T + (max_chunk / unit) * unit - 1) / ((max_chunk / unit) * unit);
    const int64_t n = by_unit < n_cap ? by_unit : n_cap;
    return n > by_max ? n : by_max;
}

static SplitPlan plan_splits(int T, int k_bits, int64_t heads, bool mma_path = false) {
    return mma_path ? plan_splits_mma(T, k_bits, heads) : plan_splits_generic(T, k_bits, heads);
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
}

// tensor-core path (decode_attn_mma.cu)
bool mma_path_eligible(const kvq_attn_args &a);
int launch_decode_attn_mma(const kvq_attn_args &a, int chunk, int n_splits, float *parts, unsigned int *counters,
                           cudaStream_t st);

}  // namespace kvq

extern "C" uint64_t kvq_decode_attn_workspace_bytes(int32_t B, int32_t nh, int32_t T) {
    using namespace kvq;
    if (B <= 0 || nh <= 0 || T <= 0) return 256;
    const int64_t heads = (int64_t)B * nh;
    int64_t ns = 1;
    for (int kb = 3; kb <= 4; ++kb) {
        const int64_t g = plan_splits_generic(T, kb, heads).n_splits, m = max_splits_mma(T, kb, heads);
        ns = g > ns ? g : ns;
        ns = m > ns ? m : ns;
    }
    uint64_t bytes = (uint64_t)heads * 4;
    bytes = (bytes + 255) / 256 * 256;
    bytes += (uint64_t)heads * ns * kPartStride * 4;
    return (bytes + 255) / 256 * 256;
}

extern "C" int kvq_decode_attn_plan(int32_t B, int32_t nh, int32_t T, int32_t k_bits, int32_t tensor_core,
                                    int32_t *chunk, int32_t *n_splits) {
    using namespace kvq;
    if (!chunk || !n_splits) return KVQ_ERR_NULL;
    if (k_bits < 1 || k_bits > 4) return KVQ_ERR_BITS;
    if (B <= 0 || nh <= 0 || T <= 0) return KVQ_ERR_SHAPE;
    const SplitPlan p = plan_splits(T, k_bits, (int64_t)B * nh, tensor_core != 0);
    *chunk = p.chunk;
    *n_splits = p.n_splits;
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
    if (a->v_bits == 3) return KVQ_ERR_UNSUPPORTED;  // upstream cannot hold 3-bit values for D = 128 either
    if (a->k_group <= 0 || a->k_group % fk != 0 || a->v_group <= 0 || a->v_group % fv != 0) return KVQ_ERR_GROUPWORD;
    if (a->Tkq % a->k_group != 0) return KVQ_ERR_DIVGROUP;
    if (kHeadDim % a->v_group != 0) return KVQ_ERR_DIVGROUP;
    if (!a->q || !a->out) return KVQ_ERR_NULL;
    if (a->Tkq > 0 && (!a->kcode || !a->kscale || !a->kmn)) return KVQ_ERR_NULL;
    if (a->Tvq > 0 && (!a->vcode || !a->vscale || !a->vmn)) return KVQ_ERR_NULL;
    const int Rk = a->T - a->Tkq, Rv = a->T - a->Tvq;
    if (Rk > 0 && (!a->kfull || a->kf_cap < Rk || a->kf_start < 0 || a->kf_start >= a->kf_cap)) return KVQ_ERR_SHAPE;
    if (Rv > 0 && (!a->vfull || a->vf_cap < Rv || a->vf_start < 0 || a->vf_start >= a->vf_cap)) return KVQ_ERR_SHAPE;
    if (Rk > 0 && (reinterpret_cast<uintptr_t>(a->kfull) % 8 || a->kf_sB % 4 || a->kf_sH % 4 || a->kf_sT % 4))
        return KVQ_ERR_ALIGN;
    if (Rv > 0 && (reinterpret_cast<uintptr_t>(a->vfull) % 4 || a->vf_sB % 2 || a->vf_sH % 2 || a->vf_sT % 2))
        return KVQ_ERR_ALIGN;

    const int64_t heads = (int64_t)a->B * a->nh;
    const bool use_mma = mma_path_eligible(*a);
    const SplitPlan plan = plan_splits(a->T, a->k_bits, heads, use_mma);
    if (heads * plan.n_splits > 2147483647LL) return KVQ_ERR_UNSUPPORTED;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    float *parts = nullptr;
    unsigned int *counters = nullptr;
    if (plan.n_splits > 1) {
        uint64_t cbytes = ((uint64_t)heads * 4 + 255) / 256 * 256;
        uint64_t need = cbytes + (uint64_t)heads * plan.n_splits * kPartStride * 4;
        if (!a->workspace || a->workspace_bytes < need) return KVQ_ERR_WORKSPACE;
        counters = static_cast<unsigned int *>(a->workspace);
        parts = reinterpret_cast<float *>(static_cast<char *>(a->workspace) + cbytes);
        int rc = record_cuda_error(cudaMemsetAsync(counters, 0, (size_t)heads * 4, st));
        if (rc) return rc;
    }
    if (use_mma) return launch_decode_attn_mma(*a, plan.chunk, plan.n_splits, parts, counters, st);
    decode_attn_kernel<<<(unsigned)(heads * plan.n_splits), kAttnThreads, 0, st>>>(*a, plan.chunk, plan.n_splits,
                                                                                   parts, counters);
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
    return kvq_decode_attn(&b, stream);                    // zeroes the counters it uses on `stream`
}
