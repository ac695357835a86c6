// Cache update fused into the attention kernels: what upstream does between projecting the new token and
// attending (models/modeling_llama_KVmix.py:111-167) -- append the token's K/V row to the fp16 tails and, when a
// group of the oldest tail tokens is due, quantize it behind the packed prefix -- done by the attention launch itself.
//
// The caller passes the cache state AFTER the update (T, Tkq, Tvq, ring starts) plus what is to be done:
//   k_new / v_new          the new token's rows; every reader of the tails takes token T-1 from here, and the CTA
//                          whose segment ends at T also stores them into the rings for the following steps;
//   k_quant / v_quant      0, or one group of tokens now lying at ring rows k_quant_slot.. / v_quant_slot.. that
//                          becomes packed tokens [Tkq - k_quant, Tkq) / [Tvq - v_quant, Tvq).  The CTA whose segment
//                          holds those positions quantizes them first; no other CTA reads them (the host only asks
//                          for this when one CTA per kv head and segment exists).
// Same arithmetic as the stand-alone quantizer (quant_core.cuh), so codes, scales and minima are bit-identical.
#pragma once
#include "quant_core.cuh"

namespace kvq {

// Keys: thread <-> channel; the group's tokens are rows of the fp16 ring (a group never wraps).
template <int KB>
__device__ __forceinline__ void fused_quant_k_group(const kvq_attn_args &a, int b, int hk, int tid) {
    constexpr int FPI = fields_per_word(KB);
    constexpr int QMAX = (1 << KB) - 1;
    const int G = a.k_quant;                                   // = k_group
    const __half *src = static_cast<const __half *>(a.kfull) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH +
                        (int64_t)a.k_quant_slot * a.kf_sT + tid;
    const int64_t st = a.kf_sT;
    float lo = __half2float(src[0]), hi = lo;
    for (int i = 1; i < G; ++i) {
        const float v = __half2float(src[i * st]);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    const float sc = (hi - lo) / (float)QMAX;
    const float rinv = __frcp_rn(sc);
    const int tok0 = a.Tkq - G;
    int32_t *pc = const_cast<int32_t *>(a.kcode) + (int64_t)b * a.kc_sB + (int64_t)hk * a.kc_sH + (int64_t)tid * a.kc_sD + tok0 / FPI;
    for (int w = 0; w < G / FPI; ++w) {
        const __half *pw = src + (int64_t)w * FPI * st;
        pc[w] = (int32_t)quant_word<KB>([&](int i) { return __half2float(pw[i * st]); }, lo, sc, rinv);
    }
    const int64_t zo = (int64_t)b * a.ks_sB + (int64_t)hk * a.ks_sH + (int64_t)tid * a.ks_sD + tok0 / G;
    static_cast<__half *>(const_cast<void *>(a.kscale))[zo] = __float2half_rn(stored_scale<QMAX>(hi - lo, sc, 0));
    static_cast<__half *>(const_cast<void *>(a.kmn))[zo] = __float2half_rn(lo);
}

// Values: thread <-> (token, channel group): v_group tokens x (128 / v_group) groups = 128 threads.
template <int VB>
__device__ __forceinline__ void fused_quant_v_group(const kvq_attn_args &a, int b, int hk, int tid) {
    constexpr int FPI = fields_per_word(VB);
    constexpr int QMAX = (1 << VB) - 1;
    const int G = a.v_group, ngv = kHeadDim / G;
    const int i = tid / ngv, jg = tid - i * ngv;               // token of the group, channel group
    const __half *src = static_cast<const __half *>(a.vfull) + (int64_t)b * a.vf_sB + (int64_t)hk * a.vf_sH +
                        (int64_t)(a.v_quant_slot + i) * a.vf_sT + jg * G;
    float lo = __half2float(src[0]), hi = lo;
    for (int c = 1; c < G; ++c) {
        const float v = __half2float(src[c]);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    const float sc = (hi - lo) / (float)QMAX;
    const float rinv = __frcp_rn(sc);
    const int t = a.Tvq - a.v_quant + i;
    int32_t *pc = const_cast<int32_t *>(a.vcode) + (int64_t)b * a.vc_sB + (int64_t)hk * a.vc_sH + (int64_t)t * a.vc_sT + jg * (G / FPI);
    for (int w = 0; w < G / FPI; ++w) {
        const __half *pw = src + w * FPI;
        pc[w] = (int32_t)quant_word<VB>([&](int e) { return __half2float(pw[e]); }, lo, sc, rinv);
    }
    const int64_t zo = (int64_t)b * a.vs_sB + (int64_t)hk * a.vs_sH + (int64_t)t * a.vs_sT + jg;
    static_cast<__half *>(const_cast<void *>(a.vscale))[zo] = __float2half_rn(stored_scale<QMAX>(hi - lo, sc, 0));
    static_cast<__half *>(const_cast<void *>(a.vmn))[zo] = __float2half_rn(lo);
}

// The update work of one segment [t0, t1) of kv head (b, hk), before its attention phases; every thread of the CTA
// calls it (it ends with a CTA barrier when it wrote packed data the CTA is about to read).
template <int KB, int VB>
__device__ __forceinline__ void fused_cache_update(const kvq_attn_args &a, int b, int hk, int t0, int t1, int tid) {
    if (!a.k_new) return;
    bool wrote = false;
    if (a.k_quant > 0 && t0 <= a.Tkq - a.k_quant && a.Tkq - a.k_quant < t1) {
        fused_quant_k_group<KB>(a, b, hk, tid);
        wrote = true;
    }
    if (a.v_quant > 0 && t0 <= a.Tvq - a.v_quant && a.Tvq - a.v_quant < t1) {
        if constexpr (VB != 3) fused_quant_v_group<VB>(a, b, hk, tid);
        wrote = true;
    }
    if (t1 == a.T && tid < 32) {                               // the rings receive the new token for the following steps
        const int c = tid & 15;
        if (tid < 16) {
            int slot = a.kf_start + (a.T - 1 - a.Tkq);
            if (slot >= a.kf_cap) slot -= a.kf_cap;
            const uint4 v = *(reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.k_new) + (int64_t)b * a.kn_sB + (int64_t)hk * a.kn_sH) + c);
            *(reinterpret_cast<uint4 *>(static_cast<__half *>(const_cast<void *>(a.kfull)) + (int64_t)b * a.kf_sB + (int64_t)hk * a.kf_sH + (int64_t)slot * a.kf_sT) + c) = v;
        } else {
            int slot = a.vf_start + (a.T - 1 - a.Tvq);
            if (slot >= a.vf_cap) slot -= a.vf_cap;
            const uint4 v = *(reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.v_new) + (int64_t)b * a.vn_sB + (int64_t)hk * a.vn_sH) + c);
            *(reinterpret_cast<uint4 *>(static_cast<__half *>(const_cast<void *>(a.vfull)) + (int64_t)b * a.vf_sB + (int64_t)hk * a.vf_sH + (int64_t)slot * a.vf_sT) + c) = v;
        }
    }
    if (wrote) {                                               // uniform over the CTA: the conditions depend on the segment only
        __threadfence_block();
        __syncthreads();
    }
}

// fp16 tail row of token t: the ring row, or -- for the step's own token while its update is fused -- the new row.
__device__ __forceinline__ const __half *k_tail_row(const kvq_attn_args &a, const __half *kf, int b, int hk, int t) {
    if (a.k_new && t == a.T - 1) return static_cast<const __half *>(a.k_new) + (int64_t)b * a.kn_sB + (int64_t)hk * a.kn_sH;
    int s = a.kf_start + (t - a.Tkq);
    if (s >= a.kf_cap) s -= a.kf_cap;
    return kf + (int64_t)s * a.kf_sT;
}
__device__ __forceinline__ const __half *v_tail_row(const kvq_attn_args &a, const __half *vf, int b, int hk, int t) {
    if (a.v_new && t == a.T - 1) return static_cast<const __half *>(a.v_new) + (int64_t)b * a.vn_sB + (int64_t)hk * a.vn_sH;
    int s = a.vf_start + (t - a.Tvq);
    if (s >= a.vf_cap) s -= a.vf_cap;
    return vf + (int64_t)s * a.vf_sT;
}

// Device-resident cache state (kvq_attn_args.state): five ints {T, Tkq, Tvq, kf_start, vf_start} describing the cache
// BEFORE this step, a completion counter at [5].  The kernel applies upstream's window policy itself -- keep
// `window` tokens in fp16, or int(ratio * current_fp16_len) (models/modeling_llama_KVmix.py:118-126) -- to derive
// what this step does, and the last CTA to have read the state writes the state after the step back, so the launch arguments
// of a decode loop never change and a whole step can be replayed from a CUDA graph.  At most one group per step
// becomes due in steady state; the host does not switch to this mode before that (upstream's ratio policy shrinks a
// prompt's tail over several steps).
__device__ __forceinline__ int tokens_due(const kvq_attn_args &a, int cur, int group, double ratio) {
    const int keep = a.window >= 0 ? a.window : (int)(ratio * (double)cur);
    if (cur > keep && keep >= 0) {
        const int n = ((cur - keep) / group) * group;
        return n > group ? group : n;
    }
    return 0;
}

__device__ __forceinline__ void dev_state_step(const kvq_attn_args &a, kvq_attn_args &b) {
    // One thread reads the state and counts the CTA in; the others take it from shared memory.  The state may be
    // overwritten once every CTA of the grid has read it: the count is raised only after the reading thread holds the
    // values (the branch on all five loaded values keeps it behind the loads), and the CTA that completes the count -- the last
    // one to START, so nothing is left on the tail of the kernel -- publishes the state after the step (below).
    __shared__ int s_state[5];
    int *st = a.state;
    bool publish = false;
    if (threadIdx.x == 0) {
        const int v0 = st[0], v1 = st[1], v2 = st[2], v3 = st[3], v4 = st[4];
        s_state[0] = v0; s_state[1] = v1; s_state[2] = v2; s_state[3] = v3; s_state[4] = v4;
        if ((v0 | v1 | v2 | v3 | v4) >= 0) publish = atomicAdd(reinterpret_cast<unsigned int *>(st + 5), 1u) == gridDim.x - 1;
    }
    __syncthreads();
    const int T0 = s_state[0], Tkq0 = s_state[1], Tvq0 = s_state[2], ks0 = s_state[3], vs0 = s_state[4];
    const int nk = tokens_due(a, T0 - Tkq0 + 1, a.k_group, a.k_ratio);
    const int nv = tokens_due(a, T0 - Tvq0 + 1, a.v_group, a.v_ratio);
    b.T = T0 + 1;
    b.Tkq = Tkq0 + nk;
    b.Tvq = Tvq0 + nv;
    b.kf_start = ks0 + nk >= a.kf_cap ? ks0 + nk - a.kf_cap : ks0 + nk;
    b.vf_start = vs0 + nv >= a.vf_cap ? vs0 + nv - a.vf_cap : vs0 + nv;
    b.k_quant = nk;
    b.v_quant = nv;
    b.k_quant_slot = ks0;
    b.v_quant_slot = vs0;
    if (publish) {
        st[0] = b.T; st[1] = b.Tkq; st[2] = b.Tvq; st[3] = b.kf_start; st[4] = b.vf_start;
        st[5] = 0;
    }
}

// Head-sharded exchange: the rows `vals[i]` (this thread's channel `tid` of `n_heads` consecutive query heads starting
// at local head h0 of sequence b) go to every rank's gather buffer, then every rank's arrival counter is raised by
// n_heads.  Every thread of the CTA calls it (CTA barrier inside).  Plain peer stores and one system-scope
// fence + atomic per rank: no multicast, nothing waits here.
template <int N>
__device__ __forceinline__ void peer_publish(const kvq_attn_args &a, int b, int h0, int n_heads, const __half (&vals)[N], int tid) {
    if (a.n_peers <= 0) return;
    for (int p = 0; p < a.n_peers; ++p) {
        __half *dst = static_cast<__half *>(a.peer_out[p]) + (int64_t)b * a.peer_sB + (int64_t)(a.peer_head0 + h0) * a.peer_sH + tid;
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (i < n_heads) dst[(int64_t)i * a.peer_sH] = vals[i];
    }
    __syncthreads();                                           // every thread's stores are issued ...
    if (tid < a.n_peers) {
        __threadfence_system();                                // ... and ordered before the arrival count, system-wide
        atomicAdd_system(a.peer_flag[tid], (unsigned)n_heads);
    }
}

}  // namespace kvq
