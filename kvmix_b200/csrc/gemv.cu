// Stand-alone dequantising mat-vec (M = 1) over the upstream cache layout, read in place.
//
//   out[n] = fp16( sum_k in[k] * (scale[k, n/G] * code[k, n] + zero[k, n/G]) ),  fp32 accumulation
//
// The zero term is hoisted: sum_k in[k]*zero[k,g] is accumulated once per packed word instead of
// once per field, and in[k]*scale[k,g] is formed once per word.  A CTA is WX word columns x KY
// k-lanes; lanes along the word axis read consecutive words (coalesced) for both uses of the
// routine: q.K^T (K = head_dim rows, thousands of word columns) and p.V (thousands of rows,
// head_dim/fpi word columns).
#include "common.cuh"

namespace kvq {

template <int BITS>
__global__ void __launch_bounds__(256) gemv_kernel(kvq_gemv_args a, int wx_log2, int nblk) {
    constexpr int FPI = fields_per_word(BITS);
    __shared__ float red[256];
    const int WX = 1 << wx_log2, KY = 256 >> wx_log2;
    const int wx = threadIdx.x & (WX - 1), ky = threadIdx.x >> wx_log2;
    const int64_t w = (int64_t)(blockIdx.x % nblk) * WX + wx;
    const int64_t s = blockIdx.x / nblk, b = s / a.nh, h = s % a.nh, hk = h / (a.nh / a.nh_kv);
    const int64_t n_pack = (a.n_groups * a.group) / FPI;
    const bool live = w < n_pack;
    const __half *in = static_cast<const __half *>(a.fA) + b * a.a_sB + h * a.a_sH;
    const int32_t *qb = a.qB + b * a.q_sB + hk * a.q_sH + w;
    const int64_t grp = (w * FPI) / a.group;
    const __half *sp = static_cast<const __half *>(a.scale) + b * a.s_sB + hk * a.s_sH + grp;
    const __half *zp = static_cast<const __half *>(a.zero) + b * a.s_sB + hk * a.s_sH + grp;

    float acc[FPI];
#pragma unroll
    for (int i = 0; i < FPI; ++i) acc[i] = 0.f;
    float zacc = 0.f;
    if (live) {
        for (int64_t k = ky; k < a.K; k += KY) {
            const uint32_t word = (uint32_t)__ldg(qb + k * a.q_sK);
            const float x = __half2float(__ldg(in + k));
            const float xs = x * __half2float(__ldg(sp + k * a.s_sK));
            zacc = fmaf(x, __half2float(__ldg(zp + k * a.s_sK)), zacc);
#pragma unroll
            for (int i = 0; i < FPI; ++i) acc[i] = fmaf(xs, (float)field<BITS>(word, i), acc[i]);
        }
    }
    __half *out = static_cast<__half *>(a.out) + b * a.o_sB + h * a.o_sH;
#pragma unroll 1
    for (int i = 0; i < FPI; ++i) {
        red[ky * WX + wx] = acc[i] + zacc;
        __syncthreads();
        if (ky == 0 && live) {
            float v = 0.f;
            for (int j = 0; j < KY; ++j) v += red[j * WX + wx];
            out[w * FPI + i] = __float2half_rn(v);
        }
        __syncthreads();
    }
}

}  // namespace kvq

extern "C" int kvq_gemv(const kvq_gemv_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->bits < 1 || a->bits > 4) return KVQ_ERR_BITS;
    if (a->nh_kv <= 0 || a->nh % a->nh_kv != 0) return KVQ_ERR_HEADS;
    if (a->bits == 3 && a->group != 11) return KVQ_ERR_GROUP3;
    const int fpi = fields_per_word(a->bits);
    if (a->group <= 0 || a->group % fpi != 0) return KVQ_ERR_GROUPWORD;
    if (a->B < 0 || a->K < 0 || a->n_groups < 0) return KVQ_ERR_SHAPE;
    const int64_t n_pack = (a->n_groups * a->group) / fpi;
    if (n_pack > a->n_words) return KVQ_ERR_SHAPE;
    if (a->B * a->nh == 0 || n_pack == 0) return KVQ_OK;
    if (!a->fA || !a->out) return KVQ_ERR_NULL;
    if (a->K > 0 && (!a->qB || !a->scale || !a->zero)) return KVQ_ERR_NULL;
    int wx_log2 = 5;
    while (wx_log2 > 2 && (1 << (wx_log2 - 1)) >= n_pack) --wx_log2;
    const int WX = 1 << wx_log2;
    const int64_t nblk = (n_pack + WX - 1) / WX;
    if (nblk * a->B * a->nh > 2147483647LL) return KVQ_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(nblk * a->B * a->nh));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (a->bits) {
        case 1: gemv_kernel<1><<<grid, 256, 0, st>>>(*a, wx_log2, (int)nblk); break;
        case 2: gemv_kernel<2><<<grid, 256, 0, st>>>(*a, wx_log2, (int)nblk); break;
        case 3: gemv_kernel<3><<<grid, 256, 0, st>>>(*a, wx_log2, (int)nblk); break;
        case 4: gemv_kernel<4><<<grid, 256, 0, st>>>(*a, wx_log2, (int)nblk); break;
    }
    return check_launch();
}
