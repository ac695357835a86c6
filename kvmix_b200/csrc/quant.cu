// Group quantizer: fp16/fp32 -> b-bit codes packed in int32 words + per-group scale and min.
//
// Arithmetic (must be bit-identical to upstream quant_cuda/csrc/quantization_cuda.cu:553-596 with
// IEEE division; this file is compiled without fast-math):
//   mn, mx   fp32 min / max of the group
//   scale32  (mx - mn) / (2^b - 1)
//   code     clamp(roundf((x - mn) / scale32), 0, 2^b - 1), roundf = half away from zero;
//            3-bit: the 11th element of each group clamps to 3; 0/0 (constant group) -> 0
//   stored scale = scale32 narrowed to the input dtype, stored mn = mn
//
// Three kernels, one result:
//   quant_contig_kernel   groups run along the contiguous axis (values: [.., T, D], groups over D;
//                         or keys already transposed to [.., D, T]).  A thread owns one or two output
//                         words; the threads of a group combine min/max with shuffles.
//   quant_strided_kernel  groups run along a strided axis while the *other* axis is contiguous
//                         (keys left as [.., T, D], groups over T).  A thread owns two adjacent
//                         channels, keeps a whole group in registers (all loads in flight at
//                         once), and the CTA transposes words through shared memory so global
//                         writes are contiguous runs per channel.
//   quant_generic_kernel  any strides / any group-to-word relation; one thread per word.
#include "quant_core.cuh"

namespace kvq {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

struct QuantDims {
    int64_t B, H, A, S;
    int64_t x_sB, x_sH, x_sA, x_sS;
    int64_t c_sB, c_sH, c_sA;
    int64_t z_sB, z_sH, z_sA;
    int group;
    int by_div;   // stored scale: 1 = (mx-mn)/qmax, 0 = (mx-mn) * fl32(1/qmax)
};

// ---------------------------------------------------------------------------------------------
// Contiguous groups.  A thread owns WPT consecutive words (E * WPT elements, 32 where the shapes allow: 64 bytes
// of loads in flight per thread, and the per-thread index arithmetic, division and shuffles spread over enough
// elements); tpg = group / (E * WPT) threads share a group.
template <int BITS, typename T, int WPT>
__global__ void __launch_bounds__(256) quant_contig_kernel(const T *__restrict__ x, int32_t *__restrict__ code,
                                                           T *__restrict__ scale, T *__restrict__ mn, QuantDims d,
                                                           int tpg, bool vec_ok, bool linear) {
    constexpr int E = fields_per_word(BITS);
    constexpr int EW = E * WPT;
    // blockIdx.y = (b, h); inside a (b, h) slab units of WPT words are numbered linearly (32-bit index arithmetic)
    const int units_per_row = (int)(d.S / EW);
    const int total = (int)d.A * units_per_row;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = idx < total;
    if (!active) idx = total - 1;  // keep the lane alive for the shuffles
    const int b = blockIdx.y / (int)d.H, h = blockIdx.y % (int)d.H;
    int a, u;
    if (linear) { a = 0; u = idx; }                      // rows of the slab are back to back in x, code and scale
    else { a = idx / units_per_row; u = idx - a * units_per_row; }
    const T *px = x + b * d.x_sB + h * d.x_sH + a * d.x_sA + (int64_t)u * EW;

    float v[EW];
    float lo, hi;
    bool have_range = false;
    if constexpr (sizeof(T) == 2 && (EW % 8 == 0)) {
        if (vec_ok) {
            // min / max in fp16x2 on the raw loads (exact: the data are fp16; NaN operands are skipped as by fminf):
            // one instruction per two elements instead of one per element
            __half2 lo2, hi2;
#pragma unroll
            for (int j = 0; j < EW / 8; ++j) {
                uint4 q = __ldg(reinterpret_cast<const uint4 *>(px) + j);
                const __half2 *hp = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (j == 0 && k == 0) { lo2 = hp[0]; hi2 = hp[0]; }
                    else { lo2 = __hmin2(lo2, hp[k]); hi2 = __hmax2(hi2, hp[k]); }
                    float2 f = __half22float2(hp[k]);
                    v[j * 8 + 2 * k] = f.x;
                    v[j * 8 + 2 * k + 1] = f.y;
                }
            }
            lo = fminf(__low2float(lo2), __high2float(lo2));
            hi = fmaxf(__low2float(hi2), __high2float(hi2));
            have_range = true;
        } else {
#pragma unroll
            for (int i = 0; i < EW; ++i) v[i] = to_f32<T>(px[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < EW; ++i) v[i] = to_f32<T>(px[i]);
    }
    if (!have_range) {
        lo = v[0];
        hi = v[0];
#pragma unroll
        for (int i = 1; i < EW; ++i) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    }
    for (int o = 1; o < tpg; o <<= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    constexpr int QMAX = (1 << BITS) - 1;
    const float sc = (hi - lo) / (float)QMAX;
    const float rinv = __frcp_rn(sc);                          // correctly rounded 1 / sc
    uint32_t word[WPT];
#pragma unroll
    for (int k = 0; k < WPT; ++k) word[k] = quant_word<BITS>([&](int i) { return v[k * E + i]; }, lo, sc, rinv);
    if (active) {
        int32_t *pc = code + b * d.c_sB + h * d.c_sH + a * d.c_sA + u * WPT;
#pragma unroll
        for (int k = 0; k < WPT; ++k) pc[k] = (int32_t)word[k];
        if ((u & (tpg - 1)) == 0) {                           // tpg is a power of two
            const int64_t zo = b * d.z_sB + h * d.z_sH + a * d.z_sA + (u >> (__ffs(tpg) - 1));
            scale[zo] = from_f32<T>(stored_scale<QMAX>(hi - lo, sc, d.by_div));
            mn[zo] = from_f32<T>(lo);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Strided groups over s, contiguous channel axis a (x_sA == 1), fp16, A % 128 == 0.
// CTA: 256 threads = 64 channel pairs x 4 group slots; covers 128 channels x GPC groups.
template <int BITS, int G>
struct StridedCfg {
    static constexpr int FPI = fields_per_word(BITS);
    static constexpr int WPG = G / FPI;                       // words per group (1 for 3-bit)
    static constexpr int GPC = (G == 11) ? 24 : (256 / G < 4 ? 4 : 256 / G);  // groups per CTA
    static constexpr int WPC = GPC * WPG;                     // words per channel per CTA
    static constexpr int WPAD = WPC + 1;
};

// Rotary embedding applied while loading (prefill of keys straight from the k_proj output): element (b, s, c) of the
// cos / sin tables at b * r_sB + s * r_sS + c, fp16.  HF's rotate_half form (the one upstream's model files import):
// out[c] = k[c] * cos[c] + rot[c] * sin[c] with rot = (-k[c + 64], k[c - 64]) for c < 64 / c >= 64, every product and
// the sum rounded to fp16 as the framework's fp16 tensor arithmetic rounds them.
struct RopeTables {
    const __half *cos, *sin;
    int64_t r_sB, r_sS;
};

template <int BITS, int G, bool ROPE>
__global__ void __launch_bounds__(256, 3) quant_strided_kernel(const __half *__restrict__ x, int32_t *__restrict__ code,
                                                            __half *__restrict__ scale, __half *__restrict__ mn,
                                                            QuantDims d, RopeTables rope) {
    using C = StridedCfg<BITS, G>;
    __shared__ int32_t s_code[128 * C::WPAD];
    __shared__ __half s_scale[128 * (C::GPC + 2)];
    __shared__ __half s_mn[128 * (C::GPC + 2)];

    const int pair = threadIdx.x & 63, slot = threadIdx.x >> 6;
    const int64_t bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
    const int64_t a0 = (int64_t)blockIdx.y * 128;
    const int64_t g0 = (int64_t)blockIdx.x * C::GPC;          // first group of this CTA
    const int64_t n_groups = d.S / G;
    const int groups_here = (int)min((int64_t)C::GPC, n_groups - g0);
    const __half *px = x + b * d.x_sB + h * d.x_sH + (a0 + 2 * pair);
    constexpr int QMAX = (1 << BITS) - 1;
    // element pair (2 pair, 2 pair + 1) of token s of this (b, h) slab, rotated on the way in when ROPE
    const int partner = (2 * pair < 64) ? 64 : -64;
    const __half *pcos = ROPE ? rope.cos + b * rope.r_sB + 2 * pair : nullptr;
    const __half *psin = ROPE ? rope.sin + b * rope.r_sB + 2 * pair : nullptr;
    auto load = [&](int64_t s) -> __half2 {
        const __half2 k = __ldg(reinterpret_cast<const __half2 *>(px + s * d.x_sS));
        if constexpr (ROPE) {
            __half2 r = __ldg(reinterpret_cast<const __half2 *>(px + s * d.x_sS + partner));
            if (partner > 0) r = __hneg2(r);
            const __half2 cs = __ldg(reinterpret_cast<const __half2 *>(pcos + s * rope.r_sS));
            const __half2 sn = __ldg(reinterpret_cast<const __half2 *>(psin + s * rope.r_sS));
            return __hadd2_rn(__hmul2_rn(k, cs), __hmul2_rn(r, sn));
        } else {
            return k;
        }
    };

    // tokens held in registers at a time: a whole group up to 32 tokens; longer groups are walked twice anyway (min/max,
    // then codes from L1/L2), and for them 16 at a time measured 5-10 % faster for 2- and 4-bit codes (fewer live
    // registers under the 80-register cap); a 1-bit word needs 32 tokens
    constexpr int CH = G > 32 ? (BITS == 1 ? 32 : 16) : G;
    constexpr int NCH = G / CH;
    constexpr int WPCH = CH / C::FPI;                         // words per chunk (1 for the 11-token group)
    for (int g = slot; g < groups_here; g += 4) {
        const int64_t s0 = (g0 + g) * G;                      // first token of the group
        __half2 raw[CH];
        // min / max of the two channels in fp16x2 (exact: the data are fp16; NaN operands are skipped as by fminf)
        __half2 lo2 = __floats2half2_rn(65504.f, 65504.f), hi2 = __floats2half2_rn(-65504.f, -65504.f);
        bool first = true;
#pragma unroll 1
        for (int c = 0; c < NCH; ++c) {
#pragma unroll
            for (int i = 0; i < CH; ++i) raw[i] = load(s0 + c * CH + i);
            if (first) { lo2 = raw[0]; hi2 = raw[0]; first = false; }
#pragma unroll
            for (int i = 0; i < CH; ++i) { lo2 = __hmin2(lo2, raw[i]); hi2 = __hmax2(hi2, raw[i]); }
        }
        const float lo0 = __low2float(lo2), lo1 = __high2float(lo2), hi0 = __low2float(hi2), hi1 = __high2float(hi2);
        const float sc0 = (hi0 - lo0) / (float)QMAX, sc1 = (hi1 - lo1) / (float)QMAX;
        const float ri0 = __frcp_rn(sc0), ri1 = __frcp_rn(sc1);     // correctly rounded reciprocals
#pragma unroll 1
        for (int c = 0; c < NCH; ++c) {
            if (NCH > 1) {                                    // long groups: second pass over the chunk (cache hit)
#pragma unroll
                for (int i = 0; i < CH; ++i) raw[i] = load(s0 + c * CH + i);
            }
#pragma unroll
            for (int w = 0; w < WPCH; ++w) {
                const uint32_t w0 = quant_word<BITS>([&](int i) { return __low2float(raw[w * C::FPI + i]); }, lo0, sc0, ri0);
                const uint32_t w1 = quant_word<BITS>([&](int i) { return __high2float(raw[w * C::FPI + i]); }, lo1, sc1, ri1);
                s_code[(2 * pair) * C::WPAD + g * C::WPG + c * WPCH + w] = (int32_t)w0;
                s_code[(2 * pair + 1) * C::WPAD + g * C::WPG + c * WPCH + w] = (int32_t)w1;
            }
        }
        s_scale[(2 * pair) * (C::GPC + 2) + g] = __float2half_rn(stored_scale<QMAX>(hi0 - lo0, sc0, d.by_div));
        s_scale[(2 * pair + 1) * (C::GPC + 2) + g] = __float2half_rn(stored_scale<QMAX>(hi1 - lo1, sc1, d.by_div));
        s_mn[(2 * pair) * (C::GPC + 2) + g] = __float2half_rn(lo0);
        s_mn[(2 * pair + 1) * (C::GPC + 2) + g] = __float2half_rn(lo1);
    }
    __syncthreads();
    const int words_here = groups_here * C::WPG;
    int32_t *pc = code + b * d.c_sB + h * d.c_sH + a0 * d.c_sA + g0 * C::WPG;
    const int64_t zo = b * d.z_sB + h * d.z_sH + a0 * d.z_sA + g0;
    if (groups_here == C::GPC) {                              // full CTA: row lengths are compile-time constants
        for (int i = threadIdx.x; i < 128 * C::WPC; i += 256) {
            const int ch = i / C::WPC, w = i % C::WPC;
            pc[ch * d.c_sA + w] = s_code[ch * C::WPAD + w];
        }
        for (int i = threadIdx.x; i < 128 * C::GPC; i += 256) {
            const int ch = i / C::GPC, g = i % C::GPC;
            scale[zo + ch * d.z_sA + g] = s_scale[ch * (C::GPC + 2) + g];
            mn[zo + ch * d.z_sA + g] = s_mn[ch * (C::GPC + 2) + g];
        }
    } else {
        for (int i = threadIdx.x; i < 128 * words_here; i += 256) {
            const int ch = i / words_here, w = i % words_here;
            pc[ch * d.c_sA + w] = s_code[ch * C::WPAD + w];
        }
        for (int i = threadIdx.x; i < 128 * groups_here; i += 256) {
            const int ch = i / groups_here, g = i % groups_here;
            scale[zo + ch * d.z_sA + g] = s_scale[ch * (C::GPC + 2) + g];
            mn[zo + ch * d.z_sA + g] = s_mn[ch * (C::GPC + 2) + g];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Any layout: one thread per output word, group statistics recomputed as needed.
template <int BITS, typename T>
__global__ void __launch_bounds__(128) quant_generic_kernel(const T *__restrict__ x, int32_t *__restrict__ code,
                                                            T *__restrict__ scale, T *__restrict__ mn, QuantDims d) {
    constexpr int E = fields_per_word(BITS);
    constexpr int QMAX = (1 << BITS) - 1;
    const int64_t words_per_row = d.S / E;
    const int64_t total = d.B * d.H * d.A * words_per_row;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t row = idx / words_per_row, w = idx % words_per_row;
    const int64_t a = row % d.A, h = (row / d.A) % d.H, b = row / (d.A * d.H);
    const T *px = x + b * d.x_sB + h * d.x_sH + a * d.x_sA;
    const int64_t zo = b * d.z_sB + h * d.z_sH + a * d.z_sA;
    const int G = d.group;
    int64_t cur = -1;
    float lo = 0.f, sc = 0.f, range = 0.f;
    uint32_t word = 0;
    for (int i = 0; i < E; ++i) {
        const int64_t s = w * E + i, g = s / G;
        if (g != cur) {
            cur = g;
            float hi = -3.402823466e+38f;
            lo = 3.402823466e+38f;
            for (int j = 0; j < G; ++j) {
                const float f = to_f32<T>(px[(g * G + j) * d.x_sS]);
                lo = fminf(lo, f); hi = fmaxf(hi, f);
            }
            range = hi - lo;
            sc = range / (float)QMAX;
        }
        if (s % G == 0) {
            scale[zo + g] = from_f32<T>(stored_scale<QMAX>(range, sc, d.by_div));
            mn[zo + g] = from_f32<T>(lo);
        }
        const float n = (to_f32<T>(px[s * d.x_sS]) - lo) / sc;
        if constexpr (BITS == 3) {
            const int pos = (int)(s % G);   // position inside the 11-group (G == 11 enforced by the host)
            word |= (uint32_t)round_code(n, pos < 10 ? 7 : 3) << (i < 10 ? 3 * i : 30);
        } else {
            word |= (uint32_t)round_code(n, QMAX) << (BITS * i);
        }
    }
    code[b * d.c_sB + h * d.c_sH + a * d.c_sA + w] = (int32_t)word;
}

// ---------------------------------------------------------------------------------------------
// Extension without an upstream counterpart: 3-bit groups of 11 along an axis whose length is not a multiple of 11
// (3-bit values at head_dim 128).  Every group is one word; the last group holds S % 11 elements, its unused fields
// stay 0.  Upstream's 3-bit group rule otherwise (quantization_cuda.cu:553-596, :612-626).  One thread per word.
template <typename T>
__global__ void __launch_bounds__(128) quant_ragged3_kernel(const T *__restrict__ x, int32_t *__restrict__ code,
                                                            T *__restrict__ scale, T *__restrict__ mn, QuantDims d) {
    const int64_t words_per_row = (d.S + 10) / 11;
    const int64_t total = d.B * d.H * d.A * words_per_row;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t row = idx / words_per_row, w = idx % words_per_row;
    const int64_t a = row % d.A, h = (row / d.A) % d.H, b = row / (d.A * d.H);
    const T *px = x + b * d.x_sB + h * d.x_sH + a * d.x_sA + w * 11 * d.x_sS;
    const int n = (int)min((int64_t)11, d.S - w * 11);
    float v[11], lo = 3.402823466e+38f, hi = -3.402823466e+38f;
#pragma unroll
    for (int i = 0; i < 11; ++i) {
        v[i] = i < n ? to_f32<T>(px[i * d.x_sS]) : 0.f;
        if (i < n) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    }
    const float range = hi - lo, sc = range / 7.0f;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 11; ++i)
        if (i < n) word |= (uint32_t)round_code((v[i] - lo) / sc, i < 10 ? 7 : 3) << (i < 10 ? 3 * i : 30);
    code[b * d.c_sB + h * d.c_sH + a * d.c_sA + w] = (int32_t)word;
    const int64_t zo = b * d.z_sB + h * d.z_sH + a * d.z_sA + w;
    scale[zo] = from_f32<T>(stored_scale<7>(range, sc, d.by_div));
    mn[zo] = from_f32<T>(lo);
}

template <typename T>
static int launch_ragged3(const kvq_quant_args *a, const QuantDims &d, cudaStream_t st) {
    const int64_t total = d.B * d.H * d.A * ((d.S + 10) / 11);
    quant_ragged3_kernel<T><<<(unsigned)((total + 127) / 128), 128, 0, st>>>(
        static_cast<const T *>(a->x), a->code, static_cast<T *>(a->scale), static_cast<T *>(a->mn), d);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------
template <int BITS, typename T>
static int launch_bits(const kvq_quant_args *a, const QuantDims &d, cudaStream_t st, const RopeTables *rope = nullptr) {
    constexpr int E = fields_per_word(BITS);
    const T *x = static_cast<const T *>(a->x);
    T *sc = static_cast<T *>(a->scale), *mn = static_cast<T *>(a->mn);
    const int G = a->group;
    const int64_t total_words = d.B * d.H * d.A * (d.S / E);
    if (total_words == 0) return KVQ_OK;

    // groups along the contiguous axis
    if (!rope && a->x_sS == 1 && G % E == 0) {
        bool vec_ok = sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && d.x_sB % 8 == 0 &&
                      d.x_sH % 8 == 0 && d.x_sA % 8 == 0;
        // 32 elements (64 B of fp16 in flight) per thread where the group and the row allow it: 4 / 2 words for 4 / 2 bits
        constexpr int WMAX = (sizeof(T) == 2 && E < 32 && 32 % E == 0) ? 32 / E : 1;
        const bool wide = WMAX > 1 && vec_ok && G % (WMAX * E) == 0 && (d.S / E) % WMAX == 0;
        const int wpt = wide ? WMAX : 1;
        const int tpg = G / (E * wpt);
        const int64_t per_slab = d.A * (d.S / (E * wpt));
        if (tpg <= 32 && (tpg & (tpg - 1)) == 0 && per_slab < (1LL << 31) && d.B * d.H <= 65535) {
            const int64_t wpr = d.S / E;
            const bool linear = d.x_sA == d.S && d.c_sA == wpr && d.z_sA == d.S / G;
            dim3 grid((unsigned)((per_slab + 255) / 256), (unsigned)(d.B * d.H));
            if (wide) quant_contig_kernel<BITS, T, WMAX><<<grid, 256, 0, st>>>(x, a->code, sc, mn, d, tpg, vec_ok, linear);
            else quant_contig_kernel<BITS, T, 1><<<grid, 256, 0, st>>>(x, a->code, sc, mn, d, tpg, vec_ok, linear);
            return check_launch();
        }
    }
    // groups along a strided axis, channels contiguous (keys in [T, D] order)
    if constexpr (sizeof(T) == 2) {
        const bool ok = a->x_sA == 1 && d.A % 128 == 0 && (reinterpret_cast<uintptr_t>(x) % 4 == 0) &&
                        d.x_sB % 2 == 0 && d.x_sH % 2 == 0 && d.x_sS % 2 == 0 && d.B * d.H <= 65535 &&
                        d.A / 128 <= 65535;
        if (ok) {
            const __half *xh = reinterpret_cast<const __half *>(x);
            __half *sh = reinterpret_cast<__half *>(sc), *mh = reinterpret_cast<__half *>(mn);
            const int64_t ng = d.S / G;
#define KVQ_LAUNCH_STRIDED(GG)                                                                     \
    {                                                                                              \
        using C = StridedCfg<BITS, GG>;                                                            \
        dim3 grid((unsigned)((ng + C::GPC - 1) / C::GPC), (unsigned)(d.A / 128), (unsigned)(d.B * d.H)); \
        if (rope) quant_strided_kernel<BITS, GG, true><<<grid, 256, 0, st>>>(xh, a->code, sh, mh, d, *rope);      \
        else quant_strided_kernel<BITS, GG, false><<<grid, 256, 0, st>>>(xh, a->code, sh, mh, d, RopeTables{});   \
        return check_launch();                                                                     \
    }
            if constexpr (BITS == 3) {
                if (G == 11) KVQ_LAUNCH_STRIDED(11)
            } else {
                if (G == 32) KVQ_LAUNCH_STRIDED(32)
                if (G == 64) KVQ_LAUNCH_STRIDED(64)
                if (G == 128) KVQ_LAUNCH_STRIDED(128)
            }
#undef KVQ_LAUNCH_STRIDED
        }
    }
    if (rope) return KVQ_ERR_UNSUPPORTED;                      // rotation on the way in needs the strided-key layout
    const int64_t blocks = (total_words + 127) / 128;
    quant_generic_kernel<BITS, T><<<(unsigned)blocks, 128, 0, st>>>(x, a->code, sc, mn, d);
    return check_launch();
}

static int quant_lastdim_impl(const kvq_quant_args *a, kvq_stream_t stream, const RopeTables *rope);

}  // namespace kvq

extern "C" int kvq_quant_lastdim(const kvq_quant_args *a, kvq_stream_t stream) {
    return kvq::quant_lastdim_impl(a, stream, nullptr);
}

static int kvq::quant_lastdim_impl(const kvq_quant_args *a, kvq_stream_t stream, const RopeTables *rope) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->bits < 1 || a->bits > 4) return KVQ_ERR_BITS;
    if (a->B < 0 || a->H < 0 || a->A < 0 || a->S < 0) return KVQ_ERR_SHAPE;
    if (a->bits == 3) {
        if (a->group != 11) return KVQ_ERR_GROUP3;
        if (a->S % 11 != 0 && !a->ragged_tail) return KVQ_ERR_DIV11;
    } else {
        if (a->group <= 0 || a->S % a->group != 0) return KVQ_ERR_DIVGROUP;
        if (a->S % (32 / a->bits) != 0) return KVQ_ERR_DIVWORD;
    }
    if (a->B * a->H * a->A * a->S == 0) return KVQ_OK;
    if (!a->x || !a->code || !a->scale || !a->mn) return KVQ_ERR_NULL;
    if (a->bits == 3 && a->S % 11 != 0) {                      // the short-last-group extension
        if (rope) return KVQ_ERR_UNSUPPORTED;
        QuantDims r{a->B, a->H, a->A, a->S, a->x_sB, a->x_sH, a->x_sA, a->x_sS, a->c_sB, a->c_sH, a->c_sA,
                    a->z_sB, a->z_sH, a->z_sA, 11, a->scale_by_division ? 1 : 0};
        cudaStream_t rs = reinterpret_cast<cudaStream_t>(stream);
        return a->x_is_f32 ? launch_ragged3<float>(a, r, rs) : launch_ragged3<__half>(a, r, rs);
    }
    QuantDims d{a->B, a->H, a->A, a->S, a->x_sB, a->x_sH, a->x_sA, a->x_sS, a->c_sB, a->c_sH, a->c_sA,
                a->z_sB, a->z_sH, a->z_sA, a->group, a->scale_by_division ? 1 : 0};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define KVQ_DISPATCH(BITS)                                                             \
    case BITS:                                                                         \
        return a->x_is_f32 ? launch_bits<BITS, float>(a, d, st, rope) : launch_bits<BITS, __half>(a, d, st, rope);
    switch (a->bits) {
        KVQ_DISPATCH(1)
        KVQ_DISPATCH(2)
        KVQ_DISPATCH(3)
        KVQ_DISPATCH(4)
    }
#undef KVQ_DISPATCH
    return KVQ_ERR_BITS;
}

// ---------------------------------------------------------------------------------------------
// Functional append forms: copy the previous tensors into the front of the outputs (strided device-to-device
// copies on the same stream), then quantize the new tokens in place behind them.
namespace kvq {
static int copy_rows(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width, size_t rows,
                     cudaStream_t st) {
    if (width == 0 || rows == 0) return KVQ_OK;
    if (!src || !dst) return KVQ_ERR_NULL;
    return record_cuda_error(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, rows, cudaMemcpyDeviceToDevice, st));
}
}  // namespace kvq

extern "C" int kvq_append_k(const kvq_append_form_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->bits < 1 || a->bits > 4) return KVQ_ERR_BITS;
    if (a->B < 0 || a->H < 0 || a->A < 0 || a->S < 0 || a->old_words < 0 || a->old_groups < 0) return KVQ_ERR_SHAPE;
    if (a->bits == 3 && a->group != 11) return KVQ_ERR_GROUP3;
    if (a->group <= 0) return KVQ_ERR_DIVGROUP;
    if (a->bits == 3) {
        if (a->S % 11 != 0) return KVQ_ERR_DIV11;
    } else {
        if (a->S % a->group != 0) return KVQ_ERR_DIVGROUP;
        if (a->S % (32 / a->bits) != 0) return KVQ_ERR_DIVWORD;
    }
    const int fpi = fields_per_word(a->bits);
    const int64_t new_words = a->S / fpi, new_groups = a->S / a->group;
    const int64_t rows = a->B * a->H * a->A, W = a->old_words + new_words, Gn = a->old_groups + new_groups;
    const size_t es = a->x_is_f32 ? 4 : 2;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int rc = copy_rows(a->code, (size_t)W * 4, a->prev_code, (size_t)a->old_words * 4, (size_t)a->old_words * 4, (size_t)rows, st);
    if (rc) return rc;
    rc = copy_rows(a->scale, (size_t)Gn * es, a->prev_scale, (size_t)a->old_groups * es, (size_t)a->old_groups * es, (size_t)rows, st);
    if (rc) return rc;
    rc = copy_rows(a->mn, (size_t)Gn * es, a->prev_mn, (size_t)a->old_groups * es, (size_t)a->old_groups * es, (size_t)rows, st);
    if (rc) return rc;
    kvq_quant_args q{a->x, a->x_is_f32, a->B, a->H, a->A, a->S, a->x_sB, a->x_sH, a->x_sA, a->x_sS, a->group, a->bits, 1,
                     a->code ? a->code + a->old_words : nullptr, a->H * a->A * W, a->A * W, W,
                     a->scale ? static_cast<char *>(a->scale) + (size_t)a->old_groups * es : nullptr,
                     a->mn ? static_cast<char *>(a->mn) + (size_t)a->old_groups * es : nullptr,
                     a->H * a->A * Gn, a->A * Gn, Gn};
    return kvq_quant_lastdim(&q, stream);
}

extern "C" int kvq_append_v(const kvq_append_form_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->bits < 1 || a->bits > 4) return KVQ_ERR_BITS;
    if (a->B < 0 || a->H < 0 || a->A < 0 || a->S < 0 || a->old_tokens < 0) return KVQ_ERR_SHAPE;
    if (a->bits == 3 && a->group != 11) return KVQ_ERR_GROUP3;
    if (a->group <= 0) return KVQ_ERR_DIVGROUP;
    if (a->bits == 3) {
        if (a->S % 11 != 0) return KVQ_ERR_DIV11;
    } else {
        if (a->S % a->group != 0) return KVQ_ERR_DIVGROUP;
        if (a->S % (32 / a->bits) != 0) return KVQ_ERR_DIVWORD;
    }
    const int fpi = fields_per_word(a->bits);
    const int64_t wpt = a->S / fpi, gpt = a->S / a->group;           // words / groups per token row
    const int64_t rows = a->B * a->H, Tt = a->old_tokens + a->A;
    const size_t es = a->x_is_f32 ? 4 : 2;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int rc = copy_rows(a->code, (size_t)(Tt * wpt) * 4, a->prev_code, (size_t)(a->old_tokens * wpt) * 4,
                       (size_t)(a->old_tokens * wpt) * 4, (size_t)rows, st);
    if (rc) return rc;
    rc = copy_rows(a->scale, (size_t)(Tt * gpt) * es, a->prev_scale, (size_t)(a->old_tokens * gpt) * es,
                   (size_t)(a->old_tokens * gpt) * es, (size_t)rows, st);
    if (rc) return rc;
    rc = copy_rows(a->mn, (size_t)(Tt * gpt) * es, a->prev_mn, (size_t)(a->old_tokens * gpt) * es,
                   (size_t)(a->old_tokens * gpt) * es, (size_t)rows, st);
    if (rc) return rc;
    kvq_quant_args q{a->x, a->x_is_f32, a->B, a->H, a->A, a->S, a->x_sB, a->x_sH, a->x_sA, a->x_sS, a->group, a->bits, 1,
                     a->code ? a->code + a->old_tokens * wpt : nullptr, a->H * Tt * wpt, Tt * wpt, wpt,
                     a->scale ? static_cast<char *>(a->scale) + (size_t)(a->old_tokens * gpt) * es : nullptr,
                     a->mn ? static_cast<char *>(a->mn) + (size_t)(a->old_tokens * gpt) * es : nullptr,
                     a->H * Tt * gpt, Tt * gpt, gpt};
    return kvq_quant_lastdim(&q, stream);
}


// ---------------------------------------------------------------------------------------------
// Prompt tails: tokens [nk, L) of the keys (rotated on the way when tables are given) and [nv, L) of the values go to
// rows 0.. of the fp16 rings.  One thread per (b, h, token, 8-channel chunk j < 8) handles chunk j and chunk j + 8,
// the rotation partners.
namespace kvq {
__global__ void __launch_bounds__(256) prefill_tails_kernel(kvq_prefill_args a) {
    const int D = a.D, nkt = a.L - a.nk, nvt = a.L - a.nv;
    const int64_t per_k = (int64_t)a.B * a.Hkv * nkt * 8, per_v = (int64_t)a.B * a.Hkv * nvt * 8;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_k + per_v) return;
    const bool is_v = i >= per_k;
    if (is_v) i -= per_k;
    const int j = (int)(i & 7);
    const int n = is_v ? nvt : nkt;
    const int64_t r = (i >> 3) % n, bh = (i >> 3) / n;
    const int b = (int)(bh / a.Hkv), h = (int)(bh % a.Hkv);
    if (is_v) {
        const __half *src = static_cast<const __half *>(a.v) + b * a.v_sB + (a.nv + r) * a.v_sT + h * a.v_sH;
        __half *dst = static_cast<__half *>(a.vfull) + b * a.vf_sB + h * a.vf_sH + r * a.vf_sT;
        reinterpret_cast<uint4 *>(dst)[j] = __ldg(reinterpret_cast<const uint4 *>(src) + j);
        reinterpret_cast<uint4 *>(dst)[j + 8] = __ldg(reinterpret_cast<const uint4 *>(src) + j + 8);
        return;
    }
    const int64_t t = a.nk + r;
    const __half *src = static_cast<const __half *>(a.k) + b * a.k_sB + t * a.k_sT + h * a.k_sH;
    __half *dst = static_cast<__half *>(a.kfull) + b * a.kf_sB + h * a.kf_sH + r * a.kf_sT;
    uint4 lo = __ldg(reinterpret_cast<const uint4 *>(src) + j), hi = __ldg(reinterpret_cast<const uint4 *>(src) + j + 8);
    if (a.cos) {
        const __half *pc = static_cast<const __half *>(a.cos) + b * a.r_sB + t * a.r_sT;
        const __half *ps = static_cast<const __half *>(a.sin) + b * a.r_sB + t * a.r_sT;
        const uint4 cl = __ldg(reinterpret_cast<const uint4 *>(pc) + j), ch = __ldg(reinterpret_cast<const uint4 *>(pc) + j + 8);
        const uint4 sl = __ldg(reinterpret_cast<const uint4 *>(ps) + j), sh = __ldg(reinterpret_cast<const uint4 *>(ps) + j + 8);
        uint4 ol, oh;
        const __half2 *kl = reinterpret_cast<const __half2 *>(&lo), *kh = reinterpret_cast<const __half2 *>(&hi);
        const __half2 *c0 = reinterpret_cast<const __half2 *>(&cl), *c1 = reinterpret_cast<const __half2 *>(&ch);
        const __half2 *s0 = reinterpret_cast<const __half2 *>(&sl), *s1 = reinterpret_cast<const __half2 *>(&sh);
        __half2 *pl = reinterpret_cast<__half2 *>(&ol), *ph = reinterpret_cast<__half2 *>(&oh);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            pl[q] = __hadd2_rn(__hmul2_rn(kl[q], c0[q]), __hmul2_rn(__hneg2(kh[q]), s0[q]));
            ph[q] = __hadd2_rn(__hmul2_rn(kh[q], c1[q]), __hmul2_rn(kl[q], s1[q]));
        }
        lo = ol;
        hi = oh;
    }
    reinterpret_cast<uint4 *>(dst)[j] = lo;
    reinterpret_cast<uint4 *>(dst)[j + 8] = hi;
    (void)D;
}
}  // namespace kvq

extern "C" int kvq_prefill(const kvq_prefill_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->D != kHeadDim) return KVQ_ERR_UNSUPPORTED;
    if (a->B <= 0 || a->Hkv <= 0 || a->L <= 0) return KVQ_OK;
    if (a->nk < 0 || a->nv < 0 || a->nk > a->L || a->nv > a->L) return KVQ_ERR_TOKENS;
    if (!a->k || !a->v) return KVQ_ERR_NULL;
    if ((a->cos == nullptr) != (a->sin == nullptr)) return KVQ_ERR_NULL;
    if (a->k_bits < 1 || a->k_bits > 4 || a->v_bits < 1 || a->v_bits > 4) return KVQ_ERR_BITS;
    auto al16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (!al16(a->k) || !al16(a->v) || a->k_sB % 8 || a->k_sT % 8 || a->k_sH % 8 || a->v_sB % 8 || a->v_sT % 8 || a->v_sH % 8)
        return KVQ_ERR_ALIGN;
    if (a->cos && (!al16(a->cos) || !al16(a->sin) || a->r_sB % 8 || a->r_sT % 8)) return KVQ_ERR_ALIGN;
    if (a->nk < a->L && (!a->kfull || !al16(a->kfull) || a->kf_sB % 8 || a->kf_sH % 8 || a->kf_sT % 8)) return KVQ_ERR_ALIGN;
    if (a->nv < a->L && (!a->vfull || !al16(a->vfull) || a->vf_sB % 8 || a->vf_sH % 8 || a->vf_sT % 8)) return KVQ_ERR_ALIGN;
    if (a->nk > 0) {                                           // keys: groups over tokens, channels contiguous, read in place
        kvq_quant_args q{a->k, 0, a->B, a->Hkv, a->D, a->nk, a->k_sB, a->k_sH, 1, a->k_sT, a->k_group, a->k_bits, 0,
                         a->kcode, a->kc_sB, a->kc_sH, a->kc_sD, a->kscale, a->kmn, a->ks_sB, a->ks_sH, a->ks_sD};
        RopeTables rope{static_cast<const __half *>(a->cos), static_cast<const __half *>(a->sin), a->r_sB, a->r_sT};
        const int rc = quant_lastdim_impl(&q, stream, a->cos ? &rope : nullptr);
        if (rc) return rc;
    }
    if (a->nv > 0) {                                           // values: groups over channels
        kvq_quant_args q{a->v, 0, a->B, a->Hkv, a->nv, a->D, a->v_sB, a->v_sH, a->v_sT, 1, a->v_group, a->v_bits, 0,
                         a->vcode, a->vc_sB, a->vc_sH, a->vc_sT, a->vscale, a->vmn, a->vs_sB, a->vs_sH, a->vs_sT,
                         a->v_bits == 3 ? 1 : 0};               // 3-bit values: the short-last-group extension
        const int rc = kvq_quant_lastdim(&q, stream);
        if (rc) return rc;
    }
    const int64_t n = (int64_t)a->B * a->Hkv * ((int64_t)(a->L - a->nk) + (a->L - a->nv)) * 8;
    if (n > 0) {
        prefill_tails_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
        return check_launch();
    }
    return KVQ_OK;
}
