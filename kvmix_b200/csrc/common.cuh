// Shared device/host helpers for the kvmix_b200 kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvmix_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "kvmix_b200 kernels are written for sm_100a only"
#endif

namespace kvq {

constexpr int kHeadDim = 128;

__host__ __device__ constexpr int fields_per_word(int bits) { return bits == 3 ? 11 : 32 / bits; }

// Field i of a packed word.  3-bit words hold ten 3-bit fields and a 2-bit field at bit 30.
template <int BITS>
__device__ __forceinline__ uint32_t field(uint32_t w, int i) {
    if constexpr (BITS == 3) {
        return i < 10 ? ((w >> (3 * i)) & 7u) : (w >> 30);
    } else {
        return (w >> (BITS * i)) & ((1u << BITS) - 1u);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Records the text of the last failing CUDA call for kvq_last_cuda_error().
// Additive attention mask value for (sequence b, query head h, key position t); the caller checked a.mask != NULL.
__device__ __forceinline__ float attn_mask_at(const kvq_attn_args &a, int b, int h, int t) {
    const int64_t off = (int64_t)b * a.mask_sB + (int64_t)h * a.mask_sH + t;
    return a.mask_is_f32 ? __ldg(static_cast<const float *>(a.mask) + off)
                         : __half2float(__ldg(static_cast<const __half *>(a.mask) + off));
}
// upstream clamps masked weights from below at torch.finfo(float32).min (models/modeling_llama_KVmix.py:192)
constexpr float kMaskFloor = -3.4028234663852886e38f;

int record_cuda_error(cudaError_t e);
inline int check_launch() { return record_cuda_error(cudaGetLastError()); }

}  // namespace kvq
