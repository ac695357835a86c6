// Library-level entry points: version, error texts, last CUDA error.
#include <string.h>

#include "common.cuh"

namespace kvq {
static thread_local char g_cuda_error[256] = "";

int record_cuda_error(cudaError_t e) {
    if (e == cudaSuccess) return KVQ_OK;
    strncpy(g_cuda_error, cudaGetErrorString(e), sizeof(g_cuda_error) - 1);
    g_cuda_error[sizeof(g_cuda_error) - 1] = 0;
    return KVQ_ERR_CUDA;
}
}  // namespace kvq

extern "C" int kvq_version(void) { return 106; }   // 105: fused decode step, device-resident state, head-sharded exchange, kvq_prefill, kvq_attn_plan; 106: 3-bit values (ragged_tail)

extern "C" int kvq_features_per_int(int bits) { return (bits >= 1 && bits <= 4) ? kvq::fields_per_word(bits) : 0; }

extern "C" const char *kvq_last_cuda_error(void) { return kvq::g_cuda_error; }

extern "C" const char *kvq_error_string(int code) {
    switch (code) {
        case KVQ_OK: return "ok";
        case KVQ_ERR_BITS: return "Supported quantization bits: 1, 2, 3, 4";
        case KVQ_ERR_GROUP3: return "For 3-bit quantization, group_length must be 11";
        case KVQ_ERR_DIV11: return "For 3-bit quantization, steps must be divisible by 11";
        case KVQ_ERR_DIVGROUP: return "steps must be divisible by group_length";
        case KVQ_ERR_DIVWORD: return "steps must be divisible by (32 / quant_bits)";
        case KVQ_ERR_HEADS: return "Total heads must be divisible by KV heads";
        case KVQ_ERR_SHAPE: return "inconsistent tensor sizes";
        case KVQ_ERR_GROUPWORD: return "group size must be a multiple of the fields per packed word";
        case KVQ_ERR_TOKENS: return "inconsistent token counts";
        case KVQ_ERR_NULL: return "null pointer";
        case KVQ_ERR_UNSUPPORTED: return "configuration not supported by the sm_100a kernels";
        case KVQ_ERR_WORKSPACE: return "workspace missing or too small";
        case KVQ_ERR_ALIGN: return "pointer or stride alignment";
        case KVQ_ERR_STATIC_SCRATCH:
            return "problem too large for the built-in scratch (kvq_decode_attn_workspace_bytes exceeds KVQ_STATIC_SCRATCH_BYTES = 8 MiB): "
                   "use kvq_decode_attn with a caller-provided workspace";
        case KVQ_ERR_CUDA: return "CUDA error";
        default: return "unknown error";
    }
}
