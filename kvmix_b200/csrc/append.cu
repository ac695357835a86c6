// Ring-tail append: writes the new token's K and V rows (fp16) into the cache tails in one launch.
#include "common.cuh"

namespace kvq {

__global__ void __launch_bounds__(256) append_kv_kernel(kvq_append_args a) {
    const int per_row = a.D / 8;                               // 16-byte chunks per row
    const int64_t total = (int64_t)a.B * a.Hkv * per_row * 2;  // keys then values
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t half = total / 2;
    const bool is_v = i >= half;
    const int64_t j = is_v ? i - half : i;
    const int c = (int)(j % per_row);
    const int64_t bh = j / per_row;
    const int b = (int)(bh / a.Hkv), h = (int)(bh % a.Hkv);
    if (is_v) {
        const uint4 v = *(reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.v_new) + b * a.vn_sB + h * a.vn_sH) + c);
        *(reinterpret_cast<uint4 *>(static_cast<__half *>(a.vfull) + b * a.vf_sB + h * a.vf_sH + (int64_t)a.v_slot * a.vf_sT) + c) = v;
    } else {
        const uint4 v = *(reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.k_new) + b * a.kn_sB + h * a.kn_sH) + c);
        *(reinterpret_cast<uint4 *>(static_cast<__half *>(a.kfull) + b * a.kf_sB + h * a.kf_sH + (int64_t)a.k_slot * a.kf_sT) + c) = v;
    }
}

}  // namespace kvq

extern "C" int kvq_append_kv(const kvq_append_args *a, kvq_stream_t stream) {
    using namespace kvq;
    if (!a) return KVQ_ERR_NULL;
    if (a->B <= 0 || a->Hkv <= 0) return KVQ_OK;
    if (a->D <= 0 || a->D % 8 != 0) return KVQ_ERR_UNSUPPORTED;
    if (!a->k_new || !a->v_new || !a->kfull || !a->vfull) return KVQ_ERR_NULL;
    if (a->k_slot < 0 || a->v_slot < 0) return KVQ_ERR_SHAPE;
    auto bad = [](const void *p, int64_t s0, int64_t s1, int64_t s2) {
        return reinterpret_cast<uintptr_t>(p) % 16 != 0 || s0 % 8 != 0 || s1 % 8 != 0 || s2 % 8 != 0;
    };
    if (bad(a->k_new, a->kn_sB, a->kn_sH, 0) || bad(a->v_new, a->vn_sB, a->vn_sH, 0) ||
        bad(a->kfull, a->kf_sB, a->kf_sH, a->kf_sT) || bad(a->vfull, a->vf_sB, a->vf_sH, a->vf_sT))
        return KVQ_ERR_ALIGN;
    const int64_t total = (int64_t)a->B * a->Hkv * (a->D / 8) * 2;
    append_kv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
    return check_launch();
}


// ---------------------------------------------------------------------------------------------
// Bounded wait for the arrival counter of the head-sharded exchange (see kvq_peer_wait in the header).
namespace kvq {
__global__ void peer_wait_kernel(const uint32_t *counter, uint32_t expected, uint32_t max_polls, int32_t *status) {
    uint32_t seen = 0;
    for (uint32_t i = 0; i < max_polls; ++i) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
        if ((int32_t)(seen - expected) >= 0) return;
        __nanosleep(1000);
    }
    status[0] = 1;                                             // gave up: the host reads this after the step
    status[1] = (int32_t)seen;
}
// The same wait with the arrival target kept on the device: generation g of this counter (incremented here) waits for
// g * per_use arrivals, so the launch carries no per-step argument and replays from a CUDA graph.
__global__ void peer_wait_next_kernel(const uint32_t *counter, uint32_t per_use, uint32_t *generation, uint32_t max_polls,
                                      int32_t *status) {
    const uint32_t g = *generation + 1u;
    *generation = g;
    const uint32_t expected = g * per_use;
    uint32_t seen = 0;
    for (uint32_t i = 0; i < max_polls; ++i) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
        if ((int32_t)(seen - expected) >= 0) return;
        __nanosleep(1000);
    }
    status[0] = 1;
    status[1] = (int32_t)seen;
}
}  // namespace kvq

extern "C" int kvq_peer_wait_next(const uint32_t *counter, uint32_t per_use, uint32_t *generation, uint32_t max_polls,
                                  int32_t *status, kvq_stream_t stream) {
    using namespace kvq;
    if (!counter || !status || !generation) return KVQ_ERR_NULL;
    if (max_polls == 0 || per_use == 0) return KVQ_ERR_SHAPE;
    peer_wait_next_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(counter, per_use, generation, max_polls, status);
    return check_launch();
}

extern "C" int kvq_peer_wait(const uint32_t *counter, uint32_t expected, uint32_t max_polls, int32_t *status,
                             kvq_stream_t stream) {
    using namespace kvq;
    if (!counter || !status) return KVQ_ERR_NULL;
    if (max_polls == 0) return KVQ_ERR_SHAPE;
    peer_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(counter, expected, max_polls, status);
    return check_launch();
}
