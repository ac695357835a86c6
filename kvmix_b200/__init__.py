"""kvmix_b200: the KV-cache hot path of KVmix (group quantizer + fused dequant decode attention)
as hand-written sm_100a CUDA behind a C ABI (include/kvmix_b200.h), with the upstream ``KVmix``
extension-module functions as the Python surface.  Importing the package does not need a GPU;
calling an operator needs the built library and CUDA tensors -- there is no CPU fallback.
"""
from .ops import (decode_attention, features_per_int, process_key_quantization_cuda,  # noqa: F401
                  process_value_quantization_cuda, quantize_into, quantize_pack_last_dim_cuda, quantized_gemm)
from .cache import (CapturedDecodeStep, KVmixLayerCache, KVmixPast, attention_step, kv_bytes_per_head,  # noqa: F401
                    split_point)

__all__ = ["quantize_pack_last_dim_cuda", "quantized_gemm", "process_key_quantization_cuda",
           "process_value_quantization_cuda", "decode_attention", "quantize_into", "KVmixLayerCache", "CapturedDecodeStep",
           "attention_step", "KVmixPast", "kv_bytes_per_head", "split_point", "features_per_int"]
