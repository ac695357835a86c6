"""Drop-in for the upstream ``KVmix`` extension module (quant_cuda/csrc/pybind.cpp:6-15).

``import KVmix`` in models/modeling_llama_KVmix.py:9 and models/modeling_mistral_KVmix.py:37
resolves to this module when the repository root is on sys.path; the four exported names keep
upstream's positional signatures and are served by the sm_100a library in kvmix_b200.
"""
from kvmix_b200.ops import (process_key_quantization_cuda, process_value_quantization_cuda,  # noqa: F401
                            quantize_pack_last_dim_cuda, quantized_gemm)
