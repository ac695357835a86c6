"""Test infrastructure: compile the upstream KVmix CUDA extension, unmodified, for sm_100a.

The upstream extension (quant_cuda/csrc/{pybind.cpp,quantization_cuda.cu,
dequantization_gemv_cuda.cu}, built upstream by quant_cuda/setup.py:32-47) is compiled
from the sources where they lie in the mounted reference tree; nothing is copied.  Two
variants are produced, both only into ``oracle/_ref/``:

* ``KVmix_ref_fast``  -- upstream's own nvcc flags (``-O3 --use_fast_math``,
  quant_cuda/setup.py:15-29): the kernel a user of upstream would run.
* ``KVmix_ref_ieee``  -- same sources without ``--use_fast_math``: IEEE division and
  rounding, which is what the CPU restatement in this folder states bit-exactly.

The modules have no CPU path, so they can only be *executed* on a machine with a GPU; there
they are used by ``tests/golden/make_golden.py`` and ``tests/golden/make_attn_golden.py`` to pin the CPU
restatement and by ``bench.py``'s ``upstream_gpu`` leg (through ``oracle/upstream_torch.py``) as the clearly
labelled "kernel to beat on the same GPU".  Nothing in the product imports them.

Usage:  python oracle/build_ref.py --ref /path/to/upstream/tree [--variant fast|ieee|both]
        (or the tree's path in the environment variable KVMIX_REFERENCE)
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

COMMON_NVCC = [
    "-O3", "-std=c++17", "-DENABLE_BF16",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
]


def _includes():
    import torch.utils.cpp_extension as ce
    inc = ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    return [f"-I{p}" for p in inc]


def _run(cmd):
    print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build(ref, variant):
    import torch
    import torch.utils.cpp_extension as ce
    name = f"KVmix_ref_{variant}"
    src = os.path.join(ref, "quant_cuda", "csrc")
    work = os.path.join(OUT, f"obj_{variant}")
    os.makedirs(work, exist_ok=True)
    defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc_flags = COMMON_NVCC + (["--use_fast_math"] if variant == "fast" else [])
    inc = _includes() + [f"-I{src}"]
    jobs = []
    for f in ("quantization_cuda.cu", "dequantization_gemv_cuda.cu"):
        obj = os.path.join(work, f.replace(".cu", ".o"))
        jobs.append((obj, ["nvcc", "-c", os.path.join(src, f), "-o", obj] + nvcc_flags + defs + inc))
    obj = os.path.join(work, "pybind.o")
    jobs.append((obj, ["g++", "-c", os.path.join(src, "pybind.cpp"), "-o", obj, "-O3", "-std=c++17",
                       "-fPIC", "-DENABLE_BF16"] + defs + inc))
    with ThreadPoolExecutor(max_workers=3) as ex:
        list(ex.map(lambda j: _run(j[1]), jobs))
    so = os.path.join(OUT, name + sysconfig.get_config_var("EXT_SUFFIX"))
    libs = [f"-L{p}" for p in ce.library_paths("cuda")]
    _run(["g++", "-shared", "-o", so] + [j[0] for j in jobs] + libs +
         ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"])
    print("built", so)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("KVMIX_REFERENCE"),
                    help="root of the upstream KVmix tree (default: $KVMIX_REFERENCE)")
    ap.add_argument("--variant", default="both", choices=["fast", "ieee", "both"])
    a = ap.parse_args()
    if not a.ref:
        ap.error("give the upstream tree with --ref or KVMIX_REFERENCE")
    if not os.path.isdir(os.path.join(a.ref, "quant_cuda", "csrc")):
        print("reference tree not present; nothing to build")
        return 0
    os.makedirs(OUT, exist_ok=True)
    for v in (["fast", "ieee"] if a.variant == "both" else [a.variant]):
        build(a.ref, v)
    return 0


if __name__ == "__main__":
    sys.exit(main())
