"""In-tree build of the sm_100a extension (``himuon_b200/csrc`` -> ``csrc/build/himuon_b200_C.so``).

nvcc cross-compiles for ``sm_100a`` without a GPU; the resulting shared object is loaded
directly by :mod:`himuon_b200._ext` so no JIT step runs on the training machine.
"""

from __future__ import annotations

import os

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
BUILD_DIR = os.path.join(CSRC, "build")
EXT_NAME = "himuon_b200_C"

CUDA_SOURCES = [
    "gemm_sm100.cu",
    "gemm2_sm100.cu",
    "optim_kernels.cu",
    "model_kernels.cu",
    "attention_sm100.cu",
    "attention_kv64_sm100.cu", "attention_bwd_sm100.cu",
    "ns5_sm100.cu",
    "comm_kernels.cu",
    "soap_kernels.cu",
    "rmsnorm_bwd_noalloc.cu",
]
CPP_SOURCES = ["bindings.cpp", "symm.cpp", "vmm.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--use_fast_math",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def sources() -> list[str]:
    out = []
    for name in CUDA_SOURCES + CPP_SOURCES:
        path = os.path.join(CSRC, name)
        if os.path.exists(path):
            out.append(path)
    return out


def so_path() -> str:
    return os.path.join(BUILD_DIR, EXT_NAME + ".so")


def build(verbose: bool = False):
    """Compile every source for sm_100a and return the loaded extension module."""
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    return cpp_extension.load(
        name=EXT_NAME,
        sources=sources(),
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=["-lcudart"],
        build_directory=BUILD_DIR,
        with_cuda=True,
        verbose=verbose,
    )


if __name__ == "__main__":
    build(verbose=True)
    print("built", so_path())
