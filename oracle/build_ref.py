"""Compiles the reference's own top-p CUDA kernel (csrc/src/sampling.cu + csrc/include/sampling.cuh
of tsinghua-ideal/Twilight) for sm_100a, from the sources where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY: the resulting extension is the GPU-side checker for the top-p pruner.
Nothing is copied from the reference; its three FlashInfer helper headers come from the
flashinfer package installed in this image.  The reference's own build path
(flashinfer.jit.load_cuda_ops of flashinfer 0.2.0) does not exist in the installed flashinfer,
so torch.utils.cpp_extension is used with the same sources and include directories.

    python oracle/build_ref.py [/path/to/Twilight]
"""
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "twilight_ref_sampling"


def build(ref_root: str = "/root/reference", verbose: bool = False):
    ref = Path(ref_root)
    src = ref / "csrc" / "src" / "sampling.cu"
    if not src.exists():
        return None
    import flashinfer
    import torch.utils.cpp_extension as ext
    inc = Path(flashinfer.__file__).parent / "data" / "include"
    OUT.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    ext.load(name=NAME, sources=[str(src)],
             extra_include_paths=[str(ref / "csrc" / "include"), str(ref / "csrc" / "src"), str(inc)],
             # FLASHINFER_ENABLE_BF16 is the reference's own switch for the bf16 branch of its fp16 entry
             # point (csrc/src/pytorch_extension_utils.h:23-57)
             extra_cflags=["-DFLASHINFER_ENABLE_BF16"],
             extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo",
                                "-DFLASHINFER_ENABLE_BF16",
                                # torch's default -D__CUDA_NO_HALF_*: the FlashInfer headers need them off
                                "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                                "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
                                "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT162_OPERATORS__"],
             build_directory=str(OUT), is_python_module=False, verbose=verbose)
    return OUT / f"{NAME}.so"


def load():
    """Imports the prebuilt extension (oracle/_ref/twilight_ref_sampling.so); None if absent."""
    so = OUT / f"{NAME}.so"
    if not so.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", verbose=True))
