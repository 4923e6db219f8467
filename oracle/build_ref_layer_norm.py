"""Builds the reference's own LayerNorm extension for sm_100 into oracle/_ref/ (test and benchmark infrastructure).

The reference ships one native component on this path: protenix/model/layer_norm/kernel/{layer_norm_cuda.cpp,
layer_norm_cuda_kernel.cu} (pybind11 + ATen, built by protenix/model/layer_norm/torch_ext_compile.py:21-97 with
torch.utils.cpp_extension.load).  This recipe compiles those two files WHERE THEY LIE in the reference tree, with the
reference's own flags and the sm_100 target it adds when nvcc knows it (torch_ext_compile.py:51-64), and leaves
fast_layer_norm_cuda_v2.so under oracle/_ref/ (git-ignored; it travels to the GPU box with the built library).
Nothing is copied into this repository.  The product never loads it: bench.py --micro times it beside
px_layer_norm_fwd when the file is present.

    python oracle/build_ref_layer_norm.py [/path/to/reference]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "fast_layer_norm_cuda_v2"


def build(ref_root: str = "/root/reference") -> str:
    from torch.utils.cpp_extension import load

    kdir = os.path.join(ref_root, "protenix", "model", "layer_norm", "kernel")
    srcs = [os.path.join(kdir, "layer_norm_cuda.cpp"), os.path.join(kdir, "layer_norm_cuda_kernel.cu")]
    if not all(os.path.exists(s) for s in srcs):
        raise FileNotFoundError(f"reference LayerNorm sources not found under {kdir}")
    os.makedirs(OUT, exist_ok=True)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    flags = ["-O3", "-DVERSION_GE_1_1", "-DVERSION_GE_1_3", "-DVERSION_GE_1_5"]
    load(name=NAME, sources=srcs, extra_include_paths=[kdir], build_directory=OUT, extra_cflags=flags,
         extra_cuda_cflags=flags + ["--use_fast_math", "-std=c++17", "-maxrregcount=32", "-U__CUDA_NO_HALF_OPERATORS__",
                                    "-U__CUDA_NO_HALF_CONVERSIONS__", "--expt-relaxed-constexpr",
                                    "--expt-extended-lambda", "-gencode", "arch=compute_100,code=sm_100"],
         is_python_module=False, verbose=False)
    return os.path.join(OUT, NAME + ".so")


def load_if_built():
    """The built extension as a Python module, or None when oracle/_ref does not hold it."""
    path = os.path.join(OUT, NAME + ".so")
    if not os.path.exists(path):
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
