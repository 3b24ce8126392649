"""Builds the reference's own CUDA extension for sm_100a into oracle/_ref/ (test infrastructure).

The two source files are compiled where they lie in the reference checkout
(csrc/attention_ext.cpp, csrc/flash_double_backward_v7.cu; the reference's setup.py:14-31 lists the
same two files and links cublas); nothing is copied into this repository, and oracle/_ref/ is
git-ignored.  The module is named `attention_cuda_ref` so that it can be loaded beside this
repository's `attention_cuda`.  Only tests and comparison scripts load it, as a checker.

    python oracle/build_ref.py [path-to-reference-checkout]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "attention_cuda_ref"


def built_path():
    p = os.path.join(OUT, NAME + ".so")
    return p if os.path.exists(p) else None


def build(reference_root="/root/reference", verbose=False):
    src = [os.path.join(reference_root, "csrc", f) for f in ("attention_ext.cpp", "flash_double_backward_v7.cu")]
    if not all(os.path.exists(s) for s in src):
        return None
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=src, build_directory=OUT, with_cuda=True, verbose=verbose,
         extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"],
         extra_ldflags=["-lcublas"], is_python_module=False)
    return built_path()


def load_module():
    """Imports the built module (None when it has not been built)."""
    p = built_path()
    if p is None:
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch symbols)
    spec = importlib.util.spec_from_file_location(NAME, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print(build(root, verbose=True))
