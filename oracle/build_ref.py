"""Builds the reference's own CUDA extension for sm_100a into oracle/_ref/ (test infrastructure).

The two source files are compiled where they lie in the reference checkout
(csrc/attention_ext.cpp, csrc/flash_double_backward_v7.cu; the reference's setup.py:14-31 lists the
same two files and links cublas); nothing is copied into this repository, and oracle/_ref/ is
git-ignored.  The module is named `attention_cuda_ref` so that it can be loaded beside this
repository's `attention_cuda`.  Only tests and comparison scripts load it, as a checker.

    python oracle/build_ref.py <path-to-reference-checkout>

`compile_python_reference()` byte-compiles the reference's TTT model file
(e2e/ttt_pytorch/model.py: its `make_sw_causal_mask`, `reference_attention`,
`v7_kernel_attention`, `CausalLM` and `meta_step`) where it lies into
oracle/_ref/ref_ttt_model.bin, so that the drop-in tests and the CPU arm of the bench can run the
reference's own Python code on a machine that has no checkout.  `load_python_reference()` imports it.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "attention_cuda_ref"


def built_path():
    p = os.path.join(OUT, NAME + ".so")
    return p if os.path.exists(p) else None


PY_NAME = "ref_ttt_model"


def python_reference_path():
    p = os.path.join(OUT, PY_NAME + ".bin")
    return p if os.path.exists(p) else None


def compile_python_reference(reference_root):
    """Byte-compiles e2e/ttt_pytorch/model.py of the checkout into oracle/_ref/ (git-ignored);
    returns the path of the byte-code file, or None when the checkout does not have the file."""
    import py_compile
    src = os.path.join(reference_root, "e2e", "ttt_pytorch", "model.py")
    if not os.path.exists(src):
        return None
    os.makedirs(OUT, exist_ok=True)
    return py_compile.compile(src, cfile=os.path.join(OUT, PY_NAME + ".bin"), dfile="e2e/ttt_pytorch/model.py", doraise=True)


def load_python_reference():
    """Imports the byte-compiled reference model module (None when it has not been compiled).
    Its `v7_kernel_attention` does `from attention import flash_attention_v7` at call time, so
    whichever `attention.py` is first on sys.path serves it."""
    p = python_reference_path()
    if p is None:
        return None
    import importlib.machinery
    import importlib.util
    loader = importlib.machinery.SourcelessFileLoader(PY_NAME, p)
    spec = importlib.util.spec_from_loader(PY_NAME, loader)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[PY_NAME] = mod          # dataclasses look their module up by name
    loader.exec_module(mod)
    return mod


def build(reference_root, verbose=False):
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
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1], verbose=True))
    print(compile_python_reference(sys.argv[1]))
