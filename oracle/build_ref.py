"""Compile the reference's own host codec (src/huffman.cpp, src/utils.cpp) as a CPU-only
torch extension into oracle/_ref/ -- a checker for the C restatement, never product code.

The sources are compiled where they lie under the reference tree (REF=/path/to/reference);
nothing is copied.  The reference's own build system is not run:
its setup.py also compiles the CUDA kernels, which this checker does not need.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "kvc_ref_huffman"


def build(ref_root=None, verbose=False):
    if ref_root is None:
        from . import ref_root as _rr
        ref_root = _rr.require()
    ext = os.path.join(ref_root, "kvcomp_cuda_extension")
    if not os.path.isdir(ext):
        raise FileNotFoundError("reference tree not found at %s" % ref_root)
    os.makedirs(OUT, exist_ok=True)
    from torch.utils.cpp_extension import load
    return load(name=NAME,
                sources=[os.path.join(HERE, "ref_binding.cpp"),
                         os.path.join(ext, "src", "huffman.cpp"),
                         os.path.join(ext, "src", "utils.cpp")],
                extra_include_paths=[os.path.join(ext, "include")],
                extra_cflags=["-O2"], build_directory=OUT, verbose=verbose)


def load_prebuilt():
    """Import oracle/_ref/kvc_ref_huffman.so if it was built earlier; None otherwise."""
    so = os.path.join(OUT, NAME + ".so")
    if not os.path.exists(so):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch symbols must be loaded first)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    from oracle import ref_root as _rr
    m = build(_rr.require(), verbose="-v" in sys.argv)
    print("built", m.__file__)
