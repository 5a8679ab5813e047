"""Compile the reference's own CUDA operator module (export_kvcomp.cpp, src/*.cu, src/*.cpp),
unmodified and from where it lies under the reference tree, for sm_100a into baseline/_ref/.

    REF=/path/to/reference python oracle/build_ref_cuda.py

The result (baseline/_ref/kvcomp_cuda.so) is a checker and the GPU kernel to compare with; the
package never imports it.  nvcc cross-compiles, so the build needs no GPU; running the module's
kernels does.  The reference's setup.py is not run (it wants to write into its own tree); the same
five sources and the same -O3 are given to torch's extension builder here, plus the arch flag the
reference's setup.py leaves to the environment.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
NAME = "kvcomp_cuda"


def build(ref_root=None, verbose=False):
    if ref_root is None:
        sys.path.insert(0, os.path.dirname(HERE))
        from oracle import ref_root as _rr
        ref_root = _rr.require()
    ext = os.path.join(ref_root, "kvcomp_cuda_extension")
    if not os.path.isdir(ext):
        raise FileNotFoundError("reference tree not found at %s" % ref_root)
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    src = os.path.join(ext, "src")
    return load(name=NAME,
                sources=[os.path.join(ext, "export_kvcomp.cpp")]
                + [os.path.join(src, f) for f in sorted(os.listdir(src)) if f.endswith((".cpp", ".cu"))],
                extra_include_paths=[os.path.join(ext, "include")],
                extra_cflags=["-O3"],
                extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a"],
                build_directory=OUT, verbose=verbose)


def load_prebuilt():
    """Import baseline/_ref/kvcomp_cuda.so if it was built earlier; None otherwise."""
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
    m = build(verbose="-v" in sys.argv)
    print("built", m.__file__)
