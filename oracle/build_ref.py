"""Compile the reference's own host extension (CPU arms of ``torch.ops.quactlize.*``) into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path imports this file or anything it builds; only the parity
tests, the smoke check and the CPU-baseline leg of the benchmark load the resulting library, and only as the
checker / the timed CPU reference.

The sources are compiled where they lie in the read-only reference checkout (``QUACTLIZE_REFERENCE_ROOT`` or ``--ref``,
else a directory named ``reference`` beside this repository); nothing is copied.  The reference extension is host C++ that needs
CUTLASS/CuTe *headers* only; the stock CUTLASS tree vendored with flashinfer serves.  Sources compiled
(paths inside the reference project):

    quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp        k-quant CPU arms, artifact producers, op registry
    quactlize/csrc/preprocess/thop/ppu_backend.cpp             the dlopen seam (QUACTLIZE_PPU_LIB)
    quactlize/csrc/preprocess/thop/weight_preprocess_ops.cpp   GPTQ pack / quantise helpers
    quactlize/csrc/preprocess/cutlass_kernels/cutlass_preprocessors.cpp

Usage:  python oracle/build_ref.py            (no-op when the library already exists)
"""
import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "quactlize_ref_C"


def ref_root() -> str:
    """The reference checkout: QUACTLIZE_REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    return os.environ.get("QUACTLIZE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def built_library():
    hits = sorted(glob.glob(os.path.join(OUT, NAME + "*.so")))
    return hits[0] if hits else None


def build(verbose: bool = False):
    """Returns the path of the built library, or None when the reference checkout is not present."""
    lib = built_library()
    if lib:
        return lib
    root = ref_root()
    if not os.path.isdir(os.path.join(root, "quactlize", "csrc")):
        return None
    import flashinfer
    from torch.utils import cpp_extension
    cutlass = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass", "include")
    os.makedirs(OUT, exist_ok=True)
    pre = os.path.join(root, "quactlize", "csrc", "preprocess")
    cpp_extension.load(
        name=NAME,
        sources=[os.path.join(pre, "thop", "gguf_prepass_ops.cpp"),
                 os.path.join(pre, "thop", "ppu_backend.cpp"),
                 os.path.join(pre, "thop", "weight_preprocess_ops.cpp"),
                 os.path.join(pre, "cutlass_kernels", "cutlass_preprocessors.cpp")],
        extra_include_paths=[pre, os.path.join(root, "quactlize", "include"), cutlass, "/usr/local/cuda/include"],
        extra_cflags=["-std=c++17", "-O2", "-DUSE_AIU=1", "-Wno-unused-function", "-Wno-sign-compare"],
        extra_ldflags=["-ldl"], is_python_module=False, build_directory=OUT, verbose=verbose)
    return built_library()


if __name__ == "__main__":
    if "--ref" in sys.argv:
        os.environ["QUACTLIZE_REFERENCE_ROOT"] = sys.argv[sys.argv.index("--ref") + 1]
    lib = build(verbose="-v" in sys.argv)
    print(lib or "reference checkout not present; nothing built")
