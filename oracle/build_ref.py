"""Build the UNMODIFIED reference CUDA extensions into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this.

The four reference extensions (``qk_ext``, ``av_ext`` of sapa/setup.py:16-37 and
``dqk``, ``dav`` of deformsapa/setup.py:16-37) are compiled from the sources where
they lie in the reference checkout (never copied), with the reference's own NVCC
defines (sapa/setup.py:5-9) plus an explicit sm_100a ``-gencode``.  Outputs go only
into ``oracle/_ref/`` (git-ignored).  The built modules are the strongest checker
this repository has: parity tests run them on the GPU next to the new kernels.

The reference's ``setup.py`` is not executed; this file is the whole recipe.

    python oracle/build_ref.py [--reference DIR]
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# name -> sources relative to the reference root
EXTENSIONS = {
    "qk_ext": [
        "sapa/sapa/src/cuda/qk_cuda.cpp",
        "sapa/sapa/src/cuda/qk_cuda_kernel.cu",
        "sapa/sapa/src/qk_ext.cpp",
    ],
    "av_ext": [
        "sapa/sapa/src/cuda/av_cuda.cpp",
        "sapa/sapa/src/cuda/av_cuda_kernel.cu",
        "sapa/sapa/src/av_ext.cpp",
    ],
    "dqk": [
        "deformsapa/deformsapa/src/cuda/deform_qk_cuda.cpp",
        "deformsapa/deformsapa/src/cuda/deform_qk_cuda_kernel.cu",
        "deformsapa/deformsapa/src/deform_qk.cpp",
    ],
    "dav": [
        "deformsapa/deformsapa/src/cuda/deform_av_cuda.cpp",
        "deformsapa/deformsapa/src/cuda/deform_av_cuda_kernel.cu",
        "deformsapa/deformsapa/src/deform_av.cpp",
    ],
}

NVCC_DEFINES = [
    "-D__CUDA_NO_HALF_OPERATORS__",
    "-D__CUDA_NO_HALF_CONVERSIONS__",
    "-D__CUDA_NO_HALF2_OPERATORS__",
]


def built(name: str) -> bool:
    return os.path.exists(os.path.join(OUT, name + ".so"))


def build(reference: str, force: bool = False) -> list[str]:
    """Compile every reference extension that is not built yet; returns names built."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils.cpp_extension import load

    done = []
    for name, rel in EXTENSIONS.items():
        if built(name) and not force:
            continue
        srcs = [os.path.join(reference, r) for r in rel]
        missing = [s for s in srcs if not os.path.exists(s)]
        if missing:
            raise FileNotFoundError(f"reference sources missing: {missing}")
        bdir = os.path.join(OUT, "_build_" + name)
        os.makedirs(bdir, exist_ok=True)
        load(
            name=name,
            sources=srcs,
            extra_cflags=["-DWITH_CUDA", "-O2"],
            extra_cuda_cflags=["-DWITH_CUDA", "-O2",
                               "-gencode", "arch=compute_100a,code=sm_100a"] + NVCC_DEFINES,
            build_directory=bdir,
            with_cuda=True,
            is_python_module=False,   # do not import here: just produce the .so
            verbose=False,
        )
        so = os.path.join(bdir, name + ".so")
        os.replace(so, os.path.join(OUT, name + ".so"))
        shutil.rmtree(bdir, ignore_errors=True)
        done.append(name)
    return done


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SAPA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"),
                    help="path of a tiny-smart/sapa checkout (default: $SAPA_REFERENCE, else a `reference` folder next to this repository)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.reference):
        print(f"reference checkout not found at {a.reference}; nothing built", file=sys.stderr)
        return 0
    os.makedirs(OUT, exist_ok=True)
    names = build(a.reference, a.force)
    print("built:", names, "->", OUT)
    return 0


if __name__ == "__main__":
    sys.exit(main())
