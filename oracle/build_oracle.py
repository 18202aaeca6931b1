"""Build recipe for the CPU checkers (test infrastructure, never part of the product path).

Two artefacts are produced, both only under ``oracle/_ref/`` (git-ignored):

* ``liboracle_conv.so`` -- the plain-C restatement in ``oracle/oracle_conv.c``.
* the reference project's own Cython kernels (``im2row_nhwc_cython`` ...), compiled from the
  ``.pyx`` files where they lie in the mounted reference checkout.  This step only runs when
  that checkout is present; the sources are never copied into this repository.  The modules are
  built with ``-march=x86-64-v3`` instead of the reference's ``-march=native`` so the binaries
  also run on a different host CPU.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
GCC = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"

# Cython modules of the reference that lie on (or right beside) the convolution path.
REF_MODULES = [
    "im2row_nhwc_cython", "im2col_nchw_cython", "add_nhwc_cython", "add_nchw_cython",
    "transpose_cython", "bn_inference_cython", "bn_relu_inference_cython", "relu_cython",
    "bn_training_cython", "eltw_sum_cython", "max_pool_2d_nhwc_cython", "max_pool_2d_nchw_cython",
    "average_pool_2d_nhwc_cython", "average_pool_2d_nchw_cython",
    # not on the path, but the reference package refuses to import without them
    # (pydtnn/cython_modules/__init__.py:20-41); needed only to generate golden vectors
    "argmax_cython", "depthwise_conv_cython", "im2col_1ch_nchw_cython", "im2row_1ch_nhwc_cython",
    "pointwise_conv_cython",
]


def _run(cmd):
    subprocess.run(cmd, check=True)


def _newer(src, dst):
    return (not os.path.exists(dst)) or os.path.getmtime(src) > os.path.getmtime(dst)


def build_c_oracle(force=False):
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "oracle_conv.c")
    dst = os.path.join(OUT, "liboracle_conv.so")
    if force or _newer(src, dst):
        _run([GCC, "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-o", dst, src, "-lm"])
    return dst


def build_reference_kernels(ref_root="/root/reference", force=False):
    """Compile the reference's Cython kernels into oracle/_ref (no-op without the checkout)."""
    pyx_dir = os.path.join(ref_root, "pydtnn", "cython_modules")
    if not os.path.isdir(pyx_dir):
        return []
    import numpy
    os.makedirs(os.path.join(OUT, "gen"), exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    inc = ["-I" + numpy.get_include(), "-I" + sysconfig.get_paths()["include"]]
    built = []
    for mod in REF_MODULES:
        pyx = os.path.join(pyx_dir, mod + ".pyx")
        c_file = os.path.join(OUT, "gen", mod + ".c")
        so = os.path.join(OUT, mod + ext)
        if force or _newer(pyx, so):
            _run([sys.executable, "-m", "cython", "-3", "-o", c_file, pyx])
            _run([GCC, "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-g0", "-w",
                  "-DNPY_NO_DEPRECATED_API=NPY_1_7_API_VERSION", *inc, "-o", so, c_file])
        built.append(so)
    return built


if __name__ == "__main__":
    print(build_c_oracle(force="--force" in sys.argv))
    for p in build_reference_kernels(force="--force" in sys.argv):
        print(p)
