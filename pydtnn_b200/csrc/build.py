"""Compile the CUDA sources in this directory into ``pydtnn_b200/libb2c.so`` for sm_100a.

    python pydtnn_b200/csrc/build.py [--force] [-v] [--variant profile|switches]

Two development variants of the tensor-core kernel can be built next to the product library (they are never loaded
by the package; ``role_profile.py`` in this directory loads them by path):

* ``--variant profile``  -> ``pydtnn_b200/libb2c_profile.so`` (``-DB2C_TC_PROFILE``): every warp role of CTA 0 adds up
  the cycles it spends waiting and working (slots named in ``role_profile.py``), read with ``b2c_debug_prof``.
* ``--variant switches`` -> ``pydtnn_b200/libb2c_switches.so`` (``-DB2C_TC_SWITCHES``): the environment variable
  ``B2C_TC_DBG`` switches parts of the kernel off to see what the rest costs (results are then wrong): 2 = one MMA of
  three, 4 = transform warps do no work, 32 = no MMA, 64 = no TMA loads; values add.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
SOURCES = ["api.cu", "conv_fma.cu", "conv_tc.cu", "aux_ops.cu"]
OUT = os.path.join(PKG, "libb2c.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]
VARIANTS = {None: ("", [], OUT),
            "profile": (".profile", ["-DB2C_TC_PROFILE"], os.path.join(PKG, "libb2c_profile.so")),
            "switches": (".switches", ["-DB2C_TC_SWITCHES"], os.path.join(PKG, "libb2c_switches.so"))}


def build(force=False, verbose=False, variant=None):
    suffix, defines, out = VARIANTS[variant]
    srcs = [os.path.join(HERE, s) for s in SOURCES]
    deps = srcs + [os.path.join(HERE, "b2c_common.cuh"), os.path.join(os.path.dirname(PKG), "include", "b2c.h")]
    deps += [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cuh")]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    objs = []
    procs = []
    for s in srcs:
        o = s[:-3] + suffix + ".o"
        objs.append(o)
        procs.append((s, subprocess.Popen([NVCC, *FLAGS, *defines, "-c", s, "-o", o], stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        text, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(text)
        if p.returncode:
            failed = True
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([NVCC, "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    return out


if __name__ == "__main__":
    variant = sys.argv[sys.argv.index("--variant") + 1] if "--variant" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, variant=variant))
