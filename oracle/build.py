"""Build recipe for the CPU oracle (test infrastructure, never imported by the product).

    python oracle/build.py          # oracle/libmp_oracle.so  (C restatement, gcc + OpenMP)
    python oracle/build.py --ref    # additionally oracle/_ref/  (the reference's own C++ CPU
                                    #  extensions, compiled from its sources where they lie)
    python oracle/build.py --ref-cuda   # additionally oracle/_ref/cuda/ (the reference's own CUDA
                                    #  extensions, recompiled unmodified for sm_100a: the GPU
                                    #  implementation this library replaces, for side-by-side
                                    #  parity and timing on the same device)

    python oracle/build.py --ref-terms  # additionally oracle/_ref/libref_terms.so (the reference's
                                    #  stereo term builders, MPLayers/aux/aux.cpp, unmodified)

The reference sources are only read, never copied; the `--ref` outputs go to `oracle/_ref/`,
which is git-ignored.  `--ref` needs the reference checkout (path in $MPL_REFERENCE_DIR,
default the directory mounted next to this repository) and is skipped when it is absent.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libmp_oracle.so")
SRC = os.path.join(HERE, "mp_oracle.c")
REF_OUT = os.path.join(HERE, "_ref")


def reference_dir():
    """The reference checkout: $MPL_REFERENCE_DIR, else a directory `reference` next to this repository."""
    default = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return os.environ.get("MPL_REFERENCE_DIR", default)


def _cpu_has_fma():
    try:
        with open("/proc/cpuinfo") as f:
            return " fma " in f.read()
    except OSError:
        return False


def build_oracle(force=False):
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    cmd = [cc, "-O2", "-std=c11", "-fopenmp", "-fPIC", "-shared", "-ffp-contract=off"]
    if _cpu_has_fma():
        cmd.append("-mfma")  # fmaf() becomes one instruction; nothing else is contracted
    cmd += [SRC, "-o", LIB, "-lm"]
    subprocess.check_call(cmd)
    return LIB


def build_reference_cpu(force=False):
    """Compile the reference's TRWP / ISGMR C++ CPU extensions (forward only) into oracle/_ref/.

    Sources used (unmodified, read in place): MPLayers/TRWP/TRWP.cpp, MPLayers/ISGMR/ISGMR.cpp,
    MPLayers/common.cpp, tools/cpp/utils.cpp.  USE_CUDA is left undefined, so only the CPU path
    (ForwardCPU) is compiled.  Returns the output directory, or None if the reference is absent.
    """
    ref = reference_dir()
    if not os.path.isdir(os.path.join(ref, "MPLayers")):
        return None
    os.makedirs(REF_OUT, exist_ok=True)
    os.environ["CXX"] = "/usr/bin/g++"  # the default wrapper compiler cannot link OpenMP here
    from torch.utils.cpp_extension import load
    mp = os.path.join(ref, "MPLayers")
    for name in ("TRWP", "ISGMR"):
        bdir = os.path.join(REF_OUT, "build_" + name)
        so = os.path.join(REF_OUT, name + ".so")
        if os.path.exists(so) and not force:
            continue
        os.makedirs(bdir, exist_ok=True)
        load(name=name,
             sources=[os.path.join(mp, name, name + ".cpp"), os.path.join(mp, "common.cpp"),
                      os.path.join(ref, "tools", "cpp", "utils.cpp")],
             extra_include_paths=[mp, os.path.join(mp, name), os.path.join(ref, "tools", "cpp")],
             extra_cflags=["-O3", "-fopenmp", "-Wno-deprecated-declarations", "-w",
                           "-DMAX_DISPARITY=256", "-DTORCH_VERSION_MAJOR=2"],
             extra_ldflags=["-fopenmp"], build_directory=bdir, verbose=False)
        built = os.path.join(bdir, name + ".so")
        os.replace(built, so)
    return REF_OUT


_REF_CUDA = {
    # name: (directory under MPLayers, .cpp, .cu files, extra macros) -- MPLayers/setup.py:86-128
    "TRWP": ("TRWP", "TRWP.cpp", ["TRWP_forward.cu", "TRWP_backward.cu"], []),
    "ISGMR": ("ISGMR", "ISGMR.cpp", ["ISGMR_forward.cu", "ISGMR_backward.cu"], []),
    "TRWP_hard_soft": ("TRWP_hard_soft", "TRWP.cpp",
                       ["TRWP_forward.cu", "TRWP_backward.cu", "TRWP_forward_soft.cu",
                        "TRWP_backward_soft.cu", "TRWP_swbp.cu"], ["-DUSE_HARD", "-DUSE_SOFT"]),
}


def build_reference_cuda(force=False, names=("TRWP", "ISGMR", "TRWP_hard_soft")):
    """Compile the reference's TRWP / ISGMR / TRWP_hard_soft CUDA extensions for sm_100a into
    oracle/_ref/cuda/.

    Sources used (unmodified, read in place): the extension's .cpp and .cu files under MPLayers/,
    MPLayers/common.cpp, tools/cpp/utils.cpp, tools/cuda/cudaUtils.cu, with the reference's own
    macros (USE_CUDA, USE_HARD / USE_SOFT, MAX_DISPARITY=256 as in its "stereo" build,
    MPLayers/setup.py:28,62-63,86,113) and its nvcc flags except the architecture (sm_35 there).
    Returns the output directory, or None if the reference is absent.
    """
    ref = reference_dir()
    if not os.path.isdir(os.path.join(ref, "MPLayers")):
        return None
    out = os.path.join(REF_OUT, "cuda")
    os.makedirs(out, exist_ok=True)
    os.environ["CXX"] = "/usr/bin/g++"
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    mp = os.path.join(ref, "MPLayers")
    for name in names:
        bdir = os.path.join(out, "build_" + name)
        so = os.path.join(out, name + ".so")
        if os.path.exists(so) and not force:
            continue
        os.makedirs(bdir, exist_ok=True)
        sub, cpp, cus, macros = _REF_CUDA[name]
        load(name=name,
             sources=[os.path.join(mp, sub, cpp), os.path.join(mp, "common.cpp")] +
                     [os.path.join(mp, sub, c) for c in cus] +
                     [os.path.join(ref, "tools", "cpp", "utils.cpp"),
                      os.path.join(ref, "tools", "cuda", "cudaUtils.cu")],
             extra_include_paths=[mp, os.path.join(mp, sub), os.path.join(ref, "tools", "cpp"),
                                  os.path.join(ref, "tools", "cuda")],
             extra_cflags=["-O3", "-fopenmp", "-w", "-DUSE_CUDA", "-DMAX_DISPARITY=256",
                           "-DTORCH_VERSION_MAJOR=2"] + macros,
             extra_cuda_cflags=["-O3", "--expt-relaxed-constexpr", "-w", "-DUSE_CUDA",
                                "-DMAX_DISPARITY=256", "-DTORCH_VERSION_MAJOR=2"] + macros,
             extra_ldflags=["-fopenmp"], with_cuda=True, build_directory=bdir, verbose=False)
        os.replace(os.path.join(bdir, name + ".so"), so)
    return out


def build_reference_terms(force=False):
    """Compile the reference's stereo term builders (MPLayers/aux/aux.cpp: computeDSI, computeCues,
    computeSmoothnessContext) into oracle/_ref/libref_terms.so, with the macros of its own build
    (USE_OPENCV, USE_FLOAT; MPLayers/setup.py:39-56).

    aux.cpp is a template over the image container and only touches rows, cols, channels() and
    ptr(y, x); OpenCV's C++ headers are not installed here, so the include path carries a stand-in
    container with exactly those members (oracle/mat_standin/), and oracle/ref_terms_shim.cpp wraps
    the three functions in C entry points.  The arithmetic compiled is the reference's, unmodified.
    Returns the library path, or None if the reference is absent.
    """
    ref = reference_dir()
    src = os.path.join(ref, "MPLayers", "aux", "aux.cpp")
    if not os.path.exists(src):
        return None
    os.makedirs(REF_OUT, exist_ok=True)
    so = os.path.join(REF_OUT, "libref_terms.so")
    if os.path.exists(so) and not force:
        return so
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([cxx, "-O3", "-std=c++11", "-w", "-fPIC", "-shared", "-DUSE_OPENCV", "-DUSE_FLOAT",
                           "-I", os.path.join(HERE, "mat_standin"), "-I", os.path.join(ref, "MPLayers", "aux"),
                           "-I", os.path.join(ref, "tools", "cpp"), os.path.join(HERE, "ref_terms_shim.cpp"), src,
                           os.path.join(ref, "tools", "cpp", "utils.cpp"), "-o", so])
    return so


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference_cpu(force="--force" in sys.argv))
    if "--ref-terms" in sys.argv:
        print(build_reference_terms(force="--force" in sys.argv))
    if "--ref-cuda" in sys.argv:
        print(build_reference_cuda(force="--force" in sys.argv))
