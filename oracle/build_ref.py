"""Compile the reference's own GEMM extension (blockquant_ext_src/{blockquant_ext.cpp,gemm.cu})
for sm_100a, from the sources where they lie in the reference checkout, into
``oracle/_ref/blockquant_ext.so`` -- TEST INFRASTRUCTURE: the on-device oracle of the GEMM tests.

    python oracle/build_ref.py /path/to/HBQ        (or: HBQ_REFERENCE_DIR=/path/to/HBQ python oracle/build_ref.py)

Nothing is copied into this repository; only the built module lands in ``oracle/_ref/`` (which
is git-ignored).  The flags are those of the reference's setup.py (-O3 --use_fast_math
--expt-relaxed-constexpr) with the architecture set to sm_100a.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HBQ_REFERENCE_DIR")
    if not ref or not os.path.isdir(os.path.join(ref, "blockquant_ext_src")):
        raise SystemExit("usage: build_ref.py REFERENCE_DIR (a checkout of SeoLabCornell/HBQ), or set HBQ_REFERENCE_DIR")
    src = os.path.join(ref, "blockquant_ext_src")
    cu, cpp = os.path.join(src, "gemm.cu"), os.path.join(src, "blockquant_ext.cpp")
    so = os.path.join(OUT, "blockquant_ext.so")
    if os.path.exists(so) and all(os.path.getmtime(so) > os.path.getmtime(f) for f in (cu, cpp, __file__)):
        print("up to date:", so)
        return
    os.makedirs(OUT, exist_ok=True)
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for d in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", d]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DTORCH_EXTENSION_NAME=blockquant_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DNDEBUG"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    o_cu, o_cpp = os.path.join(OUT, "gemm.o"), os.path.join(OUT, "blockquant_ext.o")
    if not (os.path.exists(o_cu) and os.path.getmtime(o_cu) > os.path.getmtime(cu)):   # ~5 min: keep it
        subprocess.check_call(["nvcc", "-c", cu, "-o", o_cu + ".tmp", "-O3", "--use_fast_math", "--expt-relaxed-constexpr",
                               "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--threads", "8",
                               "-Xcompiler", "-fPIC", *defs, *inc], env=env)
        os.replace(o_cu + ".tmp", o_cu)
    subprocess.check_call(["g++", "-c", cpp, "-o", o_cpp, "-O3", "-std=c++17", "-fPIC", *defs, *inc], env=env)
    libdirs = ce.library_paths("cuda")
    ld = []
    for d in libdirs:
        ld += [f"-L{d}", f"-Wl,-rpath,{d}"]
    subprocess.check_call(["g++", "-shared", o_cu, o_cpp, "-o", so, *ld, "-lc10", "-lc10_cuda", "-ltorch_cpu",
                           "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"], env=env)
    os.remove(o_cpp)
    print("built:", so)


if __name__ == "__main__":
    main()
