"""Compile the EDDL v1.1 host sources in place with plain g++.

The reference's CMake superbuild needs network access and Eigen, so it is not used: every C++ source under
``<reference>/src`` is compiled where it lies into objects under a git-ignored ``_ref`` directory.  The reference tree is
the directory ``$EDDL_REFERENCE`` names, or a checkout called ``reference`` beside this repository.  Two users:

* ``eddl_b200/build.py`` links the objects built with ``-DcGPU`` (never ``-DcCUDNN``: cuDNN calls are inlined in the
  layer code and would bypass the ``gpu_*`` boundary) with the B200 backend, so that the reference's ``Net`` runs on
  ``CS_GPU`` unmodified (``baseline/_ref/libeddl_b200_dropin.so``);
* ``oracle/build_ref.py`` links the objects built without ``-DcGPU`` into the parity checker / CPU baseline.

Eigen 3.4.0 (cmake/eigen.CMakeLists.txt.in:8) is replaced by the stand-in header in ``baseline/eigen_standin``: it only
lets the reference's host headers compile and supplies the CPU GEMM; no GPU arithmetic comes from it.  Excluded sources:
FPGA backend, the socket "distributed" draft, the reference's own CUDA backend (``src/hardware/gpu``), and the generated
protobuf file (ONNX compiles to stubs without ``-DcPROTO``).  No ``-Ofast/-ffast-math`` (the reference disables them for
correctness runs, CMakeLists.txt:14,189-198).
"""
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("EDDL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
CUDA_INC = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"

COMMON = ["-std=c++14", "-O2", "-fopenmp", "-fPIC", "-w", "-DEDDL_LINUX",
          "-mavx2", "-mfma", "-ffp-contract=off",
          "-I" + os.path.join(HERE, "eigen_standin"),
          "-I" + os.path.join(REF, "include"), "-I" + os.path.join(REF, "src")]

def reference_sources():
    out = []
    for d, _, fs in os.walk(os.path.join(REF, "src")):
        for f in fs:
            p = os.path.join(d, f)
            if not f.endswith(".cpp"):
                continue
            rel = os.path.relpath(p, REF)
            if ("hardware/fpga" in rel or "hardware/gpu" in rel or "distributed" in rel
                    or "onnx.pb" in rel or "layers/fpga" in rel or rel.endswith("apis/fpga.cpp")):
                continue
            out.append(p)
    return sorted(out)


def _compile(args):
    src, obj, flags = args
    if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return None
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    extra = ["-include", "stdexcept"]  # descriptor_reduce.cpp:100 relies on a transitive include
    cmd = ["g++"] + flags + extra + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        return "FAILED %s\n%s" % (src, r.stderr[-3000:])
    return None


def compile_objects(objdir, flags, jobs=None):
    srcs = reference_sources()
    tasks = []
    for s in srcs:
        rel = os.path.relpath(s, os.path.join(REF, "src")).replace("/", "__")
        tasks.append((s, os.path.join(objdir, rel[:-4] + ".o"), flags))
    with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count()) as ex:
        errs = [e for e in ex.map(_compile, tasks) if e]
    if errs:
        raise RuntimeError("\n".join(errs[:5]))
    return [t[1] for t in tasks]


def have_reference():
    return os.path.isdir(os.path.join(REF, "src"))


def build_gpu_host_objects():
    """baseline/_ref/obj_gpu/*.o : the reference host code compiled with -DcGPU."""
    outdir = os.path.join(ROOT, "baseline", "_ref", "obj_gpu")
    return compile_objects(outdir, COMMON + ["-DcGPU", "-I" + CUDA_INC])


if __name__ == "__main__":
    if not have_reference():
        sys.exit("reference sources not found at " + REF)
    print(len(build_gpu_host_objects()), "objects")
