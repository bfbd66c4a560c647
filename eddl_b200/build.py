"""Build the eddl_b200 native libraries in-tree.

``build_kernels()``  nvcc (sm_100a) -> ``eddl_b200/lib/libeddl_b200.so``: the CUDA kernels and
                     the C ABI declared in ``include/eddl_b200.h``.  Needs nothing but the
                     CUDA toolkit and NCCL.
``build_dropin()``   g++ -> ``baseline/_ref/libeddl_b200_dropin.so``: the C++ shim that defines
                     EDDL's ``gpu_*`` functions on top of the C ABI (``eddl_b200/shim``), the
                     distributed entry points and the net harness, linked with EDDL's own host
                     sources compiled with ``-DcGPU`` (``baseline/build_host.py``).  Needs the EDDL
                     source tree; skipped when it is absent (the prebuilt library is used).
"""
import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _nvcc_one(args):
    src, obj, headers, verbose = args
    if not _newer(obj, [src] + headers):
        return ""
    cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr[-6000:]))
    return r.stderr


def build_kernels(verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "eddl_b200.h"))
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    tasks = [(s, os.path.join(objdir, os.path.basename(s)[:-3] + ".o"), headers, verbose) for s in srcs]
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count()) as ex:
        logs = list(ex.map(_nvcc_one, tasks))
    if verbose:
        sys.stderr.write("".join(logs))
    lib = os.path.join(LIBDIR, "libeddl_b200.so")
    objs = [t[1] for t in tasks]
    if _newer(lib, objs):
        cmd = [NVCC, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                     "-lnccl", "-lcuda", "-Xlinker", "-rpath,$ORIGIN"]
        subprocess.run(cmd, check=True)
    return lib


def _host_recipe():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import build_host
    return build_host


def build_dropin():
    recipe = _host_recipe()
    outdir = os.path.join(ROOT, "baseline", "_ref")
    lib = os.path.join(outdir, "libeddl_b200_dropin.so")
    if not recipe.have_reference():
        return lib if os.path.exists(lib) else None
    kernels = build_kernels()
    objs = recipe.build_gpu_host_objects()
    mine = sorted(os.path.join(PKG, "shim", f) for f in os.listdir(os.path.join(PKG, "shim")) if f.endswith(".cpp"))
    mine.append(os.path.join(PKG, "host", "net_harness.cpp"))
    hdrs = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    flags = recipe.COMMON + ["-DcGPU", "-I" + recipe.CUDA_INC, "-I" + os.path.join(ROOT, "include")]
    shim_objs = []
    for s in mine:
        o = os.path.join(outdir, "obj_shim", os.path.basename(s)[:-4] + ".o")
        os.makedirs(os.path.dirname(o), exist_ok=True)
        if _newer(o, [s] + hdrs):
            subprocess.run(["g++"] + flags + ["-c", s, "-o", o], check=True)
        shim_objs.append(o)
    # every gpu_* symbol the reference host code needs and the shim does not define becomes
    # a stub that throws (no CPU fallback): generated from the mangled names, not committed
    stubs_cpp = os.path.join(outdir, "obj_shim", "trap_stubs.cpp")
    stubs_o = stubs_cpp[:-4] + ".o"
    undefined = _undefined_gpu_symbols(objs, shim_objs)
    body = ['#include <stdexcept>\n#include <string>\n',
            'static void eddlb200_trap(const char *n) { throw std::runtime_error(std::string("[eddl_b200] ") + n + " is not implemented in the B200 backend (no CPU fallback)"); }\n']
    for mangled, pretty in undefined:
        body.append('extern "C" void %s() { eddlb200_trap("%s"); }\n' % (mangled, pretty.replace('"', "'")))
    text = "".join(body)
    if not os.path.exists(stubs_cpp) or open(stubs_cpp).read() != text:
        open(stubs_cpp, "w").write(text)
    if _newer(stubs_o, [stubs_cpp]):
        subprocess.run(["g++", "-fPIC", "-O1", "-c", stubs_cpp, "-o", stubs_o], check=True)
    if _newer(lib, objs + shim_objs + [stubs_o, kernels]):
        cmd = (["g++", "-shared", "-Wl,-Bsymbolic", "-o", lib, "-fopenmp"] + shim_objs + [stubs_o] + objs +
               ["-L" + LIBDIR, "-leddl_b200", "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart",
                "-Wl,-rpath,$ORIGIN/../../eddl_b200/lib", "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64"),
                "-Wl,--no-undefined", "-lpthread"])
        subprocess.run(cmd, check=True)
    return lib


def _undefined_gpu_symbols(ref_objs, shim_objs):
    def syms(objs, flag):
        out = {}
        r = subprocess.run(["nm", flag] + objs, capture_output=True, text=True)
        for line in r.stdout.splitlines():
            parts = line.split()
            if len(parts) >= 2 and parts[-2] in ("U", "T", "W", "B", "D"):
                out[parts[-1]] = parts[-2]
        return out
    und = {s for s, k in syms(ref_objs, "-u").items() if k == "U"}
    defined = {s for s, k in syms(ref_objs + shim_objs, "--defined-only").items()}
    need = sorted(s for s in und - defined if s.startswith("_Z") and ("gpu" in s))
    if not need:
        return []
    r = subprocess.run(["c++filt"] + need, capture_output=True, text=True)
    pretty = r.stdout.splitlines()
    return [(m, p) for m, p in zip(need, pretty) if p.startswith("gpu_") or p.startswith("_gpu_")
            or p.startswith("cpu2gpu") or p.startswith("gpu2cpu") or "gpu" in p.split("(")[0]]


if __name__ == "__main__":
    what = sys.argv[1:] or ["kernels"]
    if "kernels" in what:
        print(build_kernels(verbose="-v" in what))
    if "dropin" in what:
        print(build_dropin())
