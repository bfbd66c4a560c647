"""TEST INFRASTRUCTURE ONLY: the reference's own CPU implementation as a shared library.

Links the EDDL v1.1 host sources, compiled in place WITHOUT ``-DcGPU`` by the recipe in ``baseline/build_host.py``, with
``oracle/ref_capi.cpp`` and the net harness into ``oracle/_ref/libeddl_ref_cpu.so``: the parity checker (the
reference's ``cpu_*`` functions and its ``Net`` driven on ``CS_CPU``) and the timed CPU baseline.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import build_host  # noqa: E402

REF = build_host.REF
COMMON = build_host.COMMON
have_reference = build_host.have_reference


def build_cpu():
    """oracle/_ref/libeddl_ref_cpu.so = reference CPU objects + oracle/ref_capi.cpp + the net harness."""
    outdir = os.path.join(HERE, "_ref")
    objs = build_host.compile_objects(os.path.join(outdir, "obj_cpu"), COMMON)
    lib = os.path.join(outdir, "libeddl_ref_cpu.so")
    mine = [os.path.join(HERE, "ref_capi.cpp"), os.path.join(ROOT, "eddl_b200", "host", "net_harness.cpp")]
    newest = max(os.path.getmtime(p) for p in objs + mine)
    if os.path.exists(lib) and os.path.getmtime(lib) >= newest:
        return lib
    cmd = ["g++", "-shared", "-Wl,-Bsymbolic", "-o", lib] + COMMON + mine + objs + ["-lpthread"]
    subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    if not have_reference():
        sys.exit("reference sources not found at " + REF)
    print(build_cpu())
