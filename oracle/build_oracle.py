"""Build recipe for the checker libraries (test infrastructure, never shipped).

* ``oracle/liboracle.so``      - the C restatement in ``attention_oracle.c``;
  plain gcc, -O2, no fast-math, FMA contraction off, so the fp32 summation
  order written in the source is the order executed.
* ``oracle/_ref/libref_cpu.so`` - the reference project's own
  ``cpu_attention`` (src/demo.cu:28-70), compiled from the reference checkout
  where it lies (never copied), with its ``main`` renamed away and a stub for
  the one library symbol the file links against.  Only built when a reference
  checkout is present; the built file travels with the repo to machines that
  have no checkout.
* ``oracle/_ref/libref_gpu.so`` - the reference project's ``mma.sync`` kernel
  (kernels/flash_attention.cu) compiled unchanged for sm_100a, used only as a
  same-box GPU comparison line by the benchmark.
* ``oracle/_ref/flash_bench`` / ``flash_demo`` - the reference's two
  executables (src/bench.cu, src/demo.cu) compiled unchanged against THIS
  repository's header and library: the drop-in proof.  Needs the product
  library to have been built first.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_OUT = os.path.join(HERE, "_ref")
# the reference checkout: FA_REFERENCE_DIR, else a directory "reference" next to this repository
REFERENCE = os.environ.get("FA_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

# Itanium-mangled name of cpu_attention(const float*, const float*, const float*,
# float*, float*, int, int, float, bool) as the reference file defines it.
REF_CPU_SYMBOL = "_Z13cpu_attentionPKfS0_S0_PfS1_iifb"
# transformer::launch_flash_attention(const transformer::FlashAttentionParams&)
REF_LAUNCH_SYMBOL = "_ZN11transformer22launch_flash_attentionERKNS_20FlashAttentionParamsE"


def _run(cmd: list[str]) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        raise RuntimeError("oracle build step failed: " + cmd[0])


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.exists(s) and os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "attention_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if force or not _newer(out, src):
        _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off",
              "-fno-fast-math", src, "-o", out, "-lm"])
    return out


def have_reference() -> bool:
    return os.path.isfile(os.path.join(REFERENCE, "src", "demo.cu"))


def build_ref_cpu(force: bool = False) -> str | None:
    """cpu_attention out of the reference's src/demo.cu, as a shared object."""
    out = os.path.join(REF_OUT, "libref_cpu.so")
    if not have_reference():
        return out if os.path.exists(out) else None
    demo = os.path.join(REFERENCE, "src", "demo.cu")
    stub = os.path.join(HERE, "ref_link_stub.cu")
    if not force and _newer(out, demo, stub):
        return out
    os.makedirs(REF_OUT, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    obj = os.path.join(REF_OUT, "demo_ref.o")
    stub_obj = os.path.join(REF_OUT, "ref_link_stub.o")
    # -O2, no --use_fast_math: this object is the parity oracle, not a speed run.
    common = [nvcc, "-std=c++17", "-O2", *ARCH, "-include", "cstdint",
              "-Xcompiler", "-fPIC,-ffp-contract=off"]
    _run(common + ["-Dmain=ref_demo_main", "-c", demo, "-o", obj])
    _run(common + ["-I", os.path.join(REFERENCE, "include"), "-c", stub, "-o", stub_obj])
    _run([nvcc, "-shared", *ARCH, obj, stub_obj, "-o", out, "-lcudart"])
    return out


def build_ref_gpu(force: bool = False) -> str | None:
    """The reference's own mma.sync kernel, recompiled unchanged for sm_100a."""
    out = os.path.join(REF_OUT, "libref_gpu.so")
    if not have_reference():
        return out if os.path.exists(out) else None
    src = os.path.join(REFERENCE, "kernels", "flash_attention.cu")
    if not force and _newer(out, src):
        return out
    os.makedirs(REF_OUT, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    _run([nvcc, "-std=c++17", "-O3", "--use_fast_math", "-lineinfo", *ARCH,
          "-include", "cstdint", "-Xcompiler", "-fPIC", "-shared", src, "-o", out,
          "-lcudart"])
    return out


def build_ref_executables(product_lib_dir: str, force: bool = False) -> list[str]:
    """flash_bench / flash_demo from the reference sources, unchanged, against
    this repository's include/flash_attention.h and libfa_b200.so.

    The reference files include "../include/flash_attention.h" relative to
    their own directory, so they are compiled through a staging directory of
    symlinks: <stage>/src/*.cu -> reference, <stage>/include -> this repo."""
    outs = [os.path.join(REF_OUT, n) for n in ("flash_bench", "flash_demo")]
    if not have_reference():
        return [o for o in outs if os.path.exists(o)]
    lib = os.path.join(product_lib_dir, "libfa_b200.so")
    hdr = os.path.join(ROOT, "include", "flash_attention.h")
    if not os.path.exists(lib):
        raise RuntimeError("build the product library before the reference executables")
    os.makedirs(REF_OUT, exist_ok=True)
    stage = os.path.join(REF_OUT, "stage")
    os.makedirs(os.path.join(stage, "src"), exist_ok=True)
    inc_link = os.path.join(stage, "include")
    if os.path.islink(inc_link):
        os.unlink(inc_link)
    os.symlink(os.path.join(ROOT, "include"), inc_link)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    for name, out in (("bench", outs[0]), ("demo", outs[1])):
        ref_src = os.path.join(REFERENCE, "src", name + ".cu")
        link = os.path.join(stage, "src", name + ".cu")
        if os.path.islink(link):
            os.unlink(link)
        os.symlink(ref_src, link)
        if not force and _newer(out, ref_src, lib, hdr):
            continue
        rpath = os.path.relpath(product_lib_dir, REF_OUT)
        _run([nvcc, "-std=c++17", "-O3", "--use_fast_math", "-lineinfo", *ARCH, link,
              "-o", out, "-L", product_lib_dir, "-lfa_b200",
              "-Xlinker", "-rpath=$ORIGIN/" + rpath, "-lcudart"])
    return outs


def build_all(force: bool = False) -> dict:
    res = {"oracle": build_oracle(force)}
    res["ref_cpu"] = build_ref_cpu(force)
    res["ref_gpu"] = build_ref_gpu(force)
    return res


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
