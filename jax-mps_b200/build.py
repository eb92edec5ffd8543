"""Builds libb200core.so (the C-ABI core: parser, plan compiler, runtime and
the hand-written sm_100a kernels) in-tree with nvcc, and the PJRT veneer when
the PJRT C API header is available. No GPU is needed to build."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "b200" / "libb200core.so"
SOURCES = ["parser.cc", "codegen.cc", "compiler.cc", "runtime.cc", "kernels.cu", "gemm16.cu"]


def _nccl_include() -> str:
    try:
        import nvidia.nccl  # type: ignore
        p = Path(nvidia.nccl.__path__[0]) / "include"
        if (p / "nccl.h").exists():
            return str(p)
    except Exception:
        pass
    return "/usr/include"


def needs_build() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(CSRC.glob("*.cc")) + list(CSRC.glob("*.cu")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + \
        [HERE.parent / "include" / "b200_core.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    build_dir = HERE / "build"
    build_dir.mkdir(exist_ok=True)
    common = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", str(CSRC), "-I", _nccl_include(),
              "-diag-suppress", "177,186"]
    procs = []
    for s in SOURCES:
        o = build_dir / (s.rsplit(".", 1)[0] + ".o")
        objs.append(str(o))
        cmd = [nvcc, *common, "-c", str(CSRC / s), "-o", str(o)]
        if s.endswith(".cu"):
            cmd.insert(1, "-Xptxas=-v")
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{out}")
        if verbose and out.strip():
            print(out)
    link = [nvcc, "-shared", "-o", str(OUT), *objs, "-cudart", "static", "-ldl", "-lpthread",
            "-Xlinker", "--exclude-libs,ALL"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
