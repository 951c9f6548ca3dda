"""Builds plast_b200/libplast_b200.so from plast_b200/csrc with nvcc for sm_100a.

    python -m plast_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and has no PyTorch dependency. Objects go to
plast_b200/csrc/build/; a source is recompiled when it or any header is newer than its object.
-fmad=false keeps every fp32 multiply and add a separate rounding, which is what a sequence of
separate plast ops produces.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
ROOT = PKG.parent
LIB = PKG / "libplast_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",
    "-Xcompiler", "-fPIC,-O2,-fvisibility=default",
    "-I", str(ROOT / "include"),
    "-I", str(CSRC),
    "-I", str(OBJ),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libplast_b200.so")
    return exe


def _host_compiler() -> list[str]:
    # The CC/CXX environment may point at a toolchain without the standard headers nvcc needs.
    gxx = "/usr/bin/g++"
    return ["-ccbin", gxx] if os.path.exists(gxx) else []


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _stale(src: Path, obj: Path, headers_mtime: float) -> bool:
    if not obj.exists():
        return True
    m = obj.stat().st_mtime
    return src.stat().st_mtime > m or headers_mtime > m


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    # the device side of the elementwise engine as a string literal, for the NVRTC chain compiler
    dev_src = (CSRC / "ew_kernel_device.cuh").read_text()
    inc = OBJ / "ew_kernel_device_src.inc"
    text = 'R"PBSRC(' + dev_src + ')PBSRC"\n'
    if not inc.exists() or inc.read_text() != text:
        inc.write_text(text)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h"))
    headers_mtime = max(h.stat().st_mtime for h in headers)
    jobs = []
    objs = []
    for src in _sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(src, obj, headers_mtime):
            cmd = [nvcc, *_host_compiler(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        if verbose:
            print(" ".join(cmd), flush=True)
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for src, p in pool.map(run, jobs):
                if p.returncode != 0:
                    sys.stderr.write(p.stdout + p.stderr)
                    raise RuntimeError(f"nvcc failed on {src.name}")
                if verbose or ptxas_info:
                    sys.stderr.write(p.stdout + p.stderr)
    need_link = force or bool(jobs) or not LIB.exists() or any(
        o.stat().st_mtime > LIB.stat().st_mtime for o in objs)
    if need_link:
        cmd = [nvcc, *_host_compiler(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB), *map(str, objs), "-cudart", "static", "-Xlinker", "-z,defs"]
        if verbose:
            print(" ".join(cmd), flush=True)
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link of libplast_b200.so failed")
    return LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills per kernel")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.ptxas_info))


if __name__ == "__main__":
    main()
