"""Builds libshield_v_cuda.so (strict) and libshield_v_cuda_experimental.so for sm_100a, in tree.

    python -m shield_sisa_b200.build [--force]

Kernels are compiled by nvcc for sm_100a only (`-gencode arch=compute_100a,code=sm_100a -lineinfo`), host sources by
the system g++ (C++17); objects land in shield_sisa_b200/lib/obj.  The compute revision baked into the library is the
SHA-256 of all sources under csrc/ and include/, so a certificate issued for one build never matches another.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INC = ROOT / "include"
LIB = PKG / "lib"
OBJ = LIB / "obj"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA / "bin" / "nvcc")
CXX = "/usr/bin/g++"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", f"-I{INC}", f"-I{CSRC / 'kernels'}"]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-ffp-contract=off", "-Wall", "-Wextra",
             f"-I{INC}", f"-I{CSRC}", f"-I{CUDA / 'include'}"]


def sources():
    cu = sorted((CSRC / "kernels").glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    return cu, cpp


def revision() -> str:
    h = hashlib.sha256()
    files = sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.cpp")) +
                   list(CSRC.rglob("*.hpp")) + list(INC.glob("*.h")))
    for f in files:
        h.update(f.relative_to(ROOT).as_posix().encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def build(force: bool = False, verbose: bool = False, dev_probes: bool = False) -> list[Path]:
    """dev_probes: compile the kernels with -DSHVK_DEV_PROBES (timing probes read from the environment; for
    measurements only, never the build that is shipped or tested)."""
    cu, cpp = sources()
    rev = revision() + ("-probes" if dev_probes else "")
    OBJ.mkdir(parents=True, exist_ok=True)
    stamp = LIB / "revision.txt"
    libs = [LIB / "libshield_v_cuda.so", LIB / "libshield_v_cuda_experimental.so"]
    if not force and stamp.exists() and stamp.read_text() == rev and all(p.exists() for p in libs):
        return libs
    jobs = []
    objs_common = []
    for src in cu:
        o = OBJ / (src.stem + ".cu.o")
        objs_common.append(o)
        jobs.append([NVCC, *NVCC_FLAGS, *(["-DSHVK_DEV_PROBES=1"] if dev_probes else []), "-c", str(src), "-o", str(o)])
    api_objs = {}
    for src in cpp:
        if src.name == "api.cpp":
            for variant, extra in (("strict", []), ("experimental", ["-DSHV_CUDA_EXPERIMENTAL=1"])):
                o = OBJ / f"api.{variant}.o"
                api_objs[variant] = o
                jobs.append([CXX, *CXX_FLAGS, f'-DSHV_CUDA_REVISION="{rev}"', *extra, "-c", str(src), "-o", str(o)])
        else:
            o = OBJ / (src.stem + ".o")
            objs_common.append(o)
            jobs.append([CXX, *CXX_FLAGS, "-c", str(src), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    for lib, variant in zip(libs, ("strict", "experimental")):
        _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs_common),
              str(api_objs[variant]), "-Xlinker", "--no-undefined", "-lpthread"])
    stamp.write_text(rev)
    if verbose:
        print(f"built {libs[0].name} and {libs[1].name}, revision {rev}")
    return libs


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, dev_probes="--dev-probes" in sys.argv)
