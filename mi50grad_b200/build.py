"""In-tree build of the native library (sm_100a only).

`python -m mi50grad_b200.build` compiles every file under csrc/ with nvcc and
links `mi50grad_b200/lib/libb200grad.so`.  The reference builds its kernels with
a Makefile plus mtime-checked JIT compilation at run time (reference:
Makefile:100-123, src/inference/engine.py:39-76); here there is one ahead-of-time
build, and the loader refuses to run on a GPU without it.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "libb200grad.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-diag-suppress", "177"]


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _stale(out: Path, deps) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    nvcc = nvcc_path()
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    jobs = []
    for src in sources():
        obj = OBJDIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *ARCH, *NVCC_FLAGS, "-I", str(CSRC)]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, r in ex.map(run, jobs):
                if verbose or ptxas_info or r.returncode:
                    sys.stderr.write(f"[build] {src.name}\n{r.stdout}{r.stderr}")
                if r.returncode:
                    raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr}")
    objs = [str(OBJDIR / (s.stem + ".o")) for s in sources()]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, *ARCH, "-shared", "-o", str(LIB), *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return LIB


if __name__ == "__main__":
    p = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(p)
