"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_native/libvolta_kernels.so``  – every sm_100a CUDA kernel plus its ``extern "C"`` launcher
  (compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``; cross-compiles without a GPU).
* ``_native/libvolta_host.so``     – host-only C++17 runtime pieces (tokenizer, Jinja subset, output
  parser, HTTP front end, GGUF block codecs, CPU oracle).

The Python side binds both with ``ctypes`` (raw device pointers + the current CUDA stream), so no
torch headers are compiled and a full rebuild takes seconds per translation unit.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_native"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr", "-diag-suppress", "177,550",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {cmd[0]} (exit {r.returncode})")
    if os.environ.get("VOLTA_BUILD_VERBOSE"):
        sys.stderr.write(r.stdout + r.stderr)


def _build_lib(name: str, srcs: list[Path], headers: list[Path], compiler: list[str],
               flags: list[str], link: list[str], force: bool) -> Path:
    OUT.mkdir(exist_ok=True)
    lib = OUT / f"lib{name}.so"
    stamp = OUT / f"{name}.stamp"
    objdir = OUT / f"obj_{name}"
    objdir.mkdir(exist_ok=True)
    jobs = []
    for s in srcs:
        dig = _digest([s] + headers, " ".join(flags))
        obj = objdir / (s.stem + ".o")
        tag = objdir / (s.stem + ".sha")
        if force or not obj.exists() or not tag.exists() or tag.read_text() != dig:
            jobs.append((s, obj, tag, dig))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_run, compiler + flags + ["-I", str(CSRC), "-c", str(s), "-o", str(o)])
                    for s, o, _, _ in jobs]
            for f in futs:
                f.result()
        for _, _, tag, dig in jobs:
            tag.write_text(dig)
    objs = [str(objdir / (s.stem + ".o")) for s in srcs]
    whole = _digest([Path(o) for o in objs], name)
    if jobs or not lib.exists() or not stamp.exists() or stamp.read_text() != whole:
        _run(compiler + ["-shared", "-o", str(lib)] + objs + link)
        stamp.write_text(whole)
    return lib


def build_kernels(force: bool = False) -> Path:
    nvcc = _nvcc()
    lib = OUT / "libvolta_kernels.so"
    if nvcc is None:
        if lib.exists():
            return lib
        raise RuntimeError("nvcc not found and libvolta_kernels.so is not built")
    srcs = sorted((CSRC / "cuda").glob("*.cu"))
    headers = sorted((CSRC / "cuda").glob("*.cuh")) + sorted((CSRC / "cuda").glob("*.h"))
    return _build_lib("volta_kernels", srcs, headers, [nvcc], NVCC_FLAGS,
                      ["-Xcompiler", "-fPIC", "-lcudart"], force)


def build_host(force: bool = False) -> Path:
    cxx = shutil.which("g++")
    lib = OUT / "libvolta_host.so"
    if cxx is None:
        if lib.exists():
            return lib
        raise RuntimeError("g++ not found and libvolta_host.so is not built")
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    headers = sorted((CSRC / "host").glob("*.h")) + sorted((CSRC / "host").glob("*.inc"))
    if not srcs:
        return lib
    return _build_lib("volta_host", srcs, headers, [cxx], CXX_FLAGS, ["-pthread", "-ldl"], force)


def build_all(force: bool = False) -> dict[str, Path]:
    return {"kernels": build_kernels(force), "host": build_host(force)}


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv)
    for k, v in libs.items():
        print(k, v)
