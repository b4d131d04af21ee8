"""Builds the native libraries of this package in-tree with nvcc / g++ for sm_100a.

    python -m tinyinfer_b200.build [--force]

Outputs (tinyinfer_b200/lib/):
    libtinyinfer_backend.so     operator ABI (ti_v2_*, ti_b200_*) + every CUDA kernel
    libtinyinfer_llm.so         model ABI (ti_llm_*) with its own copy of the kernels
    libtinyinfer_host_codec.so  host quantisation codec (ti_host_*), no CUDA
    tinyinfer_server            epoll batching server (built when its sources exist)
No GPU is needed to build (nvcc cross-compiles); the libraries refuse to run without one.
"""
from __future__ import annotations

import argparse
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
SRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG / "lib" / "obj"
INCLUDE = PKG.parent / "include"

NVCC = "nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", f"-I{INCLUDE}", f"-I{SRC}"]


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > stamp for s in sources)


def _run(cmd):
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + result.stdout + result.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")
    return result


def build(force: bool = False, verbose: bool = False) -> dict:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = list(SRC.glob("*.cuh")) + list(SRC.glob("*.hpp")) + list(INCLUDE.glob("*.h"))
    objects = {
        "kernels": (SRC / "kernels.cu", ARCH + ["-Xptxas", "-v"] if verbose else ARCH),
        "backend_api": (SRC / "backend_api.cpp", []),
        "attention_static_scratch": (SRC / "attention_static_scratch.cu", ARCH),
        "llm_runtime": (SRC / "llm_runtime.cpp", []),
    }
    jobs = []
    for name, (source, extra) in objects.items():
        obj = OBJ / f"{name}.o"
        if force or _stale(obj, [source] + headers):
            jobs.append([NVCC, *COMMON, *extra, "-c", str(source), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=4) as pool:
        for result in pool.map(_run, jobs):
            if verbose:
                sys.stderr.write(result.stderr)
    backend, llm, codec = LIB / "libtinyinfer_backend.so", LIB / "libtinyinfer_llm.so", LIB / "libtinyinfer_host_codec.so"
    shared_objects = [OBJ / "kernels.o", OBJ / "backend_api.o", OBJ / "attention_static_scratch.o"]
    if force or _stale(backend, shared_objects):
        _run([NVCC, "-shared", "-cudart", "shared", "-Xlinker", "-Bsymbolic", "-o", str(backend), *map(str, shared_objects)])
    # The model library carries its own copy of the kernels instead of depending on the backend
    # library by name: a process may also hold another library called libtinyinfer_backend.so
    # (the parity tests load the reference build), and a by-name dependency would bind to it.
    if force or _stale(llm, [OBJ / "llm_runtime.o", *shared_objects]):
        _run([NVCC, "-shared", "-cudart", "shared", "-Xlinker", "-Bsymbolic", "-o", str(llm), str(OBJ / "llm_runtime.o"),
              *map(str, shared_objects)])
    if force or _stale(codec, [SRC / "host_codec.cpp"] + list(INCLUDE.glob("*.h"))):
        _run(["g++", "-std=c++17", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fPIC", "-shared", "-Wall", "-Wextra",
              f"-I{INCLUDE}", "-o", str(codec), str(SRC / "host_codec.cpp")])
    built = {"backend": backend, "llm": llm, "host_codec": codec}
    server_src = SRC / "server" / "main.cpp"
    if server_src.exists():
        server = LIB / "tinyinfer_server"
        deps = list((SRC / "server").glob("*"))
        if force or _stale(server, deps + [llm]):
            _run(["g++", "-std=c++17", "-O2", "-pthread", "-Wall", f"-I{INCLUDE}", f"-I{SRC / 'server'}", "-o", str(server),
                  str(server_src), f"-L{LIB}", "-ltinyinfer_llm", "-Wl,-rpath,$ORIGIN"])
        built["server"] = server
    return built


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true", help="print ptxas register / spill report")
    args = parser.parse_args()
    for key, path in build(args.force, args.verbose).items():
        print(f"{key}: {path}")
