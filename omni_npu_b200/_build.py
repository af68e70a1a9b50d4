"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_C.so``       CUDA kernels for sm_100a (``csrc/**/*.cu``) + ``csrc/bindings.cpp``
                  registering ``torch.ops.omni_b200.*``.
* ``_runtime.so`` host-only C++ runtime pieces (``csrc/runtime``, ``csrc/alloc``):
                  KV block allocator, scheduler helpers, VMM sleep-mode allocator.

Kernels are compiled one translation unit per ``.cu`` file with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (no torch headers in device
code, so a file builds in seconds) and linked together with the bindings,
which are compiled by the host compiler against the torch headers.  Objects are
rebuilt only when their source (or a header) is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _cuda_home() -> str:
    return str(Path(_nvcc()).resolve().parent.parent)


def _newest_header_mtime() -> float:
    m = 0.0
    for ext in ("*.cuh", "*.h", "*.hpp"):
        for p in CSRC.rglob(ext):
            m = max(m, p.stat().st_mtime)
    return m


def _stale(src: Path, obj: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or hdr_mtime > t or Path(__file__).stat().st_mtime > t


def _run(cmd: list[str], log: Path | None = None) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def cuda_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cu"))


def runtime_sources() -> list[Path]:
    out: list[Path] = []
    for d in ("runtime", "alloc"):
        out += sorted((CSRC / d).glob("*.cpp"))
    return out


def build(force: bool = False, verbose: bool = False) -> dict:
    """Compile everything that is out of date.  Returns the paths of the libraries."""
    import torch  # noqa: F401  (import first: the headers' location comes from it)
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    nvcc = _nvcc()
    cuda_home = _cuda_home()
    jobs: list[tuple[list[str], Path | None]] = []
    objs: list[Path] = []

    for src in cuda_sources():
        obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hdr_mtime):
            jobs.append(([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                         obj.with_suffix(".log")))

    inc = []
    for p in ce.include_paths("cuda") if hasattr(ce, "include_paths") else []:
        inc += ["-I", p]
    inc += ["-I", os.path.join(cuda_home, "include")]
    import sysconfig
    inc += ["-I", sysconfig.get_paths()["include"]]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", 1))
    bind_src = CSRC / "bindings.cpp"
    bind_obj = OBJ / "bindings.cpp.o"
    if force or _stale(bind_src, bind_obj, hdr_mtime):
        jobs.append((["g++", *CXX_FLAGS, f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, "-c", str(bind_src),
                      "-o", str(bind_obj)], None))

    rt_objs: list[Path] = []
    for src in runtime_sources():
        obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        rt_objs.append(obj)
        if force or _stale(src, obj, hdr_mtime):
            jobs.append((["g++", *CXX_FLAGS, "-I", os.path.join(cuda_home, "include"), "-I", str(CSRC),
                          "-c", str(src), "-o", str(obj)], None))

    if jobs:
        if verbose:
            print(f"[omni_npu_b200] compiling {len(jobs)} translation units", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _run(j[0], j[1]), jobs))

    lib_c = PKG / "_C.so"
    lib_rt = PKG / "_runtime.so"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    if jobs or not lib_c.exists():
        _run(["g++", "-shared", "-o", str(lib_c), *map(str, objs), str(bind_obj),
              f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
              f"-L{cuda_home}/lib64", "-lcudart", f"-Wl,-rpath,{torch_lib}",
              f"-Wl,-rpath,{cuda_home}/lib64"])
    if rt_objs and (jobs or not lib_rt.exists()):
        _run(["g++", "-shared", "-o", str(lib_rt), *map(str, rt_objs), "-ldl", "-lpthread"])
    return {"_C": lib_c, "_runtime": lib_rt if rt_objs else None}


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose=True)
    print(out)
