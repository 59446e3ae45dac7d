"""In-tree build of the native extension ``hipress_b200/_C*.so`` for sm_100a.

``python -m hipress_b200.build`` (or ``build()``) compiles

* every ``csrc/kernels/*.cu`` with ``nvcc -gencode arch=compute_100a,code=sm_100a``
  (the kernels include no torch header, so each file takes seconds),
* every ``csrc/**/*.cpp`` with ``g++`` against the torch headers,

and links them into one shared object placed inside the package, plus
``libhipress_kernels.so``: the same kernels and CPU codecs behind a C ABI with
no torch or Python dependency.  Objects are cached under ``build/`` and rebuilt
when a source or any header is newer.  The reference builds one extension with
``CUDAExtension(..., nvcc: ['-O3'])`` and no architecture flag
(ref setup.py:5-18); there is no install step here: the built object is
imported from the source tree.

``python -m hipress_b200.build --sanitize thread|address`` builds the host runtime's stress
test under ThreadSanitizer or AddressSanitizer instead (see ``build_sanitized``).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
PKG = ROOT / "hipress_b200"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
# -ffp-contract=off: the CPU codecs must round exactly like baseline x86-64
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-Wall", "-Wno-unused-function",
             "-fvisibility=hidden"]


def _ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def _newest_header() -> float:
    newest = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for p in CSRC.rglob(pat):
            newest = max(newest, p.stat().st_mtime)
    return newest


_TORCH_MARKERS = ("#include <torch/", "#include <ATen/", "#include <c10/", "#include <pybind11/")


def _needs_torch(src: Path, _seen: set | None = None) -> bool:
    """True if the file, or a project header it includes, pulls in torch headers."""
    seen = _seen if _seen is not None else set()
    if src in seen or not src.exists():
        return False
    seen.add(src)
    text = src.read_text()
    if any(m in text for m in _TORCH_MARKERS):
        return True
    for line in text.splitlines():
        line = line.strip()
        if line.startswith('#include "'):
            inc = line.split('"')[1]
            for base in (src.parent, CSRC):
                if _needs_torch((base / inc).resolve(), seen):
                    return True
    return False


def _run(cmd: list[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(shlex.quote(c) for c in cmd)
                           + "\n" + proc.stdout + proc.stderr)


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames \
        else ce.include_paths(cuda=True)
    lib = ce.library_paths(device_type="cuda") if "device_type" in ce.library_paths.__code__.co_varnames \
        else ce.library_paths(cuda=True)
    return torch, inc, lib


def build(verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile what is out of date and return the path of the Python extension."""
    OBJ.mkdir(parents=True, exist_ok=True)
    torch, inc, lib = _torch_paths()
    hdr_time = _newest_header()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = str(Path(cuda_home) / "bin" / "nvcc")
    py_inc = sysconfig.get_paths()["include"]

    cu_srcs = sorted((CSRC / "kernels").glob("*.cu"))
    # sources that need torch / pybind11 vs. those that are plain C++
    torch_srcs = sorted(p for p in CSRC.rglob("*.cpp") if _needs_torch(p))
    plain_srcs = sorted(p for p in CSRC.rglob("*.cpp") if p not in torch_srcs)

    tasks = []

    def obj_of(src: Path) -> Path:
        return OBJ / (str(src.relative_to(CSRC)).replace("/", "__") + ".o")

    def stale(src: Path, obj: Path) -> bool:
        return (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)

    for src in cu_srcs:
        obj = obj_of(src)
        if stale(src, obj):
            tasks.append(([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                          obj.with_suffix(".log")))
    for src in plain_srcs:
        obj = obj_of(src)
        if stale(src, obj):
            tasks.append((["g++", *CXX_FLAGS, "-I", str(CSRC), "-I", f"{cuda_home}/include",
                           "-c", str(src), "-o", str(obj)], None))
    for src in torch_srcs:
        obj = obj_of(src)
        if stale(src, obj):
            cmd = ["g++", *CXX_FLAGS, "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                   "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
                   "-I", str(CSRC), "-I", py_inc, "-I", f"{cuda_home}/include"]
            for i in inc:
                cmd += ["-isystem", i]
            cmd += ["-c", str(src), "-o", str(obj)]
            tasks.append((cmd, None))

    if tasks:
        if verbose:
            print(f"[hipress_b200.build] compiling {len(tasks)} translation units", file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
            for fut in [ex.submit(_run, cmd, log) for cmd, log in tasks]:
                fut.result()

    cu_objs = [str(obj_of(s)) for s in cu_srcs]
    plain_objs = [str(obj_of(s)) for s in plain_srcs]
    torch_objs = [str(obj_of(s)) for s in torch_srcs]

    ext = PKG / ("_C" + _ext_suffix())
    all_objs = cu_objs + plain_objs + torch_objs
    newest_obj = max(Path(o).stat().st_mtime for o in all_objs)
    if not ext.exists() or ext.stat().st_mtime < newest_obj:
        # link under a temporary name and rename: a reader (an import in another process, a copy
        # of the tree) never sees a half-written library
        tmp = ext.with_name(ext.name + ".tmp")
        cmd = ["g++", "-shared", "-o", str(tmp), *all_objs]
        for l in lib:
            cmd += ["-L", l, f"-Wl,-rpath,{l}"]
        cmd += ["-L", f"{cuda_home}/lib64", f"-Wl,-rpath,{cuda_home}/lib64",
                "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                "-lcublasLt", "-lcudart", "-ldl", "-lpthread"]
        _run(cmd)
        os.replace(tmp, ext)

    # torch-free C ABI library (kernels + CPU codecs + c_api)
    clib = PKG / "libhipress_kernels.so"
    c_objs = cu_objs + plain_objs
    if c_objs and (not clib.exists() or clib.stat().st_mtime < max(Path(o).stat().st_mtime for o in c_objs)):
        tmp = clib.with_name(clib.name + ".tmp")
        _run(["g++", "-shared", "-o", str(tmp), *c_objs, "-L", f"{cuda_home}/lib64",
              f"-Wl,-rpath,{cuda_home}/lib64", "-lcudart", "-ldl", "-lpthread"])
        os.replace(tmp, clib)
    return ext


SANITIZERS = {"thread": ["-fsanitize=thread"], "address": ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"]}


def build_sanitized(kind: str, target: str = "runtime") -> Path:
    """Build the host runtime's stress test (tests/cpp/runtime_stress.cpp: WorkerPool,
    FinishQueue, AgeWatchdog -- the plain-C++ parts, which need neither torch nor a GPU) with
    ThreadSanitizer (``thread``) or AddressSanitizer + UBSan (``address``) and return the
    executable.  Run it directly; a sanitizer report makes it exit non-zero.  The reference
    has no such check and carries unsynchronised shared state in exactly these parts
    (ref hp_cuda.cpp:789, 930)."""
    if kind not in SANITIZERS:
        raise ValueError(f"sanitizer must be one of {sorted(SANITIZERS)}")
    out_dir = ROOT / "build" / "sanitize"
    out_dir.mkdir(parents=True, exist_ok=True)
    if target == "codec":
        # ``target="codec"``: the threaded CPU codecs (tests/cpp/codec_threads.cpp + codec_cpu.cpp)
        exe = out_dir / f"codec_threads_{kind}"
        srcs = [ROOT / "tests" / "cpp" / "codec_threads.cpp", CSRC / "codec_cpu" / "codec_cpu.cpp"]
        deps = srcs + list((CSRC / "common").glob("*.h")) + [CSRC / "codec_cpu" / "codec_cpu.h"]
        extra = ["-ffp-contract=off"]
    elif target == "runtime":
        exe = out_dir / f"runtime_stress_{kind}"
        srcs = [ROOT / "tests" / "cpp" / "runtime_stress.cpp"]
        deps = srcs + list((CSRC / "runtime").glob("*.h"))
        extra = []
    else:
        raise ValueError("target must be 'runtime' or 'codec'")
    newest = max(p.stat().st_mtime for p in deps)
    if not exe.exists() or exe.stat().st_mtime < newest:
        _run(["g++", "-std=c++17", "-O1", "-g", *extra, *SANITIZERS[kind], "-I", str(CSRC), *map(str, srcs),
              "-o", str(exe), "-lpthread"])
    return exe


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the cached nvcc logs."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        out.append(f"== {log.name}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    if len(sys.argv) >= 3 and sys.argv[1] == "--sanitize":
        print(build_sanitized(sys.argv[2], *(sys.argv[3:4])))   # optional third word: runtime | codec
    else:
        print(build(verbose=True))
