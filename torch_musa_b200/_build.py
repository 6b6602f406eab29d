"""In-tree native build for torch_musa_b200 (sm_100a only).

Two shared objects are produced next to this file:

* ``libb200_kernels.so`` -- every hand-written CUDA kernel, compiled by nvcc with
  ``-gencode arch=compute_100a,code=sm_100a``.  The translation units include no
  torch header (plain C ABI: raw pointers, sizes, ``cudaStream_t``) so each one
  cross-compiles in seconds and can be driven from C, ctypes or the C++ layer.
* ``_C.so`` -- the C++ runtime (device/stream/event/guard, caching allocators,
  hooks, generator), the ATen op registrations for the PrivateUse1 dispatch key,
  the process-group backend and the CPython bindings.  Compiled by g++ against
  the installed torch headers and linked to ``libb200_kernels.so``.

The reference builds the same split with CMake (``libmusa_kernels.so`` +
``libmusa_python.so`` + ``_MUSAC``; reference CMakeLists.txt:223-225,
setup.py:173-190); here one small incremental driver (depfile + flag hash per
object, parallel jobs) replaces build.sh/CMake because nothing has to be
patched or code-generated.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG.parent / "build" / "obj"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
# The system compiler on purpose (not $CXX): the extension must share libstdc++ with the installed torch;
# a wrapper compiler that links libstdc++ statically yields a second, uninitialised copy of the iostream
# locale state inside _C.so.  Override with B200_CXX if you know the toolchains match.
CXX = os.environ.get("B200_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")

GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _torch_paths():
    import torch  # noqa: F401  (slow first import is expected)
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = ce.library_paths()
    return inc, lib


def _nccl_include():
    try:
        import nvidia.nccl  # type: ignore

        p = Path(nvidia.nccl.__path__[0]) / "include"
        if (p / "nccl.h").exists():
            return [str(p)]
    except Exception:
        pass
    return ["/usr/include"]


def _nccl_lib():
    try:
        import nvidia.nccl  # type: ignore

        p = Path(nvidia.nccl.__path__[0]) / "lib"
        if p.exists():
            return str(p)
    except Exception:
        pass
    return None


def _needs_rebuild(src: Path, obj: Path, sig: str) -> bool:
    stamp = obj.with_suffix(obj.suffix + ".sig")
    dep = obj.with_suffix(obj.suffix + ".d")
    if not obj.exists() or not stamp.exists() or stamp.read_text() != sig:
        return True
    t = obj.stat().st_mtime
    if src.stat().st_mtime > t:
        return True
    if dep.exists():
        txt = dep.read_text().replace("\\\n", " ")
        parts = txt.split(":", 1)
        if len(parts) == 2:
            for f in parts[1].split():
                # only headers of this repo can change between builds
                if f.startswith(str(PKG)):
                    try:
                        if os.stat(f).st_mtime > t:
                            return True
                    except OSError:
                        return True
    return False


def _run(cmd, what):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        err = [l for l in (r.stdout + "\n" + r.stderr).splitlines() if "error" in l or "Error" in l][:25]
        msg = f"[b200 build] FAILED {what}\n$ {' '.join(map(shlex.quote, cmd))}\n" + "\n".join(err) + "\n"
        if os.environ.get("B200_BUILD_FULL_LOG", "0") == "1":
            msg += r.stdout[-8000:] + "\n" + r.stderr[-16000:] + "\n"
        raise RuntimeError(msg)
    return r


def _compile_many(jobs, nproc):
    # jobs: list of (src, obj, cmd, sig)
    todo = [j for j in jobs if _needs_rebuild(j[0], j[1], j[3])]
    if not todo:
        return 0

    def one(j):
        src, obj, cmd, sig = j
        obj.parent.mkdir(parents=True, exist_ok=True)
        r = _run(cmd, str(src.relative_to(PKG)))
        obj.with_suffix(obj.suffix + ".sig").write_text(sig)
        return src, r

    failures = []
    with cf.ThreadPoolExecutor(max_workers=nproc) as ex:
        futs = [ex.submit(one, j) for j in todo]
        for f in futs:
            try:
                src, r = f.result()
            except RuntimeError as e:
                failures.append(str(e))
                continue
            if verbose_ptxas() and r.stderr.strip():
                sys.stderr.write(r.stderr)
            print(f"[b200 build] compiled {src.relative_to(PKG)}", flush=True)
    if failures:
        raise RuntimeError("native build failed:\n" + "\n".join(failures))
    return len(todo)


def verbose_ptxas() -> bool:
    return os.environ.get("B200_BUILD_PTXAS_V", "0") == "1"


def build(verbose: bool = True, jobs: int | None = None) -> dict:
    """Compile (incrementally) both shared objects.  Returns their paths."""
    nproc = jobs or int(os.environ.get("MAX_JOBS", os.cpu_count() or 4))
    tinc, tlib = _torch_paths()
    py_inc = sysconfig.get_paths()["include"]

    # ---------------------------------------------------------------- kernels
    cu_srcs = sorted((CSRC / "kernels").rglob("*.cu"))
    nvcc_flags = [
        "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "--expt-extended-lambda",
        "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
        "--threads", "2", "-I", str(CSRC), "-I", str(CSRC / "kernels"),
        "-DNDEBUG",
    ] + GENCODE
    if verbose_ptxas():
        nvcc_flags += ["-Xptxas", "-v"]
    kjobs = []
    for s in cu_srcs:
        o = OBJ / "kernels" / (s.relative_to(CSRC / "kernels").as_posix().replace("/", "__") + ".o")
        cmd = [NVCC, *nvcc_flags, "-MD", "-MF", str(o) + ".d", "-c", str(s), "-o", str(o)]
        sig = hashlib.sha1(" ".join(nvcc_flags).encode()).hexdigest()
        kjobs.append((s, o, cmd, sig))

    # -------------------------------------------------------------------- C++
    cpp_srcs = sorted(p for p in CSRC.rglob("*.cpp"))
    cxx_flags = [
        "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function",
        "-Wno-unknown-pragmas", "-Wno-sign-compare", "-Wno-unused-variable",
        "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
        "-DUSE_C10D_NCCL", "-DUSE_CUDA",
        "-I", str(CSRC), "-I", py_inc, "-I", str(CUDA_HOME / "include"),
    ]
    for i in tinc:
        cxx_flags += ["-isystem", i]
    for i in _nccl_include():
        cxx_flags += ["-isystem", i]
    # developer builds of the host runtime: B200_BUILD_ASAN=1 / B200_BUILD_TSAN=1 (the device code is unaffected; an
    # instrumented _C.so needs the sanitizer runtime preloaded into python: LD_PRELOAD=$(g++ -print-file-name=libasan.so))
    sanitize = []
    if os.environ.get("B200_BUILD_ASAN", "0") == "1":
        sanitize = ["-fsanitize=address", "-fno-omit-frame-pointer", "-g"]
    elif os.environ.get("B200_BUILD_TSAN", "0") == "1":
        sanitize = ["-fsanitize=thread", "-fno-omit-frame-pointer", "-g"]
    cxx_flags += sanitize
    cjobs = []
    for s in cpp_srcs:
        o = OBJ / "cpp" / (s.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        cmd = [CXX, *cxx_flags, "-MD", "-MF", str(o) + ".d", "-c", str(s), "-o", str(o)]
        sig = hashlib.sha1(" ".join(cxx_flags).encode()).hexdigest()
        cjobs.append((s, o, cmd, sig))

    n1 = _compile_many(kjobs + cjobs, nproc)

    # ------------------------------------------------------------------- link
    klib = PKG / "libb200_kernels.so"
    kobjs = [str(j[1]) for j in kjobs]
    if n1 or not klib.exists() or any(os.stat(o).st_mtime > klib.stat().st_mtime for o in kobjs):
        cmd = [NVCC, "-shared", "-o", str(klib), *kobjs, *GENCODE, "-cudart", "shared",
               "-Xlinker", "-soname,libb200_kernels.so", "-L", str(CUDA_HOME / "lib64"), "-lcudart"]
        _run(cmd, "link libb200_kernels.so")
        if verbose:
            print(f"[b200 build] linked {klib.name}", flush=True)

    clib = PKG / "_C.so"
    cobjs = [str(j[1]) for j in cjobs]
    if n1 or not clib.exists() or any(os.stat(o).st_mtime > clib.stat().st_mtime for o in cobjs) \
            or klib.stat().st_mtime > clib.stat().st_mtime:
        cmd = [CXX, "-shared", "-o", str(clib), *cobjs, *sanitize[:1], "-L", str(PKG), "-lb200_kernels",
               "-Wl,-rpath,$ORIGIN", "-Wl,--no-as-needed"]
        for l in tlib:
            cmd += ["-L", l, f"-Wl,-rpath,{l}"]
        nl = _nccl_lib()
        if nl:
            cmd += ["-L", nl, f"-Wl,-rpath,{nl}", "-l:libnccl.so.2"]
        else:
            cmd += ["-lnccl"]
        cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
                "-L", str(CUDA_HOME / "lib64"), "-lcudart", "-ldl", "-lpthread"]
        _run(cmd, "link _C.so")
        if verbose:
            print(f"[b200 build] linked {clib.name}", flush=True)
    return {"kernels": str(klib), "core": str(clib), "recompiled": n1}


if __name__ == "__main__":
    build()
