"""Building user extensions against the blackwell backend: thin wrappers over ``torch.utils.cpp_extension`` that
add the sm_100a code generation flags (bypassing torch's own arch list), this package's kernel header directory
and its kernel library, so a user ``.cu`` file can call the C API of ``libb200_kernels.so`` or define new ops
for the PrivateUse1 dispatch key.

    from torch_musa_b200.utils.extension import B200Extension, BuildExtension, load, load_inline

Parity: reference torch_musa/utils/musa_extension.py:368 (MUSAExtension), :489 (BuildExtension), :1066 (load),
:1346 (load_inline).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def include_paths() -> List[str]:
    return [os.path.join(_PKG, "csrc"), os.path.join(_PKG, "csrc", "kernels")]


def library_paths() -> List[str]:
    return [_PKG]


def _nvcc_flags(extra: Optional[Sequence[str]]) -> List[str]:
    flags = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", *ARCH_FLAGS]
    return flags + [f for f in (extra or []) if f not in flags]


def B200Extension(name: str, sources: Sequence[str], *, extra_compile_args=None, include_dirs=None, library_dirs=None,
                  libraries=None, link_kernel_library: bool = True, **kw):
    """A ``setuptools`` extension (for ``setup.py``) compiled for sm_100a against this backend."""
    from torch.utils.cpp_extension import CUDAExtension

    eca = dict(extra_compile_args or {}) if isinstance(extra_compile_args, dict) else {"cxx": list(extra_compile_args or [])}
    eca["nvcc"] = _nvcc_flags(eca.get("nvcc"))
    eca.setdefault("cxx", [])
    libs = list(libraries or [])
    ldirs = list(library_dirs or [])
    if link_kernel_library:
        libs.append("b200_kernels")
        ldirs += library_paths()
        kw.setdefault("runtime_library_dirs", []).extend(library_paths())
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return CUDAExtension(name, list(sources), extra_compile_args=eca, include_dirs=list(include_dirs or []) + include_paths(),
                         library_dirs=ldirs, libraries=libs, **kw)


def BuildExtension(*args, **kw):
    from torch.utils.cpp_extension import BuildExtension as _BE

    return _BE(*args, **kw)


BuildExtension.with_options = lambda **options: __import__("torch.utils.cpp_extension", fromlist=["BuildExtension"]).BuildExtension.with_options(**options)


def load(name: str, sources: Sequence[str], *, extra_cflags=None, extra_cuda_cflags=None, extra_ldflags=None,
         extra_include_paths=None, build_directory: Optional[str] = None, verbose: bool = False,
         link_kernel_library: bool = True, **kw):
    """JIT-compile and import an extension (``build_directory`` defaults to torch's extension cache)."""
    from torch.utils.cpp_extension import load as _load

    ld = list(extra_ldflags or [])
    if link_kernel_library:
        ld += [f"-L{p}" for p in library_paths()] + ["-lb200_kernels"] + [f"-Wl,-rpath,{p}" for p in library_paths()]
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return _load(name, list(sources), extra_cflags=list(extra_cflags or []),
                 extra_cuda_cflags=_nvcc_flags(extra_cuda_cflags), extra_ldflags=ld,
                 extra_include_paths=list(extra_include_paths or []) + include_paths(),
                 build_directory=build_directory, verbose=verbose, **kw)


def load_inline(name: str, cpp_sources, cuda_sources=None, functions=None, *, extra_cuda_cflags=None, extra_ldflags=None,
                extra_include_paths=None, verbose: bool = False, link_kernel_library: bool = True, **kw):
    from torch.utils.cpp_extension import load_inline as _li

    ld = list(extra_ldflags or [])
    if link_kernel_library:
        ld += [f"-L{p}" for p in library_paths()] + ["-lb200_kernels"] + [f"-Wl,-rpath,{p}" for p in library_paths()]
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return _li(name, cpp_sources, cuda_sources=cuda_sources, functions=functions,
               extra_cuda_cflags=_nvcc_flags(extra_cuda_cflags), extra_ldflags=ld,
               extra_include_paths=list(extra_include_paths or []) + include_paths(), verbose=verbose, **kw)
