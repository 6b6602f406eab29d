"""Packaging for torch_musa_b200: ``pip install .`` compiles the two in-tree shared objects for sm_100a with the
package's own build driver and registers the backend with PyTorch's autoload entry point, so ``import torch`` makes
``torch.blackwell`` and the ``blackwell`` device available without an explicit import.
(The reference registers itself the same way: reference setup.py:237-241.)"""
import importlib.util
import os

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _native_build():
    spec = importlib.util.spec_from_file_location("_b200_build", os.path.join(ROOT, "torch_musa_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(verbose=True)


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("B200_SKIP_NATIVE_BUILD", "0") != "1":
            _native_build()
        super().run()


setup(
    name="torch_musa_b200",
    version="0.2.0",
    description="Blackwell-native (sm_100a) out-of-tree PyTorch device backend: device `blackwell`, collective backend `bccl`",
    packages=find_packages(include=["torch_musa_b200", "torch_musa_b200.*"]),
    package_data={"torch_musa_b200": ["*.so", "csrc/kernels/*.h", "csrc/compile/AotShim.h"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6"],
    cmdclass={"build_py": BuildWithKernels},
    entry_points={"torch.backends": ["torch_musa_b200 = torch_musa_b200:_autoload"]},
    zip_safe=False,
)
