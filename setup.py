"""Packaging: `pip install --no-build-isolation .` builds the native libraries in-tree with nvcc / g++
(`dlslime_b200/_build.py`) and installs the package with them. Environment switches follow the reference's
(`BUILD_NVLINK`, default ON: the CUDA kernel library; set it to OFF to install the host runtime only)."""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        import importlib.util

        spec = importlib.util.spec_from_file_location("_slime_build", os.path.join(HERE, "dlslime_b200", "_build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_host()
        mod.build_torch_plugin()
        if os.environ.get("BUILD_NVLINK", "ON").upper() not in ("OFF", "0", "FALSE"):
            mod.build_cuda()
        super().run()


setup(
    name="dlslime-b200",
    version="0.1.0",
    description="B200-native communication runtime with the capabilities of DLSlime",
    packages=find_packages(include=["dlslime_b200", "dlslime_b200.*"]),
    package_data={"dlslime_b200": ["*.so", "_C/*"]},
    include_package_data=True,
    python_requires=">=3.10",
    install_requires=["torch"],
    entry_points={"console_scripts": ["nanoctrl=dlslime_b200.nanoctrl.__main__:main", "dlslime-cache=dlslime_b200.cache.cli:main"]},
    cmdclass={"build_py": BuildNative},
    zip_safe=False,
)
