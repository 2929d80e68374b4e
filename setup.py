"""Packaging: `pip install --no-build-isolation .` builds the native libraries in-tree with nvcc / g++
(`dlslime_b200/_build.py`) and installs the package with them. Environment switches follow the reference's
`slime_option` set (`BUILD_RDMA`, `BUILD_NVLINK`, `BUILD_PYTHON`, `BUILD_TORCH_PLUGIN`, `BUILD_ASCEND_DIRECT`,
`BUILD_BENCH`, `BUILD_TEST`; ON|OFF|TRUE|FALSE): e.g. `BUILD_NVLINK=OFF` installs the host runtime only,
`BUILD_RDMA=OFF` leaves the RDMA transport out, `BUILD_TORCH_PLUGIN=OFF` skips the c10d backend."""
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
        mod.build_all()
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
