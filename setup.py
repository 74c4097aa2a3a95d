"""Build entry, in the place of the reference's RoDe_SDDMM/setup.py (a CUDAExtension named
`rode_sddmm_cuda` built from its binding and its kernels).

    python setup.py build_ext --inplace      # what the reference's README tells users to run
    pip install -e . --no-build-isolation    # optional: makes `rode_b200` importable anywhere

Both run the in-tree recipe of rode_b200/build.py: nvcc compiles the kernels for sm_100a into
rode_b200/librode_b200.so (the C ABI), then the torch binding rode_b200/rode_sddmm_cuda*.so is
compiled against it.  The binaries stay inside the source tree.
"""
import os
import sys

from setuptools import Command, find_packages, setup

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class BuildExt(Command):
    description = "build librode_b200.so (nvcc, sm_100a) and the torch binding, in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree"),
                    ("force", "f", "rebuild even if up to date")]

    def initialize_options(self):
        self.inplace = 1
        self.force = 0

    def finalize_options(self):
        pass

    def run(self):
        from rode_b200 import build

        print("built", build.build_library(force=bool(self.force)))
        print("built", build.build_torch_extension(force=bool(self.force)))


setup(
    name="rode_b200",
    version="0.1.0",
    description="RoDe row-decomposition SpMM / SDDMM hot path for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["rode_b200", "rode_b200.*"]),
    package_data={"rode_b200": ["*.so", "csrc/*", "torch_ext/*"]},
    cmdclass={"build_ext": BuildExt},
    python_requires=">=3.9",
)
