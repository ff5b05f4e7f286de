"""Packaging of teramoe_b200.

The native extension is one target (sm_100a) built by ``teramoe_b200/_build.py`` into ``teramoe_b200/_ext/``; this file
only hooks that build into setuptools, so that

    python setup.py build_ext --inplace      # or: pip install --no-build-isolation -e .

leaves a ready-to-import tree.  ``import teramoe_b200`` also builds on first use when the extension is missing or
older than its sources, so the explicit step is optional on a machine with nvcc.

Reference counterpart: setup.py:1-140 (torch CUDAExtension with arch list 9.0;10.0, NVSHMEM discovery and build-time
macros); here there is one architecture, no NVSHMEM and one optional macro (TMOE_WITH_GATHER4).
"""
import importlib.util
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_build_module():
    # by path, so that the package (which imports torch-heavy modules) is not imported while setuptools runs
    spec = importlib.util.spec_from_file_location("_teramoe_b200_build", os.path.join(HERE, "teramoe_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


class BuildNative(Command):
    description = "compile the CUDA extension for sm_100a into teramoe_b200/_ext/"
    user_options = [("inplace", "i", "accepted for compatibility: the build is always in the source tree")]
    boolean_options = ["inplace"]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        so = _load_build_module().build(verbose=bool(os.environ.get("VERBOSE")))
        print(f"built {so}")


class BuildPyWithNative(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


setup(
    name="teramoe_b200",
    version="0.2.0",
    description="Expert-parallel MoE layer for B200 (sm_100a): fused dispatch / GEMM / combine kernels over NVLink",
    packages=find_packages(include=["teramoe_b200", "teramoe_b200.*", "teramoe", "teramoe.*"]),
    package_data={"teramoe_b200": ["csrc/*", "_ext/*.so", "_ext/*.hash"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
    zip_safe=False,
)
