"""``python setup.py build_ext --inplace`` builds the CUDA extension next to the package, as the reference's
setup.py does for its own (setup.py:7-31), but for sm_100a.  The same sources are also built on first use
(ampere_kv_engine_b200/kernels/build.py); both give ampere_kv_engine_b200/_C.so."""

import os
import sys

from setuptools import Command, find_packages, setup

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class BuildExt(Command):
    description = "compile csrc/*.cu and bindings.cpp for sm_100a into ampere_kv_engine_b200/_C.so"
    user_options = [("inplace", "i", "build next to the package (always)"), ("force", "f", "rebuild")]

    def initialize_options(self):
        self.inplace = 1
        self.force = 0

    def finalize_options(self):
        pass

    def run(self):
        from ampere_kv_engine_b200.kernels import build
        print(build.build(verbose=True, force=bool(self.force)))


setup(
    name="ampere_kv_engine_b200",
    version="0.1.0",
    description="A small Qwen3 inference engine for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["ampere_kv_engine_b200", "ampere_kv_engine_b200.*"]),
    package_data={"ampere_kv_engine_b200": ["csrc/*", "_C.so"]},
    cmdclass={"build_ext": BuildExt},
    scripts=["bin/trace_run"],
)
