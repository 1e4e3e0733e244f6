"""``pip install .`` builds the native parts first (CUDA kernels for sm_100a with nvcc, the C++ planner with
pybind11: ``distca_b200/build.py``) so that the wheel carries ``_kernels.so`` and ``_planner*.so`` next to the
Python sources. The reference ships a pure-Python package and builds its kernels with CMake by hand
(setup.py:3, csrc/CMakeLists.txt)."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNativeThenPy(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_distca_b200_build", os.path.join(HERE, "distca_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if os.environ.get("DISTCA_SKIP_NATIVE_BUILD", "0") != "1":
            mod.build_all(force=False)
        super().run()


setup(cmdclass={"build_py": BuildNativeThenPy})
