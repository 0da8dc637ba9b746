"""Builds the native parts in-tree (g++ / nvcc for sm_100a) before packaging; `pip install -e .` works."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        import importlib.util
        import os

        spec = importlib.util.spec_from_file_location("_fastb_build", os.path.join(os.path.dirname(os.path.abspath(__file__)), "fast_b200", "_build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative})
