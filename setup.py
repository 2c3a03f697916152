"""Packaging: ``pip install --no-build-isolation -e .`` (or ``python setup.py build_ext --inplace``)
compiles ``torchcomms_b200/_comms.so`` in-tree for sm_100a with the package's own build driver
(``torchcomms_b200/_build.py``: nvcc + the PyTorch C++ extension toolchain, no GPU needed) and ships
it as package data.  Metadata lives in ``pyproject.toml``."""
import importlib.util
import os

from setuptools import Command, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_extension(force: bool = False) -> str:
    # Load the build driver by path: importing the package would need the extension it builds.
    spec = importlib.util.spec_from_file_location("_b200c_build", os.path.join(ROOT, "torchcomms_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return str(mod.build(verbose=bool(os.environ.get("B200COMMS_VERBOSE_BUILD")), force=force))


class BuildExt(Command):
    description = "compile torchcomms_b200/_comms.so in-tree (sm_100a)"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree"), ("force", "f", "rebuild even if up to date")]
    boolean_options = ["inplace", "force"]

    def initialize_options(self):
        self.inplace = True
        self.force = False

    def finalize_options(self):
        pass

    def run(self):
        print("built", _build_extension(force=bool(self.force)))


class BuildPy(build_py):
    def run(self):
        if not os.environ.get("B200COMMS_SKIP_EXT_BUILD"):
            _build_extension()
        super().run()


setup(cmdclass={"build_ext": BuildExt, "build_py": BuildPy})
