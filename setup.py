"""``pip install --no-build-isolation [-e] .`` compiles the native parts in the source tree (nvcc for sm_100a through
``rocshmem_b200/_build.py``, the same step as ``python -m rocshmem_b200._build``) and then installs the package.
An editable install copies nothing, so the built ``.so`` files stay next to their sources; a regular install
packages them (the bindings find the runtime library through ``$ORIGIN/lib``)."""
import importlib.util
import os

from setuptools import Distribution, setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

HERE = os.path.dirname(os.path.abspath(__file__))


def _native_build():
    # Load the build module by path: importing the package would try to load the not yet built extension.
    spec = importlib.util.spec_from_file_location("_rocshmem_b200_build", os.path.join(HERE, "rocshmem_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build(with_tests=False)


class BuildPy(build_py):
    def run(self):
        _native_build()
        super().run()


class Develop(develop):
    def run(self):
        _native_build()
        super().run()


class BinaryDistribution(Distribution):
    """The package carries compiled libraries: wheels get a platform tag instead of "any"."""

    def has_ext_modules(self):
        return True


setup(cmdclass={"build_py": BuildPy, "develop": Develop}, distclass=BinaryDistribution)
