"""Packaging for msamp (B200).  ``pip install -e .`` builds the sm_100a kernel library in-tree with nvcc.

Extra commands: ``python setup.py build_kernels`` (force a rebuild), ``python setup.py lint``, ``python setup.py test``.
"""
import os
import subprocess
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _build_kernels(force=False):
    sys.path.insert(0, ROOT)
    from msamp.ops.build import build
    return build(force=force)


class BuildKernels(Command):
    description = 'compile msamp/ops/csrc/*.cu into msamp/ops/libmsamp_b200.so'
    user_options = [('force', 'f', 'rebuild everything')]

    def initialize_options(self):
        self.force = False

    def finalize_options(self):
        pass

    def run(self):
        print(_build_kernels(bool(self.force)))


class BuildPyWithKernels(build_py):
    def run(self):
        try:
            _build_kernels()
        except Exception as e:    # nvcc missing: the package still works on CPU
            print(f'warning: kernel library not built ({e})')
        super().run()


class Lint(Command):
    description = 'flake8 over the package and the tests'
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        sys.exit(subprocess.call([sys.executable, '-m', 'flake8', '--max-line-length', '140', 'msamp', 'tests', 'bench.py']))


class Test(Command):
    description = 'run the CPU test-suite (use `pytest -m gpu` on a B200 for the rest)'
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        sys.exit(subprocess.call([sys.executable, '-m', 'pytest', '-q', '-m', 'not gpu', 'tests']))


setup(
    name='msamp-b200',
    version='0.4.0',
    description='FP8 mixed-precision training for NVIDIA B200: MS-AMP-compatible API on hand-written sm_100a kernels',
    packages=find_packages(include=['msamp', 'msamp.*']),
    package_data={'msamp.ops': ['libmsamp_b200.so', 'csrc/*']},
    python_requires='>=3.10',
    install_requires=['torch>=2.4', 'numpy'],
    cmdclass={'build_kernels': BuildKernels, 'build_py': BuildPyWithKernels, 'lint': Lint, 'test': Test},
)
