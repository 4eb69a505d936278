"""Installs the package and, with ``python setup.py build_native``, compiles its two native libraries ahead of
their first use (``nvcc -gencode arch=compute_100a,code=sm_100a`` for the kernels, ``g++`` for the host
library).  Nothing else is compiled at install time: the sources ship with the package and
``yalis_b200.native`` builds them beside itself at the first call that needs them."""

from setuptools import Command, setup


class build_native(Command):
    description = "compile libyalis_host and libyalis_cuda (sm_100a) into yalis_b200/_build"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        from yalis_b200 import native
        print(native.build("host"))
        print(native.build("cuda"))


setup(cmdclass={"build_native": build_native})
