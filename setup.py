"""`pip install -e .` builds the sm_100a extension in-tree (nvcc required, no GPU needed) and installs the package."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithExtension(build_py):
    def run(self):
        import os
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from odc_b200 import build as native
        native.build()
        super().run()


setup(cmdclass={"build_py": BuildWithExtension})
