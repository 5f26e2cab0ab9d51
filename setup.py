"""``pip install .`` builds ``rtp_b200/lib/librtp_b200.so`` with nvcc for sm_100a (``rtp_b200/csrc/build.py``) and ships
it inside the package; the CUDA sources travel too, so an installed package can rebuild itself.  Counterpart of the
reference's setup.py (which has no extension to build)."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    spec = importlib.util.spec_from_file_location("_rtp_b200_build", os.path.join(HERE, "rtp_b200", "csrc", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("RTP_B200_SKIP_NVCC") != "1":
            _load_builder().build()      # in-tree: package_data picks the library up from rtp_b200/lib
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
