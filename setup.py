"""Packaging. ``python setup.py build_ext --inplace`` (or ``python -m autodist_b200.ops.build``) compiles the sm_100a
extension in-tree; the protobuf messages need no ``protoc`` step (descriptors are built in Python)."""
import os

from setuptools import Command, find_packages, setup


def read_version():
    """The release number lives in the ``VERSION`` file at the repository root (one line, ``major.minor.patch``); a build of
    an untagged tree appends ``.dev0+<short commit>`` when ``AUTODIST_DEV_VERSION=1`` and git is available (the role of the
    reference's ``GENVER`` script)."""
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "VERSION")) as f:
        version = f.read().strip()
    if os.environ.get("AUTODIST_DEV_VERSION") == "1":
        try:
            import subprocess
            sha = subprocess.run(["git", "rev-parse", "--short", "HEAD"], cwd=here, capture_output=True, text=True, check=True).stdout.strip()
            version = f"{version}.dev0+{sha}"
        except (OSError, subprocess.CalledProcessError):
            pass
    return version


class BuildKernels(Command):
    description = "compile the sm_100a CUDA extension in-tree"
    user_options = [("inplace", "i", "kept for compatibility: the build is always in-tree")]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        from autodist_b200.ops import build
        print(build.build(verbose=True))


setup(
    name="autodist_b200",
    version=read_version(),
    description="Blackwell-native auto-distribution training engine for PyTorch",
    packages=find_packages(include=["autodist_b200", "autodist_b200.*"]),
    package_data={"autodist_b200": ["csrc/*", "_ext/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pyyaml", "protobuf>=4"],
    cmdclass={"build_ext": BuildKernels},
)
