"""Packaging. ``python setup.py build_ext --inplace`` (or ``python -m autodist_b200.ops.build``) compiles the sm_100a
extension in-tree; the protobuf messages need no ``protoc`` step (descriptors are built in Python)."""
from setuptools import Command, find_packages, setup


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
    version="0.1.0",
    description="Blackwell-native auto-distribution training engine for PyTorch",
    packages=find_packages(include=["autodist_b200", "autodist_b200.*"]),
    package_data={"autodist_b200": ["csrc/*", "_ext/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pyyaml", "protobuf>=4"],
    cmdclass={"build_ext": BuildKernels},
)
