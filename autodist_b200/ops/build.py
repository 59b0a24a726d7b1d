"""In-tree build of the sm_100a extension.

``build()`` compiles every ``.cu`` / ``.cpp`` under ``autodist_b200/csrc`` for
``compute_100a / sm_100a`` with ninja and leaves ``_adb200_C.so`` under
``autodist_b200/_ext`` so that the shared object travels with the source tree.
"""
import glob
import hashlib
import os

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
EXT_DIR = os.path.join(os.path.dirname(HERE), "_ext")
NAME = "_adb200_C"

CUDA_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
              "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def source_digest():
    h = hashlib.sha1()
    for path in sources() + sorted(glob.glob(os.path.join(CSRC, "*.h"))):
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def so_path():
    return os.path.join(EXT_DIR, NAME + ".so")


def is_current():
    stamp = os.path.join(EXT_DIR, "digest.txt")
    return os.path.exists(so_path()) and os.path.exists(stamp) and open(stamp).read().strip() == source_digest()


def build(verbose=False):
    from torch.utils import cpp_extension
    os.makedirs(EXT_DIR, exist_ok=True)
    if is_current():
        return so_path()
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "8")
    cpp_extension.load(name=NAME, sources=sources(), extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=CUDA_FLAGS, extra_include_paths=[CSRC], build_directory=EXT_DIR,
                       verbose=verbose, is_python_module=False)
    with open(os.path.join(EXT_DIR, "digest.txt"), "w") as f:
        f.write(source_digest())
    return so_path()


if __name__ == "__main__":
    print(build(verbose=True))
