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
    for path in sources() + sorted(glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))):
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


HOST_NAME = "_adb200_host"


def host_so_path():
    return os.path.join(EXT_DIR, HOST_NAME + ".so")


def build_host(verbose=False):
    """Host-only extension (no device code) under ``csrc/host``: the C++ model of the synchronisation protocol and the
    background batch feeder."""
    from torch.utils import cpp_extension
    os.makedirs(EXT_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    h = hashlib.sha1()
    for path in srcs:
        with open(path, "rb") as f:
            h.update(f.read())
    stamp = os.path.join(EXT_DIR, "host_digest.txt")
    if os.path.exists(host_so_path()) and os.path.exists(stamp) and open(stamp).read().strip() == h.hexdigest():
        return host_so_path()
    build_dir = os.path.join(EXT_DIR, "host")
    os.makedirs(build_dir, exist_ok=True)
    cpp_extension.load(name=HOST_NAME, sources=srcs, extra_cflags=["-O2", "-std=c++17", "-pthread"], extra_ldflags=["-pthread"],
                       build_directory=build_dir, verbose=verbose, is_python_module=False)
    import shutil
    shutil.copyfile(os.path.join(build_dir, HOST_NAME + ".so"), host_so_path())
    with open(stamp, "w") as f:
        f.write(h.hexdigest())
    return host_so_path()


def load_host():
    """Import the host-only extension, building it first if needed."""
    import importlib.util
    import sys
    if HOST_NAME in sys.modules:
        return sys.modules[HOST_NAME]
    path = build_host()
    spec = importlib.util.spec_from_file_location(HOST_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[HOST_NAME] = mod
    return mod


if __name__ == "__main__":
    print(build(verbose=True))
    print(build_host(verbose=True))
