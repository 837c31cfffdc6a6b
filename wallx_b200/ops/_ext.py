"""Loader and builder of the in-tree sm_100a extension.

The extension is built in-tree (``wallx_b200/_build/_wallx_C.so``) so that the binary travels
with the source tree. On a machine with a GPU the ops refuse to run without it: there is no
silent PyTorch fallback for CUDA tensors.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)
CSRC = os.path.join(_PKG, "csrc")
BUILD_DIR = os.path.join(_PKG, "_build")
EXT_NAME = "_wallx_C"

SOURCES = [
    "bindings.cpp",
    "kernel_bindings.cpp",
    "blocks.cpp",
    "gemm.cu",
    "kernels.cu",
    "attention.cu",
    "comm.cu",
    "index.cu",
    "decode.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]

# Debug variant: the same sources with -DWX_CHECK (range checks in the kernels, csrc/check.cuh), built into its own
# directory and loaded instead of the release build when WALLX_CHECKED=1.
CHECKED = os.environ.get("WALLX_CHECKED", "0") == "1"
CHECKED_NAME = "_wallx_C_checked"
CHECKED_DIR = os.path.join(_PKG, "_build_checked")

_lock = threading.Lock()
_mod = None
_tried = False


def so_path(checked: bool = None) -> str:
    checked = CHECKED if checked is None else checked
    return os.path.join(CHECKED_DIR, CHECKED_NAME + ".so") if checked else os.path.join(BUILD_DIR, EXT_NAME + ".so")


def build(verbose: bool = False, checked: bool = False):
    """Compile every CUDA source for sm_100a (cross-compiles without a GPU) and load the result.
    ``checked`` builds the debug variant with the kernels' range checks compiled in."""
    global _mod, _tried
    from torch.utils import cpp_extension

    out_dir = CHECKED_DIR if checked else BUILD_DIR
    os.makedirs(out_dir, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    mod = cpp_extension.load(
        name=CHECKED_NAME if checked else EXT_NAME,
        sources=srcs,
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS + (["-DWX_CHECK"] if checked else []),
        extra_include_paths=[CSRC],
        build_directory=out_dir,
        verbose=verbose,
        with_cuda=True,
    )
    if checked == CHECKED:
        with _lock:
            _mod = mod
            _tried = True
    return mod


def _load_prebuilt():
    path = so_path()
    if not os.path.exists(path):
        # a `setup.py build_ext --inplace` build carries the interpreter tag in its file name
        import glob

        tagged = sorted(glob.glob(os.path.join(BUILD_DIR, EXT_NAME + ".*.so")))
        if not tagged:
            return None
        path = tagged[-1]
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    name = CHECKED_NAME if CHECKED else EXT_NAME
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


def get(required: bool = True):
    """Return the extension module; raise if it is missing and ``required``."""
    global _mod, _tried
    if _mod is None and not _tried:
        with _lock:
            if _mod is None and not _tried:
                _tried = True
                try:
                    _mod = _load_prebuilt()
                except Exception as e:  # pragma: no cover - depends on the box
                    if required:
                        raise RuntimeError(f"wallx_b200: cannot load {so_path()}: {e}") from e
                    _mod = None
    if _mod is None and required:
        raise RuntimeError(
            "wallx_b200: the sm_100a extension is not built "
            f"({so_path()} missing). Run `python -c 'import __graft_entry__ as g; g.build()'`."
        )
    return _mod


def available() -> bool:
    return get(required=False) is not None


class LaunchCounter:
    """Counts kernel launches issued through the extension (each binding knows how many kernels it
    launches). Used by the benchmark to report how many of our kernels ran in the timed region."""

    PER_CALL = {"rms_norm_bwd": 2, "column_sum": 2}  # gemm_ag: one kernel (copy CTAs are part of its grid)

    def __init__(self, mod):
        self._mod = mod
        self.total = 0
        self.by_name = {}

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        if not callable(fn):
            return fn
        base = self.PER_CALL.get(name, 1)

        def wrapped(*a, **k):
            n = base
            if name == "attn_bwd":
                n = 3 if a[11] == a[12] else 5
            if name in ("read_status", "status_tensor", "block_launch_count"):
                n = 0
            if name in ("block_fwd", "block_bwd"):  # one host call, many kernels: the C++ side counts them
                before = self._mod.block_launch_count()
                out = fn(*a, **k)
                n = self._mod.block_launch_count() - before
                self.total += n
                self.by_name[name] = self.by_name.get(name, 0) + n
                return out
            self.total += n
            self.by_name[name] = self.by_name.get(name, 0) + n
            return fn(*a, **k)

        self.__dict__[name] = wrapped
        return wrapped

    @staticmethod
    def install() -> "LaunchCounter":
        global _mod
        real = get()
        c = LaunchCounter(real)
        _mod = c
        return c

    def uninstall(self) -> None:
        global _mod
        _mod = self._mod
