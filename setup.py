"""Build script: compiles the CUDA extension for sm_100a in-tree and installs the Python packages.

``python setup.py build_ext --inplace`` (or ``pip install -e . --no-build-isolation``) produces
``wallx_b200/_build/_wallx_C.so``, the same file that ``wallx_b200.ops._ext.build()`` JIT-builds.
Reference build: setup.py:9-49 (one CUDAExtension, arch taken from the device or the environment;
here the target is fixed: compute_100a / sm_100a, and no CUTLASS include directory is needed).
"""
import os

from setuptools import find_packages, setup


def extensions():
    from torch.utils.cpp_extension import CUDAExtension

    here = os.path.dirname(os.path.abspath(__file__))
    import importlib.util

    spec = importlib.util.spec_from_file_location("_wx_ext", os.path.join(here, "wallx_b200", "ops", "_ext.py"))
    ext = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ext)
    src = [os.path.join("wallx_b200", "csrc", s) for s in ext.SOURCES]
    return [CUDAExtension(name="wallx_b200._build._wallx_C", sources=src,
                          extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": list(ext.NVCC_FLAGS)})]


def cmdclass():
    from torch.utils.cpp_extension import BuildExtension

    return {"build_ext": BuildExtension.with_options(use_ninja=True)}


setup(
    name="wallx_b200",
    version="0.1.0",
    description="Blackwell-native VLA training and inference framework (WALL-OSS capabilities)",
    packages=find_packages(include=["wallx_b200*", "wall_x*"]),
    package_data={"wallx_b200": ["utils/*.json", "csrc/*"]},
    ext_modules=extensions(),
    cmdclass=cmdclass(),
    python_requires=">=3.10",
)
