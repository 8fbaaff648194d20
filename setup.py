"""Build and packaging of ``transformerengine_b200`` (reference counterpart: ``setup.py`` + ``build_tools/``).

    python setup.py build_ext --inplace        # compiles transformerengine_b200/_teb200_C*.so in the tree
    python -m pip install --no-build-isolation . # installs the package with the compiled extension
    python setup.py bdist_wheel                # a wheel with the extension inside

Build switches (environment):

    TEB200_CUDA_ARCHS       gencode targets, default "100a" (the kernels use tcgen05 / TMEM / TMA: sm_100a only)
    TEB200_BUILD_FAST_MATH  "0" drops --use_fast_math (activation / softmax intrinsics), default "1"
    TEB200_BUILD_LINEINFO   "0" drops -lineinfo, default "1"
    TEB200_BUILD_DEBUG      "1" compiles with -G -O0 for cuda-gdb, default "0"
    MAX_JOBS                parallel compile jobs (ninja)

The same sources and flags are used by ``__graft_entry__.build()`` / ``ops/_ext.build()`` (JIT build into
the tree); both routes produce an extension module named ``_teb200_C`` next to the Python sources.
"""
import glob
import os

from setuptools import find_packages, setup

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("transformerengine_b200", "csrc")


def _sources():
    cpp = sorted(glob.glob(os.path.join(CSRC, "**", "*.cpp"), recursive=True))
    cu = sorted(glob.glob(os.path.join(CSRC, "**", "*.cu"), recursive=True))
    return cpp + cu


def _nvcc_flags():
    archs = os.environ.get("TEB200_CUDA_ARCHS", "100a").replace(",", ";").split(";")
    flags = []
    for a in archs:
        a = a.strip()
        if not a:
            continue
        if not a.startswith("100"):
            raise SystemExit(f"TEB200_CUDA_ARCHS={a}: the kernels need sm_100a (tcgen05, TMEM)")
        flags += ["-gencode", f"arch=compute_{a},code=sm_{a}"]
    flags += ["-std=c++17", "--expt-relaxed-constexpr",
              "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
              "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__"]
    if os.environ.get("TEB200_BUILD_DEBUG", "0") == "1":
        flags += ["-G", "-O0"]
    else:
        flags += ["-O3"]
        if os.environ.get("TEB200_BUILD_LINEINFO", "1") == "1":
            flags += ["-lineinfo"]
    if os.environ.get("TEB200_BUILD_FAST_MATH", "1") == "1":
        flags += ["--use_fast_math"]
    return flags


def _extension():
    from torch.utils.cpp_extension import CUDAExtension

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return CUDAExtension(
        name="transformerengine_b200._teb200_C",
        sources=_sources(),
        include_dirs=[os.path.join(ROOT, CSRC, "include")],
        extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": _nvcc_flags()},
    )


def _cmdclass():
    from torch.utils.cpp_extension import BuildExtension

    return {"build_ext": BuildExtension.with_options(use_ninja=True)}


if __name__ == "__main__":
    setup(
        name="transformerengine_b200",
        version="0.2.0",
        description="Blackwell-native low-precision transformer library (PyTorch front end, sm_100a kernels)",
        packages=find_packages(include=["transformerengine_b200", "transformerengine_b200.*"]),
        package_data={"transformerengine_b200": ["csrc/**/*", "csrc/include/teb200/*"]},
        ext_modules=[_extension()],
        cmdclass=_cmdclass(),
        python_requires=">=3.10",
        install_requires=["torch>=2.6"],
        zip_safe=False,
    )
