"""Builds the native extension `deep_ep._C` in-tree for NVIDIA B200 (sm_100a).

    python setup.py build_ext --inplace

`csrc/python_api.cpp` holds the host runtime (C++20, compiled by g++); `csrc/kernels/*.cu` hold the
kernels and their launchers (compiled by nvcc with `-gencode arch=compute_100a,code=sm_100a`).
The shared host/device headers live inside the Python package (`deep_ep/include`) because the
runtime JIT compiles kernels against them.
"""
import glob
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
# torch's own arch list would add `-gencode` flags for other GPUs; the explicit flag below is the only target.
os.environ['TORCH_CUDA_ARCH_LIST'] = '10.0a'
# Link against the shared libstdc++ that PyTorch itself uses: a toolchain that links the C++ runtime
# statically gives this module a second, private copy, and exceptions that cross into pybind11's shared
# translators then crash.
if os.path.exists('/usr/bin/g++') and os.path.exists('/usr/bin/gcc'):
    os.environ['CC'], os.environ['CXX'] = '/usr/bin/gcc', '/usr/bin/g++'

sources = ['csrc/python_api.cpp'] + sorted(glob.glob('csrc/kernels/*.cu'))
include_dirs = [os.path.join(ROOT, 'deep_ep', 'include'), os.path.join(ROOT, 'csrc')]
cxx_flags = ['-O3', '-std=c++20', '-Wno-deprecated-declarations', '-Wno-unused-variable', '-Wno-sign-compare', '-Wno-reorder']
nvcc_flags = ['-O3', '-std=c++20', '-lineinfo', '--expt-relaxed-constexpr',
              '-gencode', 'arch=compute_100a,code=sm_100a', '-Xptxas', '-v']

setup(
    name='deep_ep',
    version='1.0.0',
    packages=find_packages(include=['deep_ep', 'deep_ep.*']),
    package_data={'deep_ep': ['include/deep_ep/**/*']},
    ext_modules=[CUDAExtension(
        name='deep_ep._C',
        sources=sources,
        include_dirs=include_dirs,
        extra_compile_args={'cxx': cxx_flags, 'nvcc': nvcc_flags},
    )],
    cmdclass={'build_ext': BuildExtension.with_options(use_ninja=True)},
)
