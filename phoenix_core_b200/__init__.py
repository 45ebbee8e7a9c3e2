"""B200-native quaternion Conv2D / Dense operators behind the UpStride engine's operator API.

The package holds the CUDA backend (``csrc/``: hand-written sm_100a kernels behind a C ABI declared in
``include/phoenix_core_b200.h``), the C++ operator layer mirroring ``upstride::conv2DFwd`` & co.
(``cpp/``), and this Python host layer used by the tests, the benchmark and the data-parallel harness.
"""
from . import _lib
from .descriptors import (Algebra, Conv2DBwdDescriptor, Conv2DFwdDescriptor, DataFormat, DenseBwdDescriptor,
                          DenseFwdDescriptor, FilterLayout, Padding, compute_windowed_output_size_and_padding)
from .context import Context, ConvFp16ComputePolicy
from .ops import KeptInput, conv2DBwd, conv2DFwd, denseBwd, denseFwd, getSmMargin, setSmMargin

__all__ = [
    "Algebra", "Padding", "DataFormat", "FilterLayout", "Conv2DFwdDescriptor", "Conv2DBwdDescriptor",
    "DenseFwdDescriptor", "DenseBwdDescriptor", "compute_windowed_output_size_and_padding", "Context",
    "ConvFp16ComputePolicy", "conv2DFwd", "conv2DBwd", "denseFwd", "denseBwd", "setSmMargin", "getSmMargin", "KeptInput",
]
