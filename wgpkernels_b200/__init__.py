"""B200-native (sm_100a) INT8 weight linear behind the `wgpkernels.int8` API of WGPKernels.

    from wgpkernels_b200 import int8 as wq
    wq.load_library(); y = wq.linear(x, weight, scale, bias)

The kernels live in one C-ABI shared library (`wgpkernels_b200/csrc`, built by `python -m wgpkernels_b200.build`)
that exports the reference's `wq8_*` entry points; `wgpkernels_b200.int8` is the host-side mirror of the
reference's Python module (same functions, arguments and errors).
"""
__version__ = "0.1.0"
