"""B200-native execution path behind the pytorch-rs (`torch_rs`) operator surface.

`_abi` binds the C ABI of libtrs_cuda.so (include/trs_cuda.h); `_device` wraps device buffers,
streams and events.  The tensor surface is added on top of these.
"""
from . import _abi, _device  # noqa: F401
