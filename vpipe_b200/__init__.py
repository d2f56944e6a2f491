"""vpipe_b200 -- B200 (sm_100a) implementation of vpipe's 4-bit affine
group-quantized linear: QMV (decode), QMM (prefill / DiT), dequantizer and
forward quantizer, behind the C ABI declared in ``include/vpq.h``.

The product is ``libvpq.so`` (hand-written CUDA, built in-tree by
``python -m vpipe_b200.build``). This package is the thin Python loader used by
the tests and the benchmark: ctypes bindings that pass torch tensors' device
pointers straight through. There is no CPU or PyTorch fallback: if the library
is missing or no sm_100 device is present, calls raise.
"""
from ._lib import VpqError, lib, lib_path, status_string  # noqa: F401
from . import ops, synth, shard  # noqa: F401

__all__ = ["VpqError", "lib", "lib_path", "status_string", "ops", "synth", "shard"]
