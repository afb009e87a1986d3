"""B200-native KV-cache hot path of jetstream-pytorch.

Python surface = the reference's own module layout
(cache_manager, page_attention_manager, attention_kernel, quantize, layers),
device side = libjpt_b200.so (hand-written CUDA for sm_100a, C ABI in
include/jpt_b200.h).  There is no CPU or eager fallback.
"""

from jetstream_pytorch_b200 import _lib  # noqa: F401

__all__ = ["attention_kernel", "cache_manager", "environment", "insert", "layers", "page_attention_manager",
           "quantize"]
