"""ctypes binding of libjpt_b200.so (the C ABI declared in include/jpt_b200.h).

There is no fallback: if the library is missing or a call fails, the caller
gets an exception.
"""

import ctypes
import os
import queue

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libjpt_b200.so")

BF16, F32, INT8 = 0, 1, 2
MASK_NONE, MASK_LENGTH, MASK_RING, MASK_ADD = 0, 1, 2, 3

_DTYPES = {torch.bfloat16: BF16, torch.float32: F32, torch.int8: INT8}

c_void_p, c_int, c_i64, c_size_t, c_float = (
    ctypes.c_void_p,
    ctypes.c_int,
    ctypes.c_int64,
    ctypes.c_size_t,
    ctypes.c_float,
)


class PeerExchangeStruct(ctypes.Structure):
  """Mirror of `struct jpt_peer_exchange` (include/jpt_b200.h)."""
  _fields_ = [("rank", c_int), ("world", c_int), ("batch", c_int), ("buffers", c_void_p * 8),
              ("wait_cycles", ctypes.c_longlong)]


class TpSumStruct(ctypes.Structure):
  """Mirror of `struct jpt_tp_sum`."""
  _fields_ = [("rank", c_int), ("world", c_int), ("buffers", c_void_p * 8), ("buffer_bytes", c_size_t),
              ("wait_cycles", ctypes.c_longlong)]


class AttnParams(ctypes.Structure):
  """Mirror of `struct jpt_attn_params`."""

  _fields_ = [
      ("q", c_void_p), ("q_dtype", c_int),
      ("B", c_int), ("Hq", c_int), ("Hkv", c_int), ("Tq", c_int), ("D", c_int),
      ("k", c_void_p), ("v", c_void_p), ("kv_dtype", c_int), ("paged", c_int),
      ("S", c_int),
      ("kv_b", c_i64), ("kv_h", c_i64), ("kv_s", c_i64),
      ("page_size", c_int), ("kv_page", c_i64),
      ("page_table", c_void_p), ("max_pages", c_int),
      ("k_scale", c_void_p), ("v_scale", c_void_p), ("scale_dtype", c_int),
      ("sc_b", c_i64), ("sc_s", c_i64),
      ("mask_mode", c_int), ("start", c_void_p), ("end", c_void_p),
      ("mask", c_void_p), ("mk_b", c_i64), ("mk_r", c_i64),
      ("sm_scale", c_float),
      ("o", c_void_p), ("m", c_void_p), ("l", c_void_p),
      ("workspace", c_void_p), ("workspace_bytes", c_size_t),
      ("num_splits", c_int), ("force_generic", c_int), ("logit_rounding", c_int),
  ]


class NewTokenStruct(ctypes.Structure):
  """Mirror of `struct jpt_new_token`."""
  _fields_ = [("xk", c_void_p), ("xv", c_void_p), ("in_dtype", c_int), ("write_cache", c_int),
              ("k_quant", c_void_p), ("v_quant", c_void_p), ("k_scale", c_void_p), ("v_scale", c_void_p),
              ("pos", c_void_p), ("pos_count", c_int), ("pos_host", c_int),
              ("px", ctypes.POINTER(PeerExchangeStruct))]


_SIGNATURES = {
    "jpt_last_error_string": (ctypes.c_char_p, []),
    "jpt_version": (c_int, []),
    "jpt_launch_count": (ctypes.c_longlong, []),
    "jpt_kv_quant_append_dense": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 8
                                  + [c_void_p, c_int, c_int] + [c_int] * 4 + [c_i64] * 5
                                  + [c_void_p, c_void_p, c_void_p]),
    "jpt_peer_exchange_bytes": (ctypes.c_size_t, [c_int, c_int]),
    "jpt_peer_exchange_alloc": (c_int, [ctypes.c_size_t, ctypes.POINTER(c_void_p)]),
    "jpt_peer_exchange_free": (c_int, [c_void_p]),
    "jpt_peer_exchange_export": (c_int, [c_void_p, c_void_p]),
    "jpt_peer_exchange_import": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "jpt_peer_exchange_release": (c_int, [c_void_p]),
    "jpt_peer_exchange_status": (c_int, [c_void_p, c_void_p]),
    "jpt_kv_quant_append_dense_peers": (c_int, [c_void_p, c_void_p, c_int] + [c_void_p] * 8
                                        + [c_void_p, c_int, c_int] + [c_int] * 4 + [c_i64] * 5
                                        + [c_void_p, c_void_p]),
    "jpt_kv_scatter_rows": (c_int, [c_void_p] * 4 + [c_int, c_void_p, c_int, c_int, c_int]
                            + [c_int] * 5 + [c_i64] * 4 + [c_void_p]),
    "jpt_kv_append_paged": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_i64, c_int, c_void_p] + [c_int] * 5 + [c_void_p]),
    "jpt_page_token_indices": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "jpt_prefill_insert_dense": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                         c_void_p] + [c_int] * 8 + [c_i64] * 10 + [c_void_p]),
    "jpt_prefill_insert_paged": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                         c_void_p, c_void_p] + [c_int] * 7 + [c_i64] * 5 + [c_void_p]),
    "jpt_enable_peer_access": (c_int, [c_int, c_int]),
    "jpt_w8a16_linear_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "jpt_w8a16_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jpt_w8a16_split_levels": (c_int, [c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jpt_w8a16_linear_from_levels": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "jpt_w8a16_tp_buffer_bytes": (c_size_t, [c_int, c_int]),
    "jpt_w8a16_linear_tp": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t,
                                    ctypes.POINTER(TpSumStruct), c_void_p]),
    "jpt_w8a16_tp_status": (c_int, [ctypes.POINTER(TpSumStruct), c_void_p]),
    "jpt_rmsnorm": (c_int, [c_void_p, c_void_p, ctypes.c_float, c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jpt_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "jpt_quantize_tokens": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "jpt_flash_decode": (c_int, [ctypes.POINTER(AttnParams), c_void_p]),
    "jpt_flash_decode_static": (c_int, [ctypes.POINTER(AttnParams), c_void_p]),
    "jpt_decode_update_attend": (c_int, [ctypes.POINTER(AttnParams), ctypes.POINTER(NewTokenStruct), c_void_p]),
    "jpt_flash_decode_workspace_bytes": (c_size_t, [ctypes.POINTER(AttnParams)]),
    "jpt_flash_decode_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "jpt_flash_decode_status": (c_int, [c_void_p, c_void_p]),
    "jpt_merge_partials": (c_int, [c_void_p] * 6 + [c_int, c_void_p, c_int, c_i64, c_int, c_void_p]),
}

EXPORTS = tuple(_SIGNATURES)

_lib = None


def lib():
  """Loads the CUDA library once.  Raises if it has not been built."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise RuntimeError(
          f"{LIB_PATH} is missing: build it with `python -m jetstream_pytorch_b200.build` "
          "(there is no CPU or eager fallback)"
      )
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
      fn = getattr(handle, name)
      fn.restype, fn.argtypes = res, args
    _lib = handle
  return _lib


def check(rc):
  """Turns a non-zero status into an exception."""
  if rc == 0:
    return
  msg = lib().jpt_last_error_string().decode()
  if rc < 0:
    raise ValueError(f"libjpt_b200 argument error {rc}: {msg}")
  raise RuntimeError(f"libjpt_b200 CUDA error {rc}: {msg}")


def dt(t):
  try:
    return _DTYPES[t.dtype if isinstance(t, torch.Tensor) else t]
  except KeyError as e:
    raise ValueError(f"unsupported dtype {e}") from None


def ptr(t):
  """Device pointer of a CUDA tensor (None -> NULL)."""
  if t is None:
    return None
  if not t.is_cuda:
    raise ValueError("libjpt_b200 works on CUDA tensors only; got a tensor on " + str(t.device))
  return t.data_ptr()


def stream():
  return torch.cuda.current_stream().cuda_stream


def as_i32(x, device):
  """A position / length / index argument as an int32 CUDA tensor."""
  if isinstance(x, torch.Tensor):
    if x.device != device:
      x = x.to(device, non_blocking=True)
    return x if x.dtype == torch.int32 else x.to(torch.int32)
  import numpy as np

  return torch.as_tensor(np.asarray(x).astype(np.int32)).to(device, non_blocking=True)


Empty = queue.Empty
