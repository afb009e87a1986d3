"""KV insert quantiser, device side.

Mirror of `quantize_tensor` / `dequantize_tensor`,
jetstream_pt/quantize.py:24-83, restricted to what the KV-cache path calls:
8 bit, symmetric, per-token over (heads, head_dim) -- `reduce_axis=(-3,-1)` on a
[1,H,L,D] prefix (jetstream_pt/engine.py:428-432) or `(1,2)` on [L,H,D]
(engine.py:547-553).  Weight quantisation is outside this package.
"""

import torch

from jetstream_pytorch_b200 import _lib

EPS = 1e-5


def quantize_tensor(w, reduce_axis, n_bit=8, symmetric=True, block_size=-1):
  """Returns (codes int8, scales keepdim in w's dtype, None)."""
  if n_bit != 8 or not symmetric or block_size > 0:
    raise NotImplementedError("only 8-bit symmetric per-token KV quantisation is provided")
  if isinstance(reduce_axis, int):
    reduce_axis = (reduce_axis,)
  axes = tuple(sorted(a % w.ndim for a in reduce_axis))
  w = w.contiguous()
  if w.ndim == 4 and axes == (1, 3) and w.shape[0] == 1:
    _, h, l, d = w.shape
    token_major, scale_shape = 0, (1, 1, l, 1)
  elif w.ndim == 3 and axes == (1, 2):
    l, h, d = w.shape
    token_major, scale_shape = 1, (l, 1, 1)
  else:
    raise NotImplementedError(f"quantize_tensor: layout {tuple(w.shape)} / axes {reduce_axis} is not a KV layout")
  codes = torch.empty(w.shape, dtype=torch.int8, device=w.device)
  scales = torch.empty(scale_shape, dtype=w.dtype, device=w.device)
  _lib.check(_lib.lib().jpt_quantize_tokens(_lib.ptr(w), _lib.dt(w), token_major, h, l, d, _lib.ptr(codes),
                                            _lib.ptr(scales), _lib.stream()))
  return codes, scales, None


def dequantize_tensor(w, scale, zero_point=None):
  """jetstream_pt/quantize.py:78-83."""
  if zero_point is not None:
    return (w - zero_point) * scale
  return w * scale
