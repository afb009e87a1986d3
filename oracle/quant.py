"""Oracle (test infrastructure): the two int8 KV quantisers of the reference.

They are written with explicit fp32 arithmetic and an explicit rounding to the
storage dtype after every operation, which is what eager torch on CPU (and XLA's
CPU backend without excess precision) does for bf16 tensors; the golden vectors
produced by the reference's own code confirm the chain bit for bit.
"""

import torch


def _rt(x32, dtype):
  """Round an fp32 intermediate to the storage dtype and come back to fp32."""
  return x32.to(dtype).to(torch.float32)


def local_amax(val: torch.Tensor):
  """max |val| over (heads, dim) per (batch, token) in fp32: the partial that a
  rank holding only some KV heads contributes; the reference gets the full
  maximum from GSPMD's reduction over the sharded head axis
  (jetstream_pt/cache_manager.py:404-410, 532-535)."""
  return val.to(torch.float32).abs().amax(dim=(-3, -1), keepdim=True)


def quantize_decode(val: torch.Tensor, amax=None):
  """`Int8KVCacheGenerate.quantize`, jetstream_pt/cache_manager.py:532-537.

  val [B, H, T, D] (bf16 or fp32).  scale = amax(|val|) over (H, D) / 127, one
  per (batch, token); codes = (val / scale) cast to int8, i.e. truncated toward
  zero, with no clamp and no epsilon.  An all-zero token has scale 0 and 0/0 =
  NaN, which the cast turns into code 0.
  `amax` (fp32 [B,1,T,1]) replaces the local maximum when the heads are sharded
  and the caller has max-reduced `local_amax` over the ranks.
  Returns (codes int8 [B,H,T,D], scale [B,1,T,1] in val's dtype).
  """
  dt = val.dtype
  v = val.to(torch.float32)
  a = v.abs().amax(dim=(-3, -1), keepdim=True) if amax is None else amax.to(torch.float32)
  s = _rt(a / 127.0, dt)
  t = _rt(v / s, dt)
  t = torch.where(torch.isnan(t), torch.zeros_like(t), t)
  codes = torch.trunc(t).clamp(-128, 127).to(torch.int8)
  return codes, s.to(dt)


def quantize_insert(w: torch.Tensor, reduce_axis):
  """`quantize_tensor(w, reduce_axis, 8, symmetric=True, block_size=-1)`,
  jetstream_pt/quantize.py:24-75 (the branch the KV insert uses,
  jetstream_pt/engine.py:427-432 and 545-553).

  max = clamp(amax(|w|), min=1e-5); scale = max / 127;
  codes = clamp(round_half_even(w * (1 / scale)), -128, 127).
  Returns (codes int8, scale keepdim in w's dtype).
  """
  if isinstance(reduce_axis, int):
    reduce_axis = (reduce_axis,)
  dt = w.dtype
  v = w.to(torch.float32)
  a = v.abs().amax(dim=tuple(reduce_axis), keepdim=True)
  eps = torch.tensor(1e-5, dtype=dt).to(torch.float32)
  a = torch.maximum(a, eps)
  s = _rt(a / 127.0, dt)
  r = _rt(1.0 / s, dt)
  t = _rt(v * r, dt)
  codes = torch.round(t).clamp(-128, 127).to(torch.int8)
  return codes, s.to(dt)


def dequantize(codes, scale):
  """`dequantize_tensor`, jetstream_pt/quantize.py:78-83 (symmetric)."""
  return codes * scale
