"""Oracle (test infrastructure): the weight-only int8 per-channel linear layer.

Restates `WeightOnlyPerChannelQuantizedLinear` of the reference
(jetstream_pt/layers.py:69-166) for symmetric 8-bit weights without activation
quantisation, and the per-channel weight quantiser it loads its buffers with
(jetstream_pt/quantize.py:24-76, 86-99).

Pin: the weight quantiser is checked bit for bit against the reference's own
`quantize_weight_from_nn_linear`, and `forward` against the reference's own
`forward`, both executed unmodified by tests/golden/make_golden.py.  The
reference's `F.linear(bf16 inputs, int8 weight)` only exists under torch_xla2,
where the product follows jax's type promotion (int8 -> bfloat16, bfloat16
result); the generator stands in for that one call with
`F.linear(inputs, weight.to(inputs.dtype))` on CPU torch (fp32 accumulation,
one rounding to bf16).  The accumulation ORDER of an XLA backend is not
reproducible here, so the forward is pinned within `w8a16_tolerance` (in the
fixtures all outputs but one in 30,000 are identical; that one is a sum that
cancels to almost nothing), not bit for bit.
"""

import torch

EPS = 1e-5


def quantize_weight(weight: torch.Tensor):
  """`quantize_tensor(weight, (1,), 8, True)` followed by `load_q_weight_helper`
  (quantize.py:58-76, 86-93): per output channel, scale = max(amax|w|, 1e-5) /
  127 in the weight's dtype, codes = clamp(round(w * (1 / scale)), -128, 127).
  Returns (codes int8 [N, K], scale bf16 [N])."""
  max_val = weight.abs().amax(dim=1, keepdim=True).clamp(min=EPS)
  scales = max_val / 127
  codes = torch.clamp(torch.round(weight * (1.0 / scales)), -128, 127).to(torch.int8)
  return codes, scales.squeeze(-1).to(torch.bfloat16)


def w8a16_linear(x: torch.Tensor, w_q: torch.Tensor, scale: torch.Tensor):
  """layers.py:137-154 with `quantize_activation` off and symmetric weights:
  result = F.linear(x, W) (a bf16 tensor), then result * weight_scaler (bf16).
  The dot products are taken exactly (float64: |sum| < 2^53 for bf16 x int8
  terms of any K in use), so the first rounding is the correctly rounded one."""
  dot = x.to(torch.float64) @ w_q.to(torch.float64).t()
  first = dot.to(torch.float32).to(torch.bfloat16)
  return (first.to(torch.float32) * scale.to(torch.float32)).to(torch.bfloat16)


def w8a16_tolerance(x: torch.Tensor, w_q: torch.Tensor, scale: torch.Tensor):
  """Largest |difference| allowed between an implementation of this layer and
  `w8a16_linear`, per output element: a bf16 rounding that falls the other way
  moves a value by up to 2^-7 of itself, and there are two roundings (2^-6);
  plus an error of 2^-15 of a row's
  amax|x| per activation element, summed over the channel's |weights| (the
  device kernel holds the activations as two int8 levels, exact to 2^-16 of the
  row's amax)."""
  exact = (x.to(torch.float64) @ w_q.to(torch.float64).t()) * scale.to(torch.float64)
  amax = x.to(torch.float64).abs().amax(dim=-1, keepdim=True)
  wsum = w_q.to(torch.float64).abs().sum(dim=1) * scale.to(torch.float64).abs()
  return exact.abs() * 2.0 ** -6 + amax * wsum * 2.0 ** -15


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float):
  """`RMSNorm.forward`, jetstream_pt/layers.py:345-350, for bf16 x and a bf16
  weight: the norm in fp32 (`x.float()`), rounded to x's dtype (`type_as`), times
  the weight (bf16 product).  Pinned bit for bit against the reference's own class
  (tests/golden/linear.npz)."""
  xf = x.float()
  normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)
  return normed * weight


def silu_mul(a: torch.Tensor, b: torch.Tensor):
  """The gate of `FeedForward.forward`, third_party/llama/model_exportable.py:85:
  `F.silu(a) * b` on bf16 tensors (each op rounds to bf16)."""
  return torch.nn.functional.silu(a) * b


def feed_forward(x, w1, s1, w2, s2, w3, s3):
  """model_exportable.py:84-86 with the weight-only int8 layers."""
  return w8a16_linear(silu_mul(w8a16_linear(x, w1, s1), w8a16_linear(x, w3, s3)), w2, s2)
