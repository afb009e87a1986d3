"""GPU parity of the weight-only int8 linear layer (tcgen05 integer MMAs fed by
the copy engine) against the oracle and against the reference's own layer
(tests/golden/linear.npz)."""

import pytest
import torch

from golden_io import load
from oracle import linear as ol

pytestmark = pytest.mark.gpu

DEV = "cuda"


def layer_for(w_q, scale):
  from jetstream_pytorch_b200.layers import WeightOnlyPerChannelQuantizedLinear

  n, k = w_q.shape
  lin = WeightOnlyPerChannelQuantizedLinear(k, n, device=DEV)
  lin._load_quantized_weights(w_q, scale)
  return lin


def check(lin, x, w_q, scale, want=None):
  y = lin(x.to(DEV))
  torch.cuda.synchronize()
  assert lin.kernel_status() == 0
  y = y.cpu()
  exp = ol.w8a16_linear(x, w_q, scale).reshape(y.shape)
  tol = ol.w8a16_tolerance(x, w_q, scale).reshape(y.shape)
  err = (y.float() - exp.float()).abs().double()
  assert (err <= tol).all(), f"max excess {(err - tol).max().item()}"
  same = (y.view(torch.int16) == exp.view(torch.int16)).float().mean().item()
  assert same > 0.95, same  # (a rounding boundary is crossed by about one output in sixty)
  if want is not None:
    assert ((y.float() - want.float()).abs().double() <= tol).all()
  return y


@pytest.mark.parametrize("tag", ["small", "batch"])
def test_linear_against_the_reference_layer(tag):
  g = load("linear")
  x, w, s, want = g[f"{tag}_x"], g[f"{tag}_weight"], g[f"{tag}_weight_scaler"], g[f"{tag}_y"]
  lin = layer_for(w, s)
  y = check(lin, x, w, s, want)
  assert y.shape == want.shape and y.dtype == torch.bfloat16
  assert not y[0, 1].any()  # the all-zero row of activations


@pytest.mark.parametrize("m,k,n", [(1, 128, 128), (3, 256, 100), (8, 512, 384), (17, 1024, 1000), (96, 2048, 512),
                                   (128, 1024, 256), (33, 8192, 640), (300, 512, 384)])
def test_linear_shapes(m, k, n):
  """Ragged batch sizes (padded to eight level rows), output channels that are
  not a multiple of the 256-channel tile, K split over the CTAs of a cluster,
  more than 128 rows (taken in blocks)."""
  g = torch.Generator().manual_seed(m * 131 + n)
  w = torch.randn(n, k, generator=g) * 0.03
  w_q, scale = ol.quantize_weight(w)
  x = (torch.randn(m, k, generator=g) * torch.rand(m, 1, generator=g) * 4).to(torch.bfloat16)
  lin = layer_for(w_q, scale)
  check(lin, x, w_q, scale)


def test_linear_is_deterministic_and_linear_in_the_scale():
  """Size-independent properties at a model-sized layer (Llama-2-70B's output
  projection, 8192 x 8192, batch 96): two runs agree bit for bit; doubling every
  channel scale doubles the output exactly (powers of two commute with the bf16
  roundings); extreme codes (+-127 / -128 everywhere) do not overflow the int32
  sums."""
  g = torch.Generator().manual_seed(5)
  m, k, n = 96, 8192, 8192
  w_q = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
  w_q[0] = 127
  w_q[1] = -128
  scale = (torch.rand(n, generator=g) * 0.01 + 1e-3).to(torch.bfloat16)
  x = torch.randn(m, k, generator=g).to(torch.bfloat16)
  x[0] = 3.0  # every level of the row at +127: the largest sums
  lin = layer_for(w_q, scale)
  y1 = lin(x.to(DEV)).clone()
  y2 = lin(x.to(DEV))
  assert torch.equal(y1, y2)
  lin._load_quantized_weights(w_q, (scale.float() * 2).to(torch.bfloat16))
  y3 = lin(x.to(DEV))
  torch.cuda.synchronize()
  assert lin.kernel_status() == 0
  assert torch.equal(y3.float(), y1.float() * 2)
  # a sample of the rows against the oracle (the full product takes the CPU a while in float64)
  rows = [0, 1, 50, 95]
  exp = ol.w8a16_linear(x[rows], w_q[:512], scale[:512])
  tol = ol.w8a16_tolerance(x[rows], w_q[:512], scale[:512])
  got = y1.cpu()[rows][:, :512]
  assert ((got.float() - exp.float()).abs().double() <= tol).all()
  assert got[0, 0].item() == exp[0, 0].item() and got[0, 1].item() == exp[0, 1].item()


def test_linear_rejects_what_it_does_not_take():
  from jetstream_pytorch_b200.layers import WeightOnlyPerChannelQuantizedLinear

  lin = WeightOnlyPerChannelQuantizedLinear(256, 128, device=DEV)
  with pytest.raises(NotImplementedError):
    lin(torch.zeros(4, 256, dtype=torch.float32, device=DEV))
  with pytest.raises(NotImplementedError):
    WeightOnlyPerChannelQuantizedLinear(200, 128, device=DEV)
