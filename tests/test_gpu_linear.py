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
                                   (128, 1024, 256), (33, 8192, 640), (300, 512, 384), (9, 384, 300), (9, 640, 300),
                                   (96, 768, 520), (128, 896, 256), (96, 8192, 10240)])
def test_linear_shapes(m, k, n):
  """Ragged batch sizes (padded to eight level rows), output channels that are
  not a multiple of the 256-channel tile, K split over clusters of 1 to 8 CTAs
  (3, 5, 6 and 7 K steps give clusters of that size; 10240 channels one of 3 with
  uneven shares), more than 128 rows (taken in blocks)."""
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


def ulp_close(got, want, min_same):
  """bf16 results of the same formula evaluated with another fp32 library (sum
  order, rsqrt, exp): all but a few identical, none further than the
  neighbouring bf16 value."""
  gi, wi = got.view(torch.int16).int(), want.view(torch.int16).int()
  same = (gi == wi).float().mean().item()
  assert same >= min_same, same
  assert (gi - wi).abs().max().item() <= 1


def test_rmsnorm_against_the_reference_class():
  from jetstream_pytorch_b200.layers import RMSNorm

  g = load("linear")
  x, w, eps, want = g["norm_x"], g["norm_weight"], float(g["norm_eps"]), g["norm_y"]
  norm = RMSNorm(x.shape[-1], eps=eps, device=DEV)
  norm.weight.data.copy_(w)
  y = norm(x.to(DEV)).cpu()
  assert y.shape == want.shape
  ulp_close(y, want, 0.999)
  assert not y[0, 1].any()
  y2, lv = norm(x.to(DEV), with_levels=True)
  assert torch.equal(y2.cpu(), y)
  assert lv.rows == 18 and lv.features == 512


@pytest.mark.parametrize("m,k", [(1, 128), (96, 8192), (37, 28672), (128, 1024)])
def test_rmsnorm_and_silu_mul_shapes(m, k):
  from jetstream_pytorch_b200.layers import RMSNorm, silu_mul

  g = torch.Generator().manual_seed(k + m)
  x = (torch.randn(m, k, generator=g) * 3).to(torch.bfloat16)
  w = (1 + 0.2 * torch.randn(k, generator=g)).to(torch.bfloat16)
  norm = RMSNorm(k, eps=1e-5, device=DEV)
  norm.weight.data.copy_(w)
  ulp_close(norm(x.to(DEV)).cpu(), ol.rmsnorm(x, w, 1e-5), 0.999)
  b = torch.randn(m, k, generator=g).to(torch.bfloat16)
  ulp_close(silu_mul(x.to(DEV), b.to(DEV)).cpu(), ol.silu_mul(x, b), 0.999)
  # more rows than levels are kept for: the plain kernels take any number
  if m == 1:
    xx = x.repeat(300, 1)
    assert torch.equal(norm(xx.to(DEV)).cpu(), norm(x.to(DEV)).cpu().repeat(300, 1))


def test_levels_from_the_producers_equal_the_layer_s_own_split():
  """A linear layer fed with the levels that RMSNorm, the gate or
  `ActivationLevels.of` left behind returns what it returns on the bf16 tensor
  itself, bit for bit; the feed-forward block equals its three layers and the gate
  called one by one, and the oracle within the layers' tolerance."""
  from jetstream_pytorch_b200.layers import ActivationLevels, FeedForward, RMSNorm, silu_mul

  g = torch.Generator().manual_seed(77)
  m, dim, hidden = 96, 1024, 2816
  ff = FeedForward(dim, hidden, device=DEV)
  ws = {}
  for name, (n, k) in (("w1", (hidden, dim)), ("w2", (dim, hidden)), ("w3", (hidden, dim))):
    wq, sc = ol.quantize_weight(torch.randn(n, k, generator=g) * 0.03)
    getattr(ff, name)._load_quantized_weights(wq, sc)
    ws[name] = (wq, sc)
  x = torch.randn(3, 32, dim, generator=g).to(torch.bfloat16)
  norm = RMSNorm(dim, eps=1e-5, device=DEV)
  norm.weight.data.copy_((1 + 0.1 * torch.randn(dim, generator=g)).to(torch.bfloat16))
  xd = x.to(DEV)
  y, lv = norm(xd, with_levels=True)
  assert torch.equal(ff.w1(y, levels=lv), ff.w1(y))
  assert torch.equal(ff.w3(y, levels=ActivationLevels.of(y)), ff.w3(y))
  a, b = ff.w1(y), ff.w3(y)
  h, hl = silu_mul(a, b, with_levels=True)
  assert torch.equal(h, silu_mul(a, b))
  assert torch.equal(ff.w2(h, levels=hl), ff.w2(h))
  out = ff(y, levels=lv)
  assert torch.equal(out, ff.w2(h)) and torch.equal(out, ff(y))
  assert out.shape == (3, 32, dim)
  torch.cuda.synchronize()
  assert ff.w1.kernel_status() == 0 and ff.w2.kernel_status() == 0
  # each step against the oracle on the step's own inputs
  yc, ac, bc, hc = y.cpu().reshape(m, dim), a.cpu().reshape(m, hidden), b.cpu().reshape(m, hidden), h.cpu().reshape(m, hidden)
  for got, xin, (wq, sc) in ((ac, yc, ws["w1"]), (bc, yc, ws["w3"]), (out.cpu().reshape(m, dim), hc, ws["w2"])):
    err = (got.float() - ol.w8a16_linear(xin, wq, sc).float()).abs().double()
    assert (err <= ol.w8a16_tolerance(xin, wq, sc)).all()
  ulp_close(hc, ol.silu_mul(ac, bc), 0.999)
