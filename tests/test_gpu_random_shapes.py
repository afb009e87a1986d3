"""Randomly drawn shapes and valid ranges through the int8 head_dim-128 attention paths (the tcgen05
kernel with 8 or 2 softmax rows, copy-engine and thread-copy row loads, left-aligned and ring ranges,
dense and paged caches) and through the fused decode step, against the CPU oracle.  Every case is
seeded; the draw favours the edges (empty, one token, full, wrap over the end, lengths around the
128-token tile)."""

import pytest
import torch

from oracle import attention as oa
from oracle import cache as oc
from oracle.quant import quantize_insert
from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu

DEV = "cuda"
LENGTHS = [64, 128, 192, 256, 320, 384, 512, 640, 1024, 1536]


def _divisor_block(s):
  return max(c for c in range(1, min(512, s) + 1) if s % c == 0)  # the reference's grid is S // bk blocks


def _edge_lengths(g, b, s):
  edges = torch.tensor([0, 1, 2, 127, 128, 129, 255, 256, 257, s - 1, s])
  edges = edges[(edges >= 0) & (edges <= s)]
  n = torch.randint(0, s + 1, (b,), generator=g)
  pick = torch.rand(b, generator=g) < 0.5
  n[pick] = edges[torch.randint(0, len(edges), (int(pick.sum()),), generator=g)]
  return n


def _draw(seed):
  g = torch.Generator().manual_seed(9000 + seed)
  b = int(torch.randint(1, 13, (1,), generator=g))
  hkv = [1, 2, 3, 4, 8][int(torch.randint(0, 5, (1,), generator=g))]
  rep = [1, 2, 3, 4, 8][int(torch.randint(0, 5, (1,), generator=g))]
  s = LENGTHS[int(torch.randint(0, len(LENGTHS), (1,), generator=g))]
  ring = bool(torch.randint(0, 2, (1,), generator=g))
  return g, b, hkv, rep, s, ring


@pytest.mark.parametrize("seed", range(24))
def test_random_int8_ragged_attention(seed):
  """(JPT_NO_TMA=1 in the environment runs the same cases through the thread-copy row loads.)"""
  from jetstream_pytorch_b200 import attention_kernel as ak

  g, b, hkv, rep, s, ring = _draw(seed)
  d, hq = 128, hkv * rep
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  k, ks = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  v, vs = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  n = _edge_lengths(g, b, s)
  if ring:
    n = n.clamp(max=s - 1)  # start == end means empty there: a ring holds at most S - 1 tokens
    start = torch.randint(0, s, (b,), generator=g)
    end = (start + n) % s
  else:
    start, end = torch.zeros(b, dtype=torch.int64), n
  c = lambda t: t.to(DEV)
  o, (m, l) = ak.ragged_mha(c(q), c(k), c(v), 0, c(start), c(end), None, None, c(ks), c(vs), ring=ring)
  eo, (em, el) = oa.ragged_mha(q, k, v, 0, start, end, ks, vs, bk=_divisor_block(s), wrap=ring)
  what = f"seed {seed}: B={b} Hkv={hkv} rep={rep} S={s} ring={ring} n={n.tolist()}"
  assert attention_close(o, eo), what + " " + describe(o, eo)
  live = torch.isfinite(em)
  assert torch.equal(torch.isfinite(m.cpu()), live), what
  assert torch.allclose(m.cpu()[live], em[live], atol=1e-3, rtol=1e-3), what
  assert torch.allclose(l.cpu()[live], el[live], atol=1e-3, rtol=1e-3), what
  assert not o.cpu()[~live].any(), what
  assert ak.kernel_status() == 0


@pytest.mark.parametrize("seed", range(12))
def test_random_fused_decode_step(seed):
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  g, b, hkv, rep, s, ring = _draw(100 + seed)
  rep = {3: 2}.get(rep, rep)
  d, hq = 128, hkv * rep
  ck, ks = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  cv, vs = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  xk = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  if ring:
    pos = int(torch.randint(0, s, (1,), generator=g))
    n = _edge_lengths(g, b, s).clamp(max=s - 2)  # the ring must not become completely full
    start, end, input_pos = (pos - n) % s, torch.full((b,), pos), [pos]
  else:
    n = _edge_lengths(g, b, s).clamp(max=s - 1)  # room for the new token
    start, end, input_pos = torch.zeros(b, dtype=torch.int64), n.clone(), n.clone()
  data = JetEngineEnvironmentData(testing=True, batch_size=b, cache_sequence_length=s, ring_buffer=ring)
  data.quant_config.enable_kv_quantization = True
  env = JetEngineEnvironment(data, device=DEV)
  c = lambda t: t.to(DEV) if isinstance(t, torch.Tensor) else t
  cache = Int8KVCacheGenerate(c(ck).clone(), c(cv).clone(), c(ks).clone(), c(vs).clone(), c(input_pos), env=env)
  if not cache.fused_step_supported(c(q), c(xk)):
    pytest.skip("shape not taken by the fused launch")
  r, (o, m, l) = cache.update_and_attend(c(q), c(xk), c(xv), 0, c(start), c(end), ring=ring)
  e = oc.int8_update(ck, cv, ks, vs, xk, xv, input_pos, ring_buffer=ring, lazy=False)
  what = f"seed {seed}: B={b} Hkv={hkv} rep={rep} S={s} ring={ring} n={n.tolist()}"
  for i in (0, 1, 2, 3, 4, 5, 6, 7):
    assert torch.equal(r[i].cpu(), e[i]), what + f": element {i} of the update tuple differs"
  e_end = (end + 1) % s if ring else end + 1
  eo, (em, el) = oa.ragged_mha(q, e[0], e[1], 0, start, e_end, e[4], e[5], bk=_divisor_block(s), wrap=ring)
  assert attention_close(o, eo), what + " " + describe(o, eo)
  assert torch.allclose(l.cpu(), el, atol=1e-3, rtol=1e-3), what
  assert ak.kernel_status() == 0


@pytest.mark.parametrize("seed", range(12))
def test_random_bf16_ragged_attention(seed):
  """The same draw with unquantised caches (the mma.sync kernel and its in-kernel merge)."""
  from jetstream_pytorch_b200 import attention_kernel as ak

  g, b, hkv, rep, s, ring = _draw(200 + seed)
  d, hq = 128, hkv * rep
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  k = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
  v = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
  n = _edge_lengths(g, b, s)
  if ring:
    n = n.clamp(max=s - 1)
    start = torch.randint(0, s, (b,), generator=g)
    end = (start + n) % s
  else:
    start, end = torch.zeros(b, dtype=torch.int64), n
  c = lambda t: t.to(DEV)
  o, (m, l) = ak.ragged_mha(c(q), c(k), c(v), 0, c(start), c(end), None, None, None, None, ring=ring)
  eo, (em, el) = oa.ragged_mha(q, k, v, 0, start, end, None, None, bk=_divisor_block(s), wrap=ring)
  what = f"seed {seed}: B={b} Hkv={hkv} rep={rep} S={s} ring={ring} n={n.tolist()}"
  assert attention_close(o, eo), what + " " + describe(o, eo)
  live = torch.isfinite(em)
  assert torch.allclose(l.cpu()[live], el[live], atol=1e-3, rtol=1e-3), what
  assert not o.cpu()[~live].any(), what
  assert ak.kernel_status() == 0
