"""The fused decode step (`Int8KVCacheGenerate.update_and_attend`, C entry point
`jpt_decode_update_attend`): one launch that quantises and writes the step's new
token and attends to the cache including it.  Cache state must equal that of
the separate `update` bit for bit; attention must match the oracle's update +
attention over the extended range."""

import pytest
import torch

from oracle import attention as oa
from oracle import cache as oc
from oracle.quant import quantize_insert
from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu

DEV = "cuda"


def make_env(**kw):
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  d = JetEngineEnvironmentData(testing=True, **kw)
  d.quant_config.enable_kv_quantization = True
  return JetEngineEnvironment(d, device=DEV)


def _case(seed, b, hq, hkv, s, d, ring, in_dtype=torch.bfloat16):
  g = torch.Generator().manual_seed(seed)
  ck, ks = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  cv, vs = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  ks, vs = ks.to(in_dtype), vs.to(in_dtype)
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  xk = torch.randn(b, hkv, 1, d, generator=g).to(in_dtype)
  xv = (torch.randn(b, hkv, 1, d, generator=g) * 2).to(in_dtype)
  xk[1] = 0  # an all-zero token: scale 0, codes 0
  if ring:
    pos = int(torch.randint(0, s, (1,), generator=g))
    start = torch.randint(0, s, (b,), generator=g)
    n = torch.randint(0, s - 1, (b,), generator=g)
    n[0] = 0  # no token yet: the new one alone
    start = (pos - n) % s  # the existing tokens end where the new one goes
    end = torch.full((b,), pos)
    input_pos = [pos]
  else:
    n = torch.randint(0, s, (b,), generator=g)
    n[0] = 0
    if b > 2:
      n[2] = s - 1
    start = torch.zeros(b, dtype=torch.int64)
    end = n.clone()
    input_pos = n.clone()
  return ck, cv, ks, vs, q, xk, xv, start, end, input_pos


@pytest.mark.parametrize("ring", [False, True])
@pytest.mark.parametrize("shape", [(6, 32, 4, 512, 128), (5, 8, 2, 300, 128), (96, 64, 8, 2048, 128), (3, 4, 4, 64, 128)])
def test_fused_step_equals_update_then_attention(shape, ring):
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  b, hq, hkv, s, d = shape
  ck, cv, ks, vs, q, xk, xv, start, end, input_pos = _case(401, b, hq, hkv, s, d, ring)
  env = make_env(batch_size=b, cache_sequence_length=s, ring_buffer=ring)
  dev = lambda x: x.to(DEV) if isinstance(x, torch.Tensor) else x
  fused = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
  plain = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
  for call in range(2):  # twice: the exchange slots in the workspace carry a launch number
    r, (o, m, l) = fused.update_and_attend(dev(q), dev(xk), dev(xv), 0, dev(start), dev(end), ring=ring)
    rp = plain.update(dev(xk), dev(xv), 0)
    for i, (got, want) in enumerate(zip(r, rp)):
      assert torch.equal(got, want), f"call {call}: element {i} of the update tuple differs"
    # the oracle: update, then attention over the range extended by the new token
    e = oc.int8_update(ck, cv, ks, vs, xk, xv, input_pos, ring_buffer=ring, lazy=False)
    assert torch.equal(r[0].cpu(), e[0]) and torch.equal(r[4].cpu(), e[4])
    if ring:
      e_start, e_end = start, (end + 1) % s
      full = (end - start) % s == s - 1  # the ring would become completely full: start == end means empty there
    else:
      e_start, e_end = start, end + 1
      full = torch.zeros(b, dtype=torch.bool)
    bk = max(c for c in range(1, min(512, s) + 1) if s % c == 0)  # the reference's grid is S // bk blocks
    eo, (em, el) = oa.ragged_mha(q, e[0], e[1], 0, e_start, e_end, e[4], e[5], bk=bk, wrap=ring)
    ok = ~full
    assert attention_close(o[ok], eo[ok]), f"call {call}: {describe(o[ok], eo[ok])}"
    assert torch.allclose(m.cpu()[ok], em[ok], atol=1e-3, rtol=1e-3)
    assert torch.allclose(l.cpu()[ok], el[ok], atol=1e-3, rtol=1e-3)
  assert ak.kernel_status() == 0


def test_fused_step_lazy_stash_and_float32_token():
  """Lazy update: nothing is written to the cache, the stash receives codes and
  scales, the attention still includes the new token.  Float32 new tokens use
  float32 scale caches."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  b, hq, hkv, s, d = 7, 32, 8, 384, 128
  for in_dtype in (torch.bfloat16, torch.float32):
    ck, cv, ks, vs, q, xk, xv, start, end, input_pos = _case(402, b, hq, hkv, s, d, False, in_dtype)
    env = make_env(batch_size=b, cache_sequence_length=s, ring_buffer=False, lazy_cache_update=True,
                   bf16_enable=in_dtype == torch.bfloat16)
    dev = lambda x: x.to(DEV)
    c = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
    r, (o, m, l) = c.update_and_attend(dev(q), dev(xk), dev(xv), 0, dev(start), dev(end))
    assert torch.equal(c.cache_k.cpu(), ck) and torch.equal(c.k_scaler.cpu(), ks), "a lazy step must not touch the cache"
    e = oc.int8_update(ck, cv, ks, vs, xk, xv, input_pos, ring_buffer=False, lazy=False)
    assert torch.equal(r[2].cpu(), e[2]) and torch.equal(r[3].cpu(), e[3])
    assert torch.equal(r[6].cpu(), e[6]) and torch.equal(r[7].cpu(), e[7])
    assert torch.equal(c.new_ks.cpu(), e[2]) and torch.equal(c.new_k_scaler.cpu(), e[6])
    c.finalize()
    assert torch.equal(c.cache_k.cpu(), e[0]) and torch.equal(c.cache_v.cpu(), e[1])
    assert torch.equal(c.k_scaler.cpu(), e[4]) and torch.equal(c.v_scaler.cpu(), e[5])
    eo, (em, el) = oa.ragged_mha(q, e[0], e[1], 0, start, end + 1, e[4], e[5], bk=128)
    assert attention_close(o, eo), describe(o, eo)
    assert torch.allclose(l.cpu(), el, atol=1e-3, rtol=1e-3)


def test_fused_step_lone_rank_wait_runs_out():
  """World of two, the second rank absent: the launch returns after the wait
  limit, raises the exchange status, and has used its own amax."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from test_gpu_bounded_waits import _LoneRankExchange

  b, hq, hkv, s, d = 8, 16, 2, 256, 128
  ck, cv, ks, vs, q, xk, xv, start, end, input_pos = _case(403, b, hq, hkv, s, d, False)
  env = make_env(batch_size=b, cache_sequence_length=s, ring_buffer=False)
  dev = lambda x: x.to(DEV)
  px = _LoneRankExchange(b, wait_cycles=4_000_000)
  try:
    c = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
    r, (o, m, l) = c.update_and_attend(dev(q), dev(xk), dev(xv), 0, dev(start), dev(end), peers=px)
    torch.cuda.synchronize()
    assert px.status() == 1
    e = oc.int8_update(ck, cv, ks, vs, xk, xv, input_pos, ring_buffer=False, lazy=False)
    assert torch.equal(r[0].cpu(), e[0]) and torch.equal(r[6].cpu(), e[6])
  finally:
    px.close()


def test_fused_step_full_cache_is_reported():
  """A sequence whose cache has no row left for the new token: the launch attends to the existing
  tokens of that sequence, writes nothing for it, and the workspace's status word reads 3; the other
  sequences are unaffected, and the word is cleared by the read."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  b, hq, hkv, s, d = 4, 16, 2, 256, 128
  ck, cv, ks, vs, q, xk, xv, start, end, input_pos = _case(404, b, hq, hkv, s, d, False)
  end[3] = s          # full: the token has nowhere to go
  input_pos[3] = s    # (out of range: not written)
  env = make_env(batch_size=b, cache_sequence_length=s, ring_buffer=False)
  dev = lambda x: x.to(DEV)
  assert ak.kernel_status() == 0
  c = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
  r, (o, m, l) = c.update_and_attend(dev(q), dev(xk), dev(xv), 0, dev(start), dev(end))
  torch.cuda.synchronize()
  assert ak.kernel_status() == 3
  assert ak.kernel_status() == 0
  assert torch.equal(r[0][3].cpu(), ck[3]), "the full sequence's cache must be untouched"
  ok = torch.tensor([True, True, True, False])
  e = oc.int8_update(ck, cv, ks, vs, xk, xv, torch.where(ok, input_pos, torch.zeros_like(input_pos)), ring_buffer=False, lazy=False)
  eo, (em, el) = oa.ragged_mha(q, e[0], e[1], 0, start, end + 1, e[4], e[5], bk=128)
  assert attention_close(o[ok], eo[ok]), describe(o[ok], eo[ok])
  # the full sequence: its existing tokens alone
  fo, _ = oa.ragged_mha(q, ck, cv, 0, start, end, ks, vs, bk=128)
  assert attention_close(o[3:], fo[3:]), describe(o[3:], fo[3:])


def test_fused_step_state_survives_other_shapes_on_the_workspace():
  """The fused launch keeps a launch counter and exchange words in the workspace between calls; launches
  of other shapes in between (whose partial results use the same workspace) must not disturb them."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  b, hq, hkv, s, d = 6, 32, 4, 512, 128
  ck, cv, ks, vs, q, xk, xv, start, end, input_pos = _case(405, b, hq, hkv, s, d, False)
  env = make_env(batch_size=b, cache_sequence_length=s, ring_buffer=False)
  dev = lambda x: x.to(DEV)
  fused = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
  plain = Int8KVCacheGenerate(dev(ck).clone(), dev(cv).clone(), dev(ks).clone(), dev(vs).clone(), dev(input_pos), env=env)
  g = torch.Generator().manual_seed(406)
  for call in range(3):
    r, _ = fused.update_and_attend(dev(q), dev(xk), dev(xv), 0, dev(start), dev(end))
    rp = plain.update(dev(xk), dev(xv), 0)
    for i, (got, want) in enumerate(zip(r, rp)):
      assert torch.equal(got, want), f"call {call}: element {i} of the update tuple differs"
    # other shapes on the same workspace: a long bf16 cache with few sequences (many partial pieces) ...
    ob, oh, os_, od = 2, 8, 4096, 128
    k2 = torch.randn(ob, oh, os_, od, generator=g).to(torch.bfloat16).to(DEV)
    q2 = torch.randn(ob, oh, 1, od, generator=g).to(torch.bfloat16).to(DEV)
    ak.ragged_mha(q2, k2, k2, 0, torch.zeros(ob, dtype=torch.int32, device=DEV),
                  torch.full((ob,), os_, dtype=torch.int32, device=DEV), None, None, None, None)
    # ... and the split-K kernel (head_dim 64)
    k3 = torch.randn(3, 2, 1024, 64, generator=g).to(torch.bfloat16).to(DEV)
    q3 = torch.randn(3, 2, 1, 64, generator=g).to(torch.bfloat16).to(DEV)
    ak.ragged_mha(q3, k3, k3, 0, torch.zeros(3, dtype=torch.int32, device=DEV),
                  torch.full((3,), 1024, dtype=torch.int32, device=DEV), None, None, None, None)
  assert ak.kernel_status() == 0
