"""GPU parity: the CUDA path (through the Python boundary and the C ABI) against
the golden vectors produced by the reference's own code and against the CPU
oracle on seeded inputs.  Bit-exact for codes, scales, tables and cache
contents; attention outputs within 2e-2 absolute and 1e-2 relative (both, see
parity_tools.py) and m, l within 1e-3 rel."""

import math
import queue
import types

import numpy as np
import pytest
import torch

from golden_io import load
from parity_tools import attention_close, describe
from oracle import attention as oa
from oracle import cache as oc
from oracle import insert as oi
from oracle import pages as op
from oracle.quant import quantize_decode, quantize_insert

pytestmark = pytest.mark.gpu

DEV = "cuda"
ATOL, RTOL = 2e-2, 1e-2


def cu(t):
  return t.to(DEV) if isinstance(t, torch.Tensor) else t


def same(a, b):
  return torch.equal(a.cpu(), b.cpu())


def close(a, b, atol=ATOL, rtol=RTOL):
  ok = attention_close(a, b, atol, rtol)
  if not ok:
    print(describe(a, b))
  return ok


def close_elementwise(a, b, atol, rtol):
  """|a - b| <= atol + rtol |b| per element: for scalars per row (m, l)."""
  return torch.allclose(a.float().cpu(), b.float().cpu(), atol=atol, rtol=rtol)


def make_env(**kw):
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  testing = kw.pop("testing", True)
  kv_quant = kw.pop("kv_quant", False)
  d = JetEngineEnvironmentData(testing=testing, **kw)
  d.quant_config.enable_kv_quantization = kv_quant
  return JetEngineEnvironment(d, device=DEV)


# ---------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------


def test_quantize_tensor_bit_exact_with_reference():
  from jetstream_pytorch_b200.quantize import quantize_tensor

  g = load("quantizers")
  for tag in ("bf16", "f32"):
    w = cu(g[f"insert_in_{tag}"])
    c, s, z = quantize_tensor(w, (-3, -1))
    assert z is None
    assert same(c, g[f"insert_codes_{tag}"]) and same(s, g[f"insert_scale_{tag}"])
    wt = w[0].permute(1, 0, 2).contiguous()
    c, s, _ = quantize_tensor(wt, (1, 2))
    assert same(c, g[f"insert_codes_t_{tag}"]) and same(s, g[f"insert_scale_t_{tag}"])


def test_decode_quantize_bit_exact_with_reference():
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = load("quantizers")
  env = make_env(batch_size=24, cache_shape=(24, 4, 8, 32))
  for tag in ("bf16", "f32"):
    x = cu(g[f"decode_in_{tag}"])
    cache = Int8KVCacheGenerate.empty((24, 4, 8, 32), DEV, env)
    c, s = cache.quantize(x)
    assert same(c, g[f"decode_codes_{tag}"]) and same(s, g[f"decode_scale_{tag}"])


@pytest.mark.parametrize("shape", [(96, 8, 1, 128), (8, 32, 1, 128), (5, 3, 1, 24), (7, 40, 1, 128)])
def test_decode_quantize_matches_oracle(shape):
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = torch.Generator().manual_seed(21)
  x = torch.randn(shape, generator=g).to(torch.bfloat16)
  x[1] = 0
  x[2] *= 1e-4
  env = make_env(batch_size=shape[0])
  cache = Int8KVCacheGenerate.empty((shape[0], shape[1], 4, shape[3]), DEV, env)
  c, s = cache.quantize(cu(x))
  oc_, os_ = quantize_decode(x)
  assert same(c, oc_) and same(s, os_)


# ---------------------------------------------------------------------------
# int8 dense cache
# ---------------------------------------------------------------------------

NAMES8 = ("ck", "cv", "kq", "vq", "ks", "vs", "kscale", "vscale")


def test_int8_update_ring_and_per_slot_bit_exact_with_reference():
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = load("int8_cache")
  xk, xv = cu(g["xk"]), cu(g["xv"])
  for mode, pos, ring in (("ring", [5], True), ("ring", torch.tensor([5]), True),
                          ("slot", g["slot_pos"], False), ("slot", g["slot_pos"].to(torch.int32), False)):
    env = make_env(batch_size=4, ring_buffer=ring)
    c = Int8KVCacheGenerate(cu(g["ring_in_ck"]).clone(), cu(g["ring_in_cv"]).clone(),
                            cu(g["ring_in_ks"]).clone(), cu(g["ring_in_vs"]).clone(), cu(pos), env=env)
    r = c.update(xk, xv, 1)
    assert r[0] is c.cache_k and r[4] is c.k_scaler
    for n, t in zip(NAMES8, r):
      assert same(t, g[f"{mode}_out_{n}"]), (mode, n)
      assert tuple(t.shape) == tuple(g[f"{mode}_out_{n}"].shape), (mode, n)


def test_int8_lazy_stacked_finalize_bit_exact_with_reference():
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = load("int8_cache")
  nl = g["lazy_xk"].shape[0]
  for new_stacked in (True, False):
    env = make_env(batch_size=4, ring_buffer=False, lazy_cache_update=True, generate_cache_stacked=True,
                   new_cache_stacked=new_stacked, num_layers=nl)
    c = Int8KVCacheGenerate(cu(g["lazy_in_ck"]).clone(), cu(g["lazy_in_cv"]).clone(),
                            cu(g["lazy_in_ks"]).clone(), cu(g["lazy_in_vs"]).clone(), cu(g["slot_pos"]), env=env)
    for layer in range(nl):
      r = c.update(cu(g["lazy_xk"][layer]), cu(g["lazy_xv"][layer]), layer)
      assert same(r[0], g["lazy_in_ck"])  # cache untouched until finalize
    if new_stacked:
      assert same(c.new_ks, g["lazy_new_ks"]) and same(c.new_k_scaler, g["lazy_new_k_scaler"])
    c.finalize()
    for n, t in zip(("ck", "cv", "ks", "vs"), (c.cache_k, c.cache_v, c.k_scaler, c.v_scaler)):
      assert same(t, g[f"lazy_out_{n}"]), n


def test_int8_lazy_unstacked_and_ring_lazy_match_oracle():
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = load("int8_cache")
  xk, xv, pos = g["xk"], g["xv"], g["slot_pos"]
  ins = [g[f"ring_in_{n}"] for n in ("ck", "cv", "ks", "vs")]
  env = make_env(batch_size=4, ring_buffer=False, lazy_cache_update=True)
  c = Int8KVCacheGenerate(*[cu(t).clone() for t in ins], cu(pos), env=env)
  c.update(cu(xk), cu(xv), 0)
  c.finalize()
  kq, ks = quantize_decode(xk)
  vq, vs = quantize_decode(xv)
  assert same(c.cache_k, oc.finalize_rows(ins[0], kq, pos)) and same(c.cache_v, oc.finalize_rows(ins[1], vq, pos))
  assert same(c.k_scaler, oc.finalize_rows(ins[2], ks, pos)) and same(c.v_scaler, oc.finalize_rows(ins[3], vs, pos))
  # ring + lazy: K/V written at finalize, scalers left alone (reference quirk)
  env = make_env(batch_size=4, ring_buffer=True, lazy_cache_update=True)
  c = Int8KVCacheGenerate(*[cu(t).clone() for t in ins], [9], env=env)
  c.update(cu(xk), cu(xv), 0)
  assert same(c.cache_k, ins[0])
  c.finalize()
  assert same(c.cache_k, oc.finalize_ring(ins[0], kq, 9)) and same(c.k_scaler, ins[2])


def test_int8_update_large_shapes_full_cache_equality():
  """Llama-2-70B-shaped slots (B=96, 8 KV heads, D=128): every byte of the cache
  and of the scalers equals the oracle's, including untouched rows."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = torch.Generator().manual_seed(31)
  b, h, s, d = 96, 8, 256, 128
  ck = torch.randint(-127, 128, (b, h, s, d), generator=g).to(torch.int8)
  cv = torch.randint(-127, 128, (b, h, s, d), generator=g).to(torch.int8)
  ks = torch.rand(b, 1, s, 1, generator=g).to(torch.bfloat16)
  vs = torch.rand(b, 1, s, 1, generator=g).to(torch.bfloat16)
  xk = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  pos = torch.randint(0, s, (b,), generator=g)
  env = make_env(batch_size=b, ring_buffer=False)
  c = Int8KVCacheGenerate(cu(ck), cu(cv), cu(ks), cu(vs), cu(pos), env=env)
  r = c.update(cu(xk), cu(xv), 0)
  exp = oc.int8_update(ck, cv, ks, vs, xk, xv, pos, ring_buffer=False, lazy=False)
  for n, t, e in zip(NAMES8, r, exp):
    assert same(t, e), n


def test_int8_update_head_sharded_two_phase_equals_unsharded():
  """KV heads split over two "ranks" (emulated on one GPU): local amax per
  rank, element-wise max (the all-reduce), update with the reduced amax.  Codes,
  scales and cache rows equal the unsharded oracle's slice."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  g = torch.Generator().manual_seed(33)
  b, h, s, d = 12, 8, 64, 128
  xk = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  xk[3] = 0
  pos = torch.randint(0, s, (b,), generator=g)
  ck = torch.zeros(b, h, s, d, dtype=torch.int8)
  sk = torch.ones(b, 1, s, 1, dtype=torch.bfloat16)
  exp = oc.int8_update(ck, ck, sk, sk, xk, xv, pos, ring_buffer=False, lazy=False)
  env = make_env(batch_size=b, ring_buffer=False)
  halves = [slice(0, 4), slice(4, 8)]
  caches = [Int8KVCacheGenerate(cu(ck[:, hs]).contiguous(), cu(ck[:, hs]).contiguous(), cu(sk).clone(),
                                cu(sk).clone(), cu(pos), env=env) for hs in halves]
  amax = [c.local_amax(cu(xk[:, hs]).contiguous(), cu(xv[:, hs]).contiguous()) for c, hs in zip(caches, halves)]
  red = torch.maximum(amax[0], amax[1])
  for c, hs in zip(caches, halves):
    r = c.update(cu(xk[:, hs]).contiguous(), cu(xv[:, hs]).contiguous(), 0, amax=red)
    assert same(r[0], exp[0][:, hs]) and same(r[1], exp[1][:, hs])
    assert same(r[2], exp[2][:, hs]) and same(r[3], exp[3][:, hs])
    assert same(r[4], exp[4]) and same(r[5], exp[5]) and same(r[6], exp[6]) and same(r[7], exp[7])


# ---------------------------------------------------------------------------
# bf16 / fp32 dense cache
# ---------------------------------------------------------------------------


def test_float_cache_bit_exact_with_reference():
  from jetstream_pytorch_b200.cache_manager import KVCacheGenerate

  g = load("float_cache")
  xk, xv, pos = cu(g["xk"]), cu(g["xv"]), cu(g["slot_pos"])
  env = make_env(batch_size=4, ring_buffer=True)
  c = KVCacheGenerate(cu(g["in_ck"]).clone(), cu(g["in_cv"]).clone(), [5], None, env=env)
  rk, rv = c.update(xk, xv, 0)
  assert same(rk, g["ring_out_ck"]) and same(rv, g["ring_out_cv"])
  env = make_env(batch_size=4, ring_buffer=False)
  c = KVCacheGenerate(cu(g["in_ck"]).clone(), cu(g["in_cv"]).clone(), pos, None, env=env)
  rk, rv = c.update(xk, xv, 0)
  assert same(rk, g["slot_out_ck"]) and same(rv, g["slot_out_cv"])
  env = make_env(batch_size=4, ring_buffer=False, generate_cache_stacked=True, num_layers=3)
  c = KVCacheGenerate(cu(g["stk_in_ck"]).clone(), cu(g["stk_in_cv"]).clone(), pos, None, env=env)
  c.update(xk, xv, 2)
  assert same(c.cache_k, g["stk_out_ck"]) and same(c.cache_v, g["stk_out_cv"])
  for new_stacked in (True, False):
    env = make_env(batch_size=4, ring_buffer=False, lazy_cache_update=True, generate_cache_stacked=True,
                   new_cache_stacked=new_stacked, num_layers=3)
    c = KVCacheGenerate(cu(g["stk_in_ck"]).clone(), cu(g["stk_in_cv"]).clone(), pos, None, env=env)
    for layer in range(3):
      c.update(cu(g["lazy_xk"][layer]), cu(g["lazy_xv"][layer]), layer)
    c.finalize()
    assert same(c.cache_k, g["lazy_out_ck"]) and same(c.cache_v, g["lazy_out_cv"])


def test_float32_cache_rows():
  from jetstream_pytorch_b200.cache_manager import KVCacheGenerate

  g = torch.Generator().manual_seed(32)
  ck, cv = torch.randn(3, 2, 10, 6, generator=g), torch.randn(3, 2, 10, 6, generator=g)
  xk, xv = torch.randn(3, 2, 1, 6, generator=g), torch.randn(3, 2, 1, 6, generator=g)
  pos = torch.tensor([9, 0, 4])
  env = make_env(batch_size=3, ring_buffer=False, bf16_enable=False)
  c = KVCacheGenerate(cu(ck), cu(cv), cu(pos), None, env=env)
  rk, rv = c.update(cu(xk), cu(xv), 0)
  assert same(rk, oc.append_per_slot(ck, xk, pos)) and same(rv, oc.append_per_slot(cv, xv, pos))


# ---------------------------------------------------------------------------
# pages
# ---------------------------------------------------------------------------


def test_pages_scenario_bit_exact_with_reference():
  from jetstream_pytorch_b200.cache_manager import KVCachePrefill, PageKVCacheGenerate
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = load("pages")
  _, p, ps, _ = g["in_ck"].shape
  b, maxp = g["after_insert_page_indices"].shape
  pam = PageAttentionManager(b, p, ps, maxp)
  ck, cv = cu(g["in_ck"]).clone(), cu(g["in_cv"]).clone()
  caches = [(ck, cv)]
  for i, (slot, length) in enumerate(g["inserts"].tolist()):
    pre = KVCachePrefill()
    pre.update(cu(g[f"prefix_k{i}"]), cu(g[f"prefix_v{i}"]), 0)
    n, idx = pam.reserve_pages_insert(slot, length)
    caches = pam.insert_prefill_cache([pre.state()], caches, idx, None, None)
  assert same(caches[0][0], g["after_insert_ck"]) and same(caches[0][1], g["after_insert_cv"])
  env = make_env(batch_size=b, ring_buffer=False, paged_attention_total_num_pages=p, paged_attention_page_size=ps)
  for step in range(3):
    lens = g[f"step{step}_lens"].numpy()
    pam.fill_new_pages(lens)
    # device-side table walk agrees with the host one
    pi_dev, _ = pam.device_tables(DEV)
    dpti, dn, dlen = pam.get_page_token_indices_device(cu(torch.as_tensor(lens, dtype=torch.int32)), pi_dev)
    pti = pam.get_page_token_indices(lens)
    n = int(dn.item())
    assert n == pti.shape[1]
    assert np.array_equal(dpti[:, :n].cpu().numpy(), pti)
    assert np.array_equal(dlen.cpu().numpy(), pam.lengths)
    c = PageKVCacheGenerate(caches[0][0], caches[0][1], pam, torch.as_tensor(pti), None, env=env)
    k, v = c.update(cu(g[f"step{step}_xk"]), cu(g[f"step{step}_xv"]))
    assert same(k, g[f"step{step}_ck"]) and same(v, g[f"step{step}_cv"])
  comp = pam.get_compress_kv_cache(caches, 5)
  assert same(comp[0][0], g["compress_slot5_k"])


def test_reference_known_answers_paged_cache_on_gpu():
  """tests/test_page_attention.py:48-145 and tests/test_kv_cache_manager.py:48-119
  of the reference, replayed through the CUDA path."""
  from jetstream_pytorch_b200.cache_manager import PageKVCacheGenerate
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  env = make_env(batch_size=5, ring_buffer=False, paged_attention_total_num_pages=20, paged_attention_page_size=4)
  pam = PageAttentionManager(3, 20, 4, 4)
  cache = PageKVCacheGenerate.empty((1, 6, 4, 2), DEV, env)
  k = torch.arange(6).reshape(1, 1, 3, 2).to(torch.bfloat16).to(DEV)
  _, idx = pam.reserve_pages_insert(0, 3)
  out = pam.insert_prefill_cache([(k, k)], [cache.state()], idx, None, None)
  assert out[0][0][0, 0].tolist() == [[0, 1], [2, 3], [4, 5], [0, 0]]
  assert out[0][1][0, 0].tolist() == [[0, 1], [2, 3], [4, 5], [0, 0]]

  pam = PageAttentionManager(3, 20, 4, 4)
  cache = PageKVCacheGenerate.empty((1, 20, 4, 2), DEV, env)
  k = torch.arange(12).reshape(1, 1, 6, 2).to(torch.bfloat16).to(DEV)
  _, idx = pam.reserve_pages_insert(0, 6)
  out = pam.insert_prefill_cache([(k, k)], [cache.state()], idx, None, None)
  exp = torch.arange(16)
  exp[12:] = 0
  assert torch.equal(out[0][0][:, :2].float().cpu(), exp.reshape(1, 2, 4, 2).float())
  assert not out[0][0][:, 2:].any()

  pam = PageAttentionManager(5, 20, 4, 4)
  cache = PageKVCacheGenerate.empty((1, 20, 4, 2), DEV, env)
  caches = [cache.state()]
  for length, slot in ((3, 0), (8, 1), (13, 3)):
    k = torch.arange(length * 2).reshape(1, 1, length, 2).to(torch.bfloat16).to(DEV)
    _, idx = pam.reserve_pages_insert(slot, length)
    caches = pam.insert_prefill_cache([(k, k)], caches, idx, None, None)
  lens = np.asarray([3, 8, 0, 13, 0])
  pam.fill_new_pages(lens)
  pti = pam.get_page_token_indices(lens)
  c = PageKVCacheGenerate(caches[0][0], caches[0][1], pam, torch.as_tensor(pti), None, env=env)
  xk = torch.arange(-1, -11, -1).reshape(5, 1, 1, 2).to(torch.bfloat16).to(DEV)
  kk, _ = c.update(xk, xk)
  assert kk[0, 0].tolist() == [[0, 1], [2, 3], [4, 5], [-1, -2]]
  assert kk[0, 7].tolist() == [[-3, -4], [0, 0], [0, 0], [0, 0]]
  assert kk[0, 6].tolist() == [[24, 25], [-7, -8], [0, 0], [0, 0]]


def test_paged_llama3_8b_shape_insert_append_exact():
  """Llama-3-8B paged shapes (8 KV heads, D=128, page 64) on a smaller pool:
  shuffled free list, 1024-token insert, one append per sequence; pools
  compared byte for byte with the oracle."""
  from jetstream_pytorch_b200.cache_manager import PageKVCacheGenerate
  from jetstream_pytorch_b200.insert import insert_page_attention_with_reservation
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = torch.Generator().manual_seed(41)
  b, h, p, ps, d, maxp = 8, 8, 192, 64, 128, 32
  order = torch.randperm(p, generator=g).tolist()
  pam = PageAttentionManager(b, p, ps, maxp, free_page_order=order)
  ora = op.PageTableOracle(b, p, ps, maxp, free_order=order)
  ck = torch.randn(h, p, ps, d, generator=g).to(torch.bfloat16)
  cv = torch.randn(h, p, ps, d, generator=g).to(torch.bfloat16)
  dk, dv = cu(ck).clone(), cu(cv).clone()
  lens = np.zeros(b, dtype=np.int64)
  for slot, length in ((0, 1024), (3, 700), (5, 64), (6, 1)):
    pk = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
    pv = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
    insert_page_attention_with_reservation(pam, [(cu(pk), cu(pv))], length, [(dk, dv)], slot)
    _, idx = ora.reserve_pages_insert(slot, length)
    ck, cv = oi.insert_paged(ck, pk, idx, ps), oi.insert_paged(cv, pv, idx, ps)
    lens[slot] = length
  assert same(dk, ck) and same(dv, cv)
  assert np.array_equal(pam.page_indices, ora.page_indices)
  env = make_env(batch_size=b, ring_buffer=False, paged_attention_total_num_pages=p, paged_attention_page_size=ps)
  for _ in range(2):
    pam.fill_new_pages(lens)
    ora.fill_new_pages(lens)
    pti = pam.get_page_token_indices(lens)
    assert np.array_equal(pti, ora.get_page_token_indices(lens))
    xk = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
    xv = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
    PageKVCacheGenerate(dk, dv, pam, pti, None, env=env).update(cu(xk), cu(xv))
    ck, cv = oc.paged_append(ck, xk, pti, ps), oc.paged_append(cv, xv, pti, ps)
    lens = np.where(lens == 0, 0, lens + 1)
  assert same(dk, ck) and same(dv, cv)
  # pool exhaustion surfaces as queue.Empty, like the reference
  big = cu(torch.zeros(1, h, 2048, d, dtype=torch.bfloat16))
  with pytest.raises(queue.Empty):
    for _ in range(p // 32 + 1):
      insert_page_attention_with_reservation(pam, [(big, big)], 2048, [(dk, dv)], 7)


def test_paged_int8_extension_insert_and_append_exact():
  from jetstream_pytorch_b200.cache_manager import PageKVCacheGenerate
  from jetstream_pytorch_b200.insert import insert_page_attention_with_reservation
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = torch.Generator().manual_seed(42)
  b, h, p, ps, d, maxp = 4, 8, 40, 64, 128, 8
  pam = PageAttentionManager(b, p, ps, maxp)
  ck = torch.zeros(h, p, ps, d, dtype=torch.int8)
  cv = torch.zeros(h, p, ps, d, dtype=torch.int8)
  sk = torch.ones(1, p, ps, 1, dtype=torch.bfloat16)
  sv = torch.ones(1, p, ps, 1, dtype=torch.bfloat16)
  dk, dv, dsk, dsv = cu(ck).clone(), cu(cv).clone(), cu(sk).clone(), cu(sv).clone()
  lens = np.zeros(b, dtype=np.int64)
  for slot, length in ((1, 300), (2, 128)):
    pk = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
    pv = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
    n_before = pam.unused_pages.qsize()
    insert_page_attention_with_reservation(pam, [(cu(pk), cu(pv))], length, [(dk, dv)], slot,
                                           cache_scales=[(dsk, dsv)])
    idx = pam.page_indices[slot, :n_before - pam.unused_pages.qsize()]
    ck, sk = oi.insert_paged_int8(ck, sk, pk, idx, ps)
    cv, sv = oi.insert_paged_int8(cv, sv, pv, idx, ps)
    lens[slot] = length
  assert same(dk, ck) and same(dsk, sk) and same(dv, cv) and same(dsv, sv)
  env = make_env(batch_size=b, ring_buffer=False, paged_attention_total_num_pages=p, paged_attention_page_size=ps)
  pam.fill_new_pages(lens)
  pti = pam.get_page_token_indices(lens)
  xk = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  PageKVCacheGenerate(dk, dv, pam, pti, None, env=env, k_scaler=dsk, v_scaler=dsv).update(cu(xk), cu(xv))
  kq, ks = quantize_decode(xk)
  vq, vs = quantize_decode(xv)
  ck, cv = oc.paged_append(ck, kq, pti, ps), oc.paged_append(cv, vq, pti, ps)
  sk, sv = oc.paged_append(sk, ks, pti, ps), oc.paged_append(sv, vs, pti, ps)
  assert same(dk, ck) and same(dsk, sk) and same(dv, cv) and same(dsv, sv)


# ---------------------------------------------------------------------------
# dense prefill insert
# ---------------------------------------------------------------------------


@pytest.mark.parametrize("int8", [False, True])
def test_paged_insert_of_stacked_layers_is_one_launch_with_the_same_result(int8):
  """Layers that are views of stacked tensors go through one launch
  (jpt_prefill_insert_paged with NL layers); separately allocated layers take a
  launch each.  Pools and scale pools must come out identical."""
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  nl, h, pages, ps, d, length = 3, 4, 12, 16, 128, 37
  g = torch.Generator().manual_seed(77)
  pre_k = cu(torch.randn(nl, 1, h, length, d, generator=g).to(torch.bfloat16))
  pre_v = cu(torch.randn(nl, 1, h, length, d, generator=g).to(torch.bfloat16))
  dt = torch.int8 if int8 else torch.bfloat16
  results = []
  for stacked in (True, False):
    if stacked:
      pk, pv = torch.zeros((nl, h, pages, ps, d), dtype=dt, device="cuda"), torch.zeros((nl, h, pages, ps, d), dtype=dt, device="cuda")
      sk, sv = (torch.zeros((nl, 1, pages, ps, 1), dtype=torch.bfloat16, device="cuda") for _ in range(2))
      pools = [(pk[i], pv[i]) for i in range(nl)]
      scales = [(sk[i], sv[i]) for i in range(nl)]
    else:
      pools = [(torch.zeros((h, pages, ps, d), dtype=dt, device="cuda"), torch.zeros((h, pages, ps, d), dtype=dt, device="cuda"))
               for _ in range(nl)]
      scales = [(torch.zeros((1, pages, ps, 1), dtype=torch.bfloat16, device="cuda"),
                 torch.zeros((1, pages, ps, 1), dtype=torch.bfloat16, device="cuda")) for _ in range(nl)]
      # fresh allocations may happen to lie at a constant step; in reverse order they never count as stacked
      pools, scales = pools[::-1], scales[::-1]
    pam = PageAttentionManager(4, pages, ps, 4)
    _, idx = pam.reserve_pages_insert(1, length)
    before = _lib.lib().jpt_launch_count()
    pam.insert_prefill_cache([(pre_k[i], pre_v[i]) for i in range(nl)], pools, idx, decode_scales=scales if int8 else None)
    torch.cuda.synchronize()
    results.append((_lib.lib().jpt_launch_count() - before, pools, scales))
  (n_one, pools_a, scales_a), (n_many, pools_b, scales_b) = results
  assert n_one == 1 and n_many == nl
  for (ka, va), (kb, vb) in zip(pools_a, pools_b):
    assert torch.equal(ka, kb) and torch.equal(va, vb)
  if int8:
    for (ka, va), (kb, vb) in zip(scales_a, scales_b):
      assert torch.equal(ka, kb) and torch.equal(va, vb)
    assert pools_a[1][0].abs().max() > 0


@pytest.mark.parametrize("quant", [False, True])
def test_dense_insert_no_wrap_and_wrap_match_oracle(quant):
  from jetstream_pytorch_b200.insert import insert_dense

  g = torch.Generator().manual_seed(51)
  b, h, s, d, length = 4, 8, 256, 128, 100
  prefix = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
  prefix[0, :, 7, :] = 0
  if quant:
    cache = torch.randint(-127, 128, (b, h, s, d), generator=g).to(torch.int8)
    scaler = torch.rand(b, 1, s, 1, generator=g).to(torch.bfloat16)
  else:
    cache = torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
    scaler = None
  for wrap, pos in ((False, 17), (False, 200), (False, -5), (True, 17), (True, 200), (True, 255)):
    dk, dv = cu(cache).clone(), cu(cache).clone()
    dsk = cu(scaler).clone() if quant else None
    dsv = cu(scaler).clone() if quant else None
    insert_dense(cu(prefix), cu(prefix), dk, dv, 2, pos, wrap=wrap, k_scaler=dsk, v_scaler=dsv)
    fn = oi.insert_wrap if wrap else oi.insert_no_wrap
    exp = fn(cache, prefix, 2, pos, scaler=scaler, quantize=quant)
    if quant:
      assert same(dk, exp[0]) and same(dv, exp[0]) and same(dsk, exp[1]) and same(dsv, exp[1]), (wrap, pos)
    else:
      assert same(dk, exp) and same(dv, exp), (wrap, pos)


def test_engine_insert_bookkeeping_and_stacked_int8():
  from jetstream_pytorch_b200.insert import insert

  g = torch.Generator().manual_seed(52)
  nl, b, h, s, d, lpad, seq_len = 2, 3, 2, 64, 16, 24, 20
  prefix = [(torch.randn(1, h, lpad, d, generator=g).to(torch.bfloat16),
             torch.randn(1, h, lpad, d, generator=g).to(torch.bfloat16)) for _ in range(nl)]
  # left aligned, stacked int8
  env = make_env(batch_size=b, ring_buffer=False, cache_sequence_length=s, num_layers=nl, testing=False,
                 kv_quant=True)
  ck = torch.zeros(nl, b, h, s, d, dtype=torch.int8)
  sk = torch.ones(nl, b, 1, s, 1, dtype=torch.bfloat16)
  dck, dcv, dsk, dsv = cu(ck).clone(), cu(ck).clone(), cu(sk).clone(), cu(sk).clone()
  mask = torch.full((b, s), float("-inf"), device=DEV)
  start = torch.zeros(b, dtype=torch.int32, device=DEV)
  ipos = torch.zeros(b, dtype=torch.int32, device=DEV)
  insert(env, [(cu(k), cu(v)) for k, v in prefix], seq_len, [(dck, dcv)], [(dsk, dsv)], 1, 0, mask=mask,
         start=start, input_pos=ipos)
  ek, esk, ev, esv = ck, sk, ck, sk
  for i, (pk, pv) in enumerate(prefix):
    ek, esk = oi.insert_no_wrap(ek, pk, 1, 0, layer=i, scaler=esk, quantize=True)
    ev, esv = oi.insert_no_wrap(ev, pv, 1, 0, layer=i, scaler=esv, quantize=True)
  assert same(dck, ek) and same(dcv, ev) and same(dsk, esk) and same(dsv, esv)
  assert same(mask[1], oi.insert_mask_row(s, 0, seq_len, False)) and int(ipos[1]) == seq_len
  # ring buffer, wrapping insert, bf16 unstacked
  env = make_env(batch_size=b, ring_buffer=True, cache_sequence_length=s, num_layers=nl)
  caches = [(torch.randn(b, h, s, d, generator=g).to(torch.bfloat16),
             torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)) for _ in range(nl)]
  dev_caches = [(cu(k).clone(), cu(v).clone()) for k, v in caches]
  cur = 10  # start_insert = -10 -> wraps
  insert(env, [(cu(k), cu(v)) for k, v in prefix], seq_len, dev_caches, None, 2, cur, mask=mask, start=start)
  for (k, v), (pk, pv), (dk, dv) in zip(caches, prefix, dev_caches):
    assert same(dk, oi.insert_wrap(k, pk, 2, (cur - seq_len) % s))
    assert same(dv, oi.insert_wrap(v, pv, 2, (cur - seq_len) % s))
  assert same(mask[2], oi.insert_mask_row(s, (cur - seq_len) % s, cur, True))
  assert int(start[2]) == (cur - seq_len) % s


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------


def test_dense_and_flash_attention_against_reference_outputs():
  from jetstream_pytorch_b200 import attention_kernel as ak

  g = load("attention")
  for tag, tol in (("bf16", (ATOL, RTOL)), ("f32", (1e-4, 1e-4))):
    for tq in (1, 2):
      pre = f"{tag}_t{tq}_"
      xq, k, v, mask = (cu(g[pre + n]) for n in ("xq", "k", "v", "mask"))
      kq, vq, ks, vs = (cu(g[pre + n]) for n in ("kq", "vq", "ks", "vs"))
      assert close(ak.dense_attention(xq, k, v, None, None, mask), g[pre + "dense_float"], *tol)
      assert close(ak.dense_attention(xq, kq, vq, ks, vs, mask), g[pre + "dense_int8"], *tol)
      o, (m, l) = ak.flash_attention(xq, k, v, 0, None, None, mask)
      assert close(o, g[pre + "flash_float_o"], *tol)
      assert close_elementwise(m, g[pre + "flash_float_m"], 1e-3, 1e-3) and close_elementwise(l, g[pre + "flash_float_l"], 1e-3, 1e-3)
      assert tuple(m.shape) == tuple(g[pre + "flash_float_m"].shape)
      o, (m, l) = ak.flash_attention(xq, kq, vq, 0, ks, vs, mask)
      assert close(o, g[pre + "flash_int8_o"], *tol)
      assert close_elementwise(m, g[pre + "flash_int8_m"], 1e-3, 1e-3) and close_elementwise(l, g[pre + "flash_int8_l"], 1e-3, 1e-3)


def _ragged_case(seed, b, hq, hkv, s, d, int8, ring, dtype=torch.bfloat16, tq=1):
  g = torch.Generator().manual_seed(seed)
  q = torch.randn(b, hq, tq, d, generator=g).to(dtype)
  k = torch.randn(b, hkv, s, d, generator=g).to(dtype)
  v = torch.randn(b, hkv, s, d, generator=g).to(dtype)
  ks = vs = None
  if int8:
    k, ks = quantize_insert(k, (-3, -1))
    v, vs = quantize_insert(v, (-3, -1))
  if ring:
    start = torch.randint(0, s, (b,), generator=g)
    end = torch.randint(0, s, (b,), generator=g)
    end[0] = start[0]  # empty row
    if b > 2:
      start[1], end[1] = s - 3, 2  # short wrap
      start[2], end[2] = 5, 4      # nearly full ring
  else:
    start = torch.zeros(b, dtype=torch.int64)
    end = torch.randint(1, s + 1, (b,), generator=g)
    end[0] = 0
    if b > 2:
      end[1], end[2] = 1, s
  return q, k, v, ks, vs, start, end


def _check_ragged(case, ring, **kw):
  from jetstream_pytorch_b200 import attention_kernel as ak

  q, k, v, ks, vs, start, end = case
  o, (m, l) = ak.ragged_mha(cu(q), cu(k), cu(v), 0, cu(start), cu(end), None, None, cu(ks), cu(vs), ring=ring, **kw)
  eo, (em, el) = oa.ragged_mha(q, k, v, 0, start, end, ks, vs, bk=min(512, k.shape[-2]), wrap=ring)
  assert tuple(o.shape) == tuple(eo.shape) and tuple(m.shape) == tuple(em.shape)
  assert close(o, eo)
  live = torch.isfinite(em)
  assert torch.equal(torch.isfinite(m.cpu()), live)
  assert torch.allclose(m.cpu()[live], em[live], atol=1e-3, rtol=1e-3)
  assert torch.allclose(l.cpu()[live], el[live], atol=1e-3, rtol=1e-3)
  assert not l.cpu()[~live].any() and not o.cpu()[~live].any()


@pytest.mark.parametrize("int8", [True, False])
@pytest.mark.parametrize("ring", [False, True])
@pytest.mark.parametrize("shape", [(5, 8, 2, 96, 16), (4, 4, 4, 70, 40), (3, 6, 2, 33, 128)])
def test_ragged_mha_small_shapes_match_oracle(int8, ring, shape):
  b, hq, hkv, s, d = shape
  _check_ragged(_ragged_case(61, b, hq, hkv, s, d, int8, ring), ring)


@pytest.mark.parametrize("splits", [1, 3, 8])
def test_ragged_mha_generic_kernel_splitk(splits):
  _check_ragged(_ragged_case(62, 4, 8, 2, 300, 64, True, True), True, num_splits=splits, force_generic=True)


@pytest.mark.parametrize("int8", [True, False])
@pytest.mark.parametrize("ring", [False, True])
@pytest.mark.parametrize("heads", [(64, 8), (32, 8), (32, 32), (16, 8), (32, 2), (24, 2)])
def test_ragged_mha_head_dim_128_matches_oracle(int8, ring, heads):
  hq, hkv = heads
  _check_ragged(_ragged_case(63, 6, hq, hkv, 512, 128, int8, ring), ring)


@pytest.mark.parametrize("kernel", [0, 2])
def test_ragged_mha_llama2_70b_shape_full_size(kernel):
  """The Llama-2-70B-shaped ragged decode at full size: B=96, 64 q / 8 kv heads, D=128, S=2048,
  int8 KV with per-token scales, left aligned and ring; through the tcgen05
  kernel (0) and the mma.sync kernel (2)."""
  for ring in (False, True):
    _check_ragged(_ragged_case(64, 96, 64, 8, 2048, 128, True, ring), ring, force_generic=kernel)


@pytest.mark.parametrize("int8", [True, False])
def test_ragged_fast_and_generic_kernels_agree(int8):
  from jetstream_pytorch_b200 import attention_kernel as ak

  q, k, v, ks, vs, start, end = _ragged_case(65, 8, 64, 8, 1024, 128, int8, True)
  args = (cu(q), cu(k), cu(v), 0, cu(start), cu(end), None, None, cu(ks), cu(vs))
  o1, (m1, l1) = ak.ragged_mha(*args, ring=True)
  o2, (m2, l2) = ak.ragged_mha(*args, ring=True, force_generic=True)
  assert close(o1, o2)
  live = torch.isfinite(m2)
  assert torch.allclose(m1[live], m2[live], atol=1e-3, rtol=1e-3)
  assert torch.allclose(l1[live], l2[live], atol=1e-3, rtol=1e-3)
  # force_generic=2: the mma.sync kernel where the tcgen05 one would have been picked (int8, <= 8 rows)
  o3, (m3, l3) = ak.ragged_mha(*args, ring=True, force_generic=2)
  assert close(o3, o2)
  assert torch.allclose(m3[live], m2[live], atol=1e-3, rtol=1e-3)
  assert torch.allclose(l3[live], l2[live], atol=1e-3, rtol=1e-3)


def test_ragged_mha_bf16_cache_llama3_8b_shape_full_size():
  """The Llama-3-8B attention shape with a dense bf16 cache: B=32, 32 q /
  8 kv heads, D=128, S=2048 (the paged form of it is covered further down)."""
  for ring in (False, True):
    _check_ragged(_ragged_case(67, 32, 32, 8, 2048, 128, False, ring), ring)


def test_ragged_mqa_per_head_entry_points_and_stacked_layout():
  from jetstream_pytorch_b200 import attention_kernel as ak

  q, k, v, ks, vs, start, end = _ragged_case(66, 4, 8, 2, 128, 128, True, True, tq=1)
  # stacked cache [NL,B,H,S,D], pick layer 1
  k5 = torch.stack([torch.zeros_like(k), k])
  v5 = torch.stack([torch.zeros_like(v), v])
  ks5 = torch.stack([torch.ones_like(ks), ks])
  vs5 = torch.stack([torch.ones_like(vs), vs])
  o, (m, l) = ak.ragged_mha(cu(q), cu(k5), cu(v5), 1, cu(start), cu(end), None, None, cu(ks5), cu(vs5))
  eo, (em, el) = oa.ragged_mha(q, k5, v5, 1, start, end, ks5, vs5, bk=128)
  assert close(o, eo)
  # one KV head through ragged_mqa (ring) and ragged_mqa_reference (left aligned)
  qg = q.reshape(4, 2, 4, 128)
  for h in range(2):
    o, (m, l) = ak.ragged_mqa(cu(qg[:, h]), cu(k[:, h]), cu(v[:, h]), 0, cu(start), cu(end),
                              k_scaler=cu(ks.squeeze(-1)), v_scaler=cu(vs.squeeze(-1)), quantized=True)
    eo, (em, el) = oa.ragged_mha(q, k, v, 0, start, end, ks, vs, bk=128, wrap=True)
    assert close(o, eo[:, h]) and tuple(m.shape) == (4, 4)
    o, _ = ak.ragged_mqa_reference(cu(qg[:, h]), cu(k[:, h]), cu(v[:, h]), 0, cu(start), cu(end),
                                   k_scaler=cu(ks.squeeze(-1)), v_scaler=cu(vs.squeeze(-1)), quantized=True)
    eo, _ = oa.ragged_mha(q, k, v, 0, start, end, ks, vs, bk=128, wrap=False)
    assert close(o, eo[:, h])


@pytest.mark.parametrize("int8", [False, True])
def test_dense_attention_decode_config1_shape(int8):
  """Llama-2-7B-shaped dense decode: batch 8, 32 heads (MHA), D=128, S=2048, q padded to
  two rows, causal-by-position mask."""
  from jetstream_pytorch_b200 import attention_kernel as ak

  g = torch.Generator().manual_seed(67)
  b, h, s, d = 8, 32, 2048, 128
  q = torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16)
  q = torch.nn.functional.pad(q, (0, 0, 0, 1))
  k = torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
  v = torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
  pos = torch.randint(0, s, (b,), generator=g)
  mask = torch.full((b, 1, 1, s), float("-inf"))
  for i in range(b):
    mask[i, :, :, :int(pos[i]) + 1] = 0
  mask = mask.to(torch.bfloat16)
  ks = vs = None
  if int8:
    k, ks = quantize_insert(k, (-3, -1))
    v, vs = quantize_insert(v, (-3, -1))
  o = ak.dense_attention(cu(q), cu(k), cu(v), cu(ks), cu(vs), cu(mask))
  eo = oa.dense_attention(q, k, v, ks, vs, mask)
  assert close(o[:, :, :1], eo[:, :, :1])


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("heads", [(32, 8), (8, 8), (4, 1)])
def test_paged_attention_matches_dense_equivalent(int8, heads):
  from jetstream_pytorch_b200 import attention_kernel as ak

  hq, hkv = heads
  g = torch.Generator().manual_seed(68)
  b, p, ps, d, maxp = 6, 64, 64, 128, 8
  kp = torch.randn(hkv, p, ps, d, generator=g).to(torch.bfloat16)
  vp = torch.randn(hkv, p, ps, d, generator=g).to(torch.bfloat16)
  ksp = vsp = None
  if int8:
    kp, ks = quantize_insert(kp.permute(1, 0, 2, 3).reshape(1, p, hkv, ps, d).permute(0, 2, 1, 3, 4).reshape(1, hkv, p * ps, d), (-3, -1))
    vp, vs = quantize_insert(vp.permute(1, 0, 2, 3).reshape(1, p, hkv, ps, d).permute(0, 2, 1, 3, 4).reshape(1, hkv, p * ps, d), (-3, -1))
    kp, vp = kp.reshape(hkv, p, ps, d), vp.reshape(hkv, p, ps, d)
    ksp, vsp = ks.reshape(1, p, ps, 1), vs.reshape(1, p, ps, 1)
  lengths = torch.tensor([1, 64, 65, 300, 512, 0])
  table = torch.randperm(p, generator=g)[:b * maxp].reshape(b, maxp).to(torch.int32)
  q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
  o = ak.call_paged_attention(None, cu(q), cu(kp), cu(vp), lengths.numpy(), table.numpy(), k_scaler=cu(ksp),
                              v_scaler=cu(vsp))
  eo = oa.paged_attention(q, kp, vp, lengths, table.numpy(), k_scale_pages=ksp, v_scale_pages=vsp)
  assert tuple(o.shape) == (b, hq, d)
  assert close(o, eo)
  o1 = ak.call_paged_attention(None, cu(q), cu(kp), cu(vp), cu(lengths), cu(table), sm_scale=1.0, k_scaler=cu(ksp),
                               v_scaler=cu(vsp))
  eo1 = oa.paged_attention(q, kp, vp, lengths, table.numpy(), sm_scale=1.0, k_scale_pages=ksp, v_scale_pages=vsp)
  assert close(o1, eo1)


def test_merge_partials_matches_reference_formula():
  from jetstream_pytorch_b200 import attention_kernel as ak

  g = torch.Generator().manual_seed(69)
  o1 = torch.randn(4, 8, 1, 128, generator=g).to(torch.bfloat16)
  o2 = torch.randn(4, 8, 1, 128, generator=g).to(torch.bfloat16)
  m1, m2 = torch.randn(4, 8, 1, 1, generator=g), torch.randn(4, 8, 1, 1, generator=g)
  l1, l2 = torch.rand(4, 8, 1, 1, generator=g) + 0.1, torch.rand(4, 8, 1, 1, generator=g) + 0.1
  m1[0], l1[0], o1[0] = -float("inf"), 0, 0  # an empty existing side passes the new side through
  out = ak.merge_partials(cu(o1), cu(m1), cu(l1), cu(o2), cu(m2), cu(l2))
  exp = oa.merge_partials(o1.float(), m1, l1, o2.float(), m2, l2)
  assert out.dtype == torch.float32
  assert torch.allclose(out.cpu()[1:], exp[1:], atol=1e-5, rtol=1e-5)
  assert torch.allclose(out.cpu()[0], o2[0].float(), atol=1e-6)


# ---------------------------------------------------------------------------
# the boundary callers, driven like the reference's tests drive them
# ---------------------------------------------------------------------------


@pytest.mark.parametrize("ring_buffer", [True, False])
def test_int8_attention_kernel_tracks_float_kernel(ring_buffer):
  """tests/test_quantization.py:155-284 of the reference (test_kv_kernel): the
  int8 caller and the float caller agree to 1e-2 on the same cache contents, in
  ring mode (dense attention) and in left-aligned lazy mode (ragged + flash +
  merge), at the reference's shapes [4,2,100,2], float32."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate, KVCacheGenerate
  from jetstream_pytorch_b200.layers import AttentionKernel, Int8KVAttentionKernel
  from jetstream_pytorch_b200.quantize import quantize_tensor

  g = torch.Generator().manual_seed(123)
  flags = dict(ring_buffer=ring_buffer, ragged_mha=not ring_buffer, flash_attention=not ring_buffer,
               generate_cache_stacked=not ring_buffer, new_cache_stacked=not ring_buffer,
               lazy_cache_update=not ring_buffer, batch_size=4, bf16_enable=False, num_layers=3, block_size=100)
  env = make_env(**flags)
  batch = 4
  shape = (3, batch, 2, 100, 2) if not ring_buffer else (batch, 2, 100, 2)
  cache_k = torch.randn(shape, generator=g).to(DEV)
  cache_v = torch.randn(shape, generator=g).to(DEV)
  start = torch.zeros(batch, dtype=torch.int32, device=DEV)
  # per-token quantisation of the existing cache over (heads, dim), batch by batch
  def quant(c):
    flat = c.reshape(-1, *c.shape[-3:])
    codes, scales = [], []
    for i in range(flat.shape[0]):
      q, s, _ = quantize_tensor(flat[i:i + 1].contiguous(), (-3, -1))
      codes.append(q)
      scales.append(s)
    codes = torch.cat(codes).reshape(c.shape)
    scales = torch.cat(scales).reshape(*c.shape[:-3], 1, c.shape[-2], 1)
    return codes, scales
  ck_i, ks_i = quant(cache_k)
  cv_i, vs_i = quant(cache_v)
  xq = torch.randn(batch, 2, 1, 2, generator=g).to(DEV)
  xk = torch.randn(batch, 2, 1, 2, generator=g).to(DEV)
  xv = torch.randn(batch, 2, 1, 2, generator=g).to(DEV)

  def get_var(position):
    pos = [position] if ring_buffer else torch.full((batch,), position, dtype=torch.int64, device=DEV)
    mask = torch.full((batch, 1, 1, 100), float("-inf"), device=DEV)
    mask[..., :position] = 0
    return pos, mask

  def run(attn, cache, layer, position):
    pos, mask = get_var(position)
    attn.layer_id = layer
    cache.input_pos = pos
    ret = attn(xq, xk, xv, mask, cache, start=start, end=pos if not ring_buffer else None)
    cache.finalize()
    return ret

  fcache = KVCacheGenerate(cache_k.clone(), cache_v.clone(), None, None, env)
  fattn = AttentionKernel(env, 0)
  float_res = [run(fattn, fcache, 1, 57), run(fattn, fcache, 1, 58), run(fattn, fcache, 2, 3)]
  env8 = make_env(kv_quant=True, **flags)
  icache = Int8KVCacheGenerate(ck_i, cv_i, ks_i, vs_i, None, None, env8)
  iattn = Int8KVAttentionKernel(env8, 0)
  int_res = [run(iattn, icache, 1, 57), run(iattn, icache, 1, 58), run(iattn, icache, 2, 3)]
  for f, i in zip(float_res, int_res):
    assert tuple(f.shape) == (batch, 2, 1, 2)
    assert torch.allclose(f.float(), i.float(), atol=0.01)


def test_int8_kv_cache_roundtrip_like_reference_test_kv_cache():
  """tests/test_quantization.py:72-153 of the reference (test_kv_cache):
  dequantised rows reproduce the inputs to 0.1 at the written positions."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate

  for ring in (True, False):
    flags = dict(ring_buffer=ring, generate_cache_stacked=not ring, new_cache_stacked=not ring,
                 lazy_cache_update=not ring, batch_size=4, num_layers=3, kv_quant=True)
    env = make_env(**flags)
    shape = (4, 2, 100, 2) if ring else (3, 4, 2, 100, 2)
    cache = Int8KVCacheGenerate.empty(shape, DEV, env)
    g = torch.Generator().manual_seed(7)
    k = torch.randn(4, 2, 1, 2, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(4, 2, 1, 2, generator=g).to(torch.bfloat16).to(DEV)
    for layer, pos in ((1, 57), (1, 58), (2, 3)):
      cache.input_pos = [pos] if ring else torch.full((4,), pos, device=DEV)
      cache.update(k, v, layer_id=layer)
      cache.finalize()
      new_k = cache.cache_k * cache.k_scaler
      new_v = cache.cache_v * cache.v_scaler
      if ring:
        assert torch.allclose(k.float(), new_k[:, :, pos:pos + 1].float(), atol=0.1)
        assert torch.allclose(v.float(), new_v[:, :, pos:pos + 1].float(), atol=0.1)
      else:
        assert torch.allclose(k.float(), new_k[layer, :, :, pos:pos + 1].float(), atol=0.1)
        assert torch.allclose(v.float(), new_v[layer, :, :, pos:pos + 1].float(), atol=0.1)


def test_attention_kernel_caller_against_oracle_decode_step():
  """One decode step through the boundary caller in every mode, against the
  oracle's composition of update + attention (+ merge): ring/dense (MHA
  shape family), left-aligned lazy ragged GQA, paged."""
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate, PageKVCacheGenerate
  from jetstream_pytorch_b200.layers import AttentionKernel, Int8KVAttentionKernel
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = torch.Generator().manual_seed(71)
  # --- ring, int8, MHA, dense attention with mask
  b, h, s, d = 4, 8, 256, 128
  ck, ks = quantize_insert(torch.randn(b, h, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  cv, vs = quantize_insert(torch.randn(b, h, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  xq, xk, xv = (torch.randn(b, h, 1, d, generator=g).to(torch.bfloat16) for _ in range(3))
  pos = 77
  mask = torch.full((b, 1, 1, s), float("-inf"))
  mask[..., :pos + 1] = 0
  mask = mask.to(torch.bfloat16)
  env = make_env(batch_size=b, ring_buffer=True, testing=False, kv_quant=True)
  cache = Int8KVCacheGenerate(cu(ck), cu(cv), cu(ks), cu(vs), [pos], env=env)
  out = Int8KVAttentionKernel(env, 0)(cu(xq), cu(xk), cu(xv), cu(mask), cache)
  e = oc.int8_update(ck, cv, ks, vs, xk, xv, [pos], ring_buffer=True, lazy=False)
  eo = oa.dense_attention(torch.nn.functional.pad(xq, (0, 0, 0, 1)), e[0], e[1], e[4], e[5], mask)[:, :, :1]
  assert same(cache.cache_k, e[0]) and same(cache.k_scaler, e[4])
  assert close(out, eo)
  # --- left aligned, lazy, stacked, int8, GQA ragged + flash + merge
  nl, b, hq, hkv, s, d = 2, 6, 32, 8, 512, 128
  ck5, ks5 = quantize_insert(torch.randn(nl * b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  cv5, vs5 = quantize_insert(torch.randn(nl * b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  ck5, cv5 = ck5.reshape(nl, b, hkv, s, d), cv5.reshape(nl, b, hkv, s, d)
  ks5, vs5 = ks5.reshape(nl, b, 1, s, 1), vs5.reshape(nl, b, 1, s, 1)
  xq = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  xk = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  ipos = torch.randint(1, s, (b,), generator=g)
  start = torch.zeros(b, dtype=torch.int64)
  env = make_env(batch_size=b, ring_buffer=False, testing=False, kv_quant=True, num_layers=nl)
  cache = Int8KVCacheGenerate(cu(ck5).clone(), cu(cv5).clone(), cu(ks5).clone(), cu(vs5).clone(), cu(ipos), env=env)
  out = Int8KVAttentionKernel(env, 1)(cu(xq), cu(xk), cu(xv), None, cache, start=cu(start), end=cu(ipos))
  cache.finalize()
  eo1, (em1, el1) = oa.ragged_mha(xq, ck5, cv5, 1, start, ipos, ks5, vs5)
  kq, ksn = quantize_decode(xk)
  vq, vsn = quantize_decode(xv)
  eo2, (em2, el2) = oa.flash_attention(xq, kq, vq, 1, ksn, vsn, None)
  exp = oa.merge_partials(eo1.reshape(b, hq, 1, d).float(), em1.reshape(b, hq, 1, 1), el1.reshape(b, hq, 1, 1),
                          eo2.float(), em2, el2)
  assert close(out, exp)
  assert same(cache.cache_k[1], oc.finalize_rows(ck5, torch.stack([torch.zeros_like(kq), kq]), ipos)[1])
  # --- paged, bf16, GQA
  b, hq, hkv, p, ps, d, maxp = 4, 32, 8, 48, 64, 128, 8
  pam = PageAttentionManager(b, p, ps, maxp)
  kp = torch.randn(hkv, p, ps, d, generator=g).to(torch.bfloat16)
  vp = torch.randn(hkv, p, ps, d, generator=g).to(torch.bfloat16)
  lens = np.asarray([100, 0, 64, 255])
  for slot in range(b):
    if lens[slot]:
      pam.reserve_pages_insert(slot, int(lens[slot]))
  pam.fill_new_pages(lens)
  pti = pam.get_page_token_indices(lens)
  env = make_env(batch_size=b, ring_buffer=False, testing=False, paged_attention_total_num_pages=p,
                 paged_attention_page_size=ps)
  cache = PageKVCacheGenerate(cu(kp).clone(), cu(vp).clone(), pam, pti, None, env=env)
  xq = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  xk = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  xv = torch.randn(b, hkv, 1, d, generator=g).to(torch.bfloat16)
  out = AttentionKernel(env, 0)(cu(xq), cu(xk), cu(xv), None, cache)
  ek, ev = oc.paged_append(kp, xk, pti, ps), oc.paged_append(vp, xv, pti, ps)
  eo = oa.paged_attention(xq[:, :, 0], ek, ev, pam.lengths, pam.page_indices)
  assert same(cache.cache_k, ek)
  assert close(out[:, :, 0], eo)


def test_attention_kernels_never_gave_up_on_a_wait():
  """Runs after the attention tests of this file: the bounded waits inside the
  persistent kernel must never have timed out."""
  from jetstream_pytorch_b200 import attention_kernel as ak

  q, k, v, ks, vs, start, end = _ragged_case(70, 4, 32, 8, 256, 128, True, True)
  ak.ragged_mha(cu(q), cu(k), cu(v), 0, cu(start), cu(end), None, None, cu(ks), cu(vs), ring=True)
  assert ak.kernel_status() == 0


def test_argument_errors_are_reported_not_launched():
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.insert import insert_dense

  q = torch.zeros(2, 6, 1, 128, dtype=torch.bfloat16, device=DEV)
  k = torch.zeros(2, 4, 64, 128, dtype=torch.bfloat16, device=DEV)
  with pytest.raises(ValueError):
    ak.dense_attention(q, k, k)  # 6 query heads over 4 KV heads
  # masks that do not broadcast against the grouped scores [B,Hkv,rep*Tq,S] are refused before the launch
  q2 = torch.zeros(2, 8, 2, 128, dtype=torch.bfloat16, device=DEV)  # rep 2, Tq 2: 4 rows per KV head
  for bad in ((2, 1, 2, 64), (3, 1, 1, 64), (2, 1, 3, 64), (2, 2, 4, 64), (2, 1, 4, 63)):
    with pytest.raises(ValueError):
      ak.dense_attention(q2, k, k, mask=torch.zeros(bad, dtype=torch.bfloat16, device=DEV))
  ak.dense_attention(q2, k, k, mask=torch.zeros((1, 1, 4, 64), dtype=torch.bfloat16, device=DEV))
  cache = torch.zeros(2, 4, 64, 128, dtype=torch.int8, device=DEV)
  pre = torch.zeros(1, 4, 100, 128, dtype=torch.bfloat16, device=DEV)
  sc = torch.ones(2, 1, 64, 1, dtype=torch.bfloat16, device=DEV)
  with pytest.raises(ValueError):
    insert_dense(pre, pre, cache, cache.clone(), 0, 0, k_scaler=sc, v_scaler=sc.clone())  # L > S without wrap
