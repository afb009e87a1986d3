"""GPU parity at the sizes the benchmark configurations state: the paged bf16
Llama-3-8B-shaped decode step (batch 32, 4096-page pool) and the int8 paged
prefill-insert burst (32 stacked layers, batch-128 pool)."""

import numpy as np
import pytest
import torch

from oracle import attention as oa
from oracle import cache as oc
from oracle import insert as oi
from oracle import pages as op
from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu

DEV = "cuda"


def test_paged_bf16_llama3_8b_step_at_full_size():
  """B=32, 32 q / 8 kv heads, D=128, page 64, 4096-page pool per layer,
  lengths uniform in [1, 2048], page tables from a seeded shuffled free list;
  a 1024-token prefill insert into the free slot, one decode append per
  sequence, then paged attention (both softmax-scale conventions).  Pools are
  compared byte for byte, attention within tolerance."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import PageKVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData
  from jetstream_pytorch_b200.insert import insert_page_attention_with_reservation
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  b, hq, hkv, d, ps, p, maxp = 32, 32, 8, 128, 64, 4096, 33
  rng = np.random.RandomState(1001)
  order = rng.permutation(p).tolist()
  lens0 = rng.randint(1, 2049, size=b)
  free_slot = 17
  lens0[free_slot] = 0
  pam = PageAttentionManager(b, p, ps, maxp, free_page_order=order)
  ora = op.PageTableOracle(b, p, ps, maxp, free_order=order)
  for slot in range(b):
    if lens0[slot]:
      pam.reserve_pages_insert(slot, int(lens0[slot]))
      ora.reserve_pages_insert(slot, int(lens0[slot]))
  gen = torch.Generator(device=DEV).manual_seed(1001)
  dk = torch.randn((hkv, p, ps, d), generator=gen, device=DEV).to(torch.bfloat16)
  dv = torch.randn((hkv, p, ps, d), generator=gen, device=DEV).to(torch.bfloat16)
  ck, cv = dk.cpu(), dv.cpu()
  pk = torch.randn((1, hkv, 1024, d), generator=gen, device=DEV).to(torch.bfloat16)
  pv = torch.randn((1, hkv, 1024, d), generator=gen, device=DEV).to(torch.bfloat16)
  insert_page_attention_with_reservation(pam, [(pk, pv)], 1024, [(dk, dv)], free_slot)
  _, idx = ora.reserve_pages_insert(free_slot, 1024)
  ck, cv = oi.insert_paged(ck, pk.cpu(), idx, ps), oi.insert_paged(cv, pv.cpu(), idx, ps)
  lens = lens0.copy()
  lens[free_slot] = 1024
  assert np.array_equal(pam.page_indices, ora.page_indices)
  # one decode step: page reservation on boundaries, index walk, append
  pam.fill_new_pages(lens)
  ora.fill_new_pages(lens)
  pti = pam.get_page_token_indices(lens)
  assert np.array_equal(pti, ora.get_page_token_indices(lens))
  xk = torch.randn((b, hkv, 1, d), generator=gen, device=DEV).to(torch.bfloat16)
  xv = torch.randn((b, hkv, 1, d), generator=gen, device=DEV).to(torch.bfloat16)
  data = JetEngineEnvironmentData(batch_size=b, ring_buffer=False, testing=True, paged_attention_total_num_pages=p,
                                  paged_attention_page_size=ps)
  env = JetEngineEnvironment(data, device=DEV)
  PageKVCacheGenerate(dk, dv, pam, pti, None, env=env).update(xk, xv)
  ck, cv = oc.paged_append(ck, xk.cpu(), pti, ps), oc.paged_append(cv, xv.cpu(), pti, ps)
  assert torch.equal(dk.cpu(), ck) and torch.equal(dv.cpu(), cv), "pools differ from the oracle's after insert + append"
  assert np.array_equal(np.asarray(pam.lengths), ora.lengths)
  q = torch.randn((b, hq, d), generator=gen, device=DEV).to(torch.bfloat16)
  for sm_scale in (None, 1.0):
    o = ak.call_paged_attention(env, q, dk, dv, pam.lengths, pam.page_indices, sm_scale=sm_scale)
    eo = oa.paged_attention(q.cpu(), ck, cv, ora.lengths, ora.page_indices, sm_scale=sm_scale)
    assert attention_close(o, eo), describe(o, eo)


def test_int8_paged_insert_burst_of_stacked_layers_at_full_size():
  """Four inserts of L in {2048, 128} x 32 stacked layers into the int8 paged
  pool of a batch of 128 (8 KV heads, D=128, page 64, 4096 pages per layer):
  one launch per insert.  The oracle runs on a compact pool that holds only
  the pages the inserts touch (its semantics are per page index); every other
  page of the GPU pools must still hold its initial pattern."""
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  nl, bsz, hkv, d, ps, maxp = 32, 128, 8, 128, 64, 32
  p = bsz * maxp
  rng = np.random.RandomState(1004)
  pam = PageAttentionManager(bsz, p, ps, maxp, free_page_order=rng.permutation(p).tolist())
  pool_k = torch.full((nl, hkv, p, ps, d), 7, dtype=torch.int8, device=DEV)
  pool_v = torch.full((nl, hkv, p, ps, d), 7, dtype=torch.int8, device=DEV)
  sc_k = torch.ones((nl, 1, p, ps, 1), dtype=torch.bfloat16, device=DEV)
  sc_v = torch.ones((nl, 1, p, ps, 1), dtype=torch.bfloat16, device=DEV)
  pools = [(pool_k[i], pool_v[i]) for i in range(nl)]
  scales = [(sc_k[i], sc_v[i]) for i in range(nl)]
  gen = torch.Generator(device=DEV).manual_seed(1004)
  lengths = [2048, 128, 2048, 128]
  slots = rng.choice(bsz, size=len(lengths), replace=False)
  touched, plan = [], []
  for length, slot in zip(lengths, slots):
    pre_k = torch.randn((nl, 1, hkv, length, d), generator=gen, device=DEV).to(torch.bfloat16)
    pre_v = torch.randn((nl, 1, hkv, length, d), generator=gen, device=DEV).to(torch.bfloat16)
    _, idx = pam.reserve_pages_insert(int(slot), length)
    idx = np.asarray(idx).copy()
    before = _lib.lib().jpt_launch_count()
    pam.insert_prefill_cache([(pre_k[i], pre_v[i]) for i in range(nl)], pools, idx, decode_scales=scales)
    assert _lib.lib().jpt_launch_count() - before == 1, "stacked layers must go through one launch"
    plan.append((pre_k.cpu(), pre_v.cpu(), idx, len(touched)))
    touched += idx.tolist()
  torch.cuda.synchronize()
  touched_t = torch.as_tensor(touched, device=DEV)
  for layer in range(nl):
    ek = torch.full((hkv, len(touched), ps, d), 7, dtype=torch.int8)
    ev = ek.clone()
    esk = torch.ones((1, len(touched), ps, 1), dtype=torch.bfloat16)
    esv = esk.clone()
    for pre_k, pre_v, idx, base in plan:
      local = np.arange(base, base + len(idx))
      ek, esk = oi.insert_paged_int8(ek, esk, pre_k[layer], local, ps)
      ev, esv = oi.insert_paged_int8(ev, esv, pre_v[layer], local, ps)
    assert torch.equal(pool_k[layer][:, touched_t].cpu(), ek), f"layer {layer}: K codes"
    assert torch.equal(pool_v[layer][:, touched_t].cpu(), ev), f"layer {layer}: V codes"
    assert torch.equal(sc_k[layer][:, touched_t].cpu(), esk), f"layer {layer}: K scales"
    assert torch.equal(sc_v[layer][:, touched_t].cpu(), esv), f"layer {layer}: V scales"
  untouched = torch.ones(p, dtype=torch.bool, device=DEV)
  untouched[touched_t] = False
  for layer in range(nl):
    assert bool((pool_k[layer][:, untouched] == 7).all()) and bool((pool_v[layer][:, untouched] == 7).all())
    assert bool((sc_k[layer][:, untouched] == 1).all()) and bool((sc_v[layer][:, untouched] == 1).all())
