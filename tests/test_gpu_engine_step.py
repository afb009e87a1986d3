"""The decode step around the KV cache (`jetstream_pytorch_b200.engine`):
bookkeeping against what the reference's `generate_impl` produced, and whole
decode steps (cache objects, attention callers, paged driver with device-side
page indices) against the oracle's composition."""

import numpy as np
import pytest
import torch

from golden_io import load
from oracle import attention as oa
from oracle import cache as oc
from oracle import pages as op
from oracle.quant import quantize_decode, quantize_insert
from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu

DEV = "cuda"


def make_env(**kw):
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  kv_quant = kw.pop("kv_quant", False)
  d = JetEngineEnvironmentData(testing=True, **kw)
  d.quant_config.enable_kv_quantization = kv_quant
  return JetEngineEnvironment(d, device=DEV)


@pytest.mark.parametrize("name", ["ring", "left"])
def test_generate_bookkeeping_bit_exact_with_reference(name):
  from jetstream_pytorch_b200.engine import DecodeState, KVCacheEngine

  g = load("engine_step")
  b, s, bk, vocab, steps = (int(v) for v in g["geometry"])
  ring = name == "ring"
  env = make_env(batch_size=b, cache_sequence_length=s, block_size=bk, num_layers=1, ring_buffer=ring,
                 lazy_cache_update=not ring, cache_shape=(b, 1, s, 8))
  seen = []

  def model(params, tokens, input_pos, caches, mask, start, rbi, rbk):
    seen.append((mask.clone(), rbi.clone(), rbk.clone(), caches[0].input_pos))
    new = torch.zeros(b, 1, 1, 8, dtype=torch.bfloat16, device=DEV)
    caches[0].update(new, new, 0)  # every layer of a real model does this once per step
    logits = torch.zeros(b, 1, vocab, device=DEV)
    logits[torch.arange(b), 0, (tokens[:, 0].long() * 3 + 1) % vocab] = 1
    return logits

  engine = KVCacheEngine(env, model)
  state = engine.init_decode_state()
  state = DecodeState(g[f"{name}_in_tokens"].to(DEV), state.caches, state.cache_scales,
                      int(g[f"{name}_in_current_position"]), g[f"{name}_in_lens"].to(DEV),
                      g[f"{name}_in_start"].to(DEV), g[f"{name}_in_input_pos"].to(DEV),
                      g[f"{name}_in_mask"].to(DEV).to(torch.bfloat16))
  for step in range(steps):
    pre = f"{name}_step{step}_"
    state, data = engine.generate(None, state)
    mask, rbi, rbk, idx = seen[-1]
    assert torch.equal(mask.float().cpu().reshape(b, s), g[pre + "model_mask"].reshape(b, s))
    assert torch.equal(rbi.cpu().long(), g[pre + "ragged_batch_index"].long())
    assert torch.equal(rbk.cpu().long(), g[pre + "ragged_block_index"].long())
    want_idx = g[pre + "model_input_indexes"].reshape(-1).long()
    got_idx = torch.as_tensor(idx).reshape(-1).long().cpu()
    assert torch.equal(got_idx, want_idx)
    assert torch.equal(state.tokens.cpu(), g[pre + "tokens"]) and torch.equal(state.lens.cpu(), g[pre + "lens"])
    assert torch.equal(state.input_pos.cpu(), g[pre + "input_pos"])
    assert torch.equal(state.mask.float().cpu(), g[pre + "mask"])
    assert state.current_position == int(g[pre + "current_position"])
    assert torch.equal(data.cpu(), g[pre + "data"])


def test_left_aligned_int8_decode_steps_match_oracle():
  """Insert two prompts, then three decode steps of a one-layer "model" (the
  int8 attention caller over a stacked lazy cache): caches, scalers, positions
  and attention outputs against the oracle's composition."""
  from jetstream_pytorch_b200.engine import KVCacheEngine, Prefix
  from jetstream_pytorch_b200.layers import Int8KVAttentionKernel
  from oracle import insert as oi

  gen = torch.Generator().manual_seed(301)
  b, hq, hkv, s, d, vocab = 4, 16, 4, 256, 128, 50
  env = make_env(batch_size=b, cache_sequence_length=s, block_size=128, num_layers=1, ring_buffer=False,
                 lazy_cache_update=True, ragged_mha=True, flash_attention=True, generate_cache_stacked=True,
                 new_cache_stacked=True, cache_shape=(b, hkv, s, d), kv_quant=True)
  eq = torch.randn(vocab, hq * d, generator=gen).to(torch.bfloat16)
  ek = torch.randn(vocab, hkv * d, generator=gen).to(torch.bfloat16)
  ev = torch.randn(vocab, hkv * d, generator=gen).to(torch.bfloat16)
  deq, dek, dev_ = eq.to(DEV), ek.to(DEV), ev.to(DEV)
  outs = []

  def model(params, tokens, input_pos, caches, mask, start, rbi, rbk):
    t = tokens[:, 0].long()
    xq, xk, xv = deq[t].reshape(b, hq, 1, d), dek[t].reshape(b, hkv, 1, d), dev_[t].reshape(b, hkv, 1, d)
    o = Int8KVAttentionKernel(env, 0)(xq, xk, xv, mask, caches[0], start=start, end=input_pos,
                                      ragged_batch_index=rbi, ragged_block_index=rbk)
    outs.append(o)
    return o.reshape(b, 1, hq * d)[..., :vocab].float()

  engine = KVCacheEngine(env, model)
  state = engine.init_decode_state()
  ck = torch.zeros(1, b, hkv, s, d, dtype=torch.int8)
  cv = torch.zeros(1, b, hkv, s, d, dtype=torch.int8)
  ks = torch.ones(1, b, 1, s, 1, dtype=torch.bfloat16)
  vs = torch.ones(1, b, 1, s, 1, dtype=torch.bfloat16)
  ipos = np.zeros(b, dtype=np.int64)
  tokens = np.zeros((b, 1), dtype=np.int64)
  for slot, length, tok in ((1, 100, 7), (3, 129, 11)):
    pk = torch.randn(1, hkv, length, d, generator=gen).to(torch.bfloat16)
    pv = torch.randn(1, hkv, length, d, generator=gen).to(torch.bfloat16)
    state = engine.insert(Prefix(torch.tensor([[tok]]), [(pk.to(DEV), pv.to(DEV))], length), state, slot)
    ck, ks = oi.insert_no_wrap(ck, pk, slot, 0, layer=0, scaler=ks, quantize=True)
    cv, vs = oi.insert_no_wrap(cv, pv, slot, 0, layer=0, scaler=vs, quantize=True)
    ipos[slot], tokens[slot] = length, tok
  assert torch.equal(state.caches[0][0].cpu(), ck) and torch.equal(state.cache_scales[0][0].cpu(), ks)
  start = torch.zeros(b, dtype=torch.int64)
  for step in range(3):
    state, _ = engine.generate(None, state)
    t = torch.as_tensor(tokens[:, 0])
    xq, xk, xv = eq[t].reshape(b, hq, 1, d), ek[t].reshape(b, hkv, 1, d), ev[t].reshape(b, hkv, 1, d)
    end = torch.as_tensor(ipos)
    o1, (m1, l1) = oa.ragged_mha(xq, ck, cv, 0, start, end, ks, vs, bk=128)
    kq, ksn = quantize_decode(xk)
    vq, vsn = quantize_decode(xv)
    o2, (m2, l2) = oa.flash_attention(xq, kq, vq, 0, ksn, vsn, None)
    exp = oa.merge_partials(o1.reshape(b, hq, 1, d).float(), m1.reshape(b, hq, 1, 1), l1.reshape(b, hq, 1, 1),
                            o2.float(), m2, l2)
    active = ipos > 0
    assert attention_close(outs[-1][active], exp[active]), describe(outs[-1][active], exp[active])
    # lazy finalize writes every slot's row at its input_pos (idle slots: position 0)
    ck = oc.finalize_rows(ck, kq.unsqueeze(0), end)
    cv = oc.finalize_rows(cv, vq.unsqueeze(0), end)
    ks = oc.finalize_rows(ks, ksn.unsqueeze(0), end)
    vs = oc.finalize_rows(vs, vsn.unsqueeze(0), end)
    assert torch.equal(state.caches[0][0].cpu(), ck) and torch.equal(state.caches[0][1].cpu(), cv), f"step {step}"
    assert torch.equal(state.cache_scales[0][0].cpu(), ks) and torch.equal(state.cache_scales[0][1].cpu(), vs)
    logits = exp.reshape(b, 1, hq * d)[..., :vocab]
    tokens = state.tokens.cpu().numpy().astype(np.int64)  # follow the GPU's argmax (ties aside, checked below)
    ipos = np.where(ipos == 0, 0, ipos + 1)
    assert np.array_equal(state.input_pos.cpu().numpy(), ipos)
    top = logits[:, 0].float().topk(2, dim=-1)
    clear = (top.values[:, 0] - top.values[:, 1]) > 0.05  # only where the oracle's argmax is not a near tie
    assert np.array_equal(tokens[clear.numpy() & active, 0], top.indices[:, 0].numpy()[clear.numpy() & active])


def test_paged_decode_steps_with_device_side_indices_match_host_path():
  """`generate_page_attention` computes the (page, offset, slot) triples on the
  device and keeps reservation on the host without reading the GPU.  Pools,
  tables and attention must equal the reference's host-driven sequence
  (fill_new_pages -> get_page_token_indices -> update -> paged attention) step
  by step, including steps that cross a page boundary."""
  from jetstream_pytorch_b200.engine import KVCacheEngine, Prefix
  from jetstream_pytorch_b200.layers import AttentionKernel
  from oracle import insert as oi

  gen = torch.Generator().manual_seed(302)
  b, hq, hkv, d, ps, p, vocab, s = 4, 16, 4, 128, 16, 64, 50, 128
  env = make_env(batch_size=b, cache_sequence_length=s, num_layers=1, ring_buffer=False,
                 paged_attention_total_num_pages=p, paged_attention_page_size=ps, cache_shape=(hkv, p, ps, d))
  eq = torch.randn(vocab, hq * d, generator=gen).to(torch.bfloat16)
  ek = torch.randn(vocab, hkv * d, generator=gen).to(torch.bfloat16)
  ev = torch.randn(vocab, hkv * d, generator=gen).to(torch.bfloat16)
  deq, dek, dev_ = eq.to(DEV), ek.to(DEV), ev.to(DEV)
  outs = []

  def model(params, tokens, input_pos, caches, mask, start, rbi, rbk):
    t = tokens[:, 0].long()
    xq, xk, xv = deq[t].reshape(b, hq, 1, d), dek[t].reshape(b, hkv, 1, d), dev_[t].reshape(b, hkv, 1, d)
    o = AttentionKernel(env, 0)(xq, xk, xv, mask, caches[0], start=start, end=input_pos)
    outs.append(o)
    return o.reshape(b, 1, hq * d)[..., :vocab].float()

  engine = KVCacheEngine(env, model)
  state = engine.init_decode_state()
  ora = op.PageTableOracle(b, p, ps, s // ps)
  ck, cv = state.caches[0][0].cpu().clone(), state.caches[0][1].cpu().clone()
  lens = np.zeros(b, dtype=np.int64)
  tokens = np.zeros((b, 1), dtype=np.int64)
  for slot, length, tok in ((0, 15, 3), (2, 31, 9), (3, 40, 21)):
    pk = torch.randn(1, hkv, length, d, generator=gen).to(torch.bfloat16)
    pv = torch.randn(1, hkv, length, d, generator=gen).to(torch.bfloat16)
    state = engine.insert(Prefix(torch.tensor([[tok]]), [(pk.to(DEV), pv.to(DEV))], length), state, slot)
    _, idx = ora.reserve_pages_insert(slot, length)
    ck, cv = oi.insert_paged(ck, pk, idx, ps), oi.insert_paged(cv, pv, idx, ps)
    lens[slot], tokens[slot] = length, tok
  for step in range(3):  # slots 0 and 2 cross a page boundary at step 1
    state, _ = engine.generate(None, state)
    ora.fill_new_pages(lens)
    pti = ora.get_page_token_indices(lens)
    t = torch.as_tensor(tokens[:, 0])
    xq, xk, xv = eq[t].reshape(b, hq, 1, d), ek[t].reshape(b, hkv, 1, d), ev[t].reshape(b, hkv, 1, d)
    ck, cv = oc.paged_append(ck, xk, pti, ps), oc.paged_append(cv, xv, pti, ps)
    exp = oa.paged_attention(xq[:, :, 0], ck, cv, ora.lengths, ora.page_indices)
    assert torch.equal(state.caches[0][0].cpu(), ck) and torch.equal(state.caches[0][1].cpu(), cv), f"step {step}"
    assert np.array_equal(engine.page_attention_manager.page_indices, ora.page_indices)
    assert np.array_equal(np.asarray(engine.page_attention_manager.lengths), ora.lengths)
    active = lens > 0
    got = outs[-1][:, :, 0]
    assert attention_close(got[active], exp[active]), describe(got[active], exp[active])
    lens = np.where(lens == 0, 0, lens + 1)
    assert np.array_equal(state.input_pos.cpu().numpy(), lens)
    tokens = state.tokens.cpu().numpy().astype(np.int64)
