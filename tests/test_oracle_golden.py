"""The CPU oracle against vectors produced by the reference's own code
(tests/golden/make_golden.py) and against the reference's known-answer tests."""

import numpy as np
import torch

from golden_io import load
from oracle import attention as oa
from oracle import cache as oc
from oracle import insert as oi
from oracle import pages as op
from oracle.quant import quantize_decode, quantize_insert


def test_quantizers_bit_exact():
  g = load("quantizers")
  for tag in ("bf16", "f32"):
    c, s = quantize_insert(g[f"insert_in_{tag}"], (-3, -1))
    assert torch.equal(c, g[f"insert_codes_{tag}"])
    assert torch.equal(s, g[f"insert_scale_{tag}"])
    wt = g[f"insert_in_{tag}"][0].permute(1, 0, 2).contiguous()
    c, s = quantize_insert(wt, (1, 2))
    assert torch.equal(c, g[f"insert_codes_t_{tag}"])
    assert torch.equal(s, g[f"insert_scale_t_{tag}"])
    c, s = quantize_decode(g[f"decode_in_{tag}"])
    assert torch.equal(c, g[f"decode_codes_{tag}"])
    assert torch.equal(s, g[f"decode_scale_{tag}"])


def test_int8_cache_update_bit_exact():
  g = load("int8_cache")
  xk, xv = g["xk"], g["xv"]
  names = ("ck", "cv", "kq", "vq", "ks", "vs", "kscale", "vscale")
  r = oc.int8_update(g["ring_in_ck"], g["ring_in_cv"], g["ring_in_ks"], g["ring_in_vs"],
                     xk, xv, [5], ring_buffer=True, lazy=False)
  for n, t in zip(names, r):
    assert torch.equal(t, g[f"ring_out_{n}"]), n
  r = oc.int8_update(g["ring_in_ck"], g["ring_in_cv"], g["ring_in_ks"], g["ring_in_vs"],
                     xk, xv, g["slot_pos"], ring_buffer=False, lazy=False)
  for n, t in zip(names, r):
    assert torch.equal(t, g[f"slot_out_{n}"]), n


def test_int8_lazy_finalize_bit_exact():
  g = load("int8_cache")
  nl = g["lazy_xk"].shape[0]
  kq, ks, vq, vs = [], [], [], []
  for layer in range(nl):
    r = oc.int8_update(None, None, None, None, g["lazy_xk"][layer], g["lazy_xv"][layer],
                       g["slot_pos"], ring_buffer=False, lazy=True)
    kq.append(r[2]); vq.append(r[3]); ks.append(r[6]); vs.append(r[7])
  kq, vq, ks, vs = (torch.stack(t) for t in (kq, vq, ks, vs))
  assert torch.equal(kq, g["lazy_new_ks"])
  assert torch.equal(ks, g["lazy_new_k_scaler"])
  pos = g["slot_pos"]
  assert torch.equal(oc.finalize_rows(g["lazy_in_ck"], kq, pos), g["lazy_out_ck"])
  assert torch.equal(oc.finalize_rows(g["lazy_in_cv"], vq, pos), g["lazy_out_cv"])
  assert torch.equal(oc.finalize_rows(g["lazy_in_ks"], ks, pos), g["lazy_out_ks"])
  assert torch.equal(oc.finalize_rows(g["lazy_in_vs"], vs, pos), g["lazy_out_vs"])


def test_float_cache_bit_exact():
  g = load("float_cache")
  xk, xv, pos = g["xk"], g["xv"], g["slot_pos"]
  assert torch.equal(oc.append_ring(g["in_ck"], xk, 5), g["ring_out_ck"])
  assert torch.equal(oc.append_ring(g["in_cv"], xv, 5), g["ring_out_cv"])
  assert torch.equal(oc.append_per_slot(g["in_ck"], xk, pos), g["slot_out_ck"])
  assert torch.equal(oc.append_per_slot(g["stk_in_ck"], xk, pos, layer=2), g["stk_out_ck"])
  assert torch.equal(oc.append_per_slot(g["stk_in_cv"], xv, pos, layer=2), g["stk_out_cv"])
  assert torch.equal(oc.finalize_rows(g["stk_in_ck"], g["lazy_xk"], pos), g["lazy_out_ck"])
  assert torch.equal(oc.finalize_rows(g["stk_in_cv"], g["lazy_xv"], pos), g["lazy_out_cv"])


def test_pages_scenario_bit_exact():
  g = load("pages")
  h, p, ps, d = g["in_ck"].shape
  b, maxp = g["after_insert_page_indices"].shape
  pt = op.PageTableOracle(b, p, ps, maxp)
  ck, cv = g["in_ck"], g["in_cv"]
  for i, (slot, length) in enumerate(g["inserts"].tolist()):
    n, idx = pt.reserve_pages_insert(slot, length)
    assert np.array_equal(idx, g[f"insert_pages{i}"].numpy())
    ck = oi.insert_paged(ck, g[f"prefix_k{i}"], idx, ps)
    cv = oi.insert_paged(cv, g[f"prefix_v{i}"], idx, ps)
  assert torch.equal(ck, g["after_insert_ck"]) and torch.equal(cv, g["after_insert_cv"])
  assert np.array_equal(pt.page_indices, g["after_insert_page_indices"].numpy())
  for step in range(3):
    lens = g[f"step{step}_lens"].numpy()
    pt.fill_new_pages(lens)
    pti = pt.get_page_token_indices(lens)
    assert np.array_equal(pti, g[f"step{step}_pti"].numpy())
    assert np.array_equal(pt.page_indices, g[f"step{step}_page_indices"].numpy())
    assert np.array_equal(pt.lengths, g[f"step{step}_lengths"].numpy())
    ck = oc.paged_append(ck, g[f"step{step}_xk"], pti, ps)
    cv = oc.paged_append(cv, g[f"step{step}_xv"], pti, ps)
    assert torch.equal(ck, g[f"step{step}_ck"]) and torch.equal(cv, g[f"step{step}_cv"])
  comp = op.compress_cache(ck, pt.page_indices[5], pt.lengths[5])
  assert torch.equal(comp, g["compress_slot5_k"])


def test_reference_known_answers_page_manager():
  """tests/test_page_attention.py:48-203 and tests/test_kv_cache_manager.py:48-119
  of the reference, replayed on the oracle."""
  # single page, zero tail
  pt = op.PageTableOracle(3, 20, 4, 4)
  cache = torch.zeros((1, 6, 4, 2), dtype=torch.bfloat16)
  k = torch.arange(6).reshape(1, 1, 3, 2).to(torch.bfloat16)
  n, idx = pt.reserve_pages_insert(0, 3)
  out = oi.insert_paged(cache, k, idx, 4)
  assert out[0, 0].tolist() == [[0, 1], [2, 3], [4, 5], [0, 0]]
  # two pages, untouched remainder
  pt = op.PageTableOracle(3, 20, 4, 4)
  cache = torch.zeros((1, 20, 4, 2), dtype=torch.bfloat16)
  k = torch.arange(12).reshape(1, 1, 6, 2).to(torch.bfloat16)
  n, idx = pt.reserve_pages_insert(0, 6)
  out = oi.insert_paged(cache, k, idx, 4)
  exp = torch.arange(16); exp[12:] = 0
  assert torch.equal(out[:, :2].float(), exp.reshape(1, 2, 4, 2).float())
  assert not out[:, 2:].any()
  # decode reservation and the sentinel
  pt = op.PageTableOracle(3, 20, 4, 4)
  pt.reserve_pages_insert(1, 8)
  pt.fill_new_pages(np.asarray([0, 8, 0]))
  assert pt.page_indices[1].tolist() == [0, 1, 2, 19]
  assert pt.page_indices[0].tolist() == [19, 19, 19, 19]
  # page / token indices
  pt = op.PageTableOracle(5, 20, 4, 4)
  pt.reserve_pages_insert(1, 8); pt.reserve_pages_insert(3, 13); pt.reserve_pages_insert(0, 3)
  lens = np.asarray([3, 8, 0, 13, 0])
  pt.fill_new_pages(lens)
  pti = pt.get_page_token_indices(lens)
  assert pti[0].tolist() == [6, 7, 5] and pti[1].tolist() == [3, 4, 9]
  # update after three inserts
  pt = op.PageTableOracle(5, 20, 4, 4)
  cache = torch.zeros((1, 20, 4, 2), dtype=torch.bfloat16)
  for length, slot in ((3, 0), (8, 1), (13, 3)):
    k = torch.arange(length * 2).reshape(1, 1, length, 2).to(torch.bfloat16)
    n, idx = pt.reserve_pages_insert(slot, length)
    cache = oi.insert_paged(cache, k, idx, 4)
  pt.fill_new_pages(lens)
  pti = pt.get_page_token_indices(lens)
  xk = torch.arange(-1, -11, -1).reshape(5, 1, 1, 2).to(torch.bfloat16)
  cache = oc.paged_append(cache, xk, pti, 4)
  assert cache[0, 0].tolist() == [[0, 1], [2, 3], [4, 5], [-1, -2]]
  assert cache[0, 7].tolist() == [[-3, -4], [0, 0], [0, 0], [0, 0]]
  assert cache[0, 6].tolist() == [[24, 25], [-7, -8], [0, 0], [0, 0]]


def test_attention_against_reference_outputs():
  g = load("attention")
  for tag, tol in (("bf16", 2e-2), ("f32", 1e-5)):
    for tq in (1, 2):
      pre = f"{tag}_t{tq}_"
      xq, k, v, mask = g[pre + "xq"], g[pre + "k"], g[pre + "v"], g[pre + "mask"]
      kq, vq, ks, vs = g[pre + "kq"], g[pre + "vq"], g[pre + "ks"], g[pre + "vs"]
      o = oa.dense_attention(xq, k, v, None, None, mask)
      assert torch.allclose(o.float(), g[pre + "dense_float"].float(), atol=tol, rtol=tol)
      o = oa.dense_attention(xq, kq, vq, ks, vs, mask)
      assert torch.allclose(o.float(), g[pre + "dense_int8"].float(), atol=tol, rtol=tol)
      o, (m, l) = oa.flash_attention(xq, k, v, 0, None, None, mask)
      assert torch.allclose(o.float(), g[pre + "flash_float_o"].float(), atol=tol, rtol=tol)
      assert torch.allclose(m.float(), g[pre + "flash_float_m"].float(), atol=1e-4, rtol=1e-4)
      assert torch.allclose(l.float(), g[pre + "flash_float_l"].float(), atol=1e-4, rtol=1e-4)
      o, (m, l) = oa.flash_attention(xq, kq, vq, 0, ks, vs, mask)
      assert torch.allclose(o.float(), g[pre + "flash_int8_o"].float(), atol=tol, rtol=tol)
      assert torch.allclose(l.float(), g[pre + "flash_int8_l"].float(), atol=1e-4, rtol=1e-4)


def test_ragged_restatement_against_the_reference_kernel_bodies():
  """`ragged.npz` holds what the reference's own `ragged_mha` (left aligned,
  attention_kernel.py:255-329 through pallas_call and vmap) and ring kernel body
  (attention_kernel.py:22-109) return when executed on a sequential grid
  interpreter.  The restatement runs the same fp32 op sequence on the same
  library, so it must agree to fp32 round-off."""
  import golden_inputs

  g = load("ragged")
  for name in golden_inputs.RAGGED_CASES:
    x = golden_inputs.ragged_inputs(name)
    assert golden_inputs.checksum(x) == int(g[name + "_checksum"]), "seeded inputs differ from the fixture's"
    o, (m, l) = oa.ragged_mha(x["q"], x["k"], x["v"], x["layer"], x["start"], x["end"], x["ks"], x["vs"],
                              bk=x["bk"], wrap=x["ring"])
    tol = 1e-6 if x["q"].dtype == torch.float32 else 0.0
    assert torch.allclose(o.float(), g[name + "_o"].float(), atol=tol, rtol=tol), name
    assert torch.allclose(m, g[name + "_m"], atol=1e-6, rtol=1e-6), name
    assert torch.allclose(l, g[name + "_l"], atol=1e-6, rtol=1e-6), name


def test_engine_insert_bit_exact():
  """`engine_insert.npz`: the reference's `PyTorchEngine.insert` (engine.py:
  371-648) executed on ring / left-aligned, stacked / per-layer, int8 / bf16
  caches, and its paged insert with reservation (650-672)."""
  g = load("engine_insert")
  b, h, s, d, nl, lpad, seq_len = (int(v) for v in g["geometry"])
  for name in ("ring_nowrap_i8", "ring_wrap_i8", "ring_edge_i8", "ring_nowrap_bf16", "ring_wrap_bf16", "left_i8",
               "left_i8_stacked", "left_bf16_stacked"):
    ring, stacked, quant, cur, slot = (int(v) for v in g[name + "_args"])
    n = 1 if stacked else nl
    caches = [(g[f"{name}_in_ck{i}"], g[f"{name}_in_cv{i}"]) for i in range(n)]
    scales = [(g[f"{name}_in_ks{i}"], g[f"{name}_in_vs{i}"]) for i in range(n)] if quant else []
    prefix = [(g[f"{name}_prefix_k{i}"], g[f"{name}_prefix_v{i}"]) for i in range(nl)]
    oc_, os_, mask, start, ipos, lens = oi.engine_insert(bool(ring), bool(stacked), bool(quant), s, cur, seq_len,
                                                         prefix, caches, scales, slot)
    for i in range(n):
      assert torch.equal(oc_[i][0], g[f"{name}_out_ck{i}"]) and torch.equal(oc_[i][1], g[f"{name}_out_cv{i}"]), name
      if quant:
        assert torch.equal(os_[i][0], g[f"{name}_out_ks{i}"]) and torch.equal(os_[i][1], g[f"{name}_out_vs{i}"]), name
    assert torch.equal(mask, g[f"{name}_out_mask"][slot]), name
    assert int(g[f"{name}_out_start"][slot]) == start and int(g[f"{name}_out_input_pos"][slot]) == ipos
    assert int(g[f"{name}_out_lens"][slot]) == lens
    other = [i for i in range(b) if i != slot]
    assert torch.isinf(g[f"{name}_out_mask"][other]).all()  # rows of the other slots are untouched
  p, ps, maxp, slot, seq_len = (int(v) for v in g["paged_geometry"])
  table = op.PageTableOracle(b, p, ps, maxp)
  table.reserve_pages_insert(0, 6)
  _, idx = table.reserve_pages_insert(slot, seq_len)
  for i in range(nl):
    assert torch.equal(oi.insert_paged(g[f"paged_in_ck{i}"], g[f"paged_prefix_k{i}"], idx, ps), g[f"paged_out_ck{i}"])
    assert torch.equal(oi.insert_paged(g[f"paged_in_cv{i}"], g[f"paged_prefix_v{i}"], idx, ps), g[f"paged_out_cv{i}"])
  assert np.array_equal(table.page_indices, g["paged_out_page_indices"].numpy())
  assert np.array_equal(table.lengths, g["paged_out_lengths"].numpy())
  assert torch.equal(oi.insert_mask_row(s, 0, seq_len, False), g["paged_out_mask"][slot])


def test_engine_step_bookkeeping_matches_reference():
  """`engine_step.npz`: three decode steps of the reference's `generate_impl`
  with a stand-in model, ring buffer and left aligned."""
  from oracle import engine as oe

  g = load("engine_step")
  b, s, bk, vocab, steps = (int(v) for v in g["geometry"])
  for name, ring in (("ring", True), ("left", False)):
    tokens, lens = g[f"{name}_in_tokens"].numpy(), g[f"{name}_in_lens"].numpy()
    start, ipos = g[f"{name}_in_start"].numpy(), g[f"{name}_in_input_pos"].numpy()
    mask, cur = g[f"{name}_in_mask"].numpy(), int(g[f"{name}_in_current_position"])
    for step in range(steps):
      pre = f"{name}_step{step}_"
      rb, ri = oe.ragged_block_indices(start, ipos, s, bk)
      assert np.array_equal(rb.reshape(-1), g[pre + "ragged_batch_index"].numpy())
      assert np.array_equal(ri.reshape(-1), g[pre + "ragged_block_index"].numpy())
      nxt = g[pre + "tokens"].numpy()
      model_mask, mask, ipos, lens, cur, data = oe.decode_step_bookkeeping(ring, not ring, s, tokens, lens, ipos, mask,
                                                                           cur, nxt)
      assert np.array_equal(model_mask, g[pre + "model_mask"].numpy().reshape(b, s))
      assert np.array_equal(mask, g[pre + "mask"].numpy())
      assert np.array_equal(ipos, g[pre + "input_pos"].numpy()) and np.array_equal(lens, g[pre + "lens"].numpy())
      assert cur == int(g[pre + "current_position"])
      assert np.array_equal(data, g[pre + "data"].numpy())
      tokens = nxt


def test_ragged_restatement_consistent_with_pinned_dense():
  """The unpinned ragged restatements agree with the pinned flash_attention on
  the same valid set (left aligned and ring wrap)."""
  g = torch.Generator().manual_seed(11)
  b, hq, hkv, s, d = 5, 8, 2, 64, 16
  xq = torch.randn(b, hq, 1, d, generator=g)
  k = torch.randn(b, hkv, s, d, generator=g)
  v = torch.randn(b, hkv, s, d, generator=g)
  kq, ks = quantize_insert(k, (-3, -1))
  vq, vs = quantize_insert(v, (-3, -1))
  start = torch.tensor([0, 0, 0, 0, 0])
  end = torch.tensor([64, 1, 33, 16, 0])
  o, (m, l) = oa.ragged_mha(xq, kq, vq, 0, start, end, ks, vs, bk=16)
  mask = torch.full((b, 1, 1, s), float("-inf"))
  for i in range(b):
    mask[i, :, :, :int(end[i])] = 0
  fo, (fm, fl) = oa.flash_attention(xq[:4], kq[:4], vq[:4], 0, ks[:4], vs[:4], mask[:4])
  assert torch.allclose(o[:4].reshape(4, hq, 1, d), fo, atol=1e-5, rtol=1e-4)
  assert torch.allclose(m[:4].reshape(4, hq, 1, 1), fm, atol=1e-5)
  assert torch.allclose(l[:4].reshape(4, hq, 1, 1), fl, rtol=1e-4)
  assert not o[4].any() and torch.isinf(m[4]).all() and not l[4].any()
  # ring wrap
  start = torch.tensor([10, 50, 63, 5, 7])
  end = torch.tensor([40, 20, 1, 4, 7])
  o, (m, l) = oa.ragged_mha(xq, kq, vq, 0, start, end, ks, vs, bk=16, wrap=True)
  pos = torch.arange(s)
  mask = torch.full((b, 1, 1, s), float("-inf"))
  for i in range(4):
    st, en = int(start[i]), int(end[i])
    ok = (pos >= st) & (pos < en) if st <= en else (pos >= st) | (pos < en)
    mask[i, 0, 0, ok] = 0
  fo, (fm, fl) = oa.flash_attention(xq[:4], kq[:4], vq[:4], 0, ks[:4], vs[:4], mask[:4])
  assert torch.allclose(o[:4].reshape(4, hq, 1, d), fo, atol=1e-5, rtol=1e-4)
  assert torch.allclose(l[:4].reshape(4, hq, 1, 1), fl, rtol=1e-4)
  assert not o[4].any() and not l[4].any()  # start == end counts as empty


def test_insert_restatements():
  g = torch.Generator().manual_seed(12)
  b, h, s, d, length = 3, 2, 32, 8, 12
  cache = torch.zeros(b, h, s, d, dtype=torch.int8)
  scaler = torch.ones(b, 1, s, 1, dtype=torch.bfloat16)
  prefix = torch.randn(1, h, length, d, generator=g).to(torch.bfloat16)
  c1, s1 = oi.insert_no_wrap(cache, prefix, 1, 4, scaler=scaler, quantize=True)
  c2, s2 = oi.insert_wrap(cache, prefix, 1, 4, scaler=scaler, quantize=True)
  assert torch.equal(c1, c2) and torch.equal(s1, s2)
  c3, s3 = oi.insert_wrap(cache, prefix, 1, 28, scaler=scaler, quantize=True)
  assert torch.equal(c3[1][:, 28:], c1[1][:, 4:8]) and torch.equal(c3[1][:, :8], c1[1][:, 8:16])
  assert torch.equal(s3[1][:, :8], s1[1][:, 8:16])
  assert not c3[0].any() and not c3[2].any()
  m = oi.insert_mask_row(8, 6, 2, wrap=True)
  assert m.tolist() == [0, 0] + [float("-inf")] * 4 + [0, 0]


def test_w8a16_linear_against_the_reference_layer():
  """`linear.npz`: the reference's own `quantize_weight_from_nn_linear` (bit for
  bit) and `forward` (within `w8a16_tolerance`, more than 99 % of the outputs
  identical: the oracle rounds the exact dot product, the reference a float32
  accumulation)."""
  from oracle import linear as ol

  g = load("linear")
  codes, scale = ol.quantize_weight(g["small_w"])
  assert torch.equal(codes, g["small_weight"])
  assert torch.equal(scale, g["small_weight_scaler"])
  assert (g["small_weight"][3] == 0).all()  # the all-zero channel keeps the clamped scale
  # the package's module quantises a float weight the same way (offline work in plain torch)
  from jetstream_pytorch_b200.layers import WeightOnlyPerChannelQuantizedLinear

  lin = WeightOnlyPerChannelQuantizedLinear(g["small_w"].shape[1], g["small_w"].shape[0])
  lin.quantize_weight_from_nn_linear(g["small_w"])
  assert torch.equal(lin.weight, g["small_weight"]) and torch.equal(lin.weight_scaler, g["small_weight_scaler"])
  for tag in ("small", "batch"):
    x, w, s, want = g[f"{tag}_x"], g[f"{tag}_weight"], g[f"{tag}_weight_scaler"], g[f"{tag}_y"]
    got = ol.w8a16_linear(x, w, s)
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    same = (got.view(torch.int16) == want.view(torch.int16)).float().mean().item()
    assert same > 0.99, same
    # (the outputs that differ are sums that cancel to almost nothing, where the reference's float32
    # accumulation error shows; they stay far inside the absolute term of the tolerance)
    assert ((got.float() - want.float()).abs().double() <= ol.w8a16_tolerance(x, w, s)).all()


def test_rmsnorm_against_the_reference_class():
  """`linear.npz`: the reference's own `RMSNorm` on bf16 inputs with a bf16 weight, bit for bit."""
  from oracle import linear as ol

  g = load("linear")
  y = ol.rmsnorm(g["norm_x"], g["norm_weight"], float(g["norm_eps"]))
  assert y.dtype == torch.bfloat16 and torch.equal(y, g["norm_y"])
  assert not g["norm_y"][0, 1].any()
