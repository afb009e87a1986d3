"""The allocation-free attention entry point (`jpt_flash_decode_static`).

Some callers cannot give the attention kernels a workspace: a serving loop
whose device memory pool is fixed and already handed out, or a host that forbids
cudaMalloc once it is running (the call synchronises the device).  For them the
library carries its own scratch array, and `static_scratch=True` makes the
Python shim call that entry point without creating any workspace tensor.

This file is collected last on purpose: if it fails, a run that stops at the
first failure has already run every other test.  The test must pass in a fresh
process as well as after the other tests, so it relies on nothing they leave
behind and checks two calls in a row (the scratch keeps the previous call's
contents).
"""

import pytest
import torch

from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu


def _case(seed, b, hq, hkv, s, d):
  from oracle.quant import quantize_insert

  g = torch.Generator().manual_seed(seed)
  q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
  k, ks = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  v, vs = quantize_insert(torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16), (-3, -1))
  start = torch.randint(0, s, (b,), generator=g)
  end = torch.randint(0, s, (b,), generator=g)
  end[0] = start[0]  # one empty row
  return [t.cuda() for t in (q, k, v, ks, vs, start, end)]


def _check(o, m, l, o_ref, m_ref, l_ref, what):
  assert attention_close(o, o_ref), f"{what}: {describe(o, o_ref)}"
  live = torch.isfinite(m_ref)
  assert torch.equal(torch.isfinite(m.cpu()), live.cpu()), what
  assert torch.allclose(m.cpu()[live.cpu()], m_ref.cpu()[live.cpu()], atol=1e-3, rtol=1e-3), what
  assert torch.allclose(l.cpu()[live.cpu()], l_ref.cpu()[live.cpu()], atol=1e-3, rtol=1e-3), what


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
  """Two calls in a row through `jpt_flash_decode_static`, each checked against
  the workspace entry point AND against the CPU oracle."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from oracle import attention as oa

  for call, (seed, shape) in enumerate(((91, (24, 64, 8, 1024, 128)), (92, (9, 32, 8, 640, 128)))):
    q, k, v, ks, vs, start, end = _case(seed, *shape)
    args = (q, k, v, 0, start, end, None, None, ks, vs)
    o_ref, (m_ref, l_ref) = ak.ragged_mha(*args, ring=True)
    before = torch.cuda.memory_allocated()
    o, (m, l) = ak.ragged_mha(*args, ring=True, static_scratch=True)
    torch.cuda.synchronize()
    # only the three result tensors were created by the call
    grown = torch.cuda.memory_allocated() - before
    assert grown <= o.numel() * 2 + (m.numel() + l.numel()) * 4 + 3 * 512, f"call {call}: {grown} bytes"
    _check(o, m, l, o_ref, m_ref, l_ref, f"call {call} vs the workspace entry point")
    # the reference's grid is S // bk blocks: bk must divide the cache length (640 in the second case)
    eo, (em, el) = oa.ragged_mha(q.cpu(), k.cpu(), v.cpu(), 0, start.cpu(), end.cpu(), ks.cpu(), vs.cpu(),
                                 bk=128, wrap=True)
    _check(o, m, l, eo, em, el, f"call {call} vs the oracle")
  assert ak.kernel_status() == 0


def test_static_scratch_holds_split_k_partials_of_the_scalar_kernel():
  """A float32 cache takes the scalar kernel; with three splits its partial
  results live in the built-in array behind the header."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from oracle import attention as oa

  g = torch.Generator().manual_seed(93)
  b, hq, hkv, s, d = 5, 8, 2, 300, 64
  q = torch.randn(b, hq, 1, d, generator=g)
  k = torch.randn(b, hkv, s, d, generator=g)
  v = torch.randn(b, hkv, s, d, generator=g)
  end = torch.tensor([300, 1, 0, 150, 299])
  start = torch.zeros(b, dtype=torch.int64)
  for _ in range(2):
    o, (m, l) = ak.ragged_mha(q.cuda(), k.cuda(), v.cuda(), 0, start.cuda(), end.cuda(), None, None, None, None,
                              num_splits=3, static_scratch=True)
    eo, (em, el) = oa.ragged_mha(q, k, v, 0, start, end, None, None, bk=300)
    assert attention_close(o, eo, 1e-4, 1e-4), describe(o, eo)
    live = torch.isfinite(em)
    assert torch.allclose(l.cpu()[live], el[live], atol=1e-3, rtol=1e-3)


def test_static_scratch_rejects_shapes_beyond_its_size():
  from jetstream_pytorch_b200 import attention_kernel as ak

  # a float32 cache takes the scalar split-K kernel, whose partials for this
  # shape need far more than the 16 MiB built into the library
  b, hq, hkv, s, d = 64, 64, 64, 256, 128
  q = torch.zeros(b, hq, 1, d, device="cuda")
  k = torch.zeros(b, hkv, s, d, device="cuda")
  with pytest.raises(ValueError, match="scratch"):
    ak._flash_decode(q, k, k, sm_scale=1.0, kv_strides=(k.stride(0), k.stride(1), k.stride(2)), n_kv_heads=hkv,
                     seq=s, num_splits=32, static_scratch=True)
