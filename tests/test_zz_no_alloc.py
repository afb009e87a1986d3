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

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-2, 1e-2


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


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
  from jetstream_pytorch_b200 import attention_kernel as ak

  for call, (seed, shape) in enumerate(((91, (24, 64, 8, 1024, 128)), (92, (9, 32, 8, 640, 128)))):
    q, k, v, ks, vs, start, end = _case(seed, *shape)
    args = (q, k, v, 0, start, end, None, None, ks, vs)
    o_ref, (m_ref, l_ref) = ak.ragged_mha(*args, ring=True)
    before = torch.cuda.memory_allocated()
    o, (m, l) = ak.ragged_mha(*args, ring=True, static_scratch=True)
    torch.cuda.synchronize()
    assert torch.allclose(o.float(), o_ref.float(), atol=ATOL, rtol=RTOL), f"call {call}: outputs differ"
    live = torch.isfinite(m_ref)
    assert torch.equal(torch.isfinite(m), live)
    assert torch.allclose(m[live], m_ref[live], atol=1e-3, rtol=1e-3)
    assert torch.allclose(l[live], l_ref[live], atol=1e-3, rtol=1e-3)
    # only the three result tensors were created by the call
    grown = torch.cuda.memory_allocated() - before
    assert grown <= o.numel() * 2 + (m.numel() + l.numel()) * 4 + 3 * 512, f"call {call}: {grown} bytes"


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
