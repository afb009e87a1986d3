"""GPU parity against vectors that the reference's own code produced for the
ragged kernels and the engine's insert path (tests/golden/make_golden.py ran the
reference's Pallas kernel bodies and `PyTorchEngine.insert` on an interpreter
and stored the results)."""

import numpy as np
import pytest
import torch

import golden_inputs
from golden_io import load
from parity_tools import attention_close, describe

pytestmark = pytest.mark.gpu

DEV = "cuda"


def cu(t):
  return t.to(DEV) if isinstance(t, torch.Tensor) else t


@pytest.mark.parametrize("name", list(golden_inputs.RAGGED_CASES))
@pytest.mark.parametrize("kernel", [0, 1, 2])
def test_ragged_kernels_against_the_reference_kernel_bodies(name, kernel):
  """`ragged_mha` (left aligned) and the ring-buffer form against `ragged.npz`,
  through every kernel that can take the shape: 0 = automatic choice (tcgen05
  for int8 D=128 with up to 8 grouped rows, mma.sync for bf16 D=128), 1 = the
  scalar split-K kernel, 2 = mma.sync instead of tcgen05."""
  from jetstream_pytorch_b200 import attention_kernel as ak

  g = load("ragged")
  x = golden_inputs.ragged_inputs(name)
  assert golden_inputs.checksum(x) == int(g[name + "_checksum"]), "seeded inputs differ from the fixture's"
  if kernel == 2 and not (x["k"].dtype == torch.int8 and x["q"].shape[-1] == 128):
    pytest.skip("only int8 head_dim-128 shapes have two tensor-core kernels")
  o, (m, l) = ak.ragged_mha(cu(x["q"]), cu(x["k"]), cu(x["v"]), x["layer"], cu(x["start"]), cu(x["end"]), None, None,
                            cu(x["ks"]), cu(x["vs"]), ring=x["ring"], force_generic=kernel)
  eo, em, el = g[name + "_o"], g[name + "_m"], g[name + "_l"]
  tight = x["q"].dtype == torch.float32
  assert attention_close(o, eo, *((1e-4, 1e-4) if tight else ())), describe(o, eo)
  live = torch.isfinite(em)
  assert torch.equal(torch.isfinite(m.cpu()), live)
  assert torch.allclose(m.cpu()[live], em[live], atol=1e-3, rtol=1e-3)
  # The reference stores 1 instead of 0 as the denominator of a row none of whose
  # blocks ran (attention_kernel.py:104, 324: l_next_safe); such rows have m = -inf.
  assert torch.allclose(l.cpu()[live], el[live], atol=1e-3, rtol=1e-3)
  assert not o.cpu()[~live].any() and not l.cpu()[~live].any()


CASES = ("ring_nowrap_i8", "ring_wrap_i8", "ring_edge_i8", "ring_nowrap_bf16", "ring_wrap_bf16", "left_i8",
         "left_i8_stacked", "left_bf16_stacked")


@pytest.mark.parametrize("name", CASES)
def test_engine_insert_bit_exact_with_reference(name):
  """`insert.insert` against what `PyTorchEngine.insert` (engine.py:371-648)
  returned for the same state: caches, scalers and the slot's bookkeeping rows."""
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData
  from jetstream_pytorch_b200.insert import insert

  g = load("engine_insert")
  b, h, s, d, nl, lpad, seq_len = (int(v) for v in g["geometry"])
  ring, stacked, quant, cur, slot = (int(v) for v in g[name + "_args"])
  n = 1 if stacked else nl
  data = JetEngineEnvironmentData(batch_size=b, cache_sequence_length=s, num_layers=nl, ring_buffer=bool(ring),
                                  generate_cache_stacked=bool(stacked), testing=True)
  data.quant_config.enable_kv_quantization = bool(quant)
  env = JetEngineEnvironment(data, device=DEV)
  assert env.generate_cache_stacked == bool(stacked)
  caches = [(cu(g[f"{name}_in_ck{i}"]).clone(), cu(g[f"{name}_in_cv{i}"]).clone()) for i in range(n)]
  scales = [(cu(g[f"{name}_in_ks{i}"]).clone(), cu(g[f"{name}_in_vs{i}"]).clone()) for i in range(n)] if quant else None
  prefix = [(cu(g[f"{name}_prefix_k{i}"]), cu(g[f"{name}_prefix_v{i}"])) for i in range(nl)]
  mask = torch.full((b, s), float("-inf"), device=DEV)
  start = torch.full((b, 1), 3, dtype=torch.int32, device=DEV)
  ipos = torch.full((b, 1), 4, dtype=torch.int32, device=DEV)
  lens = torch.full((b, 1), 9, dtype=torch.int32, device=DEV)
  insert(env, prefix, seq_len, caches, scales, slot, cur, mask=mask, start=start, input_pos=ipos, lens=lens)
  for i in range(n):
    assert torch.equal(caches[i][0].cpu(), g[f"{name}_out_ck{i}"]), f"K cache {i}"
    assert torch.equal(caches[i][1].cpu(), g[f"{name}_out_cv{i}"]), f"V cache {i}"
    if quant:
      assert torch.equal(scales[i][0].cpu(), g[f"{name}_out_ks{i}"]), f"K scaler {i}"
      assert torch.equal(scales[i][1].cpu(), g[f"{name}_out_vs{i}"]), f"V scaler {i}"
  assert torch.equal(mask.cpu(), g[f"{name}_out_mask"])
  assert torch.equal(start.cpu(), g[f"{name}_out_start"])
  assert torch.equal(ipos.cpu(), g[f"{name}_out_input_pos"])
  assert torch.equal(lens.cpu(), g[f"{name}_out_lens"])


def test_engine_paged_insert_with_reservation_bit_exact_with_reference():
  """engine.py:650-672 -> 583-625 on bf16 pools, two layers."""
  from jetstream_pytorch_b200.insert import insert_page_attention_with_reservation
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = load("engine_insert")
  b, h, s, d, nl, lpad, _ = (int(v) for v in g["geometry"])
  p, ps, maxp, slot, seq_len = (int(v) for v in g["paged_geometry"])
  pam = PageAttentionManager(b, p, ps, maxp)
  pam.reserve_pages_insert(0, 6)
  pools = [(cu(g[f"paged_in_ck{i}"]).clone(), cu(g[f"paged_in_cv{i}"]).clone()) for i in range(nl)]
  prefix = [(cu(g[f"paged_prefix_k{i}"]), cu(g[f"paged_prefix_v{i}"])) for i in range(nl)]
  insert_page_attention_with_reservation(pam, prefix, seq_len, pools, slot)
  for i in range(nl):
    assert torch.equal(pools[i][0].cpu(), g[f"paged_out_ck{i}"]) and torch.equal(pools[i][1].cpu(), g[f"paged_out_cv{i}"])
  assert np.array_equal(pam.page_indices, g["paged_out_page_indices"].numpy())
  assert np.array_equal(np.asarray(pam.lengths), g["paged_out_lengths"].numpy())
