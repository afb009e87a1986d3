"""CPU-only checks: the C-ABI library loads and exports every symbol the header
declares, the host-side page manager reproduces the reference's tables, and the
environment derives the reference's mode flags."""

import ctypes
import os
import queue
import re

import numpy as np
import pytest

from golden_io import load

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
  text = open(os.path.join(ROOT, "include", "jpt_b200.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(jpt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.build import build_library

  build_library()
  handle = ctypes.CDLL(_lib.LIB_PATH)
  declared = _header_functions()
  assert len(declared) >= 12
  for name in declared:
    assert hasattr(handle, name), f"{name} declared in include/jpt_b200.h but not exported"
  assert sorted(_lib.EXPORTS) == declared
  assert _lib.lib().jpt_version() >= 100


def test_attn_params_struct_matches_header():
  from jetstream_pytorch_b200 import _lib

  text = open(os.path.join(ROOT, "include", "jpt_b200.h")).read()
  body = text[text.index("typedef struct jpt_attn_params {"):text.index("} jpt_attn_params;")]
  body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
  names = []
  for decl in body.split("{", 1)[1].split(";"):
    decl = decl.strip()
    if not decl:
      continue
    for part in decl.split(","):
      names.append(re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", part.strip())[0])
  assert names == [f[0] for f in _lib.AttnParams._fields_]


def test_page_manager_host_tables_match_reference():
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  g = load("pages")
  _, p, ps, _ = g["in_ck"].shape
  b, maxp = g["after_insert_page_indices"].shape
  pam = PageAttentionManager(b, p, ps, maxp)
  for i, (slot, length) in enumerate(g["inserts"].tolist()):
    n, idx = pam.reserve_pages_insert(slot, length)
    assert np.array_equal(idx, g[f"insert_pages{i}"].numpy())
  assert np.array_equal(pam.page_indices, g["after_insert_page_indices"].numpy())
  for step in range(3):
    lens = g[f"step{step}_lens"].numpy()
    pam.fill_new_pages(lens)
    pti = pam.get_page_token_indices(lens)
    assert np.array_equal(pti, g[f"step{step}_pti"].numpy())
    assert np.array_equal(pam.page_indices, g[f"step{step}_page_indices"].numpy())
    assert np.array_equal(pam.lengths, g[f"step{step}_lengths"].numpy())


def test_page_manager_known_answers_and_exhaustion():
  """tests/test_page_attention.py:147-203 of the reference (host part)."""
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  pam = PageAttentionManager(3, 20, 4, 4)
  pam.reserve_pages_insert(1, 8)
  pam.fill_new_pages(np.asarray([0, 8, 0]))
  assert pam.page_indices[1].tolist() == [0, 1, 2, 19]
  assert pam.page_indices[0].tolist() == [19, 19, 19, 19]
  pam = PageAttentionManager(5, 20, 4, 4)
  pam.reserve_pages_insert(1, 8); pam.reserve_pages_insert(3, 13); pam.reserve_pages_insert(0, 3)
  lens = np.asarray([3, 8, 0, 13, 0])
  pam.fill_new_pages(lens)
  pti = pam.get_page_token_indices(lens)
  assert pti[0].tolist() == [6, 7, 5] and pti[1].tolist() == [3, 4, 9] and pti[2].tolist() == [0, 1, 3]
  # exhaustion raises queue.Empty like the reference's Queue.get(block=False)
  pam = PageAttentionManager(2, 3, 4, 4)
  pam.reserve_pages_insert(0, 8)
  with pytest.raises(queue.Empty):
    pam.reserve_pages_insert(1, 8)
  # recycling (extension): freed pages return in table order
  pam = PageAttentionManager(2, 4, 4, 4)
  pam.reserve_pages_insert(0, 7)
  pam.reserve_pages_insert(1, 5)
  pam.free_pages_resource(0)
  assert pam.page_indices[0].tolist() == [3, 3, 3, 3] and pam.lengths[0] == 0
  _, idx = pam.reserve_pages_insert(0, 8)
  assert idx.tolist() == [0, 1]


def test_environment_mode_flags():
  """jetstream_pt/environment.py:163-188."""
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  d = JetEngineEnvironmentData(ring_buffer=True, cache_shape=(4, 2, 16, 8), num_layers=3)
  e = JetEngineEnvironment(d, device="cpu")
  assert not (e.lazy_cache_update or e.ragged_mha or e.flash_attention or e.generate_cache_stacked)
  assert e.cache_shape == (4, 2, 16, 8)
  d = JetEngineEnvironmentData(ring_buffer=False, cache_shape=(4, 2, 16, 8), num_layers=3)
  e = JetEngineEnvironment(d, device="cpu")
  assert e.lazy_cache_update and e.ragged_mha and e.flash_attention and e.new_cache_stacked
  assert e.cache_shape == (3, 4, 2, 16, 8)
  d = JetEngineEnvironmentData(ring_buffer=False, testing=True, ragged_mha=True, cache_shape=(4, 2, 16, 8))
  e = JetEngineEnvironment(d, device="cpu")
  assert e.ragged_mha and not e.lazy_cache_update
  d = JetEngineEnvironmentData(ring_buffer=False, paged_attention_total_num_pages=16, cache_shape=(2, 16, 4, 8))
  e = JetEngineEnvironment(d, device="cpu")
  assert e.page_attention and not e.lazy_cache_update and not e.generate_cache_stacked


def test_cuda_only_entry_points_reject_cpu_tensors():
  import torch

  from jetstream_pytorch_b200 import quantize

  with pytest.raises(ValueError):
    quantize.quantize_tensor(torch.zeros(1, 2, 3, 16, dtype=torch.bfloat16), (-3, -1))
