"""Tolerance checks shared by the GPU parity tests.

Attention outputs must be within 2e-2 absolute AND 1e-2 relative of the
expected values.  "Relative" is measured per output row (the head_dim vector of
one query row): max |actual - expected| over the row against max |expected| over
the row, the usual vector form; an element-wise relative error is meaningless
for the near-zero components every row has.  A row whose expected values are
all zero (an empty sequence) must be exactly zero.
"""

import torch

ATOL, RTOL = 2e-2, 1e-2


def attention_errors(actual, expected):
  """(max absolute error, max row-relative error) as floats."""
  a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
  err = (a - e).abs()
  row_err = err.amax(dim=-1)
  row_ref = e.abs().amax(dim=-1)
  rel = torch.where(row_ref > 0, row_err / row_ref.clamp_min(1e-30), torch.where(row_err > 0, float("inf"), 0.0))
  return float(err.max()) if err.numel() else 0.0, float(rel.max()) if rel.numel() else 0.0


def attention_close(actual, expected, atol=ATOL, rtol=RTOL):
  """True when BOTH bounds hold: every element within `atol`, every row within
  `rtol` of its largest expected magnitude."""
  if tuple(actual.shape) != tuple(expected.shape):
    return False
  abs_err, rel_err = attention_errors(actual, expected)
  return abs_err <= atol and rel_err <= rtol


def describe(actual, expected):
  abs_err, rel_err = attention_errors(actual, expected)
  return f"max abs err {abs_err:.3e} (limit {ATOL}), max row-relative err {rel_err:.3e} (limit {RTOL})"
