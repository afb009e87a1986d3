"""Tolerance checks shared by the GPU parity tests.

Attention outputs must be within 2e-2 absolute AND 1e-2 relative of the
expected values.  The absolute bound holds for every element.  "Relative" is
measured per output row (the head_dim vector of one query row) in the usual
norm-wise form, ||actual - expected||_2 / ||expected||_2: an element-wise
relative error is meaningless for the near-zero components every row has, and
a max-norm ratio would fail on a single bf16 rounding flip (one bf16 ulp is up
to 0.8 % of its element, and the reference rounds its own output to bf16, in
the ragged kernel after every block).  A row whose expected values are all zero
(an empty sequence) must be exactly zero.
"""

import torch

ATOL, RTOL = 2e-2, 1e-2


def attention_errors(actual, expected):
  """(max absolute error, max row-relative error) as floats."""
  a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
  err = a - e
  row_err = torch.linalg.vector_norm(err, dim=-1)
  row_ref = torch.linalg.vector_norm(e, dim=-1)
  rel = torch.where(row_ref > 0, row_err / row_ref.clamp_min(1e-30), torch.where(row_err > 0, float("inf"), 0.0))
  return float(err.abs().max()) if err.numel() else 0.0, float(rel.max()) if rel.numel() else 0.0


def attention_close(actual, expected, atol=ATOL, rtol=RTOL):
  """True when BOTH bounds hold: every element within `atol`, every row within
  `rtol` of the expected row in the 2-norm."""
  if tuple(actual.shape) != tuple(expected.shape):
    return False
  abs_err, rel_err = attention_errors(actual, expected)
  return abs_err <= atol and rel_err <= rtol


def describe(actual, expected):
  abs_err, rel_err = attention_errors(actual, expected)
  return f"max abs err {abs_err:.3e} (limit {ATOL}), max row-relative err {rel_err:.3e} (limit {RTOL})"
