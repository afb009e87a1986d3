"""Torch-backed stand-ins for the packages the reference imports but this
machine lacks (jax, jax.numpy, jax.experimental.pallas, torch_xla2), so that the
reference's own modules can be imported UNMODIFIED from a read-only checkout and
the parts of them that are plain torch / numpy can be executed to produce golden
vectors.

Only `make_golden.py` (run once, on a machine that has the reference checkout)
uses this file.  Nothing here is arithmetic of its own: every function forwards
to the torch op with the same meaning, arrays are torch tensors carrying the two
jax-array idioms the reference uses (`x.at[idx].set(v)`, `x.jax()`, `x._elem =`).

`jax.experimental.pallas` is emulated as a sequential grid interpreter: that is
what `pallas_call(..., interpret=True)` does in JAX.  `pallas_call` walks the
grid in row-major order, evaluates every BlockSpec's index map (scalar-prefetch
operands first, as PrefetchScalarGridSpec passes them), hands the kernel body
`Ref` objects that are views of the selected blocks, and `program_id` / `when`
read the interpreter's state.  The reference's kernel bodies run unmodified on
these objects.  `jax.random` and the third-party paged-attention kernel are NOT
emulated; calling them raises.
"""

import contextlib
import math
import sys
import types

import numpy as np
import torch


class JTensor(torch.Tensor):
  """torch.Tensor with the jax-array / XLATensor2 idioms the reference uses."""

  @staticmethod
  def wrap(t):
    if isinstance(t, JTensor):
      return t
    if isinstance(t, torch.Tensor):
      return t.as_subclass(JTensor)
    return t

  def jax(self):
    return self

  @property
  def _elem(self):
    return self

  @_elem.setter
  def _elem(self, value):
    # `tensor._elem = new_array` rebinds the wrapped array in XLATensor2.
    self.data = torch.as_tensor(value).data

  @property
  def at(self):
    return _At(self)

  def transpose(self, *axes):
    if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
      return self.permute(*axes[0])
    if len(axes) == self.ndim and self.ndim != 2:
      return self.permute(*axes)
    return super().transpose(*axes)

  def astype(self, dtype):
    return self.to(dtype)

  def max(self, *a, axis=None, **k):  # jax: values only, never (values, indices)
    if axis is None and not a and not k:
      return super().max()
    if axis is None:
      return super().max(*a, **k)
    return JTensor.wrap(torch.amax(self.as_subclass(torch.Tensor), dim=axis))

  def sum(self, *a, axis=None, **k):
    if axis is None:
      return super().sum(*a, **k)
    return JTensor.wrap(torch.sum(self.as_subclass(torch.Tensor), dim=axis))

  def block_until_ready(self):
    return self


class _At:

  def __init__(self, arr):
    self.arr = arr

  def __getitem__(self, idx):
    return _AtIdx(self.arr, idx)


class _AtIdx:

  def __init__(self, arr, idx):
    self.arr, self.idx = arr, idx

  def set(self, value):
    out = self.arr.clone()
    idx = self.idx
    if not isinstance(idx, tuple):
      idx = (idx,)
    idx = tuple(
        torch.as_tensor(np.asarray(i)) if isinstance(i, (list, np.ndarray)) else i
        for i in idx
    )
    if any(isinstance(i, torch.Tensor) and i.ndim > 0 for i in idx):
      # numpy / jax: an integer beside index arrays is itself an advanced index
      # (the broadcast dimensions then lead when a slice separates them)
      # (a one-element index array: torch would treat a 0-d tensor like the int)
      idx = tuple(torch.tensor([int(i)]) if isinstance(i, (int, np.integer)) else i for i in idx)
    value = torch.as_tensor(value)
    out[idx] = value.to(out.dtype)
    return JTensor.wrap(out)


def _tree_map(fn, tree):
  if isinstance(tree, (list, tuple)):
    return type(tree)(_tree_map(fn, t) for t in tree)
  if isinstance(tree, dict):
    return {k: _tree_map(fn, v) for k, v in tree.items()}
  return fn(tree)


def _mod(name):
  m = types.ModuleType(name)
  sys.modules[name] = m
  return m


def _unavailable(what):

  def f(*a, **k):
    raise RuntimeError(f"{what} is not emulated by the import shim")

  return f


class ShapeDtypeStruct:

  def __init__(self, shape, dtype):
    self.shape, self.dtype = tuple(shape), dtype


class Ref:
  """What a Pallas kernel body sees of one operand: a view of the block its
  BlockSpec selected.  `ref[...]` reads the block, `ref[...] = x` writes it
  through to the operand; `ref[i]` reads one element of a scalar-prefetch
  operand."""

  def __init__(self, view):
    self.value = view

  shape = property(lambda self: self.value.shape)
  dtype = property(lambda self: self.value.dtype)

  def __getitem__(self, idx):
    return JTensor.wrap(self.value[idx].clone())

  def __setitem__(self, idx, v):
    self.value[idx] = torch.as_tensor(v).to(self.value.dtype)


class BlockSpec:

  def __init__(self, block_shape=None, index_map=None):
    # the reference passes both by keyword
    self.block_shape, self.index_map = block_shape, index_map

  def select(self, operand, grid_pos, scalar_refs):
    """The block of `operand` for this grid position: a block index b along a
    dimension of block size n covers [b*n, (b+1)*n); a block size of None takes
    element b and drops the dimension."""
    index = self.index_map(*grid_pos, *scalar_refs)
    view = operand
    dim = 0
    for b, n in zip(index, self.block_shape):
      b = int(b)
      if n is None:
        view = view.select(dim, b)
      else:
        view = view.narrow(dim, b * n, n)
        dim += 1
    return Ref(view)


class PrefetchScalarGridSpec:

  def __init__(self, num_scalar_prefetch, grid, in_specs, out_specs):
    self.num_scalar_prefetch, self.grid = num_scalar_prefetch, tuple(grid)
    self.in_specs, self.out_specs = list(in_specs), list(out_specs)


_GRID_POS = []  # stack of grid positions of the pallas_call being interpreted


def pallas_call(kernel, grid_spec, out_shape, **_unused):
  """Sequential interpreter of a pallas_call with a PrefetchScalarGridSpec."""

  def run(*operands):
    import itertools

    n = grid_spec.num_scalar_prefetch
    scalars = [None if x is None else Ref(torch.as_tensor(x).as_subclass(torch.Tensor)) for x in operands[:n]]
    ins = [torch.as_tensor(x).as_subclass(torch.Tensor) for x in operands[n:]]
    assert len(ins) == len(grid_spec.in_specs)
    outs = [torch.zeros(tuple(o.shape), dtype=o.dtype) for o in out_shape]
    for pos in itertools.product(*[range(g) for g in grid_spec.grid]):
      _GRID_POS.append(pos)
      try:
        in_refs = [sp.select(x, pos, scalars) for sp, x in zip(grid_spec.in_specs, ins)]
        out_refs = [sp.select(x, pos, scalars) for sp, x in zip(grid_spec.out_specs, outs)]
        kernel(*scalars, *in_refs, *out_refs)
      finally:
        _GRID_POS.pop()
    return [JTensor.wrap(o) for o in outs]

  return run


def install():
  """Registers the stand-in modules in sys.modules (idempotent)."""
  if "jax" in sys.modules and getattr(sys.modules["jax"], "_IS_SHIM", False):
    return
  jax = _mod("jax")
  jax._IS_SHIM = True

  def jit(f=None, **_kw):
    if f is None:
      return lambda g: g
    return f

  jax.jit = jit
  jax.named_scope = lambda name: contextlib.nullcontext()
  jax.Array = torch.Tensor

  def vmap(fn, in_axes=0, out_axes=0):
    """Maps `fn` over one axis of the arguments whose in_axes entry is not None."""

    def mapped(*args):
      axes = in_axes if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
      n = next(a.shape[ax] for a, ax in zip(args, axes) if ax is not None)
      results = []
      for i in range(n):
        results.append(fn(*[a if ax is None else a.select(ax, i) for a, ax in zip(args, axes)]))

      def stack(items):
        if isinstance(items[0], (tuple, list)):
          return type(items[0])(stack([it[j] for it in items]) for j in range(len(items[0])))
        return JTensor.wrap(torch.stack(list(items), dim=out_axes))

      return stack(results)

    return mapped

  jax.vmap = vmap
  jax.default_device = lambda d: contextlib.nullcontext()
  jax.devices = lambda *a: ["cpu"]
  jax.config = types.SimpleNamespace(update=lambda *a, **k: None)
  jax.ShapeDtypeStruct = ShapeDtypeStruct

  tree_util = _mod("jax.tree_util")
  tree_util.register_pytree_node = lambda *a, **k: None
  tree_util.tree_map = _tree_map
  jax.tree_util = tree_util

  sharding = _mod("jax.sharding")

  class _Dummy:

    def __init__(self, *a, **k):
      pass

  sharding.Mesh = _Dummy
  sharding.PartitionSpec = _Dummy
  sharding.NamedSharding = _Dummy
  sharding.Sharding = _Dummy
  jax.sharding = sharding

  lax = _mod("jax.lax")

  def dynamic_update_slice(operand, update, start_indices):
    out = operand.clone()
    sl = []
    for s, n, full in zip(start_indices, update.shape, operand.shape):
      s = int(s)
      s = max(0, min(s, full - n))  # jax clamps start indices
      sl.append(slice(s, s + n))
    out[tuple(sl)] = update.to(out.dtype)
    return JTensor.wrap(out)

  def dynamic_slice_in_dim(operand, start_index, slice_size, axis=0):
    start_index = int(start_index)
    return JTensor.wrap(operand.narrow(axis, start_index, slice_size))

  lax.dynamic_update_slice = dynamic_update_slice
  lax.dynamic_slice_in_dim = dynamic_slice_in_dim
  lax.with_sharding_constraint = lambda x, s: x
  lax.div = lambda a, b: torch.div(a, b, rounding_mode="trunc")
  lax.cond = lambda p, t, f, *ops: t(*ops) if bool(p) else f(*ops)

  def dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
    (lc, rc), (lb, rb) = dimension_numbers
    assert not lb and not rb and len(lc) == 1 and len(rc) == 1
    out = torch.tensordot(lhs, rhs, dims=(list(lc), list(rc)))
    if preferred_element_type is not None:
      out = out.to(preferred_element_type)
    return JTensor.wrap(out)

  def broadcasted_iota(dtype, shape, dimension):
    view = [1] * len(shape)
    view[dimension] = shape[dimension]
    return JTensor.wrap(torch.arange(shape[dimension], dtype=dtype).reshape(view).expand(*shape))

  def broadcast_in_dim(operand, shape, broadcast_dimensions):
    view = [1] * len(shape)
    for src, dst in enumerate(broadcast_dimensions):
      view[dst] = operand.shape[src]
    return JTensor.wrap(operand.reshape(view).expand(*shape))

  lax.dot_general = dot_general
  lax.broadcasted_iota = broadcasted_iota
  lax.broadcast_in_dim = broadcast_in_dim
  jax.lax = lax

  rnd = _mod("jax.random")
  rnd.key = rnd.PRNGKey = rnd.split = rnd.uniform = rnd.normal = _unavailable(
      "jax.random"
  )
  jax.random = rnd

  jnp = _mod("jax.numpy")
  jnp.bfloat16, jnp.float32, jnp.float16 = (
      torch.bfloat16,
      torch.float32,
      torch.float16,
  )
  jnp.int8, jnp.int32, jnp.int64 = torch.int8, torch.int32, torch.int64
  jnp.inf = float("inf")
  jnp.ndarray = torch.Tensor

  def _w(fn):
    return lambda *a, **k: JTensor.wrap(fn(*a, **k))

  def _strip_device(k):
    k.pop("device", None)
    return k

  jnp.arange = lambda *a, **k: JTensor.wrap(torch.arange(*a, **_strip_device(k)))
  jnp.zeros = lambda shape, dtype=torch.float32, **k: JTensor.wrap(
      torch.zeros(tuple(shape), dtype=dtype)
  )
  jnp.ones = lambda shape, dtype=torch.float32, **k: JTensor.wrap(
      torch.ones(tuple(shape), dtype=dtype)
  )
  jnp.full = lambda shape, v, dtype=None, **k: JTensor.wrap(
      torch.full(tuple(shape), v, dtype=dtype)
  )
  jnp.asarray = jnp.array = lambda x, dtype=None: JTensor.wrap(
      torch.as_tensor(np.asarray(x) if not isinstance(x, torch.Tensor) else x)
      if dtype is None
      else torch.as_tensor(
          np.asarray(x) if not isinstance(x, torch.Tensor) else x
      ).to(dtype)
  )
  jnp.reshape = lambda x, shape: JTensor.wrap(x.reshape(tuple(shape)))
  jnp.squeeze = lambda x, axis=None: JTensor.wrap(
      x.squeeze() if axis is None else x.squeeze(axis)
  )
  def expand_dims(x, axis):
    for ax in sorted(axis) if isinstance(axis, (tuple, list)) else (axis,):
      x = x.unsqueeze(ax)
    return JTensor.wrap(x)

  jnp.expand_dims = expand_dims
  jnp.broadcast_to = lambda x, shape: JTensor.wrap(x.expand(*shape))
  jnp.ones_like = lambda x, **k: JTensor.wrap(torch.ones_like(_t(x)))
  jnp.transpose = lambda x, axes: JTensor.wrap(x.permute(*axes))
  def _t(x):
    return x.value if isinstance(x, Ref) else x

  def where(cond, a, b):
    cond = torch.as_tensor(_t(cond))
    if cond.dtype != torch.bool:
      cond = cond != 0
    return JTensor.wrap(torch.where(cond, _t(a), _t(b)))

  jnp.where = where
  jnp.logical_and = lambda a, b: JTensor.wrap(torch.logical_and(torch.as_tensor(a), torch.as_tensor(b)))
  jnp.logical_or = lambda a, b: JTensor.wrap(torch.logical_or(torch.as_tensor(a), torch.as_tensor(b)))
  jnp.exp = _w(torch.exp)
  jnp.sqrt = lambda x: math.sqrt(x) if isinstance(x, (int, float)) else JTensor.wrap(torch.sqrt(x))
  jnp.maximum = _w(torch.maximum)
  jnp.dot = _w(torch.matmul)
  jnp.full_like = lambda x, v, **k: JTensor.wrap(torch.full_like(_t(x), v))
  jnp.array_equal = lambda a, b: bool(
      torch.equal(torch.as_tensor(a).float(), torch.as_tensor(b).float())
  )
  jnp.zeros_like = lambda x, **k: JTensor.wrap(torch.zeros_like(_t(x)))
  jnp.concatenate = lambda xs, axis=0: JTensor.wrap(torch.cat(list(xs), axis))

  def pad(array, pad_width, mode="constant"):
    assert mode == "constant"
    flat = []
    for lo, hi in reversed(pad_width):
      flat += [lo, hi]
    return JTensor.wrap(torch.nn.functional.pad(array, flat))

  jnp.pad = pad
  jax.numpy = jnp

  exp = _mod("jax.experimental")
  jax.experimental = exp
  pallas = _mod("jax.experimental.pallas")
  pallas.pallas_call = pallas_call
  pallas.program_id = lambda axis: _GRID_POS[-1][axis]
  pallas.when = lambda cond: (lambda fn: fn() if bool(cond) else None)
  pallas.BlockSpec = BlockSpec
  exp.pallas = pallas
  tpu = _mod("jax.experimental.pallas.tpu")
  tpu.PrefetchScalarGridSpec = PrefetchScalarGridSpec
  pallas.tpu = tpu
  _mod("jax.experimental.pallas.ops")
  _mod("jax.experimental.pallas.ops.tpu")
  _mod("jax.experimental.pallas.ops.tpu.paged_attention")
  pak = _mod(
      "jax.experimental.pallas.ops.tpu.paged_attention.paged_attention_kernel"
  )
  pak.paged_attention = _unavailable("pallas paged_attention")
  sm = _mod("jax.experimental.shard_map")
  sm.shard_map = lambda f, mesh=None, in_specs=None, out_specs=None, **k: f
  exp.shard_map = sm

  x2 = _mod("torch_xla2")

  class _Env:

    def __enter__(self):
      return self

    def __exit__(self, *a):
      return False

    def j2t_iso(self, tree):
      return _tree_map(JTensor.wrap, tree)

    t2j_iso = j2t_iso
    to_xla = j2t_iso

  _env = _Env()
  x2.default_env = lambda: _env
  interop = _mod("torch_xla2.interop")
  interop.call_jax = lambda f, *a, **k: f(*a, **k)
  interop.call_torch = lambda f, *a, **k: f(*a, **k)
  x2.interop = interop
  tensor = _mod("torch_xla2.tensor")
  tensor.XLATensor2 = JTensor
  tensor.t2j = JTensor.wrap
  tensor.j2t = JTensor.wrap
  x2.tensor = tensor


def import_reference(reference_root):
  """Returns (cache_manager, page_attention_manager, attention_kernel, quantize)
  imported from `<reference_root>/jetstream_pt` with the shim installed."""
  install()
  if reference_root not in sys.path:
    sys.path.insert(0, reference_root)
  # The package __init__ pulls in the serving engine (absent dependencies);
  # register an empty package object so only the submodules asked for load.
  import importlib
  import os

  pkg = types.ModuleType("jetstream_pt")
  pkg.__path__ = [os.path.join(reference_root, "jetstream_pt")]
  sys.modules["jetstream_pt"] = pkg
  mods = []
  for name in (
      "torchjax",
      "quantize",
      "page_attention_manager",
      "cache_manager",
      "attention_kernel",
  ):
    mods.append(importlib.import_module(f"jetstream_pt.{name}"))
  _, quantize, pam, cm, ak = mods
  return cm, pam, ak, quantize


class _AnyModule(types.ModuleType):
  """Module whose every attribute is a placeholder class: enough for `import x`,
  `class C(x.Base)` and annotations that name x.Something."""

  def __getattr__(self, name):
    if name.startswith("__"):
      raise AttributeError(name)
    cls = type(name, (), {"__init__": lambda self, *a, **k: None, "__class_getitem__": classmethod(lambda c, i: c)})
    setattr(self, name, cls)
    return cls


def import_reference_engine(reference_root):
  """Returns the reference's `jetstream_pt.engine` module.  Its insert functions
  (`PyTorchEngine._insert_no_wrap`, `_insert_wrap`, `insert`) are jnp code on
  arrays; everything else the module imports (serving API, tokenizers, model
  definitions, flax, etils) is replaced by placeholder modules and never run."""
  import dataclasses
  import importlib

  import_reference(reference_root)
  for name in ("etils", "etils.epath", "flax", "jetstream", "jetstream.engine", "jetstream.engine.engine_api",
               "jetstream.engine.tokenizer_api", "jetstream.engine.tokenizer_pb2", "jetstream.engine.token_utils",
               "jetstream.engine.sampling_utils", "jetstream_pt.hf_tokenizer", "jetstream_pt.environment",
               "jetstream_pt.third_party", "jetstream_pt.third_party.llama",
               "jetstream_pt.third_party.llama.model_exportable", "jetstream_pt.third_party.llama.model_args",
               "jetstream_pt.third_party.gemma", "jetstream_pt.third_party.gemma.config",
               "jetstream_pt.third_party.gemma.model", "jetstream_pt.third_party.mixtral",
               "jetstream_pt.third_party.mixtral.config", "jetstream_pt.third_party.mixtral.model"):
    if name not in sys.modules:
      sys.modules[name] = _AnyModule(name)
      parent, _, child = name.rpartition(".")
      if parent and parent in sys.modules:
        setattr(sys.modules[parent], child, sys.modules[name])
  sys.modules["flax"].struct = types.SimpleNamespace(dataclass=dataclasses.dataclass)
  return importlib.import_module("jetstream_pt.engine")


def import_reference_layers(reference_root):
  """Returns the reference's `jetstream_pt.layers` module (for its quantised
  linear layer).  `jetstream_pt.environment` cannot be imported under Python
  3.12 (a dataclass field with an unhashable dataclass default), so the one name
  layers.py takes from it, the `QuantizationConfig` record, is provided here with
  the same fields and defaults (environment.py:31-40); absl and model_base are
  placeholders."""
  import dataclasses
  import importlib

  import_reference(reference_root)
  for name in ("absl", "absl.flags", "jetstream_pt.model_base"):
    if name not in sys.modules:
      sys.modules[name] = _AnyModule(name)

  @dataclasses.dataclass(frozen=True)
  class QuantizationConfig:
    enable_weight_quantization: bool = False
    num_bits_weight: int = 8
    is_blockwise_weight: bool = False
    block_size_weight: int = 128
    is_symmetric_weight: bool = True
    enable_activation_quantization: bool = False
    enable_kv_quantization: bool = False
    exclude_layers: object = None

  env = sys.modules.get("jetstream_pt.environment")
  if env is None or isinstance(env, _AnyModule):
    env = types.ModuleType("jetstream_pt.environment")
    sys.modules["jetstream_pt.environment"] = env
  env.QuantizationConfig = QuantizationConfig
  return importlib.import_module("jetstream_pt.layers")
