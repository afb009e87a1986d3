"""Benchmark of the KV-cache hot path: int8 quantise+append followed by ragged
decode attention, Llama-2-70B-shaped (batch 96, 64 query / 8 KV heads, head_dim
128, cache length 2048, int8 KV with per-token scales, per-sequence lengths
uniform in [1, 2048]), over NL layers that each own their cache buffers.

One "step" = one decode step of the KV path through all NL layers (per layer:
fused quantise+append of the new token, then ragged attention over the
sequence's valid range, split-K merged).  tokens/s = batch / step time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (under torchrun): KV heads are sharded across ranks like the reference's
default sharding; per layer the ranks max-reduce the per-token amax (NCCL) so
codes and scales equal the single-GPU ones.  Inputs are seeded synthetic data.
"""

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

B, HQ, HKV, D, S = 96, 64, 8, 128, 2048
METRIC = "decode KV update+attention tokens/s"
UNIT = "tokens/s"
WORKLOAD = "ragged int8 decode, Llama-2-70B-shaped GQA (B=96, 64q/8kv heads, D=128, S=2048, lens~U[1,2048])"


def peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      return float(json.load(f)["hbm_gbs"]), "measured"
  return 6650.0, "fallback"


def make_lengths(seed=1002):
  g = torch.Generator().manual_seed(seed)
  return torch.randint(1, S + 1, (B,), generator=g)  # valid tokens AFTER the append


def attention_bytes(lens, hkv):
  n = int(lens.sum())
  return n * hkv * D * 2 + n * 2 * 2 + 2 * B * (HQ * hkv // HKV) * D * 2 + B * (HQ * hkv // HKV) * 8


def append_bytes(hkv):
  return 2 * B * hkv * D * 2 + 2 * B * hkv * D * 1 * 2 + 2 * B * 2 * 2


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------


class ClockSampler(threading.Thread):
  """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

  REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

  def __init__(self, index):
    super().__init__(daemon=True)
    self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
    self._stop_evt = threading.Event()
    self.ok = False
    try:
      import pynvml

      pynvml.nvmlInit()
      self.nv = pynvml
      try:
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
      except Exception:  # pylint: disable=broad-except
        self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
      self._reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
          pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
      self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
      self.ok = True
    except Exception:  # pylint: disable=broad-except
      self.ok = False

  def run(self):
    while self.ok and not self._stop_evt.is_set():
      try:
        self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
        bits = self._reasons_fn(self.h)
        for bit, name in self.REASONS.items():
          if bits & bit:
            self.reasons.add(name)
      except Exception:  # pylint: disable=broad-except
        break
      time.sleep(0.02)

  def stop(self):
    self._stop_evt.set()
    if self.is_alive():
      self.join(timeout=2)
    return {
        "sm_mhz": statistics.median(self.samples) if self.samples else None,
        "sm_max_mhz": self.max_mhz,
        "reasons": sorted(self.reasons),
        "samples": len(self.samples),
    }


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on the host cores
# ---------------------------------------------------------------------------


def cpu_layer_inputs(seed):
  g = torch.Generator().manual_seed(seed)
  ck = torch.randint(-127, 128, (B, HKV, S, D), generator=g, dtype=torch.int8)
  cv = torch.randint(-127, 128, (B, HKV, S, D), generator=g, dtype=torch.int8)
  ks = (torch.rand(B, 1, S, 1, generator=g) * 0.03 + 0.01).to(torch.bfloat16)
  vs = (torch.rand(B, 1, S, 1, generator=g) * 0.03 + 0.01).to(torch.bfloat16)
  q = torch.randn(B, HQ, 1, D, generator=g).to(torch.bfloat16)
  xk = torch.randn(B, HKV, 1, D, generator=g).to(torch.bfloat16)
  xv = torch.randn(B, HKV, 1, D, generator=g).to(torch.bfloat16)
  return ck, cv, ks, vs, q, xk, xv


def cpu_layer_step(inputs, lens):
  """One layer of the workload on the CPU oracle: update (per-slot write) then
  left-aligned ragged attention."""
  from oracle import attention as oa
  from oracle import cache as oc

  ck, cv, ks, vs, q, xk, xv = inputs
  pos = lens - 1
  r = oc.int8_update(ck, cv, ks, vs, xk, xv, pos, ring_buffer=False, lazy=False)
  o, (m, l) = oa.ragged_mha(q, r[0], r[1], 0, torch.zeros(B, dtype=torch.int64), lens, r[4], r[5])
  return o


def time_cpu(layers_per_step, steps, warmup, nl):
  torch.set_num_threads(os.cpu_count())
  lens = make_lengths()
  inputs = cpu_layer_inputs(7)
  for _ in range(warmup):
    cpu_layer_step(inputs, lens)
  t0 = time.perf_counter()
  for _ in range(steps):
    for _ in range(layers_per_step):
      cpu_layer_step(inputs, lens)
  dt = (time.perf_counter() - t0) / steps
  per_layer = dt / layers_per_step
  return B / (per_layer * nl), dt * 1e3, per_layer


def run_reference(args):
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  nl = args.layers
  steps = max(1, min(args.steps, 5))
  warmup = max(1, min(args.warmup, 1))
  value, ms, per_layer = time_cpu(1, steps, warmup, nl)
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
      "steps": steps, "warmup": warmup, "ms_per_step": per_layer * nl * 1e3, "higher_is_better": True,
      "scaling": "strong", "vs_baseline": None, "dtype": "int8 KV / bf16 q / fp32 accumulate", "data": "synthetic",
      "config": {"workload": WORKLOAD, "layers": nl, "global_batch": B},
      "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                       "sample": f"1 of {nl} layers per step (all 96 sequences), {steps} steps; tokens/s "
                                 f"extrapolated to {nl} layers"},
      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "note": "the reference needs JAX / torch_xla2, absent here: this is the torch-CPU restatement of its "
              "update + ragged attention (oracle/), all host threads",
  }
  print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# CUDA arm
# ---------------------------------------------------------------------------


def run_insert_burst(args, dev):
  """BASELINE config 4: 64 prefill inserts, each scattering and quantising a prefix of
  L in {128..2048} tokens x 32 layers into pages of an int8 paged cache (batch 128,
  page size 64).  The whole burst (2048 launches) replays as one CUDA graph; the line
  reports the HBM rate of the fused quantise + scatter against its algorithmic bytes."""
  import numpy as np
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  nl, bi, ps, hk, maxp, n_ins = min(32, args.layers), 128, 64, HKV, 32, 64  # --layers below 32 shrinks the case (profiling)
  pages = bi * maxp
  rng = np.random.RandomState(1004)
  lens = rng.choice([128, 256, 512, 1024, 2048], size=n_ins)
  gen = torch.Generator(device=dev).manual_seed(1004)
  # layers are views of stacked tensors, as a serving engine keeps them: the insert is then one launch per prefix
  pre_k = torch.randn((nl, 1, hk, 2048, D), generator=gen, device=dev).to(torch.bfloat16)
  pre_v = torch.randn((nl, 1, hk, 2048, D), generator=gen, device=dev).to(torch.bfloat16)
  pool_k = torch.zeros((nl, hk, pages, ps, D), dtype=torch.int8, device=dev)
  pool_v = torch.zeros((nl, hk, pages, ps, D), dtype=torch.int8, device=dev)
  sc_k = torch.zeros((nl, 1, pages, ps, 1), dtype=torch.bfloat16, device=dev)
  sc_v = torch.zeros((nl, 1, pages, ps, 1), dtype=torch.bfloat16, device=dev)
  pre = [(pre_k[i], pre_v[i]) for i in range(nl)]
  pools = [(pool_k[i], pool_v[i]) for i in range(nl)]
  scales = [(sc_k[i], sc_v[i]) for i in range(nl)]
  launches0 = _lib.lib().jpt_launch_count()
  pam = PageAttentionManager(bi, pages, ps, maxp, free_page_order=rng.permutation(pages))
  plan = []
  nbytes = 0
  for j, L in enumerate(lens):
    L = int(L)
    n_pages, idx = pam.reserve_pages_insert(j, L)
    plan.append((L, torch.as_tensor(np.asarray(idx), dtype=torch.int32, device=dev)))
    nbytes += nl * (2 * L * hk * D * 2 + 2 * n_pages * ps * hk * D + 2 * n_pages * ps * 2)

  def burst():
    for L, upd in plan:
      pam.insert_prefill_cache([(k[:, :, :L], v[:, :, :L]) for k, v in pre], pools, upd, decode_scales=scales)

  burst()
  torch.cuda.synchronize()
  launches = _lib.lib().jpt_launch_count() - launches0
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph):
    burst()
  for _ in range(max(3, args.warmup)):
    graph.replay()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(args.steps):
    graph.replay()
  e1.record()
  torch.cuda.synchronize()
  ms = e0.elapsed_time(e1) / args.steps
  peak, kind = peaks()
  gbs = nbytes / (ms * 1e-3) / 1e9
  print(json.dumps({"only": "insert", "layers": nl, "workload": "64 inserts x 32 layers (or --layers), L in {128,256,512,1024,2048}, int8 paged "
                    "cache (batch 128, page 64, 8 kv heads, D=128), quantise on insert", "launches_per_burst": int(launches),
                    "tokens_per_burst": int(lens.sum()), "ms_per_burst": ms, "algorithmic_bytes": nbytes,
                    "achieved_gbs": gbs, "peak": peak, "peak_kind": kind, "frac": gbs / peak,
                    "inserts_per_s": n_ins / (ms * 1e-3)}), flush=True)


def run_cuda(args):
  import torch.distributed as dist

  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if world != args.gpus:
    raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  if HKV % world:
    raise SystemExit("KV heads (8) must divide by the number of GPUs")
  hkv, hq = HKV // world, HQ // world
  nl = args.layers
  lib = _lib.lib()
  if args.only == "insert":
    run_insert_burst(args, dev)
    return

  # ---- device-resident state: every layer owns its cache (>> L2 in total)
  lens = make_lengths()
  lens_d = lens.to(dev, torch.int32)
  pos_d = (lens - 1).to(dev, torch.int32)
  gen = torch.Generator(device=dev).manual_seed(1002 + rank)
  ck = torch.empty((nl, B, hkv, S, D), dtype=torch.int8, device=dev)
  cv = torch.empty((nl, B, hkv, S, D), dtype=torch.int8, device=dev)
  for i in range(nl):
    ck[i] = torch.randint(-127, 128, (B, hkv, S, D), generator=gen, device=dev, dtype=torch.int8)
    cv[i] = torch.randint(-127, 128, (B, hkv, S, D), generator=gen, device=dev, dtype=torch.int8)
  sgen = torch.Generator(device=dev).manual_seed(77)  # scales are replicated across ranks
  ks = (torch.rand((nl, B, 1, S, 1), generator=sgen, device=dev) * 0.03 + 0.01).to(torch.bfloat16)
  vs = (torch.rand((nl, B, 1, S, 1), generator=sgen, device=dev) * 0.03 + 0.01).to(torch.bfloat16)
  hq_all = torch.randn((nl, B, hq, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  hk_all = torch.randn((nl, B, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  hv_all = torch.randn((nl, B, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)

  data = JetEngineEnvironmentData(batch_size=B, cache_sequence_length=S, num_layers=nl, ring_buffer=False,
                                  testing=True, cache_shape=(B, hkv, S, D))
  data.quant_config.enable_kv_quantization = True
  env = JetEngineEnvironment(data, device=dev, rank=rank, world_size=world)  # eager per-slot writes, unstacked
  caches = [Int8KVCacheGenerate(ck[i], cv[i], ks[i], vs[i], pos_d, env=env) for i in range(nl)]
  start_d = torch.zeros(B, dtype=torch.int32, device=dev)

  # Head-sharded scales need the amax over all ranks: inside the append launch over NVLink
  # peer memory (default), or as local_amax + NCCL all_reduce(MAX) + update (--amax-exchange nccl).
  px = None
  if world > 1 and args.amax_exchange == "peers":
    from jetstream_pytorch_b200.cache_manager import PeerAmaxExchange
    px = PeerAmaxExchange.with_torch_distributed(B)

  def layer_step(i, q, xk, xv):
    amax = None
    if world > 1 and px is None:
      amax = caches[i].local_amax(xk, xv)
      dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    r = caches[i].update(xk, xv, i, amax=amax, peers=px)
    o, _ = ak.ragged_mha(q, r[0], r[1], i, start_d, lens_d, None, None, r[4], r[5])
    return o

  def device_step():
    out = None
    for i in range(nl):
      out = layer_step(i, hq_all[i], hk_all[i], hv_all[i])
    return out

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  if args.only:
    # One kernel alone, launched eagerly: the command line for profiler captures.
    fg = 2 if args.attn_kernel == "mma" else 0  # the mma.sync kernel instead of the tcgen05 one
    if args.only == "attention" and args.kv == "bf16":  # the same shape with an unquantised cache
      ckb = torch.randn((nl, B, hkv, S, D), generator=gen, device=dev, dtype=torch.bfloat16)
      cvb = torch.randn((nl, B, hkv, S, D), generator=gen, device=dev, dtype=torch.bfloat16)

    def only_fn():
      for i in range(nl):
        if args.only == "attention" and args.kv == "bf16":
          ak.ragged_mha(hq_all[i], ckb[i], cvb[i], i, start_d, lens_d, None, None, None, None)
        elif args.only == "attention":
          ak.ragged_mha(hq_all[i], ck[i], cv[i], i, start_d, lens_d, None, None, ks[i], vs[i], force_generic=fg)
        else:
          caches[i].update(hk_all[i], hv_all[i], i)
    for _ in range(max(3, args.warmup)):
      only_fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
      only_fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.steps * nl)
    nbytes = attention_bytes(lens, hkv) if args.only == "attention" else append_bytes(hkv)
    if args.only == "attention" and args.kv == "bf16":
      nbytes = int(lens.sum()) * hkv * D * 2 * 2 + 2 * B * hq * D * 2
    # eager launches: for kernels shorter than the host's ~35 us per call this is the host's pace, not the kernel's
    print(json.dumps({"only": args.only, "kv": args.kv, "attn_kernel": args.attn_kernel, "layers": nl,
                      "launches": nl * (args.steps + max(3, args.warmup)), "us_per_eager_call": us,
                      "algorithmic_bytes": nbytes, "gbs_at_that_pace": nbytes / us / 1e3}), flush=True)
    return

  # ---- warm-up (also sizes the split-K workspace), then try a CUDA graph of one step
  for _ in range(max(3, args.warmup)):
    device_step()
  torch.cuda.synchronize()
  graph = None
  if not args.no_graph:  # with N > 1 the NCCL max-reductions are captured too
    try:
      graph = torch.cuda.CUDAGraph()
      with torch.cuda.graph(graph):
        device_step()
      graph.replay()
      torch.cuda.synchronize()
    except Exception as e:  # pylint: disable=broad-except
      print(f"[bench] CUDA graph capture unavailable ({e}); timing eager launches", file=sys.stderr)
      graph = None
      torch.cuda.synchronize()

  def timed_steps(fn, k):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(k):
      fn()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
      t = torch.tensor([ms], device=dev)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      ms = float(t.item())
    return ms / k

  step_fn = graph.replay if graph is not None else device_step
  sampler = ClockSampler(local_rank)
  sampler.start()
  launches0 = lib.jpt_launch_count()
  ms_step = timed_steps(step_fn, args.steps)
  launches = lib.jpt_launch_count() - launches0
  if graph is not None:
    # replays do not pass through the library: count the launches captured in one step
    c0 = lib.jpt_launch_count()
    device_step()
    torch.cuda.synchronize()
    launches = (lib.jpt_launch_count() - c0) * args.steps

  # ---- per-kernel timing for the roofline: attention only, then append only
  def attn_only():
    for i in range(nl):
      ak.ragged_mha(hq_all[i], ck[i], cv[i], i, start_d, lens_d, None, None, ks[i], vs[i])

  def append_only():
    for i in range(nl):
      caches[i].update(hk_all[i], hv_all[i], i)

  reps = max(1, args.steps // 2)
  attn_fn, app_fn = attn_only, append_only
  if not args.no_graph and graph is not None:
    try:
      g_attn, g_app = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
      attn_only(); append_only(); torch.cuda.synchronize()
      with torch.cuda.graph(g_attn):
        attn_only()
      with torch.cuda.graph(g_app):
        append_only()
      attn_fn, app_fn = g_attn.replay, g_app.replay
    except Exception:  # pylint: disable=broad-except
      torch.cuda.synchronize()
  for _ in range(3):
    attn_fn(); app_fn()
  ms_attn = timed_steps(attn_fn, reps) / nl
  ms_app = timed_steps(app_fn, reps) / nl
  clocks = sampler.stop()

  # ---- end to end through the public API with HOST buffers
  q_h = hq_all.cpu().pin_memory()
  k_h = hk_all.cpu().pin_memory()
  v_h = hv_all.cpu().pin_memory()
  o_h = torch.empty((nl, B, hq, 1, D), dtype=torch.bfloat16).pin_memory()
  q_s, k_s, v_s = torch.empty_like(hq_all), torch.empty_like(hk_all), torch.empty_like(hv_all)
  o_s = torch.empty((nl, B, hq, 1, D), dtype=torch.bfloat16, device=dev)
  copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
  compute = torch.cuda.current_stream()
  chunk = max(1, nl // 8)

  def e2e_step():
    """Layers are pipelined in chunks: H2D of chunk c+1 and D2H of chunk c-1
    overlap the kernels of chunk c."""
    in_evt = []
    copy_in.wait_stream(compute)
    with torch.cuda.stream(copy_in):
      for c0 in range(0, nl, chunk):
        sl = slice(c0, min(nl, c0 + chunk))
        q_s[sl].copy_(q_h[sl], non_blocking=True)
        k_s[sl].copy_(k_h[sl], non_blocking=True)
        v_s[sl].copy_(v_h[sl], non_blocking=True)
        e = torch.cuda.Event()
        e.record(copy_in)
        in_evt.append(e)
    for ci, c0 in enumerate(range(0, nl, chunk)):
      compute.wait_event(in_evt[ci])
      for i in range(c0, min(nl, c0 + chunk)):
        o_s[i].copy_(layer_step(i, q_s[i], k_s[i], v_s[i]).reshape(B, hq, 1, D))
      e = torch.cuda.Event()
      e.record(compute)
      copy_out.wait_event(e)
      with torch.cuda.stream(copy_out):
        sl = slice(c0, min(nl, c0 + chunk))
        o_h[sl].copy_(o_s[sl], non_blocking=True)
    compute.wait_stream(copy_out)
    compute.wait_stream(copy_in)

  for _ in range(2):
    e2e_step()
  ms_e2e = timed_steps(e2e_step, max(2, args.steps // 2))
  h2d = q_h.numel() * 2 + k_h.numel() * 2 + v_h.numel() * 2
  d2h = o_h.numel() * 2

  def leave():
    """Ranks leave together.  With NCCL work captured in CUDA graphs the process
    group teardown has been seen to block, so multi-rank runs skip it and exit
    once every rank has finished its GPU work."""
    if world > 1:
      torch.cuda.synchronize()
      dist.barrier()
      torch.cuda.synchronize()
      sys.stdout.flush()
      sys.stderr.flush()
      os._exit(0)

  if rank != 0:
    leave()
    return

  peak, peak_kind = peaks()
  a_bytes = attention_bytes(lens, hkv)
  achieved = a_bytes / (ms_attn * 1e-3) / 1e9
  app_gbs = append_bytes(hkv) / (ms_app * 1e-3) / 1e9
  line = {
      "metric": METRIC, "value": B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
      "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
      "vs_baseline": None, "dtype": "int8 KV / bf16 q / fp32 accumulate", "data": "synthetic",
      "config": {"workload": WORKLOAD, "layers": nl, "global_batch": B, "kv_heads_per_gpu": hkv,
                 "parallelism": f"kv-head sharding x{world}",
                 "amax_exchange": ("in-kernel over NVLink peer memory" if px is not None else
                                   ("nccl all_reduce" if world > 1 else "none")),
                 "peer_exchange_status": (px.status() if px is not None else None), "l2": "each layer has its own cache buffers "
                 f"({2 * B * hkv * S * D * nl / 2**30:.1f} GiB per GPU in total, >> 126 MB L2)",
                 "cuda_graph": graph is not None},
      "us_per_layer": ms_step * 1e3 / nl,
      "roofline": {"bound": "hbm", "kernel": "flash_decode_i8_umma_kernel (tcgen05; pieces merged in-kernel)", "achieved": achieved, "peak": peak,
                   "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                   "frac_of_8000_nominal": achieved / 8000.0, "algorithmic_bytes_per_launch": a_bytes,
                   "us_per_launch": ms_attn * 1e3,
                   # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload on one GPU
                   # (ncu capture summarised in profiles/flash_decode_i8_umma__ragged_llama2_70b_b96_s2048.md)
                   "traffic": 194.54e6 if world == 1 else None},
      "kernels": {"kv_quant_append": {"us_per_launch": ms_app * 1e3, "algorithmic_bytes": append_bytes(hkv),
                                      "achieved_gbs": app_gbs}},
      "e2e": {"value": B / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
              "d2h_bytes_per_step": d2h},
      "gpu_launches": int(launches),
      "clocks": clocks,
  }
  if world == 1 and not args.no_cpu_baseline:
    v, _, per_layer = time_cpu(1, 3, 1, nl)
    line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                            "sample": f"1 of {nl} layers (all 96 sequences) x 3 repeats, {per_layer:.2f} s per "
                                      f"layer; tokens/s extrapolated to {nl} layers"}
  print(json.dumps(line), flush=True)
  leave()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
  ap.add_argument("--layers", type=int, default=80)
  ap.add_argument("--no-graph", action="store_true")
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--amax-exchange", choices=["peers", "nccl"], default="peers",
                  help="N > 1: how the per-token amax is max-reduced over the ranks")
  ap.add_argument("--only", choices=["attention", "append", "insert"], default=None,
                  help="launch just this kernel (no graph, no end-to-end leg): for profiler captures")
  ap.add_argument("--kv", choices=["int8", "bf16"], default="int8", help="with --only attention: cache dtype")
  ap.add_argument("--attn-kernel", choices=["auto", "mma"], default="auto",
                  help="with --only attention: 'mma' forces the mma.sync kernel for the int8 cache")
  args = ap.parse_args()
  if args.impl == "reference":
    run_reference(args)
  else:
    run_cuda(args)


if __name__ == "__main__":
  main()
