"""Benchmark of the KV-cache hot path: int8 quantise+append followed by ragged
decode attention, Llama-2-70B-shaped (batch 96, 64 query / 8 KV heads, head_dim
128, cache length 2048, int8 KV with per-token scales, per-sequence lengths
uniform in [1, 2048]), over NL layers that each own their cache buffers.

One "step" = one decode step of the KV path through all NL layers (per layer:
the quantise+append launch of the new token, then the ragged attention launch
over the sequence's valid range, split pieces merged in-kernel; or both in one
launch, jpt_decode_update_attend: the default when the KV heads are sharded,
where it hides the amax exchange; `--fused` / `--unfused` choose).  tokens/s =
batch / step time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (under torchrun): KV heads are sharded across ranks like the reference's
default sharding; the per-token amax is max-reduced over the ranks inside the
append launch (NVLink peer memory), so codes and scales equal the single-GPU
ones; the line's `parity` key reports the check of exactly that against the CPU
oracle.  At N = 1 the line also carries `kernels`: the other workloads of the
path (dense int8 MHA decode, paged bf16 decode, the prefill-insert burst, the
bf16 cache of the same shape, the ring sub-case), each timed alone.
Inputs are seeded synthetic data.
"""

import argparse
import hashlib
import json
import os
import re
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
DTYPE = "int8 KV / bf16 q / fp32 accumulate"
ATTENTION_PROFILE = os.path.join(ROOT, "profiles", "flash_decode_i8_umma__ragged_llama2_70b_b96_s2048.md")
ATTENTION_SOURCE = os.path.join(ROOT, "jetstream_pytorch_b200", "csrc", "attention_umma.cu")


def peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      return float(json.load(f)["hbm_gbs"]), "measured"
  return 6650.0, "fallback"


def make_lengths(seed=1002):
  g = torch.Generator().manual_seed(seed)
  return torch.randint(1, S + 1, (B,), generator=g)  # valid tokens AFTER the append


def make_ring_ranges(seed=1003):
  """start, end uniform over the ring, wrap allowed, never start == end (that means empty)."""
  g = torch.Generator().manual_seed(seed)
  start = torch.randint(0, S, (B,), generator=g)
  end = torch.randint(0, S, (B,), generator=g)
  end = torch.where(end == start, (end + 1) % S, end)
  n = torch.where(start < end, end - start, S - start + end)
  return start, end, n


def attention_bytes(tokens, batch, hq, hkv, kv_bytes=1, scales=True, ml=True):
  """K and V rows of the valid tokens, their scales once, q in, o (and m, l) out."""
  n = int(tokens)
  out = n * hkv * D * 2 * kv_bytes + 2 * batch * hq * D * 2
  if scales:
    out += n * 2 * 2
  if ml:
    out += batch * hq * 8
  return out


def append_bytes(batch, hkv):
  return 2 * batch * hkv * D * 2 + 2 * batch * hkv * D * 1 * 2 + 2 * batch * 2 * 2


def profiled_traffic():
  """DRAM bytes one attention launch of this workload moved in the committed
  profiler summary, or (None, why) when the kernel source changed since."""
  try:
    text = open(ATTENTION_PROFILE).read()
    traffic = re.search(r"traffic_bytes_per_launch:\s*([0-9.e+]+)", text)
    sha = re.search(r"kernel_source_sha256:\s*([0-9a-f]+)", text)
    if not traffic or not sha:
      return None, "the profile summary does not state it"
    now = hashlib.sha256(open(ATTENTION_SOURCE, "rb").read()).hexdigest()
    if not now.startswith(sha.group(1)):
      return None, "the kernel source changed after the profiler capture"
    return float(traffic.group(1)), "profiler capture of one launch of this workload"
  except OSError as e:
    return None, str(e)


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


def cpu_layer_inputs(layer):
  """Seeded inputs of one layer, all 8 KV heads, on the host.  The CUDA arm
  uploads layer 0 from here (each rank its own heads), so the two arms and the
  parity check work on the same numbers."""
  g = torch.Generator().manual_seed(7000 + layer)
  ck = torch.randint(-127, 128, (B, HKV, S, D), generator=g, dtype=torch.int8)
  cv = torch.randint(-127, 128, (B, HKV, S, D), generator=g, dtype=torch.int8)
  ks = (torch.rand(B, 1, S, 1, generator=g) * 0.0075 + 0.0025).to(torch.bfloat16)
  vs = (torch.rand(B, 1, S, 1, generator=g) * 0.0075 + 0.0025).to(torch.bfloat16)
  q = torch.randn(B, HQ, 1, D, generator=g).to(torch.bfloat16)
  xk = torch.randn(B, HKV, 1, D, generator=g).to(torch.bfloat16)
  xv = torch.randn(B, HKV, 1, D, generator=g).to(torch.bfloat16)
  return ck, cv, ks, vs, q, xk, xv


def cpu_layer_step(inputs, lens):
  """One layer of the workload on the CPU oracle: update (per-slot write) then
  left-aligned ragged attention.  Returns the update's 8-tuple and (o, m, l)."""
  from oracle import attention as oa
  from oracle import cache as oc

  ck, cv, ks, vs, q, xk, xv = inputs
  pos = lens - 1
  r = oc.int8_update(ck, cv, ks, vs, xk, xv, pos, ring_buffer=False, lazy=False)
  o, (m, l) = oa.ragged_mha(q, r[0], r[1], 0, torch.zeros(B, dtype=torch.int64), lens, r[4], r[5])
  return r, (o, m, l)


def run_reference(args):
  """The reference's CPU path (its torch-CPU restatement: the reference itself
  needs JAX) on all host threads.  A step of this arm is a bounded sample of
  the workload's step: `layers_timed_per_step` of the NL layers (all 96
  sequences each), chosen so that the steps asked for end within about a
  minute; `value` scales the measured step to NL layers and `scaled_from` says
  by how much."""
  if int(os.environ.get("RANK", "0")) != 0:
    return
  torch.set_num_threads(os.cpu_count())
  nl, steps, warmup = args.layers, max(1, args.steps), max(0, args.warmup)
  lens = make_lengths()
  inputs = cpu_layer_inputs(0)
  t0 = time.perf_counter()
  cpu_layer_step(inputs, lens)  # untimed: first touch of the buffers, thread pool start
  t_one = time.perf_counter() - t0
  per_step = max(1, min(nl, int(60.0 / ((steps + warmup) * max(t_one, 1e-3)))))
  def step():
    for _ in range(per_step):
      cpu_layer_step(inputs, lens)
  for _ in range(warmup):
    step()
  t0 = time.perf_counter()
  for _ in range(steps):
    step()
  ms_sample = (time.perf_counter() - t0) / steps * 1e3
  factor = nl / per_step
  value = B / (ms_sample * factor * 1e-3)
  line = {
      "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
      "steps": steps, "warmup": warmup, "ms_per_step": ms_sample, "higher_is_better": True,
      "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
      "config": {"workload": WORKLOAD, "layers": nl, "global_batch": B},
      "scaled_from": {"layers_timed_per_step": per_step, "layers": nl, "factor": factor,
                      "note": "ms_per_step is the time of the sample actually run; value = batch / (ms_per_step x factor)"},
      "cpu_baseline": {"value": value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                       "sample": f"{per_step} of {nl} layers per step (all 96 sequences, the seeded inputs of layer 0 "
                                 f"of the CUDA arm), {steps} steps after {warmup} warm-up steps"},
      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "note": "the reference needs JAX / torch_xla2, absent here: this is the torch-CPU restatement of its "
              "update + ragged attention (oracle/), all host threads",
  }
  print(json.dumps(line), flush=True)


def time_cpu_baseline(nl, inputs, lens):
  """Bounded sample for the CUDA arm's line: repeats of one layer for about ten seconds."""
  torch.set_num_threads(os.cpu_count())
  cpu_layer_step(inputs, lens)
  t0 = time.perf_counter()
  reps = 0
  while reps < 30 and time.perf_counter() - t0 < 10.0:
    cpu_layer_step(inputs, lens)
    reps += 1
  per_layer = (time.perf_counter() - t0) / reps
  return B / (per_layer * nl), per_layer, reps


# ---------------------------------------------------------------------------
# CUDA arm: timing helpers
# ---------------------------------------------------------------------------


def graph_of(fn):
  """Runs `fn` once eagerly (sizes workspaces), then captures it."""
  fn()
  torch.cuda.synchronize()
  g = torch.cuda.CUDAGraph()
  with torch.cuda.graph(g):
    fn()
  g.replay()
  torch.cuda.synchronize()
  return g


def time_replays(replay, reps, warm=3):
  for _ in range(warm):
    replay()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(reps):
    replay()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1) / reps


def kernel_entry(us, nbytes, peak, **extra):
  gbs = nbytes / us / 1e3
  out = {"us_per_launch": us, "algorithmic_bytes": int(nbytes), "achieved_gbs": gbs, "frac": gbs / peak}
  out.update(extra)
  return out


# ---------------------------------------------------------------------------
# the other workloads of the path, each timed alone (one GPU)
# ---------------------------------------------------------------------------


def peer_insert(reps, nl=32):
  """Prefill -> decode hand-over inside one box (one process, two GPUs): a 2048-token bf16 prefix of `nl`
  layers (8 KV heads, D=128) that lies on cuda:1 goes into the int8 page pools of cuda:0 with the insert
  quantiser.  Timed: the insert of a prefix already on cuda:0; the insert kernel of cuda:0 reading the
  prefix from cuda:1 over NVLink (one pass); and a peer copy to cuda:0 followed by the local insert."""
  from jetstream_pytorch_b200 import insert as ins
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  if torch.cuda.device_count() < 2:
    return {"unavailable": "needs two GPUs in one process"}
  d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
  h, l, d, b, p, ps, maxp = 8, 2048, 128, 8, 512, 64, 40
  g = torch.Generator().manual_seed(1)
  spk = torch.randn(nl, 1, h, l, d, generator=g).to(torch.bfloat16)
  spv = torch.randn(nl, 1, h, l, d, generator=g).to(torch.bfloat16)
  loc, rem = (spk.to(d0), spv.to(d0)), (spk.to(d1), spv.to(d1))
  kp = torch.zeros(nl, h, p, ps, d, dtype=torch.int8, device=d0)
  vp = torch.zeros_like(kp)
  ksp = torch.zeros(nl, 1, p, ps, 1, dtype=torch.bfloat16, device=d0)
  vsp = torch.zeros_like(ksp)
  pam = PageAttentionManager(b, p, ps, maxp)
  _, upd = pam.reserve_pages_insert(0, l)
  upd = torch.as_tensor(np.asarray(upd).astype(np.int32)).to(d0)
  pools = [(kp[i], vp[i]) for i in range(nl)]
  scales = [(ksp[i], vsp[i]) for i in range(nl)]
  stage = (torch.empty_like(loc[0]), torch.empty_like(loc[1]))

  def run(src):
    pam.insert_prefill_cache([(src[0][i], src[1][i]) for i in range(nl)], pools, upd, None, None, decode_scales=scales)

  def copy_then_insert():
    stage[0].copy_(rem[0], non_blocking=True)
    stage[1].copy_(rem[1], non_blocking=True)
    run(stage)

  ins.prefix_on_peer(rem[0], d0)  # access enabled and streams ordered once: the captures below hold the kernel alone
  order_streams, ins.prefix_on_peer = ins.prefix_on_peer, lambda *a, **k: None
  out = {"workload": f"2048-token bf16 prefix x {nl} layers (8 KV heads, D=128) into int8 pages of cuda:0",
         "prefix_bytes": 2 * nl * l * h * d * 2}
  try:
    with torch.cuda.device(d0):
      for key, f, graph in (("same_gpu", lambda: run(loc), True), ("peer_read_by_insert_kernel", lambda: run(rem), True),
                            ("peer_copy_then_insert", copy_then_insert, False)):
        for _ in range(3):
          f()
        torch.cuda.synchronize(d0)
        torch.cuda.synchronize(d1)
        fn = f
        if graph:  # (a copy between devices cannot be captured: that leg is timed eagerly)
          gr = torch.cuda.CUDAGraph()
          with torch.cuda.graph(gr):
            f()
          fn = gr.replay
        fn()
        torch.cuda.synchronize(d0)
        torch.cuda.synchronize(d1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(max(3, reps)):
          fn()
        e1.record()
        torch.cuda.synchronize(d0)
        torch.cuda.synchronize(d1)
        us = e0.elapsed_time(e1) * 1e3 / max(3, reps)
        out[key] = {"us": us, "prefix_gbs": out["prefix_bytes"] / us / 1e3}
  finally:
    ins.prefix_on_peer = order_streams
  return out


def extra_dense_int8_mha(dev, peak, reps):
  """Dense int8 KV decode step, Llama-2-7B-shaped MHA: batch 8, 32 heads,
  D=128, S=2048; quantise+append (ring: one shared position; per-slot
  positions) then dense attention under a causal-by-position mask, q padded to
  two rows as the caller does for MHA.  Four cache sets rotate (512 MiB in
  total, beyond the L2)."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import Int8KVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData

  b, h, sets = 8, 32, 4
  gen = torch.Generator(device=dev).manual_seed(1001)
  ck = torch.randint(-127, 128, (sets, b, h, S, D), generator=gen, device=dev, dtype=torch.int8)
  cv = torch.randint(-127, 128, (sets, b, h, S, D), generator=gen, device=dev, dtype=torch.int8)
  ks = (torch.rand((sets, b, 1, S, 1), generator=gen, device=dev) * 0.0075 + 0.0025).to(torch.bfloat16)
  vs = (torch.rand((sets, b, 1, S, 1), generator=gen, device=dev) * 0.0075 + 0.0025).to(torch.bfloat16)
  q = torch.randn((b, h, 2, D), generator=gen, device=dev).to(torch.bfloat16)
  q[:, :, 1] = 0
  xk = torch.randn((b, h, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  xv = torch.randn((b, h, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  pos = torch.randint(0, S, (b,), generator=torch.Generator().manual_seed(1001))
  mask = torch.full((b, 1, 1, S), float("-inf"))
  for i in range(b):
    mask[i, :, :, :int(pos[i]) + 1] = 0
  mask = mask.to(torch.bfloat16).to(dev)
  tokens = int((pos + 1).sum())
  out = {}
  for name, ring in (("per_slot", False), ("ring", True)):
    data = JetEngineEnvironmentData(batch_size=b, cache_sequence_length=S, ring_buffer=ring, testing=True)
    data.quant_config.enable_kv_quantization = True
    env = JetEngineEnvironment(data, device=dev)
    ipos = torch.tensor([1000], dtype=torch.int32, device=dev) if ring else pos.to(dev, torch.int32)
    caches = [Int8KVCacheGenerate(ck[i], cv[i], ks[i], vs[i], ipos, env=env) for i in range(sets)]

    def update_all():
      for c in caches:
        c.update(xk, xv, 0)

    def attend_all():
      for i in range(sets):
        ak.dense_attention(q, ck[i], cv[i], ks[i], vs[i], mask)

    def step_all():
      for i, c in enumerate(caches):
        r = c.update(xk, xv, 0)
        ak.dense_attention(q, r[0], r[1], r[4], r[5], mask)

    us_app = time_replays(graph_of(update_all).replay, reps) * 1e3 / sets
    us_att = time_replays(graph_of(attend_all).replay, reps) * 1e3 / sets
    us_step = time_replays(graph_of(step_all).replay, reps) * 1e3 / sets
    out[name] = {
        "us_per_step": us_step,
        "append": kernel_entry(us_app, append_bytes(b, h), peak),
        "attention": kernel_entry(us_att, attention_bytes(tokens, b, 2 * h, h, ml=False) + S * b * 2, peak,
                                  note="mask-range pre-pass + tcgen05 kernel; the bytes include the mask rows"),
    }
  out["workload"] = "dense int8 MHA decode, B=8, 32 heads, D=128, S=2048, positions~U[0,2048), 4 rotating cache sets"
  return out


def extra_paged_bf16(dev, peak, reps):
  """Paged bf16 decode step, Llama-3-8B GQA shape: 32 q / 8 kv heads, D=128,
  page 64, 4096-page pool, batch 32, lengths uniform in [1, 2048], seeded
  shuffled free list: append of one token per sequence, paged attention, and
  the insert of a 1024-token prefill.  Two pools rotate (2 GiB in total)."""
  from jetstream_pytorch_b200 import attention_kernel as ak
  from jetstream_pytorch_b200.cache_manager import PageKVCacheGenerate
  from jetstream_pytorch_b200.environment import JetEngineEnvironment, JetEngineEnvironmentData
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  b, hq, hkv, ps, p, maxp, sets = 32, 32, 8, 64, 4096, 33, 2
  rng = np.random.RandomState(1001)
  lens = rng.randint(1, 2049, size=b)
  free_slot = 17
  lens[free_slot] = 0
  pam = PageAttentionManager(b, p, ps, maxp, free_page_order=rng.permutation(p).tolist())
  for slot in range(b):
    if lens[slot]:
      pam.reserve_pages_insert(slot, int(lens[slot]))
  gen = torch.Generator(device=dev).manual_seed(1001)
  pools = [(torch.randn((hkv, p, ps, D), generator=gen, device=dev).to(torch.bfloat16),
            torch.randn((hkv, p, ps, D), generator=gen, device=dev).to(torch.bfloat16)) for _ in range(sets)]
  pre_k = torch.randn((1, hkv, 1024, D), generator=gen, device=dev).to(torch.bfloat16)
  pre_v = torch.randn((1, hkv, 1024, D), generator=gen, device=dev).to(torch.bfloat16)
  _, idx = pam.reserve_pages_insert(free_slot, 1024)
  idx = torch.as_tensor(np.asarray(idx), dtype=torch.int32, device=dev)
  lens[free_slot] = 1024
  pam.fill_new_pages(lens)
  pti = torch.as_tensor(pam.get_page_token_indices(lens), dtype=torch.int32, device=dev)
  lengths = torch.as_tensor(np.asarray(pam.lengths), dtype=torch.int32, device=dev)
  table = torch.as_tensor(pam.page_indices, dtype=torch.int32, device=dev)
  xk = torch.randn((b, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  xv = torch.randn((b, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  q = torch.randn((b, hq, D), generator=gen, device=dev).to(torch.bfloat16)
  data = JetEngineEnvironmentData(batch_size=b, ring_buffer=False, testing=True, paged_attention_total_num_pages=p,
                                  paged_attention_page_size=ps)
  env = JetEngineEnvironment(data, device=dev)
  caches = [PageKVCacheGenerate(k, v, pam, pti, None, env=env) for k, v in pools]

  def append_all():
    for c in caches:
      c.update(xk, xv)

  def attend_all():
    for k, v in pools:
      ak.call_paged_attention(env, q, k, v, lengths, table)

  def insert_all():
    for k, v in pools:
      pam.insert_prefill_cache([(pre_k, pre_v)], [(k, v)], idx)

  tokens = int(np.asarray(pam.lengths).sum())
  pages = int(sum(-(-int(n) // ps) for n in np.asarray(pam.lengths)))
  us_app = time_replays(graph_of(append_all).replay, reps) * 1e3 / sets
  us_att = time_replays(graph_of(attend_all).replay, reps) * 1e3 / sets
  us_ins = time_replays(graph_of(insert_all).replay, reps) * 1e3 / sets
  n_active = int((lens > 0).sum())
  return {
      "workload": "paged bf16 decode, B=32, 32q/8kv heads, D=128, page 64, 4096-page pool, lens~U[1,2048], "
                  "shuffled free list, 2 rotating pools",
      "append": kernel_entry(us_app, 2 * n_active * hkv * D * 2 * 2 + 3 * n_active * 4, peak),
      "attention": kernel_entry(us_att, attention_bytes(tokens, b, hq, hkv, kv_bytes=2, scales=False, ml=False)
                                + pages * 4, peak),
      "insert_1024": kernel_entry(us_ins, 2 * 1024 * hkv * D * 2 * 2, peak),
  }


def extra_bf16_dense(dev, peak, reps, lens):
  """The bench shape with an unquantised bf16 cache (mma.sync kernel), 3 rotating cache sets."""
  from jetstream_pytorch_b200 import attention_kernel as ak

  sets = 3
  gen = torch.Generator(device=dev).manual_seed(1005)
  ck = torch.randn((sets, B, HKV, S, D), generator=gen, device=dev, dtype=torch.bfloat16)
  cv = torch.randn((sets, B, HKV, S, D), generator=gen, device=dev, dtype=torch.bfloat16)
  q = torch.randn((B, HQ, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  start = torch.zeros(B, dtype=torch.int32, device=dev)
  lens_d = lens.to(dev, torch.int32)

  def attend_all():
    for i in range(sets):
      ak.ragged_mha(q, ck[i], cv[i], 0, start, lens_d, None, None, None, None)

  us = time_replays(graph_of(attend_all).replay, reps) * 1e3 / sets
  return kernel_entry(us, attention_bytes(int(lens.sum()), B, HQ, HKV, kv_bytes=2, scales=False), peak,
                      workload="the bench shape with a bf16 cache (B=96, 64q/8kv, S=2048), 3 rotating cache sets")


def extra_insert_burst(dev, peak, reps, nl=32):
  """Prefill-insert and quantise burst: 64 inserts, each scattering and
  quantising a prefix of L in {128..2048} tokens x 32 stacked layers into pages
  of an int8 paged cache (batch 128, page 64, 8 KV heads): one launch per
  insert, the whole burst replayed as one CUDA graph."""
  from jetstream_pytorch_b200 import _lib
  from jetstream_pytorch_b200.page_attention_manager import PageAttentionManager

  bi, ps, hk, maxp, n_ins = 128, 64, HKV, 32, 64
  pages = bi * maxp
  rng = np.random.RandomState(1004)
  lens = rng.choice([128, 256, 512, 1024, 2048], size=n_ins)
  gen = torch.Generator(device=dev).manual_seed(1004)
  pre_k = torch.randn((nl, 1, hk, 2048, D), generator=gen, device=dev).to(torch.bfloat16)
  pre_v = torch.randn((nl, 1, hk, 2048, D), generator=gen, device=dev).to(torch.bfloat16)
  pool_k = torch.zeros((nl, hk, pages, ps, D), dtype=torch.int8, device=dev)
  pool_v = torch.zeros((nl, hk, pages, ps, D), dtype=torch.int8, device=dev)
  sc_k = torch.zeros((nl, 1, pages, ps, 1), dtype=torch.bfloat16, device=dev)
  sc_v = torch.zeros((nl, 1, pages, ps, 1), dtype=torch.bfloat16, device=dev)
  pre = [(pre_k[i], pre_v[i]) for i in range(nl)]
  pools = [(pool_k[i], pool_v[i]) for i in range(nl)]
  scales = [(sc_k[i], sc_v[i]) for i in range(nl)]
  pam = PageAttentionManager(bi, pages, ps, maxp, free_page_order=rng.permutation(pages))
  plan, nbytes = [], 0
  for j, length in enumerate(lens):
    length = int(length)
    n_pages, idx = pam.reserve_pages_insert(j, length)
    plan.append((length, torch.as_tensor(np.asarray(idx), dtype=torch.int32, device=dev)))
    nbytes += nl * (2 * length * hk * D * 2 + 2 * n_pages * ps * hk * D + 2 * n_pages * ps * 2)

  def burst():
    for length, upd in plan:
      pam.insert_prefill_cache([(k[:, :, :length], v[:, :, :length]) for k, v in pre], pools, upd, decode_scales=scales)

  c0 = _lib.lib().jpt_launch_count()
  burst()
  torch.cuda.synchronize()
  launches = _lib.lib().jpt_launch_count() - c0
  ms = time_replays(graph_of(burst).replay, reps)
  gbs = nbytes / (ms * 1e-3) / 1e9
  return {"workload": f"64 inserts x {nl} stacked layers, L in {{128,256,512,1024,2048}}, int8 paged cache (batch 128, "
                      "page 64, 8 kv heads, D=128), quantise on insert",
          "launches_per_burst": int(launches), "tokens_per_burst": int(lens.sum()), "ms_per_burst": ms,
          "algorithmic_bytes": int(nbytes), "achieved_gbs": gbs, "frac": gbs / peak,
          "inserts_per_s": n_ins / (ms * 1e-3)}


def extra_w8a16_linear(dev, peak, reps, eager=False):
  """The weight stream of a decode step: the weight-only int8 linear layer at the
  bench model's projection shapes (Llama-2-70B, batch 96), each over rotating
  weight sets larger than L2, replayed as one CUDA graph."""
  from jetstream_pytorch_b200.layers import WeightOnlyPerChannelQuantizedLinear

  out = {}
  gen = torch.Generator(device=dev).manual_seed(1006)
  shapes = (("wo_8192x8192", 8192, 8192), ("w_up_8192x28672", 8192, 28672), ("w_down_28672x8192", 28672, 8192))
  for name, k, n in (shapes[:1] if eager is True else [] if eager else shapes):  # (eager: for profiler captures)
    sets = max(3, int(300e6 // (k * n)) + 1)
    layers = []
    for _ in range(sets):
      lin = WeightOnlyPerChannelQuantizedLinear(k, n, device=dev)
      lin._load_quantized_weights(torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8, device=dev),
                                  torch.rand(n, generator=gen, device=dev) * 0.01)
      layers.append(lin)
    x = torch.randn((B, k), generator=gen, device=dev).to(torch.bfloat16)

    def run_all():
      for lin in layers:
        lin(x)

    if eager:
      run_all()
      us = time_replays(run_all, reps) * 1e3 / sets
    else:
      us = time_replays(graph_of(run_all).replay, reps) * 1e3 / sets
    status = max(lin.kernel_status() for lin in layers)
    nbytes = n * k + B * k * 2 + B * n * 2 + n * 2  # int8 weights, bf16 activations in and out, bf16 scales
    out[name] = kernel_entry(us, nbytes, peak, kernel_status=status, rotating_weight_sets=sets)
    del layers
    torch.cuda.empty_cache()
  out["workload"] = "y = bf16(bf16(x W^T) * scale), x bf16 [96, K], W int8 [N, K]: level split + tcgen05 GEMM launches"
  if not eager or eager == "ffn":
    # the feed-forward block behind its norm: RMSNorm (writes the levels of its result), w1 and w3 on those
    # levels, the gate (writes the levels of its result), w2: five launches, 705 MB of weights
    from jetstream_pytorch_b200.layers import FeedForward, RMSNorm

    dim, hidden, sets = 8192, 28672, 2
    blocks = []
    for _ in range(sets):
      ff = FeedForward(dim, hidden, device=dev)
      for lin in (ff.w1, ff.w2, ff.w3):
        lin._load_quantized_weights(
            torch.randint(-127, 128, (lin.out_features, lin.in_features), generator=gen, dtype=torch.int8, device=dev),
            torch.rand(lin.out_features, generator=gen, device=dev) * 0.002)
      blocks.append((RMSNorm(dim, eps=1e-5, device=dev), ff))
    x = torch.randn((B, dim), generator=gen, device=dev).to(torch.bfloat16)

    def run_blocks():
      for norm, ff in blocks:
        y, lv = norm(x, with_levels=True)
        ff(y, levels=lv)

    if eager:
      run_blocks()
      us = time_replays(run_blocks, reps) * 1e3 / sets
    else:
      us = time_replays(graph_of(run_blocks).replay, reps) * 1e3 / sets
    nbytes = 3 * dim * hidden + 3 * hidden * 2 + dim * 2 + B * 2 * (2 * dim + 3 * hidden + dim)
    out["ffn_block_8192_28672"] = kernel_entry(
        us, nbytes, peak, launches=5, kernel_status=max(ff.w2.kernel_status() for _, ff in blocks),
        workload="RMSNorm -> w1, w3 -> silu-mul -> w2 at batch 96 (weights, scales, norm weight, activations in and out)")
    del blocks
    torch.cuda.empty_cache()
  return out


def linear_tp(dev, peak, reps, rank, world):
  """The row-parallel projections of the bench model (`wo` 8192 -> 8192, `w2`
  28672 -> 8192) at batch 96 with their input features sharded over the ranks:
  the sum over the ranks inside the GEMM's epilogue (peer stores over NVLink)
  against the same GEMM followed by an NCCL all-reduce of its bf16 result.
  Times are the maximum over the ranks; bytes are one rank's."""
  import torch.distributed as dist

  from jetstream_pytorch_b200.layers import TensorParallelSum, WeightOnlyPerChannelQuantizedLinear

  out = {}
  tp = TensorParallelSum.with_torch_distributed(8192) if world > 1 else TensorParallelSum(8192, 0, 1, lambda h: [h])
  gen = torch.Generator(device=dev).manual_seed(1007 + rank)

  def max_over_ranks(ms):
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

  for name, k_all, n in (("wo_8192x8192", 8192, 8192), ("w_down_28672x8192", 28672, 8192)):
    k = k_all // world
    sets = max(3, int(300e6 // (k * n)) + 1)
    layers = []
    for _ in range(sets):
      lin = WeightOnlyPerChannelQuantizedLinear(k, n, device=dev)
      lin._load_quantized_weights(torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8, device=dev),
                                  torch.full((n,), 0.002, device=dev))
      layers.append(lin)
    x = torch.randn((B, k), generator=gen, device=dev).to(torch.bfloat16)

    def fused():
      for lin in layers:
        lin(x, tp=tp)

    def with_nccl():
      for lin in layers:
        y = lin(x)
        if world > 1:
          dist.all_reduce(y)

    entry = {}
    for label, fn in (("sum_in_kernel", fused), ("gemm_then_nccl_all_reduce", with_nccl)):
      if world > 1:
        dist.barrier()
      try:
        ms = time_replays(graph_of(fn).replay, reps)
        how = "graph"
      except Exception as e:  # pylint: disable=broad-except
        torch.cuda.synchronize()
        fn()
        ms = time_replays(fn, reps)
        how = f"eager ({type(e).__name__})"
      entry[label] = {"us_per_layer": max_over_ranks(ms) * 1e3 / sets, "launches": how}
    nbytes = n * k + B * k * 2 + B * n * 2 + n * 2
    us = entry["sum_in_kernel"]["us_per_layer"]
    entry.update(algorithmic_bytes_per_rank=int(nbytes), achieved_gbs_per_rank=nbytes / us / 1e3, frac=nbytes / us / 1e3 / peak,
                 nvlink_bytes_out_per_rank=int((world - 1) * B * n * 4), rotating_weight_sets=sets,
                 kernel_status=max(lin.kernel_status() for lin in layers), tp_status=tp.status())
    out[name] = entry
    del layers
    torch.cuda.empty_cache()
  if world > 1:
    dist.barrier()
  tp.close()
  return out


# ---------------------------------------------------------------------------
# CUDA arm
# ---------------------------------------------------------------------------


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
  h0, q0 = rank * hkv, rank * hq
  nl = args.layers
  lib = _lib.lib()
  peak, peak_kind = peaks()
  if args.only == "insert":
    print(json.dumps({"only": "insert", **extra_insert_burst(dev, peak, args.steps, nl=min(32, nl))}), flush=True)
    return
  if args.only == "peer-insert":
    print(json.dumps({"only": "peer-insert", **peer_insert(args.steps, nl=min(32, nl))}), flush=True)
    return
  if args.only == "linear-tp":
    res = linear_tp(dev, peak, args.steps, rank, world)
    if rank == 0:
      print(json.dumps({"only": "linear-tp", "n_gpus": world, **res}), flush=True)
    if world > 1:
      dist.barrier()
      dist.destroy_process_group()
    return
  if args.only in ("linear", "ffn"):
    print(json.dumps({"only": args.only,
                      **extra_w8a16_linear(dev, peak, args.steps, eager=True if args.only == "linear" else "ffn")}), flush=True)
    return

  # ---- device-resident state: every layer owns its cache (>> L2 in total).  Layer 0 comes from
  # the seeded host inputs that the reference arm and the parity check use; the others are drawn
  # on the device (host generation of 32 GB of codes would take minutes).
  lens = make_lengths()
  lens_d = lens.to(dev, torch.int32)
  pos_d = (lens - 1).to(dev, torch.int32)
  gen = torch.Generator(device=dev).manual_seed(1002 + rank)
  ck = torch.empty((nl, B, hkv, S, D), dtype=torch.int8, device=dev)
  cv = torch.empty((nl, B, hkv, S, D), dtype=torch.int8, device=dev)
  for i in range(1, nl):
    ck[i] = torch.randint(-127, 128, (B, hkv, S, D), generator=gen, device=dev, dtype=torch.int8)
    cv[i] = torch.randint(-127, 128, (B, hkv, S, D), generator=gen, device=dev, dtype=torch.int8)
  sgen = torch.Generator(device=dev).manual_seed(77)  # scales are replicated across ranks
  ks = (torch.rand((nl, B, 1, S, 1), generator=sgen, device=dev) * 0.0075 + 0.0025).to(torch.bfloat16)
  vs = (torch.rand((nl, B, 1, S, 1), generator=sgen, device=dev) * 0.0075 + 0.0025).to(torch.bfloat16)
  hq_all = torch.randn((nl, B, hq, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  hk_all = torch.randn((nl, B, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  hv_all = torch.randn((nl, B, hkv, 1, D), generator=gen, device=dev).to(torch.bfloat16)
  host0 = cpu_layer_inputs(0)
  ck[0], cv[0] = host0[0][:, h0:h0 + hkv].to(dev), host0[1][:, h0:h0 + hkv].to(dev)
  ks[0], vs[0] = host0[2].to(dev), host0[3].to(dev)
  hq_all[0] = host0[4][:, q0:q0 + hq].to(dev)
  hk_all[0], hv_all[0] = host0[5][:, h0:h0 + hkv].to(dev), host0[6][:, h0:h0 + hkv].to(dev)

  data = JetEngineEnvironmentData(batch_size=B, cache_sequence_length=S, num_layers=nl, ring_buffer=False,
                                  testing=True, cache_shape=(B, hkv, S, D))
  data.quant_config.enable_kv_quantization = True
  env = JetEngineEnvironment(data, device=dev, rank=rank, world_size=world)  # eager per-slot writes, unstacked
  caches = [Int8KVCacheGenerate(ck[i], cv[i], ks[i], vs[i], pos_d, env=env) for i in range(nl)]
  start_d = torch.zeros(B, dtype=torch.int32, device=dev)
  # outputs the steps write into (fixed addresses: graph replays and the end-to-end leg read them)
  o_s = torch.empty((nl, B, hq, 1, D), dtype=torch.bfloat16, device=dev)
  m_s = torch.empty((nl, B, hq, 1), dtype=torch.float32, device=dev)
  l_s = torch.empty((nl, B, hq, 1), dtype=torch.float32, device=dev)

  # Head-sharded scales need the amax over all ranks: inside the append launch over NVLink
  # peer memory (default), or as local_amax + NCCL all_reduce(MAX) + update (--amax-exchange nccl).
  px = None
  if world > 1 and args.amax_exchange == "peers":
    from jetstream_pytorch_b200.cache_manager import PeerAmaxExchange
    px = PeerAmaxExchange.with_torch_distributed(B)

  # The step's form: measured faster as two launches on one GPU (49 against 51 us per layer) and as one
  # fused launch when the KV heads are sharded (the amax exchange then hides under the attention).
  fused = (args.fused or (world > 1 and not args.unfused)) and (world == 1 or px is not None)
  existing_d = lens_d - 1  # tokens in the cache before the step's new one

  def layer_step(i, q, xk, xv):
    if fused:  # update and attention of the layer as ONE launch
      r, _ = caches[i].update_and_attend(q, xk, xv, i, start_d, existing_d, peers=px, out=(o_s[i], m_s[i], l_s[i]))
      return r
    amax = None
    if world > 1 and px is None:
      amax = caches[i].local_amax(xk, xv)
      dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    r = caches[i].update(xk, xv, i, amax=amax, peers=px)
    ak.ragged_mha(q, r[0], r[1], i, start_d, lens_d, None, None, r[4], r[5], out=(o_s[i], m_s[i], l_s[i]))
    return r

  def device_step():
    for i in range(nl):
      layer_step(i, hq_all[i], hk_all[i], hv_all[i])

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
    nbytes = attention_bytes(lens.sum(), B, hq, hkv) if args.only == "attention" else append_bytes(B, hkv)
    if args.only == "attention" and args.kv == "bf16":
      nbytes = attention_bytes(lens.sum(), B, hq, hkv, kv_bytes=2, scales=False)
    # eager launches: for kernels shorter than the host's ~35 us per call this is the host's pace, not the kernel's
    print(json.dumps({"only": args.only, "kv": args.kv, "attn_kernel": args.attn_kernel, "layers": nl,
                      "launches": nl * (args.steps + max(3, args.warmup)), "us_per_eager_call": us,
                      "algorithmic_bytes": nbytes, "gbs_at_that_pace": nbytes / us / 1e3}), flush=True)
    return

  # ---- warm-up (also sizes the attention workspace), then a CUDA graph of one step
  warmup = max(3, args.warmup)
  for _ in range(warmup):
    device_step()
  torch.cuda.synchronize()
  graph = None
  if not args.no_graph:
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

  # ---- per-kernel timing for the roofline: attention only (left aligned, then ring), append only
  ring_start, ring_end, ring_n = make_ring_ranges()
  ring_start_d, ring_end_d = ring_start.to(dev, torch.int32), ring_end.to(dev, torch.int32)

  def attn_only():
    for i in range(nl):
      ak.ragged_mha(hq_all[i], ck[i], cv[i], i, start_d, lens_d, None, None, ks[i], vs[i], out=(o_s[i], m_s[i], l_s[i]))

  def attn_ring_only():
    for i in range(nl):
      ak.ragged_mha(hq_all[i], ck[i], cv[i], i, ring_start_d, ring_end_d, None, None, ks[i], vs[i], ring=True,
                    out=(o_s[i], m_s[i], l_s[i]))

  def append_only():
    for i in range(nl):
      caches[i].update(hk_all[i], hv_all[i], i, peers=px)

  # the same caches under multi-head attention: one query head per KV head (Llama-2-7B/13B-like grouping)
  q_mha = hq_all[:, :, ::HQ // HKV].contiguous()
  o_mha = torch.empty_like(q_mha)

  def attn_mha_only():
    for i in range(nl):
      ak.ragged_mha(q_mha[i], ck[i], cv[i], i, start_d, lens_d, None, None, ks[i], vs[i], out=(o_mha[i], None, None))

  def two_launch_layer(i):
    r = caches[i].update(hk_all[i], hv_all[i], i, peers=px)
    ak.ragged_mha(hq_all[i], r[0], r[1], i, start_d, lens_d, None, None, r[4], r[5], out=(o_s[i], m_s[i], l_s[i]))

  def fused_only():  # the step's other form: append and attention of a layer in one launch
    for i in range(nl):
      caches[i].update_and_attend(hq_all[i], hk_all[i], hv_all[i], i, start_d, existing_d, peers=px,
                                  out=(o_s[i], m_s[i], l_s[i]))

  reps = max(1, args.steps // 2)
  legs = {"attn": attn_only, "ring": attn_ring_only, "append": append_only}
  if world == 1:
    legs["mha"] = attn_mha_only
  if not fused and (world == 1 or px is not None):
    legs["fused"] = fused_only
  if fused:
    legs["two_launch"] = lambda: [two_launch_layer(i) for i in range(nl)]
  if world > 1 and px is None:
    del legs["append"]  # the two-phase form is three launches and a collective: not a kernel on its own
  if graph is not None:
    for name in list(legs):
      try:
        legs[name] = graph_of(legs[name]).replay
      except Exception:  # pylint: disable=broad-except
        torch.cuda.synchronize()
  ms_leg = {}
  for name, fn in legs.items():
    for _ in range(3):
      fn()
    ms_leg[name] = timed_steps(fn, reps) / nl
  clocks = sampler.stop()

  # ---- parity of this run's own state against the CPU oracle (outside every timed region):
  # one more step of layer 0 on the seeded host inputs; every rank's codes, scales, written
  # cache rows and attention rows are gathered and compared with the unsharded oracle.
  r0 = layer_step(0, hq_all[0], hk_all[0], hv_all[0])
  torch.cuda.synchronize()
  rows = torch.arange(B, device=dev)
  mine = {
      "k_quant": r0[2].reshape(B, hkv, D), "v_quant": r0[3].reshape(B, hkv, D),
      "k_scale": r0[6].reshape(B).view(torch.int16), "v_scale": r0[7].reshape(B).view(torch.int16),
      "k_row": ck[0][rows, :, pos_d.long()], "v_row": cv[0][rows, :, pos_d.long()],
      "ks_row": ks[0][rows, 0, pos_d.long(), 0].view(torch.int16), "vs_row": vs[0][rows, 0, pos_d.long(), 0].view(torch.int16),
      "o": o_s[0].reshape(B, hkv, (HQ // HKV), D).view(torch.int16), "l": l_s[0].reshape(B, hkv, HQ // HKV),
  }
  gathered = {}
  for name, t in mine.items():
    t = t.contiguous()
    if world > 1:  # as bytes: NCCL has no 16-bit integer type
      raw = t.view(torch.uint8).reshape(-1)
      got = [torch.empty_like(raw) for _ in range(world)]
      dist.all_gather(got, raw)
      parts = [g.view(t.dtype).reshape(t.shape) for g in got]
    else:
      parts = [t]
    gathered[name] = [p.cpu() for p in parts]
  parity = None
  if rank == 0:
    er, (eo, em, el) = cpu_layer_step(host0, lens)
    pos = (lens - 1).long()
    ar = torch.arange(B)
    bit_exact = True
    for name in ("k_scale", "v_scale", "ks_row", "vs_row"):
      want = {"k_scale": er[6].reshape(B), "v_scale": er[7].reshape(B), "ks_row": er[4][ar, 0, pos, 0],
              "vs_row": er[5][ar, 0, pos, 0]}[name].view(torch.int16)
      bit_exact &= all(torch.equal(p, want) for p in gathered[name])  # scales are replicated: every rank holds all
    for name, want in (("k_quant", er[2].reshape(B, HKV, D)), ("v_quant", er[3].reshape(B, HKV, D)),
                       ("k_row", er[0][ar, :, pos]), ("v_row", er[1][ar, :, pos])):
      bit_exact &= torch.equal(torch.cat(gathered[name], dim=1), want)
    got_o = torch.cat(gathered["o"], dim=1).view(torch.bfloat16).float()
    err = (got_o - eo.float()).abs()
    row_rel = (torch.linalg.vector_norm(got_o - eo.float(), dim=-1)
               / torch.linalg.vector_norm(eo.float(), dim=-1).clamp_min(1e-30)).max()
    got_l = torch.cat(gathered["l"], dim=1)
    attn_ok = bool(err.max() <= 2e-2 and row_rel <= 1e-2 and torch.allclose(got_l, el, rtol=1e-3, atol=1e-3))
    parity = {"sharded_update_bit_exact": bool(bit_exact), "attention_within_tolerance": attn_ok, "ranks": world,
              "attention_max_abs_err": float(err.max()), "attention_max_row_rel_err": float(row_rel),
              "checked": "layer 0 on the seeded host inputs: quantised token, scales, written cache rows (bit for bit) "
                         "and attention rows (2e-2 abs per element, 1e-2 relative per row in the 2-norm; l 1e-3) of all ranks against the "
                         "unsharded CPU oracle"}

  # ---- end to end through the public API with HOST buffers: pinned inputs go in, outputs come
  # back, every step; the layers are pipelined in chunks (H2D of chunk c+1 and D2H of chunk c-1
  # overlap the kernels of chunk c), each chunk's launches replayed as one CUDA graph.
  q_h = hq_all.cpu().pin_memory()
  k_h = hk_all.cpu().pin_memory()
  v_h = hv_all.cpu().pin_memory()
  o_h = torch.empty((nl, B, hq, 1, D), dtype=torch.bfloat16).pin_memory()
  q_s, k_s, v_s = torch.empty_like(hq_all), torch.empty_like(hk_all), torch.empty_like(hv_all)
  copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
  compute = torch.cuda.current_stream()
  chunk = max(1, nl // max(1, args.e2e_chunks))
  chunks = [(c0, min(nl, c0 + chunk)) for c0 in range(0, nl, chunk)]

  def chunk_fn(c0, c1):
    def run():
      for i in range(c0, c1):
        layer_step(i, q_s[i], k_s[i], v_s[i])
    return run

  chunk_run = [chunk_fn(c0, c1) for c0, c1 in chunks]
  if graph is not None:
    try:
      chunk_run = [graph_of(fn).replay for fn in chunk_run]
    except Exception as e:  # pylint: disable=broad-except
      print(f"[bench] end-to-end leg runs eager launches ({e})", file=sys.stderr)
      torch.cuda.synchronize()
      chunk_run = [chunk_fn(c0, c1) for c0, c1 in chunks]

  def e2e_step():
    in_evt = []
    copy_in.wait_stream(compute)
    with torch.cuda.stream(copy_in):
      for c0, c1 in chunks:
        q_s[c0:c1].copy_(q_h[c0:c1], non_blocking=True)
        k_s[c0:c1].copy_(k_h[c0:c1], non_blocking=True)
        v_s[c0:c1].copy_(v_h[c0:c1], non_blocking=True)
        e = torch.cuda.Event()
        e.record(copy_in)
        in_evt.append(e)
    for ci, (c0, c1) in enumerate(chunks):
      compute.wait_event(in_evt[ci])
      chunk_run[ci]()
      e = torch.cuda.Event()
      e.record(compute)
      copy_out.wait_event(e)
      with torch.cuda.stream(copy_out):
        o_h[c0:c1].copy_(o_s[c0:c1], non_blocking=True)
    compute.wait_stream(copy_out)
    compute.wait_stream(copy_in)

  for _ in range(3):
    e2e_step()
  ms_e2e = timed_steps(e2e_step, max(2, args.steps // 2))
  h2d = q_h.numel() * 2 + k_h.numel() * 2 + v_h.numel() * 2
  d2h = o_h.numel() * 2
  attn_status = ak.kernel_status()
  px_status = px.status() if px is not None else None

  def leave():
    """Ranks leave together.  With collectives captured in CUDA graphs the process
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

  a_bytes = attention_bytes(lens.sum(), B, hq, hkv)
  achieved = a_bytes / (ms_leg["attn"] * 1e-3) / 1e9
  traffic, traffic_src = profiled_traffic() if world == 1 else (None, "captured on one GPU holding all 8 KV heads only")
  kernels = {"attention_ring": kernel_entry(ms_leg["ring"] * 1e3, attention_bytes(ring_n.sum(), B, hq, hkv), peak,
                                            workload="same caches, start,end~U[0,2048) with wrap (ring semantics)")}
  if "mha" in ms_leg:
    kernels["attention_mha"] = kernel_entry(
        ms_leg["mha"] * 1e3, attention_bytes(lens.sum(), B, hkv, hkv, ml=False), peak,
        workload="same caches, one query head per KV head (multi-head attention): the kernel's two-row variant")
  if "append" in ms_leg:
    kernels["kv_quant_append"] = kernel_entry(ms_leg["append"] * 1e3, append_bytes(B, hkv), peak)
  if "two_launch" in ms_leg:
    kernels["append_then_attention"] = kernel_entry(
        ms_leg["two_launch"] * 1e3, a_bytes + append_bytes(B, hkv), peak,
        workload="the step's layer as TWO launches (append with the exchange, then attention; `--unfused` makes it the step)")
  if "fused" in ms_leg:
    kernels["decode_update_attend"] = kernel_entry(
        ms_leg["fused"] * 1e3, a_bytes + append_bytes(B, hkv), peak,
        workload="the step's layer as ONE launch (jpt_decode_update_attend: quantise + append + attention; `--fused` makes it the step)")
  line = {
      "metric": METRIC, "value": B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
      "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
      "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
      "config": {"workload": WORKLOAD, "layers": nl, "global_batch": B, "kv_heads_per_gpu": hkv,
                 "parallelism": f"kv-head sharding x{world}",
                 "amax_exchange": ("in-kernel over NVLink peer memory" if px is not None else
                                   ("nccl all_reduce" if world > 1 else "none")),
                 "peer_exchange_status": px_status, "attention_status": attn_status,
                 "l2": "each layer has its own cache buffers "
                       f"({2 * B * hkv * S * D * nl / 2**30:.1f} GiB per GPU in total, >> 126 MB L2)",
                 "cuda_graph": graph is not None,
                 "launches_per_layer": "1 (fused quantise + append + attention)" if fused else "2 (append, attention)"},
      "us_per_layer": ms_step * 1e3 / nl,
      "roofline": {"bound": "hbm", "kernel": "flash_decode_i8_umma_kernel (tcgen05; pieces merged in-kernel), timed alone without the new token",
                   "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                   "frac_of_8000_nominal": achieved / 8000.0, "algorithmic_bytes_per_launch": a_bytes,
                   "us_per_launch": ms_leg["attn"] * 1e3, "traffic": traffic, "traffic_source": traffic_src},
      "kernels": kernels,
      "parity": parity,
      "e2e": {"value": B / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
              "d2h_bytes_per_step": d2h, "launches": "one CUDA graph per chunk of layers" if graph is not None else "eager"},
      "gpu_launches": int(launches),
      "clocks": clocks,
  }
  ok = parity["sharded_update_bit_exact"] and parity["attention_within_tolerance"] and not attn_status and not px_status
  if world == 1 and not args.no_extras:
    # free the 80-layer state first: the other workloads bring their own caches
    del caches, ck, cv, ks, vs, graph, legs, chunk_run, r0, mine
    torch.cuda.empty_cache()
    xreps = max(3, args.steps // 2)
    try:
      kernels["dense_int8_mha"] = extra_dense_int8_mha(dev, peak, xreps)
      torch.cuda.empty_cache()
      kernels["paged_bf16"] = extra_paged_bf16(dev, peak, xreps)
      torch.cuda.empty_cache()
      kernels["attention_bf16_cache"] = extra_bf16_dense(dev, peak, xreps, lens)
      torch.cuda.empty_cache()
      kernels["prefill_insert_burst"] = extra_insert_burst(dev, peak, max(2, xreps // 2))
      torch.cuda.empty_cache()
      kernels["w8a16_linear"] = extra_w8a16_linear(dev, peak, xreps)
      torch.cuda.empty_cache()
    except Exception as e:  # pylint: disable=broad-except
      kernels["error"] = f"{type(e).__name__}: {e}"
      torch.cuda.synchronize()
  if world == 1 and not args.no_cpu_baseline:
    v, per_layer, n = time_cpu_baseline(nl, host0, lens)
    line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                            "sample": f"1 of {nl} layers (all 96 sequences) x {n} repeats, {per_layer:.2f} s per "
                                      f"layer; tokens/s scaled to {nl} layers"}
  print(json.dumps(line), flush=True)
  if not ok:
    print("[bench] parity or kernel status check FAILED (see the line's parity / config keys)", file=sys.stderr)
    sys.stdout.flush()
    if world > 1:
      os._exit(1)
    raise SystemExit(1)
  leave()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
  ap.add_argument("--layers", type=int, default=80)
  ap.add_argument("--no-graph", action="store_true")
  ap.add_argument("--e2e-chunks", type=int, default=16,
                  help="end-to-end leg: the layers are pipelined (copy in, compute, copy out) in this many chunks")
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--fused", action="store_true",
                  help="per layer one launch that appends the new token and attends (the default when N > 1)")
  ap.add_argument("--unfused", action="store_true",
                  help="per layer the append launch, then the attention launch (the default when N = 1)")
  ap.add_argument("--no-extras", action="store_true", help="skip the other workloads' kernels (N = 1 runs them by default)")
  ap.add_argument("--amax-exchange", choices=["peers", "nccl"], default="peers",
                  help="N > 1: how the per-token amax is max-reduced over the ranks")
  ap.add_argument("--only", choices=["attention", "append", "insert", "peer-insert", "linear", "ffn", "linear-tp"], default=None,
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
