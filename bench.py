"""Headline benchmark: decode tokens/s of a Llama-3-8B-shaped Q4_0 model at batch 1 on B200, with the achieved HBM
bandwidth of the decode kernel against the measured peak, plus records of the other configurations of the path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step (one token through all blocks, head and arg-max).  Weights, embeddings and prompt ids are seeded
synthetic data of the configuration's shapes and distributions (no checkpoint or dataset is involved).  For N > 1 (launched by
torch.distributed.run) every rank decodes its own sequence on its own GPU for the headline metric (the model fits one GPU:
replicas, no data-path collective); the sharded configurations run over all N ranks and are reported in their own records:
  "moe"     configs[3], one OLMoE-shaped MXFP8 MoE layer over 4096 tokens on one GPU (N == 1)
  "batched" configs[2] shape, Qwen2-7B-shaped Q8_0 decode with 8 (and, as "batch_32", 32) sequences in lock-step on one GPU (N == 1)
  "ep_moe"  the same layer expert-parallel over the N ranks (N > 1)
  "tp70b"   configs[4], Llama-3-70B-shaped Q4_0 decode at batch 1: unsharded on one GPU at N == 1, tensor-parallel over N ranks else
Prints ONE JSON line on rank 0.
"""
import argparse, json, os, sys, time, threading, pathlib
import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC, UNIT = "decode tokens/s (8B-shape Q4_0, bs1)", "tokens/s"
NCU_TRAFFIC_RATIO = 1.006      # dram__bytes_read + write per launch / algorithmic bytes, from the committed ncu summary of qgemv_kernel
WORKLOAD = "configs[1]: Llama-3-8B-shaped decode, Q4_0 linears, fp16 embeddings/norms, fp16 KV cache, batch 1, prompt 512 random ids, greedy"
PROMPT_LEN, MAX_CONTEXT = 512, 2048


def llama3_8b_config():
  from tinygrad_b200.model import TransformerConfig
  return TransformerConfig(num_blocks=32, dim=4096, hidden_dim=14336, n_heads=32, n_kv_heads=8, norm_eps=1e-5, vocab_size=128256, head_dim=128,
                           rope_theta=500000.0, rope_dim=128, v_head_dim=128, max_context=MAX_CONTEXT, kv_dtype="float16")


def llama3_70b_config(max_context: int = 2048):
  from tinygrad_b200.model import TransformerConfig
  return TransformerConfig(num_blocks=80, dim=8192, hidden_dim=28672, n_heads=64, n_kv_heads=8, norm_eps=1e-5, vocab_size=128256, head_dim=128,
                           rope_theta=500000.0, rope_dim=128, v_head_dim=128, max_context=max_context, kv_dtype="float16")


def measured_peaks() -> dict:
  p = ROOT / "MEASURED_PEAKS.json"
  if p.exists():
    d = json.loads(p.read_text())
    return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json)"}
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback (6.65 TB/s, 1.59 PFLOP/s: an earlier measurement on this pool)"}


class ClockSampler:
  """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""
  def __init__(self, index: int):
    self.samples, self.stop_flag, self.thread, self.h = [], False, None, None
    try:
      import pynvml
      pynvml.nvmlInit()
      self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
      self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
    except Exception as e:   # no NVML: report that instead of a number
      self.err = repr(e)

  def _run(self):
    nv = self.nv
    while not self.stop_flag:
      try:
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        try: reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception: reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        self.samples.append((mhz, reasons))
      except Exception: pass
      time.sleep(0.01)

  def __enter__(self):
    if self.h is not None:
      self.thread = threading.Thread(target=self._run, daemon=True); self.thread.start()
    return self

  def __exit__(self, *a):
    self.stop_flag = True
    if self.thread: self.thread.join()

  def summary(self) -> dict:
    if self.h is None or not self.samples: return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable: " + getattr(self, "err", "no samples")]}
    names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}
    seen = set()
    for _, r in self.samples:
      for bit, n in names.items():
        if r & bit: seen.add(n)
    return {"sm_mhz": float(np.median([m for m, _ in self.samples])), "sm_max_mhz": float(self.max_mhz), "reasons": sorted(seen),
            "samples": len(self.samples)}


def _use_all_host_threads():
  """torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm uses every thread this process may run on."""
  n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
  os.environ["OMP_NUM_THREADS"] = str(n)


def _block_linear_shapes(cfg):
  qd, kvd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
  return [(qd, cfg.dim), (kvd, cfg.dim), (kvd, cfg.dim), (cfg.dim, qd), (cfg.hidden_dim, cfg.dim), (cfg.hidden_dim, cfg.dim), (cfg.dim, cfg.hidden_dim)]


class CpuPortModel:
  """The linears of the whole model as raw Q4_0 blocks in host memory, for the C restatement of the reference's fused
  dequant-linear arithmetic (oracle/qgemv_cpu.c).  Every block has its own copy of the weights (4.2 GB in all for configs[1]):
  a step streams all of them from memory, as the reference does.  The values of block i are those of block i % 2 (generating
  7.5 G random quants on the host would take longer than the measurement); attention and norms are left out (< 1 % of the work)."""
  def __init__(self, cfg, seed: int = 0):
    _use_all_host_threads()
    from oracle import cpu_gemv
    from tinygrad_b200 import synth
    self.cfg, self.gemv = cfg, cpu_gemv.qgemv
    self.shapes = _block_linear_shapes(cfg)
    rng = np.random.default_rng(seed)
    base = [[synth.q4_0_blocks(o, i, rng) for o, i in self.shapes] for _ in range(min(2, cfg.num_blocks))]
    self.blocks = [[w.copy() for w in base[b % len(base)]] for b in range(cfg.num_blocks)]
    self.head = synth.q4_0_blocks(cfg.vocab_size, cfg.dim, rng)
    self.xs = {k: rng.standard_normal(k).astype(np.float32) for k in {i for _, i in self.shapes}}
    self.threads = cpu_gemv.n_threads()

  def step(self) -> None:
    for blk in self.blocks:
      for w, (o, i) in zip(blk, self.shapes): self.gemv(2, w, self.xs[i], o, i)
    self.gemv(2, self.head, self.xs[self.cfg.dim], self.cfg.vocab_size, self.cfg.dim)


def run_reference(args, rank):
  """The reference arm: the CPU implementation of the same path on the host cores (the C restatement of tinygrad's fused
  dequant-linear arithmetic; tinygrad's own CPU device needs clang, which this image lacks).  Every step is timed as it runs:
  all 32 blocks' linears and the vocabulary head, each block streaming its own weights."""
  if rank != 0: return
  m = CpuPortModel(llama3_8b_config())
  for _ in range(max(1, args.warmup)): m.step()
  t0 = time.perf_counter()
  for _ in range(args.steps): m.step()
  total = time.perf_counter() - t0
  v = args.steps / total
  sample_txt = ("each step = the 7 Q4_0 linears of all 32 blocks (own weight copy per block, 4.2 GB streamed) + the vocabulary head, raw GGUF blocks, "
                "fp32 activations; attention / norms omitted")
  print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic", "config": {"workload": WORKLOAD},
                    "cpu_baseline": {"value": v, "unit": UNIT, "cores": m.threads, "kind": "port", "sample": sample_txt},
                    "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


MOE_SHAPE = dict(T=4096, D=2048, F=1024, E=64, k=8)     # configs[3]: OLMoE-1B-7B-shaped layer


def moe_record(reps: int = 30) -> dict:
  """configs[3] on one GPU: one MXFP8 MoE FFN layer over 4096 tokens, timed with CUDA events (whole layer, then each phase alone).
  FLOPs are counted on the routed (unpadded) rows only: T * k * 3 * 2 * d * f."""
  from tinygrad_b200 import runtime, moe, _lib
  from tinygrad_b200._lib import BF16
  T, D, F, E, k = (MOE_SHAPE[n] for n in "TDFEk")
  rng = np.random.default_rng(0)
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.02) for s in ((E, F, D), (E, F, D), (E, D, F)))
  m = moe.MxMoE(wg, wu, wd, k, moe.ROUTE_SOFTMAX_TOPK)
  x = runtime.DeviceBuffer.from_numpy(moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32)))
  logits = runtime.DeviceBuffer.from_numpy(rng.standard_normal((T, E), dtype=np.float32))
  st = runtime.Stream()
  for _ in range(5): m(x, logits, T, stream=st)
  st.synchronize()
  e0, e1 = runtime.Event(), runtime.Event()
  e0.record(st)
  for _ in range(reps): m(x, logits, T, stream=st)
  e1.record(st); st.synchronize()
  ms = e0.elapsed_ms(e1) / reps
  phase_ms = {}
  for name, fn in m.phases(x, logits, T, st).items():
    runtime.synchronize()
    e0.record(st)
    for _ in range(reps): fn()
    e1.record(st); st.synchronize()
    phase_ms[name] = round(e0.elapsed_ms(e1) / reps, 4)
  flops = T * k * 3 * 2 * D * F
  pk = measured_peaks()
  fp8_peak = 2 * pk["bf16_tflops"]
  status = runtime.mx_status()
  return {"workload": "configs[3] one layer: OLMoE-shaped MXFP8 MoE FFN, 4096 tokens, 64 experts top-8, d 2048, f 1024, one GPU",
          "ms_per_layer": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "frac": round(flops / ms / 1e9 / fp8_peak, 4),
          "peak": f"2 x bf16 burst = {fp8_peak:.0f} TFLOP/s ({pk['source']}; no fp8 figure is measured)", "phase_ms": phase_ms,
          "contraction": "tcgen05.mma kind::mxf8f6f4.block_scale, TMEM accumulators", "wait_status": status}


def batched_record(B: int = 8, steps: int = 32) -> dict:
  """configs[2] shape (Qwen2-7B, Q8_0) decoding B sequences in lock-step after 128-token prompts: every Linear streams its weights once per step
  for all B rows (few-row fused GEMV on the int8 tensor cores), attention and arg-max per sequence; one CUDA graph per step."""
  from tinygrad_b200 import runtime, synth
  from tinygrad_b200.model import Transformer, TransformerConfig
  cfg = TransformerConfig(num_blocks=28, dim=3584, hidden_dim=18944, n_heads=28, n_kv_heads=4, norm_eps=1e-6, vocab_size=152064, head_dim=128,
                          rope_theta=1000000.0, rope_dim=128, v_head_dim=128, max_context=1024, kv_dtype="float16", qkv_bias=True)
  model = Transformer(cfg, synth.LazyDenseState(cfg, synth.Q8_0, seed=0, distinct_blocks=4), ggml_type=synth.Q8_0, batch=B)
  rng = np.random.default_rng(5)
  prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, 128)] for _ in range(B)]
  gen = model.generate_batch(prompts)
  for _ in range(4): next(gen)
  e0, e1 = runtime.Event(), runtime.Event()
  model.stream.synchronize()
  e0.record(model.stream)
  for _ in range(steps): model.decode_batch_step()
  e1.record(model.stream); model.stream.synchronize()
  ms = e0.elapsed_ms(e1) / steps
  pk = measured_peaks()
  kv = 2 * cfg.n_kv_heads * cfg.head_dim * 2 * cfg.num_blocks * (128 + 4 + steps // 2) * B
  gbs = (model.weight_bytes + kv) / ms / 1e6
  return {"workload": f"configs[2] shape: Qwen2-7B-shaped Q8_0 decode, batch {B} in lock-step, prompt 128 per sequence, greedy", "ms_per_step": round(ms, 3),
          "tokens_per_s": round(B * 1e3 / ms, 1), "step_hbm_gbs": round(gbs, 1), "step_frac_of_peak": round(gbs / pk["hbm_gbs"], 4),
          "wait_status": runtime.device_status()}


def ep_moe_record(ranks, reps: int = 10) -> dict:
  """configs[3] expert-parallel over all ranks: experts split contiguously, tokens split at the input; device time of the slowest rank.
  Every rank also computes its token shard on one GPU alone and compares bit for bit."""
  from tinygrad_b200 import runtime, moe, expert_parallel as ep
  from tinygrad_b200.runtime import DeviceBuffer
  T, D, F, E, k = (MOE_SHAPE[n] for n in "TDFEk")
  G, r = ranks.world, ranks.rank
  rng = np.random.default_rng(7)                                   # every rank draws the same full problem
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.02) for s in ((E, F, D), (E, F, D), (E, D, F)))
  x = moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32))
  logits = rng.standard_normal((T, E), dtype=np.float32)
  T_l, E_l = T // G, E // G
  from tinygrad_b200 import tensor_parallel as tpar
  sl = slice(r * E_l, (r + 1) * E_l)
  dx, dl = DeviceBuffer.from_numpy(x[r * T_l:(r + 1) * T_l]), DeviceBuffer.from_numpy(logits[r * T_l:(r + 1) * T_l])
  full = moe.MxMoE(wg, wu, wd, k, 1)
  ref = full(DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(logits), T).numpy()[r * T_l:(r + 1) * T_l]
  del full
  res = {}
  for name in ("peer", "nccl"):
    if name == "peer":
      shard = ep.PeerExpertParallelMoE(tpar.TPGroup(ranks, "peer"), wg[sl], wu[sl], wd[sl], E, k, T, 1)
      shard.connect()
    else: shard = ep.ExpertParallelMoE(ranks, wg[sl], wu[sl], wd[sl], E, k, T, 1)
    runtime.synchronize(); ranks.barrier()
    out = shard(dx, dl, T_l).numpy()
    for _ in range(3): shard(dx, dl, T_l)
    runtime.synchronize(); ranks.barrier()
    ms = ranks.max(shard.timed(dx, dl, T_l, reps))
    same = ranks.sum(float(np.array_equal(out, ref))) == G
    status = ranks.max(float(runtime.mx_status()))
    res[name] = {"ms_per_layer": round(ms, 4), "bit_identical_to_one_gpu": bool(same), "wait_status": int(status), "exchange": shard.exchange_kind}
    del shard
  flops = T * k * 3 * 2 * D * F
  best = res["peer"]
  return {"workload": f"configs[3] one layer, expert-parallel x{G}: {E_l} experts and {T_l} tokens per rank", "ms_per_layer": best["ms_per_layer"],
          "tflops": round(flops / best["ms_per_layer"] / 1e9, 1), "bit_identical_to_one_gpu": best["bit_identical_to_one_gpu"] and res["nccl"]["bit_identical_to_one_gpu"],
          "exchange": best["exchange"], "by_exchange": res}


def tp70b_record(ranks, steps: int, warmup: int) -> dict:
  """configs[4]: Llama-3-70B-shaped Q4_0 decode at batch 1, prompt 1024.  One rank: the whole model on one GPU (39 GB).  N ranks: tensor
  parallel (column-split QKV / gate / up / head, row-split O / down).  Values of block i are those of block i % 4 (own device memory
  per block; generating 70 G random quants on the host would dominate the run).  The prompt's KV cache is left zero (a decode step's cost
  does not depend on the cached values): the step reads 1024+ cached positions per block like the real thing."""
  from tinygrad_b200 import runtime, synth, tensor_parallel as tpar
  from tinygrad_b200.model import Transformer
  cfg, G = llama3_70b_config(), ranks.world
  prompt_len = 1024
  t0 = time.time()
  if G == 1:
    model = Transformer(cfg, synth.LazyDenseState(cfg, synth.Q4_0, seed=0, distinct_blocks=4), ggml_type=synth.Q4_0)
  else:
    tp = tpar.TPGroup(ranks)
    lc = tpar.local_config(cfg, G)
    sd = synth.LazyDenseState(lc, synth.Q4_0, seed=0, embd_vocab=cfg.vocab_size, linear_seed=1 + ranks.rank, distinct_blocks=4)
    model = Transformer(cfg, sd, ggml_type=synth.Q4_0, tp=tp)
  t_build = time.time() - t0
  prompt = [int(t) for t in np.random.default_rng(7).integers(0, cfg.vocab_size, prompt_len)]
  model.set_state(prompt, prompt_len - 1)
  for _ in range(max(3, warmup)): model.step()
  runtime.synchronize(); ranks.barrier()
  e0, e1 = runtime.Event(), runtime.Event()
  e0.record(model.stream)
  for _ in range(steps): model.step()
  e1.record(model.stream)
  runtime.synchronize(); ranks.barrier()
  ms = ranks.max(e0.elapsed_ms(e1)) / steps
  tok = float(model.read_token(prompt_len + 1))
  same = ranks.max(tok) == ranks.sum(tok) / G                 # every rank sampled the same token
  status = runtime.device_status()
  pk = measured_peaks()
  kv_bytes = 2 * model.config.n_kv_heads * cfg.head_dim * 2 * cfg.num_blocks * (prompt_len + max(3, warmup) + steps // 2)
  per_gpu = model.weight_bytes + kv_bytes
  rec = {"workload": f"configs[4]: Llama-3-70B-shaped Q4_0 decode bs1 at position {prompt_len}, " + ("one GPU" if G == 1 else f"tensor-parallel x{G}"),
         "tokens_per_s": round(1e3 / ms, 2), "ms_per_step": round(ms, 4), "n_gpus": G, "engine": model.engine, "weight_gb_per_gpu": round(model.weight_bytes / 1e9, 3),
         "hbm_gbs_per_gpu": round(per_gpu / ms / 1e6, 1), "frac_of_hbm_peak_per_gpu": round(per_gpu / ms / 1e6 / pk["hbm_gbs"], 4),
         "ranks_agree": bool(same), "wait_status": status, "model_build_s": round(t_build, 1)}
  if G > 1: rec["collective"] = model.tp.kind
  return rec


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=256)
  ap.add_argument("--warmup", type=int, default=8)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--engine", default=None, choices=["step", "chain"], help="one-token engine (default: the whole-step kernel where it takes the model)")
  ap.add_argument("--only", default="", help="comma list of records to run besides the headline (moe, batched, ep_moe, tp70b); default: all that apply")
  ap.add_argument("--skip-cpu-baseline", action="store_true")
  ap.add_argument("--workload", default="decode", choices=["decode", "moe", "batch"], help="moe / batch: only that record (short runs for profiling)")
  args = ap.parse_args()
  rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
  if args.impl == "reference": return run_reference(args, rank)
  if args.warmup < 3: args.warmup = 3
  extras = set(args.only.split(",")) - {""} if args.only else {"moe", "batched", "ep_moe", "tp70b"}

  from tinygrad_b200 import build, runtime, synth, _lib
  from tinygrad_b200.model import Transformer
  build.build_lib()
  if args.workload == "moe":
    runtime.set_device(local)
    print(json.dumps({"moe": moe_record(reps=max(args.steps, 1))}), flush=True)
    return
  if args.workload == "batch":
    runtime.set_device(local)
    print(json.dumps({"batched": batched_record(steps=max(min(args.steps, 64), 1))}), flush=True)
    return
  from tinygrad_b200.replicas import Ranks
  ranks = Ranks(backend="nccl")
  runtime.set_device(local)
  cfg, qtype = llama3_8b_config(), synth.Q4_0
  t_build = time.time()
  model = Transformer(cfg, synth.LazyDenseState(cfg, qtype, seed=rank), ggml_type=qtype, engine=args.engine)
  t_build = time.time() - t_build
  prompt = [int(t) for t in np.random.default_rng(1000 + rank).integers(0, cfg.vocab_size, PROMPT_LEN)]
  # the prompt (outside the timed decode region) goes through the tensor-core GEMM path; the second pass is timed (the first allocates)
  for _ in range(2):
    model.set_state(prompt, 0)
    t_pf = time.time()
    model.prefill(0, PROMPT_LEN - 1)
    model.stream.synchronize()
    t_pf = time.time() - t_pf
  prefill_info = {"tokens": PROMPT_LEN - 1, "ms": round(1e3 * t_pf, 2), "tokens_per_s": round((PROMPT_LEN - 1) / t_pf, 1),
                  "note": "host wall clock around the whole prompt pass (second call), tcgen05 dequant GEMMs"}

  def barrier():
    runtime.synchronize(); ranks.barrier(); runtime.synchronize()

  if PROMPT_LEN + args.warmup + args.steps + 2 > MAX_CONTEXT:
    raise SystemExit(f"--steps {args.steps} does not fit the {MAX_CONTEXT}-token context after a {PROMPT_LEN}-token prompt")
  e0, e1 = runtime.Event(), runtime.Event()
  sampler = ClockSampler(local)
  with sampler:
    # ---- device-resident: tokens feed back on the device, K steps back to back
    for _ in range(args.warmup): model.step()
    barrier()
    e0.record(model.stream)
    for _ in range(args.steps): model.step()
    e1.record(model.stream)
    barrier()
    ms_dev = ranks.max(e0.elapsed_ms(e1))
    # ---- end to end: per step, the token id goes host->device from pinned memory, the sampled id comes back
    pin_in, pin_out = runtime.PinnedBuffer((1,), np.int32), runtime.PinnedBuffer((1,), np.int32)
    lib = _lib.load()
    pos = PROMPT_LEN - 1                      # rewind to the end of the prompt: same positions as the device-resident pass
    model.set_state([], pos)
    pin_in.array[0] = prompt[-1]
    def e2e_step(p):
      lib.b200q_memcpy_h2d(model.tokens.ptr + 4 * p, pin_in.ptr, 4, model.stream.ptr)
      model.step()
      lib.b200q_memcpy_d2h(pin_out.ptr, model.tokens.ptr + 4 * (p + 1), 4, model.stream.ptr)
      model.stream.synchronize()
      pin_in.array[0] = pin_out.array[0]
    for _ in range(args.warmup): e2e_step(pos); pos += 1
    barrier()
    e0.record(model.stream)
    t0 = time.perf_counter()
    for _ in range(args.steps): e2e_step(pos); pos += 1
    e1.record(model.stream)
    barrier()
    ms_e2e = ranks.max(max(e0.elapsed_ms(e1), 1e3 * (time.perf_counter() - t0)))
    ms_gemv = None
    if model.engine == "chain":   # the dominant kernel alone: every GEMV launch of one step, chained, weights cold (4.2 GB >> L2)
      g = model.gemv_only_graph()
      for _ in range(3): g.launch()
      barrier()
      e0.record(model.stream)
      for _ in range(20): g.launch()
      e1.record(model.stream)
      barrier()
      ms_gemv = e0.elapsed_ms(e1) / 20
  wait_status = runtime.device_status()
  pk = measured_peaks()
  peak = pk["hbm_gbs"]
  kv_bytes_per_pos = 2 * cfg.n_kv_heads * cfg.head_dim * 2 * cfg.num_blocks
  step_bytes = model.weight_bytes + kv_bytes_per_pos * (PROMPT_LEN + args.warmup + args.steps // 2) + 2 * cfg.dim + 4 * cfg.vocab_size
  ms_step = ms_dev / args.steps
  if model.engine == "step":
    # one launch = one step: algorithmic bytes = every weight block once + the cached K/V rows + the embedding row + the logits
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                "kernel": "decode_step_kernel<Q4_0, fp16 KV> (the whole step is one launch)", "peak_source": pk["source"], "launches_timed": args.steps,
                "bytes_per_launch": step_bytes, "us_per_launch_avg": 1e3 * ms_step}
    launches = args.steps
  else:
    shapes = model.gemv_launches()
    gemv_bytes = sum(o * i // 32 * 18 + 4 * i + 4 * o for o, i in shapes)
    achieved = gemv_bytes / (ms_gemv * 1e-3) / 1e9
    # DRAM bytes per launch are not measured here (that takes ncu): the captures of this kernel inside a decode step read 1.005-1.007 x
    # the algorithmic bytes from DRAM (profiles/qgemv_q4_0_o_proj_and_gate_up_in_decode_step.md), which is what `traffic` scales by
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_RATIO * gemv_bytes / len(shapes), "traffic_source": f"ncu capture of two launches: dram bytes = {NCU_TRAFFIC_RATIO} x algorithmic",
                "kernel": "qgemv_kernel<Q4_0> (the GEMV launches of a step alone, chained)", "peak_source": pk["source"], "launches_timed": len(shapes) * 20,
                "bytes_per_launch_avg": gemv_bytes / len(shapes), "us_per_launch_avg": 1e3 * ms_gemv / len(shapes)}
    launches = model.launches_per_step * args.steps
  out = {"metric": METRIC, "value": world * args.steps / (ms_dev * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
         "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
         "config": {"workload": WORKLOAD, "parallelism": f"replicas x{world}", "engine": model.engine,
                    "l2": "inputs larger than L2 (4.2 GB of weights per step vs 126 MB)",
                    "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9, "step_frac_of_peak": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
                    "wait_status": wait_status, "model_build_s": round(t_build, 1)},
         "roofline": roofline,
         "e2e": {"value": world * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
         "gpu_launches": launches, "clocks": sampler.summary(), "prefill": prefill_info}
  del model
  # ---- the other configurations of the path, each in its own record
  if world == 1 and "moe" in extras: out["moe"] = moe_record()
  if world == 1 and "batched" in extras:
    out["batched"] = batched_record()
    b32 = batched_record(B=32, steps=16)       # 4 passes of 8 rows over the weights per Linear
    out["batched"]["batch_32"] = {k: b32[k] for k in ("ms_per_step", "tokens_per_s", "wait_status")}
  if world > 1 and "ep_moe" in extras: out["ep_moe"] = ep_moe_record(ranks)
  if "tp70b" in extras: out["tp70b"] = tp70b_record(ranks, min(args.steps, 64), args.warmup)
  if rank == 0 and not args.skip_cpu_baseline and world == 1:
    m = CpuPortModel(cfg)
    m.step()
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < 10.0: m.step(); reps += 1
    out["cpu_baseline"] = {"value": reps / (time.perf_counter() - t0), "unit": UNIT, "cores": m.threads, "kind": "port",
                           "sample": f"C restatement of the fused dequant-linears, {reps} whole steps (all 32 blocks, own weights per block, + the head); attention/norms omitted"}
  if rank == 0: print(json.dumps(out), flush=True)
  if world > 1: os._exit(0)      # captured graphs hold NCCL work: leave without tearing the process group down
  ranks.close()


if __name__ == "__main__":
  main()
