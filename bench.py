"""Headline benchmark: decode tokens/s of a Llama-3-8B-shaped Q4_0 model at batch 1 on B200,
plus the achieved HBM bandwidth of the quant GEMV kernel against the measured peak.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step (one token through all blocks, head and arg-max).  Weights,
embeddings, prompt ids are seeded synthetic data of the configuration's shapes (no
checkpoint or dataset is involved).  For N > 1 (launched by torch.distributed.run) every
rank decodes its own sequence on its own GPU: replicas, no data-path collective.
Prints ONE JSON line on rank 0.
"""
import argparse, json, os, sys, time, threading, pathlib
import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC, UNIT = "decode tokens/s (8B-shape Q4_0, bs1)", "tokens/s"
WORKLOAD = "configs[1]: Llama-3-8B-shaped decode, Q4_0 linears, fp16 embeddings/norms, fp16 KV cache, batch 1, prompt 512 random ids, greedy"
PROMPT_LEN, MAX_CONTEXT = 512, 2048


def llama3_8b_config():
  from tinygrad_b200.model import TransformerConfig
  return TransformerConfig(num_blocks=32, dim=4096, hidden_dim=14336, n_heads=32, n_kv_heads=8, norm_eps=1e-5, vocab_size=128256, head_dim=128,
                           rope_theta=500000.0, rope_dim=128, v_head_dim=128, max_context=MAX_CONTEXT, kv_dtype="float16")


def qwen2_7b_config():
  from tinygrad_b200.model import TransformerConfig
  return TransformerConfig(num_blocks=28, dim=3584, hidden_dim=18944, n_heads=28, n_kv_heads=4, norm_eps=1e-6, vocab_size=152064, head_dim=128,
                           rope_theta=1000000.0, rope_dim=128, v_head_dim=128, max_context=MAX_CONTEXT, kv_dtype="float16", qkv_bias=True)


def measured_peaks():
  p = ROOT / "MEASURED_PEAKS.json"
  if p.exists():
    return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
  return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


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


def cpu_port_block_seconds(cfg, reps_budget_s: float, seed: int = 0):
  """Time the C restatement on the host cores: the 7 linears of one block and the head, raw GGUF blocks.
  Returns (seconds per block, seconds for the head, threads, repetitions)."""
  _use_all_host_threads()
  from oracle import cpu_gemv
  from tinygrad_b200 import synth
  qd, kvd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
  shapes = [(qd, cfg.dim), (kvd, cfg.dim), (kvd, cfg.dim), (cfg.dim, qd), (cfg.hidden_dim, cfg.dim), (cfg.hidden_dim, cfg.dim), (cfg.dim, cfg.hidden_dim)]
  rng = np.random.default_rng(seed)
  ws = [synth.q4_0_blocks(o, i, rng) for o, i in shapes]
  head = synth.q4_0_blocks(cfg.vocab_size, cfg.dim, rng)
  xs = {k: rng.standard_normal(k).astype(np.float32) for k in {i for _, i in shapes}}
  def block():
    for w, (o, i) in zip(ws, shapes): cpu_gemv.qgemv(2, w, xs[i], o, i)
  block(); cpu_gemv.qgemv(2, head, xs[cfg.dim], cfg.vocab_size, cfg.dim)      # warm
  t0, reps = time.perf_counter(), 0
  while True:
    block(); reps += 1
    if time.perf_counter() - t0 > reps_budget_s * 0.7: break
  t_blk = (time.perf_counter() - t0) / reps
  t0, hreps = time.perf_counter(), 0
  while True:
    cpu_gemv.qgemv(2, head, xs[cfg.dim], cfg.vocab_size, cfg.dim); hreps += 1
    if time.perf_counter() - t0 > reps_budget_s * 0.3: break
  t_head = (time.perf_counter() - t0) / hreps
  return t_blk, t_head, cpu_gemv.n_threads(), reps


def run_reference(args, rank):
  """The reference arm: the CPU implementation of the same path on the host cores (the C restatement
  of tinygrad's fused dequant-linear arithmetic; tinygrad's own CPU device needs clang, which this image lacks)."""
  if rank != 0: return
  _use_all_host_threads()
  from oracle import cpu_gemv
  from tinygrad_b200 import synth
  cfg = llama3_8b_config()
  qd, kvd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
  shapes = [(qd, cfg.dim), (kvd, cfg.dim), (kvd, cfg.dim), (cfg.dim, qd), (cfg.hidden_dim, cfg.dim), (cfg.hidden_dim, cfg.dim), (cfg.dim, cfg.hidden_dim)]
  rng = np.random.default_rng(0)
  ws = [synth.q4_0_blocks(o, i, rng) for o, i in shapes]
  head = synth.q4_0_blocks(cfg.vocab_size, cfg.dim, rng)
  xs = {k: rng.standard_normal(k).astype(np.float32) for k in {i for _, i in shapes}}
  def sample():
    t0 = time.perf_counter()
    for w, (o, i) in zip(ws, shapes): cpu_gemv.qgemv(2, w, xs[i], o, i)
    t1 = time.perf_counter()
    cpu_gemv.qgemv(2, head, xs[cfg.dim], cfg.vocab_size, cfg.dim)
    return (t1 - t0) * cfg.num_blocks + (time.perf_counter() - t1)       # one block's linears x 32 + the head = one token
  for _ in range(args.warmup): sample()
  total = sum(sample() for _ in range(args.steps))
  v = args.steps / total
  threads = cpu_gemv.n_threads()
  sample_txt = "each step = the 7 Q4_0 linears of ONE block (timed, x32 blocks) + the vocab head, raw GGUF blocks, fp32 activations; attention/norms omitted"
  print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                    "data": "synthetic", "config": {"workload": WORKLOAD},
                    "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_txt},
                    "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_gemv_probe(args):
  """Micro-benchmark of one GEMV shape (profiling aid; prints its own JSON line, not the headline).
  Rotates over enough distinct weight buffers that every launch reads HBM-cold weights."""
  from tinygrad_b200 import build, runtime, synth, quant
  build.build_lib()
  runtime.set_device(0)
  n_out, n_in = (int(v) for v in args.gemv_shape.split("x"))
  wbytes = n_out * n_in // 32 * 18
  n_rot = max(2, -(-args.rotate_mb * (1 << 20) // wbytes))
  raw = synth.q4_0_blocks(n_out, n_in, np.random.default_rng(0))
  ws = [quant.repack(raw, n_out, n_in, synth.Q4_0) for _ in range(n_rot)]
  x = runtime.DeviceBuffer.from_numpy(np.random.default_rng(1).standard_normal(n_in).astype(np.float32))
  y = runtime.DeviceBuffer.empty((n_out,), np.float32)
  st = runtime.Stream()
  fl = 0 if args.no_pdl else 1
  lib = __import__("tinygrad_b200._lib", fromlist=["load"]).load()
  xq = runtime.DeviceBuffer(lib.b200q_xq_bytes(n_in), zero=True) if args.probe_xq else None   # an all-zero record times like any other
  res = runtime.DeviceBuffer.empty((n_out,), np.float32, zero=True) if args.probe_residual else None
  def enqueue(n):
    for i in range(n): quant.gemv(ws[i % n_rot].buf.ptr, synth.Q4_0, n_out, n_in, x, y, flags=fl, stream=st, xq_in=xq, residual=res, max_ctas=args.gemv_ctas)
  enqueue(args.warmup); st.synchronize()
  g = runtime.Graph(st)
  with g: enqueue(args.steps)
  g.launch(); st.synchronize()
  e0, e1 = runtime.Event(), runtime.Event()
  e0.record(st); g.launch(); e1.record(st); st.synchronize()
  us = 1e3 * e0.elapsed_ms(e1) / args.steps
  peak, src = measured_peaks()
  gbs = (wbytes + 4 * n_in + 4 * n_out) / us / 1e3
  print(json.dumps({"workload": f"gemv probe Q4_0 {n_out}x{n_in}, {n_rot} rotating weight buffers", "us_per_launch": us, "gbs": gbs,
                    "frac_of_peak": gbs / peak, "peak_source": src, "launches": args.steps, "pdl": not args.no_pdl}))


def run_moe_probe(args):
  """One OLMoE-shaped MXFP8 MoE FFN layer over 4096 tokens (configs[3], single GPU); prints its own JSON line.
  FLOPs counted on the useful (routed, unpadded) rows only: T * k * 3 * 2 * d * f."""
  from tinygrad_b200 import build, runtime, moe
  build.build_lib()
  runtime.set_device(0)
  T, D, F, E, k = 4096, 2048, 1024, 64, 8
  rng = np.random.default_rng(0)
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.02) for s in ((E, F, D), (E, F, D), (E, D, F)))
  m = moe.MxMoE(wg, wu, wd, k, moe.ROUTE_SOFTMAX_TOPK)
  x = runtime.DeviceBuffer.from_numpy(moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32)))
  logits = runtime.DeviceBuffer.from_numpy(rng.standard_normal((T, E), dtype=np.float32))
  st = runtime.Stream()
  for _ in range(max(3, args.warmup)): m(x, logits, T, stream=st)
  st.synchronize()
  e0, e1 = runtime.Event(), runtime.Event()
  steps = min(args.steps, 50)
  e0.record(st)
  for _ in range(steps): m(x, logits, T, stream=st)
  e1.record(st); st.synchronize()
  ms = e0.elapsed_ms(e1) / steps
  # each phase alone, back to back on the same buffers
  lib = __import__("tinygrad_b200._lib", fromlist=["load"]).load()
  from tinygrad_b200._lib import BF16
  r, ws = m.last_routing, m._ws
  phases = {
    "route": lambda: ws["r"].run(logits, st),
    "zero_fill": lambda: (ws["a_q"].zero_(st), ws["a_e8"].zero_(st)),
    "dispatch_quantize": lambda: lib.b200q_quantize_mxfp8(x.ptr, BF16, T, D, r.dest_row.ptr, k, ws["a_q"].ptr, ws["a_e8"].ptr, st.ptr),
    "gate_up_gemm": lambda: lib.b200q_grouped_mxfp8_gemm(ws["a_q"].ptr, ws["a_e8"].ptr, m.gu_q.ptr, m.gu_e8.ptr, r.off.ptr, E, r.m_l, 2 * F, D, ws["h"].ptr, st.ptr),
    "gate_up_gemm_swiglu_fused": lambda: lib.b200q_grouped_mxfp8_gemm_swiglu(ws["a_q"].ptr, ws["a_e8"].ptr, m.gu_q.ptr, m.gu_e8.ptr, r.off.ptr, E, r.m_l, 2 * F, D,
                                                                             ws["act_q"].ptr, ws["act_e8"].ptr, st.ptr),
    "swiglu_quantize_unfused": lambda: lib.b200q_swiglu_quantize_mxfp8(ws["h"].ptr, r.m_l, r.off.ptr + 4 * E, F, ws["act_q"].ptr, ws["act_e8"].ptr, st.ptr),
    "down_gemm": lambda: lib.b200q_grouped_mxfp8_gemm(ws["act_q"].ptr, ws["act_e8"].ptr, m.dn_q.ptr, m.dn_e8.ptr, r.off.ptr, E, r.m_l, D, F, ws["y"].ptr, st.ptr),
    "combine": lambda: lib.b200q_moe_combine(ws["y"].ptr, r.dest_row.ptr, r.weights.ptr, T, k, D, ws["out"].ptr, st.ptr),
  }
  phase_ms = {}
  for name, fn in phases.items():
    runtime.synchronize()
    e0.record(st)
    for _ in range(steps): fn()
    e1.record(st); st.synchronize()
    phase_ms[name] = round(e0.elapsed_ms(e1) / steps, 4)
  ms_gemm1 = phase_ms["gate_up_gemm"]
  flops = T * k * 3 * 2 * D * F
  peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {"bf16_tflops": 1590.0}
  fp8_peak = 2 * peaks["bf16_tflops"]
  print(json.dumps({"workload": "configs[3] one layer: OLMoE-shaped MXFP8 MoE FFN, 4096 tokens, 64 experts top-8, d 2048, f 1024",
                    "ms_per_layer": ms, "tflops": flops / ms / 1e9, "frac_of_fp8_peak": flops / ms / 1e9 / fp8_peak,
                    "fp8_peak": f"2 x measured bf16 burst = {fp8_peak} TFLOP/s (no fp8 entry in MEASURED_PEAKS.json)",
                    "phase_ms": phase_ms, "gate_up_gemm_ms": ms_gemm1, "gate_up_gemm_tflops": T * k * 2 * 2 * D * F / ms_gemm1 / 1e9,
                    "contraction": "tcgen05.mma kind::mxf8f6f4.block_scale, 128x256x128 tiles, TMEM accumulators"}))


def run_batch_probe(args):
  """configs[2] batched decode: B sequences in lock-step through the tensor-core GEMM path; prints its own JSON line."""
  from tinygrad_b200 import build, runtime, synth
  from tinygrad_b200.model import Transformer
  from dataclasses import replace
  build.build_lib()
  runtime.set_device(0)
  cfg, qtype = (qwen2_7b_config(), synth.Q8_0) if args.model == "qwen7b_q8" else (llama3_8b_config(), synth.Q4_0)
  if args.blocks: cfg = replace(cfg, num_blocks=args.blocks)
  B, plen = args.batch, 128
  model = Transformer(cfg, synth.LazyDenseState(cfg, qtype, seed=0), ggml_type=qtype, batch=B)
  rng = np.random.default_rng(5)
  prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, plen)] for _ in range(B)]
  gen = model.generate_batch(prompts)
  for _ in range(max(3, args.warmup)): next(gen)
  e0, e1 = runtime.Event(), runtime.Event()
  steps = min(args.steps, 64)
  model.stream.synchronize()
  e0.record(model.stream)
  for _ in range(steps): model.decode_batch_step()
  e1.record(model.stream); model.stream.synchronize()
  ms = e0.elapsed_ms(e1) / steps
  peak, src = measured_peaks()
  kv = 2 * cfg.n_kv_heads * cfg.head_dim * 2 * cfg.num_blocks * (plen + args.warmup + steps // 2) * B
  print(json.dumps({"workload": f"configs[2]-style batched decode, {args.model}, batch {B}, prompt {plen} per sequence, greedy, lock-step",
                    "ms_per_step": ms, "tokens_per_s": B * 1e3 / ms, "step_hbm_gbs": (model.weight_bytes + kv) / ms / 1e6,
                    "step_frac_of_peak": (model.weight_bytes + kv) / ms / 1e6 / peak, "peak_source": src,
                    "path": "tcgen05 dequant GEMM over the batch rows (weights streamed once per step), per-sequence attention and arg-max"}))


def run_tp_probe(args):
  """configs[4]: Llama-3-70B-shaped Q4_0 decode, batch 1, tensor-parallel over all ranks (column QKV/gate/up/head, row O/down,
  NCCL all-reduce).  Launch under torch.distributed.run; prints its own JSON line on rank 0.  Shards are generated per rank."""
  from tinygrad_b200 import build, runtime, synth, tensor_parallel as tpar
  from tinygrad_b200.replicas import Ranks
  from tinygrad_b200.model import Transformer, TransformerConfig
  build.build_lib()
  ranks = Ranks(backend="nccl")
  runtime.set_device(ranks.local)
  tp = tpar.TPGroup(ranks)
  prompt_len, ctx = (1024, 2048) if not args.blocks else (64, 256)
  cfg = TransformerConfig(num_blocks=args.blocks or 80, dim=8192, hidden_dim=28672, n_heads=64, n_kv_heads=8, norm_eps=1e-5, vocab_size=128256,
                          head_dim=128, rope_theta=500000.0, rope_dim=128, v_head_dim=128, max_context=ctx, kv_dtype="float16")
  lc = tpar.local_config(cfg, ranks.world)
  t0 = time.time()
  sd = synth.LazyDenseState(lc, synth.Q4_0, seed=0, embd_vocab=cfg.vocab_size, linear_seed=1 + ranks.rank)
  model = Transformer(cfg, sd, ggml_type=synth.Q4_0, tp=tp, use_pdl=not args.no_pdl)
  t_build = time.time() - t0
  prompt = [int(t) for t in np.random.default_rng(7).integers(0, cfg.vocab_size, prompt_len)]
  if args.skip_prefill: model.set_state(prompt, prompt_len - 1)
  else:
    model.set_state(prompt, 0)
    for _ in range(prompt_len - 1): model.step(with_head=False)
  for _ in range(max(3, args.warmup)): model.step()
  runtime.synchronize(); ranks.barrier()
  e0, e1 = runtime.Event(), runtime.Event()
  e0.record(model.stream)
  for _ in range(args.steps): model.step()
  e1.record(model.stream)
  runtime.synchronize(); ranks.barrier()
  ms = ranks.max(e0.elapsed_ms(e1))
  toks = [model.read_token(prompt_len + i) for i in range(4)]
  same = ranks.max(float(toks[0])) == ranks.sum(float(toks[0])) / ranks.world       # every rank sampled the same token
  peak, src = measured_peaks()
  total_bytes = model.weight_bytes * ranks.world
  if ranks.rank == 0:
    print(json.dumps({"workload": f"configs[4]: Llama-3-70B-shaped Q4_0 decode bs1, prompt {prompt_len}, tensor-parallel x{ranks.world}" +
                      (f" DEBUG {args.blocks} blocks" if args.blocks else ""), "tokens_per_s": args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
                      "n_gpus": ranks.world, "weight_gb_total": total_bytes / 1e9, "hbm_gbs_per_gpu": model.weight_bytes / (ms / args.steps * 1e-3) / 1e9,
                      "frac_of_hbm_peak_per_gpu": model.weight_bytes / (ms / args.steps * 1e-3) / 1e9 / peak, "collectives_per_step": 2 * cfg.num_blocks + 1,
                      "ranks_agree": bool(same), "model_build_s": round(t_build, 1)}), flush=True)
  os._exit(0)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "moe", "tp70b", "batch"])
  ap.add_argument("--batch", type=int, default=8, help="sequences of the batched-decode probe (--workload batch)")
  ap.add_argument("--gemv-shape", default="28672x4096", help="rows x K of the probe (gate+up interleaved = 28672x4096)")
  ap.add_argument("--rotate-mb", type=int, default=512)
  ap.add_argument("--probe-xq", action="store_true", help="gemv probe: hand the kernel a ready-made activation record")
  ap.add_argument("--probe-residual", action="store_true", help="gemv probe: add a residual vector in the epilogue")
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=256)
  ap.add_argument("--warmup", type=int, default=8)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--blocks", type=int, default=0, help="debug: fewer transformer blocks (the reported line is then not the headline workload)")
  ap.add_argument("--no-pdl", action="store_true")
  ap.add_argument("--gemv-ctas", type=int, default=0, help="tuning: cap on the CTAs of one GEMV launch (0 = library default)")
  ap.add_argument("--handover", default=None, help="tuning: comma list of hand-over edges (attn_o,o_gateup,gateup_down,down_qkv), 'none' or 'all'")
  ap.add_argument("--model", choices=["llama8b_q4", "qwen7b_q8"], default="llama8b_q4", help="llama8b_q4 = configs[1] (the benchmark); qwen7b_q8 = configs[2] at batch 1")
  ap.add_argument("--prefill", choices=["gemm", "steps"], default="gemm", help="how the 512-token prompt is processed before the timed decode steps")
  ap.add_argument("--skip-prefill", action="store_true", help="debug/profiling: start at the end of the prompt with an all-zero KV cache")
  ap.add_argument("--skip-cpu-baseline", action="store_true")
  args = ap.parse_args()
  rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
  if args.impl == "reference": return run_reference(args, rank)
  if args.workload == "gemv": return run_gemv_probe(args)
  if args.workload == "moe": return run_moe_probe(args)
  if args.workload == "tp70b": return run_tp_probe(args)
  if args.workload == "batch": return run_batch_probe(args)
  if args.warmup < 3: args.warmup = 3

  from tinygrad_b200 import build, runtime, synth
  from tinygrad_b200.model import Transformer
  from dataclasses import replace
  build.build_lib()
  from tinygrad_b200.replicas import Ranks
  ranks = Ranks(backend="nccl")
  runtime.set_device(local)
  global METRIC, WORKLOAD
  cfg, qtype = llama3_8b_config(), synth.Q4_0
  if args.model == "qwen7b_q8":       # configs[2] at batch 1 (a probe: the benchmark proper is configs[1])
    cfg, qtype = qwen2_7b_config(), synth.Q8_0
    METRIC = "decode tokens/s (Qwen2-7B-shape Q8_0, bs1)"
    WORKLOAD = "configs[2] at batch 1: Qwen2-7B-shaped decode, Q8_0 linears with q/k/v bias, fp16 embeddings/norms, fp16 KV cache, prompt 512 random ids, greedy"
  if args.blocks: cfg = replace(cfg, num_blocks=args.blocks)
  t_build = time.time()
  model = Transformer(cfg, synth.LazyDenseState(cfg, qtype, seed=rank), ggml_type=qtype, use_pdl=not args.no_pdl, gemv_max_ctas=args.gemv_ctas,
                      handover={None: None, 'none': False, 'all': True}.get(args.handover, args.handover))
  t_build = time.time() - t_build
  prompt = [int(t) for t in np.random.default_rng(1000 + rank).integers(0, cfg.vocab_size, PROMPT_LEN)]
  # prompt (outside the timed decode region): the tensor-core GEMM path, or one position per step through the decode kernels
  prefill_info = None
  if args.skip_prefill: model.set_state(prompt, PROMPT_LEN - 1)
  else:
    model.set_state(prompt, 0)
    for rep in range(2 if args.prefill == "gemm" else 1):      # the first GEMM-path call also allocates its row buffers: time the second
      model.set_state(prompt, 0)
      t_pf = time.time()
      if args.prefill == "gemm": model.prefill(0, PROMPT_LEN - 1)
      else:
        for _ in range(PROMPT_LEN - 1): model.step(with_head=False)
      model.stream.synchronize()
      t_pf = time.time() - t_pf
    prefill_info = {"path": args.prefill, "tokens": PROMPT_LEN - 1, "ms": round(1e3 * t_pf, 2), "tokens_per_s": round((PROMPT_LEN - 1) / t_pf, 1),
                    "note": "host wall clock around the whole prompt pass (second call)"}
  model.stream.synchronize()

  def barrier():
    runtime.synchronize()
    ranks.barrier()
    runtime.synchronize()

  max_over_ranks = ranks.max

  if PROMPT_LEN + args.warmup + args.steps + 2 > MAX_CONTEXT:
    raise SystemExit(f"--steps {args.steps} does not fit the {MAX_CONTEXT}-token context after a {PROMPT_LEN}-token prompt")
  e0, e1 = runtime.Event(), runtime.Event()
  sampler = ClockSampler(local)
  with sampler:
    # ---- device-resident: tokens feed back on the device, K graph replays back to back
    for _ in range(args.warmup): model.step()
    barrier()
    e0.record(model.stream)
    for _ in range(args.steps): model.step()
    e1.record(model.stream)
    barrier()
    ms_dev = max_over_ranks(e0.elapsed_ms(e1))
    # ---- end to end: per step, the token id goes host->device from pinned memory, the sampled id comes back
    pin_in, pin_out = runtime.PinnedBuffer((1,), np.int32), runtime.PinnedBuffer((1,), np.int32)
    lib = __import__("tinygrad_b200._lib", fromlist=["load"]).load()
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
    ms_e2e = max_over_ranks(max(e0.elapsed_ms(e1), 1e3 * (time.perf_counter() - t0)))
    # ---- the dominant kernel alone: every GEMV launch of one step, chained, weights cold (4.2 GB >> L2)
    g = model.gemv_only_graph()
    for _ in range(3): g.launch()
    barrier()
    reps = 20
    e0.record(model.stream)
    for _ in range(reps): g.launch()
    e1.record(model.stream)
    barrier()
    ms_gemv = e0.elapsed_ms(e1) / reps
  launches = model.gemv_launches()
  blk_bytes = 18 if qtype == synth.Q4_0 else 34
  gemv_bytes = sum(o * i // 32 * blk_bytes + 4 * i + 4 * o for o, i in launches)     # quant blocks + fp32 activations in + out
  peak, peak_src = measured_peaks()
  achieved = gemv_bytes / (ms_gemv * 1e-3) / 1e9
  kv_bytes_per_pos = 2 * cfg.n_kv_heads * cfg.head_dim * 2 * cfg.num_blocks
  step_bytes = model.weight_bytes + kv_bytes_per_pos * (PROMPT_LEN + args.warmup + args.steps // 2)
  if rank != 0:
    ranks.close()
    return
  value = world * args.steps / (ms_dev * 1e-3)
  out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
         "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
         "config": {"workload": WORKLOAD if not (args.blocks or args.skip_prefill) else f"DEBUG (blocks={args.blocks}, skip_prefill={args.skip_prefill}) of: " + WORKLOAD, "parallelism": f"replicas x{world}",
                    "l2": "inputs larger than L2 (4.2 GB of weights per step vs 126 MB)", "pdl": not args.no_pdl, "n_split": model.n_split, "activation_handover": sorted(model.edges),
                    "step_hbm_gbs": step_bytes / (ms_dev / args.steps * 1e-3) / 1e9, "step_frac_of_peak": step_bytes / (ms_dev / args.steps * 1e-3) / 1e9 / peak,
                    "model_build_s": round(t_build, 1)},
         "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": 1.007 * gemv_bytes / len(launches),
                      "traffic_source": "ncu dram bytes on the 28672x4096 launch = 1.007 x algorithmic (profiles/qgemv_q4_0_28672x4096.md), scaled by bytes",
                      "kernel": "qgemv_kernel<Q4_0>" if qtype == synth.Q4_0 else "qgemv_kernel<Q8_0>", "peak_source": peak_src, "launches_timed": len(launches) * reps,
                      "bytes_per_launch_avg": gemv_bytes / len(launches), "us_per_launch_avg": 1e3 * ms_gemv / len(launches)},
         "e2e": {"value": world * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
         "gpu_launches": model.launches_per_step * args.steps, "clocks": sampler.summary()}
  if prefill_info: out["prefill"] = prefill_info
  if not args.skip_cpu_baseline and world == 1:
    t_blk, t_head, threads, reps_cpu = cpu_port_block_seconds(cfg, 12.0)
    out["cpu_baseline"] = {"value": 1.0 / (t_blk * cfg.num_blocks + t_head), "unit": UNIT, "cores": threads, "kind": "port",
                           "sample": f"C restatement, {reps_cpu} repetitions of one block's 7 Q4_0 linears (x{cfg.num_blocks}) + the vocab head; attention/norms omitted"}
  print(json.dumps(out))
  ranks.close()


if __name__ == "__main__":
  main()
