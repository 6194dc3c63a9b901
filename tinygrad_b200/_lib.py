"""ctypes binding of libb200q.so.  There is no fallback: if the library is
missing or a call fails, the Python wrappers raise."""
import ctypes, pathlib
from ctypes import c_int, c_int32, c_int64, c_size_t, c_float, c_void_p, c_char_p, POINTER, Structure

import os
LIB_PATH = pathlib.Path(os.environ.get("B200Q_LIB") or pathlib.Path(__file__).resolve().parent / "libb200q.so")   # B200Q_LIB: another build of the library

Q4_0, Q8_0, Q6_K = 2, 8, 14
F32, F16, BF16 = 0, 1, 2
EPI_LINEAR, EPI_SILU_MUL = 0, 1
FLAG_PDL = 1


class GemvArgs(Structure):
  _fields_ = [("qtype", c_int), ("n_out", c_int), ("n_in", c_int), ("m", c_int), ("w_packed", c_void_p), ("x", c_void_p),
              ("x_dtype", c_int), ("y_dtype", c_int), ("norm_weight", c_void_p), ("norm_eps", c_float), ("epilogue", c_int),
              ("bias", c_void_p), ("residual", c_void_p), ("y", c_void_p), ("flags", c_int), ("max_ctas", c_int),
              ("xq_in", c_void_p), ("ss_in", c_void_p), ("ss_count", c_int), ("xq_out", c_void_p), ("xq_out_norm_weight", c_void_p),
              ("ss_out", c_void_p), ("residual_scale", c_float), ("peer_mailboxes", POINTER(c_void_p)), ("n_peers", c_int), ("peer_rank", c_int),
              ("xq_out_stage", c_void_p)]


class AttnArgs(Structure):
  _fields_ = [("qkv", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("kv_dtype", c_int), ("rope", c_void_p), ("pos", c_void_p),
              ("out", c_void_p), ("scratch", c_void_p), ("n_heads", c_int), ("n_kv_heads", c_int), ("head_dim", c_int), ("rope_dim", c_int),
              ("max_context", c_int), ("n_split", c_int), ("flags", c_int), ("xq_out", c_void_p)]


class DecodeLayer(Structure):
  _fields_ = [("qkv", c_void_p), ("qkv_bias", c_void_p), ("attn_output", c_void_p), ("gate_up", c_void_p), ("ffn_down", c_void_p),
              ("attn_norm", c_void_p), ("ffn_norm", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p)]


class DecodeStepArgs(Structure):
  _fields_ = [("layers", c_void_p), ("n_layers", c_int), ("qtype", c_int), ("dim", c_int), ("hidden_dim", c_int), ("n_heads", c_int),
              ("n_kv_heads", c_int), ("head_dim", c_int), ("rope_dim", c_int), ("max_context", c_int), ("vocab", c_int), ("embd_vocab", c_int),
              ("kv_dtype", c_int), ("norm_eps", c_float), ("token_embd", c_void_p), ("output_norm", c_void_p), ("output", c_void_p),
              ("rope", c_void_p), ("tokens", c_void_p), ("pos", c_void_p), ("x", c_void_p), ("qkv", c_void_p), ("attn", c_void_p),
              ("act", c_void_p), ("logits", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("with_head", c_int), ("profile_stamps", c_int),
              ("profile", c_void_p)]


class EpArgs(Structure):
  _fields_ = [("n_ranks", c_int), ("rank", c_int), ("n_experts", c_int), ("k", c_int), ("d_model", c_int), ("n_tokens", c_int), ("m_max", c_int),
              ("topi", c_void_p), ("dest", c_void_p), ("off", c_void_p), ("counts", c_void_p), ("counts_all", POINTER(c_void_p)),
              ("a_q", POINTER(c_void_p)), ("a_e8", POINTER(c_void_p)), ("y", POINTER(c_void_p)), ("flags", POINTER(c_void_p)),
              ("send_base", c_void_p), ("off_local", c_void_p), ("remote_row", c_void_p), ("scratch", c_void_p)]


# name -> (restype, argtypes); every symbol include/b200q.h declares
SIGNATURES = {
  "b200q_strerror": (c_char_p, [c_int]),
  "b200q_last_cuda_error": (c_char_p, []),
  "b200q_version": (c_int, []),
  "b200q_status_read_clear": (c_int, [POINTER(c_int)]),
  "b200q_device_count": (c_int, [POINTER(c_int)]),
  "b200q_set_device": (c_int, [c_int]),
  "b200q_device_props": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_size_t)]),
  "b200q_malloc": (c_int, [POINTER(c_void_p), c_size_t]),
  "b200q_free": (c_int, [c_void_p]),
  "b200q_host_alloc": (c_int, [POINTER(c_void_p), c_size_t]),
  "b200q_host_free": (c_int, [c_void_p]),
  "b200q_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
  "b200q_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
  "b200q_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
  "b200q_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
  "b200q_stream_create": (c_int, [POINTER(c_void_p)]),
  "b200q_stream_destroy": (c_int, [c_void_p]),
  "b200q_stream_synchronize": (c_int, [c_void_p]),
  "b200q_device_synchronize": (c_int, []),
  "b200q_event_create": (c_int, [POINTER(c_void_p)]),
  "b200q_event_destroy": (c_int, [c_void_p]),
  "b200q_event_record": (c_int, [c_void_p, c_void_p]),
  "b200q_event_synchronize": (c_int, [c_void_p]),
  "b200q_event_elapsed_ms": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
  "b200q_graph_begin": (c_int, [c_void_p]),
  "b200q_graph_end": (c_int, [c_void_p, POINTER(c_void_p)]),
  "b200q_graph_launch": (c_int, [c_void_p, c_void_p]),
  "b200q_graph_destroy": (c_int, [c_void_p]),
  "b200q_dequant_raw": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
  "b200q_packed_bytes": (c_size_t, [c_int, c_int, c_int]),
  "b200q_repack": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
  "b200q_dequant_packed": (c_int, [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
  "b200q_gemv": (c_int, [POINTER(GemvArgs), c_void_p]),
  "b200q_mailbox_reduce": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]),
  "b200q_ipc_export": (c_int, [c_void_p, c_void_p]),
  "b200q_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
  "b200q_ipc_close": (c_int, [c_void_p]),
  "b200q_ep_publish_counts": (c_int, [POINTER(EpArgs), c_void_p]),
  "b200q_ep_plan": (c_int, [POINTER(EpArgs), c_void_p]),
  "b200q_ep_dispatch": (c_int, [POINTER(EpArgs), c_void_p, c_void_p]),
  "b200q_ep_wait": (c_int, [POINTER(EpArgs), c_int, c_int, c_void_p]),
  "b200q_ep_signal_results": (c_int, [POINTER(EpArgs), c_void_p]),
  "b200q_ep_combine": (c_int, [POINTER(EpArgs), c_void_p, c_void_p, c_void_p]),
  "b200q_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
  "b200q_tg_gemv": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
  "b200q_embed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
  "b200q_xq_bytes": (c_size_t, [c_int]),
  "b200q_attn_min_split": (c_int, [c_int]),
  "b200q_attn_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
  "b200q_attn_decode": (c_int, [POINTER(AttnArgs), c_void_p]),
  "b200q_attn_seq_scratch_stride": (c_size_t, [c_int, c_int, c_int, c_int]),
  "b200q_attn_decode_seqs": (c_int, [POINTER(AttnArgs), c_int, c_void_p]),
  "b200q_attn_decode_static_capacity": (c_size_t, []),
  "b200q_attn_decode_static": (c_int, [POINTER(AttnArgs), c_void_p]),
  "b200q_decode_step_supported": (c_int, [POINTER(DecodeStepArgs)]),
  "b200q_decode_step_workspace_bytes": (c_size_t, [POINTER(DecodeStepArgs)]),
  "b200q_decode_step": (c_int, [POINTER(DecodeStepArgs), c_void_p]),
  "b200q_argmax_scratch_bytes": (c_size_t, []),
  "b200q_argmax_advance": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
  "b200q_advance": (c_int, [c_void_p, c_int, c_int, c_void_p]),
  "b200q_gemm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
  "b200q_qgemm": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
  "b200q_qgemm_workspace_bytes": (c_size_t, [c_int, c_int]),
  "b200q_qgemm_ws": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
  "b200q_qgemv_rows_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
  "b200q_qgemv_rows": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                               c_void_p]),
  "b200q_qgemv_rows_norm": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                   c_void_p]),
  "b200q_qgemm_skinny_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
  "b200q_qgemm_skinny": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                c_void_p]),
  "b200q_embed_rows": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
  "b200q_rmsnorm_rows": (c_int, [c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_int, c_void_p]),
  "b200q_add_rows_gated": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
  "b200q_add_rows_bf16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
  "b200q_attn_prefill": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_int, c_void_p]),
  "b200q_attn_decode_batch": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_int, c_void_p]),
  "b200q_tc_status_read_clear": (c_int, [POINTER(c_int)]),
  "b200q_quantize_mxfp8": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
  "b200q_gemv_dense": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int,
                              c_void_p]),
  "b200q_swiglu_quantize_mxfp8": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
  "b200q_moe_route_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
  "b200q_moe_rows_max": (c_int, [c_int, c_int, c_int]),
  "b200q_moe_route": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
  "b200q_moe_route_pad": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
  "b200q_moe_route_gating": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p]),
  "b200q_moe_route_tables": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
  "b200q_permute_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p]),
  "b200q_moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
  "b200q_mx_status_read_clear": (c_int, [POINTER(c_int)]),
  "b200q_grouped_mxfp8_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
  "b200q_grouped_mxfp8_gemm_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
  "b200q_fp8_absmax": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p]),
  "b200q_fp8_quantize": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
  "b200q_fp8_scale_bias": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
  "b200q_grouped_mxfp8_gemm_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                             c_void_p]),
}

_lib = None


class B200QError(RuntimeError):
  pass


def load() -> ctypes.CDLL:
  """Load the shared library (building it is the job of tinygrad_b200.build)."""
  global _lib
  if _lib is not None: return _lib
  if not LIB_PATH.exists():
    raise B200QError(f"{LIB_PATH} is missing: run `python -m tinygrad_b200.build` (there is no CPU fallback)")
  lib = ctypes.CDLL(str(LIB_PATH))
  for name, (res, args) in SIGNATURES.items():
    fn = getattr(lib, name)
    fn.restype, fn.argtypes = res, args
  _lib = lib
  return lib


def check(rc: int) -> None:
  """Raise on a negative status, like `check(status)` of tinygrad/runtime/ops_cuda.py:13-16."""
  if rc == 0: return
  lib = load()
  msg = lib.b200q_strerror(rc).decode()
  if rc == -5: msg += ": " + lib.b200q_last_cuda_error().decode()
  raise B200QError(f"b200q error {rc}: {msg}")
