"""ctypes binding of libb200grad.so.

The reference reaches its kernels through a ctypes wrapper of the HIP runtime
plus by-name kernel lookup in code objects (reference:
src/runtime/hip_dispatch.py:100-587, src/kernels/launcher.py:26-130).  Here the
library exports one C launcher per kernel and a step driver; tensors come from
PyTorch and are passed as raw device pointers with the current CUDA stream.

There is no silent fallback: importing an op on a machine with a GPU but without
the built library raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import torch

LIB_PATH = Path(os.environ.get("B200GRAD_LIB") or Path(__file__).resolve().parent.parent / "lib" / "libb200grad.so")
MAX_TP = 8
MAX_ROWS = 8

EPI_STORE_F16, EPI_SILU_PAIR, EPI_STORE_F32, EPI_FINISH = 0, 1, 2, 3
FIN_NO_COMM, FIN_NO_H_WRITE, FIN_SAVE_EXTRA, FIN_ADD_EXTRA, FIN_NO_NORM = 1, 2, 4, 8, 16
FIN_TEST_WITHHOLD_SIGNAL = 32
LIN_INT4, LIN_F16, LIN_NONE = 0, 1, 2
STEP_EMBED_TOKENS, STEP_LM_HEAD, STEP_ARGMAX, STEP_ADVANCE, STEP_NO_COMMIT_DELTA = 1, 2, 4, 8, 16
STEP_MATERIALIZE_XN = 32
STEP_SPEC, STEP_GEMM_PATH = 64, 128

vp, i32, f32, i64 = C.c_void_p, C.c_int, C.c_float, C.c_longlong


class CommCtx(C.Structure):
    _fields_ = [("tp", i32), ("rank", i32), ("part_stride", i32), ("pad0", i32),
                ("part", vp * MAX_TP), ("sig", vp * MAX_TP), ("mc_part", vp),
                ("epoch", vp), ("status", vp), ("wait_ns", i64), ("trace", vp),
                ("tpart", vp * MAX_TP), ("tsig", vp * MAX_TP), ("tile_h", i32), ("tile_flags", i32)]


class RowMeta(C.Structure):
    _fields_ = [("seq", i32), ("pos", i32), ("slot", i32), ("ctx", i32), ("mask", C.c_ulonglong)]


class SeqState(C.Structure):
    _fields_ = [("len", i32), ("token", i32), ("pad", i32 * 2)]


class LazyNorm(C.Structure):
    _fields_ = [("h", vp), ("ss", vp), ("w", vp), ("np", i32), ("H", i32), ("eps", f32), ("pad", i32)]


class GemvEpi(C.Structure):
    _fields_ = [("mode", i32), ("ldo", i32), ("n_valid", i32), ("fin_flags", i32), ("out", vp),
                ("h", vp), ("norm_w", vp), ("xn", vp), ("extra", vp), ("local_part", vp),
                ("hout", vp), ("ss_part", vp), ("eps", f32), ("ss_np", i32)]


class GemvInt4Params(C.Structure):
    _fields_ = [("qfrag", vp), ("szfrag", vp), ("x", vp),
                ("ldx", i32), ("rows", i32), ("K", i32), ("KB", i32), ("NTL", i32), ("G", i32),
                ("off32", i32), ("gshift", i32), ("k_splits", i32), ("L", i32), ("cluster_splitk", i32), ("tag_base", i32),
                ("scratch", vp), ("counters", vp), ("tag_word", vp),
                ("pf_q", vp), ("pf_KB", i32), ("pf_L", i32), ("pf_nx", i32), ("pf_ks", i32), ("pf_blocks", i32), ("pf_pad", i32), ("pf_span", vp), ("pf_span_bytes", i64),
                ("ln", LazyNorm), ("epi", GemvEpi), ("comm", CommCtx)]


class GemvF16Params(C.Structure):
    _fields_ = [("w", vp), ("x", vp), ("ldw", i32), ("ldx", i32), ("rows", i32), ("K", i32), ("N", i32),
                ("k_splits", i32), ("kslice", i32), ("scratch", vp), ("counters", vp),
                ("ln", LazyNorm), ("epi", GemvEpi), ("comm", CommCtx)]


CH_MAX_OPS = 4


class ChainOp(C.Structure):
    _fields_ = [("qfrag", vp), ("szfrag", vp), ("x", vp), ("ldx", i32), ("K", i32), ("KB", i32), ("NWT", i32),
                ("G", i32), ("off32", i32), ("gshift", i32), ("gsz", i32), ("cBase", i32), ("cRem", i32), ("pmax", i32),
                ("pad", i32),
                ("ln", LazyNorm), ("epi", GemvEpi),
                ("th_out", vp), ("tss_out", vp), ("tact_out", vp), ("th_in", vp), ("tss_in", vp), ("tact_in", vp),
                ("th_res", vp), ("in_op", i32), ("res_op", i32)]


class ChainParams(C.Structure):
    _fields_ = [("n_ops", i32), ("rows", i32), ("stages", i32), ("xf_chunks", i32), ("op", ChainOp * CH_MAX_OPS),
                ("scratch", vp), ("counters", vp), ("tag_h", vp), ("tag_ss", vp), ("tag_act", vp),
                ("tag_h_cols", i32), ("tag_ss_cols", i32), ("tag_act_cols", i32), ("pad1", i32),
                ("prof", vp), ("comm", CommCtx)]


class AttnParams(C.Structure):
    _fields_ = [("q", vp), ("ldq", i32), ("gate_off", i32), ("kcache", vp), ("vcache", vp), ("rows", vp),
                ("out", vp), ("ldo", i32), ("n_rows", i32), ("nq", i32), ("nkv", i32), ("max_seq", i32),
                ("splits", i32), ("scale", f32), ("scratch", vp), ("counters", vp)]


class DeltaParams(C.Structure):
    _fields_ = [("proj", vp), ("ld", i32), ("off_q", i32), ("off_k", i32), ("off_v", i32), ("off_z", i32),
                ("off_a", i32), ("off_b", i32), ("xn", vp), ("ldx", i32), ("H", i32), ("wa", vp), ("wb", vp),
                ("conv_w", vp), ("conv_state", vp), ("state", vp), ("A_log", vp), ("dt_bias", vp),
                ("norm_w", vp), ("seq_rows", vp), ("rows", vp), ("out", vp), ("ldo", i32), ("nk", i32),
                ("nv", i32), ("n_seqs", i32), ("eps", f32), ("commit", i32), ("ln", LazyNorm)]


class ArgmaxParams(C.Structure):
    _fields_ = [("logits", vp), ("ld", i32), ("n_rows", i32), ("vocab_local", i32), ("vocab_offset", i32),
                ("blocks", i32), ("scratch", vp), ("counters", vp), ("out_tokens", vp), ("seqs", vp),
                ("rows", vp), ("comm", CommCtx)]


class GemmTcParams(C.Structure):
    _fields_ = [("qfrag", vp), ("szfrag", vp), ("K", i32), ("KB", i32), ("NTL", i32), ("G", i32), ("off32", i32),
                ("gshift", i32), ("T", i32), ("t_tile", i32), ("n_valid", i32), ("ldo", i32), ("epi", i32),
                ("stages", i32), ("out", vp), ("status", vp), ("m_halves", i32), ("dense", i32),
                ("push", vp * MAX_TP), ("epoch", vp), ("part_stride", i64), ("push_tp", i32), ("push_rank", i32),
                ("push_per", C.c_uint), ("k_splits", i32), ("cta_pair", i32), ("pad3", i32)]


TC_EPI_STORE_F16, TC_EPI_SILU_PAIR, TC_EPI_STORE_F32, TC_EPI_RESID_F32 = 0, 1, 2, 3


class LinearDesc(C.Structure):
    _fields_ = [("kind", i32), ("K", i32), ("N", i32), ("KB", i32), ("NTL", i32), ("G", i32), ("off32", i32),
                ("gshift", i32), ("k_splits", i32), ("L", i32), ("ldw", i32), ("kslice", i32), ("pad", i32),
                ("w", vp), ("sz", vp)]


class LayerDesc(C.Structure):
    _fields_ = [("type", i32), ("type_index", i32), ("in_proj", LinearDesc), ("out_proj", LinearDesc),
                ("gate_up", LinearDesc), ("down", LinearDesc), ("attn_norm", vp), ("ffn_norm", vp), ("next_norm", vp),
                ("q_norm", vp), ("k_norm", vp), ("kcache", vp), ("vcache", vp),
                ("wa", vp), ("wb", vp), ("conv_w", vp), ("conv_state", vp), ("state", vp),
                ("A_log", vp), ("dt_bias", vp), ("la_norm", vp),
                ("off_q", i32), ("off_k", i32), ("off_v", i32), ("off_z", i32), ("off_a", i32), ("off_b", i32),
                ("ffn_kind", i32), ("q8_group", i32), ("q8_F", i32), ("pad_q8", i32),
                ("q8_w", vp * 3), ("q8_s", vp * 3), ("wab", vp)]


class SampleParams(C.Structure):
    _fields_ = [("logits", vp), ("ld", i32), ("n_rows", i32), ("vocab", i32), ("vocab_offset", i32),
                ("temperature", f32), ("top_p", f32), ("rep_penalty", f32), ("top_k", i32),
                ("past", vp), ("n_past", vp), ("max_past", i32), ("vocab_total", i32), ("seed", C.c_ulonglong),
                ("out_tokens", vp), ("dbg_ids", vp), ("dbg_probs", vp), ("comm", CommCtx)]


SAMPLE_MAX_CAND = 1024


class Quant8Params(C.Structure):
    _fields_ = [("w", vp), ("w_scale", vp), ("g_scale", vp), ("xq", vp), ("x_scale", vp), ("out", vp),
                ("K", i32), ("N", i32), ("T", i32), ("ldo", i32), ("group", i32), ("out_f16", i32),
                ("w4", i32), ("pad", i32)]


class ActQuantParams(C.Structure):
    _fields_ = [("x", vp), ("xq", vp), ("scale", vp), ("T", i32), ("K", i32), ("ldx", i32), ("pad", i32)]


class SpecStage(C.Structure):
    _fields_ = [("base", vp), ("layer_stride", i64), ("seq_stride", i64), ("off_k", i32), ("off_u", i32),
                ("off_g", i32), ("off_x", i32)]


SPEC_MAX_NODES = 16


class ModelDesc(C.Structure):
    _fields_ = [("n_layers", i32), ("H", i32), ("vocab", i32), ("vocab_local", i32), ("vocab_offset", i32),
                ("nq", i32), ("nkv", i32), ("hd", i32), ("rot", i32), ("rope_interleaved", i32),
                ("la_nk", i32), ("la_nv", i32), ("la_dk", i32), ("la_dv", i32),
                ("max_seq", i32), ("max_rows", i32), ("ar_mode", i32),
                ("attn_splits", i32), ("argmax_blocks", i32), ("n_seqs_max", i32),
                ("eps", f32), ("F_pad", i32),
                ("embed", vp), ("first_norm", vp), ("lm_head", LinearDesc),
                ("cos_tab", vp), ("sin_tab", vp),
                ("h", vp), ("xn", vp), ("proj", vp), ("ld_proj", i32), ("pad0", i32),
                ("attn_out", vp), ("ld_attn", i32), ("pad1", i32),
                ("act", vp), ("logits", vp), ("ld_logits", i32), ("pad2", i32),
                ("gemv_scratch", vp), ("gemv_counters", vp), ("attn_scratch", vp), ("attn_counters", vp),
                ("argmax_scratch", vp), ("argmax_counters", vp), ("extra", vp), ("h_tmp", vp),
                ("ss", vp), ("np", i32), ("pad3", i32),
                ("rows", vp), ("rows_tmpl", vp), ("seqs", vp), ("row_tokens", vp), ("seq_rows", vp),
                ("out_tokens", vp),
                ("max_prefill", i32), ("pad4", i32), ("p_h", vp), ("p_xn", vp), ("p_proj", vp), ("p_attn", vp),
                ("p_act", vp), ("p_partial", vp), ("p_rows", vp), ("p_rows_tmpl", vp), ("p_row_tokens", vp),
                ("tc_status", vp), ("p_ab", vp), ("coll_gather", vp * MAX_TP), ("coll_mc_gather", vp), ("coll_counters", vp),
                ("p_logits", vp), ("p_argmax_scratch", vp), ("p_argmax_counters", vp), ("p_out_tokens", vp),
                ("p_attn_scratch", vp), ("p_attn_counters", vp),
                ("p_logit_rows", i32), ("n_lin_layers", i32), ("n_full_layers", i32), ("ab_off", i32),
                ("spec", SpecStage), ("spec_acc", vp), ("spec_result", vp),
                ("state0", vp), ("conv0", vp), ("state_layer_stride", i64), ("conv_layer_stride", i64),
                ("k0", vp), ("v0", vp), ("kv_layer_stride", i64),
                ("xn_sym", vp * MAX_TP), ("xn_mc", vp), ("hlast_sym", vp * MAX_TP), ("seq_parallel", i32), ("tagged_splitk", i32),
                ("chain_scratch", vp), ("chain_counters", vp), ("chain_act_cols", i32), ("use_chain", i32),
                ("chain_tag_h", vp), ("chain_tag_ss", vp), ("chain_tag_act", vp),
                ("q8_xq", vp), ("q8_sx", vp), ("q8_gate", vp), ("q8_up", vp), ("q8_down", vp), ("q8_xn", vp),
                ("comm", CommCtx)]


_SIZE_CHECKS = {
    "b2_sizeof_comm_ctx": CommCtx, "b2_sizeof_gemv_int4_params": GemvInt4Params,
    "b2_sizeof_gemv_f16_params": GemvF16Params, "b2_sizeof_attn_params": AttnParams,
    "b2_sizeof_delta_params": DeltaParams, "b2_sizeof_argmax_params": ArgmaxParams,
    "b2_sizeof_linear_desc": LinearDesc, "b2_sizeof_layer_desc": LayerDesc,
    "b2_sizeof_model_desc": ModelDesc, "b2_sizeof_spec_stage": SpecStage, "b2_sizeof_sample_params": SampleParams, "b2_sizeof_quant8_params": Quant8Params, "b2_sizeof_act_quant_params": ActQuantParams, "b2_sizeof_gemm_tc_params": GemmTcParams, "b2_sizeof_row_meta": RowMeta, "b2_sizeof_seq_state": SeqState,
    "b2_sizeof_chain_params": ChainParams, "b2_sizeof_chain_op": ChainOp,
}

_lib: Optional[C.CDLL] = None


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library (built on first use when nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if os.environ.get("B200GRAD_NO_AUTOBUILD"):
            raise NativeLibraryMissing(f"{LIB_PATH} is missing: run `python -m mi50grad_b200.build`")
        from ..build import build_all
        build_all()
    _lib = C.CDLL(str(LIB_PATH))
    for fn, st in _SIZE_CHECKS.items():
        f = getattr(_lib, fn)
        f.restype = i32
        if f() != C.sizeof(st):
            raise RuntimeError(f"struct layout mismatch for {st.__name__}: C {f()} vs ctypes {C.sizeof(st)}")
    _lib.b2_driver_create.restype = vp
    _lib.b2_driver_launches.restype = i64
    _lib.b2_driver_chain_launches.restype = i64
    _lib.b2_driver_exchanges.restype = i64
    _lib.b2_driver_total_launches.restype = i64
    _lib.b2_driver_total_exchanges.restype = i64
    _lib.b2_chain_scratch_floats.restype = i64
    _lib.b2_gemv_int4_smem.restype = C.c_size_t
    return _lib


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    return t.data_ptr()


def stream() -> vp:
    return vp(torch.cuda.current_stream().cuda_stream)


def check(code: int, what: str = "kernel launch"):
    if code != 0:
        name = f"cudaError {code}"
        raise RuntimeError(f"{what} failed: {name}")


def null_comm() -> CommCtx:
    c = CommCtx()
    c.tp, c.rank = 1, 0
    return c
