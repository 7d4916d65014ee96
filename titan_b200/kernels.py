"""Python face of the hand-written CUDA library: argument structs and checked calls.

Every function here launches kernels of ``titan_b200/csrc`` on the given CUDA
stream and raises ``KernelError`` with the launcher's message when it refuses
its arguments.  Nothing here computes on the host and nothing falls back to a
library: if the extension cannot be built or loaded, the first call raises.
"""
from __future__ import annotations

import ctypes
import sys
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

EPI_STORE, EPI_F32, EPI_ADD, EPI_SWIGLU = 0, 1, 2, 3
F32, BF16 = 0, 1
# What the SWIGLU epilogue makes of a (gate, up) pair of sums (csrc/activation.h): silu(g) u; gelu_tanh(g) u; or, with
# g' = min(g, limit) and u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1).
ACT_SILU, ACT_GELU_TANH, ACT_SWISH_CLAMPED = 0, 1, 2
GATES = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "swish_clamped": ACT_SWISH_CLAMPED}

launch_count = 0          # launcher calls since import (a launcher starts one or two kernels)
_launch_log = None        # while a log is open: launcher name -> calls (berniehans/titan keeps such a record per launch, engine-cuda/src/dispatch_telemetry.rs:13-143)


def launch_log_start() -> None:
    """Begin counting launcher calls by name (what a step launched, and how often)."""
    global _launch_log
    _launch_log = {}


def launch_log_stop() -> dict:
    """End the count; {launcher name: calls}, in the order of first use."""
    global _launch_log
    log, _launch_log = _launch_log or {}, None
    return log


class KernelError(RuntimeError):
    pass


def timeline_attach(buffer: Optional[torch.Tensor]) -> bool:
    """Names the buffer (int64, 1 + 8 * records) in which the decode kernels' timeline probe keeps its records, or
    takes it away (None).  False if the tensor-core library was built without the probe (csrc/timeline.cuh: it is
    compiled in with TITAN_B200_NVCC_FLAGS=-DTB_TIMELINE and costs nothing otherwise)."""
    ptr = None if buffer is None else buffer.data_ptr()
    on = [int(f(c_void_p(ptr))) for f in (tlib().tb_gemm_tc_timeline, alib().tb_attn_mma_timeline)]
    return all(v == 1 for v in on)


class KvView(Structure):
    _fields_ = [("storage", c_void_p), ("table", c_void_p), ("table_width", c_int), ("ring_rows", c_int),
                ("page_size", c_int), ("num_pages", c_int), ("kv_heads", c_int), ("head_dim", c_int)]


class Batch(Structure):
    _fields_ = [("tokens", c_void_p), ("seq_of", c_void_p), ("pos_of", c_void_p), ("slot_of_seq", c_void_p),
                ("q_start", c_void_p), ("start_pos", c_void_p), ("kv_len", c_void_p),
                ("T", c_int), ("B", c_int), ("max_new", c_int), ("max_kv_len", c_int)]


class RotaryArgs(Structure):
    """What a position encoding hands to the kernels; a mixer passes it on without looking inside.
    angle_k(position) = (position + offset) * inv_freq[k]; cosines and sines are scaled by ``magnitude``."""
    _fields_ = [("inv_freq", c_void_p), ("rot", c_int), ("offset", c_float), ("magnitude", c_float), ("adjacent", c_int)]


class QkArgs(Structure):
    _fields_ = [("inp", c_void_p), ("in_stride", c_int), ("q_out", c_void_p), ("q_stride", c_int),
                ("k_out", c_void_p), ("k_stride", c_int), ("q_w", c_void_p), ("k_w", c_void_p),
                ("rope", RotaryArgs), ("eps", c_float), ("nh", c_int), ("nkv", c_int),
                ("hd", c_int), ("pos_of", c_void_p), ("seq_of", c_void_p), ("slot_of_seq", c_void_p),
                ("cache", KvView), ("append", c_int), ("T", c_int), ("zero_in", c_int), ("kv_len", c_void_p),
                ("row_sumsq", c_void_p), ("row_parts", c_int), ("row_width", c_int), ("row_eps", c_float),
                ("norm_dims", c_int), ("norm_after", c_int),
                ("v_first", c_void_p), ("v_first_stride", c_int), ("v_mix", c_void_p), ("v_keep", c_void_p), ("v_keep_stride", c_int),
                ("v_first_head", c_int), ("v_norm_dims", c_int), ("v_eps", c_float)]


class AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_int), ("kv_new", c_void_p), ("kv_stride", c_int),
                ("out", c_void_p), ("out_stride", c_int), ("cache", KvView), ("batch", Batch),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int), ("scale", c_float),
                ("chunk", c_int), ("n_splits", c_int), ("scratch", c_void_p),
                ("early_len", c_void_p), ("early_mode", c_int), ("fused_qk", POINTER(QkArgs)),
                ("hd_v", c_int), ("v_alias", c_int), ("head_blocks", c_int), ("sink", c_void_p), ("keep_first", c_int),
                ("softcap", c_float), ("rel_bias", c_void_p), ("rel_far", c_int), ("head_mix", c_void_p),
                ("head_gate", c_void_p), ("head_gate_stride", c_int)]


class LatentArgs(Structure):
    """Arguments of the kernel between the input projection of a latent-attention mixer and its attention (csrc/latent.cu)."""
    _fields_ = [("inp", c_void_p), ("in_stride", c_int), ("q_nope", c_void_p), ("qn_stride", c_int),
                ("q_abs", c_void_p), ("qa_stride", c_int), ("kv_rows", c_void_p), ("kv_stride", c_int),
                ("latent_w", c_void_p), ("eps", c_float), ("rope", RotaryArgs),
                ("H", c_int), ("dn", c_int), ("rd", c_int), ("r", c_int), ("dk", c_int), ("owner", c_int),
                ("pos_of", c_void_p), ("seq_of", c_void_p), ("slot_of_seq", c_void_p), ("kv_len", c_void_p),
                ("cache", KvView), ("append", c_int), ("T", c_int), ("q_full", c_void_p), ("qf_stride", c_int), ("kv_in", c_void_p)]


class SplitAttnArgs(Structure):
    """Arguments of the tensor-core prompt attention with keys in two parts (csrc/attention_mma.cu: tb_attn_prefill_split)."""
    _fields_ = [("q", c_void_p), ("q_stride", c_int), ("kv", c_void_p), ("kv_stride", c_int), ("k_col0", c_int), ("v_col0", c_int),
                ("tail", c_void_p), ("tail_stride", c_int), ("tail_col0", c_int), ("out", c_void_p), ("out_stride", c_int),
                ("batch", Batch), ("nh", c_int), ("dn", c_int), ("dt", c_int), ("dv", c_int), ("window", c_int), ("scale", c_float)]


class LightningArgs(Structure):
    """Arguments of the decayed linear-attention recurrence (csrc/lightning.cu)."""
    _fields_ = [("proj", c_void_p), ("stride", c_int), ("out", c_void_p), ("out_stride", c_int), ("state", c_void_p),
                ("decay", c_void_p), ("q_start", c_void_p), ("slot_of_seq", c_void_p),
                ("B", c_int), ("H", c_int), ("dk", c_int), ("dv", c_int), ("max_new", c_int), ("plain", c_int)]


class WholeNormArgs(Structure):
    """Arguments of the kernel between a fused Q | K | V projection with biases and attention whose queries and keys are
    normed over the whole projection (csrc/attention_mixed.cu: tb_qkv_whole_norm)."""
    _fields_ = [("inp", c_void_p), ("in_stride", c_int), ("bias", c_void_p), ("q_w", c_void_p), ("k_w", c_void_p), ("eps", c_float),
                ("q_count", c_int), ("k_count", c_int), ("q_out", c_void_p), ("q_stride", c_int), ("kv_out", c_void_p), ("kv_stride", c_int),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int),
                ("pos_of", c_void_p), ("seq_of", c_void_p), ("slot_of_seq", c_void_p), ("kv_len", c_void_p),
                ("cache", KvView), ("append", c_int), ("T", c_int),
                ("o_bias", c_void_p), ("o_out", c_void_p), ("o_stride", c_int), ("o_width", c_int)]


class WkvArgs(Structure):
    """Arguments of the wkv mixer's kernels (csrc/wkv.cu)."""
    _fields_ = [("h", c_void_p), ("h_stride", c_int), ("mixes", c_void_p), ("mix_stride", c_int), ("mu", c_void_p),
                ("proj", c_void_p), ("proj_stride", c_int), ("lora", c_void_p), ("lora_stride", c_int), ("w2", c_void_p),
                ("w0", c_void_p), ("decay", c_void_p), ("u", c_void_p), ("out", c_void_p), ("out_stride", c_int),
                ("state", c_void_p), ("state_stride", c_longlong), ("norm_w", c_void_p), ("y", c_void_p), ("y_stride", c_int),
                ("eps", c_float), ("q_start", c_void_p), ("slot_of_seq", c_void_p), ("seq_of", c_void_p),
                ("T", c_int), ("B", c_int), ("H", c_int), ("dk", c_int), ("W", c_int), ("rank", c_int), ("max_new", c_int)]


class HyperArgs(Structure):
    """Arguments of the kernel between two sublayers of a model with several residual streams (csrc/hyper.cu)."""
    _fields_ = [("xs", c_void_p), ("S", c_int), ("W", c_int), ("rows", c_int), ("y", c_void_p), ("mix", c_void_p), ("out_w", c_void_p),
                ("zero_y", c_int), ("in_w", c_void_p), ("norm_w", c_void_p), ("eps", c_float), ("h", c_void_p)]


class DeltaPrepArgs(Structure):
    """Arguments of the kernel between the delta-rule mixer's projections and its recurrence (csrc/recurrent.cu)."""
    _fields_ = [("proj", c_void_p), ("stride", c_int), ("taps", c_void_p), ("n_taps", c_int), ("state", c_void_p), ("state_stride", c_longlong),
                ("conv_off", c_int), ("ba", c_void_p), ("ba_stride", c_int), ("a_log", c_void_p), ("dt_bias", c_void_p),
                ("qkv", c_void_p), ("qkv_stride", c_int), ("gates", c_void_p), ("gates_stride", c_int),
                ("seq_of", c_void_p), ("q_start", c_void_p), ("slot_of_seq", c_void_p),
                ("T", c_int), ("H", c_int), ("G", c_int), ("dk", c_int), ("dv", c_int)]


class ScanArgs(Structure):
    """Arguments of the recurrences over a matrix state: the gated delta rule and the mLSTM memory (csrc/recurrent.cu)."""
    _fields_ = [("q", c_void_p), ("q_stride", c_int), ("k", c_void_p), ("k_stride", c_int), ("v", c_void_p), ("v_stride", c_int),
                ("group", c_int), ("gates", c_void_p), ("gates_stride", c_int), ("i_bias", c_void_p), ("f_bias", c_void_p), ("cap", c_float),
                ("q_scale", c_float), ("out", c_void_p), ("out_stride", c_int), ("state", c_void_p), ("state_stride", c_longlong),
                ("q_start", c_void_p), ("slot_of_seq", c_void_p), ("B", c_int), ("H", c_int), ("dk", c_int), ("dv", c_int),
                ("conv_in", c_void_p), ("conv_stride", c_int), ("conv_bf16", c_int), ("conv_channels", c_int), ("n_taps", c_int), ("conv_off", c_int)]


class SampleArgs(Structure):
    _fields_ = [("logits", c_void_p), ("ld", c_int), ("V", c_int), ("B", c_int), ("slot_of_row", c_void_p),
                ("temperature", c_void_p), ("top_k", c_void_p), ("top_p", c_void_p), ("penalty", c_void_p),
                ("seed", c_void_p), ("sequence_id", c_void_p), ("sample_step", c_void_p),
                ("last_token", c_void_p), ("seen", c_void_p), ("seen_words", c_int), ("out", c_void_p),
                ("part_best", c_void_p), ("part_idx", c_void_p), ("parts", c_int)]


_lib = None


def lib():
    """The loaded extension (built on first use)."""
    global _lib
    if _lib is None:
        l = _build.load()
        l.tb_last_error.restype = ctypes.c_char_p
        l.tb_uniform24.restype = ctypes.c_uint
        l.tb_uniform24.argtypes = [c_longlong, c_longlong, c_longlong]
        l.tb_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        l.tb_fill_random.argtypes = [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p]
        l.tb_scale_f32.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        l.tb_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]
        l.tb_gemm_simt.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_gemm_simt_gated.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_longlong, c_longlong, c_longlong, c_int, c_float, c_void_p]
        l.tb_dyt.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
        l.tb_scale_add.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        l.tb_wkv.argtypes = [POINTER(WkvArgs), c_int, c_int, c_void_p]
        l.tb_hyper.argtypes = [POINTER(HyperArgs), c_int, c_void_p]
        l.tb_polynorm.argtypes = [c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_gate_rows.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_head_norm_gate.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_float, c_void_p]
        l.tb_head_norm_gate_from.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_float, c_float, c_void_p]
        l.tb_delta_prep.argtypes = [POINTER(DeltaPrepArgs), c_int, c_void_p]
        l.tb_recurrent_scan.argtypes = [POINTER(ScanArgs), c_int, c_int, c_void_p]
        l.tb_moe_route_all.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_moe_route_scored.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_group_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_residual_group_norm.argtypes = [c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_qkv_whole_norm.argtypes = [POINTER(WholeNormArgs), c_int, c_void_p]
        l.tb_attn_mixed_prefill.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_mixed_decode.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_set_attn_mixed_tile.argtypes = [c_int]
        l.tb_rotary_rows.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, POINTER(RotaryArgs), c_int, c_float, c_void_p]
        l.tb_gemm_simt_batched.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_longlong, c_longlong, c_longlong, c_void_p]
        l.tb_gemm_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_rmsnorm_add.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        l.tb_round_rows.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p]
        l.tb_gelu_mul_table.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_latent_prep.argtypes = [POINTER(LatentArgs), c_int, c_void_p]
        l.tb_latent_append.argtypes = [c_void_p, c_int, c_int, POINTER(KvView), POINTER(Batch), c_void_p]
        l.tb_lightning_scan.argtypes = [POINTER(LightningArgs), c_int, c_void_p]
        l.tb_gated_rmsnorm.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_moe_route.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_token_gate_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_moe_plan_tiles.argtypes = [c_int, c_int]
        l.tb_moe_plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
        l.tb_moe_gather.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        l.tb_moe_grouped.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_moe_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_float, c_void_p]
        l.tb_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                     c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
        l.tb_qk_norm_rope.argtypes = [POINTER(QkArgs), c_int, c_int, c_void_p]
        l.tb_kv_append.argtypes = [c_void_p, c_int, c_int, POINTER(KvView), POINTER(Batch), c_void_p]
        l.tb_attn_prefill.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_decode.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_sample.argtypes = [POINTER(SampleArgs), c_void_p]
        l.tb_decode_prepare.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_commit_lengths.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_mark_seen.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        _lib = l
    return _lib


_tlib = None


def tlib():
    """The library of tensor-core kernels (tcgen05 / TMA / mma.sync), built and loaded when first asked for."""
    global _tlib
    if _tlib is None:
        lib()
        l = _build.load("tensor")
        l.tb_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_gemm_tc_gated.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
        l.tb_gemm_tc_normed.argtypes = [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        l.tb_gemm_tc_normed_check.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        l.tb_gemm_tc_expert_runs.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                             c_int, c_float, c_void_p]
        l.tb_gemm_tc_check.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
        _tlib = l
    return _tlib


_alib = None

# (own key dims, shared key dims, value dims) of a head that the tensor-core prompt kernel with keys in two parts is built for;
# asked before the attention library is built, so that a model of other sizes never compiles it
ATTN_SPLIT_SIZES = {(128, 64, 128)}


def alib():
    """The library of tensor-core attention kernels (tcgen05 and mma.sync), built and loaded when first asked for."""
    global _alib
    if _alib is None:
        tlib()
        l = _build.load("attention")
        l.tb_attn_decode_mma.argtypes = [POINTER(AttnArgs), c_void_p]
        l.tb_attn_decode_mma_check.argtypes = [POINTER(AttnArgs), c_int]
        l.tb_attn_prefill_mma.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_prefill_mma_check.argtypes = [POINTER(AttnArgs), c_int, c_int]
        l.tb_attn_prefill_split.argtypes = [POINTER(SplitAttnArgs), c_void_p]
        l.tb_attn_prefill_split_check.argtypes = [POINTER(SplitAttnArgs)]
        l.tb_attn_prefill_tc.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_prefill_tc_check.argtypes = [POINTER(AttnArgs), c_int, c_int]
        _alib = l
    return _alib


def _check(rc: int) -> None:
    global launch_count
    launch_count += 1
    if _launch_log is not None:
        name = sys._getframe(1).f_code.co_name
        _launch_log[name] = _launch_log.get(name, 0) + 1
    if rc:
        raise KernelError(lib().tb_last_error().decode())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dt}")


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


# --------------------------------------------------------------------------- #
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, stream: int) -> None:
    _need_cuda(table, tokens, out)
    _check(lib().tb_embed(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                          tokens.numel(), table.shape[1], table.shape[0], stream))


def fill_random(out: torch.Tensor, key: int, std: float, mean: float) -> None:
    """out[i] = normal(key, i) * std + mean (float32 or bfloat16), or 15-bit integers (int32): the counter-based
    generator of titan_b200.weights.random_init, on the device."""
    _need_cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_random: a contiguous tensor is wanted")
    code = -1 if out.dtype == torch.int32 else dtype_code(out.dtype)
    _check(lib().tb_fill_random(out.data_ptr(), code, out.numel(), key & ((1 << 64) - 1), std, mean, current_stream()))


def scale_f32(x: torch.Tensor, factor: float, stream: int) -> None:
    """x *= factor in place (float32, contiguous)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_f32: a contiguous float32 tensor is wanted")
    _check(lib().tb_scale_f32(x.data_ptr(), x.numel(), factor, stream))


def rmsnorm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, eps: float, stream: int,
            rows: Optional[torch.Tensor] = None) -> None:
    _need_cuda(x, w, y, rows)
    n = y.shape[0]
    _check(lib().tb_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), dtype_code(y.dtype), _ptr(rows), n,
                            x.shape[-1], eps, stream))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int, gate: int = ACT_SILU, limit: float = 0.0) -> None:
    """out (epilogue ``epi``) = x[M,K] . w[N,K]^T; x and out may be row-strided views.  ``gate``, ``limit``: what the
    SWIGLU epilogue makes of a pair (ACT_*)."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(lib().tb_gemm_simt_gated(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(w.dtype), M, N, K,
                                    x.stride(0), out.stride(0), epi, 1, 0, 0, 0, int(gate), float(limit), stream))


def gemm_simt_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int, batch: int,
                      x_step: int, out_step: int) -> None:
    """``batch`` products of one shape in one launch: out_z (epilogue ``epi``) = x_z[M,K] . w[z][N,K]^T, where x_z and
    out_z are the views ``x`` and ``out`` moved right by z * x_step and z * out_step columns (the heads of a mixer, side
    by side in the rows of one buffer) and ``w`` is [batch, N, K]."""
    _need_cuda(x, w, out)
    M, K = x.shape
    if w.dim() != 3 or w.shape[0] != batch or w.shape[2] != K or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_batched: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    N = w.shape[1]
    _check(lib().tb_gemm_simt_batched(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(w.dtype), M, N, K, x.stride(0),
                                      out.stride(0), epi, batch, x_step, N * K, out_step, stream))


def gemm_rows(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int) -> None:
    """out (epilogue store, float32 or add) = x[M,K] . w[N,K]^T, a warp per output element: for the few rows of a decode step and
    matrices too small to pay for a tensor-core launch."""
    _need_cuda(x, w, out)
    M, K = x.shape
    if w.shape[1] != K or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1 or x.dtype != w.dtype:
        raise KernelError(f"gemm_rows: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    want = w.dtype if epi == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_rows: this epilogue writes {want}, the output is {out.dtype}")
    _check(lib().tb_gemm_rows(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(w.dtype), M, w.shape[0], K, x.stride(0), out.stride(0), epi, stream))


def rmsnorm_add(y: torch.Tensor, w: torch.Tensor, x: torch.Tensor, eps: float, stream: int,
                lowp: Optional[torch.Tensor] = None, zero_y: bool = True) -> None:
    """x += y / sqrt(mean(y^2) + eps) * w (float32 rows): a norm on a sublayer's output, added to the residual stream.
    ``zero_y`` leaves y zeroed for the next sublayer's products to add into; ``lowp`` receives the new rows of x rounded
    to its dtype (what the next sublayer's first product reads)."""
    _need_cuda(y, w, x, lowp)
    if y.dtype != torch.float32 or x.dtype != torch.float32 or w.dtype != torch.float32 or y.shape != x.shape \
            or not (y.is_contiguous() and x.is_contiguous()) or (lowp is not None and (lowp.shape != x.shape or not lowp.is_contiguous())):
        raise KernelError("rmsnorm_add: contiguous float32 rows of one shape are wanted")
    _check(lib().tb_rmsnorm_add(y.data_ptr(), w.data_ptr(), x.data_ptr(), _ptr(lowp), dtype_code(lowp.dtype) if lowp is not None else F32,
                                x.shape[0], x.shape[1], eps, int(zero_y), stream))


def dyt(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor, y: torch.Tensor, stream: int,
        rows: Optional[torch.Tensor] = None) -> None:
    """y[r] = tanh(alpha * x[rows[r] or r]) * w + b: a norm that takes no statistics (x float32 rows, alpha one number on
    the device, y in its own dtype)."""
    _need_cuda(x, w, b, alpha, y, rows)
    if x.dtype != torch.float32 or not (x.is_contiguous() and y.is_contiguous()) or any(t.dtype != torch.float32 for t in (w, b, alpha)):
        raise KernelError("dyt: contiguous float32 rows in, float32 weight, bias and factor")
    _check(lib().tb_dyt(x.data_ptr(), w.data_ptr(), b.data_ptr(), alpha.data_ptr(), y.data_ptr(), dtype_code(y.dtype), _ptr(rows), y.shape[0],
                        x.shape[-1], stream))


def scale_add(y: torch.Tensor, scale: Optional[torch.Tensor], x: torch.Tensor, stream: int, zero_y: bool = True, norm=None,
              h: Optional[torch.Tensor] = None) -> None:
    """x += y * scale (float32 rows; ``scale`` a vector or None for 1); ``zero_y`` leaves y zeroed for the next sublayer's
    products to add into; ``norm`` = (w, b, alpha) with ``h``: h = tanh(alpha x) w + b of the NEW rows, in h's dtype."""
    _need_cuda(y, scale, x, h)
    if y.dtype != torch.float32 or x.dtype != torch.float32 or y.shape != x.shape or not (y.is_contiguous() and x.is_contiguous()) \
            or (h is not None and (h.shape != x.shape or not h.is_contiguous() or norm is None)):
        raise KernelError("scale_add: contiguous float32 rows of one shape are wanted")
    w, b, alpha = norm if h is not None else (None, None, None)
    _check(lib().tb_scale_add(y.data_ptr(), _ptr(scale), x.data_ptr(), int(zero_y), _ptr(w), _ptr(b), _ptr(alpha), _ptr(h),
                              dtype_code(h.dtype) if h is not None else F32, x.shape[0], x.shape[1], stream))


def hyper(xs: torch.Tensor, streams: int, stream: int, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
          out_w: Optional[torch.Tensor] = None, zero_y: bool = True, in_w: Optional[torch.Tensor] = None,
          norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, h: Optional[torch.Tensor] = None) -> None:
    """Between two sublayers of a model with ``streams`` residual streams, xs float32 [T, streams * W].  With ``y`` (float32 [T, W],
    the sublayer's result): every stream r becomes sum_s mix[s, r] x_s + out_w[r] * y (``zero_y`` leaves y zeroed).  With ``in_w``:
    h = the blend sum_r in_w[r] x_r of the new streams, RMS-normed with ``norm_w`` and ``eps`` into h's dtype, or, without a norm,
    as it is in float32."""
    _need_cuda(xs, y, mix, out_w, in_w, norm_w, h)
    W = xs.shape[1] // streams
    if xs.dtype != torch.float32 or not xs.is_contiguous() or xs.shape[1] != streams * W or (y is not None and (y.dtype != torch.float32 or not y.is_contiguous() or y.shape != (xs.shape[0], W))) \
            or (h is not None and (not h.is_contiguous() or h.shape != (xs.shape[0], W))) or any(t is not None and t.dtype != torch.float32 for t in (mix, out_w, in_w, norm_w)):
        raise KernelError("hyper: contiguous float32 rows of streams, a float32 result and float32 weights are wanted")
    a = HyperArgs(xs.data_ptr(), streams, W, xs.shape[0], _ptr(y), _ptr(mix), _ptr(out_w), int(zero_y), _ptr(in_w), _ptr(norm_w), eps, _ptr(h))
    _check(lib().tb_hyper(byref(a), dtype_code(h.dtype) if h is not None else F32, stream))


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, y: torch.Tensor, stream: int) -> None:
    """y = a N(z) + b N(z^2) + c N(z^3) + e row by row, N(x) = x / sqrt(mean(x^2) + eps), coef = (a, b, c, e) float32 on the device."""
    _need_cuda(z, coef, y)
    if z.dtype != y.dtype or z.shape != y.shape or z.stride(1) != 1 or y.stride(1) != 1 or coef.dtype != torch.float32 or coef.numel() != 4:
        raise KernelError("polynorm: rows of one dtype and shape and four float32 coefficients are wanted")
    _check(lib().tb_polynorm(z.data_ptr(), z.stride(0), coef.data_ptr(), eps, y.data_ptr(), y.stride(0), dtype_code(z.dtype), z.shape[0], z.shape[1], stream))


GATE_SIGMOID, GATE_SILU = 0, 1


def gate_rows(x: torch.Tensor, g: torch.Tensor, y: torch.Tensor, act: int, scale: float, stream: int) -> None:
    """y = x * act(g) * scale, element by element (act GATE_SIGMOID or GATE_SILU, in float32); row-strided views of one dtype; y may be x."""
    _need_cuda(x, g, y)
    if len({x.dtype, g.dtype, y.dtype}) != 1 or x.shape != g.shape or x.shape != y.shape or x.stride(1) != 1 or g.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gate_rows: three views of one dtype and shape are wanted")
    _check(lib().tb_gate_rows(x.data_ptr(), x.stride(0), g.data_ptr(), g.stride(0), y.data_ptr(), y.stride(0), dtype_code(x.dtype), x.shape[0], x.shape[1],
                              int(act), float(scale), stream))


def head_norm_gate(o: torch.Tensor, w: torch.Tensor, per_head: bool, g: torch.Tensor, y: torch.Tensor, heads: int, act: int, scale: float,
                   eps: float, stream: int) -> None:
    """Per head of dv = width / heads elements: y = o / sqrt(mean(o^2) + eps) * w * act(g) * scale.  o float32 [T, heads * dv]; w float32, one
    row of dv for every head or (``per_head``) heads * dv; y in the compute dtype, g in it or in float32 (row-strided views allowed)."""
    _need_cuda(o, w, g, y)
    dv = o.shape[1] // heads
    if o.dtype != torch.float32 or w.dtype != torch.float32 or g.dtype not in (y.dtype, torch.float32) or o.stride(1) != 1 or g.stride(1) != 1 or y.stride(1) != 1 \
            or o.shape[1] != heads * dv or w.numel() != (heads * dv if per_head else dv) or g.shape != o.shape or y.shape != o.shape:
        raise KernelError("head_norm_gate: float32 rows of whole heads, a gate and an output of one dtype")
    _check(lib().tb_head_norm_gate_from(o.data_ptr(), o.stride(0), w.data_ptr(), dv if per_head else 0, g.data_ptr(), g.stride(0), dtype_code(g.dtype),
                                        y.data_ptr(), y.stride(0), dtype_code(y.dtype), o.shape[0], heads, dv, int(act), float(scale), float(eps), stream))


def delta_prep(args: "DeltaPrepArgs", dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_delta_prep(byref(args), dtype_code(dtype), stream))


SCAN_DELTA, SCAN_MLSTM = 0, 1


def recurrent_scan(args: "ScanArgs", mode: int, dtype: torch.dtype, stream: int) -> None:
    """The gated delta rule (SCAN_DELTA, float32 inputs) or the mLSTM memory (SCAN_MLSTM, inputs in ``dtype``) over a step's tokens."""
    _check(lib().tb_recurrent_scan(byref(args), int(mode), dtype_code(dtype), stream))


WKV_SHIFT, WKV_DECAY, WKV_SCAN, WKV_OUT = 0, 1, 2, 3


def wkv(args: "WkvArgs", stage: int, dtype: torch.dtype, stream: int) -> None:
    """One of the wkv mixer's four kernels (WKV_SHIFT, WKV_DECAY, WKV_SCAN, WKV_OUT) on the argument block."""
    _check(lib().tb_wkv(byref(args), int(stage), dtype_code(dtype), stream))


def moe_route_all(z: torch.Tensor, top: int, correction: Optional[torch.Tensor], groups: int, keep: int, ids: torch.Tensor,
                  wts: torch.Tensor, stream: int) -> None:
    """Per row of z (float32 [T, n_all]): scores = softmax over the whole row; the ``top`` experts with the largest
    score + correction inside the ``keep`` best of ``groups`` groups of neighbours; weights = their scores over their sum."""
    _need_cuda(z, correction, ids, wts)
    _check(lib().tb_moe_route_all(z.data_ptr(), z.stride(0), z.shape[1], top, _ptr(correction), groups, keep, ids.data_ptr(), wts.data_ptr(),
                                  z.shape[0], stream))


def moe_route_scored(z: torch.Tensor, top: int, correction: Optional[torch.Tensor], groups: int, keep: int, ids: torch.Tensor,
                     wts: torch.Tensor, stream: int, sigmoid: bool, group_best: int, renorm: bool) -> None:
    """``moe_route_all`` with its three fixed choices as arguments: scores by a sigmoid an output instead of a softmax over the
    row; a group's score as the sum of its ``group_best`` largest choice scores; weights left as the chosen scores."""
    _need_cuda(z, correction, ids, wts)
    _check(lib().tb_moe_route_scored(z.data_ptr(), z.stride(0), z.shape[1], top, _ptr(correction), groups, keep, ids.data_ptr(), wts.data_ptr(),
                                     z.shape[0], int(sigmoid), int(group_best), int(renorm), stream))


def group_rmsnorm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, groups: int, eps: float, stream: int,
                  rows: Optional[torch.Tensor] = None) -> None:
    """RMS norm of float32 rows in ``groups`` equal runs, each with its own mean square, one weight over the row."""
    _need_cuda(x, w, y, rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous():
        raise KernelError("group_rmsnorm: contiguous float32 rows are wanted")
    _check(lib().tb_group_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), dtype_code(y.dtype), _ptr(rows), y.shape[0], x.shape[-1],
                                  groups, eps, stream))


def residual_group_norm(y: torch.Tensor, mult: float, x: torch.Tensor, stream: int, norm_w: Optional[torch.Tensor] = None, groups: int = 1,
                        eps: float = 0.0, h: Optional[torch.Tensor] = None) -> None:
    """x += mult * y (float32 rows), y left zeroed; with ``h``: h = the grouped RMS norm of the NEW rows times norm_w, in h's dtype."""
    _need_cuda(y, x, norm_w, h)
    if y.dtype != torch.float32 or x.dtype != torch.float32 or y.shape != x.shape or not (y.is_contiguous() and x.is_contiguous()) \
            or (h is not None and (h.shape != x.shape or not h.is_contiguous() or norm_w is None)):
        raise KernelError("residual_group_norm: contiguous float32 rows of one shape are wanted")
    _check(lib().tb_residual_group_norm(y.data_ptr(), float(mult), x.data_ptr(), _ptr(norm_w), _ptr(h),
                                        dtype_code(h.dtype) if h is not None else F32, x.shape[0], x.shape[1], groups, eps, stream))


def qkv_whole_norm(args: "WholeNormArgs", out_dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_qkv_whole_norm(byref(args), dtype_code(out_dtype), stream))


def attn_mixed_prefill(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_mixed_prefill(byref(args), dtype_code(dtype), stream))


def set_attn_mixed_tile(on: bool) -> None:
    """Prompt attention with blended heads: the kernel that stages a round's keys and values in shared memory for two queries
    and all heads (default), or (off) the one-query kernel that every size falls back to; the tests compare the two."""
    lib().tb_set_attn_mixed_tile(int(on))


def attn_mixed_decode(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_mixed_decode(byref(args), dtype_code(dtype), stream))


def rotary_rows(x: torch.Tensor, pos_of: torch.Tensor, heads: int, hd: int, rope: RotaryArgs, scale_from: int, scale: float, stream: int) -> None:
    """Rotates ``heads`` heads of ``hd`` elements that lie side by side from column 0 of the float32 rows ``x``, in place, by the
    rows' positions; heads from ``scale_from`` on are multiplied by ``scale`` afterwards."""
    _need_cuda(x, pos_of)
    if x.dtype != torch.float32 or x.stride(-1) != 1:
        raise KernelError("rotary_rows: float32 rows are wanted")
    _check(lib().tb_rotary_rows(x.data_ptr(), x.stride(0), pos_of.data_ptr(), x.shape[0], heads, hd, byref(rope), scale_from, scale, stream))


def round_rows(x: torch.Tensor, out: torch.Tensor, stream: int) -> None:
    """out = x rounded to bfloat16 (x float32, both contiguous and of one shape)."""
    _need_cuda(x, out)
    if x.dtype != torch.float32 or out.dtype != torch.bfloat16 or x.shape != out.shape or not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("round_rows: float32 in, bfloat16 out, one shape, contiguous")
    _check(lib().tb_round_rows(x.data_ptr(), out.data_ptr(), x.numel(), stream))


def gelu_mul_table(z: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, offset: int, g: torch.Tensor, stream: int) -> None:
    """g[t] = gelu_tanh(z[t]) * table[tokens[t], offset : offset + D]  (z, g [T, D] and the table in one dtype)."""
    _need_cuda(z, table, tokens, g)
    if not (z.is_contiguous() and g.is_contiguous() and table.is_contiguous()) or z.dtype != table.dtype or g.dtype != z.dtype:
        raise KernelError("gelu_mul_table: contiguous tensors of one dtype are wanted")
    _check(lib().tb_gelu_mul_table(z.data_ptr(), table.data_ptr(), tokens.data_ptr(), g.data_ptr(), dtype_code(z.dtype), z.shape[0],
                                   z.shape[1], table.shape[1], int(offset), table.shape[0], stream))


def latent_prep(args: "LatentArgs", out_dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_latent_prep(byref(args), dtype_code(out_dtype), stream))


def latent_append(rows: torch.Tensor, cache: KvView, batch: Batch, stream: int) -> None:
    _check(lib().tb_latent_append(rows.data_ptr(), rows.stride(0), dtype_code(rows.dtype), byref(cache), byref(batch), stream))


def lightning_scan(args: "LightningArgs", dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_lightning_scan(byref(args), dtype_code(dtype), stream))


def gated_rmsnorm(o: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, y: torch.Tensor, eps: float, stream: int) -> None:
    """y = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate), row by row; o float32, gate and y in the compute dtype (row-strided views allowed)."""
    _need_cuda(o, w, gate, y)
    if o.dtype != torch.float32 or gate.dtype != y.dtype or o.stride(1) != 1 or gate.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gated_rmsnorm: float32 rows in, gate and output of one dtype")
    _check(lib().tb_gated_rmsnorm(o.data_ptr(), o.stride(0), w.data_ptr(), gate.data_ptr(), gate.stride(0), y.data_ptr(), y.stride(0),
                                  dtype_code(y.dtype), o.shape[0], o.shape[1], eps, stream))


def moe_route(z: torch.Tensor, experts: int, top: int, has_gate: bool, ids: torch.Tensor, wts: torch.Tensor,
              gate: Optional[torch.Tensor], stream: int) -> None:
    """Per row of z (float32 [T, experts (+1)]): the ``top`` largest logits' indices and their softmax weights; the last
    column's sigmoid into ``gate`` if the row has one more column than experts."""
    _need_cuda(z, ids, wts, gate)
    _check(lib().tb_moe_route(z.data_ptr(), z.stride(0), experts, top, int(has_gate), ids.data_ptr(), wts.data_ptr(), _ptr(gate),
                              z.shape[0], stream))


def token_gate_rows(x: torch.Tensor, w: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, offset: int, g: torch.Tensor, stream: int) -> None:
    """g[t] = gelu_tanh(x[t] . w^T) * table[tokens[t], offset : offset + D] in one kernel, for a few rows (one dtype throughout)."""
    _need_cuda(x, w, table, tokens, g)
    if not (w.is_contiguous() and g.is_contiguous() and table.is_contiguous()) or x.stride(1) != 1 or len({x.dtype, w.dtype, table.dtype, g.dtype}) != 1:
        raise KernelError("token_gate_rows: contiguous tensors of one dtype are wanted")
    _check(lib().tb_token_gate_rows(x.data_ptr(), x.stride(0), w.data_ptr(), table.data_ptr(), tokens.data_ptr(), g.data_ptr(), dtype_code(w.dtype),
                                    x.shape[0], x.shape[1], w.shape[0], table.shape[1], int(offset), table.shape[0], stream))


def moe_plan_tiles(pairs: int, experts: int) -> int:
    return int(lib().tb_moe_plan_tiles(pairs, experts))


class MoePlan:
    """The (token, choice) pairs grouped by expert, as views of one int32 buffer: ``perm`` sorted row -> pair, ``inverse``
    pair -> sorted row, ``offsets`` [E + 1] first sorted row of every expert, and the row tiles of the grouped product."""

    def __init__(self, buffer: torch.Tensor, pairs: int, experts: int):
        P, tiles = pairs, moe_plan_tiles(pairs, experts)
        if buffer.numel() < self.size(pairs, experts) or buffer.dtype != torch.int32:
            raise KernelError("moe_plan: the plan's buffer is too small")
        at = 0
        def cut(n):
            nonlocal at
            at += n
            return buffer[at - n: at]
        self.rank, self.perm, self.inverse = cut(P), cut(P), cut(P)
        self.tile_e, self.tile_row0, self.tile_rows = cut(tiles), cut(tiles), cut(tiles)
        self.n_tiles, self.offsets = cut(1), cut(experts + 1)
        self.tiles, self.pairs, self.experts = tiles, P, experts

    @staticmethod
    def size(pairs: int, experts: int) -> int:
        return 3 * pairs + 3 * moe_plan_tiles(pairs, experts) + 1 + experts + 1


def moe_plan(ids: torch.Tensor, experts: int, buffer: torch.Tensor, stream: int) -> MoePlan:
    """Groups the (token, choice) pairs by expert into ``buffer`` (int32 scratch of MoePlan.size elements)."""
    plan = MoePlan(buffer, ids.numel(), experts)
    _check(lib().tb_moe_plan(ids.data_ptr(), plan.pairs, experts, plan.rank.data_ptr(), plan.perm.data_ptr(), plan.tile_e.data_ptr(),
                             plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr(), plan.n_tiles.data_ptr(), plan.tiles,
                             plan.offsets.data_ptr(), plan.inverse.data_ptr(), stream))
    return plan


def moe_gather(x: torch.Tensor, plan: MoePlan, top: int, out: torch.Tensor, stream: int) -> None:
    """out[r] = x[plan.perm[r] // top]: the tokens' rows in the plan's order (out [P, K] contiguous, x's dtype)."""
    _need_cuda(x, out)
    if out.dtype != x.dtype or not out.is_contiguous() or x.stride(1) != 1 or out.shape != (plan.pairs, x.shape[1]):
        raise KernelError("moe_gather: a contiguous [pairs, K] output of the input's dtype is wanted")
    _check(lib().tb_moe_gather(x.data_ptr(), x.stride(0), plan.perm.data_ptr(), top, out.data_ptr(), dtype_code(x.dtype), plan.pairs, x.shape[1], stream))


def moe_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, plan, top: int, stream: int,
                gate: int = ACT_SILU, limit: float = 0.0) -> None:
    """The experts' products over the plan's tiles on the CUDA cores.  mode 0: x [T, K] tokens, w [E, 2F, K] (gate and up
    rows interleaved), out [P, F] in sorted order; mode 1: x [P, K] sorted rows, w [E, N, K], out float32 [P, N] in pair order."""
    _need_cuda(x, w, out)
    _check(lib().tb_moe_grouped(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), dtype_code(w.dtype), mode,
                                plan.perm.data_ptr(), plan.tile_e.data_ptr(), plan.tile_row0.data_ptr(), plan.tile_rows.data_ptr(),
                                plan.n_tiles.data_ptr(), plan.tiles, w.shape[1], w.shape[2], top, w.shape[0], int(gate), float(limit), stream))


def moe_rows(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, ids: torch.Tensor, top: int, stream: int,
             gate: int = ACT_SILU, limit: float = 0.0) -> None:
    """The same two products for a few pairs, a warp per output, without a plan (pair order in and out)."""
    _need_cuda(x, w, out, ids)
    n_out = w.shape[1] // 2 if mode == 0 else w.shape[1]
    _check(lib().tb_moe_rows(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), dtype_code(w.dtype), mode,
                             ids.data_ptr(), ids.numel(), n_out, w.shape[2], top, w.shape[0], int(gate), float(limit), stream))


def moe_combine(y: torch.Tensor, wts: torch.Tensor, shared_y: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                out: torch.Tensor, top: int, stream: int, where: Optional[torch.Tensor] = None,
                ids: Optional[torch.Tensor] = None, n_real: int = 0, x: Optional[torch.Tensor] = None) -> None:
    """out[t] += sum_k wts[t, k] * y[row of pair t * top + k] (+ gate[t] * shared_y[t]); everything float32.  The row of
    pair p is p, or ``where[p]`` if y is in another order (a plan's ``inverse``).  With ``ids``, ``n_real`` and ``x``: a
    pair whose expert is ``n_real`` or beyond has no matrices; its output is the token's own input row x[t]."""
    _need_cuda(y, wts, shared_y, gate, out, where, ids, x)
    _check(lib().tb_moe_combine(y.data_ptr(), wts.data_ptr(), _ptr(shared_y), _ptr(gate), out.data_ptr(), out.shape[0], out.shape[1], top,
                                _ptr(where), _ptr(ids), int(n_real), _ptr(x), x.stride(0) if x is not None else 0,
                                dtype_code(x.dtype) if x is not None else F32, stream))


def gemm_tc_accepts(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int) -> bool:
    """Whether the tensor-core kernel's alignment rules hold for this product."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    return tlib().tb_gemm_tc_check(x.shape[0], w.shape[0], x.shape[1], x.stride(0), out.stride(0), epi,
                                  x.data_ptr(), w.data_ptr(), out.data_ptr()) == 0


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int, splits: int = 0, ordered: bool = False,
            gate: int = ACT_SILU, limit: float = 0.0) -> None:
    """out (epilogue ``epi``) = x[M,K] . w[N,K]^T on the tcgen05 tensor cores (bfloat16 operands).  ``ordered``: partial
    sums along K add up in a fixed order (the K slices of a decode product inside a thread-block cluster, no prompt tile
    cut along K), so that the same inputs give the same bits on every run; the default lets float32 reductions meet at
    L2 in the order they arrive, which is faster and differs from run to run in the last bits."""
    _need_cuda(x, w, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    want = torch.bfloat16 if epi in (EPI_STORE, EPI_SWIGLU) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: this epilogue writes {want}, the output is {out.dtype}")
    M, K_ = x.shape
    N = w.shape[0]
    if w.shape[1] != K_ or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(tlib().tb_gemm_tc_gated(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K_, x.stride(0), out.stride(0), epi,
                                  -1 if ordered and not splits else splits, int(gate), float(limit), stream))


def gemm_tc_expert_runs(x: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, w_down: torch.Tensor, y: torch.Tensor, first, stream: int,
                        gate: int = ACT_SILU, limit: float = 0.0) -> None:
    """For every run s of rows [first[s], first[s + 1]): act = swiglu(x . w_gate_up[s]^T), y = act . w_down[s]^T (float32), on the
    tensor cores, the runs spread over a few side streams (w_gate_up [E, 2F, H] with gate and up rows interleaved, w_down [E, H, F])."""
    global launch_count
    _need_cuda(x, w_gate_up, act, w_down, y)
    E, F2, H = w_gate_up.shape
    if (x.dtype != torch.bfloat16 or act.dtype != torch.bfloat16 or y.dtype != torch.float32 or w_down.shape != (E, H, F2 // 2)
            or not (w_gate_up.is_contiguous() and w_down.is_contiguous()) or len(first) != E + 1 or first[-1] > x.shape[0]
            or x.stride(1) != 1 or act.stride(1) != 1 or y.stride(1) != 1 or act.shape[1] != F2 // 2):
        raise KernelError("gemm_tc_expert_runs: shapes or dtypes do not fit")
    arr = (c_int * len(first))(*first)
    launch_count += 2 * sum(1 for a, b in zip(first, first[1:]) if b > a) - 1
    _check(tlib().tb_gemm_tc_expert_runs(x.data_ptr(), x.stride(0), w_gate_up.data_ptr(), act.data_ptr(), act.stride(0), w_down.data_ptr(),
                                        y.data_ptr(), y.stride(0), arr, E, H, F2 // 2, int(gate), float(limit), stream))


def gemm_tc_normed_accepts(x: torch.Tensor, norm_w: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int,
                           sumsq: Optional[torch.Tensor]) -> bool:
    """Can the product run with the RMS norm of its input folded in (tb_gemm_tc_normed)?"""
    if x.dtype != torch.float32 or norm_w.dtype != torch.float32 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != w.shape[1] or norm_w.numel() != x.shape[1]:
        return False
    return tlib().tb_gemm_tc_normed_check(x.shape[0], w.shape[0], x.shape[1], x.stride(0), out.stride(0), epi, x.data_ptr(),
                                         norm_w.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(sumsq)) == 0


def gemm_tc_normed(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int,
                   sumsq: Optional[torch.Tensor] = None, ordered: bool = False) -> None:
    """out (epilogue ``epi``) = rmsnorm(x; norm_w, eps) . w^T for the rows of a decode step, the norm folded into the
    product: x is the float32 residual stream.  EPI_SWIGLU: complete.  EPI_ADD: ``out`` (float32) receives the products
    of the rows times the norm's weight WITHOUT the rows' scales, and ``sumsq`` [slices, 32] (float32; ``gemm_tc_normed_slices``
    rows of it are written) the rows' sums of squares per K slice; the consumer multiplies row m by
    1/sqrt(sum_z sumsq[z, m] / K + eps).  ``ordered``: as for ``gemm_tc``."""
    _need_cuda(x, norm_w, w, out, sumsq)
    want = torch.bfloat16 if epi == EPI_SWIGLU else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc_normed: this epilogue writes {want}, the output is {out.dtype}")
    _check(tlib().tb_gemm_tc_normed(x.data_ptr(), x.stride(0), norm_w.data_ptr(), eps, w.data_ptr(), out.data_ptr(), x.shape[0],
                                   w.shape[0], x.shape[1], out.stride(0), epi, _ptr(sumsq), int(bool(ordered)), stream))


def gemm_tc_normed_slices(w: torch.Tensor, epi: int, rows: int = 1, ordered: bool = False) -> int:
    """K slices that gemm_tc_normed cuts this product into (one row of partial sums of squares each) for a step of
    ``rows`` rows; ``ordered``: as it cuts when the slices add up in a fixed order (a cluster per tile: fewer fit)."""
    return int(tlib().tb_gemm_tc_normed_slices(w.shape[0], w.shape[1], epi, int(rows), int(bool(ordered))))


def gemm_tc_error() -> int:
    """Error word of the tensor-core kernels (0: none); synchronises the device and clears the word."""
    return int(tlib().tb_gemm_tc_error())


def qk_norm_rope(args: QkArgs, in_dtype: torch.dtype, out_dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_qk_norm_rope(byref(args), dtype_code(in_dtype), dtype_code(out_dtype), stream))


def kv_append(kv: torch.Tensor, cache: KvView, batch: Batch, stream: int) -> None:
    _check(lib().tb_kv_append(kv.data_ptr(), kv.stride(0), dtype_code(kv.dtype), byref(cache), byref(batch), stream))


def attn_prefill(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_prefill(byref(args), dtype_code(dtype), stream))


def attn_decode(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_decode(byref(args), dtype_code(dtype), stream))


def attn_decode_mma_accepts(args: AttnArgs, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and alib().tb_attn_decode_mma_check(byref(args), BF16) == 0


def attn_decode_mma(args: AttnArgs, stream: int) -> None:
    """Decode attention on tensor cores (bfloat16, head_dim 64 or 128), then the merge of the splits."""
    _check(alib().tb_attn_decode_mma(byref(args), stream))


def set_attn_decode_cluster(on: bool) -> None:
    """Decode attention with up to 16 splits: merge them inside a thread-block cluster (on by default) or through
    scratch memory and the merge kernel."""
    alib().tb_attn_decode_set_cluster(int(bool(on)))


def set_attn_decode_late_trigger(on: bool) -> None:
    """Decode attention lets the kernel after it start once its own pages have been requested and read (on by
    default), or at once: the next kernel's first weight requests then queue in front of the pages."""
    alib().tb_attn_decode_set_late_trigger(int(bool(on)))


# Where the tensor-core prompt kernels take keys and values from: nowhere they can (0), the step's own rows (every
# sequence starts at position 0), or the cache's pages (the step's keys are appended already; no ring).
KV_NOWHERE, KV_FROM_STEP, KV_FROM_CACHE = 0, 1, 2


def attn_prefill_mma_accepts(args: AttnArgs, dtype: torch.dtype, source: int) -> bool:
    return dtype == torch.bfloat16 and alib().tb_attn_prefill_mma_check(byref(args), BF16, int(source)) == 0


def attn_prefill_mma(args: AttnArgs, source: int, stream: int) -> None:
    """Causal attention of prompts and continuation chunks on tensor cores (bfloat16, head_dim 64 or 128)."""
    _check(alib().tb_attn_prefill_mma(byref(args), int(source), stream))


def attn_prefill_split_accepts(args: "SplitAttnArgs") -> bool:
    return alib().tb_attn_prefill_split_check(byref(args)) == 0


def attn_prefill_split(args: "SplitAttnArgs", stream: int) -> None:
    """Causal (windowed) attention of prompts that start at position 0 on tensor cores, a key being [a part of its own head |
    a part all heads share] and values of their own width (bfloat16; keys of 128 + 64, values of 128)."""
    _check(alib().tb_attn_prefill_split(byref(args), stream))


def attn_prefill_tc_accepts(args: AttnArgs, dtype: torch.dtype, source: int) -> bool:
    return dtype == torch.bfloat16 and alib().tb_attn_prefill_tc_check(byref(args), BF16, int(source)) == 0


def attn_prefill_tc(args: AttnArgs, source: int, stream: int) -> None:
    """Causal attention of prompts and continuation chunks on the tcgen05 tensor cores (bfloat16, head_dim 128)."""
    _check(alib().tb_attn_prefill_tc(byref(args), int(source), stream))


def attn_tc_error() -> int:
    return int(alib().tb_attn_tc_error())


def attn_mma_error() -> int:
    return int(alib().tb_attn_mma_error())


def sample(args: SampleArgs, stream: int) -> None:
    _check(lib().tb_sample(byref(args), stream))


def set_sample_team(ctas: int) -> None:
    """CTAs (a thread-block cluster) that share a row that is not greedy: 0 = by the size of the vocabulary
    (8 from 65,536 tokens, 4 from 16,384, else 1), or 1, 2, 4, 8."""
    lib().tb_sample_set_team(int(ctas))


def mark_seen(tokens, seq_of, slot_of_seq, seen: torch.Tensor, T: int, stream: int) -> None:
    _check(lib().tb_mark_seen(tokens.data_ptr(), seq_of.data_ptr(), slot_of_seq.data_ptr(), seen.data_ptr(),
                              seen.shape[1], T, stream))


def decode_prepare(slot_of_seq, seq_len, last_token, feed_last: bool, tokens, pos_of, start_pos, kv_len, stream: int) -> None:
    _check(lib().tb_decode_prepare(slot_of_seq.data_ptr(), seq_len.data_ptr(), last_token.data_ptr(), int(feed_last),
                                   tokens.data_ptr(), pos_of.data_ptr(), start_pos.data_ptr(), kv_len.data_ptr(),
                                   slot_of_seq.numel(), stream))


def commit_lengths(slot_of_seq, kv_len, seq_len, stream: int) -> None:
    _check(lib().tb_commit_lengths(slot_of_seq.data_ptr(), kv_len.data_ptr(), seq_len.data_ptr(), slot_of_seq.numel(), stream))


def wait_errors() -> dict:
    """The error words of the kernels whose waits are bounded (a wait that gave up leaves a code there and the
    step's result is invalid).  Reads and clears them; synchronises the device.  Empty if all is well, and
    if the tensor-core library was never loaded."""
    if _tlib is None:
        return {}
    found = {"gemm_tc": gemm_tc_error()}
    if _alib is not None:
        found.update({"attn_prefill_tc": attn_tc_error(), "attn_mma": attn_mma_error()})
    return {k: v for k, v in found.items() if v}


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel launched afterwards (on by default)."""
    lib().tb_set_pdl(int(bool(on)))


def set_gemm_tail_split(on: bool) -> None:
    """Prompt products with the ADD epilogue: cut the tiles of a last, partly filled round along K (on by default) or keep them whole."""
    tlib().tb_gemm_tc_set_tail_split(int(bool(on)))


def set_gemm_pair(on: bool) -> None:
    """Prompt products on pairs of CTAs that share one MMA (on by default) or on single CTAs."""
    tlib().tb_gemm_tc_set_pair(int(bool(on)))


def set_gemm_swap_below(m: int) -> None:
    """Products with fewer rows than this run in swap mode (weights on the 128-row side): 128 by default, at most 129."""
    tlib().tb_gemm_tc_set_swap_below(int(m))


def set_gemm_plain_tile(which: int) -> None:
    """Prompt products: 0 lets the launcher choose the tile shape (default), 1 forces CTA pairs with 256 x 256 tiles
    (from 256 x 256 outputs on), 2 single CTAs with 128 x 256 tiles, 3 single CTAs with 128 x 128 tiles."""
    tlib().tb_gemm_tc_set_plain_tile(int(which))


def gemm_pair_clusters(epi: int) -> int:
    """CTA pairs the device holds at once for the pair kernel of this epilogue (0: it cannot run)."""
    return int(tlib().tb_gemm_tc_pair_clusters(int(epi)))


def uniform24(seed: int, sequence: int, step: int) -> int:
    return int(lib().tb_uniform24(seed, sequence, step))
