"""ctypes binding of the C ABI declared in include/leopard_b200.h.

There is no CPU fallback: if the shared library is missing or a call fails, a `NativeError` is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libleopard_b200.so"

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SWIGLU = 0, 1, 2, 3
LOGITS_NONE, LOGITS_LAST, LOGITS_ALL = 0, 1, 2


class NativeError(RuntimeError):
    pass


_vp, _ll, _i, _f, _sz = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_size_t


class VitDims(C.Structure):
    _fields_ = [(n, _i) for n in ("layers", "hidden", "ffn", "heads", "head_dim", "head_stride", "grid", "tokens",
                                  "patch_k", "patch_k_pad")] + [("eps", _f)]


class VitLayerWeights(C.Structure):
    _fields_ = [(n, _vp) for n in ("ln1_g", "ln1_b", "ln2_g", "ln2_b", "qkv_w", "qkv_b", "out_w", "out_b", "fc1_w",
                                   "fc1_b", "fc2_w", "fc2_b", "qkv_wf", "qkv_c1", "qkv_c2", "fc1_wf", "fc1_c1", "fc1_c2")]


class VitWeights(C.Structure):
    _fields_ = [("patch_w", _vp), ("patch_b", _vp), ("pos", _vp), ("layers", C.POINTER(VitLayerWeights)),
                ("post_g", _vp), ("post_b", _vp)]


class ProjWeights(C.Structure):
    _fields_ = [("w1", _vp), ("b1", _vp), ("w2", _vp), ("b2", _vp), ("act", _i)]


class DecDims(C.Structure):
    _fields_ = [(n, _i) for n in ("layers", "hidden", "ffn", "heads", "kv_heads", "head_dim", "vocab")] + [("eps", _f)]


class DecLayerWeights(C.Structure):
    _fields_ = [(n, _vp) for n in ("ln1_g", "qkv_w", "o_w", "ln2_g", "gateup_w", "down_w", "qkv_wf", "gateup_wf")]


class DecWeights(C.Structure):
    _fields_ = [("layers", C.POINTER(DecLayerWeights)), ("final_g", _vp), ("lm_head", _vp), ("inv_freq", _vp)]


class GemmDesc(C.Structure):
    """lp_gemm_desc (include/leopard_b200.h)."""
    _fields_ = [("A", _vp), ("lda", _ll), ("W", _vp), ("ldw", _ll), ("C", _vp), ("ldc", _ll), ("M", _i), ("N", _i), ("K", _i),
                ("bias", _vp), ("residual", _vp), ("ldr", _ll), ("res_row_mod", _i), ("act", _i), ("out_fp32", _i),
                ("block_n", _i), ("norm_mode", _i), ("stats_in", _vp), ("stats_in_parts", _i), ("colsum", _vp),
                ("norm_eps", _f), ("stats_out", _vp), ("stats_out_parts", _i), ("rope_cos", _vp), ("rope_sin", _vp),
                ("rope_heads", _i), ("a_t", _i), ("b_t", _i)]


NORM_NONE, NORM_RMS, NORM_LAYER = 0, 1, 2
TP_ALLGATHER, TP_REDUCE_SCATTER = 1, 2


class TpDesc(C.Structure):
    """lp_tp_desc (include/leopard_b200.h)."""
    _fields_ = [("tp_size", _i), ("tp_rank", _i), ("seg_rows", _i), ("mode", _i), ("epoch", C.c_uint), ("peer_A", _vp * 8),
                ("peer_stage", _vp * 8), ("counter", _vp), ("recycle", _vp), ("signal_local", _vp), ("signal_peer", _vp * 8)]


class ProfileRecord(C.Structure):
    _fields_ = [("kind", _i), ("a", _i), ("b", _i), ("c", _i), ("ms", _f)]


_P = C.POINTER

EPI_NONE, EPI_XIELU, EPI_SILU_GATE, EPI_RELU2, EPI_CLAMP_GLU = 0, 1, 2, 3, 4
GATED_EPIS = (EPI_SILU_GATE, EPI_CLAMP_GLU)      # W = [gate rows; up rows], half as many output columns
RET_FINISH_GATED_NORM, RET_FINISH_RAW = 0, 1
QKNORM_NONE, QKNORM_HEAD, QKNORM_FULL = 0, 1, 2
ROT_HALF, ROT_INTERLEAVED = 0, 1
RETENTION_CHUNK = 32


class LinearDesc(C.Structure):
    """lp_linear_desc (include/leopard_b200.h)."""
    _fields_ = [("A", _vp), ("lda", _ll), ("a_batch", _ll), ("a_fp32", _i), ("W", _vp), ("ldw", _ll), ("w_batch", _ll), ("C", _vp),
                ("ldc", _ll), ("c_batch", _ll), ("c_fp32", _i), ("M", _i), ("N", _i), ("K", _i), ("batch", _i), ("epi", _i),
                ("epi_a", _f), ("epi_b", _f), ("c_accum", _i), ("c_scale", _f), ("bias", _vp), ("row_scale", _vp), ("gate", _vp), ("ldg", _ll)]


class WindowAttnDesc(C.Structure):
    """lp_window_attn_desc (include/leopard_b200.h)."""
    _fields_ = [("qkv", _vp), ("ld", _ll), ("q_off", _i), ("k_off", _i), ("v_off", _i), ("heads", _i), ("kv_heads", _i), ("dim", _i),
                ("vdim", _i), ("norm_mode", _i), ("q_gain", _vp), ("k_gain", _vp), ("eps", _f), ("inv_freq", _vp), ("rot_dims", _i),
                ("rot_layout", _i), ("rot_mscale", _f), ("v_inv_freq", _vp), ("v_rot_dims", _i), ("v_rot_layout", _i), ("cache", _vp),
                ("page_size", _i), ("page_table", _vp), ("max_pages", _i), ("pooled", _vp), ("pooled_table", _vp),
                ("max_pooled_pages", _i), ("pool", _i), ("window", _i), ("keep_first", _i), ("scale", _f), ("softcap", _f), ("sink", _i),
                ("q_bias", _vp), ("k_bias", _vp), ("v_bias", _vp), ("v_norm", _i), ("talk", _vp), ("g_off", _i), ("chunk", _i), ("kv_shared", _i)]


class MinGRUDesc(C.Structure):
    """lp_mingru_desc (include/leopard_b200.h)."""
    _fields_ = [("zxg", _vp), ("ld", _ll), ("z_off", _i), ("x_off", _i), ("g_off", _i), ("width", _i), ("z_bias", _vp), ("x_bias", _vp),
                ("state", _vp), ("slot_stride", _ll), ("out", _vp), ("ldo", _ll), ("out_fp32", _i)]


class RetentionDesc(C.Structure):
    """lp_retention_desc (include/leopard_b200.h)."""
    _fields_ = [("qkvg", _vp), ("ld", _ll), ("q_off", _i), ("k_off", _i), ("v_off", _i), ("g_off", _i), ("heads", _i), ("dim", _i),
                ("vdim", _i), ("decay", _vp), ("inv_freq", _vp), ("rot_dims", _i), ("rot_layout", _i), ("rot_mscale", _f),
                ("k_scale", _f), ("eps", _f), ("state", _vp), ("slot_stride", _ll), ("out", _vp), ("ldo", _ll), ("out_fp32", _i),
                ("in_act", _i), ("finish", _i)]


class LatentDesc(C.Structure):
    """lp_latent_desc (include/leopard_b200.h)."""
    _fields_ = [("q", _vp), ("ldq", _ll), ("dkv", _vp), ("lddkv", _ll), ("heads", _i), ("dim", _i), ("rot_dim", _i), ("kv_rank", _i),
                ("c_gain", _vp), ("eps", _f), ("inv_freq", _vp), ("rot_dims", _i), ("rot_layout", _i), ("rot_mscale", _f),
                ("cache", _vp), ("page_size", _i), ("page_table", _vp), ("max_pages", _i), ("window", _i), ("scale", _f),
                ("sink", _vp), ("gate", _vp), ("ldg", _ll)]


class MLSTMDesc(C.Structure):
    """lp_mlstm_desc (include/leopard_b200.h)."""
    _fields_ = [("proj", _vp), ("ld", _ll), ("q_off", _i), ("k_off", _i), ("v_off", _i), ("g_off", _i), ("i_off", _i), ("f_off", _i),
                ("heads", _i), ("dim", _i), ("vdim", _i), ("i_bias", _vp), ("f_bias", _vp), ("gate_cap", _f), ("q_scale", _f),
                ("eps", _f), ("out_gain", _vp), ("state", _vp), ("slot_stride", _ll), ("out", _vp), ("ldo", _ll), ("out_fp32", _i)]


# name -> (restype, argtypes); must list EVERY symbol include/leopard_b200.h declares (tests/test_abi.py checks)
_SIGS = {
    "lp_last_error": (C.c_char_p, []),
    "lp_abi_version": (_i, []),
    "lp_gemm_bf16": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _vp, _vp, _ll, _i, _i, _i, _i, _vp]),
    "lp_gemm_bf16_ex": (_i, [C.POINTER(GemmDesc), _vp]),
    "lp_gemm_pick_block_n": (_i, [_i, _i, _i]),
    "lp_row_stats": (_i, [_vp, _ll, _i, _i, _vp, _vp]),
    "lp_model_set_fused_norm": (_i, [_i]),
    "lp_model_set_chained_projector": (_i, [_i]),
    "lp_gemm_set_pair_mode": (_i, [_i]),
    "lp_gemm_streamk_workspace_bytes": (_sz, []),
    "lp_gemm_set_streamk_workspace": (_i, [_vp, _sz]),
    "lp_gemm_set_streamk": (_i, [_i]),
    "lp_gemm_set_tma_residual": (_i, [_i]),
    "lp_gemm_set_raster_balance": (_i, [_i]),
    "lp_gemm_set_epilogue_sleep": (_i, [_i]),
    "lp_gemm_bf16_tp": (_i, [C.POINTER(GemmDesc), C.POINTER(TpDesc), _vp]),
    "lp_tp_reduce": (_i, [C.POINTER(TpDesc), _vp, _ll, _vp, _ll, _vp, _ll, _i, _vp]),
    "lp_parity_split": (_i, [_vp, _ll, _i, _i, _vp, _ll, _i, _vp]),
    "lp_parity_norm": (_i, [_vp, _ll, _vp, _vp, _vp, _ll, _i, _i, _f, _i, _vp]),
    "lp_parity_act": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _vp]),
    "lp_parity_add": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _vp]),
    "lp_parity_rope": (_i, [_vp, _ll, _i, _i, _i, _vp, _vp, _vp]),
    "lp_parity_softmax": (_i, [_vp, _ll, _i, _i, _f, _i, _vp]),
    "lp_set_prefill_pdl": (_i, [_i]),
    "lp_attention_fwd": (_i, [_vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _ll, _i, _vp]),
    "lp_attention_set_pingpong": (_i, [_i]),
    "lp_model_set_attention_variant": (_i, [_i]),
    "lp_attention_cross": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _ll, _vp]),
    "lp_layernorm": (_i, [_vp, _ll, _vp, _vp, _vp, _ll, _i, _i, _f, _i, _vp]),
    "lp_rmsnorm": (_i, [_vp, _ll, _vp, _vp, _ll, _i, _i, _f, _vp]),
    "lp_norm_set_variant": (_i, [_i]),
    "lp_rope_table": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "lp_rope_inplace": (_i, [_vp, _ll, _i, _i, _i, _i, _vp, _vp, _vp]),
    "lp_embed_merge": (_i, [_vp, _i, _ll, _i, _vp, _ll, _ll, _vp, _ll, _i, _vp, _ll, _i, _i, _vp, _vp]),
    "lp_im2col_patch14": (_i, [_vp, _i, _vp, _ll, _i, _i, _i, _i, _vp]),
    "lp_cross_entropy": (_i, [_vp, _i, _ll, _vp, _vp, _i, _i, _vp]),
    "lp_pixel_shuffle": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _vp]),
    "lp_vit_workspace_bytes": (_sz, [_P(VitDims), _i]),
    "lp_vit_forward": (_i, [_P(VitDims), _P(VitWeights), _vp, _i, _i, _vp, _ll, _i, _vp, _sz, _vp]),
    "lp_vit_layers_workspace_bytes": (_sz, [_P(VitDims), _i]),
    "lp_vit_layers": (_i, [_P(VitDims), _P(VitWeights), _vp, _P(_i), _i, _vp, _ll, _vp, _sz, _vp]),
    "lp_project_workspace_bytes": (_sz, [_i, _i]),
    "lp_project": (_i, [_P(ProjWeights), _vp, _i, _i, _i, _vp, _ll, _vp, _sz, _vp]),
    "lp_decoder_workspace_bytes": (_sz, [_P(DecDims), _i, _i]),
    "lp_decoder_prefill": (_i, [_P(DecDims), _P(DecWeights), _vp, _vp, _P(_i), _i, _vp, _ll, _vp, _ll, _i, _i, _vp,
                                _sz, _vp]),
    "lp_decode_workspace_bytes": (_sz, [_P(DecDims)]),
    "lp_decode_step": (_i, [_P(DecDims), _P(DecWeights), _vp, _ll, _vp, _i, _vp, _ll, _vp, _vp, _sz, _vp]),
    "lp_decode_greedy_step": (_i, [_P(DecDims), _P(DecWeights), _vp, _ll, _vp, _vp, _vp, _ll, _vp, _i, _vp, _sz, _vp]),
    "lp_decode_graph_create": (_i, [_P(DecDims), _P(DecWeights), _vp, _ll, _vp, _vp, _vp, _ll, _vp, _i, _vp, _sz,
                                    _P(_vp)]),
    "lp_decode_graph_launch": (_i, [_vp, _vp]),
    "lp_decode_graph_destroy": (None, [_vp]),
    "lp_decode_set_mode": (_i, [_i]),
    "lp_decode_set_prefetch": (_i, [_i, _i]),
    "lp_image_frontend_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "lp_image_frontend": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _i, C.c_double, _P(_f), _P(_f), _vp, _sz, _vp]),
    "lp_image_resize_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "lp_image_resize": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp, C.c_double, _P(_f), _P(_f), _vp, _sz, _vp]),
    "lp_decode_debug_stamps": (_i, [_vp]),
    "lp_attention_bwd_workspace_bytes": (_sz, [_i, _i, _i]),
    "lp_attention_bwd": (_i, [_vp, _ll, _vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _ll, _vp, _sz, _vp]),
    "lp_transpose_bf16": (_i, [_vp, _ll, _i, _i, _vp, _ll, _vp]),
    "lp_layernorm_bwd_workspace_bytes": (_sz, [_i]),
    "lp_layernorm_bwd": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _i, _i, _f, _vp, _sz, _vp]),
    "lp_pixel_unshuffle": (_i, [_vp, _ll, _vp, _ll, _i, _i, _i, _vp]),
    "lp_rowmod_sum": (_i, [_vp, _ll, _i, _i, _i, _vp, _vp]),
    "lp_rmsnorm_bwd_workspace_bytes": (_sz, [_i]),
    "lp_rmsnorm_bwd": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _i, _i, _f, _vp, _sz, _vp]),
    "lp_swiglu_fwd": (_i, [_vp, _ll, _vp, _ll, _i, _i, _vp]),
    "lp_swiglu_bwd": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _vp]),
    "lp_gelu_bwd": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _vp]),
    "lp_colsum_bf16": (_i, [_vp, _ll, _i, _i, _vp, _vp]),
    "lp_ce_fwd_bwd": (_i, [_vp, _i, _ll, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp]),
    "lp_embed_bwd": (_i, [_vp, _ll, _vp, _i, _ll, _vp, _ll, _i, _ll, _vp]),
    "lp_gather_rows_bf16": (_i, [_vp, _ll, _vp, _i, _i, _vp, _ll, _vp]),
    "lp_softmax_bwd": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _i, _i, _i, _f, _vp]),
    "lp_accumulate_f32": (_i, [_vp, _vp, _ll, _vp]),
    "lp_grad_norm_workspace_bytes": (_sz, []),
    "lp_sumsq_accum": (_i, [_vp, _ll, _vp, _vp]),
    "lp_grad_norm_finish": (_i, [_vp, _f, _vp, _vp]),
    "lp_adamw_step": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _i, _vp, _vp]),
    "lp_launch_count": (_ll, []),
    "lp_linear": (_i, [C.POINTER(LinearDesc), _vp]),
    "lp_linear_grouped": (_i, [C.POINTER(LinearDesc), _vp, _i, _vp, _vp]),
    "lp_linear_tile_rows": (_i, []),
    "lp_linear_pairs": (_i, [C.POINTER(LinearDesc), _vp, _i, _i, _vp]),
    "lp_embed_rows_f32": (_i, [_vp, _i, _vp, _ll, _i, _f, _vp, _ll, _i, _vp]),
    "lp_axpy_f32": (_i, [_vp, _ll, _vp, _ll, _f, _i, _i, _vp]),
    "lp_window_attn_prep": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _vp]),
    "lp_window_attn_pool": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _i, _vp]),
    "lp_window_attn": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _vp, _ll, _i, _vp]),
    "lp_window_attn_tiles": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _ll, _i, _vp]),
    "lp_window_attn_talk": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _vp, _ll, _i, _vp]),
    "lp_window_attn_talk_tiles": (_i, [C.POINTER(WindowAttnDesc), _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _ll, _i, _vp]),
    "lp_mlstm_workspace_bytes": (_sz, [_i, _i, _i]),
    "lp_mlstm": (_i, [C.POINTER(MLSTMDesc), _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "lp_add_positions_f32": (_i, [_vp, _ll, _i, _i, _vp, _vp, _vp]),
    "lp_add_row_f32": (_i, [_vp, _ll, _vp, _i, _i, _vp]),
    "lp_token_shift_f32": (_i, [_vp, _ll, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _vp]),
    "lp_moe_route_softmax": (_i, [_vp, _ll, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp, _vp, _vp]),
    "lp_mingru_workspace_bytes": (_sz, [_i, _i]),
    "lp_mingru_prefill": (_i, [C.POINTER(MinGRUDesc), _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "lp_mingru_decode": (_i, [C.POINTER(MinGRUDesc), _i, _vp, _vp, _vp, _vp]),
    "lp_rmsnorm_f32": (_i, [_vp, _ll, _i, _i, _f, _vp, _f, _vp, _ll, _i, _vp, _ll, _vp]),
    "lp_glu_f32": (_i, [_vp, _ll, _i, _vp, _ll, _i, _i, _i, _i, _f, _f, _vp]),
    "lp_glu_scaled_f32": (_i, [_vp, _ll, _i, _vp, _ll, _i, _i, _i, _i, _f, _f, _vp, _vp]),
    "lp_dyt_f32": (_i, [_vp, _ll, _i, _i, _f, _vp, _vp, _vp, _ll, _f, _vp, _vp, _vp, _ll, _i, _vp]),
    "lp_rmsnorm_gated_f32": (_i, [_vp, _ll, _i, _i, _vp, _f, _vp, _ll, _vp, _ll, _i, _vp]),
    "lp_gated_axpy_f32": (_i, [_vp, _ll, _vp, _ll, _vp, _vp, _ll, _vp, _f, _i, _i, _vp]),
    "lp_depth_average_f32": (_i, [_vp, _ll, _ll, _vp, _i, _vp, _ll, _vp, _ll, _i, _i, _vp]),
    "lp_moe_route_sigmoid": (_i, [_vp, _ll, _i, _i, _i, _vp, _ll, _i, _i, _vp, _vp, _vp]),
    "lp_moe_sorted_weights": (_i, [_vp, _vp, _i, _vp, _vp]),
    "lp_retention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "lp_retention_prefill": (_i, [C.POINTER(RetentionDesc), _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "lp_retention_decode": (_i, [C.POINTER(RetentionDesc), _i, _vp, _vp, _vp, _vp]),
    "lp_latent_prep": (_i, [C.POINTER(LatentDesc), _i, _vp, _vp, _vp]),
    "lp_latent_attend": (_i, [C.POINTER(LatentDesc), _i, _vp, _vp, _vp, _ll, _vp, _ll, _i, _vp]),
    "lp_moe_route": (_i, [_vp, _ll, _i, _i, _i, _vp, _ll, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "lp_moe_max_tiles": (_i, [_i, _i, _i]),
    "lp_moe_align": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "lp_moe_combine": (_i, [_vp, _ll, _vp, _vp, _i, _vp, _ll, _vp, _vp, _ll, _i, _i, _vp]),
    "lp_profile_enable": (_i, [_i]),
    "lp_profile_read": (_i, [_vp, _i]),
}

_lib = None


def declared_symbols():
    return sorted(_SIGS)


def lib():
    """Load (once) and return the native library; raises NativeError when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NativeError(
                f"{LIB_PATH} not found: build it with `python -m leopard_b200.build` "
                "(or __graft_entry__.build()); leopard_b200 has no CPU fallback")
        try:
            L = C.CDLL(str(LIB_PATH))
        except OSError as e:  # pragma: no cover
            raise NativeError(f"cannot load {LIB_PATH}: {e}") from e
        for name, (restype, argtypes) in _SIGS.items():
            try:
                fn = getattr(L, name)
            except AttributeError as e:
                raise NativeError(f"{LIB_PATH} does not export {name}: rebuild the library") from e
            fn.argtypes = argtypes
            fn.restype = restype
        import os
        if os.environ.get("LEOPARD_PREFILL_PDL") is not None:  # A/B switch for the prefill kernels' launch mode
            L.lp_set_prefill_pdl(int(os.environ["LEOPARD_PREFILL_PDL"]))
        _lib = L
    return _lib


# ---- the 32-bit residual-stream entry points (csrc/lp_linear.cu, lp_stream32.cu, lp_seqmix.cu, lp_winattn.cu, lp_mingru.cu, lp_mlstm.cu, lp_moe.cu) -----------------------------------
# They need none of the tcgen05 translation units, so a model that uses only them can run from a library of its own that compiles in
# seconds (build.build_native("stream32")); the full library contains the same symbols and is preferred when it is already built.
STREAM32_LIB_PATH = PKG / "lib" / "libleopard_stream32.so"
STREAM32_SYMBOLS = ("lp_last_error", "lp_abi_version", "lp_launch_count", "lp_linear", "lp_linear_grouped", "lp_linear_tile_rows", "lp_linear_pairs",
                    "lp_embed_rows_f32", "lp_rmsnorm_f32", "lp_glu_f32", "lp_retention_workspace_bytes", "lp_retention_prefill",
                    "lp_retention_decode", "lp_latent_prep", "lp_latent_attend", "lp_moe_route", "lp_moe_max_tiles", "lp_moe_align",
                    "lp_moe_combine", "lp_axpy_f32", "lp_window_attn_prep", "lp_window_attn_pool", "lp_window_attn", "lp_window_attn_tiles",
                    "lp_mingru_workspace_bytes",
                    "lp_mingru_prefill", "lp_mingru_decode", "lp_window_attn_talk", "lp_window_attn_talk_tiles", "lp_mlstm_workspace_bytes", "lp_mlstm",
                    "lp_add_positions_f32", "lp_add_row_f32", "lp_token_shift_f32", "lp_moe_route_softmax", "lp_glu_scaled_f32", "lp_dyt_f32",
                    "lp_rmsnorm_gated_f32", "lp_gated_axpy_f32", "lp_depth_average_f32", "lp_moe_route_sigmoid", "lp_moe_sorted_weights")
STREAM32_OPTIONAL = ("lp_gemm_bf16",)      # present in the native libraries, absent from the CPU-emulated build
_stream32 = None


def bind_stream32(L):
    """Set the signatures of the 32-bit residual-stream entry points on a loaded library (the native one, or the CPU-emulated build
    of the same sources that the tests make)."""
    for name in STREAM32_SYMBOLS:
        try:
            fn = getattr(L, name)
        except AttributeError as e:
            raise NativeError(f"the library does not export {name}: rebuild it") from e
        fn.restype, fn.argtypes = _SIGS[name]
    for name in STREAM32_OPTIONAL:
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = _SIGS[name]
    return L


def stream32_lib(build: bool = True):
    """The native library with the 32-bit residual-stream entry points: the full library when it is built and current, else the small
    one (built on first use when `build`)."""
    global _stream32
    if _stream32 is None:
        from . import build as _build
        if _lib is not None or _build.is_current():
            _stream32 = lib()
        else:
            if build:
                _build.build_native(component="stream32")
            if not STREAM32_LIB_PATH.exists():
                raise NativeError(f"{STREAM32_LIB_PATH} not found: build it with `python -m leopard_b200.build stream32`")
            try:
                _stream32 = bind_stream32(C.CDLL(str(STREAM32_LIB_PATH)))
            except OSError as e:  # pragma: no cover
                raise NativeError(f"cannot load {STREAM32_LIB_PATH}: {e}") from e
    return _stream32


def check_on(L, rc: int, what: str):
    """`check` for a call made on library L (its own error text)."""
    if rc != 0:
        msg = L.lp_last_error()
        raise NativeError(f"{what} failed (status {rc}): {msg.decode() if msg else '?'}")


_streamk_ws = None   # the device buffer handed to lp_gemm_set_streamk_workspace (kept alive here)


def ensure_streamk_workspace(device=None):
    """Give the GEMM its stream-K workspace (include/leopard_b200.h: lp_gemm_set_streamk_workspace) on the process's GPU — one
    process per GPU, one compute stream, as everywhere in this package.  LEOPARD_STREAMK=0 leaves the stream-K tail off."""
    global _streamk_ws
    import os
    import torch
    L = lib()
    if os.environ.get("LEOPARD_STREAMK", "1") == "0" or not torch.cuda.is_available():
        return None
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    if dev.index is None:                   # "cuda" and "cuda:<current>" are the same device
        dev = torch.device("cuda", torch.cuda.current_device())
    if _streamk_ws is not None:
        if _streamk_ws.device != dev:      # a second device in one process: the single workspace cannot serve both
            check(L.lp_gemm_set_streamk_workspace(None, 0), "lp_gemm_set_streamk_workspace")
        return _streamk_ws
    with torch.cuda.device(dev):
        ws = torch.zeros(int(L.lp_gemm_streamk_workspace_bytes()), dtype=torch.uint8, device=dev)
    check(L.lp_gemm_set_streamk_workspace(C.c_void_p(ws.data_ptr()), ws.numel()), "lp_gemm_set_streamk_workspace")
    _streamk_ws = ws
    return ws


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().lp_last_error()
        raise NativeError(f"{what} failed (status {rc}): {msg.decode() if msg else '?'}")


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
