"""ctypes binding of include/crabml_cuda.h (the drop-in C ABI)."""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libcrabml_cuda.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "crabml_cuda.h")
RUNNER_HEADER = os.path.join(os.path.dirname(HERE), "include", "crabml_runner.h")
SEQOPS_HEADER = os.path.join(os.path.dirname(HERE), "include", "crabml_seqops.h")
ZATORAX_HEADER = os.path.join(os.path.dirname(HERE), "include", "crabml_zatorax.h")

CC_OK, CC_ERR_TENSOR, CC_ERR_CUDA, CC_ERR_ARG, CC_ERR_UNSUPPORTED = 0, 1, 2, 3, 4
CC_MAX_DIMS = 4

# GGMLType ids (crabml-core/src/gguf.rs:86-108)
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1 = 0, 1, 2, 3, 6, 7, 8, 9
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_K = 10, 11, 12, 13, 14, 15
I32, BF16 = 26, 30
ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_SWISH, ACT_SIGMOID = 0, 1, 2, 3, 4
ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1
ROPE_LLAMA, ROPE_NEOX = 0, 1
QK_NORM_NONE, QK_NORM_HEAD, QK_NORM_ROW = 0, 1, 2
ROPE_NEIGHBOURS, ROPE_HALVES = 0, 1


class TensorError(Exception):
    """ErrorKind::TensorError (crabml-core/src/error.rs:24-25)."""


class CudaError(RuntimeError):
    pass


class cc_view(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("ndim", C.c_int32), ("shape", C.c_int64 * CC_MAX_DIMS), ("strides", C.c_int64 * CC_MAX_DIMS)]


class cc_device_options(C.Structure):
    _fields_ = [("device_ordinal", C.c_int32), ("debug_named_tensors", C.c_int32), ("lazy", C.c_int32),
                ("exact_order", C.c_int32), ("pool_bytes", C.c_uint64)]


def declared_symbols():
    """Every CC_API prototype name in the headers (used by the CPU-side export test)."""
    out = []
    for h in (HEADER, RUNNER_HEADER, SEQOPS_HEADER, ZATORAX_HEADER):
        with open(h) as f:
            out += re.findall(r"^CC_API [\w\s\*]+?\b(c[cz]r?_\w*)\(", f.read(), flags=re.M)
    return out


class ccr_llama_config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_heads", "n_kv_heads", "n_layers", "embedding_dim", "hidden_dim", "seq_len", "vocab_size", "rope_dim")] + \
               [("rms_norm_eps", C.c_float), ("use_f16_kv_cache", C.c_int32), ("shard_rank", C.c_int32), ("shard_world", C.c_int32), ("hidden_local", C.c_int32),
                ("arch", C.c_int32)]


class ccr_llama_weights(C.Structure):
    _pp = C.POINTER(C.c_void_p)
    _fields_ = [("token_embed", C.c_void_p), ("wq", _pp), ("wk", _pp), ("wv", _pp), ("wo", _pp), ("ffn_gate", _pp),
                ("ffn_down", _pp), ("ffn_up", _pp), ("rms_att", _pp), ("rms_ffn", _pp), ("rms_final", C.c_void_p),
                ("output_weight", C.c_void_p), ("bq", _pp), ("bk", _pp), ("bv", _pp)]


class czr_layer_config(C.Structure):            # include/crabml_zatorax.h
    _fields_ = [(n, C.c_int32) for n in ("mixer", "heads", "kv_heads", "dim", "vdim", "conv", "window", "kv_from")] + [("scale", C.c_float)] + \
               [(n, C.c_int32) for n in ("has_mlp", "experts", "top", "groups", "keep_groups", "expert_ff", "shared_ff")]


class czr_config(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("width", C.c_int32), ("vocab", C.c_int32), ("norm_eps", C.c_float), ("chunk", C.c_int32)]


CZR_WEIGHT_FIELDS = ("norm1", "norm2", "q", "k", "v", "o", "q_conv", "k_conv", "v_conv", "b", "a", "a_log", "dt_bias", "out_norm", "g", "q_norm", "k_norm",
                     "r1", "r2", "router", "correction", "e_gate", "e_up", "e_down", "s_gate", "s_up", "s_down")


class czr_layer_weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in CZR_WEIGHT_FIELDS]


class cmr_layer_config(C.Structure):            # include/crabml_meresun.h
    _fields_ = [(n, C.c_int32) for n in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "window")] + [("scale", C.c_float), ("rot_mag", C.c_float)] + \
               [(n, C.c_int32) for n in ("ff_kind", "ff", "experts", "top", "groups", "keep_groups")] + [("limit", C.c_float)]


class cmr_config(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("width", C.c_int32), ("vocab", C.c_int32), ("norm_eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("norm_groups", "loop_start", "loop_stop", "loop_times", "side_dim", "chunk", "max_seq")]


CMR_WEIGHT_FIELDS = ("norm1", "h_stack", "dq_norm", "uq", "dkv_norm", "uk", "uv", "uk_t", "uv_f32", "sink", "rot_freq", "o", "rg1_b", "rg2_b", "down", "act",
                     "router", "correction", "e_gate", "e_up", "e_down", "side_table", "side_gate", "side_proj", "side_norm")


class cmr_layer_weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in CMR_WEIGHT_FIELDS]


class cvr_layer_config(C.Structure):            # include/crabml_vuzinex.h
    _fields_ = [(n, C.c_int32) for n in ("mixer", "heads", "kv_heads", "dim", "vdim", "window", "block", "left_gate")] + [("scale", C.c_float), ("rot_mag", C.c_float)] + \
               [(n, C.c_int32) for n in ("right", "r_heads", "r_dim", "r_vdim", "r_rank")] + \
               [(n, C.c_float) for n in ("gate_cap", "tau", "r_q_scale", "left_scale", "right_scale")] + \
               [(n, C.c_int32) for n in ("s_heads", "s_vdim", "s_state", "s_groups", "s_conv", "s_norm_groups", "ff")]


class cvr_config(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("width", C.c_int32), ("vocab", C.c_int32), ("norm_eps", C.c_float), ("residual_mult", C.c_float), ("logit_scale", C.c_float)] + \
               [(n, C.c_int32) for n in ("loop_start", "loop_stop", "loop_times")] + [(n, C.c_int64) for n in ("hash_buckets", "hash_mul_prev", "hash_mul_cur")] + \
               [("chunk", C.c_int32), ("max_seq", C.c_int32)]


CVR_WEIGHT_FIELDS = ("norm_a", "norm_b", "norm_c", "norm_d", "h_stack", "h_bias", "q_norm", "k_norm", "sink", "rot_freq", "left_o", "right_norm", "right_o", "gate_bias_i",
                     "gate_bias_f", "decay_up", "decay_bias", "in", "conv", "conv_bias", "dt_bias", "a_log", "d_skip", "s_norm", "s_o", "gate_up", "gate_up_bias", "down",
                     "down_bias")


class cvr_layer_weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in CVR_WEIGHT_FIELDS]


class clr_layer_config(C.Structure):            # include/crabml_lifesun.h
    _fields_ = [(n, C.c_int32) for n in ("heads", "kv_heads", "dim", "vdim", "window", "block", "qk_norm", "left_gate")] + [("scale", C.c_float), ("softcap", C.c_float)] + \
               [(n, C.c_int32) for n in ("right", "r_width", "r_blocks", "r_conv", "r_heads", "r_dim", "r_vdim")] + \
               [(n, C.c_float) for n in ("r_rate", "left_scale", "right_scale")] + [("ff", C.c_int32)]


class clr_config(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("width", C.c_int32), ("vocab", C.c_int32), ("norm_eps", C.c_float), ("logit_scale", C.c_float)] + \
               [(n, C.c_int32) for n in ("loop_start", "loop_stop", "loop_times", "chunk", "max_seq")]


CLR_WEIGHT_FIELDS = ("norm_w", "norm_b", "h_stack", "q_norm", "k_norm", "sink", "rot_freq", "left_o", "right_o", "x_bias", "y_bias", "conv", "conv_bias", "gate_w", "gate_b",
                     "lam", "r_rot_freq", "decay", "down")


class clr_layer_weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in CLR_WEIGHT_FIELDS]


class cc_route_params(C.Structure):              # include/crabml_seqops.h
    _fields_ = [(n, C.c_int32) for n in ("score", "top", "n_groups", "keep_groups", "group_top", "renormalise")] + [("renorm_eps", C.c_float)]


class cc_glu_params(C.Structure):
    _fields_ = [("act", C.c_int32), ("alpha", C.c_float), ("limit", C.c_float), ("up_shift", C.c_float)]


_lib = None


def load_library(build_if_missing: bool = True):
    """Loads the in-tree .so; builds it with nvcc first when it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    alt = os.environ.get("CRABML_CUDA_LIB")          # developer A/B: another build of the same library
    if alt:
        build_if_missing = False
    if build_if_missing:
        from . import build as _build
        if _build.needs_build():
            _build.build()
    if not os.path.exists(LIB_PATH):
        raise CudaError(f"{LIB_PATH} is missing: run `python -m crabml_b200.build` (no CPU fallback exists)")
    L = C.CDLL(alt if alt else LIB_PATH)
    vp, i32, i64, u64, sz, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_size_t, C.c_float
    pv = C.POINTER(cc_view)
    pp = C.POINTER(C.c_void_p)
    sig = {
        "cc_device_create": (i32, [C.POINTER(cc_device_options), pp]),
        "cc_device_destroy": (None, [vp]),
        "cc_last_error": (C.c_char_p, [vp]),
        "cc_device_synchronize": (i32, [vp]),
        "cc_device_launch_count": (u64, [vp]),
        "cc_device_flush": (i32, [vp]),
        "cc_lazy_stats": (i32, [vp, C.POINTER(u64)]),
        "cc_test_mega_barrier_floor": (i32, [vp, i32, C.POINTER(f32)]),
        "cc_lazy_mega_profile": (i32, [vp, C.POINTER(u64), C.POINTER(i32), i32, C.POINTER(i32)]),
        "cc_lazy_mega_variant": (i32, [vp]),
        "cc_device_stream": (vp, [vp]),
        "cc_tensor_from_cpu": (i32, [vp, vp, sz, C.POINTER(i64), i32, i32, pp]),
        "cc_tensor_alloc": (i32, [vp, C.POINTER(i64), i32, i32, pp]),
        "cc_tensor_retain": (None, [vp]),
        "cc_tensor_release": (None, [vp]),
        "cc_tensor_dtype": (i32, [vp]),
        "cc_tensor_capacity": (i64, [vp]),
        "cc_tensor_dup": (i32, [vp, pv, pp]),
        "cc_tensor_export_f32": (i32, [vp, pv, vp, sz]),
        "cc_copy_rows_from": (i32, [vp, pv, pv, C.POINTER(i64), i32]),
        "cc_concatenate": (i32, [vp, pv, pv, i32]),
        "cc_contiguous": (i32, [vp, pv, pp]),
        "cc_rope_inplace": (i32, [vp, pv, i32, i64, i64]),
        "cc_rms_norm_inplace": (i32, [vp, pv, f32]),
        "cc_softmax_inplace": (i32, [vp, pv, i32]),
        "cc_silu_inplace": (i32, [vp, pv]),
        "cc_gelu_inplace": (i32, [vp, pv]),
        "cc_mul_inplace": (i32, [vp, pv, pv]),
        "cc_add_inplace": (i32, [vp, pv, pv]),
        "cc_scale_inplace": (i32, [vp, pv, f32]),
        "cc_matmul_vec": (i32, [vp, pv, pv, pp]),
        "cc_batch_matmul": (i32, [vp, pv, pv, pp]),
        "cc_debug_tensor_tap": (i32, [vp, C.c_char_p, pv]),
        "cc_dump_debug_tensor": (i32, [vp, C.c_char_p, vp, C.POINTER(sz)]),
        "cc_test_quantize_activation": (i32, [vp, pv, i32, vp, sz]),
        "cc_tensor_synth": (i32, [vp, C.POINTER(i64), i32, i32, u64, u64, f32, pp]),
        "cc_test_export_blocks": (i32, [vp, vp, vp, sz]),
        "cc_tensor_synth_slice": (i32, [vp, C.POINTER(i64), i32, i32, u64, u64, f32, i64, i64, i64, i64, pp]),
        "cc_comm_create": (i32, [vp, i32, i32, vp]),
        "cc_comm_connect": (i32, [vp, vp]),
        "cc_comm_nccl_unique_id": (i32, [vp, vp]),
        "cc_comm_connect_local": (i32, [vp, vp]),
        "cc_device_set_sm_limit": (i32, [vp, i32]),
        "cc_comm_init_nccl": (i32, [vp, vp]),
        "cc_comm_rank": (i32, [vp]),
        "cc_comm_world_size": (i32, [vp]),
        "cc_all_reduce_sum_inplace": (i32, [vp, pv]),
        "cc_all_gather": (i32, [vp, pv, pv]),
        "cc_bench_timer_begin": (i32, [vp]),
        "cc_bench_timer_end": (i32, [vp, C.POINTER(f32)]),
    }
    sig.update({
        "ccr_runner_create": (i32, [vp, C.POINTER(ccr_llama_config), C.POINTER(ccr_llama_weights), i32, pp]),
        "ccr_runner_destroy": (None, [vp]),
        "ccr_runner_last_error": (C.c_char_p, [vp]),
        "ccr_runner_forward": (i32, [vp, C.POINTER(i64), i32, i64, vp]),
        "ccr_runner_kv_cache_len": (i64, [vp]),
        "ccr_runner_generate_greedy": (i32, [vp, C.POINTER(i64), i32, i32, i64, C.POINTER(i64), C.POINTER(i32)]),
        "ccr_runner_generate_greedy_ex": (i32, [vp, C.POINTER(i64), i32, i32, i64, C.POINTER(i64), C.POINTER(i32), vp]),
        "cc_argmax_to_slot": (i32, [vp, pv, i32, i64]),
        "cc_copy_rows_from_slot": (i32, [vp, pv, pv, i32]),
        "cc_slot_set": (i32, [vp, i32, i64]),
        "cc_read_history": (i32, [vp, i64, i64, C.POINTER(i64)]),
        "cc_tensor_export_f32_async": (i32, [vp, pv, vp, C.c_size_t]),
        "cc_host_alloc": (i32, [vp, C.c_size_t, pp]),
        "cc_host_free": (None, [vp, vp]),
    })
    # sequence-mixing / routing ops (include/crabml_seqops.h) and the Zatorax runner (include/crabml_zatorax.h)
    sig.update({
        "cc_tensor_zero": (i32, [vp, pv]),
        "cc_rms_norm_gain": (i32, [vp, pv, pv, pv, f32, i32]),
        "cc_gated_head_rms_norm": (i32, [vp, pv, pv, pv, i32, f32, i32]),
        "cc_glu_inplace": (i32, [vp, pv, pv, i32]),
        "cc_short_conv": (i32, [vp, pv, pv, pv, i32, i32, i32, f32, f32, pp]),
        "cc_gated_delta_rule": (i32, [vp, pv, pv, pv, pv, pv, pv, pv, pv, i32, i32, i32, i32, pp]),
        "cc_kv_ring_append": (i32, [vp, pv, pv, pv, pv, pv, f32, i64, i32, i32, i32]),
        "cc_window_attention": (i32, [vp, pv, pv, f32, pv, pv, i64, i32, i32, i32, i32, i32, f32, pv, pv, pp]),
        "cc_moe_route": (i32, [vp, pv, pv, pv, i32, i32, i32, i32, pp, pp]),
        "cc_moe_experts": (i32, [vp, pv, pv, pv, pv, pv, pv, i32, i32, i32, pp]),
        "cc_group_rms_norm": (i32, [vp, pv, pv, pv, i32, f32]),
        "cc_poly_norm": (i32, [vp, pv, pv, f32]),
        "cc_gated_sum": (i32, [vp, pv, i32, pv, pv, pv, pv, pv, pv]),
        "cc_window_attention_sink": (i32, [vp, pv, pv, f32, pv, pv, i64, i32, i32, i32, i32, i32, f32, pv, pv, pv, pp]),
        "cc_rope_pairs": (i32, [vp, pv, i32, i32, i32, pv, f32, i64]),
        "cc_latent_ring_append": (i32, [vp, pv, pv, pv, f32, i32, pv, f32, i64]),
        "cc_split_cols": (i32, [vp, pv, i32, C.POINTER(i32), pp]),
        "cc_head_project": (i32, [vp, pv, pv, i32, i32, pv, f32, i64, pp]),
        "cc_head_concat_shared": (i32, [vp, pv, pv, i32, i32, i32, pp]),
        "cc_moe_route_ex": (i32, [vp, pv, pv, pv, C.POINTER(cc_route_params), pp, pp]),
        "cc_moe_experts_glu": (i32, [vp, pv, pv, pv, pv, pv, pv, i32, i32, C.POINTER(cc_glu_params), pp]),
        "cc_rms_norm_gain_mult": (i32, [vp, pv, pv, pv, f32, f32]),
        "cc_gated_group_rms_norm": (i32, [vp, pv, pv, pv, pv, i32, f32, i32]),
        "cc_glu_halves": (i32, [vp, pv, pv, i32, pp]),
        "cc_add_row_bias": (i32, [vp, pv, pv]),
        "cc_scaled_sum": (i32, [vp, pv, pv, f32, pv, f32]),
        "cc_pair_hash_rows_add": (i32, [vp, pv, pv, C.POINTER(i64), i32, i32, pv, i64, i64, i64]),
        "cc_short_conv_bias": (i32, [vp, pv, pv, pv, pv, i32, pp]),
        "cc_masked_attention": (i32, [vp, pv, pv, pv, i64, i32, i32, i32, i32, i32, i32, f32, pv, pp]),
        "cc_matrix_memory": (i32, [vp, pv, pv, pv, pv, pv, pv, pv, f32, f32, pv, pv, i32, i32, i32, pp]),
        "cc_decayed_linear_attention": (i32, [vp, pv, pv, pv, pv, pv, f32, f32, pv, i32, i32, i32, pp]),
        "cc_state_space_scan": (i32, [vp, pv, pv, pv, pv, pv, pv, i32, i32, i32, i32, pp]),
        "cc_layer_norm": (i32, [vp, pv, pv, pv, pv, f32]),
        "cc_head_gate": (i32, [vp, pv, pv, i32, i32]),
        "cc_rope_halves_two": (i32, [vp, pv, pv, i32, i32, i32, pv, f32, i64]),
        "cc_short_conv_biases": (i32, [vp, pv, pv, pv, pv, pv, i32, pp]),
        "cc_qk_prepare_append": (i32, [vp, pv, pv, pv, pv, pv, i32, pv, pv, f32, pv, i32, i32, f32, i64, i32, i32, i32, i32]),
        "cc_scaled_sum_accumulate": (i32, [vp, pv, pv, f32, pv, f32, pv]),
        "cc_concat_cols": (i32, [vp, pv, pv, pp]),
        "cc_rope_halves": (i32, [vp, pv, i32, i32, i32, pv, f32, i64]),
        "cc_masked_attention_capped": (i32, [vp, pv, pv, pv, i64, i32, i32, i32, i32, i32, i32, f32, f32, pv, pp]),
        "cc_retention": (i32, [vp, pv, pv, pv, pv, f32, pv, i32, i32, i32, pp]),
        "cc_gated_diagonal_recurrence": (i32, [vp, pv, pv, pv, pv, f32, i32, pv, pv, i32, pv, pp]),
        "clr_runner_create": (i32, [vp, C.POINTER(clr_config), C.POINTER(clr_layer_config), C.POINTER(clr_layer_weights), vp, vp, vp, vp, vp, pp]),
        "cvr_runner_create": (i32, [vp, C.POINTER(cvr_config), C.POINTER(cvr_layer_config), C.POINTER(cvr_layer_weights), vp, vp, vp, vp, pp]),
        "csr_runner_destroy": (None, [vp]),
        "csr_runner_last_error": (C.c_char_p, [vp]),
        "csr_last_create_error": (C.c_char_p, []),
        "csr_seq_open": (i32, [vp, C.POINTER(i32)]),
        "csr_seq_close": (i32, [vp, i32]),
        "csr_seq_len": (i64, [vp, i32]),
        "csr_runner_stats": (i32, [vp, C.POINTER(i64)]),
        "csr_runner_step": (i32, [vp, i32, C.POINTER(i64), i32, C.POINTER(i32), i32, vp]),
        "csr_runner_generate_greedy": (i32, [vp, i32, C.POINTER(i64), i32, i32, i64, C.POINTER(i64), C.POINTER(i32)]),
        "cmr_runner_create": (i32, [vp, C.POINTER(cmr_config), C.POINTER(cmr_layer_config), C.POINTER(cmr_layer_weights), vp, vp, vp, pp]),
        "czr_runner_create": (i32, [vp, C.POINTER(czr_config), C.POINTER(czr_layer_config), C.POINTER(czr_layer_weights), vp, vp, vp, pp]),
        "czr_last_create_error": (C.c_char_p, []),
        "czr_runner_destroy": (None, [vp]),
        "czr_runner_last_error": (C.c_char_p, [vp]),
        "czr_seq_open": (i32, [vp, C.POINTER(i32)]),
        "czr_seq_close": (i32, [vp, i32]),
        "czr_seq_len": (i64, [vp, i32]),
        "czr_runner_stats": (i32, [vp, C.POINTER(i64)]),
        "czr_runner_step": (i32, [vp, i32, C.POINTER(i64), i32, C.POINTER(i32), i32, vp]),
        "czr_runner_generate_greedy": (i32, [vp, i32, C.POINTER(i64), i32, i32, i64, C.POINTER(i64), C.POINTER(i32)]),
    })
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    # optional entry points (later build stages); bound when present
    _lib = L
    return L
