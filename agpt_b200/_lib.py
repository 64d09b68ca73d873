"""ctypes binding of libagpt_b200.so (the C ABI declared in include/agpt_b200.h).

There is no fallback: if the shared library is missing, loading raises with the build
command, and every compute entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# AGPT_B200_LIB selects another build of the same library (same ABI), e.g. one compiled with different flags
SO = os.environ.get("AGPT_B200_LIB") or os.path.join(HERE, "libagpt_b200.so")

vp, i32, i64, u64, f32, f64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_double
P32, P64 = C.POINTER(C.c_int32), C.POINTER(C.c_int64)


class TrieInfo(C.Structure):
    _fields_ = [("radix_count", i32), ("n_depth_files", i32), ("total_edge_chars", i64), ("total_counts", i64),
                ("leveled_nodes", i64),
                ("parent", P32), ("first_char_depth", P32), ("edge_len", P32), ("edge_mass", P32),
                ("endpoint_depth", P32), ("subtree_key", P32),
                ("edge_off", P64), ("edge_tok", P32), ("cnt_off", P64), ("cnt_tok", P32), ("cnt_val", P32),
                ("edge_start", P32)]


class GroupInfo(C.Structure):
    _fields_ = [("n", i64), ("n_units", i32), ("parent", P32), ("row", P64), ("trained", C.POINTER(C.c_uint8)), ("unit_of_row", P32)]


class PlanInfo(C.Structure):
    _fields_ = [("n", i64), ("tile_m", i32), ("n_tiles", i64), ("chain_rows", i64), ("max_depth", i32),
                ("sum_depth", i64), ("sum_group_prefix", i64), ("n_groups", i64), ("n_reduce_items", i64),
                ("n_reduce_nodes", i64), ("n_reduce_multi", i64),
                ("dfs_to_node", P32), ("node_to_dfs", P32), ("parent_dfs", P32), ("depth", P32), ("sub_end", P32),
                ("device", C.c_int)]


# name -> (restype, argtypes); every symbol include/agpt_b200.h declares
SIGNATURES = {
    "agpt_b200_last_error": (C.c_char_p, []),
    "agpt_b200_version": (C.c_char_p, []),
    "cuda_batched_varlen_attention": (None, [vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, f32]),
    "cuda_batched_varlen_attention_backward": (None, [vp] * 10 + [C.c_int] * 4 + [f32]),
    "cuda_unpack_batched_attn_output": (None, [vp, vp, C.c_int, C.c_int, C.c_int]),
    "cuda_batched_varlen_attention_L_queries": (None, [vp] * 9 + [C.c_int] * 4 + [f32]),
    "cuda_batched_varlen_attention_L_queries_backward": (None, [vp] * 12 + [C.c_int] * 4 + [f32]),
    "cuda_sync": (None, []),
    "agpt_b200_synth_markov_corpus": (C.c_int, [i64, C.c_int, C.c_int, u64, vp]),
    "agpt_b200_synth_markov_corpus_repeats": (C.c_int, [i64, C.c_int, C.c_int, u64, C.c_int, vp]),
    "agpt_b200_synth_tree": (i64, [i64, C.c_int, C.c_int, f64, C.c_int, i64, u64, vp]),
    "agpt_b200_groups_create": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, i64, C.POINTER(vp)]),
    "agpt_b200_groups_count": (i64, [vp]),
    "agpt_b200_groups_get": (C.c_int, [vp, i64, C.POINTER(GroupInfo)]),
    "agpt_b200_groups_free": (None, [vp]),
    "agpt_b200_mass_weights": (C.c_int, [vp, vp, vp, vp, i64, i64, C.c_int, vp]),
    "agpt_b200_trie_build": (C.c_int, [vp, i64, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "agpt_b200_trie_load_dir": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "agpt_b200_trie_manifest": (i64, [C.c_char_p, i64, vp, vp, vp, vp]),
    "agpt_b200_trie_load_subtree": (C.c_int, [C.c_char_p, i32, C.POINTER(vp)]),
    "agpt_b200_trie_save_dir": (C.c_int, [vp, C.c_char_p, C.c_int, i32, i32, u64, C.c_char_p]),
    "agpt_b200_trie_info": (C.c_int, [vp, C.POINTER(TrieInfo)]),
    "agpt_b200_trie_free": (None, [vp]),
    "agpt_b200_token_hash": (u64, [vp, i64]),
    "agpt_b200_trie_char_tree": (C.c_int, [vp, vp, vp, vp, vp]),
    "agpt_b200_plan_create": (C.c_int, [vp, i64, C.c_int, C.c_int, C.POINTER(vp)]),
    "agpt_b200_plan_info": (C.c_int, [vp, C.POINTER(PlanInfo)]),
    "agpt_b200_plan_destroy": (None, [vp]),
    "agpt_b200_attn_bwd_workspace_bytes": (i64, [vp, C.c_int]),
    "agpt_b200_plan_units": (i64, [vp, C.c_int, i64, vp, vp]),
    "agpt_b200_partition_lpt": (C.c_int, [vp, i64, C.c_int, vp]),
    "agpt_b200_gather_rows": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
    "cuda_layer_norm_forward": (None, [vp] * 6 + [C.c_int, C.c_int]),
    "cuda_layer_norm_backward": (None, [vp] * 7 + [C.c_int, C.c_int]),
    "agpt_b200_layer_norm_fwd": (C.c_int, [vp] * 6 + [i64, C.c_int, vp]),
    "agpt_b200_layer_norm_bwd": (C.c_int, [vp] * 7 + [i64, C.c_int, vp, i64, vp]),
    "agpt_b200_layer_norm_bwd_add": (C.c_int, [vp] * 8 + [i64, C.c_int, vp, i64, vp]),
    "agpt_b200_layer_norm_bwd_workspace_bytes": (i64, [i64, C.c_int]),
    "cuda_bias_add": (None, [vp, vp, C.c_int, C.c_int]),
    "cuda_fused_bias_relu": (None, [vp] * 4 + [C.c_int, C.c_int]),
    "cuda_relu_backward": (None, [vp] * 3 + [C.c_int]),
    "cuda_softmax_rows": (None, [vp, vp, C.c_int, C.c_int]),
    "cuda_softmax_backward": (None, [vp] * 3 + [C.c_int, C.c_int]),
    "cuda_embedding_gather": (None, [vp] * 3 + [C.c_int, C.c_int]),
    "cuda_embedding_scatter_add": (None, [vp] * 3 + [C.c_int, C.c_int]),
    "agpt_b200_bias_act": (C.c_int, [vp] * 4 + [i64, C.c_int, C.c_int, vp]),
    "agpt_b200_relu_bwd": (C.c_int, [vp] * 3 + [i64, vp]),
    "agpt_b200_col_sum": (C.c_int, [vp] * 3 + [i64, C.c_int, f32, C.c_int, vp, vp, i64, vp]),
    "agpt_b200_col_sum_workspace_bytes": (i64, [i64, C.c_int]),
    "agpt_b200_softmax_rows": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "agpt_b200_softmax_bwd": (C.c_int, [vp] * 3 + [i64, C.c_int, vp]),
    "agpt_b200_embedding_gather": (C.c_int, [vp] * 3 + [i64, C.c_int, C.c_int, vp]),
    "agpt_b200_embedding_grad": (C.c_int, [vp] * 3 + [i64, C.c_int, C.c_int, C.c_int, vp, i64, vp]),
    "agpt_b200_embedding_grad_workspace_bytes": (i64, [i64, C.c_int, C.c_int]),
    "cuda_adam_bulk": (None, [vp] * 4 + [f32] * 4 + [C.c_int, C.c_int]),
    "cuda_sgd_bulk": (None, [vp, vp, f32, C.c_int]),
    "cuda_momentum_bulk": (None, [vp] * 3 + [f32, f32, C.c_int]),
    "cuda_rmsprop_bulk": (None, [vp] * 3 + [f32] * 3 + [C.c_int]),
    "cuda_weight_decay": (None, [vp, f32, f32, C.c_int]),
    "cuda_grad_clip_by_norm": (None, [vp, f32, C.c_int, vp, vp]),
    "agpt_b200_optimizer_step": (C.c_int, [C.c_int] + [vp] * 4 + [i64] + [f32] * 4 + [C.c_int, f32, f32, C.c_int, vp, vp]),
    "agpt_b200_optimizer_scratch_bytes": (i64, []),
    "agpt_b200_device_status": (C.c_int, [vp]),
    "agpt_b200_compute_lr": (f32, [f32, C.c_int, C.c_int, C.c_int, C.c_int]),
    "agpt_b200_lightning_sample": (i64, [vp, C.c_int, C.c_int, f32, i64, vp, vp, vp, vp, vp, vp, i64]),
    "agpt_b200_trie_from_suffix_order": (C.c_int, [vp, i64, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, C.POINTER(vp)]),
    "agpt_b200_suffix_order_gpu": (C.c_int, [vp, i64, C.c_int, C.c_int, vp, vp, C.POINTER(C.c_float)]),
    "agpt_b200_trie_build_gpu": (C.c_int, [vp, i64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "agpt_b200_gemm_f32": (C.c_int, [C.c_int] * 5 + [f32, vp, C.c_int, vp, C.c_int, f32, vp, C.c_int, vp, C.c_int, vp, C.c_int, C.c_int, vp,
                                     i64, vp]),
    "agpt_b200_gemm_f32_workspace_bytes": (i64, [C.c_int] * 6),
    "agpt_b200_set_gemm_impl": (C.c_int, [C.c_int]),
    "agpt_b200_rope_table": (C.c_int, [vp, vp, C.c_int, C.c_int, f32]),
    "agpt_b200_rope": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, C.c_int, C.c_int, vp]),
    "agpt_b200_rope_pair": (C.c_int, [vp, vp, vp, vp, vp, i64, C.c_int, C.c_int, C.c_int, vp]),
    "agpt_b200_kv_store_write_bf16": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "agpt_b200_attn_fwd": (C.c_int, [vp, vp, vp, vp, C.c_int, vp, vp, C.c_int, C.c_int, f32, vp]),
    "agpt_b200_attn_bwd": (C.c_int, [vp, vp, vp, vp, C.c_int, vp, vp, vp, vp, vp, vp, vp, i64, C.c_int, C.c_int, f32, vp]),
    "agpt_b200_attn_bwd_mode": (C.c_int, [vp, vp, vp, vp, C.c_int, vp, vp, vp, vp, vp, vp, vp, i64, C.c_int, C.c_int, f32, C.c_int, vp, vp]),
    "agpt_b200_set_attn_impl": (C.c_int, [C.c_int]),
    "agpt_b200_set_attn_variant": (C.c_int, [C.c_int, C.c_int]),
    "agpt_b200_attn_bwd_static": (C.c_int, [vp, vp, vp, vp, C.c_int, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, f32, vp]),
    "agpt_b200_static_scratch_bytes": (i64, []),
    "agpt_b200_loss_per_query": (C.c_int, [vp] * 11 + [i64, C.c_int, f32, f32, C.c_int, vp]),
    "agpt_b200_loss_per_node": (C.c_int, [vp] * 7 + [i64, C.c_int, vp]),
    "agpt_b200_attn_fwd_bwd_host": (C.c_int, [vp] * 10 + [C.c_int, C.c_int, C.c_int, f32]),
}

_lib = None


class AgptError(RuntimeError):
    pass


def lib():
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO):
            raise AgptError(f"{SO} is missing: build it with `python -m agpt_b200.build` (nvcc, sm_100a); "
                            "there is no CPU fallback")
        L = C.CDLL(SO)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int, what: str = ""):
    if rc < 0:
        raise AgptError(f"{what}: {lib().agpt_b200_last_error().decode()} (code {rc})")
    return rc
