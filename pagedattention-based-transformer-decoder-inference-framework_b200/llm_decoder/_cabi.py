"""ctypes binding of libpa_b200.so (include/pa_b200.h).

torch tensors only supply device pointers (`.data_ptr()`) and the current stream; every
computation on the path happens inside the hand-written sm_100a kernels.  There is no
fallback: a missing or unloadable library raises at first use.
"""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libpa_b200.so")
CORE_LIB_PATH = os.path.join(_PKG, "libpa_b200_core.so")   # build.py --core: the subset the config-driven models need

PA_OK = 0
PA_ERR_UNSUPPORTED = -2
ACT = {"": 0, None: 0, "none": 0, "relu": 1, "gelu": 2}

_lib = None

_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

_DECODE_COMMON = [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp]

_SIGS = {
    "pa_version": ([], _i32),
    "pa_error_string": ([_i32], C.c_char_p),
    "pa_device_info": ([C.POINTER(_i32)] * 3, _i32),
    "pa_page_table_clear": ([_vp, _i64, _vp], _i32),
    "pa_page_table_update": ([_vp, _i64, _vp, _vp, _i32, _vp], _i32),
    "pa_page_table_lookup": ([_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_kv_gather": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _vp], _i32),
    "pa_kv_append_f16": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_kv_append_f32": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_kv_append_f32_f16": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_kv_append_f32_i8": ([_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_kv_copy_pages": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp], _i32),
    "pa_decode_workspace_bytes": ([_i32, _i32, _i32, _i32, _i32], _sz),
    "pa_paged_decode_f16": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_f16_overlap": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_i8": ([_vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_i8_overlap": ([_vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_f32": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_f32_overlap": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp], _i32),
    "pa_attention_filtered_workspace_bytes": ([_i32, _i32, _i32], _sz),
    "pa_paged_attention_filtered": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32] + _DECODE_COMMON + [_i32, _f32, _vp, _vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_f16_partial": ([_vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _sz, _vp], _i32),
    "pa_paged_decode_i8_partial": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _sz, _vp], _i32),
    "pa_paged_decode_f16_splitkv": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_paged_decode_i8_splitkv": ([_vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_vp, _vp, _sz, _vp, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_paged_decode_f16_group": ([_vp, _vp, _vp, _vp] + _DECODE_COMMON + [_i32, _vp, _vp, _sz, _vp], _i32),
    "pa_paged_decode_i8_group": ([_vp, _vp, _vp, _vp, _vp, _vp] + _DECODE_COMMON + [_i32, _vp, _vp, _sz, _vp], _i32),
    "pa_softmax_lut_i32": ([_vp, _i32, _i32, _f32, _vp, _i32, _vp, _vp], _i32),
    "pa_softmax_temperature": ([_vp, _i32, _i32, _f32, _vp, _vp], _i32),
    "pa_topk_topp_filter": ([_vp, _i32, _i32, _i32, _f32, _i32, _f32, _vp], _i32),
    "pa_sample_from_probs": ([_vp, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_prefill_workspace_bytes": ([_i32, _i32, _i32, _i32, _i32, _i32], _sz),
    "pa_paged_prefill_f16": ([_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp, _sz, _vp], _i32),
    "pa_paged_prefill_i8": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp, _sz, _vp], _i32),
    "pa_paged_prefill_f16_tokmajor": ([_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp], _i32),
    "pa_paged_prefill_i8_tokmajor": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _vp], _i32),
    "pa_lse_combine": ([_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_quantize_i8": ([_vp, _i64, _f32, _vp, _vp], _i32),
    "pa_batch_quantize_i8": ([_vp, _vp, _i32, _i32, _vp, _vp], _i32),
    "pa_absmax": ([_vp, _i64, _vp, _vp], _i32),
    "pa_minmax_scale": ([_vp, _i64, _vp, _vp], _i32),
    "pa_batch_minmax_scale": ([_vp, _i32, _i32, _vp, _vp], _i32),
    "pa_dequantize_i8": ([_vp, _i64, _f32, _vp, _vp], _i32),
    "pa_batch_dequantize_i8": ([_vp, _vp, _i32, _i32, _vp, _vp], _i32),
    "pa_gemm_i8_workspace_bytes": ([_i32, _i32, _i32, _i32], _sz),
    "pa_gemm_i8": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _f32, _f32, _vp, _i32, _vp, _sz, _vp], _i32),
    "pa_gemm_i8_dequant": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _f32, _vp, _i32, _vp, _sz, _vp], _i32),
    "pa_gemm_i8_dynquant_workspace_bytes": ([_i32, _i32, _i32], _sz),
    "pa_gemm_i8_dynquant": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _f32, _vp, _i32, _vp, _sz, _vp], _i32),
    "pa_embedding_f32": ([_vp, _vp, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_embedding_i8": ([_vp, _f32, _vp, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_layer_norm_f32": ([_vp, _vp, _vp, _i32, _i32, _f32, _vp, _vp], _i32),
    "pa_linear_workspace_bytes": ([_i32, _i32, _i32], _sz),
    "pa_linear_f32": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp], _i32),
    "pa_linear_pack_bytes": ([_i32, _i32], _sz),
    "pa_linear_pack_f32": ([_vp, _vp, _i32, _i32, _vp], _i32),
    "pa_linear_f32_packed": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp], _i32),
    "pa_logits_f32": ([_vp, _vp, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_logits_i8": ([_vp, _vp, _f32, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_argmax_f32": ([_vp, _i32, _i32, _f32, _i32, _vp, _vp], _i32),
    "pa_logits_argmax": ([_vp, _vp, _i32, _f32, _i32, _i32, _i32, _f32, _i32, _vp, _vp, _vp, _vp], _i32),
    "pa_layer_norm_quantize_i8": ([_vp, _vp, _vp, _i32, _i32, _f32, _vp, _vp, _vp, _vp], _i32),
    "pa_row_quantize_dynamic_i8": ([_vp, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_apply_rope_f32": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    "pa_advance_positions": ([_vp, _vp, _i32, _vp], _i32),
    "pa_splitkv_exchange_bytes": ([_i32, _i32, _i32], _sz),
    "pa_p2p_alloc": ([_sz, C.POINTER(_vp), C.c_char_p], _i32),
    "pa_p2p_open": ([C.c_char_p, C.POINTER(_vp)], _i32),
    "pa_p2p_close": ([_vp], _i32),
    "pa_p2p_free": ([_vp], _i32),
    "pa_splitkv_exchange_combine": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp], _i32),
    "pa_splitkv_exchange_send": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_splitkv_exchange_recv": ([_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp], _i32),
    "pa_nccl_unique_id": ([C.c_char_p], _i32),
    "pa_nccl_init": ([C.c_char_p, _i32, _i32, C.POINTER(_vp)], _i32),
    "pa_nccl_destroy": ([_vp], _i32),
    "pa_nccl_gather_bytes": ([_i32, _i32, _i32], _sz),
    "pa_nccl_allgather_combine": ([_vp, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _sz, _vp, _vp, _vp], _i32),
    # ragged-batch sequence ops (seq_ops.cu, diff_attention.cu, moe_ops.cu)
    "pa_linear_f32_exact": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp], _i32),
    "pa_embedding_rows": ([_vp, _i32, _vp, _i32, _i32, _i32, _vp, _vp], _i32),
    "pa_rms_norm_shift": ([_vp, _i32, _i32, _f32, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_rms_norm_state_store": ([_vp, _i32, _f32, _f32, _vp, _vp, _vp, _vp, _i32, _vp, _vp], _i32),
    "pa_mingru_scan": ([_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _vp], _i32),
    "pa_mingru_chunked_workspace_bytes": ([_i32, _i32], _sz),
    "pa_mingru_scan_chunked": ([_vp, _vp, _vp, _i32, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _vp, _sz, _vp], _i32),
    "pa_gelu_inplace": ([_vp, _i64, _i32, _vp], _i32),
    "pa_silu_mul": ([_vp, _i64, _i32, _vp, _i32, _vp], _i32),
    "pa_residual_combine": ([_vp, _i64, _i32, _f32, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _vp], _i32),
    "pa_gather_rows_f32": ([_vp, _vp, _i32, _i32, _vp, _vp], _i32),
    "pa_kv_append_rows": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _vp], _i32),
    "pa_diff_attention_tile_tokens": ([_i32, _i32], _i32),
    "pa_diff_attention_mma_tile_tokens": ([_i32, _i32, _i32], _i32),
    "pa_diff_attention_mma_head_rows": ([_i32, _i32, _i32, _i32, _i32], _i32),
    "pa_diff_attention_workspace_bytes": ([_i32, _i32, _i32, _i32, _i32], _sz),
    "pa_diff_attention": ([_vp, _i64, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _i32,
                           _f32, _f32, _i32, _f32, _f32, _f32, _vp, _i32, _i32, _i32, _vp, _sz, _vp], _i32),
    "pa_router_topk": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _vp], _i32),
    "pa_moe_tile_rows": ([], _i32),
    "pa_moe_max_tiles": ([_i32, _i32], _i32),
    "pa_moe_meta_ints": ([_i32, _i32], _sz),
    "pa_moe_sort": ([_vp, _i32, _i32, _vp, _vp, _vp], _i32),
    "pa_moe_gate_up": ([_vp, _i64, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _vp, _i32, _vp], _i32),
    "pa_moe_down": ([_vp, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _vp], _i32),
    "pa_moe_gate_up_act": ([_vp, _i64, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _i32, _vp, _i32, _vp], _i32),
    "pa_moe_up": ([_vp, _i64, _vp, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _i32, _vp, _i32, _vp], _i32),
    "pa_embedding_rows_scaled": ([_vp, _i32, _vp, _i32, _i32, _i32, _f32, _vp, _vp], _i32),
    "pa_act_mul": ([_vp, _i64, _i32, _i32, _vp, _i32, _vp], _i32),
    "pa_residual_add_norm": ([_vp, _i64, _i32, _f32, _vp, _vp, _vp, _vp, _i32, _vp, _i32, _vp], _i32),
    "pa_cast_rows": ([_vp, _i64, _vp, _i32, _vp], _i32),
    # attention through a low-rank latent (latent_attention.cu)
    "pa_rope_table": ([_vp, _i32, _i32, _f32, _vp, _vp], _i32),
    "pa_rope_rows": ([_vp, _i64, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _vp], _i32),
    "pa_latent_kv_append": ([_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _i32, _vp, _f32, _vp, _vp, _vp,
                             _i32, _i32, _vp], _i32),
    "pa_rms_norm_rows": ([_vp, _i64, _i32, _i32, _f32, _vp, _vp, _i64, _i32, _i32, _vp], _i32),
    "pa_head_linear": ([_vp, _i64, _i64, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _i64, _i32, _vp], _i32),
    "pa_head_gate": ([_vp, _i64, _i64, _vp, _i64, _i32, _i32, _i64, _vp, _i32, _vp], _i32),
    "pa_latent_attention_tile_tokens": ([_i32], _i32),
    "pa_latent_attention_mma_tile_tokens": ([_i32, _i32, _i32, _i32], _i32),
    "pa_latent_attention_workspace_bytes": ([_i32, _i32, _i32, _i32], _sz),
    "pa_latent_attention": ([_vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _i32,
                             _f32, _vp, _i64, _i64, _i32, _i32, _i32, _vp, _sz, _vp], _i32),
    # pre-norm wiring, looped blocks, grouped router
    "pa_residual_add_prenorm": ([_vp, _i64, _i32, _vp, _f32, _vp, _f32, _vp, _vp, _i32, _vp, _vp, _f32, _vp, _vp, _i32, _vp], _i32),
    "pa_concat_rows": ([_vp, _vp, _i64, _i32, _vp, _i32, _vp], _i32),
    "pa_router_topk_grouped": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _vp], _i32),
    # softmax attention with score modifiers and visibility rules (masked_attention.cu)
    "pa_masked_attention_tile_tokens": ([_i32, _i32], _i32),
    "pa_masked_attention_mma_tile_tokens": ([_i32, _i32, _i32], _i32),
    "pa_masked_attention": ([_vp, _i64, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _i32,
                             _f32, _f32, _i32, _i32, _i32, _vp, _i32, _vp, _i32, _i32, _vp], _i32),
    # matrix-state recurrences (recurrence_ops.cu)
    "pa_causal_conv_silu": ([_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _vp], _i32),
    "pa_conv_state_update": ([_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _vp, _i32, _vp], _i32),
    "pa_decay_scan_workspace_bytes": ([_i32, _i32, _i32, _i32], _sz),
    "pa_decay_scan": ([_vp, _i64, _i32, _vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _i32,
                       _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _sz, _i32, _vp], _i32),
    "pa_gated_rms_norm": ([_vp, _i64, _i32, _i32, _vp, _i64, _i32, _i32, _vp, _f32, _vp, _i32, _vp], _i32),
    # sink / temperature / kept first positions / turned values; two-norm parallel wiring; polynomial activation
    "pa_masked_attention_sink": ([_vp, _i64, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _i32,
                                  _f32, _f32, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp], _i32),
    "pa_rope_kv_append": ([_vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32,
                           _i32, _i32, _vp, _vp, _i32, _i32, _vp], _i32),
    "pa_residual_add_norm2": ([_vp, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _f32, _vp, _vp, _vp, _vp, _i32,
                               _vp], _i32),
    "pa_poly_norm": ([_vp, _i64, _i32, _vp, _f32, _vp, _i32, _vp], _i32),
    "pa_logit_softcap": ([_vp, _i64, _f32, _f32, _vp], _i32),
    "pa_router_topk_biased": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32,
                               _vp], _i32),
    "pa_causal_conv": ([_vp, _i64, _i32, _i32, _i32, _vp, _vp, _i32, _vp, _vp, _i32, _vp, _i64, _i32, _vp], _i32),
}

EXPORTS = tuple(_SIGS)


class PAError(RuntimeError):
    """A non-zero status from libpa_b200.so (mirrors the reference's C++ exception ->
    pybind11 -> RuntimeError path)."""


def _missing(name, path):
    def fn(*_a, **_k):
        raise PAError(f"{name} is not in {os.path.basename(path)} (the core build); build the full library with "
                      f"`python build.py` in {_PKG}")
    return fn


def lib():
    """The loaded library: libpa_b200.so, or, where only the core subset was built (build.py --core), that one --
    entry points it does not hold raise PAError when called."""
    global _lib
    if _lib is None:
        path = LIB_PATH if os.path.exists(LIB_PATH) else CORE_LIB_PATH
        if not os.path.exists(path):
            raise PAError(
                f"{LIB_PATH} is missing: build it with `python build.py` in {_PKG} "
                "(there is no CPU or PyTorch fallback for this path)")
        handle = C.CDLL(path)
        for name, (args, res) in _SIGS.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                if path == LIB_PATH:
                    raise  # the header and the full .so disagree
                setattr(handle, name, _missing(name, path))
                continue
            fn.argtypes = args
            fn.restype = res
        _lib = handle
    return _lib


def check(status, what=""):
    if status != PA_OK:
        msg = lib().pa_error_string(status).decode()
        raise PAError(f"{what or 'pa_b200'} failed: {msg} (status {status})")


def ptr(t):
    """Device (or host) pointer of a torch tensor / None."""
    if t is None:
        return None
    return t.data_ptr()


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def device_info():
    sm, maj, mnr = _i32(), _i32(), _i32()
    check(lib().pa_device_info(C.byref(sm), C.byref(maj), C.byref(mnr)), "pa_device_info")
    return sm.value, maj.value, mnr.value
