"""B200 kernels behind the ``lite_llama.kernels`` names
(reference export list: lite_llama/kernels/__init__.py:22-39).

Every callable keeps the reference's signature and argument meaning; all of them launch
hand-written sm_100a CUDA from ``libb200lite.so`` on the current CUDA stream.
"""

from .flashattention2_nopad import flash_attention2_no_pad
from .flashdecoding import flash_decoding
from .fused_moe import fused_moe, grouped_experts, moe_align_block_size, route_sigmoid_groups, route_topk
from .gated_linear import gated_linear_scan, head_mix, head_norm_gate, swiglu_scaled
from .latent import head_linear, latent_prepare, rope_heads, rope_table
from .linear import linear, linear_simt
from .parallel_stream import branch_sum_residual, depth_mix_norms, embed_rmsnorm, gelu_mul_gather
from .rotary_heads import head_norm_rope_prepare, rope_table_freqs, rotary_frequencies
from .residual_stream import embed_positions, gelu, post_norm_residual, relu_squared, rmsnorm_from_f32, softcap_to_f32
from .sink_attention import MIXED_HEAD_MAX_KEYS, attn_prepare, mixed_head_attention, sink_attention
from .ssm import causal_conv_silu, decay_attention, gated_group_norm, gated_scan, norm_sigmoid_gate, ssm_scan
from .rope_emb import rope_emb_forward, rope_emb_inplace, rope_kv_write
from .sampling import argmax_rows
from .skip_rmsnorm import can_fuse_int8_quant, skip_rmsnorm, skip_rmsnorm_quant_int8
from .swiglu import swiglu_forward
from .update_kv_buffer import update_kv_buffer, update_kv_buffer_split
from .update_kv_index import update_kv_index
from .quantization import PackedW4, quantize_activations_int8, smoothquant_matmul, smoothquant_matmul_prequant, w4a16_matmul, w4a16_matmul_packed, w4a16_pack, w8a16_matmul

__all__ = [
    "flash_attention2_no_pad",
    "flash_decoding",
    "fused_moe",
    "moe_align_block_size",
    "route_topk",
    "route_sigmoid_groups",
    "gated_linear_scan",
    "head_norm_gate",
    "head_mix",
    "swiglu_scaled",
    "grouped_experts",
    "head_linear",
    "latent_prepare",
    "rope_heads",
    "rope_table",
    "gelu",
    "softcap_to_f32",
    "linear",
    "linear_simt",
    "embed_positions",
    "post_norm_residual",
    "rmsnorm_from_f32",
    "relu_squared",
    "attn_prepare",
    "sink_attention",
    "mixed_head_attention",
    "MIXED_HEAD_MAX_KEYS",
    "causal_conv_silu",
    "ssm_scan",
    "gated_group_norm",
    "gated_scan",
    "decay_attention",
    "norm_sigmoid_gate",
    "embed_rmsnorm",
    "depth_mix_norms",
    "branch_sum_residual",
    "gelu_mul_gather",
    "rope_table_freqs",
    "rotary_frequencies",
    "head_norm_rope_prepare",
    "argmax_rows",
    "rope_emb_forward",
    "rope_emb_inplace",
    "rope_kv_write",
    "skip_rmsnorm",
    "skip_rmsnorm_quant_int8",
    "can_fuse_int8_quant",
    "swiglu_forward",
    "update_kv_buffer",
    "update_kv_buffer_split",
    "update_kv_index",
    "w4a16_matmul",
    "w8a16_matmul",
    "smoothquant_matmul",
    "smoothquant_matmul_prequant",
    "quantize_activations_int8",
    "w4a16_pack",
    "w4a16_matmul_packed",
    "PackedW4",
]
