"""Python faces of the CUDA kernels. Each function checks its tensors, allocates the output
and launches on the current stream. float32 tensors run the true 32-bit kernels, bfloat16
tensors the serving kernels; nothing here computes on the CPU."""

from atomserve_b200.ops.attention import attention_tile_shape, paged_attention
from atomserve_b200.ops.elementwise import (
    embedding,
    partial_add_rms_norm,
    partial_add_rms_norm_fusable,
    qk_norm_rope_store,
    qk_norm_rope_store_takes_partial,
    rms_norm,
    rotary,
    silu_mul,
)
from atomserve_b200.ops.experts import combine, experts_down, experts_glu, group_by_expert, route
from atomserve_b200.ops.latent import head_matmul, head_matmul_on_tensor_cores, latent_attention, latent_prepare
from atomserve_b200.ops.library import KernelLibraryError, require_device
from atomserve_b200.ops.outnorm import capped_gates_scan, gated_token_slice, head_norm_gate, projection_norm_store, residual_out_norm
from atomserve_b200.ops.parallel_block import concat_cast, pair_embedding, residual_dual_norm
from atomserve_b200.ops.prepare import differential_combine, qk_prepare_store
from atomserve_b200.ops.recurrent import lightning_attention, linear_recurrence, plan_segments, rotary_table
from atomserve_b200.ops.linear import PartialSums, interleave_gate_up, linear, linear_glu, linear_partial, linear_relu2, linear_swiglu, swiglu_fusable
from atomserve_b200.ops.sandwich import add_normed, bias_glu, softcap_
from atomserve_b200.ops.ssm import conv_state_update, conv_steps, gate_group_norm
from atomserve_b200.ops.sampling import argmax_rows, presence_penalty, sample_rows
from atomserve_b200.ops.status import DeviceStatus, status_for
from atomserve_b200.ops.stream import activation, cast_rows, clamped_glu, embedding_scaled, gated_rms_norm, gelu, linear_for_stream, scaled_add_rms_norm

__all__ = [
    "concat_cast", "pair_embedding", "residual_dual_norm", "differential_combine", "qk_prepare_store",
    "add_normed", "bias_glu", "softcap_", "conv_state_update", "conv_steps", "gate_group_norm",
    "activation", "capped_gates_scan", "gated_token_slice", "head_norm_gate", "linear_recurrence", "projection_norm_store", "rotary_table",
    "residual_out_norm",
    "cast_rows", "clamped_glu", "combine", "embedding_scaled", "experts_down", "experts_glu", "gated_rms_norm", "gelu",
    "group_by_expert", "linear_for_stream", "head_matmul", "head_matmul_on_tensor_cores", "latent_attention", "latent_prepare", "lightning_attention", "plan_segments", "route",
    "scaled_add_rms_norm",
    "DeviceStatus",
    "KernelLibraryError",
    "PartialSums",
    "argmax_rows",
    "attention_tile_shape",
    "embedding",
    "interleave_gate_up",
    "linear",
    "linear_partial",
    "linear_glu",
    "linear_relu2",
    "linear_swiglu",
    "paged_attention",
    "partial_add_rms_norm",
    "partial_add_rms_norm_fusable",
    "presence_penalty",
    "qk_norm_rope_store",
    "qk_norm_rope_store_takes_partial",
    "require_device",
    "rms_norm",
    "rotary",
    "sample_rows",
    "silu_mul",
    "status_for",
    "swiglu_fusable",
]
