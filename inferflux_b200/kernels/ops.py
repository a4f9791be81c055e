"""Python entry points of the hand-written CUDA kernels.

Each function takes torch tensors that already live on the GPU, checks what
the kernel cannot check itself, and launches on torch's current stream through
the C interface of the kernel library.  There is no other implementation
behind these functions: a tensor that is not on a CUDA device, or a library
that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

#: kernels of this library launched since import (library matrix products are not counted)
launch_count = 0

_ERRORS = {100001: "unsupported size or element type", 100002: "misaligned pointer or stride"}


class KernelError(RuntimeError):
    pass


_sigs_done = False


def _lib():
    global _sigs_done
    lib = library()
    if not _sigs_done:
        lib.ifx_embed_gather.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        lib.ifx_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_float, c_void_p,
                                        c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_swiglu.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_convert.argtypes = [c_void_p, c_int, c_void_p, c_int, c_ll, c_void_p]
        lib.ifx_rope_table.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_double, c_void_p]
        lib.ifx_qkv_rope_kv_write.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                              c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                              c_int, c_void_p]
        lib.ifx_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_void_p]
        lib.ifx_attn_paged_generic.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int,
                                               c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.ifx_attn_prefill_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.ifx_attn_decode_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                             c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
        lib.ifx_attn_decode_prep_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_attn_decode_prep_bf16.restype = c_int
        lib.ifx_attn_decode_even_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int,
                                                  c_void_p, c_void_p]
        lib.ifx_attn_decode_even_bf16.restype = c_int
        lib.ifx_attn_decode_even_pieces.argtypes = [c_int, c_int, c_int, c_int]
        lib.ifx_attn_decode_even_pieces.restype = c_int
        lib.ifx_gemv_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll,
                                      c_int, c_int, c_void_p]
        lib.ifx_gemm_umma.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p]
        lib.ifx_gemm_umma.restype = c_int
        lib.ifx_gemm_umma_skinny.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int,
                                             c_void_p, c_void_p]
        lib.ifx_gemm_umma_skinny.restype = c_int
        lib.ifx_gemm_umma_qkv.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.ifx_gemm_umma_qkv.restype = c_int
        lib.ifx_gemm_umma_skinny_parts.argtypes = [c_int, c_int]
        lib.ifx_gemm_umma_skinny_parts.restype = c_int
        lib.ifx_gemv_bf16_plan.argtypes = [c_int, c_int, c_int]
        lib.ifx_gemv_bf16_plan.restype = c_int
        lib.ifx_attn_decode_plan.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.ifx_attn_decode_plan.restype = c_int
        lib.ifx_attn_prefill_umma.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_attn_prefill_umma_plan.argtypes = [c_int, c_int, c_int]
        lib.ifx_attn_prefill_umma_plan.restype = c_int
        lib.ifx_argmax.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.ifx_apply_penalties.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                            c_void_p, c_int, c_int, c_void_p]
        lib.ifx_apply_penalties_ring.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_apply_penalties_ring.restype = c_int
        lib.ifx_ring_append.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.ifx_ring_append.restype = c_int
        lib.ifx_sample.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_void_p]
        for name in ("ifx_embed_gather", "ifx_add_rmsnorm", "ifx_swiglu", "ifx_convert", "ifx_rope_table",
                     "ifx_qkv_rope_kv_write", "ifx_gemm_f32", "ifx_attn_paged_generic", "ifx_argmax",
                     "ifx_attn_prefill_bf16", "ifx_attn_decode_bf16", "ifx_gemv_bf16", "ifx_attn_prefill_umma",
                     "ifx_apply_penalties", "ifx_sample"):
            getattr(lib, name).restype = c_int
        c_double = ctypes.c_double
        lib.ifx_add_layernorm.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_float, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_add_layernorm_shift1.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_float, c_void_p,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_token_shift.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_void_p]
        lib.ifx_embed_sinusoid_layernorm.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_double,
                                                     c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_polynorm.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_float, c_void_p, c_ll, c_int, c_int, c_int, c_void_p]
        lib.ifx_mingru_segment.argtypes = []
        lib.ifx_mingru_scan.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.ifx_latent_prep.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p,
                                        c_void_p, c_int, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p]
        lib.ifx_attn_latent_paged.argtypes = [c_void_p, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p, c_int, c_ll, c_int,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_int, c_int, c_float, c_void_p]
        lib.ifx_attn_latent_mma.argtypes = [c_void_p, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p, c_ll, c_int, c_void_p, c_int,
                                            c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_float, c_int, c_void_p, c_void_p, c_void_p]
        lib.ifx_attn_latent_mma_plan.argtypes = [c_int, c_int, c_int, c_int]
        lib.ifx_attn_latent_mma_max_rank.argtypes = []
        lib.ifx_add_into.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_void_p]
        lib.ifx_add_rows_vector.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_gate_heads.argtypes = [c_void_p, c_int, c_ll, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, c_int, c_void_p]
        lib.ifx_gather_latents.argtypes = [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_int, c_void_p]
        c_dbl = ctypes.c_double
        lib.ifx_norm_chain.argtypes = [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_ll, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]
        lib.ifx_conv_rope_kv_write.argtypes = [c_void_p, c_int, c_ll, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                               c_ll, c_int, c_void_p]
        lib.ifx_rotate_heads.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_attn_paged_generic_ex.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int,
                                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                  c_void_p, c_int, c_int, c_int, c_float, c_int,
                                                  c_int, c_float, c_int, c_int, c_void_p, c_int, c_ll, c_int, c_int, c_void_p]
        lib.ifx_attn_prefill_bf16_ex.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                                 c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                 c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_int, c_int,
                                                 c_void_p, c_int, c_ll, c_int, c_void_p]
        lib.ifx_attn_prefill_bf16_ex.restype = c_int
        lib.ifx_retention_segment.argtypes = []
        lib.ifx_retention_scan.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
                                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.ifx_retention_finish.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_ll, c_int, c_int, c_int, c_float,
                                             c_void_p]
        lib.ifx_gelu_tanh.argtypes = [c_void_p, c_int, c_ll, c_void_p, c_int, c_ll, c_int, c_int, c_void_p]
        lib.ifx_moe_route.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]
        lib.ifx_moe_tile_rows.argtypes = [c_int]
        lib.ifx_moe_experts.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p]
        lib.ifx_moe_group.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.ifx_moe_gather_rows.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_gemm_umma_grouped.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p]
        lib.ifx_activation.argtypes = [c_void_p, c_ll, c_int, c_ll, c_void_p, c_int, c_ll, c_int, c_int, c_int, c_void_p]
        lib.ifx_causal_conv.argtypes = [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_void_p, c_ll, c_int, c_int, c_void_p]
        lib.ifx_ssm_scan.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p]
        lib.ifx_gated_group_norm.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_ll, c_int, c_int, c_int,
                                             c_float, c_void_p]
        lib.ifx_delta_rule_scan.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_ll, c_int, c_int, c_int,
                                            c_float, c_float, c_int, c_void_p, c_void_p]
        lib.ifx_head_norm_gate.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_ll, c_int, c_int, c_int,
                                           c_float, c_int, c_void_p]
        lib.ifx_qkv_norm_rope_write.argtypes = [c_void_p, c_int, c_ll, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]
        lib.ifx_add_group_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_ll, c_float, c_void_p, c_int, c_ll, c_float, c_int,
                                              c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_glu_clamped.argtypes = [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float,
                                        c_void_p]
        lib.ifx_gla_scan.argtypes = [c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_float, c_float, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_ll, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
        lib.ifx_gla_segment.argtypes = []
        lib.ifx_gla_segment.restype = c_int
        lib.ifx_attn_paged_generic_ex2.argtypes = list(lib.ifx_attn_paged_generic_ex.argtypes[:-1]) + [
            c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.ifx_attn_latent_paged_ex.argtypes = [c_void_p, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p, c_int, c_ll, c_int,
                                                 c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p]
        lib.ifx_latent_rope_prep.argtypes = [c_void_p, c_ll, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_int, c_ll, c_int, c_void_p, c_int,
                                             c_void_p]
        lib.ifx_attn_decode_bf16_ex.argtypes = list(lib.ifx_attn_decode_bf16.argtypes[:-1]) + [c_float, c_int, c_void_p, c_void_p, c_void_p]
        lib.ifx_attn_decode_bf16_ex.restype = c_int
        lib.ifx_attn_prefill_bf16_ex2.argtypes = list(lib.ifx_attn_prefill_bf16_ex.argtypes[:-1]) + [c_float, c_int, c_void_p, c_void_p, c_void_p]
        lib.ifx_attn_prefill_bf16_ex2.restype = c_int
        lib.ifx_attn_latent_mma_ex.argtypes = list(lib.ifx_attn_latent_mma.argtypes[:-1]) + [c_int, c_int, c_void_p, c_void_p]
        lib.ifx_attn_latent_mma_ex.restype = c_int
        for name in ("ifx_add_group_rmsnorm", "ifx_glu_clamped", "ifx_gla_scan", "ifx_attn_paged_generic_ex2",
                     "ifx_attn_latent_paged_ex", "ifx_latent_rope_prep"):
            getattr(lib, name).restype = c_int
        for name in ("ifx_activation", "ifx_causal_conv", "ifx_ssm_scan", "ifx_gated_group_norm", "ifx_delta_rule_scan",
                     "ifx_head_norm_gate", "ifx_qkv_norm_rope_write"):
            getattr(lib, name).restype = c_int
        for name in ("ifx_moe_group", "ifx_moe_gather_rows", "ifx_moe_combine", "ifx_gemm_umma_grouped"):
            getattr(lib, name).restype = c_int
        for name in ("ifx_norm_chain", "ifx_conv_rope_kv_write", "ifx_rotate_heads", "ifx_attn_paged_generic_ex",
                     "ifx_retention_segment", "ifx_retention_scan", "ifx_retention_finish", "ifx_gelu_tanh",
                     "ifx_moe_route", "ifx_moe_tile_rows", "ifx_moe_experts"):
            getattr(lib, name).restype = c_int
        for name in ("ifx_add_layernorm", "ifx_add_layernorm_shift1", "ifx_token_shift", "ifx_embed_sinusoid_layernorm",
                     "ifx_polynorm", "ifx_mingru_segment", "ifx_mingru_scan", "ifx_latent_prep", "ifx_attn_latent_paged", "ifx_gate_heads",
                     "ifx_add_into", "ifx_add_rows_vector", "ifx_attn_latent_mma", "ifx_attn_latent_mma_plan",
                     "ifx_attn_latent_mma_max_rank", "ifx_gather_latents"):
            getattr(lib, name).restype = c_int
        _sigs_done = True
    return lib


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        msg = _ERRORS.get(code)
        if msg is None:
            msg = f"CUDA error {code}"
            try:
                torch.cuda.synchronize()
            except RuntimeError as e:   # surfaces the sticky error text
                msg += f" ({e})"
        raise KernelError(f"{what}: {msg}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel operands must be CUDA tensors (there is no CPU path)")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]) * scale; ids int32 [N], out float32 [N, H]."""
    n, (vocab, hidden) = ids.numel(), table.shape
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32, "embed_gather: ids int32, out float32")
    _need(table.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n, hidden),
          "embed_gather: contiguous table and out [N, H]")
    _check(_lib().ifx_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), n, hidden, vocab, float(scale), _stream()),
           "embed_gather")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_partials: int = 1) -> Optional[torch.Tensor]:
    """residual (float32 [N, H]) += delta; out = RMSNorm(residual) * weight.

    With ``rows`` (int32 [R]) only those rows are normed into out [R, H] and
    the residual is left untouched.  ``delta`` may be None; with
    ``n_partials`` > 1 it is [P, N, H] float32 partial sums.  ``out`` may be
    None (only the sum is stored)."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: residual float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "add_rmsnorm: weight float32 [H]")
    n_rows = rows.numel() if rows is not None else n
    if rows is not None:
        _need(rows.dtype == torch.int32, "add_rmsnorm: rows int32")
    pstride = 0
    if delta is not None:
        _need(delta.is_contiguous(), "add_rmsnorm: delta contiguous")
        if n_partials > 1:
            _need(tuple(delta.shape) == (n_partials, n, hidden), "add_rmsnorm: partials [P, N, H]")
            pstride = n * hidden
        else:
            _need(tuple(delta.shape) == (n, hidden), "add_rmsnorm: delta [N, H]")
    if out is not None:
        _need(out.is_contiguous() and tuple(out.shape) == (n_rows, hidden), "add_rmsnorm: out [rows, H]")
    dd = _code(delta) if delta is not None else F32
    od = _code(out) if out is not None else F32
    _check(_lib().ifx_add_rmsnorm(_ptr(residual), _ptr(delta), dd, n_partials, pstride, _ptr(weight), float(eps),
                                  _ptr(out), od, _ptr(rows), n_rows, hidden, 0 if rows is not None else 1,
                                  _stream()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[m, i] = silu(gate_up[m, i]) * gate_up[m, I + i]."""
    m, two_i = gate_up.shape
    _need(two_i % 2 == 0 and tuple(out.shape) == (m, two_i // 2) and out.dtype == gate_up.dtype,
          "swiglu: gate_up [M, 2I], out [M, I] of the same type")
    _need(gate_up.is_contiguous() and out.is_contiguous(), "swiglu: contiguous operands")
    _check(_lib().ifx_swiglu(_ptr(gate_up), _ptr(out), _code(out), m, two_i // 2, _stream()), "swiglu")
    return out


def convert(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    _need(src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel(), "convert: same size, contiguous")
    _check(_lib().ifx_convert(_ptr(src), _code(src), _ptr(dst), _code(dst), src.numel(), _stream()), "convert")
    return dst


# ----------------------------------------------------------------------- rotary
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               magnitude: float = 1.0) -> None:
    """cos/sin [N, half] float32 of positions[t] * inv_freq[i] (inv_freq float64 [half]), both times ``magnitude``."""
    n, half = positions.numel(), inv_freq.numel()
    _need(positions.dtype == torch.int32 and inv_freq.dtype == torch.float64, "rope_table: int32 positions, float64 inv_freq")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
          and tuple(cos.shape) == (n, half) and tuple(sin.shape) == (n, half), "rope_table: cos/sin float32 [N, half]")
    _check(_lib().ifx_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), n, half, float(magnitude), _stream()),
           "rope_table")


def qkv_rope_kv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                      slot_map: Optional[torch.Tensor], k_layer: Optional[torch.Tensor],
                      v_layer: Optional[torch.Tensor], page_stride: int, page_size: int,
                      n_heads: int, n_kv: int, head_dim: int, partials: Optional[torch.Tensor] = None) -> None:
    """Bias add, rotate-half rotation of q (in place) and k, and the write of k
    and v into the paged cache at ``slot_map`` (page * page_size + offset).
    With ``partials`` (float32 [S, N, width], bfloat16 qkv, full rotation, head
    size a multiple of 16) the rows are the sums of the S slices instead of
    qkv's content, and qkv only receives the rotated q."""
    n, width = qkv.shape
    _need(qkv.is_contiguous() and width == (n_heads + 2 * n_kv) * head_dim, "qkv_rope_kv_write: qkv [N, (nh + 2 nkv) hd]")
    rot_dim = 2 * cos.shape[1]
    _need(tuple(cos.shape) == tuple(sin.shape) and cos.shape[0] == n and cos.dtype == torch.float32
          and cos.is_contiguous() and sin.is_contiguous(), "qkv_rope_kv_write: cos/sin float32 [N, rot/2]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "qkv_rope_kv_write: bias float32 [width]")
    if n_kv:
        _need(slot_map is not None and slot_map.dtype == torch.int32 and slot_map.numel() == n,
              "qkv_rope_kv_write: slot_map int32 [N]")
        _need(k_layer.dtype == qkv.dtype and v_layer.dtype == qkv.dtype, "qkv_rope_kv_write: cache of qkv's type")
    n_partials = 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 3
              and tuple(partials.shape[1:]) == (n, width) and qkv.dtype == torch.bfloat16
              and rot_dim == head_dim and head_dim % 16 == 0, "qkv_rope_kv_write: partial sums float32 [S, N, width]")
        n_partials = partials.shape[0]
    _check(_lib().ifx_qkv_rope_kv_write(_ptr(qkv), _code(qkv), _ptr(bias), _ptr(cos), _ptr(sin), rot_dim,
                                        _ptr(slot_map) if n_kv else None, _ptr(k_layer) if n_kv else None,
                                        _ptr(v_layer) if n_kv else None, page_stride, page_size, n, n_heads, n_kv,
                                        head_dim, _ptr(partials), n_partials, _stream()), "qkv_rope_kv_write")


# --------------------------------------------------------------- matrix product
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T + bias, all float32, plain FFMA."""
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32, "gemm_f32: float32")
    _need(w.shape[1] == k and w.is_contiguous() and tuple(out.shape) == (m, n), "gemm_f32: shapes")
    _need(a.stride(1) == 1 and out.stride(1) == 1, "gemm_f32: unit inner strides")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_f32: bias float32 [N]")
    _check(_lib().ifx_gemm_f32(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0) if m > 1 else k,
                               out.stride(0) if m > 1 else n, _stream()), "gemm_f32")
    return out


GEMV_MAX_ROWS = 16


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              swiglu: bool = False, k_splits: int = 1) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for M <= 16, bfloat16 operands,
    float32 accumulation, bfloat16 or float32 result.  With ``swiglu`` w is
    [2N, K] = [gate; up] and out = silu(x gate^T) * (x up^T).  With
    ``k_splits`` > 1 out is float32 [k_splits, M, N]: slice s is the sum over the
    s-th part of K and the caller adds the slices.  ``w`` is a parameter: the
    kernel starts to read it before the kernel launched before it has finished,
    so it must not be that kernel's output."""
    m, k = x.shape
    n = out.shape[-1]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous(), "gemv_bf16: bfloat16 operands")
    _need(w.shape == ((2 * n if swiglu else n), k), "gemv_bf16: shapes")
    _need(m <= GEMV_MAX_ROWS and k % 8 == 0, f"gemv_bf16: at most {GEMV_MAX_ROWS} rows and K a multiple of 8")
    if k_splits > 1:
        _need(tuple(out.shape) == (k_splits, m, n) and out.is_contiguous() and out.dtype == torch.float32
              and not swiglu, "gemv_bf16: partial sums are float32 [k_splits, M, N]")
        ldo = n
    else:
        _need(out.dim() == 2 and out.shape[0] == m and out.stride(1) == 1, "gemv_bf16: out [M, N]")
        ldo = out.stride(0) if m > 1 else n
    _need(x.stride(1) == 1, "gemv_bf16: unit inner strides")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n and not swiglu, "gemv_bf16: bias float32 [N]")
    _check(_lib().ifx_gemv_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), m, n, k,
                                x.stride(0) if m > 1 else k, ldo, 1 if swiglu else 0, int(k_splits),
                                _stream()), "gemv_bf16")
    return out


def gemm_umma(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              swiglu: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for many rows, on the tcgen05 tensor
    cores (TMA operands, accumulators in tensor memory), bfloat16 operands, float32
    accumulation, bfloat16 or float32 result.  With ``swiglu`` w is [2N, K] =
    [gate; up] and out = silu(x gate^T) * (x up^T), the activation applied in the
    product's epilogue.  Two SMs share each tile (cta_group::2).  A bounded wait
    that runs out sets the device's error flag (see :func:`check_device_errors`)."""
    m, k = x.shape
    n = out.shape[-1]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous(), "gemm_umma: bfloat16 operands")
    _need(w.shape == ((2 * n if swiglu else n), k), "gemm_umma: shapes")
    _need(out.dim() == 2 and out.shape[0] == m and out.stride(1) == 1 and x.stride(1) == 1,
          "gemm_umma: out [M, N], unit inner strides")
    _need(k % 8 == 0 and (m == 1 or x.stride(0) % 8 == 0), "gemm_umma: K and the row stride of x must be multiples of 8")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n and not swiglu, "gemm_umma: bias float32 [N]")
    _check(_lib().ifx_gemm_umma(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(bias), _ptr(out), out.stride(0),
                                _code(out), m, n, k, 1 if swiglu else 0, _ptr(error_flag(x.device)), _stream()),
           "gemm_umma")
    return out


QKV_EPILOGUE_HEAD_DIM = 128     # the head size gemm_umma_qkv is written for


def gemm_umma_qkv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, slot_map: Optional[torch.Tensor],
                  k_layer: Optional[torch.Tensor], v_layer: Optional[torch.Tensor], page_stride: int, page_size: int,
                  n_heads: int, n_kv: int) -> torch.Tensor:
    """The stacked q, k, v projection x[M, K] @ w[(nh + 2 nkv) * 128, K]^T of many
    rows on the tcgen05 tensor cores, with what stands between it and attention
    in its epilogue: bias, rotate-half rotation of the query and key heads
    (``cos``, ``sin`` float32 [M, 64]), the queries as bfloat16 into the first
    nh * 128 columns of ``q_out``'s rows, keys and values into the paged cache
    at ``slot_map`` (page * page_size + offset).  Head size 128 only."""
    m, k = x.shape
    hd = QKV_EPILOGUE_HEAD_DIM
    width = (n_heads + 2 * n_kv) * hd
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (width, k),
          "gemm_umma_qkv: bfloat16 x [M, K], w [(nh + 2 nkv) * 128, K]")
    _need(q_out.dtype == torch.bfloat16 and q_out.dim() == 2 and q_out.shape[0] == m and q_out.shape[1] >= n_heads * hd
          and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0, "gemm_umma_qkv: q_out bfloat16 [M, >= nh * 128]")
    _need(k % 8 == 0 and x.stride(1) == 1 and (m == 1 or x.stride(0) % 8 == 0),
          "gemm_umma_qkv: K and the row stride of x must be multiples of 8")
    _need(tuple(cos.shape) == (m, hd // 2) and tuple(sin.shape) == (m, hd // 2) and cos.dtype == torch.float32
          and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(),
          "gemm_umma_qkv: cos/sin float32 [M, 64]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "gemm_umma_qkv: bias float32 [width]")
    if n_kv:
        _need(slot_map is not None and slot_map.dtype == torch.int32 and slot_map.numel() == m
              and k_layer.dtype == torch.bfloat16 and v_layer.dtype == torch.bfloat16,
              "gemm_umma_qkv: slot_map int32 [M], bfloat16 cache")
    _check(_lib().ifx_gemm_umma_qkv(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(bias), _ptr(q_out), q_out.stride(0),
                                    _ptr(cos), _ptr(sin), _ptr(slot_map) if n_kv else None,
                                    _ptr(k_layer) if n_kv else None, _ptr(v_layer) if n_kv else None, page_stride,
                                    page_size, m, k, n_heads, n_kv, _ptr(error_flag(x.device)), _stream()), "gemm_umma_qkv")
    return q_out


SKINNY_MAX_ROWS = 256       # rows of x that gemm_umma_skinny takes


def gemm_umma_skinny_parts(n: int, k: int) -> int:
    """Into how many parts :func:`gemm_umma_skinny` cuts K for an [n, k] matrix."""
    key = ("skinny", n, k)
    if key not in _gemv_plans:
        s = int(_lib().ifx_gemm_umma_skinny_parts(n, k))
        if s < 1:
            raise KernelError(f"gemm_umma_skinny_parts: CUDA error {-s}")
        _gemv_plans[key] = s
    return _gemv_plans[key]


def gemm_umma_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Partial sums of x[M, K] @ w[N, K]^T for a few rows (up to
    SKINNY_MAX_ROWS), where the time goes to reading w once: out float32
    [S, M, N], S = ``gemm_umma_skinny_parts(N, K)`` parts of K, to be added by
    the consumer.  tcgen05 with the operands' places changed: 256 rows of w are
    the rows of a tile and the rows of x its columns."""
    m, k = x.shape
    s, m2, n = out.shape
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (n, k),
          "gemm_umma_skinny: bfloat16 x [M, K], w [N, K]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and m2 == m and 1 <= m <= SKINNY_MAX_ROWS
          and s == gemm_umma_skinny_parts(n, k), "gemm_umma_skinny: out float32 [parts, M, N]")
    _need(k % 8 == 0 and x.stride(1) == 1 and (m == 1 or x.stride(0) % 8 == 0),
          "gemm_umma_skinny: K and the row stride of x must be multiples of 8")
    _check(_lib().ifx_gemm_umma_skinny(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(out), n, m * n, m, n, k, s,
                                       _ptr(error_flag(x.device)), _stream()), "gemm_umma_skinny")
    return out


_gemv_plans = {}


def gemv_k_splits(n: int, k: int, max_splits: int = 8) -> int:
    """Into how many parts of K the weight-streaming kernel is best told to cut
    an [n, k] matrix when float32 partial sums are welcome: the kernel's own
    count of what keeps the GPU fullest.  It depends on the matrix only."""
    key = (n, k, max_splits)
    if key not in _gemv_plans:
        s = int(_lib().ifx_gemv_bf16_plan(n, k, max_splits))
        if s < 1:
            raise KernelError(f"gemv_k_splits: CUDA error {-s}")
        _gemv_plans[key] = s
    return _gemv_plans[key]


_sm_counts = {}


def sm_count(device) -> int:
    """SMs of the device (where a kernel's plan is made on the host)."""
    key = torch.device(device).index or 0
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _sm_counts[key]


_error_flags = {}


def error_flag(device) -> torch.Tensor:
    """The device word that kernels with bounded waits set when a wait runs out."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_device_errors(device) -> None:
    """Raise if a kernel reported that one of its bounded waits ran out (this
    reads one word back from the device, so it synchronises)."""
    key = torch.device(device).index or 0
    flag = _error_flags.get(key)
    if flag is not None:
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            if code == 2:
                raise KernelError("decode attention met a context longer than the bound its scratch was sized for; "
                                  "its output is invalid")
            raise KernelError("a kernel gave up waiting on a barrier (bounded wait ran out); its output is invalid")


def matmul_library(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T through the vendor library (cuBLAS via torch), bfloat16
    operands, float32 accumulation, bfloat16 or float32 result.  Stands where
    the reference calls cuBLAS (runtime/backends/cuda/native/cublas_gemm.cpp:84-102)."""
    _need(x.is_cuda and w.is_cuda, "matmul_library: CUDA tensors (there is no CPU path)")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "matmul_library: bfloat16 operands")
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


# -------------------------------------------------------------------- attention
def attn_paged_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                       v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                       tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                       entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                       n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> torch.Tensor:
    """Causal grouped-query attention of new tokens over the paged cache.

    q: first element of the query rows (row stride ``q_stride`` elements, heads
    contiguous); out [N, n_heads * head_dim]; query tiles of 16 tokens are
    listed by tile_entry / tile_q0."""
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1,
          "attn: block_tables int32 [R, B]")
    for t in (tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start):
        _need(t.dtype == torch.int32, "attn: int32 metadata")
    _need(out.is_contiguous() and out.dtype == q.dtype and k_layer.dtype == q.dtype, "attn: types")
    _need(1 <= head_dim <= 256, f"attention: head_dim {head_dim} is outside 1..256")
    _need(n_heads % n_kv == 0, "attention: n_heads must be a multiple of n_kv")
    _check(_lib().ifx_attn_paged_generic(_ptr(q), q_stride, _ptr(out), out.stride(0), _code(q), _ptr(k_layer),
                                         _ptr(v_layer), page_stride, page_size, _ptr(block_tables),
                                         block_tables.stride(0), _ptr(tile_entry), _ptr(tile_q0), n_tiles,
                                         _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_ctx_start),
                                         n_heads, n_kv, head_dim, float(scale), int(window), _stream()),
           "attn_paged_generic")
    return out


FAST_ATTENTION_HEAD_DIMS = (64, 128)


def attn_prefill_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                      v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> torch.Tensor:
    """Tensor-core attention of prompt portions over the paged cache (bfloat16,
    head_dim 64 or 128); query tiles of 64 tokens listed by tile_entry / tile_q0."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_prefill_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_prefill_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    _check(_lib().ifx_attn_prefill_bf16(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                        page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                        _ptr(tile_entry), _ptr(tile_q0), n_tiles, _ptr(entry_q_start),
                                        _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, n_kv, head_dim,
                                        float(scale), int(window), _stream()), "attn_prefill_bf16")
    return out


UMMA_ATTENTION_HEAD_DIM = 128
UMMA_ATTENTION_TILE = 256          # tokens per query tile of attn_prefill_umma


def attn_prefill_umma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                      v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                      n_splits: int = 1, tile_rows: int = 256) -> torch.Tensor:
    """Attention of prompt portions with tcgen05.mma and tensor-memory
    accumulators (bfloat16, head_dim 128); query tiles of ``tile_rows`` = 256 or
    128 tokens listed by tile_entry / tile_q0 (a block takes a tile and a head;
    with 128 the tile's key tiles are dealt out to both halves of the block:
    twice the blocks, for steps whose tiles of 256 would leave SMs idle).  With ``n_splits`` > 1 the keys of every tile are cut
    into that many parts (see :func:`attn_prefill_umma_splits`), merged by a
    second kernel.  A bounded wait that runs out sets the device error flag
    (see :func:`check_device_errors`)."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_prefill_umma: bfloat16 operands")
    _need(head_dim == UMMA_ATTENTION_HEAD_DIM, f"attn_prefill_umma: head_dim {head_dim} is not 128")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    # The kernel reads the cache through a TMA tensor map, which wants to know how many pages lie behind page 0:
    # as many as fit between the view's start and the end of the storage it is a view of.
    n_elems = k_layer.untyped_storage().nbytes() // k_layer.element_size()
    last = max(k_layer.storage_offset(), v_layer.storage_offset()) + n_kv * page_size * head_dim
    num_pages = (n_elems - last) // page_stride + 1 if n_elems >= last else 0
    _need(num_pages >= 1, "attn_prefill_umma: k_layer / v_layer are not views of page 0 of a paged pool")
    part_o = part_ml = None
    global launch_count
    if n_splits > 1:
        rows = n_tiles * n_heads * n_splits * UMMA_ATTENTION_TILE
        part_o = torch.empty(rows * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_prefill_umma(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                        page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                        _ptr(tile_entry), _ptr(tile_q0), n_tiles, _ptr(entry_q_start),
                                        _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, n_kv, head_dim,
                                        float(scale), int(window), _ptr(error_flag(q.device)), _ptr(part_o),
                                        _ptr(part_ml), int(n_splits), int(num_pages), int(tile_rows), _stream()),
           "attn_prefill_umma")
    return out


def attn_prefill_umma_splits(n_tiles: int, n_heads: int, max_keys: int) -> int:
    """Into how many parts :func:`attn_prefill_umma` is best told to cut the keys
    of its query tiles (the kernel's own count: 1 when the tiles fill the GPU)."""
    return max(1, int(_lib().ifx_attn_prefill_umma_plan(n_tiles, n_heads, (max_keys + 63) // 64)))


def attn_decode_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                     v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                     dec_entries: torch.Tensor, n_dec: int, entry_q_start: torch.Tensor,
                     entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor, part_o: Optional[torch.Tensor],
                     part_ml: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int, scale: float,
                     window: int, n_splits: int, q_temp=None, distance_toll=None) -> torch.Tensor:
    """Tensor-core attention of single decoded tokens (entries listed in
    dec_entries), the keys split ``n_splits`` ways and merged.  Scratch:
    part_o float32 [n_dec * n_heads * n_splits * head_dim], part_ml float32
    [n_dec * n_heads * n_splits * 2].  ``q_temp`` and ``distance_toll`` as in
    :func:`attn_paged_options`."""
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    r1, r2 = distance_toll if distance_toll else (None, None)
    for t in (r1, r2):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads), "attn: per-head numbers float32 [heads]")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_decode_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_dec * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.dtype == torch.float32
              and part_ml.numel() >= n_dec * n_heads * n_splits * 2, "attn_decode_bf16: scratch too small")
    global launch_count
    if n_splits > 1:
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_bf16_ex(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                          page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                          _ptr(dec_entries), n_dec, _ptr(entry_q_start), _ptr(entry_q_len),
                                          _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml), n_heads, n_kv, head_dim,
                                          float(scale), int(window), int(n_splits), coef, every, _ptr(r1), _ptr(r2),
                                          _stream()), "attn_decode_bf16")
    return out


def attn_decode_prep_bf16(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                          slot_map: Optional[torch.Tensor], partials: Optional[torch.Tensor], out: torch.Tensor,
                          k_layer: torch.Tensor, v_layer: torch.Tensor, page_stride: int, page_size: int,
                          block_tables: torch.Tensor, dec_entries: torch.Tensor, n_dec: int,
                          entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                          part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], n_heads: int, n_kv: int,
                          head_dim: int, scale: float, window: int, n_splits: int) -> torch.Tensor:
    """:func:`attn_decode_bf16` for a step of single tokens only, with the work
    of :func:`qkv_rope_kv_write` folded into the attention kernel: ``qkv`` is
    the product's output before bias and rotation (or ``partials``, float32
    [S, N, width], holds it as partial sums and qkv's content is not read);
    the kernel rotates its own query heads and writes the token's key and
    value into the cache (``slot_map`` None: the layer writes none) before it
    reads them.  Every row of qkv must be one of the decoded entries."""
    n, width = qkv.shape
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16
          and qkv.is_contiguous() and width == (n_heads + 2 * n_kv) * head_dim and n == n_dec,
          "attn_decode_prep_bf16: qkv bfloat16 [n_dec, (nh + 2 nkv) hd]")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_prep_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(tuple(cos.shape) == (n, head_dim // 2) and tuple(sin.shape) == (n, head_dim // 2) and cos.dtype == torch.float32
          and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(),
          "attn_decode_prep_bf16: cos/sin float32 [N, head_dim / 2]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "attn_decode_prep_bf16: bias float32 [width]")
    _need(slot_map is None or (slot_map.dtype == torch.int32 and slot_map.numel() == n), "attn_decode_prep_bf16: slot_map int32 [N]")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    n_partials = 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 3
              and tuple(partials.shape[1:]) == (n, width), "attn_decode_prep_bf16: partial sums float32 [S, N, width]")
        n_partials = partials.shape[0]
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_dec * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.dtype == torch.float32
              and part_ml.numel() >= n_dec * n_heads * n_splits * 2, "attn_decode_prep_bf16: scratch too small")
    global launch_count
    if n_splits > 1:
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_prep_bf16(_ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(k_layer),
                                            _ptr(v_layer), page_stride, page_size, _ptr(block_tables),
                                            block_tables.stride(0), _ptr(dec_entries), n_dec, _ptr(entry_q_start),
                                            _ptr(entry_q_len), _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml),
                                            n_heads, n_kv, head_dim, float(scale), int(window), int(n_splits),
                                            _ptr(bias), _ptr(cos), _ptr(sin), _ptr(slot_map), _ptr(partials),
                                            n_partials, n, _stream()), "attn_decode_prep_bf16")
    return out


_decode_plans = {}


def attn_decode_splits(n_dec: int, n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Into how many parts :func:`attn_decode_bf16` is best told to cut the keys
    (the kernel's own count: every block has a place on the GPU at once)."""
    key = (n_dec, n_heads, n_kv, head_dim, (max_keys + 63) // 64)
    if key not in _decode_plans:
        if len(_decode_plans) > 65536:
            _decode_plans.clear()
        s = int(_lib().ifx_attn_decode_plan(n_dec, n_heads, n_kv, head_dim, max_keys))
        if s < 1:
            raise KernelError(f"attn_decode_splits: CUDA error {-s}")
        _decode_plans[key] = s
    return _decode_plans[key]


DECODE_EVEN_MAX_ENTRIES = 1024        # single tokens per call of attn_decode_even_bf16


def attn_decode_pieces(n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Pieces per (entry, head) that :func:`attn_decode_even_bf16`'s scratch must
    have room for when no entry sees more than ``max_keys`` keys."""
    key = ("even", n_heads, n_kv, head_dim, (max_keys + 63) // 64)
    if key not in _decode_plans:
        if len(_decode_plans) > 65536:
            _decode_plans.clear()
        s = int(_lib().ifx_attn_decode_even_pieces(n_heads, n_kv, head_dim, max_keys))
        if s < 1:
            raise KernelError(f"attn_decode_pieces: CUDA error {-s}")
        _decode_plans[key] = s
    return _decode_plans[key]


def attn_decode_even_bf16(q: torch.Tensor, out: torch.Tensor, k_layer: torch.Tensor, v_layer: torch.Tensor,
                          page_stride: int, page_size: int, block_tables: torch.Tensor, dec_entries: torch.Tensor,
                          n_dec: int, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                          entry_ctx_start: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                          piece_count: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                          max_pieces: int) -> torch.Tensor:
    """Tensor-core attention of single decoded tokens (entries listed in
    dec_entries, at most DECODE_EVEN_MAX_ENTRIES) for steps whose contexts
    differ much in length: the 64-key tiles of all entries are shared out
    evenly over the blocks the GPU holds, so the longest context does not set
    the time; what several blocks share is merged by a second kernel.
    ``max_pieces`` from :func:`attn_decode_pieces`; scratch part_o float32
    [n_dec * n_heads * max_pieces * head_dim], part_ml float32 [... * 2],
    piece_count int32 [n_dec * n_heads].  A context beyond the bound that
    max_pieces was made for sets the device error flag."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_decode_even_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_even_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    _need(1 <= n_dec <= DECODE_EVEN_MAX_ENTRIES, f"attn_decode_even_bf16: 1 to {DECODE_EVEN_MAX_ENTRIES} entries")
    _need(part_o.dtype == torch.float32 and part_o.numel() >= n_dec * n_heads * max_pieces * head_dim
          and part_ml.dtype == torch.float32 and part_ml.numel() >= n_dec * n_heads * max_pieces * 2
          and piece_count.dtype == torch.int32 and piece_count.numel() >= n_dec * n_heads,
          "attn_decode_even_bf16: scratch too small")
    global launch_count
    launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_even_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                            page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                            _ptr(dec_entries), n_dec, _ptr(entry_q_start), _ptr(entry_q_len),
                                            _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml), _ptr(piece_count), n_heads,
                                            n_kv, head_dim, float(scale), int(window), int(max_pieces),
                                            _ptr(error_flag(q.device)), _stream()), "attn_decode_even_bf16")
    return out


# --------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = lowest index of the maximum of logits[r, :] (float32 [R, V])."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= r,
          "argmax: float32 logits, int32 out")
    # a wide row is cut into slices with a block each (then a second launch picks among them)
    parts = min(64, v // 2048) if r <= 65535 else 1
    part = None
    global launch_count
    if parts > 1:
        part = torch.empty((r, parts, 2), dtype=torch.int32, device=logits.device)
        launch_count += 1
    _check(_lib().ifx_argmax(_ptr(logits), logits.stride(0), _ptr(out), r, v, _ptr(part), parts, _stream()), "argmax")
    return out


def apply_penalties(logits: torch.Tensor, recent_ids: torch.Tensor, recent_counts: torch.Tensor,
                    n_recent: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "penalties: float32 logits")
    _need(recent_ids.dtype == torch.int32 and recent_counts.dtype == torch.int32 and n_recent.dtype == torch.int32
          and recent_ids.is_contiguous() and recent_counts.is_contiguous() and recent_ids.shape[0] == r
          and recent_ids.shape == recent_counts.shape, "penalties: int32 [R, W] ids and counts")
    for t in (rep, freq, pres):
        _need(t.dtype == torch.float32 and t.numel() == r, "penalties: float32 [R] parameters")
    _check(_lib().ifx_apply_penalties(_ptr(logits), logits.stride(0), _ptr(recent_ids), _ptr(recent_counts),
                                      _ptr(n_recent), recent_ids.shape[1], _ptr(rep), _ptr(freq), _ptr(pres), r, v,
                                      _stream()), "apply_penalties")


def apply_penalties_ring(logits: torch.Tensor, ring: torch.Tensor, totals: torch.Tensor, slots: torch.Tensor,
                         last_n: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    """The penalties of :func:`apply_penalties` over each row's latest tokens,
    read from rings on the device: ``ring`` int32 [n_slots, ring_size] holds a
    request's tokens in order of arrival, written round and round,
    ``totals[slot]`` how many were written in all; row r is the request in
    ``slots[r]`` (negative: leave the row alone) and counts its latest
    ``last_n[r]`` tokens (at most ring_size)."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "apply_penalties_ring: float32 logits")
    _need(ring.dtype == torch.int32 and ring.dim() == 2 and ring.is_contiguous() and totals.dtype == torch.int32
          and totals.numel() >= ring.shape[0], "apply_penalties_ring: ring int32 [slots, size], totals int32 [slots]")
    _need(slots.dtype == torch.int32 and slots.numel() >= r and last_n.dtype == torch.int32 and last_n.numel() >= r
          and all(t.dtype == torch.float32 and t.numel() >= r for t in (rep, freq, pres)),
          "apply_penalties_ring: one slot, window and penalty triple per row")
    _check(_lib().ifx_apply_penalties_ring(_ptr(logits), logits.stride(0), _ptr(ring), ring.shape[1], _ptr(totals),
                                           _ptr(slots), _ptr(last_n), _ptr(rep), _ptr(freq), _ptr(pres), r, v, _stream()),
           "apply_penalties_ring")


def ring_append(ring: torch.Tensor, totals: torch.Tensor, slots: torch.Tensor, ids: torch.Tensor) -> None:
    """ids[r] becomes the next token of the request in slots[r] (negative: skipped)."""
    _need(ring.dtype == torch.int32 and ring.dim() == 2 and ring.is_contiguous() and totals.dtype == torch.int32
          and slots.dtype == torch.int32 and ids.dtype == torch.int32 and slots.numel() >= ids.numel(),
          "ring_append: int32 operands")
    _check(_lib().ifx_ring_append(_ptr(ring), ring.shape[1], _ptr(totals), _ptr(slots), _ptr(ids), ids.numel(), _stream()),
           "ring_append")


def sample(logits: torch.Tensor, weights: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: torch.Tensor) -> torch.Tensor:
    """One token per row: argmax where temperature <= 0, else a draw from
    softmax(logits / T) restricted by top-k / top-p / min-p.  ``weights`` is
    float32 scratch of logits' shape; seeds / counters are int64 (read as
    unsigned)."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: float32 logits")
    _need(weights.dtype == torch.float32 and weights.is_contiguous() and weights.numel() >= r * v, "sample: scratch")
    _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and min_p.dtype == torch.float32
          and top_k.dtype == torch.int32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64
          and out.dtype == torch.int32, "sample: parameter types")
    _check(_lib().ifx_sample(_ptr(logits), logits.stride(0), _ptr(weights), _ptr(temperature), _ptr(top_k),
                             _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(counters), _ptr(out), r, v, _stream()),
           "sample")
    return out


# ------------------------------------- layer norm, token shift, sinusoidal embedding, PolyNorm, minGRU, latent attention
def add_layernorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None, n_partials: int = 1,
                  out32: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """residual (float32 [N, H]) += delta; out = (r - mean) / sqrt(var + eps) * weight.

    The arguments are those of :func:`add_rmsnorm`; ``out32`` (float32
    ``[rows, H]``) takes the normed rows unrounded beside ``out``."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_layernorm: residual float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "add_layernorm: weight float32 [H]")
    n_rows = rows.numel() if rows is not None else n
    if rows is not None:
        _need(rows.dtype == torch.int32, "add_layernorm: rows int32")
    pstride = 0
    if delta is not None:
        _need(delta.is_contiguous(), "add_layernorm: delta contiguous")
        if n_partials > 1:
            _need(tuple(delta.shape) == (n_partials, n, hidden), "add_layernorm: partials [P, N, H]")
            pstride = n * hidden
        else:
            _need(tuple(delta.shape)[-2:] == (n, hidden) and delta.numel() == n * hidden, "add_layernorm: delta [N, H]")
    for o in (out, out32):
        if o is not None:
            _need(o.is_contiguous() and tuple(o.shape) == (n_rows, hidden), "add_layernorm: out [rows, H]")
    if out32 is not None:
        _need(out32.dtype == torch.float32, "add_layernorm: out32 float32")
    dd = _code(delta) if delta is not None else F32
    od = _code(out) if out is not None else F32
    _check(_lib().ifx_add_layernorm(_ptr(residual), _ptr(delta), dd, n_partials, pstride, _ptr(weight), float(eps),
                                    _ptr(out), od, _ptr(out32), _ptr(rows), n_rows, hidden,
                                    0 if rows is not None else 1, _stream()), "add_layernorm")
    return out


def add_layernorm_shift1(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                         mu: torch.Tensor, state: torch.Tensor, entry_slot: torch.Tensor, out: torch.Tensor,
                         shifted: torch.Tensor, n_partials: int = 1) -> None:
    """A step of single tokens (row t is entry t): residual sum, layer norm,
    ``shifted = h + (state[slot] - h) * mu`` and ``state[slot] = h`` in one
    kernel.  state float32 [slots, H]."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_layernorm_shift1: residual float32 contiguous")
    _need(weight.dtype == torch.float32 and mu.dtype == torch.float32 and weight.numel() == hidden
          and mu.numel() == hidden, "add_layernorm_shift1: weight and mu float32 [H]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == hidden,
          "add_layernorm_shift1: state float32 [slots, H]")
    _need(entry_slot.dtype == torch.int32 and entry_slot.numel() >= n, "add_layernorm_shift1: one slot per row")
    pstride = 0
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() == n_partials * n * hidden, "add_layernorm_shift1: delta [P, N, H]")
        pstride = n * hidden if n_partials > 1 else 0
    for o in (out, shifted):
        _need(o.is_contiguous() and tuple(o.shape) == (n, hidden) and o.dtype == out.dtype, "add_layernorm_shift1: out [N, H]")
    _check(_lib().ifx_add_layernorm_shift1(_ptr(residual), _ptr(delta), _code(delta) if delta is not None else F32,
                                           n_partials, pstride, _ptr(weight), float(eps), _ptr(mu), _ptr(state),
                                           _ptr(entry_slot), _ptr(out), _ptr(shifted), _code(out), n, hidden, _stream()),
           "add_layernorm_shift1")


def token_shift(h32: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, row_entry: torch.Tensor,
                entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_slot: torch.Tensor,
                out: torch.Tensor) -> torch.Tensor:
    """out[t] = h32[t] + (before(t) - h32[t]) * mu, where before(t) is the row
    above within the same entry or, for an entry's first row, what its state
    slot holds; the slot then takes the entry's last row.  h32 float32 [N, H],
    state float32 [slots, H], row_entry int32 [N]."""
    n, hidden = h32.shape
    _need(h32.dtype == torch.float32 and h32.is_contiguous(), "token_shift: h32 float32 contiguous")
    _need(mu.dtype == torch.float32 and mu.numel() == hidden, "token_shift: mu float32 [H]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == hidden,
          "token_shift: state float32 [slots, H]")
    _need(out.is_contiguous() and tuple(out.shape) == (n, hidden), "token_shift: out [N, H]")
    for t in (row_entry, entry_q_start, entry_q_len, entry_slot):
        _need(t.dtype == torch.int32, "token_shift: int32 metadata")
    _check(_lib().ifx_token_shift(_ptr(h32), _ptr(mu), _ptr(state), _ptr(row_entry), _ptr(entry_q_start),
                                  _ptr(entry_q_len), _ptr(entry_slot), _ptr(out), _code(out), n, hidden, _stream()),
           "token_shift")
    return out


def embed_sinusoid_layernorm(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, weight: torch.Tensor,
                             eps: float, base: float, out: torch.Tensor) -> torch.Tensor:
    """out[t] = layer norm(table[ids[t]] + P(positions[t])) * weight with
    P[2i] = sin(pos * base^(-2i/H)), P[2i+1] = cos of the same angle; out float32 [N, H]."""
    n, (vocab, hidden) = ids.numel(), table.shape
    _need(ids.dtype == torch.int32 and positions.dtype == torch.int32 and positions.numel() == n,
          "embed_sinusoid_layernorm: ids and positions int32 [N]")
    _need(out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n, hidden),
          "embed_sinusoid_layernorm: contiguous table, out float32 [N, H]")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "embed_sinusoid_layernorm: weight float32 [H]")
    _check(_lib().ifx_embed_sinusoid_layernorm(_ptr(table), _code(table), _ptr(ids), _ptr(positions), _ptr(weight),
                                               float(eps), float(base), _ptr(out), n, hidden, vocab, _stream()),
           "embed_sinusoid_layernorm")
    return out


def polynorm(z: torch.Tensor, bias: Optional[torch.Tensor], coeff: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, z = z + bias first; N
    divides a row by its root mean square.  z float32 [M, F], coeff float32 [4]."""
    m, f = z.shape
    _need(z.dtype == torch.float32 and z.stride(1) == 1, "polynorm: z float32 with unit inner stride")
    _need(coeff.dtype == torch.float32 and coeff.numel() == 4, "polynorm: four float32 coefficients")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == f, "polynorm: bias float32 [F]")
    _need(out.stride(1) == 1 and tuple(out.shape) == (m, f), "polynorm: out [M, F] with unit inner stride")
    _check(_lib().ifx_polynorm(_ptr(z), z.stride(0), _ptr(bias), _ptr(coeff), float(eps), _ptr(out), out.stride(0), _code(out), m, f,
                               _stream()), "polynorm")
    return out


def mingru_segment() -> int:
    """Tokens per segment of the minGRU scan."""
    return int(_lib().ifx_mingru_segment())


def mingru_scan(proj: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, out: torch.Tensor, seg_entry: torch.Tensor, seg_t0: torch.Tensor,
                n_segments: int, entry_first_seg: torch.Tensor, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                entry_slot: torch.Tensor, n_entries: int, multi: bool) -> torch.Tensor:
    """The minGRU recurrence over a step: proj float32 [N, 3W] = the stacked
    projections [z | x | g] of every token (bias float32 [2W]: the biases of z
    and x, added here), state float32 [slots, W] (read at
    an entry's first token, written after its last), out [N, W] =
    S_t * silu(g_t)."""
    n, w3 = proj.shape
    width = w3 // 3
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and w3 == 3 * width, "mingru_scan: proj float32 [N, 3W]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width,
          "mingru_scan: state float32 [slots, W]")
    _need(out.stride(1) == 1 and tuple(out.shape) == (n, width), "mingru_scan: out [N, W] with unit inner stride")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * width, "mingru_scan: bias float32 [2W]")
    for t in (seg_entry, seg_t0, entry_first_seg, entry_q_start, entry_q_len, entry_slot):
        _need(t.dtype == torch.int32, "mingru_scan: int32 metadata")
    scratch = torch.empty(3 * n_segments * width, dtype=torch.float32, device=proj.device) if multi else None
    _check(_lib().ifx_mingru_scan(_ptr(proj), _ptr(bias), _ptr(state), _ptr(out), out.stride(0), _code(out), _ptr(seg_entry), _ptr(seg_t0), n_segments,
                                  _ptr(entry_first_seg), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_slot),
                                  n_entries, width, 1 if multi else 0, _ptr(scratch), _stream()), "mingru_scan")
    return out


def latent_prep(p: torch.Tensor, wq: torch.Tensor, wkv: torch.Tensor, eps: float, q_rank: int, kv_rank: int, n_heads: int,
                cq: torch.Tensor, cache: torch.Tensor, page_stride: int, page_size: int, slot_map: torch.Tensor,
                gate: torch.Tensor) -> None:
    """From a token's stacked down projections p = [query latent | key/value
    latent | gates] (float32): cq = unit-rms(query latent) * wq, the key/value
    latent likewise with wkv into the token's place in the paged cache, gate =
    sigmoid(gates) float32 [N, heads].  cache: the run's latent stream of page 0."""
    n = p.shape[0]
    _need(p.dtype == torch.float32 and p.stride(1) == 1 and p.shape[1] == q_rank + kv_rank + n_heads,
          "latent_prep: p float32 [N, q_rank + kv_rank + heads]")
    _need(wq.dtype == torch.float32 and wq.numel() == q_rank and wkv.dtype == torch.float32 and wkv.numel() == kv_rank,
          "latent_prep: norm weights float32")
    _need(cq.is_contiguous() and tuple(cq.shape) == (n, q_rank) and cq.dtype == cache.dtype, "latent_prep: cq [N, q_rank]")
    _need(gate.dtype == torch.float32 and gate.is_contiguous() and tuple(gate.shape) == (n, n_heads),
          "latent_prep: gate float32 [N, heads]")
    _need(slot_map.dtype == torch.int32 and slot_map.numel() >= n, "latent_prep: slot_map int32 [N]")
    _check(_lib().ifx_latent_prep(_ptr(p), p.stride(0), _ptr(wq), _ptr(wkv), float(eps), q_rank, kv_rank, n_heads,
                                  _ptr(cq), _ptr(cache), _code(cache), page_stride, page_size, _ptr(slot_map), _ptr(gate),
                                  n, _stream()), "latent_prep")


def _head_layout(t: torch.Tensor, n_heads: int, width: int, what: str):
    """(row stride, head stride) of a ``[N, heads, width]`` view whose vectors are contiguous."""
    _need(t.dim() == 3 and t.shape[1] == n_heads and t.shape[2] == width and (t.stride(2) == 1 or width == 1),
          f"{what}: a [N, heads, width] view with contiguous vectors")
    return t.stride(0), t.stride(1)


def attn_latent_paged(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_stride: int, page_size: int,
                      block_tables: torch.Tensor, tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                      scale: float, window: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of new tokens over the cached latents, which serve as
    keys and as values: q float32 ``[N, heads, kw]`` (the queries moved into
    the latent space; any view whose vectors are contiguous), out ``[N, heads,
    rank]`` in the cache's type (the weighted sums of the latents).  A cached
    row is ``kw >= rank`` wide; what lies behind the latent (a rotated key part
    shared by the heads) enters the scores only.  ``window`` > 0 hides keys j
    <= p - window; ``sink`` float32 ``[heads]`` adds ``exp(sink[h])`` to the
    softmax's denominator.  Query tiles of 16 tokens are listed by tile_entry /
    tile_q0."""
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1,
          "attn_latent: block_tables int32 [R, B]")
    for t in (tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start):
        _need(t.dtype == torch.int32, "attn_latent: int32 metadata")
    _need(q.dtype == torch.float32 and out.dtype == cache.dtype and q.shape[:2] == out.shape[:2] and out.shape[2] <= q.shape[2],
          "attn_latent: q float32 [N, heads, kw], out [N, heads, rank <= kw] of the cache's type")
    n_heads, kw, rank = q.shape[1], q.shape[2], out.shape[2]
    _need(1 <= kw <= 1024, f"attn_latent: width {kw} is outside 1..1024")
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads), "attn_latent: sink float32 [heads]")
    (q_row, q_head), (o_row, o_head) = _head_layout(q, n_heads, kw, "attn_latent q"), _head_layout(out, n_heads, rank, "attn_latent out")
    _check(_lib().ifx_attn_latent_paged_ex(_ptr(q), q_row, q_head, _ptr(out), o_row, o_head, _ptr(cache), _code(cache),
                                           page_stride, page_size, _ptr(block_tables), block_tables.stride(0), _ptr(tile_entry),
                                           _ptr(tile_q0), n_tiles, _ptr(entry_q_start), _ptr(entry_q_len),
                                           _ptr(entry_ctx_start), n_heads, rank, kw, float(scale), int(window), _ptr(sink),
                                           _stream()), "attn_latent_paged")
    return out


def latent_rope_prep(p: torch.Tensor, wkv: torch.Tensor, eps: float, n_heads: int, dim: int, rot: int, kv_rank: int,
                     cos: torch.Tensor, sin: torch.Tensor, q_plain: torch.Tensor, q_rows: torch.Tensor, cache: torch.Tensor,
                     page_stride: int, page_size: int, slot_map: torch.Tensor) -> None:
    """p float32 ``[N, n_heads * (dim + rot) + kv_rank + rot]``: a token's query heads (``dim`` plain then ``rot``
    rotating columns each), its latent and its rotating key part.  ``q_plain [N, n_heads * dim]`` (the cache's type)
    takes the plain query parts; ``q_rows`` float32 ``[N, n_heads, kv_rank + rot]`` takes the rotated query parts in
    its last ``rot`` columns; the cache row of the token (``kv_rank + rot`` wide, at ``slot_map``) takes the latent
    divided by its root mean square times ``wkv`` and the rotated key part.  Neighbouring pairs ``(2i, 2i + 1)`` rotate
    by ``cos``/``sin`` float32 ``[N, rot / 2]``."""
    n = p.shape[0]
    _need(p.dtype == torch.float32 and p.stride(1) == 1 and p.shape[1] == n_heads * (dim + rot) + kv_rank + rot,
          "latent_rope_prep: p float32 [N, heads * (dim + rot) + kv_rank + rot]")
    _need(wkv.dtype == torch.float32 and wkv.is_contiguous() and wkv.numel() == kv_rank, "latent_rope_prep: wkv float32 [kv_rank]")
    _need(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
          and tuple(cos.shape) == (n, rot // 2), "latent_rope_prep: cos/sin float32 [N, rot / 2]")
    _need(q_plain.is_contiguous() and tuple(q_plain.shape) == (n, n_heads * dim) and q_plain.dtype == cache.dtype,
          "latent_rope_prep: q_plain [N, heads * dim] of the cache's type")
    _need(q_rows.dtype == torch.float32, "latent_rope_prep: q_rows float32")
    q_row, q_head = _head_layout(q_rows, n_heads, kv_rank + rot, "latent_rope_prep q_rows")
    _need(slot_map.dtype == torch.int32 and slot_map.numel() == n, "latent_rope_prep: slot_map int32 [N]")
    _check(_lib().ifx_latent_rope_prep(_ptr(p), p.stride(0), _ptr(wkv), float(eps), n_heads, dim, rot, kv_rank, _ptr(cos),
                                       _ptr(sin), _ptr(q_plain), _ptr(q_rows), q_row, q_head, _ptr(cache), _code(cache),
                                       page_stride, page_size, _ptr(slot_map), n, _stream()), "latent_rope_prep")


def gate_heads(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, row_entry: Optional[torch.Tensor] = None,
               entry_q_len: Optional[torch.Tensor] = None, prompt_rows: bool = False) -> torch.Tensor:
    """out[t, h * width + d] = x[t, h, d] * gate[t, h]: x ``[N, heads, width]``
    (any view whose vectors are contiguous), gate float32 [N, heads], out
    contiguous ``[N, heads * width]``.  With ``row_entry`` (the entry of every
    row) and ``entry_q_len`` only the rows of entries with more than one token
    (``prompt_rows``) or with exactly one are written."""
    n, n_heads, width = x.shape
    _need(gate is None or (gate.dtype == torch.float32 and gate.is_contiguous() and tuple(gate.shape) == (n, n_heads)),
          "gate_heads: gate float32 [N, heads] (or None: the heads are gathered and rounded as they are)")
    _need(out.stride(1) == 1 and tuple(out.shape) == (n, n_heads * width), "gate_heads: out [N, heads * width], unit inner stride")
    row, head = _head_layout(x, n_heads, width, "gate_heads x")
    _check(_lib().ifx_gate_heads(_ptr(x), _code(x), row, head, _ptr(gate), _ptr(out), out.stride(0), _code(out), n, n_heads, width,
                                 _ptr(row_entry), _ptr(entry_q_len), 1 if prompt_rows else 0, _stream()), "gate_heads")
    return out


def gather_latents(cache: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                   g_entry: torch.Tensor, g_pos: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[i] = the cached latent at position g_pos[i] of entry g_entry[i] (zeros
    where its page was given back).  cache: the run's latent stream of page 0."""
    n, rank = out.shape
    _need(out.is_contiguous() and out.dtype == cache.dtype and cache.shape[-1] == rank, "gather_latents: out [n, rank] of the cache's type")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1 and g_entry.dtype == torch.int32
          and g_pos.dtype == torch.int32 and g_entry.numel() >= n and g_pos.numel() >= n, "gather_latents: int32 metadata")
    _check(_lib().ifx_gather_latents(_ptr(cache), _code(cache), page_stride, page_size, rank, _ptr(block_tables),
                                     block_tables.stride(0), _ptr(g_entry), _ptr(g_pos), _ptr(out), n, _stream()),
           "gather_latents")
    return out


def add_into(residual: torch.Tensor, delta: torch.Tensor, n_partials: int = 1) -> torch.Tensor:
    """residual (float32 [N, H]) += delta, or the sum of its ``n_partials`` slices [P, N, H] in index order."""
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and delta.is_contiguous()
          and delta.numel() == n_partials * residual.numel(), "add_into: float32 contiguous residual, delta [P, N, H]")
    _check(_lib().ifx_add_into(_ptr(residual), _ptr(delta), _code(delta), n_partials, residual.numel(), residual.numel(),
                               _stream()), "add_into")
    return residual


def add_rows_vector(a: torch.Tensor, b: torch.Tensor, v: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = a[t, :] + b[t, :] + v[:], all float32; out may be a or b."""
    n, hidden = a.shape
    for t in (a, b, out):
        _need(t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == (n, hidden), "add_rows_vector: float32 [N, H]")
    _need(v.dtype == torch.float32 and v.is_contiguous() and v.numel() == hidden, "add_rows_vector: v float32 [H]")
    _check(_lib().ifx_add_rows_vector(_ptr(a), _ptr(b), _ptr(v), _ptr(out), n, hidden, _stream()), "add_rows_vector")
    return out


LATENT_MMA_TILES = (16, 32, 64)      # (token, head) rows per tile of the tensor-core latent attention kernel


def attn_latent_mma_ok(rank: int, cache: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes this cache: bfloat16, a rank that is a multiple of 8 and not too large."""
    return cache.dtype == torch.bfloat16 and rank % 8 == 0 and 8 <= rank <= int(_lib().ifx_attn_latent_mma_max_rank())


def attn_latent_mma_splits(n_tiles: int, bm: int, rank: int, max_keys: int) -> int:
    return int(_lib().ifx_attn_latent_mma_plan(n_tiles, bm, rank, max_keys))


def attn_latent_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_stride: int, page_size: int,
                    block_tables: torch.Tensor, tile_entry: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, bm: int,
                    entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor, scale: float,
                    n_splits: int = 1, window: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`attn_latent_paged` on the tensor cores, bfloat16 cache and result.
    A tile is ``bm`` (16, 32 or 64) consecutive (token, head) rows of one entry,
    counted token by token with the heads innermost; ``tile_row0`` is a tile's
    first row within its entry.  With ``n_splits`` > 1 every tile's keys are cut
    into that many parts, which a second kernel merges.  ``out`` may be narrower than ``q``
    (``[N, heads, vrank]``, a multiple of 8): a cached row is then as wide as ``q``, its first
    ``vrank`` columns are the latent, and the rest enters the scores only.  ``window`` and ``sink``
    as in :func:`attn_latent_paged`."""
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1,
          "attn_latent_mma: block_tables int32 [R, B]")
    for t in (tile_entry, tile_row0, entry_q_start, entry_q_len, entry_ctx_start):
        _need(t.dtype == torch.int32, "attn_latent_mma: int32 metadata")
    _need(q.dtype == torch.float32 and out.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
          and q.shape[:2] == out.shape[:2] and out.shape[2] <= q.shape[2], "attn_latent_mma: q float32, out and cache bfloat16")
    _need(bm in LATENT_MMA_TILES, "attn_latent_mma: tiles of 16, 32 or 64 rows")
    n_heads, rank, vrank = q.shape[1], q.shape[2], out.shape[2]
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads), "attn_latent_mma: sink float32 [heads]")
    (q_row, q_head), (o_row, o_head) = _head_layout(q, n_heads, rank, "attn_latent_mma q"), _head_layout(out, n_heads, vrank, "attn_latent_mma out")
    _need(o_row % 2 == 0 and o_head % 2 == 0, "attn_latent_mma: out vectors on 4-byte boundaries")
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty(n_tiles * n_splits * bm * rank, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_tiles * n_splits * bm * 2, dtype=torch.float32, device=q.device)
    _check(_lib().ifx_attn_latent_mma_ex(_ptr(q), q_row, q_head, _ptr(out), o_row, o_head, _ptr(cache), page_stride, page_size,
                                         _ptr(block_tables), block_tables.stride(0), _ptr(tile_entry), _ptr(tile_row0), n_tiles,
                                         bm, _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, rank,
                                         float(scale), n_splits, _ptr(part_o), _ptr(part_ml), vrank, int(window), _ptr(sink),
                                         _stream()), "attn_latent_mma")
    return out


# ------------------------------------------------- norm chains, convolution + rotation, retention, routed experts
def _slices(t: Optional[torch.Tensor], n: int, width: int, what: str):
    """(pointer, number of slices, elements between slices) of float32 sums given as [N, W] or [P, N, W]."""
    if t is None:
        return None, 0, 0
    _need(t.dtype == torch.float32 and t.is_contiguous(), f"{what}: float32 contiguous sums")
    if t.dim() == 3:
        _need(tuple(t.shape[1:]) == (n, width), f"{what}: slices [P, {n}, {width}], got {tuple(t.shape)}")
        return _ptr(t), t.shape[0], n * width
    _need(tuple(t.shape) == (n, width), f"{what}: [{n}, {width}], got {tuple(t.shape)}")
    return _ptr(t), 1, 0


def norm_chain(residual: torch.Tensor, a: Optional[torch.Tensor], eps: float, w_a: Optional[torch.Tensor] = None,
               b: Optional[torch.Tensor] = None, w_b: Optional[torch.Tensor] = None,
               w_post: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One pass over every row, float32: ``y = a`` (``N(a) * w_a`` with a weight), with ``b`` the mean of the two
    (normed) branches; ``y = N(y) * w_post`` with a weight; ``residual += y``; ``out = N(residual) * w_next``
    (without ``w_next``, ``out`` is the stream itself rounded into its type: for a sublayer that reads the stream as it is).
    ``N(v) = v / sqrt(mean(v^2) + eps)``.  ``a`` and ``b`` are float32 ``[N, H]`` or slices ``[P, N, H]`` that are
    added first.  With ``rows`` (int32) only those rows are computed, into ``out [R, H]``, and the residual is
    left as it is."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "norm_chain: residual float32 contiguous")
    for w in (w_a, w_b, w_post, w_next):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == hidden and w.is_contiguous()), "norm_chain: weights float32 [H]")
    n_rows = rows.numel() if rows is not None else n
    if rows is not None:
        _need(rows.dtype == torch.int32, "norm_chain: rows int32")
    ap, a_parts, a_stride = _slices(a, n, hidden, "norm_chain a")
    bp, b_parts, b_stride = _slices(b, n, hidden, "norm_chain b")
    if out is not None:
        _need(out.is_contiguous() and tuple(out.shape) == (n_rows, hidden), "norm_chain: out [rows, H]")
    _check(_lib().ifx_norm_chain(ap, a_parts, a_stride, _ptr(w_a), bp, b_parts, b_stride, _ptr(w_b), _ptr(w_post),
                                 _ptr(residual), _ptr(w_next), _ptr(out), _code(out) if out is not None else F32,
                                 _ptr(rows), n_rows, hidden, float(eps), _stream()), "norm_chain")
    return out


ROT_HALF, ROT_INTERLEAVED = 0, 1


def conv_rope_kv_write(proj: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int, tail: Optional[torch.Tensor],
                       row_entry: torch.Tensor, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                       entry_slot: torch.Tensor, n_entries: int, cos: torch.Tensor, sin: torch.Tensor, layout: int,
                       n_heads: int, n_kv: int, dim: int, vdim: int, q_out: torch.Tensor, slot_map: torch.Tensor,
                       k_layer: torch.Tensor, v_layer: torch.Tensor, page_stride: int, page_size: int) -> None:
    """The first ``(n_heads + n_kv) * dim + n_kv * vdim`` columns of the float32 projection ``proj [N, W]`` (or
    slices ``[P, N, W]``) are q, k and v heads side by side.  Every channel is convolved over time with its
    ``taps`` weights ``conv_w [channels, taps]`` (None = no convolution), reading the rows before the step's
    first from ``tail [slots, taps - 1, channels]``, which is then brought up to date; q and k heads are rotated
    by ``cos``/``sin`` ``[N, r/2]`` in pairs ``(i, i + r/2)`` (``ROT_HALF``) or ``(2i, 2i + 1)``
    (``ROT_INTERLEAVED``); q goes to ``q_out [N, n_heads * dim]``, k and v into the paged cache at ``slot_map``."""
    n = q_out.shape[0]
    channels = (n_heads + n_kv) * dim + n_kv * vdim
    width = proj.shape[-1]
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and width >= channels, "conv_rope: float32 projection")
    parts, pstride = (proj.shape[0], n * width) if proj.dim() == 3 else (1, 0)
    if conv_w is not None:
        _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and tuple(conv_w.shape) == (channels, taps),
              "conv_rope: conv weights float32 [channels, taps]")
        if taps > 1:
            _need(tail is not None and tail.dtype == torch.float32 and tail.is_contiguous()
                  and tuple(tail.shape[1:]) == (taps - 1, channels), "conv_rope: tail float32 [slots, taps - 1, channels]")
    _need(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
          and cos.shape[0] == n, "conv_rope: cos/sin float32 [N, r/2]")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (n, n_heads * dim) and k_layer.dtype == q_out.dtype,
          "conv_rope: q_out [N, heads * dim] of the cache's type")
    _check(_lib().ifx_conv_rope_kv_write(_ptr(proj), parts, pstride, width, _ptr(conv_w), int(taps), _ptr(tail),
                                         _ptr(row_entry), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_slot), n,
                                         n_entries, _ptr(cos), _ptr(sin), cos.shape[1], layout, n_heads, n_kv, dim, vdim,
                                         _ptr(q_out), _code(q_out), _ptr(slot_map), _ptr(k_layer), _ptr(v_layer),
                                         page_stride, page_size, _stream()), "conv_rope_kv_write")
    if conv_w is not None and taps > 1:
        global launch_count
        launch_count += 1


def rotate_heads(x: torch.Tensor, col0: int, n_rot_heads: int, dim: int, cos: torch.Tensor, sin: torch.Tensor,
                 layout: int) -> torch.Tensor:
    """Rotates, in place, ``n_rot_heads`` heads of width ``dim`` that start at column ``col0`` of the float32 rows
    ``x [N, W]``: the first ``2 * cos.shape[1]`` dimensions of each, paired by ``layout``."""
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1, "rotate_heads: float32 rows")
    _need(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
          and cos.shape[0] == x.shape[0], "rotate_heads: cos/sin float32 [N, r/2]")
    _need(col0 + n_rot_heads * dim <= x.shape[1], "rotate_heads: heads beyond the row")
    _check(_lib().ifx_rotate_heads(_ptr(x), x.stride(0), col0, n_rot_heads, dim, _ptr(cos), _ptr(sin), cos.shape[1], layout,
                                   x.shape[0], _stream()), "rotate_heads")
    return x


def attn_paged_options(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor, v_layer: torch.Tensor,
                       page_stride: int, page_size: int, block_tables: torch.Tensor, tile_entry: torch.Tensor,
                       tile_q0: torch.Tensor, n_tiles: int, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                       entry_ctx_start: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                       v_dim: int, softcap: float = 0.0, keep_first: int = 0, sink: bool = False,
                       gate: Optional[torch.Tensor] = None, single_tokens: bool = False, q_temp=None,
                       distance_toll=None, sink_value: Optional[torch.Tensor] = None) -> torch.Tensor:
    """With ``single_tokens`` every listed tile is one token (``tile_q0`` = its place in its entry) and the kernel
    for single tokens runs (a block a token and head, its warps sharing the keys out).  Otherwise
    :func:`attn_paged_generic` with values ``v_dim`` wide, a cap on the scores (``softcap * tanh(s / softcap)``,
    0 = none), ``keep_first`` first tokens that stay visible behind the window, a sink (one more term ``exp(0)`` in
    the denominator) and an output gate: ``gate`` = float32 ``[N, W]`` or ``[P, N, W]`` sums whose first
    ``n_heads * v_dim`` columns go through a sigmoid and multiply the result element by element.
    ``q_temp`` = ``(coef, every)``: the query at position p counts ``1 + coef * ln(floor((p + 1) / every) + 1)`` times;
    ``distance_toll`` = ``(r1, r2)``, float32 ``[n_heads]`` each: the score of key j loses ``r1 * ln(1 + r2 * (p - j))``
    (after the cap); ``sink_value`` float32 ``[n_heads]``: the sink's score per head instead of 0."""
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1,
          "attn: block_tables int32 [R, B]")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    r1, r2 = distance_toll if distance_toll else (None, None)
    for t in (r1, r2, sink_value):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads), "attn: per-head numbers float32 [heads]")
    _need(out.is_contiguous() and out.dtype == q.dtype and k_layer.dtype == q.dtype and out.shape[1] == n_heads * v_dim, "attn: types")
    gp, g_parts, g_pstride, g_stride = None, 0, 0, 0
    if gate is not None:
        _need(gate.dtype == torch.float32 and gate.stride(-1) == 1 and gate.shape[-1] >= n_heads * v_dim, "attn: gate float32 rows")
        gp = _ptr(gate)
        if gate.dim() == 3:
            g_parts, g_pstride, g_stride = gate.shape[0], gate.stride(0), gate.stride(1)
        else:
            g_parts, g_pstride, g_stride = 1, 0, gate.stride(0)
    _check(_lib().ifx_attn_paged_generic_ex2(_ptr(q), q_stride, _ptr(out), out.stride(0), _code(q), _ptr(k_layer),
                                            _ptr(v_layer), page_stride, page_size, _ptr(block_tables),
                                            block_tables.stride(0), _ptr(tile_entry), _ptr(tile_q0), n_tiles,
                                            _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_ctx_start),
                                            n_heads, n_kv, head_dim, float(scale), int(window), int(v_dim), float(softcap),
                                            int(keep_first), 1 if sink else 0, gp, g_parts, g_pstride, g_stride,
                                            1 if single_tokens else 0, coef, every, _ptr(r1), _ptr(r2), _ptr(sink_value),
                                            _stream()),
           "attn_paged_options")
    return out


def _gate_slices(gate: Optional[torch.Tensor], width: int, what: str):
    if gate is None:
        return None, 0, 0, 0
    _need(gate.dtype == torch.float32 and gate.stride(-1) == 1 and gate.shape[-1] >= width, f"{what}: gate float32 rows")
    if gate.dim() == 3:
        return _ptr(gate), gate.shape[0], gate.stride(0), gate.stride(1)
    return _ptr(gate), 1, 0, gate.stride(0)


def attn_prefill_options_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor, v_layer: torch.Tensor,
                              page_stride: int, page_size: int, block_tables: torch.Tensor, tile_entry: torch.Tensor,
                              tile_q0: torch.Tensor, n_tiles: int, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                              entry_ctx_start: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                              window: int, softcap: float = 0.0, keep_first: int = 0, sink: bool = False,
                              gate: Optional[torch.Tensor] = None, q_temp=None, distance_toll=None) -> torch.Tensor:
    """:func:`attn_prefill_bf16` (tensor cores, bfloat16, keys and values both ``head_dim`` = 64 or 128 wide, query
    tiles of 64 tokens) with the options of :func:`attn_paged_options` (all but the sink's own score)."""
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    r1, r2 = distance_toll if distance_toll else (None, None)
    for t in (r1, r2):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads), "attn: per-head numbers float32 [heads]")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_prefill_options_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_prefill_options_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    gp, g_parts, g_pstride, g_stride = _gate_slices(gate, n_heads * head_dim, "attn_prefill_options_bf16")
    _check(_lib().ifx_attn_prefill_bf16_ex2(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                           page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                           _ptr(tile_entry), _ptr(tile_q0), n_tiles, _ptr(entry_q_start),
                                           _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, n_kv, head_dim,
                                           float(scale), int(window), float(softcap), int(keep_first), 1 if sink else 0,
                                           gp, g_parts, g_pstride, g_stride, coef, every, _ptr(r1), _ptr(r2), _stream()),
           "attn_prefill_options_bf16")
    return out


def retention_segment() -> int:
    """Tokens per segment of the retention scan."""
    return int(_lib().ifx_retention_segment())


def retention_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, heads: int, dim: int, vdim: int,
                   decay: torch.Tensor, k_scale: float, state: torch.Tensor, seg_entry: torch.Tensor, seg_t0: torch.Tensor,
                   n_segments: int, entry_first_seg: torch.Tensor, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                   entry_slot: torch.Tensor, n_entries: int, multi: bool, out: torch.Tensor) -> torch.Tensor:
    """``S_t = decay_h S_{t-1} + (k_scale k_t) v_t^T``, ``o_t = S_t^T q_t`` per head over the step's entries, all
    float32.  ``proj`` float32 ``[N, W]`` holds q, k (already rotated) and v heads from the given columns on;
    ``state`` float32 ``[slots, heads, dim, vdim]``; ``out`` float32 ``[N, heads * vdim]``."""
    n = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.dim() == 2 and proj.stride(1) == 1, "retention: float32 projection rows")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "retention: state float32 [slots, heads, dim, vdim]")
    _need(decay.dtype == torch.float32 and decay.numel() == heads, "retention: decay float32 [heads]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (n, heads * vdim), "retention: out float32")
    seg_b = seg_start = None
    if multi:
        seg_b = torch.empty((n_segments, heads, dim, vdim), dtype=torch.float32, device=proj.device)
        seg_start = torch.empty_like(seg_b)
    _check(_lib().ifx_retention_scan(_ptr(proj), proj.stride(0), q_col, k_col, v_col, heads, dim, vdim, _ptr(decay),
                                     float(k_scale), _ptr(state), _ptr(seg_entry), _ptr(seg_t0), n_segments,
                                     _ptr(entry_first_seg), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_slot),
                                     n_entries, 1 if multi else 0, _ptr(seg_b), _ptr(seg_start), _ptr(out), _stream()),
           "retention_scan")
    if multi:
        global launch_count
        launch_count += 2
    return out


def retention_finish(o: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, heads: int, vdim: int, eps: float) -> torch.Tensor:
    """``out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * silu(gate[t, h])``: ``o`` float32 ``[N, heads * vdim]``,
    ``gate`` float32 rows (a view with any row stride), ``out`` rows of either type with any row stride."""
    n = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1
          and out.stride(1) == 1 and tuple(out.shape) == (n, heads * vdim), "retention_finish: operands")
    _check(_lib().ifx_retention_finish(_ptr(o), _ptr(gate), gate.stride(0), _ptr(out), _code(out), out.stride(0), n, heads,
                                       vdim, float(eps), _stream()), "retention_finish")
    return out


def gelu_tanh(z: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))`` of float32 sums ``z [M, C]`` or ``[P, M, C]``."""
    m, cols = out.shape
    zp, parts, pstride = _slices(z, m, cols, "gelu_tanh")
    _need(out.stride(1) == 1, "gelu_tanh: out rows")
    _check(_lib().ifx_gelu_tanh(zp, parts, pstride, _ptr(out), _code(out), out.stride(0), m, cols, _stream()), "gelu_tanh")
    return out


def moe_route(logits: torch.Tensor, top: int, over_all: bool = False, scale: float = 1.0):
    """The ``top`` largest of every row of float32 ``logits [N, E]`` (lowest index first among equals) and their
    weights: the softmax over the chosen logits alone, or, with ``over_all``, the softmax over every expert's
    logit with the chosen scores divided by their sum (+ 1e-20); either times ``scale``.  Returns (int32
    ``[N, top]``, float32 ``[N, top]``)."""
    n, experts = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "moe_route: float32 logits")
    _need(1 <= top <= min(64, experts), f"moe_route: top {top} must be within 1..min(64, experts)")
    chosen = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    _check(_lib().ifx_moe_route(_ptr(logits), n, experts, top, int(bool(over_all)), float(scale), _ptr(chosen),
                                _ptr(weights), _stream()), "moe_route")
    return chosen, weights


#: bfloat16 steps with at least this many (token, expert) pairs run the experts' products on the tcgen05 kernel
#: (row tiles of 256 of one expert each); fewer pairs, float32 and sizes that are no multiple of 8 take the FFMA tiles.
MOE_TENSOR_CORES = True
MOE_TENSOR_CORE_PAIRS = 512
MOE_UMMA_TILE = 256


def _moe_experts_umma(x, w_gate_up, w_down, chosen, weights, n, hidden, ff, experts, top, activation) -> torch.Tensor:
    lib, dev, tile = _lib(), x.device, MOE_UMMA_TILE
    pairs = n * top
    max_tiles = pairs // tile + experts
    rows = max_tiles * tile
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(rows, dtype=torch.int32, device=dev)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
    _check(lib.ifx_moe_group(_ptr(chosen), pairs, experts, tile, max_tiles, _ptr(tile_expert), _ptr(sorted_pair),
                             _ptr(pair_row), _stream()), "moe_group")
    xs = torch.empty((rows, hidden), dtype=x.dtype, device=dev)
    _check(lib.ifx_moe_gather_rows(_ptr(x), _code(x), _ptr(sorted_pair), _ptr(xs), rows, hidden, top, _stream()), "moe_gather_rows")
    act = torch.empty((rows, ff), dtype=x.dtype, device=dev)
    flag = error_flag(dev)
    _check(lib.ifx_gemm_umma_grouped(_ptr(xs), hidden, _ptr(w_gate_up), _ptr(act), ff, BF16, rows, ff, hidden, activation, experts,
                                     _ptr(tile_expert), _ptr(flag), _stream()), "gemm_umma_grouped (gate, up)")
    y = torch.empty((rows, hidden), dtype=torch.float32, device=dev)
    _check(lib.ifx_gemm_umma_grouped(_ptr(act), ff, _ptr(w_down), _ptr(y), hidden, F32, rows, hidden, ff, 0, experts,
                                     _ptr(tile_expert), _ptr(flag), _stream()), "gemm_umma_grouped (down)")
    out = torch.empty((n, hidden), dtype=torch.float32, device=dev)
    _check(lib.ifx_moe_combine(_ptr(y), _ptr(pair_row), _ptr(weights), _ptr(out), n, hidden, top, _stream()), "moe_combine")
    return out


MOE_SWIGLU, MOE_RELU2 = 1, 2


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, chosen: torch.Tensor,
                weights: torch.Tensor, activation: int = MOE_SWIGLU) -> torch.Tensor:
    """``out[t] = sum_k weights[t, k] * W_down[e] act_e(x_t)``, ``e = chosen[t, k]``.  ``MOE_SWIGLU``: ``w_gate_up
    [E, 2F, H]`` (gate rows, then up rows) and ``act = silu(W_gate x) * (W_up x)``; ``MOE_RELU2``: ``w_gate_up [E, F, H]``
    (up rows alone) and ``act = relu(W_up x)^2``.  ``x [N, H]``, ``w_down [E, H, F]`` of one type; float32 ``[N, H]``
    out.  The pairs are sorted by expert on the device and run as tiles of one expert each."""
    n, hidden = x.shape
    experts, up_rows, _ = w_gate_up.shape
    ff, top = (up_rows // 2 if activation == MOE_SWIGLU else up_rows), chosen.shape[1]
    _need(activation in (MOE_SWIGLU, MOE_RELU2), "moe_experts: activation")
    _need(x.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and x.dtype == w_gate_up.dtype == w_down.dtype,
          "moe_experts: contiguous operands of one type")
    _need(tuple(w_down.shape) == (experts, hidden, ff) and w_gate_up.shape[2] == hidden, "moe_experts: weight shapes")
    pairs = n * top
    if (MOE_TENSOR_CORES and x.dtype == torch.bfloat16 and pairs >= MOE_TENSOR_CORE_PAIRS and hidden % 8 == 0 and ff % 8 == 0):
        return _moe_experts_umma(x, w_gate_up, w_down, chosen, weights, n, hidden, ff, experts, top, activation)
    tile = int(_lib().ifx_moe_tile_rows(pairs))
    max_tiles = pairs // tile + experts
    dev = x.device
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(max_tiles * tile, dtype=torch.int32, device=dev)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
    act = torch.empty((max_tiles * tile, ff), dtype=x.dtype, device=dev)
    y = torch.empty((max_tiles * tile, hidden), dtype=torch.float32, device=dev)
    out = torch.empty((n, hidden), dtype=torch.float32, device=dev)
    _check(_lib().ifx_moe_experts(_ptr(x), _code(x), _ptr(w_gate_up), _ptr(w_down), _ptr(chosen), _ptr(weights), n, hidden, ff,
                                  experts, top, activation, tile, max_tiles, _ptr(tile_expert), _ptr(sorted_pair), _ptr(pair_row),
                                  _ptr(act), _ptr(y), _ptr(out), _stream()), "moe_experts")
    global launch_count
    launch_count += 3
    return out


# ------------------------------------------------- activations, state-space scan, delta rule, normed q/k/v
ACT_GELU, ACT_TANH, ACT_RELU2, ACT_SILU, ACT_SIGMOID = 0, 1, 2, 3, 4


def activation(z: torch.Tensor, out: torch.Tensor, act: int) -> torch.Tensor:
    """``out = act(z)`` element by element, computed in float32 and rounded once: ``z`` float32 rows ``[M, C]`` (a view
    with any row stride) or contiguous slices ``[P, M, C]`` that are added first; ``out`` rows of either type.
    ``act``: ``ACT_GELU`` (tanh form), ``ACT_TANH``, ``ACT_RELU2`` (the square of relu), ``ACT_SILU``, ``ACT_SIGMOID``."""
    m, cols = out.shape
    _need(z.dtype == torch.float32 and z.stride(-1) == 1 and out.stride(1) == 1, "activation: float32 sums, rows out")
    if z.dim() == 3:
        _need(z.is_contiguous() and tuple(z.shape[1:]) == (m, cols), "activation: slices [P, M, C]")
        parts, pstride, zstride = z.shape[0], m * cols, cols
    else:
        _need(tuple(z.shape) == (m, cols), "activation: [M, C]")
        parts, pstride, zstride = 1, 0, z.stride(0)
    _check(_lib().ifx_activation(_ptr(z), zstride, parts, pstride, _ptr(out), _code(out), out.stride(0), m, cols, int(act),
                                 _stream()), "activation")
    return out


def causal_conv(x: torch.Tensor, col0: int, channels: int, w: torch.Tensor, bias: Optional[torch.Tensor],
                tail: Optional[torch.Tensor], row_entry: torch.Tensor, entry_q_start: torch.Tensor,
                entry_q_len: torch.Tensor, entry_slot: torch.Tensor, n_entries: int, out: torch.Tensor,
                silu: bool = True) -> torch.Tensor:
    """``out[t, c] = act(bias[c] + sum_j w[c, j] * u_(t - taps + 1 + j)[c])`` with ``u = x[:, col0 + c]`` over the
    tokens of one sequence and ``u = 0`` ahead of its first token: ``x`` float32 rows, ``w`` float32 ``[channels,
    taps]``, ``out`` float32 ``[N, channels]``.  The ``taps - 1`` inputs before the step's first row come from
    ``tail [slots, taps - 1, channels]``, which a second launch then brings up to date."""
    n, taps = x.shape[0], w.shape[1]
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and col0 + channels <= x.shape[1],
          "causal_conv: float32 rows")
    _need(w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == channels, "causal_conv: w float32 [channels, taps]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == channels), "causal_conv: bias float32 [channels]")
    _need(out.dtype == torch.float32 and out.stride(1) == 1 and tuple(out.shape) == (n, channels), "causal_conv: out")
    if taps > 1:
        _need(tail is not None and tail.dtype == torch.float32 and tail.is_contiguous()
              and tuple(tail.shape[1:]) == (taps - 1, channels), "causal_conv: tail float32 [slots, taps - 1, channels]")
    _check(_lib().ifx_causal_conv(_ptr(x), x.stride(0), col0, _ptr(w), _ptr(bias), taps, _ptr(tail) if taps > 1 else None,
                                  _ptr(row_entry), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_slot), n, n_entries,
                                  _ptr(out), out.stride(0), channels, 1 if silu else 0, _stream()), "causal_conv")
    if taps > 1:
        global launch_count
        launch_count += 1
    return out


def ssm_scan(xbc: torch.Tensor, x_col: int, b_col: int, c_col: int, dt: torch.Tensor, dt_bias: torch.Tensor,
             a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, entry_q_start: torch.Tensor,
             entry_q_len: torch.Tensor, entry_slot: torch.Tensor, n_entries: int, out: torch.Tensor, heads: int,
             groups: int, vdim: int, n_state: int) -> torch.Tensor:
    """The selective state-space recurrence, float32.  Per head ``h`` with ``B``, ``C`` of group ``h // (heads /
    groups)``: ``dt = softplus(dt_raw + dt_bias)``, ``S <- exp(-exp(a_log) dt) S + dt B x^T``, ``y = S^T C + D x``.
    ``xbc`` float32 rows hold x (``heads * vdim`` from ``x_col``), B and C (``groups * n_state`` from ``b_col``,
    ``c_col``); ``dt`` float32 rows ``[N, heads]`` (a view); ``state [slots, heads, vdim, n_state]`` is read at an
    entry's start and written at its end; ``out`` float32 ``[N, heads * vdim]``."""
    n = xbc.shape[0]
    _need(xbc.dtype == torch.float32 and xbc.stride(1) == 1 and dt.dtype == torch.float32 and dt.stride(1) == 1
          and tuple(dt.shape) == (n, heads), "ssm_scan: float32 rows")
    _need(all(v.dtype == torch.float32 and v.numel() == heads and v.is_contiguous() for v in (dt_bias, a_log, d_skip)),
          "ssm_scan: dt_bias, a_log, d float32 [heads]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, n_state),
          "ssm_scan: state float32 [slots, heads, vdim, state]")
    _need(out.dtype == torch.float32 and out.stride(1) == 1 and tuple(out.shape) == (n, heads * vdim), "ssm_scan: out")
    _check(_lib().ifx_ssm_scan(_ptr(xbc), xbc.stride(0), x_col, b_col, c_col, _ptr(dt), dt.stride(0), _ptr(dt_bias),
                               _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(entry_q_start), _ptr(entry_q_len),
                               _ptr(entry_slot), n_entries, _ptr(out), out.stride(0), heads, groups, vdim, n_state,
                               n, _stream()), "ssm_scan")
    return out


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, out: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``v = y * silu(z)``; every one of ``groups`` equal parts of a row of ``v`` is divided by its own root mean
    square (eps inside the root) and multiplied by ``w``: ``y``, ``z`` float32 rows (views), ``w`` float32 ``[C]``."""
    n, cols = y.shape
    _need(y.dtype == torch.float32 and z.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1
          and tuple(z.shape) == (n, cols) and cols % groups == 0, "gated_group_norm: float32 rows, groups dividing them")
    _need(w.dtype == torch.float32 and w.numel() == cols and w.is_contiguous() and out.stride(1) == 1
          and tuple(out.shape) == (n, cols), "gated_group_norm: w float32 [C], out [N, C]")
    _check(_lib().ifx_gated_group_norm(_ptr(y), y.stride(0), _ptr(z), z.stride(0), _ptr(w), _ptr(out), _code(out),
                                       out.stride(0), n, groups, cols // groups, float(eps), _stream()), "gated_group_norm")
    return out


def delta_rule_scan(proj: torch.Tensor, r_col: int, k_col: int, v_col: int, a_col: int, w_raw: torch.Tensor,
                    w0: torch.Tensor, a_bias: torch.Tensor, state: torch.Tensor, entry_q_start: torch.Tensor,
                    entry_q_len: torch.Tensor, entry_slot: torch.Tensor, n_entries: int, out: torch.Tensor, heads: int,
                    dim: int, vdim: int, decay_scale: float, key_eps: float) -> torch.Tensor:
    """The generalized delta rule, float32.  Per head: ``w = exp(-decay_scale * sigmoid(w_raw + w0))``, ``a =
    sigmoid(a_raw + a_bias)``, ``u = k / sqrt(sum(k^2) + key_eps)``, ``S <- diag(w) S - (a * u)(u^T S) + k v^T``
    (both terms from the old state), ``o = S^T r``.  ``proj`` float32 rows hold r, k, a_raw (``heads * dim`` each)
    and v (``heads * vdim``) from the given columns; ``w_raw`` float32 rows ``[N, heads * dim]``;
    ``state [slots, heads, vdim, dim]``; ``out`` float32 ``[N, heads * vdim]``."""
    n = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and w_raw.dtype == torch.float32 and w_raw.stride(1) == 1
          and tuple(w_raw.shape) == (n, heads * dim), "delta_rule_scan: float32 rows")
    _need(all(v.dtype == torch.float32 and v.numel() == heads * dim and v.is_contiguous() for v in (w0, a_bias)),
          "delta_rule_scan: w0 and a_bias float32 [heads * dim]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, dim),
          "delta_rule_scan: state float32 [slots, heads, vdim, dim]")
    _need(out.dtype == torch.float32 and out.stride(1) == 1 and tuple(out.shape) == (n, heads * vdim), "delta_rule_scan: out")
    # a step with portions: the unit key, decay and removal rate of all its rows by a kernel ahead of the scan
    prep = torch.empty((n, 3 * heads * dim), dtype=torch.float32, device=proj.device) if n > n_entries else None
    _check(_lib().ifx_delta_rule_scan(_ptr(proj), proj.stride(0), r_col, k_col, v_col, a_col, _ptr(w_raw), w_raw.stride(0),
                                      _ptr(w0), _ptr(a_bias), _ptr(state), _ptr(entry_q_start), _ptr(entry_q_len),
                                      _ptr(entry_slot), n_entries, _ptr(out), out.stride(0), heads, dim, vdim,
                                      float(decay_scale), float(key_eps), n, _ptr(prep) if prep is not None else None,
                                      _stream()), "delta_rule_scan")
    if prep is not None:
        global launch_count
        launch_count += 1
    return out


GATE_NONE, GATE_SIGMOID, GATE_SILU = 0, 1, 2


def head_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], w: Optional[torch.Tensor], out: torch.Tensor, heads: int,
                   vdim: int, eps: float, gate_kind: int = GATE_SIGMOID) -> torch.Tensor:
    """``out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * w[h] * g(gate[t, h])`` with ``g`` sigmoid, silu or
    absent: ``o``, ``gate`` float32 rows (views), ``w`` float32 ``[heads * vdim]`` or None, ``out`` rows of either type."""
    n = o.shape[0]
    _need(o.dtype == torch.float32 and o.stride(1) == 1 and tuple(o.shape) == (n, heads * vdim) and out.stride(1) == 1
          and tuple(out.shape) == (n, heads * vdim), "head_norm_gate: o float32 [N, heads * vdim], out alike")
    _need(gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and tuple(gate.shape) == tuple(o.shape)),
          "head_norm_gate: gate float32 rows")
    _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == heads * vdim), "head_norm_gate: w")
    _check(_lib().ifx_head_norm_gate(_ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(w),
                                     _ptr(out), _code(out), out.stride(0), n, heads, vdim, float(eps),
                                     int(gate_kind) if gate is not None else GATE_NONE, _stream()), "head_norm_gate")
    return out


MIX_NONE, MIX_STORE, MIX_BLEND = 0, 1, 2


def qkv_norm_rope_write(proj: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                        cos: torch.Tensor, sin: torch.Tensor, layout: int, n_heads: int, n_kv: int, dim: int, vdim: int,
                        v_norm: bool, mix_mode: int, mix_lambda: Optional[torch.Tensor], v_first: Optional[torch.Tensor],
                        q_out: torch.Tensor, slot_map: torch.Tensor, k_layer: torch.Tensor, v_layer: torch.Tensor,
                        page_stride: int, page_size: int) -> None:
    """The first ``(n_heads + n_kv) * dim + n_kv * vdim`` columns of the float32 projection ``proj [N, W]`` (or
    slices ``[P, N, W]``) are q, k and v heads side by side.  With ``wq`` (``wk``) all query (key) columns of a token
    are divided by their common root mean square (eps inside the root) and multiplied by that weight; q and k heads
    are rotated by ``cos``/``sin`` ``[N, r/2]``; with ``v_norm`` every value head is divided by its own root mean
    square; ``MIX_STORE`` keeps the values in ``v_first [N, n_kv * vdim]``, ``MIX_BLEND`` replaces them by
    ``(1 - lambda) v + lambda v_first``.  q goes to ``q_out``, k and v into the paged cache at ``slot_map``."""
    n = q_out.shape[0]
    channels = (n_heads + n_kv) * dim + n_kv * vdim
    width = proj.shape[-1]
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and width >= channels, "qkv_norm_rope: float32 projection")
    parts, pstride = (proj.shape[0], n * width) if proj.dim() == 3 else (1, 0)
    _need(wq is None or (wq.dtype == torch.float32 and wq.is_contiguous() and wq.numel() == n_heads * dim), "qkv_norm_rope: wq")
    _need(wk is None or (wk.dtype == torch.float32 and wk.is_contiguous() and wk.numel() == n_kv * dim), "qkv_norm_rope: wk")
    _need(cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape == sin.shape
          and cos.shape[0] == n, "qkv_norm_rope: cos/sin float32 [N, r/2]")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (n, n_heads * dim) and k_layer.dtype == q_out.dtype,
          "qkv_norm_rope: q_out [N, heads * dim] of the cache's type")
    if mix_mode != MIX_NONE:
        _need(v_first is not None and v_first.dtype == torch.float32 and v_first.is_contiguous()
              and tuple(v_first.shape) == (n, n_kv * vdim), "qkv_norm_rope: v_first float32 [N, kv_heads * vdim]")
    if mix_mode == MIX_BLEND:
        _need(mix_lambda is not None and mix_lambda.dtype == torch.float32 and mix_lambda.numel() == 1, "qkv_norm_rope: lambda")
    _check(_lib().ifx_qkv_norm_rope_write(_ptr(proj), parts, pstride, width, _ptr(wq), _ptr(wk), float(eps), _ptr(cos),
                                          _ptr(sin), cos.shape[1], layout, n_heads, n_kv, dim, vdim, int(bool(v_norm)),
                                          int(mix_mode), _ptr(mix_lambda), _ptr(v_first), _ptr(q_out), _code(q_out),
                                          _ptr(slot_map), _ptr(k_layer), _ptr(v_layer), page_stride, page_size, n,
                                          _stream()), "qkv_norm_rope_write")


def add_group_rmsnorm(residual: torch.Tensor, a, weight: torch.Tensor, eps: float, groups: int, out: Optional[torch.Tensor],
                      rows: Optional[torch.Tensor] = None, a_scale: float = 1.0, b=None, b_scale: float = 1.0) -> Optional[torch.Tensor]:
    """``residual`` (float32 ``[N, H]``) ``+= a_scale * a + b_scale * b``; ``out`` = the sum with each of ``groups``
    equal consecutive parts of a row divided by its own root mean square (eps inside the root), times ``weight``.
    ``a`` and ``b`` are None, ``[N, H]`` or slices ``[P, N, H]`` (float32 or bfloat16, both of one type).  With
    ``rows`` (int32) only those rows are normed into ``out [R, H]`` and the residual is left untouched."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_group_rmsnorm: residual float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden and groups >= 1 and hidden % groups == 0,
          "add_group_rmsnorm: weight float32 [H], groups dividing H")
    n_rows = rows.numel() if rows is not None else n
    _need(rows is None or rows.dtype == torch.int32, "add_group_rmsnorm: rows int32")

    def slices(t):
        if t is None:
            return None, 1, 0
        _need(t.is_contiguous() and tuple(t.shape[-2:]) == (n, hidden) and t.dim() in (2, 3), "add_group_rmsnorm: addends [N, H] or [P, N, H]")
        return _ptr(t), (t.shape[0] if t.dim() == 3 else 1), n * hidden
    (pa, na, sa), (pb, nb, sb) = slices(a), slices(b)
    if a is not None and b is not None:
        _need(a.dtype == b.dtype, "add_group_rmsnorm: both addends of one type")
    dd = _code(a if a is not None else b) if (a is not None or b is not None) else F32
    if out is not None:
        _need(out.is_contiguous() and tuple(out.shape) == (n_rows, hidden), "add_group_rmsnorm: out [rows, H]")
    _check(_lib().ifx_add_group_rmsnorm(_ptr(residual), pa, na, sa, float(a_scale), pb, nb, sb, float(b_scale), dd, _ptr(weight),
                                        float(eps), int(groups), _ptr(out), _code(out) if out is not None else F32, _ptr(rows),
                                        n_rows, hidden, 0 if rows is not None else 1, _stream()), "add_group_rmsnorm")
    return out


def glu_clamped(z: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, limit: float, alpha: float = 1.702,
                shift: float = 1.0) -> torch.Tensor:
    """``z`` float32 ``[M, 2I]`` or slices ``[P, M, 2I]`` (gate columns first, then up): ``g = min(z_g + b_g, limit)``,
    ``u = clamp(z_u + b_u, -limit, limit)``, ``out = g * sigmoid(alpha * g) * (u + shift)``."""
    m, inter = out.shape
    _need(z.dtype == torch.float32 and z.is_contiguous() and tuple(z.shape[-2:]) == (m, 2 * inter), "glu_clamped: z float32 [M, 2I]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * inter), "glu_clamped: bias float32 [2I]")
    _need(out.is_contiguous(), "glu_clamped: out contiguous")
    parts = z.shape[0] if z.dim() == 3 else 1
    _check(_lib().ifx_glu_clamped(_ptr(z), parts, m * 2 * inter, _ptr(bias), _ptr(out), _code(out), m, inter, float(limit),
                                  float(alpha), float(shift), _stream()), "glu_clamped")
    return out


def gla_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, z: torch.Tensor, z_bias: torch.Tensor, tau: float,
             q_scale: float, state: torch.Tensor, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
             entry_slot: torch.Tensor, n_entries: int, out: torch.Tensor, heads: int, dim: int, vdim: int,
             seg_entry: Optional[torch.Tensor] = None, seg_t0: Optional[torch.Tensor] = None,
             entry_first_seg: Optional[torch.Tensor] = None, n_segments: int = 0) -> torch.Tensor:
    """Gated linear attention, float32.  Per head ``alpha = sigmoid(z + z_bias)^(1 / tau)`` (one per key channel),
    ``S <- diag(alpha) S + k v^T``, ``o = S^T (q * q_scale)``.  ``proj`` float32 rows hold q, k (``heads * dim`` each)
    and v (``heads * vdim``) from the given columns; ``z`` float32 rows ``[N, heads * dim]``; ``state [slots, heads,
    dim, vdim]``; ``out`` float32 ``[N, heads * vdim]``.  With ``n_segments`` > 0 the step is cut into segments of
    :func:`gla_segment` tokens (``seg_entry``, ``seg_t0``, ``entry_first_seg``: int32) that run side by side, their
    starting states found one after the other in between; without, every entry is walked from its slot in one go."""
    n = proj.shape[0]
    _need(proj.dtype == torch.float32 and proj.stride(1) == 1 and z.dtype == torch.float32 and z.stride(1) == 1
          and tuple(z.shape) == (n, heads * dim), "gla_scan: float32 rows")
    _need(z_bias.dtype == torch.float32 and z_bias.is_contiguous() and z_bias.numel() == heads * dim, "gla_scan: z_bias float32 [heads * dim]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "gla_scan: state float32 [slots, heads, dim, vdim]")
    _need(out.dtype == torch.float32 and out.stride(1) == 1 and tuple(out.shape) == (n, heads * vdim), "gla_scan: out")
    _need(max(q_col, k_col) + heads * dim <= proj.shape[1] and v_col + heads * vdim <= proj.shape[1], "gla_scan: columns beyond the row")
    seg_state = seg_decay = None
    if n_segments > 0:
        seg_state = torch.empty((n_segments, heads, dim, vdim), dtype=torch.float32, device=proj.device)
        seg_decay = torch.empty((n_segments, heads, dim), dtype=torch.float32, device=proj.device)
    _check(_lib().ifx_gla_scan(_ptr(proj), proj.stride(0), q_col, k_col, v_col, _ptr(z), z.stride(0), _ptr(z_bias),
                               1.0 / float(tau), float(q_scale), _ptr(state), _ptr(entry_q_start), _ptr(entry_q_len),
                               _ptr(entry_slot), n_entries, _ptr(out), out.stride(0), heads, dim, vdim, _ptr(seg_entry),
                               _ptr(seg_t0), _ptr(entry_first_seg), int(n_segments), _ptr(seg_state), _ptr(seg_decay),
                               _stream()), "gla_scan")
    if n_segments > 0:
        global launch_count
        launch_count += 2
    return out


def gla_segment() -> int:
    """Tokens per segment of the gated linear attention scan."""
    return int(_lib().ifx_gla_segment())
