"""The compiled kernels as a ctypes library, loaded once per process.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, `load()` raises and nothing of the engine runs.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from .build import BuildError, bounds_check_wanted, build

_LIB = None

ERRORS = {
    1: "a size is outside what the kernel supports",
    2: "unknown dtype flag",
    3: "the CUDA launch failed",
    4: "a pointer or stride is misaligned",
    5: "the scratch buffer is too small",
}


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "mb_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                       c_float, c_int, c_void_p],
    "mb_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_rope_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p],
    "mb_gemm_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_void_p],
    "mb_paged_attention_simt": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                c_void_p],
    "mb_paged_attention_mma": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                               c_void_p],
    "mb_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float,
                       c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                       c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "mb_gemm_skinny_swiglu": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                              c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                              c_longlong, c_int, c_float, c_float, c_void_p, c_void_p],
    "mb_gemm_skinny_set_fed_min": [c_longlong],
    "mb_gemm_skinny_qkv_rope": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float,
                                c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                        c_int, c_void_p],
    "mb_gemm_tcgen05_withheld": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                 c_longlong, c_void_p],
    "mb_gemm_tcgen05_persistent": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p],
    "mb_gemm_pair_supports": [c_int, c_int, c_int],
    "mb_gemm_pair_tiles": [c_int, c_int],
    "mb_gemm_pair": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                     c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "mb_paged_attention_tcgen05": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "mb_paged_attention_decode_cluster_sinks": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                                c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                                c_void_p],
    "mb_paged_attention_mma_sinks": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p],
    "mb_paged_attention_decode_cluster": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_gemm_skinny_set_slices": [c_int, c_int],
    "mb_patch_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "mb_embed_positions": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                           c_int, c_int, c_int, c_void_p],
    "mb_rmsnorm_add": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int, c_float,
                       c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_gated_act": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "mb_mixed_head_attention": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_longlong, c_void_p],
    "mb_mixed_head_attention_mma": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p,
                                    c_longlong, c_void_p],
    "mb_rope_blend_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_mingru_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p],
    "mb_causal_conv": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_block_gates": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "mb_gated_recurrence_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_paged_attention_simt_sinks": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                      c_void_p, c_void_p],
    "mb_embed_scaled": [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_scaled_add_norm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_float, c_int,
                           c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "mb_softcap": [c_void_p, c_longlong, c_float, c_void_p],
    "mb_conv_act": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                    c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "mb_conv_act_update": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p],
    "mb_conv_tail_update": [c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_void_p],
    "mb_mamba2_scan": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                       c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_delta_rule_scan": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                           c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_void_p],
    "mb_gated_group_norm": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float,
                            c_int, c_void_p, c_int, c_int, c_void_p],
    "mb_latent_norm_store": [c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "mb_head_linear": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                       c_int, c_int, c_void_p],
    "mb_route_experts": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                         c_int, c_int, c_int, c_int, c_float, c_void_p],
    "mb_expert_tile_rows": [c_int, c_int, c_int],
    "mb_expert_tile_cap": [c_int, c_int, c_int],
    "mb_expert_plan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_expert_product": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_expert_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_embed_bigram": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int,
                        c_int, c_void_p],
    "mb_rmsnorm_join_add": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float,
                            c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_int, c_int,
                            c_void_p],
    "mb_masked_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_masked_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int,
                            c_float, c_float, c_float, c_int, c_int, c_void_p],
    "mb_masked_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                c_int, c_int, c_float, c_float, c_float, c_int, c_void_p],
    "mb_retention_scan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p,
                          c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_void_p],
    "mb_expert_combine_sorted": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_expert_combine": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_rmsnorm_add_pair": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int,
                            c_float, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p],
    "mb_stream_conv": [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_stream_tail_store": [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int,
                             c_int, c_void_p],
    "mb_latent_prepare": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
                          c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                          c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_rope_rows": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                     c_void_p, c_int, c_void_p],
    "mb_qk_norm_rope_store": [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                              c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_sigmoid_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p],
    "mb_sigmoid_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "mb_general_delta_scan": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_float,
                              c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int, c_void_p],
    "mb_tanh_slice": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "mb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "mb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
}


def load():
    """Build if needed, load, and declare the entry points."""
    global _LIB
    if _LIB is not None:
        return _LIB
    try:
        path = build(bounds_check=bounds_check_wanted())
    except BuildError as err:
        raise KernelError(f"the CUDA kernels could not be built: {err}") from err
    lib = ctypes.CDLL(str(path))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.mb_gemm_tcgen05_supports.argtypes = [c_int, c_int, c_int]
    lib.mb_gemm_tcgen05_supports.restype = c_int
    lib.mb_check_enabled.argtypes = []
    lib.mb_check_enabled.restype = c_int
    lib.mb_check_set_limits.argtypes = [c_int, c_int, c_void_p]
    lib.mb_check_set_limits.restype = c_int
    lib.mb_check_read.argtypes = [ctypes.POINTER(c_int), c_void_p]
    lib.mb_check_read.restype = c_int
    lib.mb_set_dependent_launch.argtypes = [c_int]
    lib.mb_set_dependent_launch.restype = None
    lib.mb_gemm_skinny_supports.argtypes = [c_int, c_int, c_int]
    lib.mb_gemm_skinny_supports.restype = c_int
    lib.mb_gemm_skinny_qkv_supports.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_gemm_skinny_qkv_supports.restype = c_int
    lib.mb_attention_tcgen05_supports.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.mb_attention_tcgen05_supports.restype = c_int
    lib.mb_attention_mma_supports.argtypes = [c_int]
    lib.mb_attention_mma_supports.restype = c_int
    lib.mb_attention_decode_raw_pays.argtypes = [c_int]
    lib.mb_attention_decode_raw_pays.restype = c_int
    lib.mb_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_attention_scratch_floats.restype = c_longlong
    lib.mb_mixed_head_mma_supports.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_mixed_head_mma_supports.restype = c_int
    lib.mb_mixed_head_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_mixed_head_scratch_floats.restype = c_longlong
    lib.mb_mamba2_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int]
    lib.mb_mamba2_scratch_floats.restype = c_longlong
    lib.mb_sigmoid_attention_mma_supports.argtypes = [c_int]
    lib.mb_sigmoid_attention_mma_supports.restype = c_int
    lib.mb_sigmoid_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_sigmoid_attention_scratch_floats.restype = c_longlong
    lib.mb_masked_attention_mma_supports.argtypes = [c_int, c_int, c_int]
    lib.mb_masked_attention_mma_supports.restype = c_int
    lib.mb_masked_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.mb_masked_attention_scratch_floats.restype = c_longlong
    _LIB = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {ERRORS.get(code, f'error {code}')}")
