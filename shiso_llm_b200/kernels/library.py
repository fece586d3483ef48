"""Loads the kernel library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, ``library()`` raises and every op with it.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from .build import BASE, BuildError, exports, library_path

_LIB = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

_SIGNATURES = {
    "shiso_embed": [P, P, P, P, I, P, I, I, I, P],
    "shiso_gather_rows": [P, P, P, I, I, P],
    "shiso_rmsnorm": [P, P, P, P, P, I, I, I, F, P],
    "shiso_swiglu": [P, P, I, I, I, P],
    "shiso_gemm_simple": [P, I, P, I, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05": [P, P, P, P, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_tokens64": [P, P, P, P, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_swiglu": [P, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05_prompt": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_prefill_attention_tc_supported": [I, I],
    "shiso_prefill_attention_tc": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, LL, F, I, P],
    "shiso_gemm_tcgen05_pair": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_supported": [I, P, P],
    "shiso_gemm_tcgen05_fused_max_tokens": [],
    "shiso_gemm_tcgen05_into_partial_rows": [I],
    "shiso_gemm_tcgen05_into": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "shiso_gemm_tcgen05_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_pair_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_prompt_scaled": [P, P, I, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_tcgen05_status": [],
    "shiso_gemm_stream": [P, P, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_stream_into": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "shiso_gemm_stream_scaled": [P, P, I, F, P, P, I, I, I, I, I, I, P],
    "shiso_gemm_stream_conv": [P, P, I, F, P, P, P, P, LL, P, P, P, I, I, I, I, I, I, P],
    "shiso_short_conv": [P, I, P, P, P, LL, P, P, P, P, I, I, I, I, I, I, P],
    "shiso_qk_norm_rope_store": [P, I, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "shiso_paged_attention": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
    "shiso_decode_attention": [P, P, P, P, I, P, P, P, P, I, I, I, I, I, F, I, I, P],
    "shiso_decode_attention_fused_supported": [I, I, I, I],
    "shiso_decode_attention_fused_max_parts": [],
    "shiso_decode_attention_fused": [P, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, P],
    "shiso_decode_attention_from_qkv": [P, P, P, P, F, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, I, P],
    "shiso_prefill_attention": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P],
    "shiso_argmax": [P, P, I, I, P, P],
    "shiso_argmax_chunked": [P, P, P, I, I, I, P, P],
    "shiso_sample": [P, P, P, P, P, P, P, P, I, I, P, P],
    "shiso_suppress": [P, P, P, I, I, I, P],
    "shiso_copy_words": [P, P, I, I, P],
    "shiso_selftest_bounded_wait": [LL, P],
    "shiso_embed_hashed_pair": [P, P, P, P, P, I, P, P, P, P, P, LL, P, I, I, I, I, F, I, I, I, P],
    "shiso_hyper_mix": [P, LL, P, P, P, P, LL, P, P, F, P, P, I, I, I, I, P],
    "shiso_token_shift_blend": [P, I, P, P, LL, P, P, P, P, P, I, I, I, I, P],
    "shiso_unary": [P, I, P, I, LL, I, P],
    "shiso_decay_recurrence_supported": [I, I],
    "shiso_decay_recurrence": [P, P, P, P, LL, LL, LL, LL, P, LL, I, P, LL, P, P, P, P, LL, P, P, P, P, I, F, P, F, F, P, I, I, I, I, I, I, P],
    "shiso_store_kv": [P, LL, P, LL, I, P, P, P, I, P, P, I, I, I, I, I, P],
    "shiso_pool_kv": [P, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, P],
    "shiso_pooled_window_attention": [P, LL, I, P, P, P, P, P, P, I, P, P, P, LL, P, I, I, I, I, I, I, F, I, I, F, P],
    "shiso_prefill_attention_tc_open": [P, LL, P, P, P, I, P, P, P, LL, P, F, I, I, I, I, I, I, LL, F, I, P],
    "shiso_prefill_attention_tc_kept": [P, LL, P, P, P, I, P, P, P, LL, I, I, I, I, I, I, LL, F, I, I, P],
    "shiso_decode_attention_from_qkv_kept": [P, P, P, P, F, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, I, I, P],
    "shiso_decode_attention_fused_kept": [P, LL, P, P, P, I, P, P, P, I, I, I, I, I, LL, F, I, I, I, P],
    "shiso_add_layernorm": [P, P, P, P, P, P, I, I, I, F, P],
    "shiso_group_rmsnorm": [P, I, LL, P, LL, P, P, I, I, I, I, I, F, P],
    "shiso_causal_conv": [P, LL, I, P, P, P, LL, P, P, P, P, I, I, I, I, I, P],
    "shiso_rotate_heads": [P, LL, LL, P, LL, LL, I, P, P, I, I, I, I, F, I, P],
    "shiso_latent_store": [P, LL, I, P, P, P, P, P, I, P, I, I, I, I, I, F, F, I, P],
    "shiso_state_recurrence": [P, P, P, P, LL, LL, LL, LL, I, P, P, P, P, P, LL, P, P, P, I, I, I, I, I, I, I, I, P],
    "shiso_head_linear": [P, LL, LL, I, P, I, P, LL, LL, I, P, LL, I, I, I, I, P],
    "shiso_moe_route": [P, LL, P, P, P, I, I, I, I, I, F, I, I, F, P],
    "shiso_routed_experts": [P, I, P, P, P, P, I, P, P, LL, P, P, P, P, I, I, I, I, I, I, I, F, P],
    "shiso_latent_attention_smem": [I, I],
    "shiso_latent_attention": [P, I, P, P, I, P, P, P, P, I, I, I, I, I, F, I, P],
    "shiso_latent_prefill_supported": [I, I],
    "shiso_latent_prefill": [P, P, P, I, P, P, P, I, I, I, I, I, I, F, P],
    "shiso_head_prepare_store": [P, LL, I, I, I, I, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, F, I, I, P],
    "shiso_masked_attention": [P, LL, I, P, P, P, I, P, P, P, LL, P, LL, P, I, I, I, I, I, I, F, F, I, I, I, I, I, P, I, P],
    "shiso_masked_attention_tiles_supported": [I, I],
    "shiso_masked_attention_tiles": [P, LL, P, P, P, I, P, P, P, LL, P, LL, P, I, I, I, I, I, I, I, F, F, I, I, I, I, I, P],
    "shiso_norm_into": [P, P, I, P, P, I, I, F, P],
    "shiso_polynorm": [P, LL, I, P, P, I, I, F, P],
    "shiso_gemm_stream_glu": [P, P, P, I, I, I, I, I, F, I, P],
    "shiso_gemm_tcgen05_glu": [P, P, P, I, I, I, I, I, F, P],
    "shiso_gemm_tcgen05_pair_glu": [P, P, P, I, I, I, I, I, F, I, P],
    "shiso_gemm_tcgen05_prompt_glu": [P, P, P, I, I, I, I, I, F, I, P],
    "shiso_gate_rows": [P, LL, P, LL, I, I, I, P],
    "shiso_embed_scaled": [P, P, P, P, I, P, I, I, I, F, P],
    "shiso_add_dyt": [P, P, P, P, P, P, F, P, I, I, I, P],
    "shiso_stream_add": [P, P, P, I, P, I, P, I, P, I, I, P],
    "shiso_glu_act": [P, P, I, I, I, I, F, P],
    "shiso_joined_norm_store": [P, LL, I, I, I, I, I, P, P, P, P, P, I, P, P, I, I, F, F, I, P],
}


class KernelLibraryError(RuntimeError):
    pass


class _Library:
    """The kernel libraries as one object: an entry point is looked up, on its first use, in the
    library of the file that defines it, which is built then if it is not yet."""

    def __init__(self):
        self._loaded = {}

    def _module(self, module: str):
        lib = self._loaded.get(module)
        if lib is not None:
            return lib
        if module != BASE:
            self._module(BASE)  # the others resolve their cross-file calls against it
        try:
            path = library_path(module)
        except BuildError as e:
            raise KernelLibraryError(f"the CUDA kernels are required and could not be built: {e}") from e
        try:
            # (never with RTLD_GLOBAL: every library carries its own copies of inline functions and
            # their static state, and a global base would lend the others its copies)
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelLibraryError(f"the CUDA kernel library {path} could not be loaded: {e}") from e
        self._loaded[module] = lib
        return lib

    def __getattr__(self, name):
        if not name.startswith("shiso_"):
            raise AttributeError(name)
        module = exports().get(name)
        if module is None:
            raise KernelLibraryError(f"no kernel file exports {name}")
        lib = self._module(module)
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"{lib._name} does not export {name}; rebuild it") from e
        if name in _SIGNATURES:
            fn.argtypes = _SIGNATURES[name]
        fn.restype = c_int
        setattr(self, name, fn)
        return fn

    def loaded(self) -> list:
        return sorted(self._loaded)


def library():
    global _LIB
    if _LIB is None:
        _LIB = _Library()
        _LIB._module(BASE)  # no kernels without it: fail here, loudly, not at the first launch
    return _LIB


def declare(name: str, argtypes) -> None:
    """Declares one more entry point (used by kernels added in their own files)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None and name in _LIB.__dict__:
        _LIB.__dict__[name].argtypes = argtypes
