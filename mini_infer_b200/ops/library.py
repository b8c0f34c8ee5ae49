"""Load the CUDA library and declare its C entry points.

There is exactly one way to run an op: through this library, on a CUDA device.
If it cannot be built or loaded the import of an op fails with the reason; no
op has a CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from typing import Optional

_lib: Optional["_Library"] = None
_lib_path: Optional[str] = None

P = c_void_p
I = c_int
F = c_float
L = c_int64

_SIGNATURES = {
    "mi_embed_gather": [P, P, I, P, I, I, I, P],
    "mi_add_rmsnorm": [P, P, P, P, I, P, I, I, I, F, P],
    "mi_qkv_post": [P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    "mi_swiglu": [P, P, I, L, I, P],
    "mi_moe_combine": [P, P, P, P, P, P, I, I, I, P],
    "mi_combine_add_rmsnorm": [P, P, P, P, P, P, I, P, P, I, P, I, I, I, F, P],
    "mi_attn_tiled": [P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_decode": [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_decode_split": [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_decode_split_form": [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, I, P],
    "mi_moe_router": [P, I, P, P, I, P, P, P, P, P, I, I, I, I, I, P, P],
    "mi_moe_permute": [P, P, P, P, P, I, I, I, P],
    "mi_grouped_gemm_plain": [P, I, P, P, I, P, P, I, I, I, I, I, I, I, F, F, P, P],
    "mi_sample_rows": [P, P, P, P, P, P, I, I, P],
    "mi_grouped_gemm_skinny": [P, P, P, P, P, I, I, I, I, I, F, F, P, P],
    "mi_moe_route_small": [P, I, P, P, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P],
    "mi_moe_norm_route_small": [P, P, P, I, F, P, I, P, P, I, P, P, P, P, I, I, I, I, I, P],
    "mi_grouped_gemm_skinny_pairs": [P, P, P, P, I, I, I, I, I, I, I, F, F, P, P],
    "mi_qkv_skinny": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "mi_dense_skinny": [P, P, P, P, I, I, I, I, P],
    "mi_gather_rows_bf16": [P, P, P, I, I, P],
    "mi_attn_prefill": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_prefill_tc": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, F, I, P],
    "mi_grouped_gemm_tc": [P, P, P, P, P, I, I, I, I, I, I, F, F, P, P],
    "mi_grouped_gemm_tc_form": [P, P, P, P, P, I, I, I, I, I, I, I, F, F, P, P],
    "mi_random_fill": [P, I, L, ctypes.c_uint, ctypes.c_uint, F, F, P],
    "mi_dense_f32": [P, P, P, I, I, I, P],
    "mi_l2_prefetch": [P, ctypes.c_ulonglong, P],
    "mi_causal_conv_silu": [P, I, P, P, I, P, L, P, P, P, P, I, I, I, I, I, P],
    "mi_delta_scan": [P, I, P, I, P, I, P, P, P, L, P, P, P, P, I, I, I, I, I, I, F, P],
    "mi_ssd_scan": [P, I, P, I, P, P, P, P, L, P, P, P, I, I, I, I, I, P],
    "mi_gated_group_rmsnorm": [P, P, I, P, I, I, P, I, I, I, I, I, F, P],
    "mi_rope_store": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P, F, I, P, L, P, P],
    "mi_attn_mix": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, I, I, I, P],
    "mi_attn_mix_tc": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, I, I, I, I, P],
    "mi_out_norm_add": [P, P, P, P, P, P, P, I, P, I, P, I, I, I, F, F, P],
    "mi_softcap_rows": [P, L, F, P],
    "mi_cast_rows": [P, P, I, L, P],
    "mi_scatter_values": [P, P, P, I, P],
    "mi_add2_rmsnorm_scalar": [P, P, P, P, P, P, P, P, I, I, I, F, P],
    "mi_geglu_tanh": [P, P, I, L, I, P],
    "mi_concat_cast": [P, P, P, P, P, I, I, I, P],
    "mi_rows_plus_vec": [P, P, P, I, I, I, P],
    "mi_attn_prefill_tc_shared": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P],
    "mi_clamped_glu": [P, P, I, L, I, F, F, P],
    "mi_dense_f32_batched": [P, P, P, I, I, I, I, I, I, L, L, L, P],
    "mi_latent_store": [P, I, I, P, P, P, F, P, P, I, I, I, I, P],
    "mi_latent_query": [P, P, P, P, P, I, I, I, I, I, I, P],
    "mi_sigmoid_gate": [P, L, L, P, I, I, P, I, I, I, I, P],
    "mi_causal_conv_residual": [P, I, P, I, P, L, P, P, P, P, I, I, I, I, I, I, P],
    "mi_norm_conv_decode": [P, P, I, F, P, P, L, P, P, P, I, I, I, I, P],
    "mi_delta_scan_form": [P, I, P, I, P, I, P, P, P, L, P, P, P, P, I, I, I, I, I, I, F, I, F, P],
    "mi_gla_scan_segments": [P, I, P, I, P, P, L, P, P, P, P, I, I, I, I, I, F, F, I, I, P, P, P, P],
    "mi_attn_mix_form": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, I, I, I, P, P],
    "mi_attn_mix_tc_form": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, I, I, I, I, P, P],
    "mi_attn_prefill_tc_logistic": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "mi_group_rmsnorm": [P, P, P, I, P, I, I, I, I, F, P],
    "mi_out_norm_add_groups": [P, P, P, P, P, P, P, I, P, I, P, I, I, I, F, F, I, P],
}


# entry points that are not launchers: name -> (argtypes, restype)
_OTHERS = {
    "mi_last_error": ([], c_char_p),
    "mi_launch_count": ([], ctypes.c_longlong),
    "mi_attn_decode_supported": ([I], c_int),
    "mi_attn_prefill_supported": ([I], c_int),
    "mi_grouped_gemm_tc_supported": ([I], c_int),
    "mi_grouped_gemm_skinny_supported": ([I], c_int),
    "mi_moe_route_small_max_tokens": ([], c_int),
    "mi_moe_norm_route_small_max_width": ([], c_int),
    "mi_set_dependent_launch": ([c_int], c_int),
    "mi_moe_norm_route_small_takes": ([c_int, c_int, c_int, c_int], c_int),
    "mi_grouped_gemm_skinny_pairs_split_inner_max_tokens": ([], c_int),
    "mi_grouped_gemm_skinny_pairs_max_tokens": ([], c_int),
    "mi_attn_prefill_tc_supported": ([I, I], c_int),
    "mi_qkv_skinny_supported": ([I, I, I], c_int),
    "mi_dense_skinny_max_rows": ([], c_int),
    "mi_delta_scan_prep_row": ([I], c_int),
    "mi_attn_mix_tc_supported": ([I, I, I, I], c_int),
    "mi_attn_mix_tc_splits": ([I], c_int),
    "mi_attn_mix_supported": ([I, I, I, I, I], c_int),
    "mi_attn_prefill_tc_shared_supported": ([I, I, I, I], c_int),
    "mi_attn_prefill_tc_logistic_supported": ([I, I, I], c_int),
    "mi_attn_decode_split_size": ([], c_int),
}

# kernels that the engine itself calls, whatever the model: embedding, norms and the residual, the dense
# products of both precision paths, weight prefetch, sampling, random weights
ENGINE_SOURCES = ("elementwise.cu", "dense_f32.cu", "moe_skinny.cu", "prefetch.cu", "sampling.cu", "random_init.cu")


class _Library:
    """The entry points of one loaded library.  A partial library (built from the sources one model needs) lacks
    the others' entry points: asking for one of those builds and loads the whole library in its place, so a
    missing kernel costs a compile, never a wrong or a missing result."""

    def __init__(self, cdll: ctypes.CDLL, path: str, sources):
        self._cdll, self.path, self.sources = cdll, path, sources          # sources None: the whole library
        for name, argtypes in _SIGNATURES.items():
            self._bind(name, argtypes, c_int)
        for name, (argtypes, restype) in _OTHERS.items():
            self._bind(name, argtypes, restype)

    def _bind(self, name, argtypes, restype) -> None:
        try:
            fn = getattr(self._cdll, name)
        except AttributeError:
            return
        fn.argtypes = argtypes
        fn.restype = restype
        self.__dict__[name] = fn

    def __getattr__(self, name):           # only reached for names that were not bound above
        if name.startswith("_"):
            raise AttributeError(name)
        try:
            return getattr(self._cdll, name)
        except AttributeError:
            if self.sources is None:
                raise
        return getattr(_load(None), name)


_loaded: list = []       # every library this process loaded (a replaced one stays: captured graphs hold its kernels)


def _load(needs) -> "_Library":
    global _lib, _lib_path
    from ..csrc.build import CORE, build, built_full
    path, sources = None, None
    if needs is not None:
        path = built_full()                 # the whole library is there already: nothing to compile
        if path is None:
            sources = frozenset(needs) | frozenset(CORE)
            path = build(only=sorted(sources))
    if path is None:
        path = build()
    try:
        cdll = ctypes.CDLL(path)
    except OSError as e:
        raise RuntimeError(f"mini_infer_b200: cannot load {path}: {e}") from e
    lib = _Library(cdll, path, sources)
    if "mi_last_error" not in lib.__dict__:
        raise RuntimeError(f"mini_infer_b200: {path} lacks the library's core entry points")
    _loaded.append(lib)
    _lib, _lib_path = lib, path
    return lib


def library(needs=None) -> "_Library":
    """The loaded library; built at the first call of a fresh checkout.  ``needs`` (names of CUDA sources): what
    the caller is going to use; when nothing is built yet, only those (and the engine's own) are compiled.  A
    call without ``needs`` takes whatever is loaded."""
    if _lib is not None:
        if needs is None or _lib.sources is None or set(needs) <= _lib.sources:
            return _lib
    if needs is not None:
        needs = set(needs) | set(ENGINE_SOURCES)
    return _load(needs)


def launch_count() -> int:
    """Kernels of this library queued so far in this process."""
    library()
    return sum(int(lib.mi_launch_count()) for lib in _loaded)


def library_path() -> Optional[str]:
    return _lib_path


class KernelError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        msg = library().mi_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} refused or failed (code {code}): {msg}")
