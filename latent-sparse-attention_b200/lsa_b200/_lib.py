"""ctypes binding of `liblsa_b200.so`, the C-ABI library of sm_100a kernels.

There is no CPU path: if the library is missing or the tensors are not on a CUDA device, every call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblsa_b200.so")
ABI_VERSION = 18

DTYPE_F32, DTYPE_BF16 = 0, 1
PAD = -1
EMPTY_KEY = -(2**63)
INT64_MAX = 2**63 - 1

_P, _I, _L, _F, _Z = c_void_p, c_int, c_int64, c_float, c_size_t

# name -> (restype, argtypes); kept in the order of include/lsa_b200.h
SIGNATURES = {
    "lsa_error_string": (ctypes.c_char_p, [_I]),
    "lsa_abi_version": (_I, []),
    "lsa_index_map": (_I, [_P, _I, _L, _I, _I, _I, _I, _L, _L, _P, _I, _I, _I, _P, _P, _P]),
    "lsa_index_map_tc": (_I, [_P, _L, _L, _L, _P, _I, _I, _P, _P, _P, _P]),
    "lsa_gemm_gelu_tc": (_I, [_P, _L, _L, _L, _P, _L, _P, _P, _P]),
    "lsa_rows_linear": (_I, [_P, _I, _I, _L, _L, _I, _P, _I, _I, _P, _P, _P]),
    "lsa_pool_keys": (_I, [_P, _I, _L, _I, _I, _P, _P]),
    "lsa_ward_merge_workspace_bytes": (_Z, [_L, _I, _I]),
    "lsa_ward_merge": (_I, [_P, _P, _F, _L, _I, _I, _I, _F, _I, _P, _P, _P, _P, _Z, _P]),
    "lsa_bucket_table": (_I, [_P, _I, _P, _L, _I, _I, _I, _I, _I, _L, _P, _P, _P, _P, _P, _P, _P]),
    "lsa_kmeans_update": (_I, [_P, _P, _P, _I, _I, _P, _P]),
    "lsa_gather_sum": (_I, [_P, _I, _P, _I, _L, _I, _I, _L, _P, _P]),
    "lsa_flat_select": (_I, [_P, _L, _I, _P, _L, _P, _P, _I, c_int32, _P, _P, _P]),
    "lsa_scan_centre": (_I, [_P, _L, _I, _P, _P, _P, _P, _P]),
    "lsa_scan_select_workspace_bytes": (_Z, [_L, _I, _L]),
    "lsa_scan_select": (_I, [_P, _L, _I, _P, _P, _P, _P, _L, _P, _P, _I, c_int32, _I, _P, _P, _P, _P, _Z, _P]),
    "lsa_dense_scores": (_I, [_P, _L, _I, _P, _P, _I, _I, _P, _L, c_int32, _P, _P, _P]),
    "lsa_flat_select_decode_workspace_bytes": (_Z, [_L, _I, _I]),
    "lsa_flat_select_decode": (_I, [_P, _L, _I, _P, _P, _P, _I, _I, _P, _P, _P, _Z, _P]),
    "lsa_flat_select_paged": (_I, [_P, _L, _I, _P, _L, _P, _I, _I, _P, _I, _I, _P, _P, _P, _Z, _P]),
    "lsa_merge_candidates": (_I, [_P, _I, _L, _I, _P, _P, _P]),
    "lsa_shape_build": (_I, [_P, _L, _L, _P, _P, _L, _I, _I, _I, _P, _P, _P, _P]),
    "lsa_shaped_select": (_I, [_P, _L, _I, _P, _L, _P, _P, _P, _I, _F, _P, _P, _I, c_int32, _P, _P, _P]),
    "lsa_shaped_select_decode": (_I, [_P, _L, _I, _P, _P, _P, _P, _I, _F, _P, _P, _I, _I, _P, _P, _P, _Z, _P]),
    "lsa_shaped_select_paged": (_I, [_P, _L, _I, _P, _L, _P, _P, _P, _I, _F, _P, _I, _I, _P, _I, _I, _P, _P, _P, _Z,
                                     _P]),
    "lsa_shaped_scores": (_I, [_P, _L, _I, _P, _L, _P, _P, _P, _I, _F, _P, _L, _P, _P]),
    "lsa_page_fingerprints": (_I, [_P, _L, _I, _P, _L, _L, _I, _P, _P, _P, _P, _P]),
    "lsa_beam_step": (_I, [_P, _L, _I, _P, _L, _P, _I, _P, _P, _I, _P, _I, _P, _P, _P, _P]),
    "lsa_beam_step_workspace_bytes": (_Z, [_L, _I, _I]),
    "lsa_beam_step_split": (_I, [_P, _L, _I, _P, _L, _P, _I, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "lsa_expand": (_I, [_P, _L, _I, _P, _P, _L, _I, _P, _P, _I, _I, _I, _P, _I, _L, _L, _I, _I, _I, _I, _P, _P, _P,
                        _P]),
    "lsa_expand_batched": (_I, [_P, _L, _I, _P, _P, _L, _I, _P, _P, _I, _I, _I, _P, _I, _L, _L, _I, _I, _I, _I, _P, _L, _P,
                                _L, _I, _I, _P, _P, _P, _P]),
    "lsa_sparse_attend_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "lsa_sparse_attend": (_I, [_P, _L, _I, _I, _L, _L, _P, _P, _L, _L, _I, _L, _L, _P, _L, _P, _P, _P, _F, _I, _P, _P,
                               _P, _P, _Z, _P]),
    "lsa_band_attend": (_I, [_P, _L, _I, _I, _L, _L, _P, _P, _L, _I, _L, _L, _L, _I, _I, _F, _P, _P, _I, _P, _P]),
    "lsa_sparse_attend_static_scratch_bytes": (_Z, []),
    "lsa_sparse_attend_static": (_I, [_P, _L, _I, _I, _L, _L, _P, _P, _L, _L, _I, _L, _L, _P, _L, _P, _F, _I, _P, _P,
                                      _P, _P]),
    "lsa_latent_attend_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "lsa_latent_attend": (_I, [_P, _L, _I, _I, _I, _L, _L, _P, _L, _L, _P, _L, _P, _F, _I, _P, _P, _P, _I, _I, _I, _I,
                               _P, _P, _Z, _P]),
    "lsa_bucket_attend_workspace_bytes": (_Z, [_L, _I, _I, _I, _L]),
    "lsa_bucket_attend": (_I, [_P, _L, _I, _I, _L, _L, _P, _P, _L, _I, _L, _L, _P, _I, _P, _P, _L, _I, _P, _P, _I, _I, _I,
                               _P, _P, _F, _P, _P, _I, _P, _P, _P, _Z, _P]),
    "lsa_lse_merge": (_I, [_P, _I, _P, _I, _L, _I, _P, _P, _P, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the kernel library, or raise: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"lsa_b200: the CUDA kernel library {LIB_PATH} is not built - run "
                "`python latent-sparse-attention_b200/build.py` (there is no CPU fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        if lib.lsa_abi_version() != ABI_VERSION:
            raise RuntimeError(f"lsa_b200: {LIB_PATH} has ABI {lib.lsa_abi_version()}, the binding wants {ABI_VERSION}")
        _lib = lib
    return _lib


class Address(int):
    """A device address that keeps its tensor alive: a tensor converted inline in an argument list
    (`ptr(x.to(torch.int32))`) must outlive the launch it is passed to, or the caching allocator may hand its block
    to the next conversion of the same call."""

    def __new__(cls, tensor: torch.Tensor):
        self = super().__new__(cls, tensor.data_ptr())
        self.tensor = tensor
        return self


def ptr(tensor: torch.Tensor | None) -> Address | None:
    """Device address of a tensor (None passes NULL). Refuses anything that is not CUDA memory."""
    if tensor is None:
        return None
    if not tensor.is_cuda:
        raise RuntimeError("lsa_b200 kernels take CUDA tensors only - there is no CPU path")
    return Address(tensor)


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(tensor: torch.Tensor) -> int:
    if tensor.dtype == torch.float32:
        return DTYPE_F32
    if tensor.dtype == torch.bfloat16:
        return DTYPE_BF16
    raise ValueError(f"expected float32 or bfloat16 - got {tensor.dtype}")


# Kernel launches made through this binding since import (a benchmark reads it before and after a step).
LAUNCHES = 0


def call(name: str, *args, launches: int = 1):
    """Call an entry point that returns a status code; raise on a refusal."""
    global LAUNCHES
    code = getattr(load(), name)(*args)
    LAUNCHES += launches
    if code != 0:
        reason = load().lsa_error_string(code).decode()
        kind = ValueError if code in (-1, -2, -3, -4, -7) else RuntimeError
        raise kind(f"{name} refused the call: {reason} (code {code})")


def query(name: str, *args) -> int:
    """Call a size query."""
    return int(getattr(load(), name)(*args))
