"""ctypes binding of libpe_b200.so, the C-ABI CUDA library (include/pe_b200.h).

There is no CPU or PyTorch fallback behind these calls: if the shared library is
missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

from .errors import PackedEncodersError

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libpe_b200.so"

PE_OK = 0
PE_ERR_ARG = -1
PE_ERR_CUDA = -2
PE_ERR_WORKSPACE = -3
PE_ERR_DEVICE = -4
PE_ERR_UNSUPPORTED = -5
_ERR_NAMES = {
    PE_ERR_ARG: "PE_ERR_ARG",
    PE_ERR_CUDA: "PE_ERR_CUDA",
    PE_ERR_WORKSPACE: "PE_ERR_WORKSPACE",
    PE_ERR_DEVICE: "PE_ERR_DEVICE",
    PE_ERR_UNSUPPORTED: "PE_ERR_UNSUPPORTED",
}
OPT_FUSED_GEGLU = 1
OPT_FUSED_ROPE = 2
OPT_GEMM_PAIR = 3
OPT_FUSED_RESIDUAL = 4


class NativeLibraryError(PackedEncodersError):
    """The CUDA library could not be loaded, or one of its calls failed."""


class PeLayerWeights(Structure):
    _fields_ = [
        ("attn_norm_w", c_void_p),
        ("wqkv", c_void_p),
        ("wo", c_void_p),
        ("mlp_norm_w", c_void_p),
        ("wi", c_void_p),
        ("wo_mlp", c_void_p),
        ("is_global", c_int32),
        ("reserved", c_int32),
    ]


class PeModel(Structure):
    _fields_ = [
        ("hidden", c_int32),
        ("n_heads", c_int32),
        ("head_dim", c_int32),
        ("intermediate", c_int32),
        ("n_layers", c_int32),
        ("vocab", c_int32),
        ("half_window", c_int32),
        ("max_positions", c_int32),
        ("eps", c_float),
        ("reserved", c_float),
        ("tok_emb", c_void_p),
        ("emb_norm_w", c_void_p),
        ("final_norm_w", c_void_p),
        ("rope_global", c_void_p),
        ("rope_local", c_void_p),
        ("layers", POINTER(PeLayerWeights)),
    ]


# name -> (restype, argtypes); mirrors include/pe_b200.h one to one.
PROTOTYPES = {
    "pe_version": (c_int, []),
    "pe_last_error": (c_char_p, []),
    "pe_device_check": (c_int, []),
    "pe_set_option": (c_int, [c_int, c_int]),
    "pe_unpad_build": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, POINTER(c_int32), c_void_p]),
    "pe_gather_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "pe_repad_scatter": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "pe_gather_rows_counted": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "pe_repad_scatter_counted": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                         c_void_p]),
    "pe_rope_table": (c_int, [c_float, c_int, c_void_p, c_void_p]),
    "pe_embed_ln": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int, c_int, c_void_p,
                            c_void_p, c_void_p]),
    "pe_add_ln": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int, c_void_p, c_void_p,
                          c_void_p]),
    "pe_rope_qk_inplace": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p,
                                   c_void_p]),
    "pe_geglu": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "pe_gemm_bf16_tn": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                c_void_p]),
    "pe_gemm_geglu_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                   c_void_p]),
    "pe_gemm_qkv_rope_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                      c_void_p, c_int, c_void_p, c_void_p]),
    "pe_gemm_residual_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                      c_void_p, c_void_p]),
    "pe_gemm_l2norm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "pe_pool_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "pe_pool_packed": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_size_t, c_void_p]),
    "pe_attn_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pe_attn_varlen": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                               c_void_p, c_size_t, c_void_p, c_void_p]),
    "pe_attn_varlen_static": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p]),
    "pe_forward_workspace_bytes": (c_size_t, [POINTER(PeModel), c_int64, c_int]),
    "pe_forward_packed": (c_int, [POINTER(PeModel), c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                  c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "pe_forward_packed_pooled": (c_int, [POINTER(PeModel), c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                         c_int, c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p]),
    "pe_read_status": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
}

_lib = None


def load(path: os.PathLike | str | None = None) -> ctypes.CDLL:
    """Load the library (once) and attach the prototypes. Raises if it is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    lib_path = Path(path) if path is not None else LIB_PATH
    if not lib_path.exists():
        raise NativeLibraryError(
            f"{lib_path} is missing: build it with `python flash-modernbert_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback path."
        )
    try:
        lib = ctypes.CDLL(str(lib_path))
    except OSError as exc:
        raise NativeLibraryError(f"could not load {lib_path}: {exc}") from exc
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise NativeLibraryError(f"{lib_path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _lib = lib
    return lib


def last_error() -> str:
    msg = load().pe_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    """Raise for a non-zero return code of a library call."""
    if rc == PE_OK:
        return
    raise NativeLibraryError(f"{what} failed with {_ERR_NAMES.get(rc, rc)}: {last_error()}")


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor, None for None."""
    return None if t is None else t.data_ptr()


def current_stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
