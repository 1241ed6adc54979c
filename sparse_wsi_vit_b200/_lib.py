"""ctypes binding of libswv_b200.so (the C ABI declared in include/swv_b200.h).

There is no fallback: if the library is missing or was built without a symbol
the import fails loudly.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SWV_B200_LIB") or os.path.join(_HERE, "csrc", "libswv_b200.so")

SWV_F32, SWV_BF16, SWV_F16 = 0, 1, 2

EXPORTS = [
    "swv_version", "swv_strerror", "swv_dsa_workspace_bytes", "swv_dsa_mask_bytes",
    "swv_dsa_indexer_topk_fwd", "swv_dsa_attn_gather_fwd", "swv_dsa_attn_masked_fwd",
    "swv_dsa_indexer_topk_static_fwd", "swv_block_sparse_attn_fwd", "swv_rope2d_apply", "swv_pool_tokens",
    "swv_nsa_importance_bytes", "swv_nsa_select_blocks_fwd", "swv_nsa_selected_attn_fwd", "swv_nsa_combine_fwd",
    "swv_nsa_workspace_bytes", "swv_nsa_attn_fwd", "swv_dsa_attn_scratch_bytes", "swv_dsa_attn_masked_count_fwd",
    "swv_dsa_attn_bwd", "swv_dsa_indexer_bwd", "swv_dsa_prologue_fwd", "swv_dsa_attn_lists_fwd",
    "swv_dsa_attn_lists_scratch_bytes", "swv_dsa_workspace_bytes_topk",
]


class SwvError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python sparse_wsi_vit_b200/csrc/build.py` "
            "(there is no CPU or PyTorch fallback for this package)")
    lib = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it with `python sparse_wsi_vit_b200/csrc/build.py --force`")
    i64p = POINTER(c_int64)
    lib.swv_version.restype = c_int
    lib.swv_strerror.restype = c_char_p
    lib.swv_strerror.argtypes = [c_int]
    lib.swv_dsa_workspace_bytes.argtypes = [c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_dsa_mask_bytes.argtypes = [c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_dsa_indexer_topk_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.swv_dsa_indexer_topk_static_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.swv_block_sparse_attn_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_int, c_void_p, c_void_p, i64p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.swv_pool_tokens.argtypes = [c_void_p, i64p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.swv_rope2d_apply.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, c_int64, c_int, c_int, c_float, c_float, c_int, c_void_p]
    lib.swv_dsa_attn_gather_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, i64p, c_void_p, i64p, c_void_p, i64p,
        c_void_p, i64p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.swv_dsa_attn_masked_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_void_p, i64p, c_int,
        c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.swv_dsa_attn_lists_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, i64p,
        c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
    lib.swv_dsa_attn_lists_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_dsa_workspace_bytes_topk.argtypes = [c_int, c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_dsa_attn_masked_count_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_void_p, i64p, c_int,
        c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    lib.swv_dsa_attn_bwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, i64p, c_int, c_void_p, i64p,
        c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_int, c_void_p, c_void_p]
    lib.swv_dsa_indexer_bwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, c_void_p, i64p, c_void_p, i64p, c_void_p,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.swv_dsa_prologue_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, i64p, c_void_p, i64p, c_int, c_void_p, c_void_p, c_float,
        c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]
    lib.swv_dsa_attn_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_nsa_importance_bytes.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_size_t)]
    lib.swv_nsa_select_blocks_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
        c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
    lib.swv_nsa_selected_attn_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
        c_int, c_void_p, c_void_p]
    lib.swv_nsa_combine_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p]
    lib.swv_nsa_workspace_bytes.argtypes = [c_int] * 10 + [POINTER(c_size_t)]
    lib.swv_nsa_attn_fwd.argtypes = [
        c_void_p, i64p, c_void_p, i64p, c_void_p, i64p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
        c_int, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
    for name in EXPORTS[2:]:
        getattr(lib, name).restype = c_int
    return lib


lib = _load()


def strerror(code: int) -> str:
    return lib.swv_strerror(int(code)).decode()


def check(rc: int, what: str):
    if rc != 0:
        raise SwvError(f"{what}: {strerror(rc)} (code {rc})")


def strides(t, n=None):
    s = t.stride()
    return (c_int64 * len(s))(*s)


def dtype_code(dt):
    import torch
    try:
        return {torch.float32: SWV_F32, torch.bfloat16: SWV_BF16, torch.float16: SWV_F16}[dt]
    except KeyError:
        raise SwvError(f"unsupported dtype {dt}") from None
