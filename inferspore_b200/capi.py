"""ctypes binding of libispore_kernels.so (the C ABI in include/ispore_kernels.h).

The library is the product; this module only loads it and declares argument
types.  There is no fallback: if the shared library has not been built
(`python -m inferspore_b200.build`) loading raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libispore_kernels.so"

ISPORE_OK = 0
ISPORE_ENULL, ISPORE_ESHAPE, ISPORE_EALIGN, ISPORE_ELAUNCH, ISPORE_ESCRATCH, ISPORE_ELIMIT = -1, -2, -3, -4, -5, -6
DEV_BAD_TOKEN_ID, DEV_KV_OVERRUN, DEV_BAD_PADDING, DEV_TIMEOUT = 1, 2, 4, 8
TOPK_MAX_K = 256

_p, _i64, _i32, _f = C.c_void_p, C.c_int64, C.c_int32, C.c_float

# name -> argument types (the return type is always int unless listed in _RESTYPES)
SIGNATURES: dict[str, list] = {
    "ispore_version": [],
    "ispore_last_error_string": [],
    "ispore_set_stream": [_p],
    "ispore_get_stream": [],
    "ispore_set_programmatic_launch": [C.c_int],
    "ispore_get_programmatic_launch": [],
    "ispore_device_status": [C.POINTER(C.c_uint), C.c_int],
}
_RESTYPES = {"ispore_last_error_string": C.c_char_p, "ispore_set_stream": None, "ispore_get_stream": _p,
             "ispore_set_programmatic_launch": None}

for _t in ("f32", "f16"):
    SIGNATURES[f"ispore_add_residual_rmsnorm_{_t}"] = [_p, _p, _p, _p, _f, _i64, _i64, _p]
    SIGNATURES[f"ispore_rmsnorm_{_t}"] = [_p, _p, _p, _f, _i64, _i64, _p]
    SIGNATURES[f"ispore_input_embedding_{_t}"] = [_p, _p, _p, _i64, _i64, _i64, _p]
    SIGNATURES[f"ispore_qkv_bias_rope_transpose_{_t}"] = (
        [_p] * 8 + [_i64] * 6 + [_i32, _f, _i32, _i32, _p]
    )
    SIGNATURES[f"ispore_rope_decode_{_t}"] = [_p, _i64, _i64, _i64, _i64, _i32, _i32, _f, _p]
    SIGNATURES[f"ispore_silu_mul_{_t}"] = [_p, _p, _i64, _i64, _p]
    SIGNATURES[f"ispore_concat_kv_{_t}"] = [_p] * 6 + [_i64] * 7 + [_p]
    SIGNATURES[f"ispore_scale_mask_softmax_{_t}"] = [_p, _p, _p, _i64, _i64, _i64, _i64, _f, _p]
    SIGNATURES[f"ispore_scale_causal_softmax_{_t}"] = [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _p]
    SIGNATURES[f"ispore_decoder_masked_mha_{_t}"] = [_p] * 5 + [_i64] * 8 + [_i32, _f, _f, _p, _i64, _p]
    SIGNATURES[f"ispore_topk_{_t}"] = [_p, _i64, _i64, _i32, _p, _p, _i32, _p, _p, _i32, _p, _f, _p, _p]
    SIGNATURES[f"ispore_topk_merge_{_t}"] = [_p, _p, _i64, _i32, _i32, _p, _p, _p, _f, _p, _p]
    SIGNATURES[f"ispore_topk_merge_strided_{_t}"] = [_p, _p, _i64, _i32, _i32, _i64, _i64, _i64, _i64, _p, _p, _p, _f, _p, _p]
    SIGNATURES[f"ispore_sampling_{_t}"] = [_p, _p, _p, _p, _i64, _i32, _f, _p]
    SIGNATURES[f"ispore_build_causal_mask_{_t}"] = [_p, _p, _p, _i64, _i64, _i64, _p]
    SIGNATURES[f"ispore_transpose_remove_padding_{_t}"] = [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p]
    SIGNATURES[f"ispore_repeat_kv_{_t}"] = [_p] * 5 + [_i64] * 8 + [_p]

SIGNATURES["ispore_decoder_masked_mha_workspace_bytes"] = [_i64] * 5
_RESTYPES["ispore_decoder_masked_mha_workspace_bytes"] = _i64
SIGNATURES["ispore_cal_padding_offset"] = [_p, _p, _p, _i64, _i64, _p]
SIGNATURES["ispore_topk_static_f32"] = [_p, _i64, _i64, _i32, _p, _p, _i32, _p, _f, _p, _p]
TOPK_STATIC_ENTRIES = 131072

_lib = None


def exported_symbols() -> list[str]:
    """Every symbol include/ispore_kernels.h declares."""
    return sorted(SIGNATURES)


def load() -> C.CDLL:
    """Loads the shared library once; raises if it is missing (no fallback path)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m inferspore_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)"
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = lib
    return _lib


class IsporeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"ispore error {code}: {message}")
        self.code = code


def check(code: int) -> None:
    if code != ISPORE_OK:
        raise IsporeError(code, (load().ispore_last_error_string() or b"").decode())


def device_status(clear: bool = True) -> int:
    flags = C.c_uint(0)
    check(load().ispore_device_status(C.byref(flags), 1 if clear else 0))
    return flags.value
