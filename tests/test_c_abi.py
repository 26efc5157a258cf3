"""The C-ABI shared library: loads, exports every declared symbol, and rejects bad
arguments with an error code before it touches a device.  No GPU needed."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "ispore_kernels.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ispore_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    from inferspore_b200 import capi

    assert declared_symbols() == capi.exported_symbols()


def test_library_exports_every_declared_symbol(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(Path(lib._name))], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (ispore_\w+)", out))
    assert set(declared_symbols()) <= exported
    # nothing but the C ABI leaks out of the library
    leaked = [s for s in re.findall(r" [TDB] (\w+)", out) if not s.startswith("ispore_") and not s.startswith("_")]
    assert leaked == []


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "ispore_kernels.h"\nint main(void){return ISPORE_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{HEADER.parent}", "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_version_and_stream_roundtrip(lib):
    assert lib.ispore_version() >= 100
    lib.ispore_set_stream(C.c_void_p(0x1234))
    assert lib.ispore_get_stream() == 0x1234
    lib.ispore_set_stream(None)
    assert lib.ispore_get_stream() in (None, 0)


def test_bad_arguments_return_codes_without_a_device(lib):
    from inferspore_b200 import capi

    one = C.c_void_p(0x1000)  # never dereferenced: every call below fails validation first
    assert lib.ispore_silu_mul_f32(None, one, 4, 8, None) == capi.ISPORE_ENULL
    assert lib.ispore_silu_mul_f16(one, one, -1, 8, None) == capi.ISPORE_ESHAPE
    assert lib.ispore_add_residual_rmsnorm_f32(one, None, None, None, 1e-6, 4, 8, None) == capi.ISPORE_ENULL
    assert lib.ispore_add_residual_rmsnorm_f16(one, None, None, one, 1e-6, 4, 0, None) == capi.ISPORE_ESHAPE
    assert lib.ispore_input_embedding_f32(one, one, None, 1, 8, 0, None) == capi.ISPORE_ENULL
    assert lib.ispore_concat_kv_f16(one, one, one, one, one, one, 3, 2, 1, 1, 1, 8, 8, None) == capi.ISPORE_ESHAPE
    assert lib.ispore_scale_mask_softmax_f32(one, one, one, 1, 0, 1, 8, 1.0, None) == capi.ISPORE_ESHAPE
    assert lib.ispore_topk_f32(one, 1, 100, 300, one, one, 8, one, one, 0, None, 1.0, None, None) == capi.ISPORE_ELIMIT
    # a uniform without a place for the sampled ids
    assert lib.ispore_topk_f32(one, 1, 100, 5, None, None, 0, one, one, 0, one, 1.0, None, None) == capi.ISPORE_ENULL
    assert lib.ispore_topk_f32(one, 1, 100, 5, None, None, 0, one, one, -1, None, 1.0, None, None) == capi.ISPORE_ESHAPE
    assert lib.ispore_sampling_f32(one, one, one, one, 1, 5, 0.0, None) == capi.ISPORE_ESHAPE
    # rotary dim larger than the head / odd head size
    args = [one] * 8 + [1, 4, 4, 2, 2, 8]
    assert lib.ispore_qkv_bias_rope_transpose_f32(*args, 16, 10000.0, 4096, 0, None) == capi.ISPORE_ESHAPE
    assert b"rotary" in lib.ispore_last_error_string()
    # empty inputs are fine and launch nothing
    assert lib.ispore_silu_mul_f32(one, one, 0, 8, None) == capi.ISPORE_OK
    assert lib.ispore_concat_kv_f32(one, one, one, one, one, one, 0, 1, 0, 1, 1, 8, 8, None) == capi.ISPORE_OK


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from inferspore_b200 import capi

    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        capi.load()


def test_ops_refuse_cpu_tensors():
    import torch

    from inferspore_b200 import ops

    with pytest.raises(ValueError, match="CUDA tensors"):
        ops.launchAct(torch.zeros(2, 2, 8), torch.zeros(2, 8))
