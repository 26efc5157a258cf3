"""Host-side behaviour of the drop-in C++ headers (inferspore_b200/compat): they build with a
plain host compiler, keep the reference's wrapper semantics, and throw std::runtime_error for
the checks the reference launchers make — all before any CUDA call.  No GPU needed."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

PROGRAM = r"""
#include <cstdio>
#include <stdexcept>
#include "src/kernels/act_kernel.h"
#include "src/kernels/attn_softmax_kernel.h"
#include "src/kernels/build_casual_mask.h"
#include "src/kernels/cal_paddingoffset.h"
#include "src/kernels/concat_past_kv.h"
#include "src/kernels/fused_addresidual_norm.h"
#include "src/kernels/fused_transpose_and_remv_pad.h"
#include "src/kernels/input_embedding.h"
#include "src/kernels/qkv_bias_and_RoPE.h"
#include "src/kernels/repeat_kv.h"
#include "src/kernels/topK.h"
#include "src/weights/llama/attention_weights.h"
#include "src/weights/llama/ffn_weights.h"
#include "src/utils/params.h"

template <typename F> static bool throws(F f) {
    try { f(); } catch (const std::runtime_error&) { return true; }
    return false;
}
#define EXPECT(c) do { if (!(c)) { std::printf("FAILED line %d: %s\n", __LINE__, #c); return 1; } } while (0)

int main() {
    float dummy[64] = {0};
    int idummy[8] = {0};
    // wrapper semantics (reference: src/utils/tensor.h)
    EXPECT(getTensorType<float>() == FP32 && getTensorType<half>() == FP16 && getTensorType<int>() == INT32);
    EXPECT(getTensorType<const float>() == FP32 && getTensorType<double>() == UNSUPPORTED);
    TensorWrapper<float> t(GPU, FP32, {4, 2, 8}, dummy);
    EXPECT(t.size() == 64 && t.numel() == 64 && t.getPtr() == dummy && t.getPtrByOffset(3) == dummy + 3);
    EXPECT(throws([&] { TensorWrapper<float> bad(GPU, FP16, {1}, dummy); }));   // dtype mismatch
    EXPECT(throws([&] { (void)t.getVal(); }));                                   // host read of a GPU tensor
    TensorWrapper<int> layer(CPU, INT32, {1}, idummy);
    EXPECT(layer.getVal() == 0);
    TensorWrapper<float> empty(GPU, FP32, {4});
    EXPECT(empty.size() == 0 && empty.data == nullptr);
    Tensor big(GPU, FP16, {32, 64, 32, 4096, 128});
    EXPECT(big.numel() == (1ll << 35));
    TensorMap m{{"a", &t}};
    EXPECT(m.isExist("a") && !m.isExist("b") && m.size() == 1 && m.at("a") == &t);
    EXPECT(throws([&] { m.at("zzz"); }));
    EXPECT(throws([&] { TensorMap bad{{"e", &empty}}; }));
    EXPECT(t.toString().find("FP32") != std::string::npos && t.DeviceString() == "GPU");
    BaseWeight<float> w;
    EXPECT(w.bias == nullptr && w.data == nullptr);                              // no indeterminate pointers
    LLaMAattentionWeights<half> aw; LLaMAFFNWeights<half> fw; (void)aw; (void)fw;
    EXPECT(Vec<float>::size == 4 && Vec<half>::size == 2);

    // launcher checks fire before anything reaches CUDA
    TensorWrapper<float> out(GPU, FP32, {4, 8}, dummy);
    TensorWrapper<float> wrong(GPU, FP32, {4, 3, 8}, dummy);
    EXPECT(throws([&] { launchAct(&wrong, &out); }));                            // shape[1] != 2 (act_kernel.cu:61)
    TensorWrapper<int> ids(GPU, INT32, {5}, idummy);
    EmbeddingWeight<float> table; table.data = dummy;
    EXPECT(throws([&] { launchInputEmbedding(&ids, &out, &table); }));           // 5 ids vs 4 rows (input_embedding.cu:35)
    TensorWrapper<int> gpu_layer(GPU, INT32, {1}, idummy);
    TensorWrapper<float> ksrc(GPU, FP32, {1, 1, 2, 4}, dummy), kdst(GPU, FP32, {1, 1, 4, 4}, dummy);
    EXPECT(throws([&] { launchConcatKVCache(&ksrc, &ksrc, &gpu_layer, &ids, &ids, &kdst, &kdst); }));  // layer id must be on the CPU
    TensorWrapper<float> null_out(GPU, FP32, {4, 8});
    BaseWeight<float> norm;
    EXPECT(throws([&] { launchFusedAddBiasResidualRMSNorm(&null_out, &null_out, norm, (float*)nullptr, 1e-6f); }));
    TensorWrapper<float> probs(GPU, FP32, {2, 100}, dummy);
    TensorWrapper<int> fid(GPU, INT32, {2, 300}, idummy);
    TensorWrapper<float> fval(GPU, FP32, {2, 300}, dummy);
    EXPECT(throws([&] { launchTopKforBeamSearch(&probs, &fid, &fval, &fid, &fval); }));  // K = 300 > limit
    TensorWrapper<int> po(GPU, INT32, {3, 5}, idummy), cum3(GPU, INT32, {3}, idummy), len3(GPU, INT32, {3}, idummy);
    EXPECT(throws([&] { launchCalPaddingoffset(&po, &cum3, &len3); }));          // cum_seqlens must be [bs + 1] (cal_paddingoffset.cu:36)
    TensorWrapper<float> cache4(GPU, FP32, {1, 2, 4, 4}, dummy);
    EXPECT(throws([&] { launchRepeatKVCache(&cache4, &cache4, &ids, &layer, &cache4, &cache4); }));  // source caches carry a layer axis
    std::printf("compat ok\n");
    return 0;
}
"""


def test_compat_headers_host_only(tmp_path):
    src = tmp_path / "compat_host.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "compat_host"
    lib_dir = ROOT / "inferspore_b200" / "lib"
    cmd = ["g++", "-std=c++11", "-Wall", f"-I{ROOT / 'inferspore_b200' / 'compat'}", f"-I{ROOT / 'include'}",
           "-I/usr/local/cuda/include", str(src), "-o", str(exe), f"-L{lib_dir}", "-lispore_kernels",
           f"-Wl,-rpath,{lib_dir}"]
    subprocess.run(cmd, check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "compat ok" in out.stdout, out.stdout + out.stderr


def test_reference_unit_tests_build_unmodified():
    """oracle/build.py compiles eleven of the reference's unit tests, untouched, against the
    drop-in headers; here: the binaries exist and link to our library (they run in the gpu suite)."""
    dropin = ROOT / "oracle" / "_ref" / "dropin"
    if not dropin.is_dir():
        pytest.skip("reference tree absent: nothing was built")
    for name in ["test_fused_addresidual_norm", "test_act", "test_input_embedding", "test_concat_kv",
                 "test_mask_softmax", "test_bias_and_RoPE", "test_casual_mask", "test_cal_paddingoffset",
                 "test_fused_trans_remv_pad", "test_repeat_kv", "test_fused_decoder_attention"]:
        exe = dropin / name
        assert exe.exists(), name
        ldd = subprocess.run(["ldd", str(exe)], capture_output=True, text=True).stdout
        assert "libispore_kernels.so" in ldd and "not found" not in ldd.split("libispore_kernels.so")[1].split("\n")[0]


def test_per_kernel_static_archives_carry_the_reference_target_names(tmp_path):
    """inferspore_b200/build.py emits one archive per CMake target of the reference's
    src/kernels/CMakeLists.txt; each defines the C-ABI symbols its launcher template calls, and a
    program that includes every launcher links against all of them together (the shared object
    that several archives contain is pulled once: no duplicate symbols)."""
    from inferspore_b200 import build as lib_build

    static = lib_build.STATIC_DIR
    needs = {
        "embeddingFunctor": ["ispore_input_embedding_f16"],
        "cal_paddingoffset": ["ispore_cal_padding_offset"],
        "build_casual_mask": ["ispore_build_causal_mask_f32"],
        "qkv_bias_and_rope": ["ispore_qkv_bias_rope_transpose_f16", "ispore_rope_decode_f32"],
        "concat_kv": ["ispore_concat_kv_f16"],
        "repeat_kv": ["ispore_repeat_kv_f16"],
        "mask_softmax": ["ispore_scale_mask_softmax_f16", "ispore_scale_causal_softmax_f32"],
        "fused_transpose_and_remv_pad": ["ispore_transpose_remove_padding_f16"],
        "fused_addresidual_norm": ["ispore_add_residual_rmsnorm_f32", "ispore_rmsnorm_f16"],
        "act": ["ispore_silu_mul_f16"],
        "topk": ["ispore_topk_f32", "ispore_topk_merge_f16", "ispore_sampling_f32"],
        "fused_decoder_self_attention": ["ispore_decoder_masked_mha_f16"],
    }
    assert set(needs) == set(lib_build.ARCHIVES)
    for target, symbols in needs.items():
        archive = static / f"lib{target}.a"
        assert archive.exists(), archive
        defined = subprocess.run(["nm", "--defined-only", str(archive)], capture_output=True, text=True).stdout
        for sym in symbols + ["ispore_last_error_string", "ispore_get_stream"]:
            assert f" T {sym}" in defined, (target, sym)
    src = tmp_path / "compat_host.cu"
    src.write_text(PROGRAM)
    exe = tmp_path / "compat_static"
    cmd = [lib_build.find_nvcc(), "-std=c++17", "-w", "-gencode", "arch=compute_100a,code=sm_100a",
           f"-I{ROOT / 'inferspore_b200' / 'compat'}", f"-I{ROOT / 'include'}", str(src), "-o", str(exe), f"-L{static}",
           *[f"-l{t}" for t in needs]]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "compat ok" in out.stdout, out.stdout + out.stderr
