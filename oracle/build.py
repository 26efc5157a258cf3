"""Builds the checker side: the C oracle and, when the reference tree is present,
the reference's own code.

    python oracle/build.py [--ref-root <reference checkout>] [--force]

TEST INFRASTRUCTURE ONLY — nothing under inferspore_b200/ imports this.

1. oracle/ispore_oracle.c  ->  oracle/libispore_oracle.so      (gcc, OpenMP)
2. if the reference tree exists:
   a. oracle/ref_wrap/*.cu + the reference kernel sources they need, compiled
      from where they lie in the reference tree, -> oracle/_ref/libref_*.so.
      These export the reference's CPU functions (from its unit tests) and its
      GPU launchers through a C ABI.
   b. eleven of the reference's unit tests (DROPIN_TESTS), unmodified, compiled against
      inferspore_b200/compat (the drop-in headers) and linked to
      libispore_kernels.so -> oracle/_ref/dropin/test_*.  They are the
      acceptance check that the reference's callers build and run against the
      new library without edits.
   Outputs go only to oracle/_ref/ (git-ignored); no reference source is copied.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
ORACLE_SO = HERE / "libispore_oracle.so"
REF_OUT = HERE / "_ref"


def _default_ref_root() -> Path:
    """The reference checkout: $ISPORE_REFERENCE_ROOT, else `reference_path` of BASELINE.json at the
    repository root.  With neither, a path that does not exist (the reference is then not built)."""
    env = os.environ.get("ISPORE_REFERENCE_ROOT")
    if env:
        return Path(env)
    try:
        import json

        return Path(json.loads((ROOT / "BASELINE.json").read_text())["reference_path"])
    except Exception:
        return ROOT / "_no_reference_tree"


DEFAULT_REF_ROOT = _default_ref_root()

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

# wrapper TU -> reference kernel sources linked into the same shared object
REF_LIBS = {
    "libref_act.so": ("ref_wrap/ref_act.cu", ["src/kernels/act_kernel.cu"]),
    "libref_embedding.so": ("ref_wrap/ref_embedding.cu", ["src/kernels/input_embedding.cu"]),
    "libref_norm.so": ("ref_wrap/ref_norm.cu", ["src/kernels/fused_addresidual_norm.cu"]),
    "libref_rope.so": ("ref_wrap/ref_rope.cu", ["src/kernels/qkv_bias_and_RoPE.cu"]),
    "libref_concat_softmax.so": (
        "ref_wrap/ref_concat_softmax.cu",
        ["src/kernels/concat_past_kv.cu", "src/kernels/attn_softmax_kernel.cu"],
    ),
    "libref_topk.so": ("ref_wrap/ref_topk.cu", ["src/kernels/topK.cu"]),
    "libref_mha.so": ("ref_wrap/ref_mha.cu", []),  # the wrapper includes the kernel file itself
    "libref_layout.so": (
        "ref_wrap/ref_layout.cu",
        ["src/kernels/build_casual_mask.cu", "src/kernels/cal_paddingoffset.cu", "src/kernels/repeat_kv.cu"],
    ),
}

DROPIN_TESTS = [
    "test_fused_addresidual_norm",
    "test_act",
    "test_input_embedding",
    "test_concat_kv",
    "test_mask_softmax",
    "test_bias_and_RoPE",
    "test_casual_mask",
    "test_cal_paddingoffset",
    "test_fused_trans_remv_pad",
    "test_repeat_kv",
    "test_fused_decoder_attention",
]
# The decode attention test calls CHECK_CUDA_ERROR, which no header of the reference defines
# (src/utils/macro.h has CHECK only); the definition comes from the command line, the file is untouched.
# unit test -> the per-kernel static archive it links in the reference's tests/unittests/CMakeLists.txt
STATIC_DROPIN = {"test_act": "act", "test_mask_softmax": "mask_softmax"}
DROPIN_FLAGS = {"test_fused_decoder_attention": ["-DCHECK_CUDA_ERROR(call)=CHECK(call)"]}


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps: list[Path]) -> bool:
    return target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists())


def build_oracle(force: bool = False) -> Path:
    src = HERE / "ispore_oracle.c"
    if force or not _newer(ORACLE_SO, [src]):
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fvisibility=hidden",
              "-Wall", "-o", str(ORACLE_SO), str(src), "-lm"])
    return ORACLE_SO


def build_reference(ref_root: Path = DEFAULT_REF_ROOT, force: bool = False) -> list[Path]:
    """Compiles the reference's own sources (where they lie) into oracle/_ref/."""
    if not (ref_root / "src" / "kernels").is_dir():
        return []
    nvcc = _nvcc()
    REF_OUT.mkdir(exist_ok=True)
    (REF_OUT / "dropin").mkdir(exist_ok=True)
    jobs: list[tuple[Path, list[str]]] = []
    for name, (wrap, kernels) in REF_LIBS.items():
        out = REF_OUT / name
        srcs = [HERE / wrap] + [ref_root / k for k in kernels]
        if force or not _newer(out, srcs):
            jobs.append((out, [nvcc, "-std=c++17", "-O2", *ARCH, "-shared", "-Xcompiler", "-fPIC", "-w",
                               f"-I{ref_root}", f"-I{HERE / 'ref_shim'}", "-o", str(out), *map(str, srcs)]))
    lib_dir = ROOT / "inferspore_b200" / "lib"
    compat = ROOT / "inferspore_b200" / "compat"
    headers = list(compat.rglob("*.h")) + [ROOT / "include" / "ispore_kernels.h", lib_dir / "libispore_kernels.so"]
    for test in DROPIN_TESTS:
        out = REF_OUT / "dropin" / test
        src = ref_root / "tests" / "unittests" / f"{test}.cu"
        if force or not _newer(out, [src, *headers]):
            jobs.append((out, [nvcc, "-std=c++17", "-O2", *ARCH, "-w", *DROPIN_FLAGS.get(test, []), f"-I{compat}",
                               f"-I{ROOT / 'include'}",
                               str(src), "-o", str(out), f"-L{lib_dir}", "-lispore_kernels",
                               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../inferspore_b200/lib"]))
    # The reference links each unit test against one per-kernel static archive (e.g. test_act against
    # `act`, tests/unittests/CMakeLists.txt); the same link line against this library's archives of
    # the same names, without the shared library:
    static_dir = lib_dir / "static"
    for test, archive in STATIC_DROPIN.items():
        out = REF_OUT / "dropin" / f"{test}_static"
        src = ref_root / "tests" / "unittests" / f"{test}.cu"
        if (static_dir / f"lib{archive}.a").exists() and (force or not _newer(out, [src, *headers, static_dir / f"lib{archive}.a"])):
            jobs.append((out, [nvcc, "-std=c++17", "-O2", *ARCH, "-w", f"-I{compat}", f"-I{ROOT / 'include'}", str(src),
                               "-o", str(out), f"-L{static_dir}", f"-l{archive}"]))
    with cf.ThreadPoolExecutor(max_workers=8) as pool:
        list(pool.map(lambda job: _run(job[1]), jobs))
    return ([REF_OUT / n for n in REF_LIBS] + [REF_OUT / "dropin" / t for t in DROPIN_TESTS] +
            [REF_OUT / "dropin" / f"{t}_static" for t in STATIC_DROPIN])


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ref-root", type=Path, default=DEFAULT_REF_ROOT)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    print(build_oracle(args.force))
    for p in build_reference(args.ref_root, args.force):
        print(p)
    return 0


if __name__ == "__main__":
    sys.exit(main())
