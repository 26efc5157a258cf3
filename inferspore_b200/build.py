"""Builds libispore_kernels.so (sm_100a only) in-tree with nvcc.

    python -m inferspore_b200.build [--force] [--verbose]

Each csrc/*.cu is compiled to an object under build/ (skipped when the object is
newer than the source and every header), then linked into
inferspore_b200/lib/libispore_kernels.so.  nvcc cross-compiles without a GPU.
`-Xptxas -v` output (registers, spills, shared memory per kernel) is kept next
to the objects as <name>.ptxas.txt.

The same objects also go into one static archive per kernel under
inferspore_b200/lib/static/, named after the reference's per-kernel CMake
targets (src/kernels/CMakeLists.txt:1-69 of m0dulo/InferSpore: embeddingFunctor,
qkv_bias_and_rope, concat_kv, mask_softmax, fused_addresidual_norm, act, topk,
...), so that a build of the reference that links `-lact` or `-ltopk` keeps its
link lines: each archive holds the objects its launcher needs plus the
library-level object (error text, stream, status word).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
OBJ_DIR = ROOT / "build" / "ispore_obj"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libispore_kernels.so"
STATIC_DIR = LIB_DIR / "static"

# reference CMake target (src/kernels/CMakeLists.txt) -> our objects that implement its launcher
ARCHIVES = {
    "embeddingFunctor": ["embedding"],
    "cal_paddingoffset": ["layout_ops"],
    "build_casual_mask": ["layout_ops"],
    "qkv_bias_and_rope": ["qkv_rope"],
    "concat_kv": ["concat_kv"],
    "repeat_kv": ["layout_ops"],
    "mask_softmax": ["softmax"],
    "fused_transpose_and_remv_pad": ["layout_ops"],
    "fused_addresidual_norm": ["rmsnorm"],
    "act": ["act"],
    "topk": ["topk"],
    "fused_decoder_self_attention": ["decoder_mha"],
}
COMMON_OBJECTS = ["c_api"]  # error text, thread-local stream, device status word, occupancy cache

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xptxas",
    "-v",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or add /usr/local/cuda/bin to PATH)")


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile_one(nvcc: str, src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ_DIR / (src.stem + ".ptxas.txt")).write_text(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return obj


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every kernel source for sm_100a and links the shared library."""
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    headers = _headers()
    todo = [s for s in sources if force or _stale(OBJ_DIR / (s.stem + ".o"), [s, *headers])]
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        list(pool.map(lambda s: _compile_one(nvcc, s, verbose), todo))
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if force or todo or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        if verbose:
            print(" ".join(cmd), flush=True)
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    build_archives(force=force or bool(todo))
    return LIB_PATH


def build_archives(force: bool = False) -> list[Path]:
    """One static archive per reference CMake target from the objects already compiled."""
    STATIC_DIR.mkdir(parents=True, exist_ok=True)
    out = []
    for target, stems in ARCHIVES.items():
        path = STATIC_DIR / f"lib{target}.a"
        objs = [OBJ_DIR / f"{stem}.o" for stem in stems + COMMON_OBJECTS]
        missing = [o for o in objs if not o.exists()]
        if missing:
            raise RuntimeError(f"archive {target}: objects missing: {missing}")
        if force or _stale(path, objs):
            path.unlink(missing_ok=True)
            proc = subprocess.run(["ar", "rcs", str(path), *map(str, objs)], capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"ar failed for {target}:\n{proc.stderr}")
        out.append(path)
    return out


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true", help="rebuild every object")
    ap.add_argument("--verbose", action="store_true", help="print the nvcc command lines")
    args = ap.parse_args(argv)
    print(build_library(force=args.force, verbose=args.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
