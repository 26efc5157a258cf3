"""Generates tests/golden/ref_cpu_vectors.npz from the reference's own CPU functions.

    python tests/golden/make_golden.py

Needs oracle/_ref/ (built by oracle/build.py where the reference tree is
mounted).  The functions run are the unmodified CPUSwiGLU, cpuEmbedding,
CPUfusedresidandRMSNorm and CPUfunc of the reference's tests/unittests/*.cu;
inputs are seeded and stored next to the outputs so the file is self-contained.
tests/test_oracle_vs_ref.py checks the oracle against this file on machines
where the reference tree (and therefore oracle/_ref/) is absent.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import binding as orc  # noqa: E402

OUT = Path(__file__).resolve().parent / "ref_cpu_vectors.npz"


def rope_case(rng, batch, seq, heads, hist):
    """Inputs for CPUfunc (head size is fixed at 128 by its `+ 64`, test_bias_and_RoPE.cu:41,62).
    Returns the flat buffer CPUfunc reads plus the q / k inputs it effectively uses."""
    d = 128
    buf = rng.standard_normal(batch * seq * 3 * heads * d).astype(np.float32)
    qb, kb = seq * heads * d, seq * heads * d
    q_in = np.empty((batch, seq, heads, d), np.float32)
    k_in = np.empty((batch, seq, heads, d), np.float32)
    for b in range(batch):
        for s in range(seq):
            for h in range(heads):
                q0 = b * qb + s * heads * d + h * d            # test_bias_and_RoPE.cu:36-37
                k0 = b * kb + s * (2 * heads) * d + h * d      # :56-57
                q_in[b, s, h] = buf[q0:q0 + d]
                k_in[b, s, h] = buf[k0:k0 + d]
    return buf, q_in, k_in, np.asarray(hist, np.int32)


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    act32 = (rng.standard_normal((4, 2, 96)) * 3).astype(np.float32)
    act16 = (rng.standard_normal((4, 2, 96)) * 3).astype(np.float16)
    out["act_in_f32"], out["act_out_f32"] = act32, orc.ref_cpu_swiglu(act32)
    out["act_in_f16"], out["act_out_f16"] = act16, orc.ref_cpu_swiglu(act16)

    table = rng.standard_normal((50, 32)).astype(np.float32)
    ids = rng.integers(0, 50, 16).astype(np.int32)
    out["emb_table"], out["emb_ids"], out["emb_out"] = table, ids, orc.ref_cpu_embedding(ids, table)

    # constant rows, zero residual / bias: the only inputs CPUfusedresidandRMSNorm is defined for
    consts = rng.standard_normal(4).astype(np.float32) * 2
    x = np.repeat(consts[:, None], 64, 1).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, 64).astype(np.float32)
    out["norm_x"], out["norm_scale"] = x, scale
    out["norm_out"] = orc.ref_cpu_fused_resid_rmsnorm(np.zeros_like(x), x, np.zeros(64, np.float32), scale, 1e-6)

    buf, q_in, k_in, hist = rope_case(rng, 2, 6, 2, [3, 0])
    q, k = orc.ref_cpu_qkv_rope(buf.reshape(2 * 6, 6, 128), np.zeros(6 * 128, np.float32), hist, 2, 6, 2, 2, 128,
                                128, 10000.0)
    out["rope_q_in"], out["rope_k_in"], out["rope_hist"], out["rope_q"], out["rope_k"] = q_in, k_in, hist, q, k
    np.savez_compressed(OUT, **out)
    print(OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
