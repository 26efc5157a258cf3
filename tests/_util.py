"""Helpers shared by the GPU parity tests: tolerances as the task states them."""
import numpy as np
import torch

REL_F32 = 1e-5   # fp32 outputs: relative
ABS_F16 = 2e-3   # fp16 outputs: absolute, against the fp32-accumulated oracle value


def dev(a, device="cuda:0"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def host(t):
    return t.detach().cpu().numpy()


def randn16(rng, shape, scale=1.0):
    return (rng.standard_normal(shape, dtype=np.float32) * scale).astype(np.float16)


def assert_close_f32(got, want, floor=0.0, what=""):
    """|got - want| <= 1e-5 * max(|want|, floor) element-wise.  `floor` (scalar or array) is the
    magnitude below which the relative test would only measure cancellation noise."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    bound = REL_F32 * np.maximum(np.abs(want), floor)
    bad = ~(np.abs(got - want) <= bound)
    if bad.any():
        i = np.argmax(np.abs(got - want) - bound)
        raise AssertionError(
            f"{what}: {bad.sum()} of {bad.size} elements beyond 1e-5 relative; worst at flat index {i}: "
            f"got {got.flat[i]!r} want {want.flat[i]!r} bound {np.broadcast_to(bound, got.shape).flat[i]!r}")


def half_ulp(v):
    """Half the spacing of binary16 at |v| (normal range; subnormal spacing below 2^-14)."""
    a = np.maximum(np.abs(np.asarray(v, np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(a)) - 11)


def assert_close_f16(got_half, want_f32, want_half=None, what=""):
    """fp16 output vs the oracle's UNROUNDED fp32 value: |got - want| <= 2e-3 absolute.  Where a
    half cannot represent the value that closely (|want| >= 8: half spacing 2^-7 or more) the bound
    is the rounding error of one half conversion, and such elements are counted and must be large.
    Returns (max_abs_err, number of elements over 2e-3, fraction bit-identical to want_half)."""
    got = np.asarray(got_half).astype(np.float64)
    want = np.asarray(want_f32, np.float64)
    err = np.abs(got - want)
    bound = np.maximum(ABS_F16, half_ulp(want) + 1e-5 * np.abs(want))
    bad = ~(err <= bound)
    if bad.any():
        i = np.argmax(err - bound)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements out of tolerance; worst at {i}: "
                             f"got {got.flat[i]!r} want {want.flat[i]!r}")
    over = err > ABS_F16
    if over.any():
        assert np.abs(want[over]).min() >= 8.0, f"{what}: element over 2e-3 that a half could have represented"
    same = None
    if want_half is not None:
        same = float(np.mean(np.asarray(got_half).view(np.uint16) == np.asarray(want_half).view(np.uint16)))
    return float(err.max()), int(over.sum()), same
