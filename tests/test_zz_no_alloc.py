"""ispore_topk_static_f32: the top-K entry point for callers that may not allocate.

Some users of the library sample from inside code that is not allowed to touch the device
allocator: a serving loop whose HBM was handed out completely at start-up (a cudaMalloc there can
fail or stall every stream), an "enqueue"-style plugin callback, a latency-critical thread.  For
them the library keeps the round-1 candidate lists in a fixed array of its own instead of
caller-provided scratch.  This test calls that entry point through the C ABI and checks it
 * against the regular entry point (which takes scratch from the caller) and against the CPU
   oracle, bit for bit, on calls in a row with different inputs — a later call finds the earlier
   call's leftovers in the shared array and must not be affected by them;
 * on a shape where the fixed array only has room for two slices per row instead of eight;
 * for the property it exists for: once one warm-up call per device has been made (that call
   loads the CUDA module and looks the array up), further calls leave the device's free memory
   and torch's allocator untouched.
The file sorts last so that a `-x` run has already executed every other test when it gets here;
it also passes on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(rows, K, dev):
    return (torch.full((rows, K), -7, dtype=torch.int32, device=dev),
            torch.full((rows, K), -7.0, dtype=torch.float32, device=dev),
            torch.full((rows,), -7, dtype=torch.int32, device=dev))


def _run_both(lib, capi, logits, K, u, temperature):
    rows, vocab = logits.shape
    dev = torch.device("cuda:0")
    d = torch.from_numpy(logits).to(dev)
    du = torch.from_numpy(u).to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    # regular entry point: scratch [rows, 8, K] from the caller
    sc_i = torch.empty((rows, 8, K), dtype=torch.int32, device=dev)
    sc_v = torch.empty((rows, 8, K), dtype=torch.float32, device=dev)
    ri, rv, rp = _outputs(rows, K, dev)
    capi.check(lib.ispore_topk_f32(d.data_ptr(), rows, vocab, K, sc_i.data_ptr(), sc_v.data_ptr(), 8, ri.data_ptr(),
                                   rv.data_ptr(), 0, du.data_ptr(), temperature, rp.data_ptr(), stream))
    # entry point under test: no scratch argument at all
    si, sv, sp = _outputs(rows, K, dev)
    capi.check(lib.ispore_topk_static_f32(d.data_ptr(), rows, vocab, K, si.data_ptr(), sv.data_ptr(), 0, du.data_ptr(),
                                          temperature, sp.data_ptr(), stream))
    torch.cuda.synchronize()
    return (ri.cpu().numpy(), rv.cpu().numpy(), rp.cpu().numpy()), (si.cpu().numpy(), sv.cpu().numpy(), sp.cpu().numpy())


def test_static_scratch_topk_matches_regular_entry_point_and_oracle(cuda, orc):
    from inferspore_b200 import capi

    lib = capi.load()
    rng = np.random.default_rng(4242)
    # call 1: the headline shape (256 x 32000, K = 50); call 2: other shape, other data, more ties;
    # call 3: rows * K = 65536, so the fixed array holds two slices per row, not eight
    cases = [
        ((rng.standard_normal((256, 32000)) * 2).astype(np.float32), 50, 1.0),
        (np.round(rng.standard_normal((37, 50000)) * 3).astype(np.float32), 64, 0.7),
        ((rng.standard_normal((1024, 9000)) * 2).astype(np.float32), 64, 1.3),
    ]
    assert cases[2][0].shape[0] * cases[2][1] * 2 == capi.TOPK_STATIC_ENTRIES
    for logits, K, temperature in cases:
        u = rng.random(logits.shape[0], dtype=np.float32)
        (ri, rv, rp), (si, sv, sp) = _run_both(lib, capi, logits, K, u, temperature)
        assert np.array_equal(si, ri), "ids differ from the caller-scratch entry point"
        assert np.array_equal(sv.view(np.uint32), rv.view(np.uint32)), "values differ"
        assert np.array_equal(sp, rp), "sampled ids differ"
        assert (si >= 0).all() and (np.diff(sv, axis=1) <= 0).all()
        want_i, want_v = orc.topk(logits, K)
        assert np.array_equal(si, want_i), "ids differ from the oracle"
        assert np.array_equal(sv.view(np.uint32), want_v.view(np.uint32)), "values differ from the oracle"
        want_p, margin = orc.sampling(want_i, want_v, u, temperature)
        decided = margin > 1e-6  # a draw that sits on a CDF boundary may fall either side in fp32
        assert np.array_equal(sp[decided], want_p[decided]), "sampled ids differ from the oracle"


def test_static_scratch_calls_do_not_allocate(cuda):
    """After one warm-up call on the device, further calls change neither the device's free memory
    nor torch's allocator state.  (The warm-up is part of the contract: the first CUDA call into a
    lazily loaded module allocates the module's image, the 1 MiB array included.)"""
    from inferspore_b200 import capi

    lib = capi.load()
    dev = torch.device("cuda:0")
    rows, vocab, K = 64, 32000, 50
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    logits = [torch.randn(rows, vocab, generator=g, device=dev) * 2 for _ in range(2)]
    u = torch.rand(rows, generator=g, device=dev)
    oi, ov, op = _outputs(rows, K, dev)
    stream = torch.cuda.current_stream().cuda_stream

    def call(x):
        capi.check(lib.ispore_topk_static_f32(x.data_ptr(), rows, vocab, K, oi.data_ptr(), ov.data_ptr(), 0,
                                              u.data_ptr(), 1.0, op.data_ptr(), stream))

    call(logits[0])  # warm-up: module load, address look-up, shared-memory attribute
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    allocated_before, reserved_before = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for i in range(4):
        call(logits[i % 2])
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before, f"device free memory moved by {free_before - free_after} bytes"
    assert torch.cuda.memory_allocated(dev) == allocated_before
    assert torch.cuda.memory_reserved(dev) == reserved_before
    assert (oi >= 0).all().item()


def test_static_scratch_limit_is_a_clear_error(cuda):
    from inferspore_b200 import capi

    lib = capi.load()
    rows, K = capi.TOPK_STATIC_ENTRIES // 64 + 1, 64  # one entry too many for even a single slice
    one = C.c_void_p(0x1000)  # never dereferenced: the size check comes first
    rc = lib.ispore_topk_static_f32(one, rows, 1000, K, one, one, 0, None, 1.0, None, None)
    assert rc == capi.ISPORE_ELIMIT
    msg = lib.ispore_last_error_string().decode()
    assert "built-in scratch" in msg and "ispore_topk_f32" in msg
