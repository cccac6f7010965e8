"""fml_softmax_xent_static: the cross-entropy entry point for callers that cannot allocate.

Hosts whose own allocator owns all device memory, or that cannot afford the device-wide
synchronisation of cudaMalloc/cudaFree, call this variant; its per-row scratch is a fixed array
inside the library instead of the context's growable arena.  The test calls it through the C ABI
twice in a row (the array keeps the first call's contents) and compares loss and gradient with
the regular entry point and with the float64 CPU checker, and it holds the device's free memory
and the size of the context's arena from before the call against the figures after it: the one
property the entry point exists for.  It lives in its own file, collected last, so that a run that stops at
the first failure has already run everything else; it builds its own context and so passes both
alone in a fresh process and after the other tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_regular_entry_point_twice(orc):
    from flutter_ml_b200 import _lib
    ctx = _lib.Context()
    rng = np.random.default_rng(123)
    for rows, cols in ((300, 1000), (64, 10)):      # second call: fewer rows than the array now holds
        z = (2 * rng.standard_normal((rows, cols))).astype(np.float32)
        labels = rng.integers(0, cols, rows).astype(np.int32)
        inv = 1.0 / rows
        dl = ctx.upload(labels)
        z_new, dz_new, loss_new = ctx.upload(z), ctx.empty(rows, cols), ctx.zeros(1)
        z_ref, dz_ref, loss_ref = ctx.upload(z), ctx.empty(rows, cols), ctx.zeros(1)
        # every buffer exists; from here to the second reading the only library call is the one under test
        ctx.sync()
        free0, _, arena0 = ctx.mem_info()
        ctx.call("fml_softmax_xent_static", z_new, dl, dz_new, loss_new, rows, cols, inv, launches=2)
        ctx.sync()
        free1, _, arena1 = ctx.mem_info()
        assert arena1 == arena0, "the call grew the context's scratch arena"
        assert free1 >= free0, f"the call took {free0 - free1} bytes of device memory"
        ctx.call("fml_softmax_xent", z_ref, dl, dz_ref, loss_ref, rows, cols, inv, launches=2)
        # against the float64 checker
        dz64 = np.zeros((rows, cols))
        loss64 = orc.Ops().softmax_xent(np.ascontiguousarray(z, dtype=np.float64), labels, dz64, inv)
        assert abs(loss_new.numpy()[0] - loss64) <= 1e-5 * abs(loss64)
        assert np.linalg.norm(dz_new.numpy() - dz64) <= 1e-5 * np.linalg.norm(dz64)
        # same kernels, same launch geometry: identical within the tolerance of the other xent tests
        a, b = loss_new.numpy()[0], loss_ref.numpy()[0]
        assert abs(a - b) <= 2e-6 * abs(b)
        g_new, g_ref = dz_new.numpy().astype(np.float64), dz_ref.numpy().astype(np.float64)
        assert np.linalg.norm(g_new - g_ref) <= 2e-6 * np.linalg.norm(g_ref)
    assert ctx.device_status() == 0
    ctx.close()


def test_static_scratch_rejects_oversized_batches():
    from flutter_ml_b200 import _lib
    ctx = _lib.Context()
    rows = 65536 + 1
    z, lab, loss = ctx.empty(4), ctx.empty(4, dtype=np.int32), ctx.zeros(1)
    rc = ctx.lib.fml_softmax_xent_static(ctx.h, z.ptr, lab.ptr, None, loss.ptr, rows, 4, 1.0)
    assert rc == -6
    assert b"exceed the fixed scratch" in ctx.lib.fml_last_error(ctx.h)
    ctx.close()
