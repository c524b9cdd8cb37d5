"""The allocation-free min/max entry point (lyap_minmax_device_noalloc).

Some hosts may not allocate device memory when they call into the library (fixed memory budget, real-time
frame loop, plug-in rules), so this entry point keeps its reduction scratch in a fixed array inside the
library.  The test drives it through the C ABI and checks it against the ordinary entry point
(lyap_minmax_device), bit for bit, on two calls in a row that share that array; the second call has
different data and a different size, so anything left over from the first would show."""
import ctypes

import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L

pytestmark = pytest.mark.gpu


def reference_minmax(engine, buf, offset_values, n, out):
    engine.minmax_device(buf.ptr + 8 * offset_values, n, out.ptr)
    return out.to_host(np.float64)


def test_noalloc_minmax_matches_regular_entry_point_twice(engine):
    rng = np.random.default_rng(12)
    n1, n2 = 3_000_001, 70_003
    v = rng.uniform(-6.0, 2.0, size=n1)
    v[::101] = -5.0                      # sentinels are filtered out (<= -4)
    v[7], v[8], v[9] = np.nan, np.inf, -np.inf
    buf = engine.alloc(8 * n1)           # the caller's own buffers; the entry point under test allocates nothing
    buf.from_host(v)
    want, got = engine.alloc(16), engine.alloc(16)

    # first call: whole array
    w1 = reference_minmax(engine, buf, 0, n1, want).copy()
    engine.sync()
    L.minmax_device_noalloc(buf.ptr, n1, got.ptr, engine_stream(engine))
    device_synchronize()
    g1 = got.to_host(np.float64).copy()
    assert np.array_equal(g1.view(np.uint64), w1.view(np.uint64))
    sel = v[np.isfinite(v) & (v > -4.0)]
    assert g1[0] == sel.min() and g1[1] == sel.max()

    # second call straight after, other data and size, same fixed scratch
    w2 = reference_minmax(engine, buf, 1_000_000, n2, want).copy()
    engine.sync()
    L.minmax_device_noalloc(buf.ptr + 8 * 1_000_000, n2, got.ptr, engine_stream(engine))
    device_synchronize()
    g2 = got.to_host(np.float64).copy()
    assert np.array_equal(g2.view(np.uint64), w2.view(np.uint64))
    assert not np.array_equal(g1, g2)

    # nothing passes the filter -> the reference's starting values (+max, lowest)
    buf.from_host(np.full(1000, -5.0))
    L.minmax_device_noalloc(buf.ptr, 1000, got.ptr, engine_stream(engine))
    device_synchronize()
    g3 = got.to_host(np.float64)
    assert g3[0] == np.finfo(np.float64).max and g3[1] == -np.finfo(np.float64).max
    for b in (buf, want, got):
        b.free()


def engine_stream(engine):
    """The entry point takes a raw cudaStream_t; the test uses NULL (the default stream)."""
    return None


def device_synchronize():
    """The engine's own stream does not wait for default-stream work, so the test waits for the device itself
    before it reads a result back through the engine."""
    cudart = ctypes.CDLL("libcudart.so.12")
    assert cudart.cudaDeviceSynchronize() == 0


def test_noalloc_rejects_oversize_and_null(engine):
    lib = engine.lib
    out = engine.alloc(16)
    st = lib.lyap_minmax_device_noalloc(out.ptr, L.NOALLOC_MAX_VALUES + 1, out.ptr, None)
    assert st == 3 and b"LYAP_NOALLOC_MAX_VALUES" in lib.lyap_last_error()
    assert lib.lyap_minmax_device_noalloc(out.ptr, 10, None, None) == 1
    assert lib.lyap_minmax_device_noalloc(None, 10, out.ptr, None) == 1
    out.free()


def test_noalloc_on_a_caller_stream_two_calls_in_order(engine):
    """The documented use: the caller's own (non-blocking) stream, two calls back to back on it with nothing in
    between -- the second starts from the scratch the first left -- then one wait for the stream."""
    cudart = ctypes.CDLL("libcudart.so.12")
    stream = ctypes.c_void_p()
    assert cudart.cudaStreamCreateWithFlags(ctypes.byref(stream), 1) == 0      # cudaStreamNonBlocking
    rng = np.random.default_rng(99)
    n1, n2 = 1_200_007, 333_331
    v = rng.uniform(-7.0, 1.5, size=n1 + n2)
    v[::53] = -5.0
    buf = engine.alloc(8 * (n1 + n2))
    buf.from_host(v)
    want1, want2, got1, got2 = (engine.alloc(16) for _ in range(4))
    w1 = reference_minmax(engine, buf, 0, n1, want1).copy()
    w2 = reference_minmax(engine, buf, n1, n2, want2).copy()
    engine.sync()
    L.minmax_device_noalloc(buf.ptr, n1, got1.ptr, stream)
    L.minmax_device_noalloc(buf.ptr + 8 * n1, n2, got2.ptr, stream)
    assert cudart.cudaStreamSynchronize(stream) == 0
    g1, g2 = got1.to_host(np.float64), got2.to_host(np.float64)
    assert np.array_equal(g1.view(np.uint64), w1.view(np.uint64))
    assert np.array_equal(g2.view(np.uint64), w2.view(np.uint64))
    assert cudart.cudaStreamDestroy(stream) == 0
    for b in (buf, want1, want2, got1, got2):
        b.free()
