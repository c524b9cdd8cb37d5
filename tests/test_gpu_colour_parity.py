"""GPU parity of the colour stage on the large benchmark frames: normalizeData's whole-frame min/max
(reference src/lyapunov_fractal.hpp:110-125), its map (:127-137) and the page's 3x3 mean + palette + byte store
(web/fractal_renderer.js:283-311,207-281,191-198), against the CPU oracle.  Bar: identical fp64 words and bytes."""
import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L
from conftest import CONFIGS, config5_frame

pytestmark = pytest.mark.gpu


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint64), b.view(np.uint64))


def oracle_rows(port, kw, **rows):
    return port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                            kw["sequence"], kw["iterations"], kw["warmup"], c=kw.get("c"), **rows)


@pytest.mark.parametrize("k", [0, 33, 255])
def test_config5_frames_whole(engine, port, k):
    """Zoom-batch frames 0 (a third of the pixels escape), 33 (the last frame that still reaches a > 4) and 255, whole:
    lambda, executed steps, min/max, normalised grid and RGBA against the oracle."""
    kw = config5_frame(k)
    r = engine.render(L.make_params(**kw), want=("lambda", "norm", "rgba"))
    lam, steps = oracle_rows(port, kw)
    assert same_bits(r["lambda"], lam) and r["stats"].executed_steps == steps
    assert (r["stats"].lambda_min, r["stats"].lambda_max) == port.minmax(lam)
    norm = port.normalize(lam)
    assert same_bits(r["norm"], norm)
    assert np.array_equal(r["rgba"], port.colorize(norm, 0))


def check_blocks(port, kw, frame_mm, norm, rgba, blocks):
    """Row blocks [y0, y1) of a frame whose normalised grid and RGBA are in `norm` / `rgba`: the oracle renders lambda for
    the block plus one row either side, normalises it with the frame's min/max and colours it; the block's own rows of
    the 3x3 mean see exactly those rows."""
    lo, hi = frame_mm
    H = kw["height"]
    seen_lo, seen_hi = np.inf, -np.inf
    for y0, y1 in blocks:
        a, b = max(0, y0 - 1), min(H, y1 + 1)
        lam, _ = oracle_rows(port, kw, y0=a, y1=b)
        mn, mx = port.minmax(lam)
        seen_lo, seen_hi = min(seen_lo, mn), max(seen_hi, mx)
        want_norm = port.normalize(lam, lo, hi)
        assert same_bits(norm[a:b], want_norm), (y0, y1)
        want_rgba = port.colorize(want_norm, 0)
        # rows whose three neighbour rows are all inside [a, b), or cut by the image edge exactly as in the frame
        first = y0 - a if a > 0 else 0
        last = (y1 - a) if b < H else (b - a)
        assert np.array_equal(rgba[a + first:a + last], want_rgba[first:last]), (y0, y1)
    # the frame's extremes bound every sampled row's (they are equal only if the extreme pixel was sampled)
    assert lo <= seen_lo and hi >= seen_hi


def test_config3_colour_stage_one_device_and_two_bands(engine, port):
    """16384^2, "BBBBBBAAAAAA", 500 + 4000: the whole frame on the device, then sampled row blocks of the normalised grid
    and of the RGBA bytes against the oracle -- first, last, interior, and the rows either side of the band edge of a
    two-band render (lyap_multi_render, both bands on this device), whose bytes must equal the one-device frame's."""
    kw = CONFIGS[3]
    one = engine.render(L.make_params(**kw), want=("norm", "rgba"))
    mm = (one["stats"].lambda_min, one["stats"].lambda_max)
    blocks = [(0, 2), (5000, 5002), (8190, 8194), (16382, 16384)]
    check_blocks(port, kw, mm, one["norm"], one["rgba"], blocks)
    with L.Multi([0, 0]) as m:
        two = m.render(L.make_params(**kw), want=("norm", "rgba"))
    assert (two["stats"].lambda_min, two["stats"].lambda_max) == mm
    assert two["stats"].executed_steps == one["stats"].executed_steps
    assert same_bits(two["norm"], one["norm"])
    assert np.array_equal(two["rgba"], one["rgba"])


def test_fp32_lambda_on_config3_and_config4_bands(engine, port):
    """(float)lambda beside the fp64 value, on bands of the two largest frames."""
    for cfg, y0, y1 in ((3, 12287, 12290), (4, 49151, 49153)):
        kw = CONFIGS[cfg]
        r = engine.render(L.make_params(**kw, row_begin=y0, row_end=y1), want=("lambda", "lambda32"))
        want, steps = oracle_rows(port, kw, y0=y0, y1=y1)
        assert same_bits(r["lambda"], want) and r["stats"].executed_steps == steps
        assert r["lambda32"].dtype == np.float32 and np.array_equal(r["lambda32"], want.astype(np.float32))


def test_config4_colour_stage_on_a_band_with_given_minmax(engine, port):
    """65536-wide rows: the device entry points on a band (normalise with a supplied min/max, colour with neighbour rows
    present above and below) against the oracle on the same rows."""
    kw = CONFIGS[4]
    y0, y1 = 32766, 32770          # straddles the 2-, 4- and 8-band boundary at row 32768
    W = kw["width"]
    rows = y1 - y0
    lam, _ = oracle_rows(port, kw, y0=y0, y1=y1)
    mn, mx = -3.9, 1.0             # any fixed pair: the band path takes the frame's min/max from outside
    d_lam, d_norm = engine.alloc(rows * W * 8), engine.alloc(rows * W * 8)
    d_rgba, d_mm = engine.alloc((rows - 2) * W * 4), engine.alloc(16)
    engine.lambda_device(L.make_params(**kw, row_begin=y0, row_end=y1), d_lam.ptr)
    d_mm.from_host(np.array([mn, mx]))
    engine.normalize_device(d_lam.ptr, rows * W, d_mm.ptr, d_norm.ptr)
    engine.colorize_device(d_norm.ptr + W * 8, W, rows - 2, 1, 1, 0, d_rgba.ptr)
    engine.sync()
    want_norm = port.normalize(lam, mn, mx)
    assert same_bits(d_lam.to_host(np.float64).reshape(rows, W), lam)
    assert same_bits(d_norm.to_host(np.float64).reshape(rows, W), want_norm)
    assert np.array_equal(d_rgba.to_host(np.uint8).reshape(rows - 2, W, 4), port.colorize(want_norm, 0)[1:-1])
    for b in (d_lam, d_norm, d_rgba, d_mm):
        b.free()
