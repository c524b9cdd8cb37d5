"""GPU parity: the CUDA engine, called through the C ABI, against the CPU oracle and the golden
vectors made from the unmodified reference header.  Bar: bit-exact (fp64 words, bytes, step counts)."""
import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L
import oracle_lib as O
from conftest import CONFIGS, config5_frame

pytestmark = pytest.mark.gpu


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint64), b.view(np.uint64))


def oracle_rows(port, kw, **rows):
    return port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                            kw["sequence"], kw["iterations"], kw["warmup"], c=kw.get("c"), **rows)


def test_golden_vectors_from_the_reference_header(engine, port, golden):
    """Every golden case: lambda, normalised and RGBA (all 7 palettes) hashes, spot values."""
    for name, case in golden["cases"].items():
        a = case["args"]
        p = L.make_params(*a[:6], sequence=a[6], iterations=a[7], warmup=a[8])
        r = engine.render(p, want=("lambda", "norm"))
        assert "%016x" % port.hash64(r["lambda"]) == case["lyapmath"]["lambda_hash"], name
        assert "%016x" % port.hash64(r["norm"]) == case["lyapmath"]["norm_hash"], name
        for x, y, lh, nh in case["spots"]:
            assert r["lambda"][y, x] == float.fromhex(lh) and r["norm"][y, x] == float.fromhex(nh), (name, x, y)
        for pname, h in case.get("rgba_hash", {}).items():
            assert "%016x" % port.hash64(engine.colorize(r["norm"], pname)) == h, (name, pname)


def test_config1_full_pipeline_bitwise(engine, port):
    kw = CONFIGS[1]
    r = engine.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"))
    lam, steps = oracle_rows(port, kw)
    assert same_bits(r["lambda"], lam)
    assert np.array_equal(r["lambda32"], lam.astype(np.float32))
    norm = port.normalize(lam)
    assert same_bits(r["norm"], norm)
    assert np.array_equal(r["rgba"], port.colorize(norm, 0))
    st = r["stats"]
    assert st.executed_steps == steps and st.nominal_steps == 512 * 512 * 1100
    assert (st.lambda_min, st.lambda_max) == port.minmax(lam)


def test_config2_full_frame_rows_and_properties(engine, port):
    """4096^2 'AABAB' 200+2000: every 64th row against the oracle; the whole frame through
    size-independent properties (band split, min/max of bands, normalise of a band)."""
    kw = CONFIGS[2]
    r = engine.render(L.make_params(**kw), want=("lambda", "norm", "rgba"))
    lam = r["lambda"]
    rows, _ = oracle_rows(port, kw, y0=5, y1=4096, row_stride=64)
    assert same_bits(lam[5:4096:64], rows)
    # bands rendered separately have the whole frame's bits
    for y0, y1 in ((0, 3), (1023, 1026), (4093, 4096)):
        band = engine.compute_fractal(L.make_params(**kw, row_begin=y0, row_end=y1))
        assert same_bits(band, lam[y0:y1])
    mn, mx = port.minmax(lam)
    assert (r["stats"].lambda_min, r["stats"].lambda_max) == (mn, mx)
    sl = slice(2000, 2016)
    assert same_bits(r["norm"][sl], port.normalize(lam[sl], mn, mx))
    # colour rows 2001..2014 depend only on norm rows 2000..2015
    assert np.array_equal(r["rgba"][2001:2015], port.colorize(r["norm"][sl], 0)[1:15])


def band_check(engine, port, kw, bands_to_check):
    for y0, y1 in bands_to_check:
        got = engine.compute_fractal(L.make_params(**kw, row_begin=y0, row_end=y1))
        want, _ = oracle_rows(port, kw, y0=y0, y1=y1)
        assert same_bits(got, want), (y0, y1)


def test_config3_band_edges(engine, port):
    """16384^2, 12-letter sequence, warm-up 500 (accumulation starts at phase 8): the rows either side
    of each of the 8 band boundaries, first and last row."""
    kw = CONFIGS[3]
    edges = [(0, 1)] + [(b * 2048 - 1, b * 2048 + 1) for b in range(1, 8)] + [(16383, 16384)]
    band_check(engine, port, kw, edges)


def test_config4_band_edges(engine, port):
    """65536^2 (more pixels than a 32-bit count holds): rows at the 8-band boundaries."""
    kw = CONFIGS[4]
    edges = [(0, 1), (8191, 8193), (32767, 32769), (57343, 57345), (65535, 65536)]
    band_check(engine, port, kw, edges)


def test_config4_large_band_indexing(engine):
    """A 4096-row band of the 65536-wide frame (2.7e8 pixels, 2 GiB of lambda) equals the same rows
    rendered as two halves: 64-bit indexing and tile walk at full width."""
    kw = CONFIGS[4]
    n = 512
    y0 = 40000
    whole = engine.compute_fractal(L.make_params(**kw, row_begin=y0, row_end=y0 + n))
    a = engine.compute_fractal(L.make_params(**kw, row_begin=y0, row_end=y0 + n // 2 + 1))
    b = engine.compute_fractal(L.make_params(**kw, row_begin=y0 + n // 2 + 1, row_end=y0 + n))
    assert same_bits(whole, np.vstack([a, b]))


def test_config5_zoom_frames_with_c(engine, port):
    """Zoom batch frames 0 (a > 4 columns escape early) and 200, sequence 'ABC' with c = 3.7:
    every 8th row against the oracle, executed-step counts on a band."""
    for k in (0, 200):
        kw = config5_frame(k)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        rows, _ = oracle_rows(port, kw, y0=k % 8, y1=1080, row_stride=8)
        assert same_bits(r["lambda"][k % 8:1080:8], rows), k
        band = L.make_params(**kw, row_begin=500, row_end=516)
        rb = engine.render(band, want=("lambda",))
        want, steps = oracle_rows(port, kw, y0=500, y1=516)
        assert same_bits(rb["lambda"], want) and rb["stats"].executed_steps == steps


def test_ui_production_call_with_mid_run_exits(engine, port):
    """The page's own call (web/fractal_renderer.js:144-154): 800x800, [0,4]^2, warm-up 100, 'AB'.
    Here r < 1 orbits underflow to 0 in mid-accumulation and keep their partial sums."""
    kw = dict(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=800, height=800, sequence="AB", iterations=1000,
              warmup=100)
    r = engine.render(L.make_params(**kw), want=("lambda", "norm", "rgba"))
    lam, steps = oracle_rows(port, kw)
    assert same_bits(r["lambda"], lam) and r["stats"].executed_steps == steps
    assert steps < 800 * 800 * 1100
    norm = port.normalize(lam)
    assert same_bits(r["norm"], norm) and np.array_equal(r["rgba"], port.colorize(norm, 0))


@pytest.mark.parametrize("shape", [(1, 1), (1, 9), (9, 1), (2, 2), (33, 17), (1025, 3), (7, 1031)])
def test_ragged_shapes(engine, port, shape):
    w, h = shape
    kw = dict(min_x=2.4, max_x=4.1, min_y=2.2, max_y=4.05, width=w, height=h, sequence="ABBAB", iterations=70, warmup=19)
    r = engine.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"))
    lam, steps = oracle_rows(port, kw)
    assert same_bits(r["lambda"], lam) and r["stats"].executed_steps == steps
    assert np.array_equal(r["lambda32"], lam.astype(np.float32))
    norm = port.normalize(lam)
    assert same_bits(r["norm"], norm) and np.array_equal(r["rgba"], port.colorize(norm, 0))


def test_step_count_edges(engine, port):
    for warmup, iterations in ((0, 1), (0, 16), (1, 0), (16, 16), (17, 31), (15, 33), (0, 0)):
        kw = dict(min_x=2.6, max_x=4.0, min_y=2.7, max_y=3.9, width=40, height=12, sequence="BA", iterations=iterations,
                  warmup=warmup)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        lam, steps = oracle_rows(port, kw)
        assert same_bits(r["lambda"], lam) and r["stats"].executed_steps == steps, (warmup, iterations)


def test_sequence_rules_on_gpu(engine, port):
    base = dict(min_x=2.6, max_x=3.9, min_y=2.7, max_y=3.8, width=48, height=20, iterations=200, warmup=20)
    a = engine.compute_fractal(L.make_params(**base, sequence="ABC"))
    b = engine.compute_fractal(L.make_params(**base, sequence="ABB"))
    assert same_bits(a, b)                                               # extension off: 'C' is B
    c = engine.compute_fractal(L.make_params(**base, sequence="ABC", c=3.7))
    want, _ = oracle_rows(port, dict(base, sequence="ABC", c=3.7))
    assert same_bits(c, want) and not same_bits(c, b)
    long_seq = "ABBABAABBBAB" * 30 + "A"                                 # 361 letters, longer than the run
    d = engine.compute_fractal(L.make_params(**base, sequence=long_seq))
    want, _ = oracle_rows(port, dict(base, sequence=long_seq))
    assert same_bits(d, want)
    # a negative / zero / huge c sends the orbit out at once; handled by the step-by-step path
    for cval in (-1.0, 0.0, 1e300):
        e = engine.compute_fractal(L.make_params(**base, sequence="ABC", c=cval))
        want, _ = oracle_rows(port, dict(base, sequence="ABC", c=cval))
        assert same_bits(e, want), cval


def test_transpose_symmetry_on_gpu(engine):
    a = engine.compute_fractal(L.make_params(min_x=2.5, max_x=4.0, min_y=3.0, max_y=3.9, width=256, height=256,
                                             sequence="AAB", iterations=300, warmup=50))
    b = engine.compute_fractal(L.make_params(min_x=3.0, max_x=3.9, min_y=2.5, max_y=4.0, width=256, height=256,
                                             sequence="BBA", iterations=300, warmup=50))
    assert same_bits(a, b.T.copy())


def test_extreme_parameters(engine, port):
    """Tiny, huge, negative and NaN-producing windows go through the step-by-step path."""
    for win in ((1e-310, 1e-300, 2.0, 3.0), (1e200, 1e300, 1.0, 2.0), (-1.0, 1.0, -1.0, 1.0), (0.5, 1.5, 1e-3, 0.9)):
        kw = dict(min_x=win[0], max_x=win[1], min_y=win[2], max_y=win[3], width=16, height=8, sequence="AB",
                  iterations=80, warmup=10)
        got = engine.render(L.make_params(**kw), want=("lambda",))
        want, steps = oracle_rows(port, kw)
        assert same_bits(got["lambda"], want) and got["stats"].executed_steps == steps, win


def test_seeded_random_cases_against_the_oracle(engine, port, kernel_path):
    """40 seeded draws of window, shape, sequence (letters A, B, C and a stray byte), step counts and the optional c:
    lambda bits, executed steps, normalised bits and RGBA bytes, with the run-time specialised kernels on and off."""
    rng = np.random.default_rng(20240607)
    for case in range(40):
        lo_x, lo_y = rng.uniform(-0.2, 3.6, size=2)
        kw = dict(min_x=float(lo_x), max_x=float(lo_x + rng.uniform(0.05, 4.3 - lo_x)),
                  min_y=float(lo_y), max_y=float(lo_y + rng.uniform(0.05, 4.3 - lo_y)),
                  width=int(rng.integers(1, 300)), height=int(rng.integers(1, 60)),
                  sequence="".join(rng.choice(list("AABBCx"), size=int(rng.integers(1, 40)))),
                  iterations=int(rng.integers(0, 700)), warmup=int(rng.integers(0, 150)))
        if rng.random() < 0.5:
            kw["c"] = float(rng.uniform(0.5, 4.1))
        kernel_path("jit" if case % 2 else "generic")
        r = engine.render(L.make_params(**kw, palette=case % 7), want=("lambda", "norm", "rgba"))
        lam, steps = oracle_rows(port, kw)
        assert same_bits(r["lambda"], lam) and r["stats"].executed_steps == steps, kw
        norm = port.normalize(lam)
        assert same_bits(r["norm"], norm) and np.array_equal(r["rgba"], port.colorize(norm, case % 7)), kw
