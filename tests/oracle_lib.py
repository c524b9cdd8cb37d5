"""ctypes access to the CPU checkers under oracle/ (test infrastructure only).

`port`  -- oracle/liboracle_port.so, this project's restatement (always present after build()).
`ref(kind)` -- oracle/_ref/libref_{lyapmath,stock}.so, the unmodified reference header; built only
where the reference sources exist, shipped prebuilt otherwise.  Returns None when absent.
"""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
c_double_p = ctypes.POINTER(ctypes.c_double)
c_u8_p = ctypes.POINTER(ctypes.c_uint8)
c_u64_p = ctypes.POINTER(ctypes.c_uint64)

PALETTES = ["cosmic", "nebula", "aurora", "solarflare", "blackhole", "psychedelic", "rainbow"]


def _dp(a):
    return a.ctypes.data_as(c_double_p)


class Port:
    def __init__(self):
        path = os.path.join(ROOT, "oracle", "liboracle_port.so")
        self.lib = L = ctypes.CDLL(path)
        for n in ("oracle_log", "oracle_exp", "oracle_sin", "oracle_cos"):
            getattr(L, n).restype = ctypes.c_double
            getattr(L, n).argtypes = [ctypes.c_double]
        L.oracle_pow.restype = ctypes.c_double
        L.oracle_pow.argtypes = [ctypes.c_double, ctypes.c_double]
        L.oracle_hash64.restype = ctypes.c_uint64
        L.oracle_hash64.argtypes = [c_u64_p, ctypes.c_uint64]
        L.oracle_lambda_rows.restype = ctypes.c_uint64
        L.oracle_lambda_rows.argtypes = [ctypes.c_double] * 4 + [ctypes.c_int] * 2 + [
            ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_double,
            ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, c_double_p]
        L.oracle_minmax.argtypes = [c_double_p, ctypes.c_uint64, c_double_p, c_double_p]
        L.oracle_normalize_with.argtypes = [c_double_p, ctypes.c_uint64, ctypes.c_double, ctypes.c_double,
                                            c_double_p]
        L.oracle_normalize.argtypes = [c_double_p, ctypes.c_uint64, c_double_p]
        L.oracle_box3.argtypes = [c_double_p, ctypes.c_int, ctypes.c_int, c_double_p]
        L.oracle_colorize.argtypes = [c_double_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, c_u8_p]
        L.oracle_palette.argtypes = [ctypes.c_double, ctypes.c_int, c_u8_p]
        L.oracle_glow.argtypes = [c_u8_p, ctypes.c_int, ctypes.c_int, c_u8_p]

    def hash64(self, arr):
        a = np.ascontiguousarray(arr)
        assert a.nbytes % 8 == 0
        return int(self.lib.oracle_hash64(a.ctypes.data_as(c_u64_p), a.nbytes // 8))

    def lambda_rows(self, min_x, max_x, min_y, max_y, width, height, sequence, iterations, warmup,
                    c=None, y0=0, y1=None, row_stride=1):
        """Rows y0, y0+stride, ... < y1 (global indices) -> (array [nrows, width], executed steps)."""
        y1 = height if y1 is None else y1
        nrows = max(0, (y1 - y0 + row_stride - 1) // row_stride)
        out = np.empty((nrows, width), dtype=np.float64)
        seq = sequence.encode("latin-1")
        steps = self.lib.oracle_lambda_rows(min_x, max_x, min_y, max_y, width, height, seq, len(seq), iterations,
                                            warmup, 0 if c is None else 1, 0.0 if c is None else c, y0, y1,
                                            row_stride, _dp(out))
        return out, int(steps)

    def minmax(self, v):
        v = np.ascontiguousarray(v, dtype=np.float64)
        mn, mx = ctypes.c_double(), ctypes.c_double()
        self.lib.oracle_minmax(_dp(v), v.size, ctypes.byref(mn), ctypes.byref(mx))
        return mn.value, mx.value

    def normalize(self, v, mn=None, mx=None):
        v = np.ascontiguousarray(v, dtype=np.float64)
        out = np.empty_like(v)
        if mn is None:
            self.lib.oracle_normalize(_dp(v), v.size, _dp(out))
        else:
            self.lib.oracle_normalize_with(_dp(v), v.size, mn, mx, _dp(out))
        return out

    def box3(self, v):
        v = np.ascontiguousarray(v, dtype=np.float64)
        h, w = v.shape
        out = np.empty_like(v)
        self.lib.oracle_box3(_dp(v), w, h, _dp(out))
        return out

    def colorize(self, norm, palette=0):
        norm = np.ascontiguousarray(norm, dtype=np.float64)
        h, w = norm.shape
        out = np.empty((h, w, 4), dtype=np.uint8)
        self.lib.oracle_colorize(_dp(norm), w, h, palette, out.ctypes.data_as(c_u8_p))
        return out

    def glow(self, rgba):
        rgba = np.ascontiguousarray(rgba, dtype=np.uint8)
        h, w, _ = rgba.shape
        out = np.empty_like(rgba)
        self.lib.oracle_glow(rgba.ctypes.data_as(c_u8_p), w, h, out.ctypes.data_as(c_u8_p))
        return out

    def palette(self, t, palette):
        rgb = (ctypes.c_uint8 * 3)()
        self.lib.oracle_palette(t, palette, rgb)
        return tuple(rgb)


class Ref:
    """The unmodified reference header behind three C entry points."""

    def __init__(self, path):
        self.lib = L = ctypes.CDLL(path)
        L.ref_compute_fractal.restype = ctypes.c_int
        L.ref_compute_fractal.argtypes = [ctypes.c_double] * 4 + [ctypes.c_int] * 2 + [
            ctypes.c_char_p, ctypes.c_int, ctypes.c_int, c_double_p]
        L.ref_normalize.restype = ctypes.c_int
        L.ref_normalize.argtypes = [c_double_p, ctypes.c_uint64, c_double_p]
        L.ref_default_params.argtypes = [c_double_p, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
        L.ref_omp_max_threads.restype = ctypes.c_int
        L.ref_omp_set_threads.argtypes = [ctypes.c_int]

    def max_threads(self):
        """Threads the header's OpenMP loop uses when it is on (it is off for frames of 100 rows or fewer, :40)."""
        return int(self.lib.ref_omp_max_threads())

    def set_threads(self, n):
        self.lib.ref_omp_set_threads(int(n))

    def compute_fractal(self, min_x, max_x, min_y, max_y, width, height, sequence, iterations, warmup):
        out = np.empty((height, width), dtype=np.float64)
        n = self.lib.ref_compute_fractal(min_x, max_x, min_y, max_y, width, height, sequence.encode("latin-1"),
                                         iterations, warmup, _dp(out))
        assert n == width * height
        return out

    def normalize(self, v):
        v = np.ascontiguousarray(v, dtype=np.float64)
        out = np.empty_like(v)
        self.lib.ref_normalize(_dp(v), v.size, _dp(out))
        return out

    def default_params(self):
        f4 = (ctypes.c_double * 4)()
        i4 = (ctypes.c_int * 4)()
        seq = ctypes.create_string_buffer(64)
        self.lib.ref_default_params(f4, i4, seq, 64)
        return list(f4), list(i4), seq.value.decode()


_port = None


def port():
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref(kind="lyapmath"):
    path = os.path.join(ROOT, "oracle", "_ref", "libref_%s.so" % kind)
    if not os.path.exists(path):
        return None
    return Ref(path)
