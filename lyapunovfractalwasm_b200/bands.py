"""Row-band sharding of one frame over ranks (one process per GPU).

A pixel's exponent depends only on its global (column, row) index, so a frame splits into
contiguous row bands with no data exchange for lambda.  The colour stage needs two things from
outside a band:
  * the whole frame's min/max (normalizeData, reference src/lyapunov_fractal.hpp:110-125): one
    all-reduce of two doubles (min, max are selections, so the result is exact in any order);
  * the neighbour bands' edge rows for the 3x3 mean (web/fractal_renderer.js:283-311): these are
    RECOMPUTED (one halo row above and below, same bits because lambda is a pure function of the
    global index) rather than exchanged.  Halo rows do not enter this rank's min/max.

`render_band` is written against a small backend interface so the same orchestration runs on the
GPU engine (GpuBackend, below) and, in the CPU tests, on a stand-in.
"""

import numpy as np


def band_rows(height, world_size, rank):
    """Rows [begin, end) owned by `rank`: contiguous, sizes differ by at most one row."""
    base, extra = divmod(height, world_size)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin, end


def halo_rows(height, begin, end):
    """(rows_above, rows_below): 1 where a neighbour row exists in the frame, else 0."""
    return (1 if begin > 0 else 0), (1 if end < height else 0)


def frame_for_rank(frame_index, world_size):
    """Round-robin owner of a frame in a batch (zoom sequences)."""
    return frame_index % world_size


def render_band(backend, params_kw, rank, world_size, allreduce_minmax, palette=0):
    """Render rank's band of the frame described by params_kw (keywords of make_params).

    allreduce_minmax(local_min, local_max) -> (global_min, global_max); the only exchange.
    Returns the backend's handle for (lambda_band, norm_band, rgba_band) and the band's row range.
    """
    height = params_kw["height"]
    begin, end = band_rows(height, world_size, rank)
    above, below = halo_rows(height, begin, end)
    lam = backend.lambda_rows(params_kw, begin - above, end + below)       # band plus halo rows
    own = backend.rows_view(lam, above, end - begin)
    lo, hi = backend.minmax(own)
    glo, ghi = allreduce_minmax(lo, hi)
    norm = backend.normalize(lam, glo, ghi)                                 # halo rows too
    rgba = backend.colorize(norm, above, end - begin, above, below, palette)
    return {"lambda": own, "norm": backend.rows_view(norm, above, end - begin), "rgba": rgba,
            "rows": (begin, end), "minmax": (glo, ghi)}


class GpuBackend:
    """render_band backend on one Engine; handles are (DeviceBuffer, row_offset, rows, width)."""

    def __init__(self, engine, make_params):
        self.e = engine
        self.make_params = make_params
        self.d_minmax = engine.alloc(16)
        self.steps = engine.alloc(8)
        self.steps.from_host(np.zeros(1, dtype=np.uint64))

    def lambda_rows(self, params_kw, r0, r1):
        kw = dict(params_kw, row_begin=r0, row_end=r1)
        p = self.make_params(**kw)
        w = p.width
        buf = self.e.alloc((r1 - r0) * w * 8)
        self.e.lambda_device(p, buf.ptr, None, self.steps.ptr)
        return (buf, 0, r1 - r0, w)

    @staticmethod
    def rows_view(handle, first, rows):
        buf, off, _n, w = handle
        return (buf, off + first, rows, w)

    @staticmethod
    def _ptr(handle):
        buf, off, _rows, w = handle
        return buf.ptr + off * w * 8

    def minmax(self, handle):
        _buf, _off, rows, w = handle
        self.e.minmax_device(self._ptr(handle), rows * w, self.d_minmax.ptr)
        mm = self.d_minmax.to_host(np.float64)
        return float(mm[0]), float(mm[1])

    def normalize(self, handle, lo, hi):
        _buf, _off, rows, w = handle
        self.d_minmax.from_host(np.array([lo, hi], dtype=np.float64))
        out = self.e.alloc(rows * w * 8)
        self.e.normalize_device(self._ptr(handle), rows * w, self.d_minmax.ptr, out.ptr)
        return (out, 0, rows, w)

    def colorize(self, norm_handle, first, rows, above, below, palette):
        buf, off, _rows, w = norm_handle
        rgba = self.e.alloc(rows * w * 4)
        self.e.colorize_device(buf.ptr + (off + first) * w * 8, w, rows, above, below, palette, rgba.ptr)
        return (rgba, rows, w)

    def executed_steps(self):
        return int(self.steps.to_host(np.uint64)[0])

    @staticmethod
    def to_host(handle, dtype=np.float64):
        if len(handle) == 3:
            buf, rows, w = handle
            return buf.to_host(np.uint8, rows * w * 4).reshape(rows, w, 4)
        buf, off, rows, w = handle
        return buf.to_host(dtype, rows * w, off * w * 8).reshape(rows, w)
