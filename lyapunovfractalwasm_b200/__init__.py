"""ctypes view of liblyap_b200.so (the C ABI in include/lyap_b200.h).

The product is the shared library and the C++23 header include/lyapunov_fractal.hpp; this module is the
thin Python binding the tests and the benchmark drive it through.  It holds no computation and no
fallback: if the library is missing or no CUDA device answers, calls raise.
"""
import ctypes
import weakref
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblyap_b200.so")

MODE_EXACT, MODE_FAST_FP64, MODE_FAST_FP32, MODE_FAST_FP64_ORBIT = 0, 1, 2, 3
PALETTES = ["cosmic", "nebula", "aurora", "solarflare", "blackhole", "psychedelic", "rainbow"]

c_double_p = ctypes.POINTER(ctypes.c_double)
c_float_p = ctypes.POINTER(ctypes.c_float)
c_u8_p = ctypes.POINTER(ctypes.c_uint8)
c_u64_p = ctypes.POINTER(ctypes.c_uint64)
PROGRESS_FN = ctypes.CFUNCTYPE(None, ctypes.c_double)


class LyapParams(ctypes.Structure):
    """struct lyap_params (include/lyap_b200.h)."""
    _fields_ = [
        ("min_x", ctypes.c_double), ("max_x", ctypes.c_double),
        ("min_y", ctypes.c_double), ("max_y", ctypes.c_double),
        ("width", ctypes.c_int32), ("height", ctypes.c_int32),
        ("sequence", ctypes.c_char_p), ("sequence_len", ctypes.c_int32),
        ("iterations", ctypes.c_int32), ("warmup", ctypes.c_int32),
        ("mode", ctypes.c_int32), ("palette", ctypes.c_int32),
        ("c_enabled", ctypes.c_int32), ("reserved0", ctypes.c_int32),
        ("c_value", ctypes.c_double),
        ("row_begin", ctypes.c_int64), ("row_end", ctypes.c_int64),
    ]


class RenderStats(ctypes.Structure):
    """struct lyap_render_stats."""
    _fields_ = [
        ("executed_steps", ctypes.c_uint64), ("nominal_steps", ctypes.c_uint64),
        ("lambda_min", ctypes.c_double), ("lambda_max", ctypes.c_double),
        ("ms_lambda", ctypes.c_float), ("ms_minmax", ctypes.c_float), ("ms_normalize", ctypes.c_float),
        ("ms_colorize", ctypes.c_float), ("ms_total_device", ctypes.c_float), ("ms_copies", ctypes.c_float),
        ("kernel_launches", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class MultiStats(ctypes.Structure):
    """struct lyap_multi_stats."""
    _fields_ = [
        ("executed_steps", ctypes.c_uint64), ("nominal_steps", ctypes.c_uint64),
        ("lambda_min", ctypes.c_double), ("lambda_max", ctypes.c_double),
        ("ms_wall", ctypes.c_float), ("ms_lambda_max", ctypes.c_float), ("ms_device_max", ctypes.c_float),
        ("ms_gather", ctypes.c_float), ("gather_bytes", ctypes.c_uint64),
        ("kernel_launches", ctypes.c_int32), ("used_nccl", ctypes.c_int32),
    ]


MULTI_GATHER_RGBA, MULTI_GATHER_LAMBDA32, MULTI_HOST_EXCHANGE = 1, 2, 4


class LyapError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("lyap status %d: %s" % (status, message))
        self.status = status


# every symbol include/lyap_b200.h declares: name -> (restype, argtypes)
_P = ctypes.c_void_p
ABI = {
    "lyap_abi_version": (ctypes.c_int, []),
    "lyap_self_test": (ctypes.c_int, []),
    "lyap_last_error": (ctypes.c_char_p, []),
    "lyap_jit_note": (ctypes.c_char_p, []),
    "lyap_last_kernel": (ctypes.c_char_p, []),
    "lyap_multi_create": (ctypes.c_int, [ctypes.POINTER(_P), ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]),
    "lyap_multi_destroy": (ctypes.c_int, [_P]),
    "lyap_multi_note": (ctypes.c_char_p, [_P]),
    "lyap_multi_render": (ctypes.c_int, [_P, ctypes.POINTER(LyapParams), ctypes.c_int32, _P, _P, _P, _P, ctypes.c_double,
                                         ctypes.POINTER(MultiStats)]),
    "lyap_multi_gathered": (ctypes.c_int, [_P, ctypes.POINTER(_P), ctypes.POINTER(_P)]),
    "lyap_multi_render_frames": (ctypes.c_int, [_P, ctypes.POINTER(LyapParams), ctypes.c_int32, ctypes.POINTER(_P),
                                                ctypes.POINTER(_P), ctypes.POINTER(RenderStats)]),
    "lyap_selector_code": (ctypes.c_int, [ctypes.POINTER(LyapParams), ctypes.c_int, ctypes.c_int64, ctypes.POINTER(ctypes.c_int)]),
    "lyap_group_patterns": (ctypes.c_int, [ctypes.POINTER(LyapParams), ctypes.POINTER(ctypes.c_int), c_u64_p, c_u64_p]),
    "lyap_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "lyap_params_default": (None, [ctypes.POINTER(LyapParams)]),
    "lyap_palette_from_name": (ctypes.c_int, [ctypes.c_char_p]),
    "lyap_device_count": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "lyap_create": (ctypes.c_int, [ctypes.POINTER(_P), ctypes.c_int]),
    "lyap_destroy": (ctypes.c_int, [_P]),
    "lyap_set_stream": (ctypes.c_int, [_P, _P]),
    "lyap_sync": (ctypes.c_int, [_P]),
    "lyap_device_alloc": (ctypes.c_int, [_P, ctypes.POINTER(_P), ctypes.c_size_t]),
    "lyap_device_free": (ctypes.c_int, [_P, _P]),
    "lyap_host_alloc": (ctypes.c_int, [ctypes.POINTER(_P), ctypes.c_size_t]),
    "lyap_host_free": (ctypes.c_int, [_P]),
    "lyap_copy_to_host": (ctypes.c_int, [_P, _P, _P, ctypes.c_size_t]),
    "lyap_copy_to_device": (ctypes.c_int, [_P, _P, _P, ctypes.c_size_t]),
    "lyap_lambda_device": (ctypes.c_int, [_P, ctypes.POINTER(LyapParams), _P, _P, _P]),
    "lyap_minmax_device": (ctypes.c_int, [_P, _P, ctypes.c_uint64, _P]),
    "lyap_normalize_device": (ctypes.c_int, [_P, _P, ctypes.c_uint64, _P, _P]),
    "lyap_colorize_device": (ctypes.c_int, [_P, _P, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32,
                                            ctypes.c_int32, ctypes.c_int32, _P]),
    "lyap_compute_fractal": (ctypes.c_int, [_P, ctypes.POINTER(LyapParams), _P, _P]),
    "lyap_normalize_data": (ctypes.c_int, [_P, _P, ctypes.c_uint64, _P]),
    "lyap_colorize": (ctypes.c_int, [_P, _P, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _P]),
    "lyap_glow_device": (ctypes.c_int, [_P, _P, ctypes.c_int32, ctypes.c_int32, _P]),
    "lyap_glow": (ctypes.c_int, [_P, _P, ctypes.c_int32, ctypes.c_int32, _P]),
    "lyap_render": (ctypes.c_int, [_P, ctypes.POINTER(LyapParams), _P, _P, _P, _P, _P,
                                   ctypes.POINTER(RenderStats)]),
    "lyap_render_multi": (ctypes.c_int, [ctypes.POINTER(LyapParams), ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), _P, _P,
                                         _P, ctypes.c_double, ctypes.POINTER(RenderStats)]),
    "lyap_render_frames": (ctypes.c_int, [ctypes.POINTER(LyapParams), ctypes.c_int32, ctypes.c_int32,
                                          ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(_P), ctypes.POINTER(_P),
                                          ctypes.POINTER(RenderStats)]),
    "lyap_minmax_device_noalloc": (ctypes.c_int, [_P, ctypes.c_uint64, _P, _P]),
    "lyap_fp64_peak": (ctypes.c_int, [_P, c_double_p]),
    "lyap_fp32_peak": (ctypes.c_int, [_P, c_double_p]),
}

_lib = None


def load_library():
    """Load liblyap_b200.so and declare every ABI symbol.  Raises if the library is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                "%s is missing: build it with `python -m lyapunovfractalwasm_b200.build` "
                "(there is no fallback implementation)" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in ABI.items():
            fn = getattr(lib, name)   # AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _check(status):
    if status != 0:
        raise LyapError(status, load_library().lyap_last_error().decode("utf-8", "replace"))


def make_params(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=800, height=600, sequence="ABABABAB",
                iterations=10000, warmup=100, mode=MODE_EXACT, palette=0, c=None, row_begin=0, row_end=0):
    """lyap_params with the reference's defaults (src/lyapunov_fractal.hpp:15-25)."""
    p = LyapParams()
    seq = sequence.encode("latin-1") if isinstance(sequence, str) else bytes(sequence)
    p._seq_keepalive = seq
    p.min_x, p.max_x, p.min_y, p.max_y = min_x, max_x, min_y, max_y
    p.width, p.height = width, height
    p.sequence, p.sequence_len = seq, len(seq)
    p.iterations, p.warmup = iterations, warmup
    p.mode = mode
    p.palette = PALETTES.index(palette) if isinstance(palette, str) else palette
    p.c_enabled = 0 if c is None else 1
    p.c_value = 0.0 if c is None else c
    p.row_begin, p.row_end = row_begin, row_end
    return p


def selector_code(params, region, step):
    """lyap_selector_code: the parameter (0 = A, 1 = B, 2 = C) the kernels use at `step` of warm-up (0) / accumulation (1)."""
    code = ctypes.c_int(-1)
    _check(load_library().lyap_selector_code(ctypes.byref(params), region, step, ctypes.byref(code)))
    return code.value


def group_patterns(params):
    """lyap_group_patterns: (groups, warm-up patterns, accumulation patterns) -- the key of a kernel instance for the sequence."""
    kg, wu, acc = ctypes.c_int(-1), ctypes.c_uint64(0), ctypes.c_uint64(0)
    _check(load_library().lyap_group_patterns(ctypes.byref(params), ctypes.byref(kg), ctypes.byref(wu), ctypes.byref(acc)))
    return kg.value, wu.value, acc.value


NOALLOC_MAX_VALUES = 1 << 32


def minmax_device_noalloc(d_values, n, d_minmax, cuda_stream=None):
    """lyap_minmax_device_noalloc on the current device: no context, no allocation (see include/lyap_b200.h)."""
    _check(load_library().lyap_minmax_device_noalloc(d_values, n, d_minmax, cuda_stream))


def render_frames(frames, devices, want=("norm", "rgba"), pinned=False):
    """lyap_render_frames: a list of lyap_params (whole frames) dealt round-robin to the device ordinals.
    Returns ({"norm": [array per frame], "rgba": [...]}, [RenderStats per frame]); with pinned=True the output
    arrays live in page-locked memory (lyap_host_alloc) that is released when the returned arrays are collected."""
    lib = load_library()
    n = len(frames)
    arr = (LyapParams * n)()
    keep = []
    for i, f in enumerate(frames):
        ctypes.memmove(ctypes.byref(arr[i]), ctypes.byref(f), ctypes.sizeof(LyapParams))
        keep.append(f)           # the sequence bytes the copies point to

    def host_array(shape, dtype):
        if not pinned:
            return np.empty(shape, dtype=dtype)
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        ptr = ctypes.c_void_p()
        _check(lib.lyap_host_alloc(ctypes.byref(ptr), nbytes))
        buf = (ctypes.c_uint8 * nbytes).from_address(ptr.value)
        a = np.frombuffer(buf, dtype=dtype).reshape(shape)
        weakref.finalize(buf, lib.lyap_host_free, ptr)
        return a

    out, ptrs = {}, {}
    for key, dtype, tail in (("norm", np.float64, ()), ("rgba", np.uint8, (4,))):
        if key in want:
            out[key] = [host_array((f.height, f.width) + tail, dtype) for f in frames]
            ptrs[key] = (_P * n)(*[a.ctypes.data for a in out[key]])
        else:
            ptrs[key] = None
    devs = (ctypes.c_int32 * len(devices))(*devices)
    stats = (RenderStats * n)()
    _check(lib.lyap_render_frames(arr, n, len(devices), devs, ptrs["norm"], ptrs["rgba"], stats))
    del keep
    return out, list(stats)


def render_multi(params, devices, want=("lambda", "norm", "rgba"), timeout_seconds=0.0):
    """lyap_render_multi: one frame over the listed device ordinals, from this process."""
    h, w = params.height, params.width
    out, ptrs = {}, {}
    for key, dtype, shape in (("lambda", np.float64, (h, w)), ("norm", np.float64, (h, w)), ("rgba", np.uint8, (h, w, 4))):
        if key in want:
            out[key] = np.empty(shape, dtype=dtype)
            ptrs[key] = out[key].ctypes.data
        else:
            ptrs[key] = None
    devs = (ctypes.c_int32 * len(devices))(*devices)
    stats = RenderStats()
    _check(load_library().lyap_render_multi(ctypes.byref(params), len(devices), devs, ptrs["lambda"], ptrs["norm"],
                                            ptrs["rgba"], timeout_seconds, ctypes.byref(stats)))
    out["stats"] = stats
    return out


class Multi:
    """lyap_multi: a set of devices kept ready for banded frames and frame batches (see include/lyap_b200.h)."""

    def __init__(self, devices, use_nccl=False):
        self.lib = load_library()
        self.devices = list(devices)
        devs = (ctypes.c_int32 * len(self.devices))(*self.devices)
        m = ctypes.c_void_p()
        _check(self.lib.lyap_multi_create(ctypes.byref(m), len(self.devices), devs, 1 if use_nccl else 0))
        self.m = m

    def note(self):
        return self.lib.lyap_multi_note(self.m).decode()

    def close(self):
        if self.m:
            self.lib.lyap_multi_destroy(self.m)
            self.m = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def render(self, params, want=("lambda", "norm", "rgba"), flags=0, timeout_seconds=0.0):
        """lyap_multi_render into fresh numpy arrays (+ 'stats')."""
        h, w = params.height, params.width
        out, ptrs = {}, {}
        for key, dtype, shape in (("lambda", np.float64, (h, w)), ("lambda32", np.float32, (h, w)),
                                  ("norm", np.float64, (h, w)), ("rgba", np.uint8, (h, w, 4))):
            if key in want:
                out[key] = np.empty(shape, dtype=dtype)
                ptrs[key] = out[key].ctypes.data
            else:
                ptrs[key] = None
        stats = MultiStats()
        _check(self.lib.lyap_multi_render(self.m, ctypes.byref(params), flags, ptrs["lambda"], ptrs["lambda32"], ptrs["norm"],
                                          ptrs["rgba"], timeout_seconds, ctypes.byref(stats)))
        out["stats"] = stats
        return out

    def gathered(self):
        """Device pointers (first device) of the gathered RGBA8 and fp32 lambda frames."""
        a, b = ctypes.c_void_p(), ctypes.c_void_p()
        _check(self.lib.lyap_multi_gathered(self.m, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def render_frames(self, frames, norm_ptrs, rgba_ptrs):
        """lyap_multi_render_frames with caller-owned host pointers (lists of ints or None); returns the stats list."""
        n = len(frames)
        arr = (LyapParams * n)()
        for i, f in enumerate(frames):
            ctypes.memmove(ctypes.byref(arr[i]), ctypes.byref(f), ctypes.sizeof(LyapParams))
        pn = (_P * n)(*norm_ptrs) if norm_ptrs is not None else None
        pr = (_P * n)(*rgba_ptrs) if rgba_ptrs is not None else None
        stats = (RenderStats * n)()
        _check(self.lib.lyap_multi_render_frames(self.m, arr, n, pn, pr, stats))
        return list(stats)


class DeviceBuffer:
    def __init__(self, engine, nbytes):
        self.engine, self.nbytes = engine, nbytes
        ptr = ctypes.c_void_p()
        _check(engine.lib.lyap_device_alloc(engine.ctx, ctypes.byref(ptr), nbytes))
        self.ptr = ptr.value

    def to_host(self, dtype, count=None, offset_bytes=0):
        dtype = np.dtype(dtype)
        count = (self.nbytes - offset_bytes) // dtype.itemsize if count is None else count
        out = np.empty(count, dtype=dtype)
        _check(self.engine.lib.lyap_copy_to_host(self.engine.ctx, out.ctypes.data, self.ptr + offset_bytes,
                                                 out.nbytes))
        return out

    def from_host(self, arr, offset_bytes=0):
        arr = np.ascontiguousarray(arr)
        _check(self.engine.lib.lyap_copy_to_device(self.engine.ctx, self.ptr + offset_bytes, arr.ctypes.data,
                                                   arr.nbytes))

    def free(self):
        if self.ptr:
            self.engine.lib.lyap_device_free(self.engine.ctx, self.ptr)
            self.ptr = None


class Engine:
    """One lyap_ctx (one GPU, one stream)."""

    def __init__(self, device=0):
        self.lib = load_library()
        ctx = ctypes.c_void_p()
        _check(self.lib.lyap_create(ctypes.byref(ctx), device))
        self.ctx = ctx

    def close(self):
        if self.ctx:
            self.lib.lyap_destroy(self.ctx)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- host-pointer API ----
    def render(self, params, want=("lambda", "norm", "rgba"), progress=None):
        """lyap_render -> dict of numpy arrays (+ 'stats')."""
        h, w = params.height, params.width
        rows = h if (params.row_begin == 0 and params.row_end == 0) else params.row_end - params.row_begin
        out = {}
        ptrs = {}
        for key, dtype, shape in (("lambda", np.float64, (rows, w)), ("lambda32", np.float32, (rows, w)),
                                  ("norm", np.float64, (rows, w)), ("rgba", np.uint8, (rows, w, 4))):
            if key in want:
                out[key] = np.empty(shape, dtype=dtype)
                ptrs[key] = out[key].ctypes.data
            else:
                ptrs[key] = None
        cb = PROGRESS_FN(progress) if progress else None
        stats = RenderStats()
        _check(self.lib.lyap_render(self.ctx, ctypes.byref(params), ptrs["lambda"], ptrs["lambda32"], ptrs["norm"],
                                    ptrs["rgba"], ctypes.cast(cb, ctypes.c_void_p) if cb else None,
                                    ctypes.byref(stats)))
        out["stats"] = stats
        return out

    def compute_fractal(self, params, progress=None):
        rows = params.height if (params.row_begin == 0 and params.row_end == 0) else params.row_end - params.row_begin
        out = np.empty((rows, params.width), dtype=np.float64)
        cb = PROGRESS_FN(progress) if progress else None
        _check(self.lib.lyap_compute_fractal(self.ctx, ctypes.byref(params), out.ctypes.data,
                                             ctypes.cast(cb, ctypes.c_void_p) if cb else None))
        return out

    def normalize_data(self, values):
        values = np.ascontiguousarray(values, dtype=np.float64)
        out = np.empty_like(values)
        _check(self.lib.lyap_normalize_data(self.ctx, values.ctypes.data if values.size else None, values.size,
                                            out.ctypes.data if values.size else None))
        return out

    def colorize(self, norm, palette=0):
        norm = np.ascontiguousarray(norm, dtype=np.float64)
        h, w = norm.shape
        out = np.empty((h, w, 4), dtype=np.uint8)
        pal = PALETTES.index(palette) if isinstance(palette, str) else palette
        _check(self.lib.lyap_colorize(self.ctx, norm.ctypes.data, w, h, pal, out.ctypes.data))
        return out

    def glow(self, rgba):
        rgba = np.ascontiguousarray(rgba, dtype=np.uint8)
        h, w, _ = rgba.shape
        out = np.empty_like(rgba)
        _check(self.lib.lyap_glow(self.ctx, rgba.ctypes.data, w, h, out.ctypes.data))
        return out

    # ---- device-pointer API ----
    def alloc(self, nbytes):
        return DeviceBuffer(self, nbytes)

    def lambda_device(self, params, d_lambda=None, d_lambda32=None, d_steps=None):
        _check(self.lib.lyap_lambda_device(self.ctx, ctypes.byref(params), d_lambda, d_lambda32, d_steps))

    def minmax_device(self, d_values, n, d_minmax):
        _check(self.lib.lyap_minmax_device(self.ctx, d_values, n, d_minmax))

    def normalize_device(self, d_values, n, d_minmax, d_out):
        _check(self.lib.lyap_normalize_device(self.ctx, d_values, n, d_minmax, d_out))

    def colorize_device(self, d_norm, width, rows, rows_above, rows_below, palette, d_rgba):
        _check(self.lib.lyap_colorize_device(self.ctx, d_norm, width, rows, rows_above, rows_below, palette, d_rgba))

    def set_stream(self, cuda_stream_handle):
        _check(self.lib.lyap_set_stream(self.ctx, cuda_stream_handle))

    def sync(self):
        _check(self.lib.lyap_sync(self.ctx))

    def fp64_peak(self):
        v = ctypes.c_double()
        _check(self.lib.lyap_fp64_peak(self.ctx, ctypes.byref(v)))
        return v.value

    def fp32_peak(self):
        v = ctypes.c_double()
        _check(self.lib.lyap_fp32_peak(self.ctx, ctypes.byref(v)))
        return v.value
