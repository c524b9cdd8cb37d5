"""The C-ABI library: loads, exports every symbol the header declares, fails loudly without a GPU."""
import ctypes
import os
import re
import subprocess

import pytest

import lyapunovfractalwasm_b200 as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lyap_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lyap_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    syms = declared_symbols()
    assert len(syms) >= 25
    assert sorted(L.ABI.keys()) == syms


def test_library_exports_every_declared_symbol():
    lib = L.load_library()
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_no_compute_calls_needed_for_these():
    lib = L.load_library()
    assert lib.lyap_abi_version() == 2
    assert lib.lyap_self_test() == 42                    # testFunction(), src/wasm_bindings.cpp:19-22
    p = L.LyapParams()
    lib.lyap_params_default(ctypes.byref(p))
    assert (p.min_x, p.max_x, p.min_y, p.max_y) == (0.0, 4.0, 0.0, 4.0)      # src/lyapunov_fractal.hpp:16-24
    assert (p.width, p.height, p.iterations, p.warmup) == (800, 600, 10000, 100)
    assert p.sequence == b"ABABABAB" and p.sequence_len == 8
    assert (p.mode, p.palette, p.c_enabled, p.row_begin, p.row_end) == (0, 0, 0, 0, 0)
    for i, n in enumerate(L.PALETTES):
        assert lib.lyap_palette_from_name(n.encode()) == i
    assert lib.lyap_palette_from_name(b"fire") == 0 and lib.lyap_palette_from_name(None) == 0
    assert lib.lyap_status_string(0) == b"ok" and lib.lyap_status_string(2) == b"empty or missing sequence"


def test_struct_layout_matches_header():
    # the C struct is 4 doubles, 2 int32, pointer, 3 int32 (+pad), 4 int32, double, 2 int64
    assert ctypes.sizeof(L.LyapParams) == 104
    assert L.LyapParams.sequence.offset == 40 and L.LyapParams.c_value.offset == 80
    assert ctypes.sizeof(L.RenderStats) == 64
    assert ctypes.sizeof(L.MultiStats) == 64 and L.MultiStats.gather_bytes.offset == 48


def test_drop_in_header_compiles_as_cxx23(tmp_path):
    src = tmp_path / "user.cpp"
    src.write_text(
        '#include "lyapunov_fractal.hpp"\n'
        "static void cb(double) {}\n"
        "int main() {\n"
        "  lyapunov::FractalComputer::ComputationParams params;   // same fields as the reference struct\n"
        "  params.min_x = 2; params.max_x = 4; params.min_y = 2; params.max_y = 4;\n"
        '  params.width = 32; params.height = 16; params.sequence = "AB"; params.iterations = 64; params.warmup = 8;\n'
        "  lyapunov::FractalComputer computer;\n"
        "  std::vector<double> fractal_data = computer.computeFractal(params, cb);\n"
        "  std::vector<double> normalized_data = lyapunov::normalizeData(fractal_data);\n"
        "  return normalized_data.size() == 512 ? 0 : 1;\n"
        "}\n")
    exe = tmp_path / "user"
    libdir = os.path.join(ROOT, "lyapunovfractalwasm_b200")
    subprocess.run(["g++", "-std=c++23", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                    "-L", libdir, "-llyap_b200", "-Wl,-rpath," + libdir, "-o", str(exe)], check=True)
    assert exe.exists()


def test_fails_loudly_without_a_device():
    """On a machine with no CUDA device creating a context is an error, not a CPU fallback."""
    lib = L.load_library()
    n = ctypes.c_int(-1)
    st = lib.lyap_device_count(ctypes.byref(n))
    if st == 0 and n.value > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(L.LyapError) as ei:
        L.Engine(0)
    assert ei.value.status == 4
    frames = [L.make_params(width=8, height=8, sequence="AB", iterations=10, warmup=2) for _ in range(3)]
    with pytest.raises(L.LyapError) as ei:          # the batch entry point: same rule, reported from its worker thread
        L.render_frames(frames, [0])
    assert ei.value.status == 4
    with pytest.raises(L.LyapError) as ei:          # the kept multi-device object: same rule
        L.Multi([0], use_nccl=True)
    assert ei.value.status == 4
    with pytest.raises(L.LyapError) as ei:          # argument errors come before any device is touched
        L.render_frames([L.make_params(width=8, height=8, sequence="", iterations=10, warmup=2)], [0])
    assert ei.value.status == 2
