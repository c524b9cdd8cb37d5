import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session", autouse=True)
def built():
    """Make sure the engine library and the CPU checkers exist (compiles them where a toolchain is present)."""
    from lyapunovfractalwasm_b200 import build
    build.build_library()
    build.build_cli()
    build.build_oracle()


@pytest.fixture(scope="session")
def port():
    import oracle_lib
    return oracle_lib.port()


@pytest.fixture(scope="session")
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "golden.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def engine():
    import lyapunovfractalwasm_b200 as L
    eng = L.Engine(0)   # raises without a GPU or without the built library: no fallback
    yield eng
    eng.close()


# which lambda kernel a launch takes for a periodic sequence: (LYAP_JIT, LYAP_PREBUILT)
KERNEL_PATHS = {
    "generic": ("0", "0"),    # patterns dispatched every two steps at run time
    "prebuilt": ("0", "1"),   # the instance compiled with the library, where the patterns match one; else generic
    "jit": ("2", "0"),        # an instance compiled by NVRTC on first use
}


@pytest.fixture()
def kernel_path():
    """choose(name) sets the two environment switches the library reads at every launch; restored afterwards."""
    old = {k: os.environ.get(k) for k in ("LYAP_JIT", "LYAP_PREBUILT")}

    def choose(name):
        os.environ["LYAP_JIT"], os.environ["LYAP_PREBUILT"] = KERNEL_PATHS[name]
    yield choose
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


# the benchmark configurations 1-4, as make_params keywords (5 is config5_frame below)
CONFIGS = {
    1: dict(min_x=2.0, max_x=4.0, min_y=2.0, max_y=4.0, width=512, height=512, sequence="AB",
            iterations=1000, warmup=100),
    2: dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=4096, height=4096, sequence="AABAB",
            iterations=2000, warmup=200),
    3: dict(min_x=3.4, max_x=4.0, min_y=2.5, max_y=3.4, width=16384, height=16384, sequence="BBBBBBAAAAAA",
            iterations=4000, warmup=500),
    4: dict(min_x=2.0, max_x=4.0, min_y=2.0, max_y=4.0, width=65536, height=65536, sequence="AB",
            iterations=1000, warmup=100),
}


def config5_frame(k):
    """Frame k of the zoom batch: centre (3.82, 3.45), half-width 0.5*0.97^k on both axes, 'ABC' with c = 3.7."""
    h = 0.5 * 0.97 ** k
    return dict(min_x=3.82 - h, max_x=3.82 + h, min_y=3.45 - h, max_y=3.45 + h, width=1920, height=1080,
                sequence="ABC", iterations=3000, warmup=300, c=3.7)
