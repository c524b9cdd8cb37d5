#!/usr/bin/env python3
"""Generate tests/golden/golden.json from the UNMODIFIED reference header.

Needs oracle/_ref/ (built by oracle/Makefile where the reference sources exist), so it runs only in
a checkout that has the reference beside it; the JSON it writes travels with the repository.

Each case stores 64-bit-word FNV hashes (see oracle_hash64) and a few spot values of
  lambda  = FractalComputer::computeFractal                      (src/lyapunov_fractal.hpp:27)
  norm    = normalizeData(lambda)                                (src/lyapunov_fractal.hpp:105)
computed twice: with this project's log/pow/exp bound into the header ("lyapmath": what the CUDA
engine must reproduce bit for bit) and with the host libm ("stock": informational, depends on the
libm build).  rgba hashes come from the restated colour stage applied to the lyapmath norm.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402

CASES = {
    # name: (min_x, max_x, min_y, max_y, width, height, sequence, iterations, warmup)
    "cfg1_512_AB": (2.0, 4.0, 2.0, 4.0, 512, 512, "AB", 1000, 100),
    "ui_default_call_200": (0.0, 4.0, 0.0, 4.0, 200, 200, "AB", 1000, 100),
    "cfg2_shape_256_AABAB": (2.5, 4.0, 2.5, 4.0, 256, 256, "AABAB", 2000, 200),
    "cfg3_shape_128_B6A6": (3.4, 4.0, 2.5, 3.4, 128, 128, "BBBBBBAAAAAA", 4000, 500),
    "abc_without_c_96": (3.3, 4.3, 2.9, 3.9, 96, 54, "ABC", 300, 30),
    "odd_333x77": (2.5, 4.2, 2.4, 4.1, 333, 77, "AABAB", 257, 37),
    "lowercase_is_b_64": (2.0, 4.0, 2.0, 4.0, 64, 64, "AbaB", 200, 20),
    "width1_height5": (2.0, 4.0, 2.0, 4.0, 1, 5, "AB", 50, 10),
    "warmup0_40": (2.0, 4.0, 2.0, 4.0, 40, 40, "AB", 100, 0),
    "struct_defaults_80x60": (0.0, 4.0, 0.0, 4.0, 80, 60, "ABABABAB", 1000, 100),
}
SPOTS = [(0, 0), (1, 2), (17, 5), (31, 40), (100, 400), (256, 256), (300, 300), (511, 511)]


def main():
    port = O.port()
    refs = {"lyapmath": O.ref("lyapmath"), "stock": O.ref("stock")}
    if refs["lyapmath"] is None:
        sys.exit("oracle/_ref is not built (needs the reference sources): run make -C oracle")
    out = {"hash": "h=1469598103934665603; per 64-bit word: h^=w; h*=1099511628211 mod 2^64", "cases": {}}
    for name, args in CASES.items():
        entry = {"args": list(args)}
        for kind, ref in refs.items():
            lam = ref.compute_fractal(*args)
            norm = ref.normalize(lam)
            entry[kind] = {"lambda_hash": "%016x" % port.hash64(lam), "norm_hash": "%016x" % port.hash64(norm)}
            if kind == "lyapmath":
                h, w = lam.shape
                entry["spots"] = [[x, y, lam[y, x].hex(), norm[y, x].hex()] for (x, y) in SPOTS if x < w and y < h]
                entry["census"] = {"sentinel": int(np.count_nonzero(lam == -5.0)),
                                   "negative": int(np.count_nonzero((lam < 0) & (lam != -5.0))),
                                   "nonnegative": int(np.count_nonzero(lam >= 0))}
                if w * h % 2 == 0:
                    for pal, pname in enumerate(O.PALETTES):
                        entry.setdefault("rgba_hash", {})[pname] = "%016x" % port.hash64(port.colorize(norm, pal))
        out["cases"][name] = entry
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote golden.json with %d cases" % len(out["cases"]))


if __name__ == "__main__":
    main()
