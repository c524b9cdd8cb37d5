"""Host logic of the step selectors: the packed table the kernels read (whole regions, or one period of the
sequence walked cyclically for runs longer than the table) against sequence[i % len]
(src/lyapunov_fractal.hpp:37).  No GPU needed."""
import random

import pytest

import lyapunovfractalwasm_b200 as L


def expected(seq, i, use_c):
    ch = seq[i % len(seq)]
    return 0 if ch == "A" else (2 if use_c and ch == "C" else 1)


def check(seq, warmup, iterations, steps, c=None):
    p = L.make_params(width=4, height=4, sequence=seq, iterations=iterations, warmup=warmup, c=c)
    for i in steps:
        if i < warmup:
            assert L.selector_code(p, 0, i) == expected(seq, i, c is not None), (seq, "warm-up", i)
        if i < iterations:
            assert L.selector_code(p, 1, i) == expected(seq, warmup + i, c is not None), (seq, "acc", i)


def test_regions_stored_whole():
    rng = random.Random(1)
    for seq in ("AB", "AABAB", "BBBBBBAAAAAA", "AxB?", "ABCAC"):
        check(seq, 203, 2001, list(range(0, 2001, 7)) + [202, 2000], c=2.5 if "C" in seq else None)
    seq = "".join(rng.choice("AB") for _ in range(1000))   # longer than it can wrap, short enough to store
    check(seq, 3000, 11000, range(0, 11000, 13))


@pytest.mark.parametrize("seq", ["A", "AB", "AABAB", "BBBBBBAAAAAA", "ABBABAABBAABABBA", "ABCAC", "AABABBA" * 9])
def test_long_runs_wrap_by_the_sequence_period(seq):
    warmup, iterations = 100003, 2_000_000_011            # neither a multiple of 16 nor of the period
    far = [0, 1, 15, 16, 17, len(seq) * 16 - 1, len(seq) * 16, len(seq) * 16 + 1, 14335, 14336, 14337, 99999, 100002,
           1_000_000_007, 2_000_000_010]
    rng = random.Random(len(seq))
    far += [rng.randrange(iterations) for _ in range(200)]
    check(seq, warmup, iterations, far, c=1.75 if "C" in seq else None)


def test_mixed_whole_warmup_and_wrapped_accumulation():
    seq = "AABAB" * 40                                     # 200 letters: one period is 200 / gcd(200, 16) = 25 words
    check(seq, 37, 500_000, [0, 36, 199, 200, 3199, 3200, 3201, 499_999])


def test_limits():
    ok_len = 448                                          # 2 * 448 words = the whole table
    seq = "".join("AB"[(i * i) % 3 == 0] for i in range(ok_len - 1)) + "A"
    rng = random.Random(3)
    check(seq, 50_000, 50_000, [rng.randrange(50_000) for _ in range(100)])
    too_long = "".join("AB"[(i * i) % 3 == 0] for i in range(449))
    p = L.make_params(width=4, height=4, sequence=too_long, iterations=20_000, warmup=20_000)
    with pytest.raises(L.LyapError) as e:
        L.selector_code(p, 1, 0)
    assert e.value.status == 3                            # LYAP_ERR_TOO_LARGE
    # the same sequence is fine while the steps fit in the table
    check(too_long, 4000, 10_000, range(0, 10_000, 97))
    p = L.make_params(width=4, height=4, sequence="AB", iterations=10, warmup=0)
    for region, step in ((0, 0), (1, 10), (1, -1), (2, 0)):
        with pytest.raises(L.LyapError):
            L.selector_code(p, region, step)
