"""Row-band sharding across ranks, run as two gloo ranks on CPU.

The orchestration under test is lyapunovfractalwasm_b200/bands.py (partition, halo rows, the one
min/max exchange).  The arithmetic is done by the CPU oracle as a stand-in backend, so the test checks
that bands + halo + exchanged min/max assemble into exactly the single-process frame."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as O
from lyapunovfractalwasm_b200 import bands

KW = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=96, height=61, sequence="AABAB", iterations=120, warmup=20)


class OracleBackend:
    """bands.render_band backend on the CPU oracle; handles are numpy arrays."""

    def __init__(self):
        self.p = O.port()

    def lambda_rows(self, kw, r0, r1):
        lam, _ = self.p.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                                    kw["sequence"], kw["iterations"], kw["warmup"], y0=r0, y1=r1)
        return lam

    @staticmethod
    def rows_view(a, first, rows):
        return a[first:first + rows]

    def minmax(self, a):
        return self.p.minmax(np.ascontiguousarray(a))

    def normalize(self, a, lo, hi):
        return self.p.normalize(a, lo, hi)

    def colorize(self, norm, first, rows, above, below, palette):
        # the oracle colours a whole array with image-edge rules; give it band + halo rows and cut
        full = self.p.colorize(norm, palette)
        return full[first:first + rows]


def test_band_rows_partition():
    for h in (1, 7, 61, 4096, 65536):
        for n in (1, 2, 3, 4, 8):
            spans = [bands.band_rows(h, n, r) for r in range(n)]
            assert spans[0][0] == 0 and spans[-1][1] == h
            assert all(spans[i][1] == spans[i + 1][0] for i in range(n - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    assert bands.band_rows(65536, 8, 3) == (3 * 8192, 4 * 8192)
    assert bands.halo_rows(61, 0, 30) == (0, 1) and bands.halo_rows(61, 30, 61) == (1, 0)
    assert [bands.frame_for_rank(k, 8) for k in (0, 7, 8, 255)] == [0, 7, 0, 7]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def allreduce(lo, hi):
        pair = torch.tensor([lo, -hi], dtype=torch.float64)      # one all-reduce serves both ends: min over (min, -max)
        dist.all_reduce(pair, op=dist.ReduceOp.MIN)
        return float(pair[0]), -float(pair[1])

    res = bands.render_band(OracleBackend(), KW, rank, world, allreduce, palette=0)
    np.savez(os.path.join(outdir, "rank%d.npz" % rank), lam=res["lambda"], norm=res["norm"], rgba=res["rgba"],
             rows=np.array(res["rows"]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_bands_over_gloo_equal_single_process(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    p = O.port()
    lam, _ = p.lambda_rows(KW["min_x"], KW["max_x"], KW["min_y"], KW["max_y"], KW["width"], KW["height"],
                           KW["sequence"], KW["iterations"], KW["warmup"])
    norm = p.normalize(lam)
    rgba = p.colorize(norm, 0)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    assert [tuple(q["rows"]) for q in parts] == [bands.band_rows(KW["height"], world, r) for r in range(world)]
    assert np.array_equal(np.vstack([q["lam"] for q in parts]).view(np.uint64), lam.view(np.uint64))
    assert np.array_equal(np.vstack([q["norm"] for q in parts]).view(np.uint64), norm.view(np.uint64))
    assert np.array_equal(np.vstack([q["rgba"] for q in parts]), rgba)
