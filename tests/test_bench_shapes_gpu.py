"""Parity at the benchmarked shapes: the workloads bench.py times (batch 64 x 4096 INT4, batch 256 x 8192 INT2, KIVI batch
32 x 16384) are built at full batch x context exactly as the bench builds them (one pool copy), the timed kernel runs once,
and two sampled rows x all heads are compared with the float64 oracle over those rows' pages.  This is the check that the
kernel the bench times does the whole job at that size; the bounds are the stated ones (max-abs <= 2e-2, relative RMS <= 1e-2).
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import pytest
import torch

from oracle import flagrot_oracle as O
from oracle import kivi_oracle as KO
from tests._util import bits

pytestmark = pytest.mark.gpu
ARGS = argparse.Namespace(ncopy=1, nsplit=0, kvseq_exchange="p2p", e2e_launch="calls")


def _bounds(got, ref, what):
    err = np.abs(got - ref)
    assert not np.isnan(got).any(), what
    assert err.max() <= 2e-2, (what, "max-abs", err.max())
    rms = math.sqrt((err ** 2).mean()) / max(math.sqrt((ref ** 2).mean()), 1e-30)
    assert rms <= 1e-2, (what, "relative RMS", rms)


@pytest.mark.parametrize("name", ["cfg2", "cfg3"])
def test_decode_workload_sampled_rows(name):
    import bench
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = bench.WORKLOADS[name]
    wl = bench.DecodeWorkload(w, 0, 1, dev, ARGS)
    wl.resident(0)                                       # append + decode, as timed
    torch.cuda.synchronize()
    assert wl.status() == 0
    rows = [1, wl.B - 2]
    npg = wl.Lloc // 16
    btr = wl.bts[0][rows].cpu().long()
    sub = wl.pools[0][btr.reshape(-1)].cpu().numpy()     # the sampled rows' pages, re-indexed 0 .. 2 npg - 1
    bt = np.arange(2 * npg, dtype=np.int32).reshape(2, npg)
    T = w["S"] + w["W"]
    with np.errstate(invalid="ignore", over="ignore"):
        ref = O.decode_reference(bits(wl.q[rows]), sub, bt, [int(wl.seq[r]) for r in rows], bench.SCALE, w["nb"], 16, True,
                                 tail=bits(wl.ring[rows]), tail_len=np.full(2, T, np.int32), tail_idx=np.arange(2), kv_start=w["S"])
    got = wl.out.view(wl.B, w["Hq"], 128)[rows].double().cpu().numpy()
    _bounds(got, ref, (name, wl.plan))


def test_kivi_workload_sampled_rows():
    import bench
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = bench.WORKLOADS["cfg4"]
    wl = bench.KiviWorkload(w, 0, 1, dev, ARGS)
    wl.resident(0)
    torch.cuda.synchronize()
    rows = [0, wl.B - 1]
    npg = wl.L // 16
    btr = wl.bts[0][rows].cpu().long()
    sub = wl.pools[0][btr.reshape(-1)].cpu().numpy()
    bt = np.arange(2 * npg, dtype=np.int32).reshape(2, npg)
    ring = wl.ring.cpu()
    ref = KO.decode_reference(bits(wl.q[rows]), sub, bt, np.full(2, wl.L - wl.W, np.int32), bench.SCALE, wl.S, wl.G,
                              ring=bits(ring[rows]), tail_len=np.full(2, wl.T, np.int32), tail_idx=np.arange(2))
    got = wl.out.view(wl.B, w["Hq"], 128)[rows].double().cpu().numpy()
    _bounds(got, ref, ("cfg4", wl.plan))
