"""HostStep: the captured step (host -> device copies, writer append, decode, copy back) gives the same output rows as the
separate launches, also after the host buffers were rewritten between replays."""
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

pytestmark = pytest.mark.gpu


def test_host_step_replay_matches_separate_launches():
    import bench
    from flagrot_releaser_b200.graphs import HostStep

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    import argparse
    w = dict(bench.WORKLOADS["cfg2"], B=3, L=768)
    st = bench.DecodeWorkload(w, 0, 1, dev, argparse.Namespace(ncopy=1, nsplit=0, kvseq_exchange="p2p", e2e_launch="calls"))
    st.resident(0)                                      # first calls outside the capture
    torch.cuda.synchronize()
    hs = HostStep([(st.q, st.q_host), (st.kv, st.kv_host), (st.slots[0], st.slots_host[0])],
                  lambda: st.resident(0), [(st.out_host, st.out)])
    assert hs.h2d_bytes == st.q_host.numel() * 2 + st.kv_host.numel() * 2 + w["B"] * 8
    assert (hs.h2d_bytes, hs.d2h_bytes) == st.copies()
    g = torch.Generator().manual_seed(11)
    for _ in range(3):
        st.q_host.copy_(torch.randn(st.q_host.shape, generator=g).bfloat16())
        st.kv_host.copy_(torch.randn(st.kv_host.shape, generator=g).bfloat16())
        st.out_host.zero_()
        hs.run()
        got = st.out_host.clone()
        # the same step with separate launches on the same inputs (the append rewrites the same slots with the same rows)
        st.q.copy_(st.q_host)
        st.kv.copy_(st.kv_host)
        st.resident(0)
        torch.cuda.synchronize()
        assert torch.equal(got, st.out.cpu())
        assert got.float().abs().max() > 0
