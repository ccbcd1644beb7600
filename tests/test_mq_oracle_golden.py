"""CPU tests of the multi-query prefill oracle and host logic against fixtures produced by the reference's own Python
(tests/golden/make_golden_mq.py): the work-list builder, float64 attention over dequantised pages with shift / sink, and the
LSE merge."""
from __future__ import annotations

import hashlib
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from flagrot_releaser_b200 import prefill_mq as MQ
from oracle import flagrot_oracle as O
from oracle import mq_oracle as MO
from _mq_cases import ATTN_CASES, PLAN_CASES, make_request_pool

GOLD = Path(__file__).resolve().parent / "golden"
REF_KCTAS = {1: 3, 2: 1, 3: 1}          # resident CTAs per SM the reference's planner assumes for its own kernels


@pytest.fixture(scope="module")
def plans():
    return np.load(GOLD / "mq_plans.npz")


@pytest.fixture(scope="module")
def attn():
    return np.load(GOLD / "mq_attn.npz")


@pytest.mark.parametrize("ci", range(len(PLAN_CASES)))
def test_plan_matches_reference(plans, ci, monkeypatch):
    monkeypatch.setattr(MQ, "KCTAS", REF_KCTAS)
    reqs, G, Hkv, shift, sink, ext = PLAN_CASES[ci]
    for nsm in (132, 148):
        for kern in (1, 3):
            tiles, items, idx, m = MQ.plan_arrays(reqs, G, Hkv, shift, nsm, kern, 2.0, 4, ext)
            key = f"c{ci}_s{nsm}_k{kern}"
            np.testing.assert_array_equal(tiles, plans[key + "_tiles"])
            np.testing.assert_array_equal(items, plans[key + "_items"])
            np.testing.assert_array_equal(idx, plans[key + "_idx"])
            assert [tiles.shape[0], items.shape[0], m, MQ.KROWS[kern], sink] == plans[key + "_meta"].tolist()


def test_build_plan_cpu_buffer(plans, monkeypatch):
    monkeypatch.setattr(MQ, "KCTAS", REF_KCTAS)
    monkeypatch.setitem(MQ._NSM, "cpu", 132)
    reqs, G, Hkv, shift, sink, ext = PLAN_CASES[-1]
    p = MQ.build_plan(reqs, G, Hkv, shift, "cpu", sink=sink, kernel=3, ext=ext, balance=False)
    key = f"c{len(PLAN_CASES) - 1}_s132_k3"
    assert p.buf.dtype == torch.int32 and p.kmin == sink and p.rows == 128 and p.kernel == 3
    np.testing.assert_array_equal(p.tiles.numpy().reshape(-1, 9), plans[key + "_tiles"])
    np.testing.assert_array_equal(p.items.numpy().reshape(-1, 4), plans[key + "_items"])
    np.testing.assert_array_equal(p.idx.numpy(), plans[key + "_idx"])
    with pytest.raises(RuntimeError):
        MQ.build_plan(reqs, G, Hkv, shift, "cpu", D=256)


def test_plan_covers_every_visible_key():
    """every tile's items tile [0, ceil(last visible key / 64)) without gaps or overlap"""
    for reqs, G, Hkv, shift, sink, ext in PLAN_CASES:
      for balance in (False, True):
        tiles, items, _, _ = MQ.plan_arrays(reqs, G, Hkv, shift, 148, 3, 2.0, 4, ext, balance)
        for ti, tl in enumerate(tiles):
            own = items[tl[6]:tl[6] + tl[7]]
            assert (own[:, 0] == ti).all() and own[0, 1] == 0
            assert (own[1:, 1] == own[:-1, 2]).all()
            last = max(0, min(tl[5], max(tl[4] + tl[3] - shift, tl[8] + 1)))
            assert own[-1, 2] == -(-last // 64)


@pytest.mark.parametrize("ci", range(len(ATTN_CASES)))
def test_attention_matches_reference(attn, ci):
    case = ATTN_CASES[ci]
    pool, bt, qb = make_request_pool(case)
    sha = hashlib.sha1(pool.tobytes() + bt.tobytes() + qb.tobytes()).digest()
    assert sha == attn[f"c{ci}_sha"].tobytes(), "seeded inputs drifted from the ones the fixture was made with"
    L, nq, W, S = case["L"], case["nq"], case["W"], case["S"]
    kk, vv = MO.request_cache(pool, bt, L - W, case["bits"], case["key_only"])
    q = O.bf16_bits_to_f32(qb)
    o, lse = MO.attention(q, kk, vv, np.arange(L - nq, L), W, 1 / math.sqrt(128), kmin=S)
    ro, rl = attn[f"c{ci}_o"], attn[f"c{ci}_lse"]
    fin = np.isfinite(rl)
    # the reference's page parsers dequantise in fp32 before the cast to float64; the oracle is float64 throughout
    np.testing.assert_allclose(lse[fin], rl[fin], rtol=0, atol=1e-4)
    assert np.isneginf(lse[~fin]).all()
    rows = fin.T[:, :, None]
    np.testing.assert_allclose(np.where(rows, o, 0), np.where(rows, ro, 0), rtol=0, atol=5e-5)


def test_lse_merge_matches_reference(attn):
    parts = [(torch.from_numpy(attn[f"merge_o{i}"]), torch.from_numpy(attn[f"merge_l{i}"])) for i in range(3)]
    np.testing.assert_allclose(MQ.ref_partial_lse_merge(parts).numpy(), attn["merge_out"], rtol=1e-6, atol=1e-6)
    two = MQ.ref_partial_lse_merge(parts[:2]).numpy()
    got = MO.bf_merge(None, parts[0][0].numpy(), parts[0][1].numpy(), parts[1][0].numpy(), parts[1][1].numpy(), None, None, None,
                      None, 0, 0, 1.0, 3)
    np.testing.assert_allclose(got, two, rtol=1e-5, atol=1e-6)


def test_item_merge_reassembles_attention():
    """partials over disjoint key ranges, merged by the oracle's item merge, equal the attention over all keys"""
    rs = np.random.RandomState(3)
    Hkv, G, nk, nt = 2, 4, 200, 5
    q = rs.randn(nt, Hkv * G, 128)
    kk, vv = rs.randn(nk, Hkv, 128), rs.randn(nk, Hkv, 128)
    pos = np.arange(nk - nt, nk)
    scale = 1 / math.sqrt(128)
    full, lse = MO.attention(q, kk, vv, pos, 0, scale)
    rows = 64
    cuts = [(0, 64), (64, 192), (192, 256)]
    opart = np.zeros((3, Hkv, rows, 128), np.float32)
    ml = np.zeros((3, Hkv, rows, 2), np.float32)
    ml[..., 0] = -np.inf
    for i, (a, b) in enumerate(cuts):
        b = min(b, nk)
        s = np.einsum("qhgd,khd->qhgk", q.reshape(nt, Hkv, G, 128), kk[a:b]) * scale * MQ.LOG2E
        s = np.where((np.arange(a, b)[None, :] <= pos[:, None])[:, None, None, :], s, -np.inf)
        mx = s.max(-1)
        p = np.where(np.isfinite(mx)[..., None], np.exp2(s - np.where(np.isfinite(mx), mx, 0)[..., None]), 0)
        o = np.einsum("qhgk,khd->qhgd", p, vv[a:b])
        for t in range(nt):
            for g in range(G):
                opart[i, :, t * G + g] = o[t, :, g]
                ml[i, :, t * G + g, 0] = mx[t, :, g]
                ml[i, :, t * G + g, 1] = p.sum(-1)[t, :, g]
    tiles = np.asarray([[0, 0, 0, nt, pos[0], nk, 0, 3, MO.NO_EXT]], np.int32)
    o2, l2 = MO.merge_items(tiles, opart, ml, G, nt)
    np.testing.assert_allclose(o2, full, atol=1e-5)
    np.testing.assert_allclose(l2, lse, atol=1e-5)
