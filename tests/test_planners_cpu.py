"""Host arithmetic of the split planners (no GPU): coverage of the context, granularity, and the choices measured on B200."""
import random

from flagrot_releaser_b200 import kernels as K
from flagrot_releaser_b200 import kivi as KV


def test_decode_planner_headline_shapes():
    # 148 SMs x 3 resident CTAs; batch 64 x 3968 page tokens, 8 kv heads, window CTAs in the launch
    assert K.plan_splits(64, 3968, 8, 444, tail=True) == (2, 1984)
    ns, ch = K.plan_splits(1, 131072 - 128, 8, 444)
    assert ns * ch >= 131072 - 128 and ch % 64 == 0 and ch <= K.MAX_CHUNK and 40 <= ns <= 64
    assert K.plan_splits(256, 8064, 8, 444)[0] == 1


def test_decode_planner_properties():
    rnd = random.Random(3)
    for _ in range(300):
        B, L, H = rnd.randint(1, 300), rnd.randint(1, 200000), rnd.choice([1, 2, 8])
        slots = rnd.choice([148, 296, 444, 592])
        ns, ch = K.plan_splits(B, L, H, slots)
        assert ch % 64 == 0 and 64 <= ch <= K.MAX_CHUNK
        assert ns == -(-L // ch) and ns <= K.MAX_SPLITS or L > K.MAX_CHUNK * K.MAX_SPLITS
        forced = K.plan_splits(B, L, H, slots, nsplit=rnd.randint(1, 8))
        assert forced[1] % 64 == 0 and forced[0] * forced[1] >= min(L, forced[0] * K.MAX_CHUNK)


def test_kivi_planner():
    assert KV.plan(32, 16384, 8, sms=148, occ=3) == (5, 3328)      # measured best of 2 .. 7 splits
    rnd = random.Random(5)
    for _ in range(300):
        B, L, H = rnd.randint(1, 300), rnd.randint(1, 200000), rnd.choice([1, 2, 8])
        ns, ch = KV.plan(B, L, H, sms=148, occ=rnd.choice([2, 3]))
        assert ch % 128 == 0 and ch >= 256
        assert ns == -(-L // ch) and ns * ch >= L
