"""Matrix-chain association (mimk_chain_order / mimk_chain_cost): the reference's price list reproduces every decision
and every cost its own test documents (lit/tensor/reassoc.mim); the B200 price list is checked for the properties it
is built on. Needs no GPU."""
import itertools

import pytest
import torch

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def R():
    entry.build()
    from mimir_b200 import reassoc
    return reassoc


def lanes(R, dims, splits, transposed=None, vec=8):
    return R.chain_cost(dims, splits, transposed, model="lanes", vec=vec)


def test_chain3_and_chain4(R):
    # lit/tensor/reassoc.mim:29-37: 4x10 . 10x2 . 2x10 right-deep costs 960, the optimum is left-deep at 448
    dims = (4, 10, 2, 10)
    assert lanes(R, dims, R.right_deep(3)) == 960
    splits, cost = R.chain_order(dims, model="lanes")
    assert cost == 448 and [s[:3] for s in splits] == [(0, 0, 1), (0, 1, 2)]
    # reassoc.mim:39-46: 30x35 . 35x15 . 15x5 . 5x10 left-deep 22800; optimum ((A (B C)) D) at 15000
    dims = (30, 35, 15, 5, 10)
    assert lanes(R, dims, R.left_deep(4)) == 22800
    splits, cost = R.chain_order(dims, model="lanes")
    assert cost == 15000 and [s[:3] for s in splits] == [(1, 1, 2), (0, 0, 2), (0, 2, 3)]


def test_idle_lanes_are_charged(R):
    # reassoc.mim:83-100: 100x4 . 4x2 . 2x8
    dims = (100, 4, 2, 8)
    for vec, written, other, moved in ((8, 4800, 3264, True), (4, 3200, 3264, False), (1, 2400, 3264, False)):
        assert lanes(R, dims, R.left_deep(3), vec=vec) == written
        assert lanes(R, dims, R.right_deep(3), vec=vec) == other
        splits, cost, reassociated = R.choose(dims, None, R.left_deep(3), model="lanes", vec=vec)
        assert reassociated == moved and cost == min(written, other)


def test_transposed_leaf_vectorises_the_contraction(R):
    # reassoc.mim:102-111: a(10x5) . b(5x8) . transpose c(9x8): as written 1120, a.(b.c^T) 1160
    dims, tr = (10, 5, 8, 9), (False, False, True)
    assert lanes(R, dims, R.left_deep(3), tr) == 1120
    assert lanes(R, dims, R.right_deep(3), tr) == 1160
    assert lanes(R, dims, R.left_deep(3)) == 1680 and lanes(R, dims, R.right_deep(3)) == 1440   # without the kvec schedule
    assert R.choose(dims, tr, R.left_deep(3), model="lanes")[2] is False


def test_attention_scores_chain(R):
    # reassoc.mim:113-131: (x wq) (x wk)^T is the chain x . wq . wk^T . x^T; as written the right factor is built
    # untransposed (x . wk) and read through a transpose, i.e. a node stored transposed
    tr = (False, False, True, True)
    written = [(0, 0, 1, False), (2, 2, 3, True), (0, 1, 3, False)]
    dims = (64, 8, 8, 8, 64)
    assert lanes(R, dims, written, tr) == 40960
    splits, cost, moved = R.choose(dims, tr, written, model="lanes")
    assert cost == 37376 and moved and [s[:3] for s in splits] == [(1, 1, 2), (1, 2, 3), (0, 0, 3)]
    dims = (4, 8, 8, 8, 4)
    assert lanes(R, dims, written, tr) == 640
    splits, cost, moved = R.choose(dims, tr, written, model="lanes")
    assert cost == 640 and not moved and splits == written       # a tie keeps the program as written


def test_order_is_optimal_against_enumeration(R):
    def brackets(lo, hi):
        if lo == hi:
            yield []
            return
        for s in range(lo, hi):
            for l, r in itertools.product(brackets(lo, s), brackets(s + 1, hi)):
                yield l + r + [(lo, s, hi, False)]
    g = torch.Generator().manual_seed(3)
    for _ in range(20):
        n = int(torch.randint(3, 7, (1,), generator=g))
        dims = [int(v) for v in torch.randint(1, 200, (n + 1,), generator=g)]
        tr = [bool(v) for v in torch.randint(0, 2, (n,), generator=g)]
        _, cost = R.chain_order(dims, tr, model="lanes")
        assert cost == min(lanes(R, dims, b, tr) for b in brackets(0, n - 1))
        # the B200 list may also build nodes transposed, so it is at least as good as every plain bracketing
        _, cost = R.chain_order(dims, tr, model="b200", dtype=torch.float32)
        assert cost <= min(R.chain_cost(dims, b, tr, model="b200", dtype=torch.float32) for b in brackets(0, n - 1)) * (1 + 1e-12)


def test_b200_price_list(R):
    # low-rank bottleneck (reassoc.mim:58-65): x (U V) forms the 768 x 768 product first, (x U) V never does
    dims = (65536, 768, 8, 768)
    splits, cost, moved = R.choose(dims, None, R.right_deep(3), model="b200")
    assert moved and [s[:3] for s in splits] == [(0, 0, 1), (0, 1, 2)]
    assert cost < R.chain_cost(dims, R.right_deep(3), model="b200")
    # tiles are whole: 129 rows cost what 256 rows cost once the product is compute-bound
    a = R.chain_cost((129, 8192, 8192), [(0, 0, 1)], model="b200")
    b = R.chain_cost((256, 8192, 8192), [(0, 0, 1)], model="b200")
    assert a == b
    # a transposed leaf on the right is free, on the left it pays a copy -- unless the node is built transposed instead
    free = R.chain_cost((4096, 4096, 4096), [(0, 0, 1)], (False, True), model="b200")
    plain = R.chain_cost((4096, 4096, 4096), [(0, 0, 1)], model="b200")
    left = R.chain_cost((4096, 4096, 4096), [(0, 0, 1)], (True, False), model="b200")
    assert free == plain < left
    dims, tr = (4096, 4096, 4096, 256), (False, True, True)      # X . (A^T . B^T): built as (B . A) and read back through a transpose
    splits, cost = R.chain_order(dims, tr, model="b200")
    assert splits == [(1, 1, 2, True), (0, 0, 2, False)]
    assert cost < R.chain_cost(dims, R.right_deep(3), tr, model="b200") < R.chain_cost(dims, R.left_deep(3), tr, model="b200")
    # the estimate for the 8192^3 bf16 product is within 15 % of the measured 0.74 ms
    assert abs(R.chain_cost((8192, 8192, 8192), [(0, 0, 1)], model="b200") / 0.74e-3 - 1) < 0.15


def test_bad_arguments(R):
    with pytest.raises(Exception):
        R.chain_cost((4, 4, 4, 4), [(0, 0, 2)])          # uses sub-chain 1..2 that no given product builds
    with pytest.raises(ValueError):
        R.chain_order((4,))
