"""Program-level recognisers (mimk_program_classify): lists of map_reduce_post descriptors whose dataflow spells softmax
or attention. Pure host logic, no device needed."""
import pytest
import torch

F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32


@pytest.fixture(scope="module")
def TL():
    import __graft_entry__ as entry
    entry.build()
    from mimir_b200 import _lib, tensor
    return tensor, _lib


class Mem:
    """Fake device addresses for operands."""

    def __init__(self):
        self.next = 0x10000

    def new(self, T, shape, dtype=F32):
        self.next += 1 << 24
        return T.Operand(self.next, dtype, shape)


def softmax_ops(T, L, P, mem, x, ax, fused=False, dtype=F32):
    """The operations `softmax m ax x` expands to (tensor.mim:1172-1176): reduce fmax, binary_ax exp(u - v), reduce add,
    binary_ax div -- or the three fuse_tensor leaves (fuse.cpp:225-245)."""
    shape = list(x.shape)
    r = len(shape)
    red = shape[:ax] + shape[ax + 1:]
    fold_sr = red + [shape[ax]]
    fold_map = [j if j < ax else (r - 1 if j == ax else j - 1) for j in range(r)]   # x read with the folded loop last
    drop = [i if i < ax else i + 1 for i in range(r - 1)]                           # an operand without axis ax
    mx = P.op(mem.new(T, red, dtype), fold_sr, L.F_MAX, float("-inf"), L.P_ID, T.proj_map(r, range(r - 1)), [T.proj_map(r, fold_map)], [x])
    if fused:
        sm = P.op(mem.new(T, red, dtype), fold_sr, L.F_ADD_SUBEXP, 0.0, L.P_ID, T.proj_map(r, range(r - 1)),
                  [T.proj_map(r, fold_map), T.proj_map(r, range(r - 1))], [x, mx])
        return P.op(mem.new(T, shape, dtype), shape, L.F_SUBEXP_DIV, 0.0, L.P_ID, T.id_map(r),
                    [T.id_map(r), T.proj_map(r, drop), T.proj_map(r, drop)], [x, mx, sm])
    e = P.op(mem.new(T, shape, dtype), shape, L.F_SUBEXP, 0.0, L.P_ID, T.id_map(r), [T.id_map(r), T.proj_map(r, drop)], [x, mx])
    sm = P.op(mem.new(T, red, dtype), fold_sr, L.F_ADD, 0.0, L.P_ID, T.proj_map(r, range(r - 1)), [T.proj_map(r, fold_map)], [e])
    return P.op(mem.new(T, shape, dtype), shape, L.F_DIV, 0.0, L.P_ID, T.id_map(r), [T.id_map(r), T.proj_map(r, drop)], [e, sm])


def matmul(T, L, P, mem, a, b, m, n, k, b_nk=False, dtype=F32):
    return P.op(mem.new(T, (m, n), dtype), (m, n, k), L.F_MULADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)),
                [T.proj_map(3, (0, 2)), T.proj_map(3, (1, 2) if b_nk else (2, 1))], [a, b])


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("shape,ax", [((64, 100), 1), ((4, 37, 6), 1), ((5, 8), 0), ((2, 3, 4), 2)])
def test_softmax_chain_is_recognised(TL, shape, ax, fused):
    T, L = TL
    mem, P = Mem(), T.Program()
    x = mem.new(T, shape)
    softmax_ops(T, L, P, mem, x, ax, fused)
    assert P.classify() == (["softmax", "absorbed", "absorbed"] + ([] if fused else ["absorbed"]))


def test_softmax_chain_is_left_alone_when_it_is_not_one(TL):
    T, L = TL
    # a temporary (the exponentials) is read by a later operation outside the chain: nothing may be skipped
    mem, P = Mem(), T.Program()
    x = mem.new(T, (16, 32))
    softmax_ops(T, L, P, mem, x, 1)
    e = P.keep[1][0]
    P.op(mem.new(T, (16, 32)), (16, 32), L.F_ADD2, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.id_map(2)], [e, e])
    assert P.classify() == ["op"] * 5
    # the sum fold runs along another axis than the max fold
    mem, P = Mem(), T.Program()
    x = mem.new(T, (8, 8))
    mx = P.op(mem.new(T, (8,)), (8, 8), L.F_MAX, float("-inf"), L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [x])
    e = P.op(mem.new(T, (8, 8)), (8, 8), L.F_SUBEXP, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.proj_map(2, (0,))], [x, mx])
    sm = P.op(mem.new(T, (8,)), (8, 8), L.F_ADD, 0.0, L.P_ID, T.proj_map(2, (0,)), [T.proj_map(2, (1, 0))], [e])
    P.op(mem.new(T, (8, 8)), (8, 8), L.F_DIV, 0.0, L.P_ID, T.id_map(2), [T.id_map(2), T.proj_map(2, (0,))], [e, sm])
    assert P.classify() == ["op"] * 4
    # an integer fold with the same maps is not a softmax
    mem, P = Mem(), T.Program()
    x = mem.new(T, (8, 8), I32)
    P.op(mem.new(T, (8,), I32), (8, 8), L.F_MAX, -(2 ** 31), L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [x])
    assert P.classify() == ["op"]
    # an empty program
    assert T.Program().classify() == []


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_chain_is_recognised(TL, fused, dtype):
    """lit/tensor/attn_exec.mim:20-22 after the projections: softmax (q * transpose_2d k) * v."""
    T, L = TL
    mem, P = Mem(), T.Program()
    n, dh = 64, 8
    x, wq = mem.new(T, (n, dh), dtype), mem.new(T, (dh, dh), dtype)
    q = matmul(T, L, P, mem, x, wq, n, dh, dh, dtype=dtype)                      # a projection in front: an ordinary operation
    k, v = mem.new(T, (n, dh), dtype), mem.new(T, (n, dh), dtype)
    s = matmul(T, L, P, mem, q, k, n, n, dh, b_nk=True, dtype=dtype)
    p = softmax_ops(T, L, P, mem, s, 1, fused, dtype)
    matmul(T, L, P, mem, p, v, n, dh, n, dtype=dtype)
    inner = 3 if fused else 4
    assert P.classify() == ["op", "attention"] + ["absorbed"] * (inner + 1)


def test_attention_needs_the_whole_shape(TL):
    T, L = TL
    # scores read by something else as well: the softmax inside still fuses, the contractions run by themselves
    mem, P = Mem(), T.Program()
    n, dh = 32, 16
    q, k, v = mem.new(T, (n, dh)), mem.new(T, (n, dh)), mem.new(T, (n, dh))
    s = matmul(T, L, P, mem, q, k, n, n, dh, b_nk=True)
    p = softmax_ops(T, L, P, mem, s, 1)
    matmul(T, L, P, mem, p, v, n, dh, n)
    P.op(mem.new(T, (n,)), (n, n), L.F_ADD, 0.0, L.P_ID, T.proj_map(2, (0,)), [T.id_map(2)], [s])
    assert P.classify() == ["op", "softmax", "absorbed", "absorbed", "absorbed", "op", "op"]
    # k not read through transpose_2d (stored [head_dim, keys]): not the program's shape
    P = T.Program()
    kt = mem.new(T, (dh, n))
    s = matmul(T, L, P, mem, q, kt, n, n, dh)
    p = softmax_ops(T, L, P, mem, s, 1)
    matmul(T, L, P, mem, p, v, n, dh, n)
    assert P.classify()[0] == "op" and "attention" not in P.classify()
    # softmax along the query axis of the scores
    P = T.Program()
    s = matmul(T, L, P, mem, q, k, n, n, dh, b_nk=True)
    p = softmax_ops(T, L, P, mem, s, 0)
    matmul(T, L, P, mem, p, v, n, dh, n)
    assert "attention" not in P.classify() and "softmax" in P.classify()


def test_a_map_feeding_one_fold_is_fused(TL):
    """fuse_map_reduce on the list level (phase/fuse.cpp:183-358): the produced tensor is read by the fold alone."""
    T, L = TL
    mem, P = Mem(), T.Program()
    shape, ax = [64, 300, 8], 1
    red = [64, 8]
    x, mean = mem.new(T, shape), mem.new(T, red)
    # d = x - mean (binary_ax along axis 1); s = sum d along axis 1 ... a centred sum
    d = P.op(mem.new(T, shape), shape, L.F_ADD2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (0, 2))], [x, mean])
    P.op(mem.new(T, red), red + [300], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [d])
    # unary map then a max fold along the last axis
    a = P.op(mem.new(T, shape), shape, L.F_FIRST, 0.0, L.P_RELU, T.id_map(3), [T.id_map(3)], [x])
    P.op(mem.new(T, [64, 300]), [64, 300, 8], L.F_MAX, float("-inf"), L.P_ID, T.proj_map(3, (0, 1)), [T.id_map(3)], [a])
    # weights over the trailing axes from the folded one on
    w = mem.new(T, [300, 8])
    xw = P.op(mem.new(T, shape), shape, L.F_MUL2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (1, 2))], [x, w])
    P.op(mem.new(T, red), red + [300], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [xw])
    assert P.classify() == ["fold_of_map", "absorbed"] * 3


def test_a_map_read_twice_or_broadcast_across_the_fold_is_not_fused(TL):
    T, L = TL
    mem, P = Mem(), T.Program()
    shape, red = [64, 300, 8], [64, 8]
    x, y = mem.new(T, shape), mem.new(T, [64, 300])
    # the produced tensor has a second reader
    sq = P.op(mem.new(T, shape), shape, L.F_MUL2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.id_map(3)], [x, x])
    P.op(mem.new(T, red), red + [300], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [sq])
    P.op(mem.new(T, shape), shape, L.F_FIRST, 0.0, L.P_RELU, T.id_map(3), [T.id_map(3)], [sq])
    assert P.classify() == ["op", "op", "op"]
    # y lacks the LAST axis while the fold runs over the middle one: no placement of the producer's operand fits
    P2 = T.Program()
    d = P2.op(mem.new(T, shape), shape, L.F_ADD2, 0.0, L.P_ID, T.id_map(3), [T.id_map(3), T.proj_map(3, (0, 1))], [x, y])
    P2.op(mem.new(T, red), red + [300], L.F_ADD, 0.0, L.P_ID, T.proj_map(3, (0, 1)), [T.proj_map(3, (0, 2, 1))], [d])
    assert P2.classify() == ["op", "op"]
    # the exponential of an incomplete softmax chain still fuses with its sum
    P3 = T.Program()
    r = 2
    xs = mem.new(T, [128, 512])
    mx = P3.op(mem.new(T, [128]), [128, 512], L.F_MAX, float("-inf"), L.P_ID, T.proj_map(r, (0,)), [T.id_map(r)], [xs])
    e = P3.op(mem.new(T, [128, 512]), [128, 512], L.F_SUBEXP, 0.0, L.P_ID, T.id_map(r), [T.id_map(r), T.proj_map(r, (0,))], [xs, mx])
    P3.op(mem.new(T, [128]), [128, 512], L.F_ADD, 0.0, L.P_ID, T.proj_map(r, (0,)), [T.id_map(r)], [e])
    assert P3.classify() == ["op", "fold_of_map", "absorbed"]
