"""Writes tests/golden/cases.npz: seeded inputs' recipes and the oracle's f64-truth outputs for small instances of
every operator on the path. Run from the repository root:  python tests/golden/make_golden.py

The oracle that produces these is pinned on the reference's own known answers (tests/test_oracle_golden.py); the
fixtures freeze its answers so that the CUDA path is also compared with numbers that no later change of the oracle or
of a kernel can move. Inputs are regenerated from the recipe (numpy PCG64 streams are stable across platforms), only
outputs (for the larger cases: sampled rows) are stored. bf16 operands are float32 draws rounded to nearest even.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle as mo  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def draw(seed, shape, std=1.0, bf16=False):
    """The input recipe shared with the tests: N(0, std) in float32, optionally rounded to bf16 bit patterns."""
    x = (np.random.default_rng(seed).standard_normal(shape).astype(np.float32) * np.float32(std)).astype(np.float32)
    return mo.to_bf16(x) if bf16 else x


CASES = {
    # name: (kind, parameters)
    "gemm_f32": ("gemm", dict(m=96, n=80, k=72, nk=False, bf16=False, seed=101)),
    "gemm_f32_nk_tc": ("gemm", dict(m=256, n=384, k=260, nk=True, bf16=False, seed=102, rows=[0, 1, 127, 128, 200, 255])),
    "gemm_bf16_nk": ("gemm", dict(m=256, n=264, k=136, nk=True, bf16=True, seed=103, rows=[0, 5, 127, 128, 129, 255])),
    "gemm_bf16_kn": ("gemm", dict(m=640, n=520, k=72, nk=False, bf16=True, seed=104, rows=[0, 63, 511, 512, 639])),
    "softmax_rows": ("softmax", dict(rows=9, cols=1027, seed=105)),
    "rmsnorm_rows": ("rmsnorm", dict(rows=5, cols=8200, seed=106, eps=1e-6)),
    "reduce_sum_ax0": ("reduce", dict(shape=(40, 33, 65), ax=0, monoid="sum", seed=107)),
    "reduce_max_ax1": ("reduce", dict(shape=(40, 33, 65), ax=1, monoid="max", seed=108)),
    "reduce_sum_ax2": ("reduce", dict(shape=(40, 33, 65), ax=2, monoid="sum", seed=109)),
    "attn_bf16_causal": ("attn", dict(bh=3, s=300, d=128, causal=True, bf16=True, seed=110, heads=[1], qrows=[0, 1, 127, 128, 129, 255, 256, 299])),
    "attn_bf16_full": ("attn", dict(bh=2, s=257, d=128, causal=False, bf16=True, seed=111, heads=[0], qrows=[0, 64, 127, 128, 255, 256])),
    "attn_f32_small": ("attn", dict(bh=2, s=64, d=8, causal=False, bf16=False, seed=112, heads=[0, 1])),
    "mlp_gated": ("mlp", dict(m=128, k=64, f=192, n=72, seed=113, rows=[0, 1, 64, 127])),
}


def inputs(kind, p):
    s = p["seed"]
    if kind == "gemm":
        b_shape = (p["n"], p["k"]) if p["nk"] else (p["k"], p["n"])
        return draw(s, (p["m"], p["k"]), 0.5, p["bf16"]), draw(s + 1000, b_shape, 0.5, p["bf16"])
    if kind == "softmax":
        return (draw(s, (p["rows"], p["cols"]), 2.0),)
    if kind == "rmsnorm":
        return draw(s, (p["rows"], p["cols"]), 2.0), (draw(s + 1000, (p["cols"],), 0.25) + np.float32(1.0)).astype(np.float32)
    if kind == "reduce":
        return (draw(s, p["shape"], 1.0),)
    if kind == "attn":
        return tuple(draw(s + 1000 * i, (p["bh"], p["s"], p["d"]), 1.0, p["bf16"]) for i in range(3))
    if kind == "mlp":
        return (draw(s, (p["m"], p["k"]), 1.0, True), draw(s + 1000, (p["k"], p["f"]), 0.1, True),
                draw(s + 2000, (p["k"], p["f"]), 0.1, True), draw(s + 3000, (p["f"], p["n"]), 0.1, True))
    raise ValueError(kind)


def truth(kind, p, ins):
    if kind == "gemm":
        return mo.gemm_truth(ins[0], ins[1], b_nk=p["nk"], bf16=p["bf16"], rows=p.get("rows"))
    if kind == "softmax":
        return mo.softmax_rows(ins[0], truth=True)
    if kind == "rmsnorm":
        return mo.rmsnorm_rows(ins[0], ins[1], p["eps"], truth=True)
    if kind == "reduce":
        return mo.reduce_axis(ins[0], p["ax"], p["monoid"], truth=True)
    if kind == "attn":
        o = mo.attention(*ins, scale=float(p["d"]) ** -0.5, causal=p["causal"], bf16=p["bf16"], heads=p.get("heads"))
        return o[:, p["qrows"]] if "qrows" in p else o
    if kind == "mlp":
        return mo.mlp_gated_truth(*ins, rows=p.get("rows"))
    raise ValueError(kind)


def main():
    out = {}
    for name, (kind, p) in CASES.items():
        out[name] = truth(kind, p, inputs(kind, p)).astype(np.float64)
        # a short checksum of the inputs guards the recipe itself
        out[name + "__insum"] = np.array([float(np.sum(np.asarray(x, dtype=np.float64))) for x in inputs(kind, p)])
    np.savez_compressed(os.path.join(HERE, "cases.npz"), **out)
    print("wrote", os.path.join(HERE, "cases.npz"), {k: v.shape for k, v in out.items() if not k.endswith("__insum")})


if __name__ == "__main__":
    main()
