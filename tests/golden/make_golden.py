"""Generates tests/golden/golden.npz from the UNMODIFIED reference CPU evaluator.

Run where oracle/_ref/libmshadow_ref.so exists (it is built from the reference headers by
oracle/Makefile).  Inputs are seeded; each case stores its inputs' seed-derived arrays and the
reference's outputs, so the fixtures stay valid on machines without the reference tree.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import cpu_checkers as cc  # noqa: E402


def main():
    ref = cc.load("ref")
    if ref is None:
        raise SystemExit("oracle/_ref/libmshadow_ref.so not built: cannot generate fixtures")
    rng = np.random.default_rng(20261125)
    out = {}

    def f32(a):
        return np.ascontiguousarray(a, dtype=np.float32)

    # element-wise expressions, all ten cases on one 24x36 problem
    shape = (24, 36)
    A, B = f32(rng.uniform(-1, 1, shape)), f32(rng.uniform(-1, 1, shape))
    Cm = f32(rng.uniform(0.5, 1.5, shape))
    bias = f32(rng.standard_normal(max(shape)))
    d0 = f32(rng.uniform(0.5, 2.0, shape))
    out.update(expr_A=A, expr_B=B, expr_C=Cm, expr_bias=bias, expr_d0=d0)
    for cid in range(10):
        out["expr_out_%d" % cid] = ref.expr_case(cid, d0.copy(), A, B, Cm, bias)

    # reductions
    M = f32(rng.standard_normal((300, 52)))
    T = f32(rng.standard_normal((6, 10, 7, 8)))
    out.update(red_M=M, red_T=T)
    for reducer in range(3):
        out["keep_lowest_%d" % reducer] = ref.reduce_keep_lowest(np.zeros(52, np.float32), M, scale=0.5,
                                                                reducer=reducer)
        out["keep_highdim_%d" % reducer] = ref.reduce_keep_highdim(np.zeros(10, np.float32), T, scale=2.0,
                                                                  reducer=reducer)

    # softmax family
    L = f32(2.0 * rng.standard_normal((12, 100)))
    lab = f32(rng.integers(0, 100, 12))
    lab[0], lab[-1] = 0, 99
    P = ref.softmax(np.zeros_like(L), L)
    out.update(sm_logits=L, sm_label=lab, sm_prob=P)
    for mode in range(4):
        out["sm_grad_%d" % mode] = ref.softmax_grad(np.zeros_like(L), P, lab, mode=mode, ignore_label=float(lab[3]),
                                                    alpha=0.1)

    # pooling, values on a coarse grid so that maxima tie
    X = f32(rng.integers(0, 6, size=(6, 14, 14)) / 4.0)
    gP = f32(rng.uniform(0, 1, (6, 6, 6)))
    out.update(pool_X=X, pool_gP=gP)
    for reducer in range(3):
        Pm = ref.pool(np.zeros((6, 6, 6), np.float32), X, 3, 3, 2, 2, reducer=reducer)
        out["pool_%d" % reducer] = Pm
        out["unpool_%d" % reducer] = ref.unpool(np.zeros_like(X), X, Pm, gP, 3, 3, 2, 2, reducer=reducer)
    X4 = f32(rng.uniform(-1, 1, (2, 12, 5, 8)))
    out["chpool_X"] = X4
    out["chpool_sum5"] = ref.chpool(np.zeros_like(X4), X4, 5, reducer=0)
    out["chpool_max3"] = ref.chpool(np.zeros_like(X4), X4, 3, reducer=1)
    out["chpool_sum3_s2"] = ref.chpool(np.zeros((2, 6, 5, 8), np.float32), X4, 3, 2, 1, reducer=0)

    # embedding backward
    k, d, n = 40, 24, 500
    idx = rng.integers(-2, k + 2, n).astype(np.int32)
    src = f32(rng.standard_normal((n, d)))
    t0 = f32(rng.standard_normal((k, d)))
    out.update(emb_idx=idx, emb_src=src, emb_t0=t0)
    out["emb_addtakegrad"] = ref.addtakegrad(t0.copy(), idx, src)
    keys, vals = np.clip(idx, 0, k - 1).astype(np.int32), np.arange(n, dtype=np.int32)
    ref.sort_by_key(keys, vals, True)
    out.update(emb_sorted=keys, emb_order=vals)
    out["emb_largebatch"] = ref.addtakegrad_largebatch(t0.copy(), keys, vals, src)
    kd, vd = np.clip(idx, 0, k - 1).astype(np.int32), np.arange(n, dtype=np.int32)
    ref.sort_by_key(kd, vd, False)
    out.update(emb_sorted_desc=kd, emb_order_desc=vd)

    # softmax over the middle axis and its gradients, IndexFill, VectorizedSort
    L3 = f32(rng.standard_normal((3, 7, 10)) * 2)
    lab3 = f32(rng.integers(0, 7, size=(3, 10)))
    P3 = ref.softmax3d(np.zeros_like(L3), L3)
    out.update(sm3_logits=L3, sm3_label=lab3, sm3_prob=P3)
    for mode in range(4):
        out["sm3_grad_%d" % mode] = ref.softmax_grad3d(np.zeros_like(L3), P3, lab3, mode=mode,
                                                       ignore_label=float(lab3[1, 2]), alpha=0.1)
    fidx = rng.integers(0, 12, size=30).astype(np.int32)
    fsrc = f32(rng.standard_normal((30, 6)))
    ft0 = f32(rng.standard_normal((12, 6)))
    out.update(fill_idx=fidx, fill_src=fsrc, fill_t0=ft0)
    out["fill_out"] = ref.index_fill(ft0.copy(), fidx, fsrc)
    seg = np.sort(rng.integers(0, 5, size=64)).astype(np.int32)
    sval = f32(rng.integers(0, 16, size=64) / 4.0)
    out.update(vsort_seg=seg, vsort_val=sval)
    out["vsort_out"] = ref.vectorized_sort(sval.copy(), seg.copy())[0]

    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote %s (%d arrays, %d bytes)" % (path, len(out), os.path.getsize(path)))


if __name__ == "__main__":
    main()
