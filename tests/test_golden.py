"""Committed fixtures produced by the unmodified reference CPU evaluator
(tests/golden/make_golden.py): the plain-C oracle must reproduce them bit for bit anywhere,
and the CUDA path must match them on a GPU within the tolerances of test_gpu_parity.py."""
import os

import numpy as np
import pytest

import cpu_checkers as cc

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
orc = cc.load("orc")


def same_bits(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


# ----------------------------------------------------------------------------- oracle (CPU)
@pytest.mark.parametrize("cid", range(10))
def test_oracle_expressions(cid):
    got = orc.expr_case(cid, G["expr_d0"].copy(), G["expr_A"], G["expr_B"], G["expr_C"], G["expr_bias"])
    assert same_bits(got, G["expr_out_%d" % cid])


@pytest.mark.parametrize("reducer", range(3))
def test_oracle_reductions(reducer):
    assert same_bits(orc.reduce_keep_lowest(np.zeros(52, np.float32), G["red_M"], scale=0.5, reducer=reducer),
                     G["keep_lowest_%d" % reducer])
    assert same_bits(orc.reduce_keep_highdim(np.zeros(10, np.float32), G["red_T"], scale=2.0, reducer=reducer),
                     G["keep_highdim_%d" % reducer])


def test_oracle_softmax_family():
    L, lab = G["sm_logits"], G["sm_label"]
    P = orc.softmax(np.zeros_like(L), L)
    assert same_bits(P, G["sm_prob"])
    for mode in range(4):
        got = orc.softmax_grad(np.zeros_like(L), P, lab, mode=mode, ignore_label=float(lab[3]), alpha=0.1)
        assert same_bits(got, G["sm_grad_%d" % mode])


@pytest.mark.parametrize("reducer", range(3))
def test_oracle_pooling(reducer):
    X, gP = G["pool_X"], G["pool_gP"]
    Pm = orc.pool(np.zeros((6, 6, 6), np.float32), X, 3, 3, 2, 2, reducer=reducer)
    assert same_bits(Pm, G["pool_%d" % reducer])
    assert same_bits(orc.unpool(np.zeros_like(X), X, Pm, gP, 3, 3, 2, 2, reducer=reducer), G["unpool_%d" % reducer])


def test_oracle_chpool():
    X4 = G["chpool_X"]
    assert same_bits(orc.chpool(np.zeros_like(X4), X4, 5, reducer=0), G["chpool_sum5"])
    assert same_bits(orc.chpool(np.zeros_like(X4), X4, 3, reducer=1), G["chpool_max3"])
    assert same_bits(orc.chpool(np.zeros((2, 6, 5, 8), np.float32), X4, 3, 2, 1, reducer=0), G["chpool_sum3_s2"])


def test_oracle_embedding():
    idx, src, t0 = G["emb_idx"], G["emb_src"], G["emb_t0"]
    assert same_bits(orc.addtakegrad(t0.copy(), idx, src), G["emb_addtakegrad"])
    keys, vals = np.clip(idx, 0, 39).astype(np.int32), np.arange(idx.size, dtype=np.int32)
    orc.sort_by_key(keys, vals, True)
    assert np.array_equal(keys, G["emb_sorted"]) and np.array_equal(vals, G["emb_order"])
    assert same_bits(orc.addtakegrad_largebatch(t0.copy(), keys, vals, src), G["emb_largebatch"])
    kd, vd = np.clip(idx, 0, 39).astype(np.int32), np.arange(idx.size, dtype=np.int32)
    orc.sort_by_key(kd, vd, False)
    assert np.array_equal(kd, G["emb_sorted_desc"]) and np.array_equal(vd, G["emb_order_desc"])


def test_oracle_softmax3d_fill_and_segment_sort():
    L3, lab3 = G["sm3_logits"], G["sm3_label"]
    P3 = orc.softmax3d(np.zeros_like(L3), L3)
    assert same_bits(P3, G["sm3_prob"])
    for mode in range(4):
        got = orc.softmax_grad3d(np.zeros_like(L3), P3, lab3, mode=mode, ignore_label=float(lab3[1, 2]), alpha=0.1)
        assert same_bits(got, G["sm3_grad_%d" % mode])
    assert same_bits(orc.index_fill(G["fill_t0"].copy(), G["fill_idx"], G["fill_src"]), G["fill_out"])
    v, s = orc.vectorized_sort(G["vsort_val"].copy(), G["vsort_seg"].copy())
    assert same_bits(v, G["vsort_out"]) and np.array_equal(s, G["vsort_seg"])


# ----------------------------------------------------------------------------- CUDA path
@pytest.fixture(scope="module")
def gpu():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import mshadow_b200
    lib = mshadow_b200.load()
    lib.init(0)
    return lib, torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def sum_close(got, want, per_row=False):
    w = want.astype(np.float64)
    rms = np.sqrt(np.mean(w ** 2, axis=-1, keepdims=True)) if per_row else np.sqrt(np.mean(w ** 2))
    return np.max(np.abs(got.astype(np.float64) - w) / np.maximum(np.abs(w), rms)) <= 1e-5


@pytest.mark.gpu
def test_gpu_matches_fixtures(gpu):
    lib, torch = gpu
    d = lambda a: dev(torch, a)  # noqa: E731
    h = lambda t: t.cpu().numpy()  # noqa: E731
    for cid in range(10):
        got = h(lib.expr_case(cid, d(G["expr_d0"]), d(G["expr_A"]), d(G["expr_B"]), d(G["expr_C"]),
                              d(G["expr_bias"])))
        want = G["expr_out_%d" % cid]
        if cid == 0:
            ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
            assert ulp.max() <= 1
        else:
            assert same_bits(got, want), cid
    for reducer in range(3):
        lo = h(lib.reduce_keep_lowest(torch.zeros(52, device="cuda"), d(G["red_M"]), scale=0.5, reducer=reducer))
        hi = h(lib.reduce_keep_highdim(torch.zeros(10, device="cuda"), d(G["red_T"]), scale=2.0, reducer=reducer))
        if reducer == 0:
            assert sum_close(lo, G["keep_lowest_0"]) and sum_close(hi, G["keep_highdim_0"])
        else:
            assert same_bits(lo, G["keep_lowest_%d" % reducer]) and same_bits(hi, G["keep_highdim_%d" % reducer])
    L, lab, P = G["sm_logits"], G["sm_label"], G["sm_prob"]
    got = h(lib.softmax(torch.zeros(L.shape, device="cuda"), d(L)))
    assert np.max(np.abs(got.astype(np.float64) - P) / P) <= 1e-5
    for mode in range(4):
        got = h(lib.softmax_grad(torch.zeros(L.shape, device="cuda"), d(P), d(lab), mode=mode,
                                 ignore_label=float(lab[3]), alpha=0.1))
        assert same_bits(got, G["sm_grad_%d" % mode])
    X, gP = G["pool_X"], G["pool_gP"]
    for reducer in range(3):
        Pm = lib.pool(torch.zeros(6, 6, 6, device="cuda"), d(X), 3, 3, 2, 2, reducer=reducer)
        assert same_bits(h(Pm), G["pool_%d" % reducer])
        U = lib.unpool(torch.zeros(X.shape, device="cuda"), d(X), Pm, d(gP), 3, 3, 2, 2, reducer=reducer)
        assert same_bits(h(U), G["unpool_%d" % reducer])
    X4 = G["chpool_X"]
    assert same_bits(h(lib.chpool(torch.zeros(X4.shape, device="cuda"), d(X4), 5, reducer=0)), G["chpool_sum5"])
    assert same_bits(h(lib.chpool(torch.zeros(X4.shape, device="cuda"), d(X4), 3, reducer=1)), G["chpool_max3"])
    assert same_bits(h(lib.chpool(torch.zeros(2, 6, 5, 8, device="cuda"), d(X4), 3, 2, 1, reducer=0)),
                     G["chpool_sum3_s2"])
    idx, src, t0 = G["emb_idx"], G["emb_src"], G["emb_t0"]
    assert sum_close(h(lib.addtakegrad(d(t0), d(idx), d(src))), G["emb_addtakegrad"], per_row=True)
    keys, vals = np.clip(idx, 0, 39).astype(np.int32), np.arange(idx.size, dtype=np.int32)
    gk, gv = lib.sort_by_key(d(keys), d(vals), True)
    assert np.array_equal(h(gk), G["emb_sorted"]) and np.array_equal(h(gv), G["emb_order"])
    assert sum_close(h(lib.addtakegrad_largebatch(d(t0), gk, gv, d(src))), G["emb_largebatch"], per_row=True)
    gk, gv = lib.sort_by_key(d(keys), d(vals), False)
    assert np.array_equal(h(gk), G["emb_sorted_desc"]) and np.array_equal(h(gv), G["emb_order_desc"])
    L3, lab3, P3 = G["sm3_logits"], G["sm3_label"], G["sm3_prob"]
    got = h(lib.softmax3d(torch.zeros(L3.shape, device="cuda"), d(L3)))
    assert np.max(np.abs(got.astype(np.float64) - P3) / P3) <= 1e-5
    for mode in range(4):
        got = h(lib.softmax_grad3d(torch.zeros(L3.shape, device="cuda"), d(P3), d(lab3), mode=mode,
                                   ignore_label=float(lab3[1, 2]), alpha=0.1))
        assert same_bits(got, G["sm3_grad_%d" % mode])
    assert same_bits(h(lib.index_fill(d(G["fill_t0"]), d(G["fill_idx"]), d(G["fill_src"]))), G["fill_out"])
    gv, gs = lib.vectorized_sort(d(G["vsort_val"]), d(G["vsort_seg"]))
    assert same_bits(h(gv), G["vsort_out"]) and np.array_equal(h(gs), G["vsort_seg"])
