"""Initialisation kernels (variable-init and sparse-connectivity snippets).

CPU part: the checker's restatement of the snippets has the distributions the
reference documents for them (initSparseConnectivitySnippet.h:170-410,
initVarSnippet.h:87-212); the reference itself checks these statistically
(tests/features/test_connect_init.py).  GPU part: the CUDA kernels reproduce the
checker bit for bit (same Philox streams) through the C ABI."""
import ctypes as C
import math

import numpy as np
import pytest

from genn_b200 import abi
from oracle import oracle

SEED = 77


def test_fixed_probability_rows_are_binomial_sorted_and_unique():
    n_pre, n_post, p = 2000, 1500, 0.08
    rl, ind, overflow = oracle.init_sparse_connectivity(abi.CONNECT_FIXED_PROBABILITY, [p, 1.0 / math.log(1.0 - p)],
                                                        n_pre, 220, np.uint16, 0, n_post, SEED, 1)
    assert not overflow
    assert abs(rl.mean() / (n_post * p) - 1.0) < 0.01
    assert abs(rl.var() / (n_post * p * (1 - p)) - 1.0) < 0.1
    rows = ind.reshape(n_pre, 220)
    for i in range(0, n_pre, 97):
        r = rows[i, :rl[i]].astype(np.int64)
        assert np.all(np.diff(r) > 0) and r.max() < n_post
    counts = np.bincount(np.concatenate([rows[i, :rl[i]] for i in range(n_pre)]), minlength=n_post)
    assert abs(counts.mean() / (n_pre * p) - 1.0) < 0.01
    assert counts.std() / math.sqrt(n_pre * p * (1 - p)) < 1.15       # columns binomial too


def test_fixed_number_total_rows_ascend_and_cover_targets_uniformly():
    n_pre, n_post, total = 500, 4000, 200000
    rng = np.random.default_rng(1)
    row_length = rng.multinomial(total, np.full(n_pre, 1.0 / n_pre)).astype(np.uint32)
    stride = int(row_length.max())
    rl, ind, overflow = oracle.init_sparse_connectivity(abi.CONNECT_FIXED_NUMBER_TOTAL, [float(total)], n_pre, stride,
                                                        np.uint32, 0, n_post, SEED, 2, row_length=row_length)
    assert not overflow and np.array_equal(rl, row_length)
    rows = ind.reshape(n_pre, stride)
    allpost = np.concatenate([rows[i, :rl[i]] for i in range(n_pre)])
    for i in range(0, n_pre, 37):
        assert np.all(np.diff(rows[i, :rl[i]].astype(np.int64)) >= 0)
    counts = np.bincount(allpost, minlength=n_post)
    assert len(allpost) == total and counts.min() > 0
    assert abs(counts.std() / math.sqrt(total / n_post) - 1.0) < 0.1     # Poisson-like column counts


def test_target_slice_keeps_indices_inside_the_slice():
    rl, ind, _ = oracle.init_sparse_connectivity(abi.CONNECT_FIXED_NUMBER_POST, [50.0], 300, 50, np.uint16, 640, 1280,
                                                 SEED, 3)
    assert np.all(rl == 50) and ind.min() >= 640 and ind.max() < 1280


def test_fixed_number_pre_gives_every_target_its_in_degree():
    rl, ind, overflow = oracle.init_sparse_connectivity(abi.CONNECT_FIXED_NUMBER_PRE, [20.0], 400, 60, np.uint32, 0, 300,
                                                        SEED, 4)
    assert not overflow and rl.sum() == 20 * 300
    rows = ind.reshape(400, 60)
    allpost = np.concatenate([rows[i, :rl[i]] for i in range(400)])
    assert np.all(np.bincount(allpost, minlength=300) == 20)


def test_variable_snippets_have_their_distributions():
    n = 200000
    u = oracle.init_var(n, np.float32, abi.INIT_UNIFORM, [-2.0, 3.0], SEED, 5)
    assert u.min() >= -2.0 and u.max() <= 3.0 and abs(u.mean() - 0.5) < 0.02
    z = oracle.init_var(n, np.float32, abi.INIT_NORMAL, [-58.0, 5.0], SEED, 6)
    assert abs(z.mean() + 58.0) < 0.05 and abs(z.std() - 5.0) < 0.05
    w = oracle.init_var(n, np.float32, abi.INIT_NORMAL_CLIPPED, [0.0878, 0.0878, 0.0, 0.12], SEED, 7)
    assert w.min() >= 0.0 and w.max() <= 0.12
    d = oracle.init_var(n, np.uint8, abi.INIT_NORMAL_CLIPPED_DELAY, [15.0, 7.5, 0.0, 42.89], SEED, 8)
    assert d.max() <= 43 and abs(d.mean() - 15.3) < 0.3          # truncation at zero shifts the mean up


# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def runner():
    lib = abi.load_library()
    h = C.c_void_p()
    abi.check(lib.b200_runner_create(0, 0.1, SEED, 1, C.byref(h)))
    yield lib, h
    lib.b200_runner_destroy(h)


def _alloc(lib, h, nbytes):
    p = C.c_void_p()
    abi.check(lib.b200_array_alloc(h, nbytes, C.byref(p)))
    return p


def _pull(lib, h, ptr, count, dtype):
    out = np.zeros(count, dtype=dtype)
    abi.check(lib.b200_array_pull(h, out.ctypes.data, ptr, out.nbytes))
    return out


def _params(v):
    return (C.c_float * 4)(*(list(v) + [0.0] * 4)[:4])


@pytest.mark.gpu
@pytest.mark.parametrize("snippet,params,dtype", [
    (abi.INIT_UNIFORM, [-2.0, 3.0], np.float32),
    (abi.INIT_NORMAL, [-58.0, 5.0], np.float32),
    (abi.INIT_NORMAL_CLIPPED, [0.0878, 0.00878, 0.0, 3.4e38], np.float32),
    (abi.INIT_NORMAL_CLIPPED_DELAY, [15.0, 7.5, 0.0, 42.89], np.uint8)])
def test_gpu_init_var_is_bit_identical_to_checker(runner, snippet, params, dtype):
    lib, h = runner
    n = 300001
    ptr = _alloc(lib, h, n * np.dtype(dtype).itemsize)
    abi.check(lib.b200_init_var(h, ptr, np.dtype(dtype).itemsize, n, snippet, _params(params), 9))
    got = _pull(lib, h, ptr, n, dtype)
    assert np.array_equal(got, oracle.init_var(n, dtype, snippet, params, SEED, 9))
    lib.b200_array_free(h, ptr)


@pytest.mark.gpu
@pytest.mark.parametrize("snippet,params,ind_dtype,stride", [
    (abi.CONNECT_FIXED_PROBABILITY, [0.08, 1.0 / math.log(0.92)], np.uint16, 220),
    (abi.CONNECT_FIXED_PROBABILITY_NO_AUTAPSE, [0.08, 1.0 / math.log(0.92)], np.uint32, 220),
    (abi.CONNECT_FIXED_NUMBER_TOTAL, [150000.0], np.uint16, None),
    (abi.CONNECT_FIXED_NUMBER_POST, [64.0], np.uint8, 64),
    (abi.CONNECT_FIXED_NUMBER_PRE, [20.0], np.uint32, 70)])
def test_gpu_connectivity_build_matches_checker(runner, snippet, params, ind_dtype, stride):
    lib, h = runner
    n_pre = 1500
    n_post = 250 if ind_dtype == np.uint8 else 1500
    begin, end = (0, n_post) if snippet != abi.CONNECT_FIXED_NUMBER_POST else (32, n_post)
    row_length = None
    if snippet == abi.CONNECT_FIXED_NUMBER_TOTAL:
        row_length = np.random.default_rng(5).multinomial(int(params[0]), np.full(n_pre, 1.0 / n_pre)).astype(np.uint32)
        stride = int(row_length.max()) + 3
    want_rl, want_ind, overflow = oracle.init_sparse_connectivity(snippet, params, n_pre, stride, ind_dtype, begin, end,
                                                                  SEED, 12, row_length=row_length)
    assert not overflow
    isz = np.dtype(ind_dtype).itemsize
    d_rl, d_ind = _alloc(lib, h, n_pre * 4), _alloc(lib, h, n_pre * stride * isz)
    if row_length is not None:
        abi.check(lib.b200_array_push(h, d_rl, row_length.ctypes.data, row_length.nbytes))
    abi.check(lib.b200_init_sparse_connectivity(h, snippet, _params(params), n_pre, n_post, stride, isz, begin, end,
                                                d_rl, d_ind, 12))
    abi.check(lib.b200_synchronize(h))
    got_rl = _pull(lib, h, d_rl, n_pre, np.uint32)
    got_ind = _pull(lib, h, d_ind, n_pre * stride, ind_dtype).reshape(n_pre, stride)
    assert np.array_equal(got_rl, want_rl)
    want_ind = want_ind.reshape(n_pre, stride)
    for i in range(n_pre):
        a, b = got_ind[i, :got_rl[i]], want_ind[i, :want_rl[i]]
        if snippet == abi.CONNECT_FIXED_NUMBER_PRE:      # row order depends on atomics: compare as multisets
            a, b = np.sort(a), np.sort(b)
        assert np.array_equal(a, b), f"row {i}"
    # per-synapse variables over the ragged rows
    d_g = _alloc(lib, h, n_pre * stride * 4)
    gp = [0.0878, 0.00878, 0.0, 3.4e38]
    abi.check(lib.b200_init_sparse_vars(h, d_rl, n_pre, stride, d_g, 4, abi.INIT_NORMAL_CLIPPED, _params(gp), 13))
    got_g = _pull(lib, h, d_g, n_pre * stride, np.float32)
    assert np.array_equal(got_g, oracle.init_sparse_vars(want_rl, stride, np.float32, abi.INIT_NORMAL_CLIPPED, gp, SEED, 13))
    for p in (d_rl, d_ind, d_g):
        lib.b200_array_free(h, p)


@pytest.mark.gpu
def test_gpu_remap_matches_checker_per_column(runner):
    lib, h = runner
    n_pre, n_post, stride = 300, 200, 40
    rl, ind, _ = oracle.init_sparse_connectivity(abi.CONNECT_FIXED_NUMBER_POST, [40.0], n_pre, stride, np.uint16, 0, n_post,
                                                 SEED, 20)
    cols = np.bincount(ind, minlength=n_post)
    cs = int(cols.max())
    want_cl, want_remap = np.zeros(n_post, np.uint32), np.zeros(n_post * cs, np.uint32)
    oracle.lib().oracle_build_remap(rl.ctypes.data, ind.ctypes.data, 2, n_pre, n_post, stride, cs,
                                    want_cl.ctypes.data, want_remap.ctypes.data)
    d_rl, d_ind = _alloc(lib, h, rl.nbytes), _alloc(lib, h, ind.nbytes)
    d_cl, d_remap = _alloc(lib, h, n_post * 4), _alloc(lib, h, n_post * cs * 4)
    abi.check(lib.b200_array_push(h, d_rl, rl.ctypes.data, rl.nbytes))
    abi.check(lib.b200_array_push(h, d_ind, ind.ctypes.data, ind.nbytes))
    abi.check(lib.b200_build_remap(h, d_rl, d_ind, 2, n_pre, n_post, stride, cs, d_cl, d_remap))
    abi.check(lib.b200_synchronize(h))
    got_cl = _pull(lib, h, d_cl, n_post, np.uint32)
    got_remap = _pull(lib, h, d_remap, n_post * cs, np.uint32).reshape(n_post, cs)
    assert np.array_equal(got_cl, want_cl)
    want_remap = want_remap.reshape(n_post, cs)
    for j in range(n_post):
        assert np.array_equal(np.sort(got_remap[j, :got_cl[j]]), np.sort(want_remap[j, :want_cl[j]]))
