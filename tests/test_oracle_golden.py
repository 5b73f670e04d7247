"""The CPU oracle against the reference's own fixtures (tests/golden/reference_fixtures.json) and against itself
(C restatement vs numpy restatement) on seeded inputs. No GPU."""
import numpy as np
import pytest

import oracle
from oracle.linq_oracle import Enumerable, InvalidOperationError, scalar_enumerable_where_select
from tests.fixture_util import PY_LAMBDAS, check_expectation, fixture_input, load_fixtures

F = np.float32


@pytest.mark.parametrize("fx", load_fixtures(), ids=lambda f: f["name"])
def test_oracle_reproduces_reference_fixture(fx):
    q = Enumerable(fixture_input(fx))
    for op, arg in fx["ops"]:
        if op == "Where":
            q = q.Where(PY_LAMBDAS[arg])
        elif op == "Select":
            q = q.Select(PY_LAMBDAS[arg])
        elif op == "Take":
            q = q.Take(arg)
        elif op == "Skip":
            q = q.Skip(arg)
    term = fx["terminal"]
    if isinstance(term, list):
        got = getattr(q, term[0])(PY_LAMBDAS[term[1]])
    else:
        got = getattr(q, term)()
    check_expectation(fx, got)


def test_c_oracle_agrees_with_numpy_oracle():
    o = oracle.c_oracle()
    x = np.random.Generator(np.random.PCG64(11)).random(1 << 20, dtype=F)
    for thr in (0.5, 0.99, 0.01):
        a = o.where_gt_select_sq_add(x, thr, 3.0)
        b = Enumerable(x).Where(lambda v: v > F(thr)).Select(lambda v: v * v + F(3)).ToArray()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        s, raw, cnt = o.where_gt_select_sq_add_sum(x, thr, 3.0)
        assert cnt == b.size and s == Enumerable(b).Sum()
    y = np.random.Generator(np.random.PCG64(7)).standard_normal(1 << 20, dtype=F)
    assert o.sum_f32(y)[0] == Enumerable(y).Sum()
    assert o.min_f32(y) == Enumerable(y).Min() and o.max_f32(y) == Enumerable(y).Max()
    assert o.average_f32(y) == Enumerable(y).Average()
    k = np.random.Generator(np.random.PCG64(8)).integers(-1000, 1001, 1 << 20, dtype=np.int32)
    assert o.sum_i32(k) == Enumerable(k).Sum() and o.min_i32(k) == k.min() and o.max_i32(k) == k.max()
    assert o.average_i32(k) == Enumerable(k).Average()
    keys = np.random.Generator(np.random.PCG64(23)).integers(-2**63, 2**63 - 1, 1 << 18, dtype=np.int64, endpoint=True)
    assert np.array_equal(o.where_mask_eq_i64(keys, 0xF, 3), keys[(keys & 0xF) == 3])


def test_oracle_does_not_contract_to_fma():
    o = oracle.c_oracle()
    x = np.random.Generator(np.random.PCG64(5)).random(1 << 16, dtype=F)
    got = o.where_gt_select_sq_add(x, -1.0, 3.0)
    fused = (x.astype(np.float64) * x.astype(np.float64) + 3.0).astype(F)
    assert np.array_equal(got, x * x + F(3))
    assert (got != fused).any()          # the input can tell the two apart, and the oracle is on the unfused side


def test_pure_python_loop_matches_vector_oracle():
    x = np.random.Generator(np.random.PCG64(1)).random(257, dtype=F)
    a = scalar_enumerable_where_select(x, lambda v: v > F(0.5), lambda v: v * v + F(3))
    b = Enumerable(x).Where(lambda v: v > F(0.5)).Select(lambda v: v * v + F(3)).ToArray()
    assert [np.float32(v) for v in a] == b.tolist()


def test_oracle_linq_exceptions_and_nan_rules():
    o = oracle.c_oracle()
    e = np.array([], dtype=F)
    assert o.sum_f32(e)[0] == 0
    for fn in (o.min_f32, o.max_f32, o.average_f32):
        with pytest.raises(oracle.InvalidOperationError):
            fn(e)
    with pytest.raises(InvalidOperationError):
        Enumerable(e).Min()
    with pytest.raises(OverflowError):
        o.sum_i32(np.full(3, 2**30, dtype=np.int32))
    with pytest.raises(OverflowError):
        Enumerable(np.full(3, 2**30, dtype=np.int32)).Sum()
    x = np.array([1.0, np.nan, -2.0, 7.5], dtype=F)
    assert np.isnan(o.min_f32(x)) and o.max_f32(x) == F(7.5)
    assert np.isnan(Enumerable(x).Min()) and Enumerable(x).Max() == F(7.5)
    assert np.isnan(o.max_f32(np.array([np.nan, np.nan], dtype=F)))


def test_cpu_simd_baseline_is_close_to_the_oracle():
    s, o = oracle.cpu_simd(), oracle.c_oracle()
    x = np.random.Generator(np.random.PCG64(31)).random(1 << 20, dtype=F)
    want, raw, _ = o.where_gt_select_sq_add_sum(x, 0.5, 3.0)
    for threads in (1, 3, s.threads):
        got = s.where_select_sum(x, 0.5, 3.0, threads)
        assert abs(float(got) - raw) <= 1e-4 * raw      # fp32 lanes, as the reference's SIMD Sum: looser than the GPU bar
    assert s.scalar_where_select_sum(x, 0.5, 3.0) == want
    assert np.array_equal(s.where_select_toarray(x, 0.5, 3.0), o.where_gt_select_sq_add(x, 0.5, 3.0))
