"""Shared helpers: load the reference fixtures and run them against either implementation."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_fixtures():
    with open(os.path.join(HERE, "golden", "reference_fixtures.json")) as f:
        return json.load(f)


def fixture_input(fx):
    inp = fx["input"]
    if isinstance(inp, dict):
        lo, hi = inp["range"]
        return np.arange(lo, hi + 1).astype(fx["dtype"])
    return np.array(inp, dtype=fx["dtype"])


# Python callables equivalent to the C# lambdas the fixtures use (for the CPU oracle).
F = np.float32
PY_LAMBDAS = {
    "x => x > 3": lambda x: x > 3, "x => x * 2": lambda x: x * np.int32(2), "x => x % 2 == 0": lambda x: x % 2 == 0,
    "x => x > 0": lambda x: x > 0, "x => x > 2": lambda x: x > 2, "x => x > 5": lambda x: x > 5, "x => x < 16": lambda x: x < 16,
    "x => x * 1.5f": lambda x: x * F(1.5), "x => x + 1": lambda x: x + np.int32(1),
    "x => x / 2": lambda x: (np.trunc(x / 2)).astype(np.int32) if hasattr(x, "astype") else np.int32(int(x / 2)),
    "x => true": lambda x: np.ones(np.shape(x), bool), "x => false": lambda x: np.zeros(np.shape(x), bool),
    "x => x < 6": lambda x: x < 6, "x => x < 100": lambda x: x < 100,
    "x => x + 42.0f": lambda x: x + F(42), "x => x * 2.0f + 1.0f": lambda x: x * F(2) + F(1),
    "x => x * 3.5f": lambda x: x * F(3.5), "x => (x * 2.0f + 10.0f) / x": lambda x: (x * F(2) + F(10)) / x,
    "x => x * 2.0f": lambda x: x * F(2),
}


def check_expectation(fx, got):
    """Assert `got` (array, scalar or bool) against whatever the fixture pins."""
    if "expect" in fx:
        exp = fx["expect"]
        if isinstance(exp, list):
            assert list(np.asarray(got).tolist()) == exp, (fx["name"], got)
        else:
            assert got == exp, (fx["name"], got)
    if "expect_len" in fx:
        got = np.asarray(got)
        assert got.size == fx["expect_len"] and got[0] == fx["expect_first"] and got[-1] == fx["expect_last"], fx["name"]
    if "expect_from_linq" in fx:
        x = fixture_input(fx)
        want = {"x + 42": lambda: x + F(42), "x * 2 + 1": lambda: x * F(2) + F(1), "x * 3.5": lambda: x * F(3.5),
                "(x * 2 + 10) / x": lambda: (x * F(2) + F(10)) / x, "x * 2": lambda: x * F(2)}[fx["expect_from_linq"]]()
        got = np.asarray(got)
        if "abs_tol" in fx:        # the reference asserts closeness only (BeApproximately)
            assert got.shape == want.shape and np.all(np.abs(got.astype(np.float64) - want) <= fx["abs_tol"]), fx["name"]
        elif "rel_tol" in fx:
            assert got.shape == want.shape and np.all(np.abs(got.astype(np.float64) - want) <= np.abs(want.astype(np.float64)) * fx["rel_tol"]), fx["name"]
        else:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), fx["name"]
