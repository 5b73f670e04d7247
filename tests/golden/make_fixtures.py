"""Writes reference_fixtures.json: the input/output pairs the reference's own tests pin for the LINQ path.

The reference is C#/.NET and cannot run in this image, so the values below were read from its test sources as text;
`src` names the file and lines inside the DotCompute tree. Inputs given as ranges are expanded here. Expected outputs
are the literals the reference asserts (never computed by this script), except `expect_from_linq`, where the
reference test itself asserts equality with System.Linq over the same lambda: there the expected column is left out
and the test compares oracle and GPU against IEEE float arithmetic done operation by operation. Where the reference
asserts only closeness (`abs_tol` / `rel_tol`, its own numbers), the fixture carries that tolerance.

Run: python tests/golden/make_fixtures.py
"""
import json
import os

T = "tests/Unit/DotCompute.Linq.Tests/ComputeQueryProviderTests.cs"
R = "tests/Integration/DotCompute.Linq.Integration.Tests/RuntimeOrchestrationTests.cs"
E = "tests/Unit/DotCompute.Linq.Tests/ComputeQueryableExtensionsTests.cs"
C = "tests/Integration/DotCompute.Linq.Tests/CpuIntegrationTests.cs"

FIX = [
    {"name": "where_gt3", "src": f"{T}:340-351", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [["Where", "x => x > 3"]], "terminal": "ToArray", "expect": [4, 5]},
    {"name": "select_times2", "src": f"{T}:354-366", "dtype": "int32", "input": [1, 2, 3],
     "ops": [["Select", "x => x * 2"]], "terminal": "ToArray", "expect": [2, 4, 6]},
    {"name": "take3", "src": f"{T}:383-395", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [["Take", 3]], "terminal": "ToArray", "expect": [1, 2, 3]},
    {"name": "skip2", "src": f"{T}:397-408", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [["Skip", 2]], "terminal": "ToArray", "expect": [3, 4, 5]},
    {"name": "even_take100", "src": f"{T}:466-479", "dtype": "int32", "input": {"range": [1, 10000]},
     "ops": [["Where", "x => x % 2 == 0"], ["Take", 100]], "terminal": "ToArray",
     "expect_len": 100, "expect_first": 2, "expect_last": 200},
    {"name": "empty_where", "src": f"{T}:482-494", "dtype": "int32", "input": [],
     "ops": [["Where", "x => x > 0"]], "terminal": "ToArray", "expect": []},
    {"name": "single_roundtrip", "src": f"{T}:496-507", "dtype": "int32", "input": [42],
     "ops": [], "terminal": "ToArray", "expect": [42]},
    {"name": "count5", "src": f"{T}:560-572", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [], "terminal": "Count", "expect": 5},
    {"name": "any_gt2", "src": f"{T}:574-586", "dtype": "int32", "input": [1, 2, 3],
     "ops": [], "terminal": ["Any", "x => x > 2"], "expect": True},
    {"name": "all_gt0", "src": f"{T}:588-599", "dtype": "int32", "input": [1, 2, 3],
     "ops": [], "terminal": ["All", "x => x > 0"], "expect": True},
    {"name": "sum15", "src": f"{T}:601-613", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [], "terminal": "Sum", "expect": 15},
    {"name": "roundtrip_1_5", "src": f"{R}:112-120", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [], "terminal": "ToArray", "expect": [1, 2, 3, 4, 5]},
    {"name": "compute_select_double", "src": f"{R}:126-137", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [["Select", "x => x * 2"]], "terminal": "ToArray", "expect": [2, 4, 6, 8, 10]},
    {"name": "compute_where_gt5", "src": f"{R}:139-151", "dtype": "int32", "input": {"range": [1, 10]},
     "ops": [["Where", "x => x > 5"]], "terminal": "ToArray", "expect": [6, 7, 8, 9, 10]},
    {"name": "where_select_where", "src": f"{R}:153-166", "dtype": "int32", "input": {"range": [1, 10]},
     "ops": [["Where", "x => x > 3"], ["Select", "x => x * 2"], ["Where", "x => x < 16"]], "terminal": "ToArray",
     "expect": [8, 10, 12, 14]},
    {"name": "float_times_1_5", "src": f"{R}:168-180", "dtype": "float32", "input": [1.0, 2.0, 3.0, 4.0],
     "ops": [["Select", "x => x * 1.5f"]], "terminal": "ToArray", "expect": [1.5, 3.0, 4.5, 6.0]},
    {"name": "empty_select", "src": f"{R}:186-196", "dtype": "int32", "input": [],
     "ops": [["Select", "x => x + 1"]], "terminal": "ToArray", "expect": []},
    {"name": "int_div2", "src": f"{R}:198-209", "dtype": "int32", "input": [10, 20, 30, 40],
     "ops": [["Select", "x => x / 2"]], "terminal": "ToArray", "expect": [5, 10, 15, 20]},
    {"name": "where_then_select", "src": f"{E}:331-345", "dtype": "int32", "input": [1, 2, 3, 4, 5],
     "ops": [["Where", "x => x > 2"], ["Select", "x => x * 2"]], "terminal": "ToArray", "expect": [6, 8, 10]},
    {"name": "always_true", "src": f"{E}:435-446", "dtype": "int32", "input": [1, 2, 3],
     "ops": [["Where", "x => true"]], "terminal": "ToArray", "expect": [1, 2, 3]},
    {"name": "always_false", "src": f"{E}:448-459", "dtype": "int32", "input": [1, 2, 3],
     "ops": [["Where", "x => false"]], "terminal": "ToArray", "expect": []},
    {"name": "where_twice", "src": f"{E}:494-508", "dtype": "int32", "input": [1, 2, 3, 4, 5, 6],
     "ops": [["Where", "x => x > 2"], ["Where", "x => x < 6"]], "terminal": "ToArray", "expect": [3, 4, 5]},
    {"name": "thousand_chain", "src": f"{E}:587-608", "dtype": "int32", "input": {"range": [1, 1000]},
     "ops": [["Where", "x => x % 2 == 0"], ["Select", "x => x * 2"], ["Where", "x => x < 100"]], "terminal": "ToArray",
     "expect_len": 24, "expect_first": 4, "expect_last": 96},
    {"name": "large_roundtrip", "src": f"{E}:225-238", "dtype": "int32", "input": {"range": [1, 10000]},
     "ops": [], "terminal": "ToArray", "expect_len": 10000, "expect_first": 1, "expect_last": 10000},
    {"name": "add42_matches_linq", "src": f"{C}:490-504", "dtype": "float32", "input": {"range": [0, 9999]},
     "ops": [["Select", "x => x + 42.0f"]], "terminal": "ToArray", "expect_from_linq": "x + 42"},
    {"name": "times3_5_approx", "src": f"{C}:505-522", "dtype": "float32", "input": {"range": [0, 9999]},
     "ops": [["Select", "x => x * 3.5f"]], "terminal": "ToArray", "expect_from_linq": "x * 3.5", "abs_tol": 0.0001},
    {"name": "complex_expression_approx", "src": f"{C}:524-541", "dtype": "float32", "input": {"range": [1, 10000]},
     "ops": [["Select", "x => (x * 2.0f + 10.0f) / x"]], "terminal": "ToArray", "expect_from_linq": "(x * 2 + 10) / x", "abs_tol": 0.001},
    {"name": "edge_values_times2", "src": f"{C}:563-581", "dtype": "float32",
     "input": [0.0, -1.0, 1.0, 1.7014117331926443e38, -1.7014117331926443e38],
     "ops": [["Select", "x => x * 2.0f"]], "terminal": "ToArray", "expect_from_linq": "x * 2", "rel_tol": 0.0001},
    {"name": "mul2add1_1000", "src": f"{C}:544-561", "dtype": "float32", "input": {"range": [0, 999]},
     "ops": [["Select", "x => x * 2.0f + 1.0f"]], "terminal": "ToArray", "expect_from_linq": "x * 2 + 1"},
    {"name": "mul2add1_10000", "src": f"{C}:544-561", "dtype": "float32", "input": {"range": [0, 9999]},
     "ops": [["Select", "x => x * 2.0f + 1.0f"]], "terminal": "ToArray", "expect_from_linq": "x * 2 + 1"},
    {"name": "mul2add1_50000", "src": f"{C}:544-561", "dtype": "float32", "input": {"range": [0, 49999]},
     "ops": [["Select", "x => x * 2.0f + 1.0f"]], "terminal": "ToArray", "expect_from_linq": "x * 2 + 1"},
]

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(out, "w") as f:
        json.dump(FIX, f, indent=1)
    print(out, len(FIX))
