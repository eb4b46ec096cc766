"""Generates tests/golden/*.json from the reference's own C++ test tables.

The reference cannot be built or imported in this environment (its Legate dependency is
absent), so its golden vectors are taken from its test sources *as data*: this script reads
``tests/cpp/integration/test_sort.cc`` and ``test_argsort.cc`` of a reference checkout as text,
extracts the input arrays, shapes and expected-result tables, and writes them as JSON.  It copies
no code.  Run:  python tests/golden/make_golden.py /path/to/reference
"""
from __future__ import annotations

import json
import os
import re
import sys


def _table(src: str, func: str):
    """Returns the nested initializer of ``expect_result`` inside ``auto <func>()``."""
    start = src.index("auto " + func + "()")
    eq = src.index("expect_result = {", start) + len("expect_result = ")
    end = src.index("};", eq) + 1
    text = src[eq:end]
    text = re.sub(r"legate::Complex<float>\(([^,()]+),\s*([^()]+?)\)", r"[\1, \2]", text)
    text = text.replace("{", "[").replace("}", "]")
    table = json.loads(text)
    # per shape: list of [axis, values] -> {axis: values}
    return [{str(ax): vals for ax, vals in shape} for shape in table]


def _array(src: str, anchor: str, nth: int = 0):
    """Returns the brace initializer following the nth occurrence of ``anchor``."""
    pos = -1
    for _ in range(nth + 1):
        pos = src.index(anchor, pos + 1)
    eq = src.index("= {", pos) + 2
    depth, i = 0, eq
    while True:
        if src[i] == "{":
            depth += 1
        elif src[i] == "}":
            depth -= 1
            if depth == 0:
                break
        i += 1
    text = src[eq:i + 1]
    text = re.sub(r"legate::Complex<float>\(([^,()]+),\s*([^()]+?)\)", r"[\1, \2]", text)
    return json.loads(text.replace("{", "[").replace("}", "]"))


def main(ref: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    sort_cc = open(os.path.join(ref, "tests/cpp/integration/test_sort.cc")).read()
    arg_cc = open(os.path.join(ref, "tests/cpp/integration/test_argsort.cc")).read()

    body = sort_cc[sort_cc.index("void sort_basic_axis()"):]
    sort_golden = {
        "source": "tests/cpp/integration/test_sort.cc:26-96,98-492,541-572",
        "shapes": _array(body, "test_shapes"),
        "int32": {"input": _array(body, "in_array1"), "expect": _table(sort_cc, "get_expect_result_int")},
        "float64": {"input": _array(body, "in_array2"), "expect": _table(sort_cc, "get_expect_result_double")},
        "complex64": {"input": _array(body, "in_array3"), "expect": _table(sort_cc, "get_expect_result_complex")},
        "empty_shapes": _array(sort_cc[sort_cc.index("void sort_empty_array()"):], "test_shapes"),
        "single_shapes": _array(sort_cc[sort_cc.index("void sort_single_item_array()"):], "test_shapes"),
    }
    with open(os.path.join(here, "sort_cc.json"), "w") as f:
        json.dump(sort_golden, f, indent=1)

    basic = arg_cc[arg_cc.index("void argsort_basic_axis()"):]
    stable = arg_cc[arg_cc.index("void argsort_basic_axis_stable()"):]
    maxdim = arg_cc[arg_cc.index("void argsort_basic_axis_max_dim()"):]
    arg_golden = {
        "source": "tests/cpp/integration/test_argsort.cc:26-204,282-410",
        "shapes": _array(basic, "test_shapes"),
        "expect": _table(arg_cc, "get_argsort_expect_result"),
        "basic": {"int32": _array(basic, "in_array1"), "float64": _array(basic, "in_array2"),
                  "complex64": _array(basic, "in_array3")},
        # inputs with duplicates that must reproduce the same table under a stable sort
        "stable": {"int32": _array(stable, "in_array1"), "float64": _array(stable, "in_array2"),
                   "complex64": _array(stable, "in_array3")},
        "maxdim": {"input": _array(maxdim, "in_array ="), "cases": []},
        # argsort_large_array: descending input of 10000 elements, expected indices count-1-j
        "large": {"count": 10000, "int32": "count - i", "float64": "count * 1.1 - i",
                  "expect": "count - 1 - j"},
    }
    for d in (4, 5, 6, 7):
        arg_golden["maxdim"]["cases"].append({
            "shapes": _array(maxdim, f"test_shapes_{d}d"),
            "expect": _table(arg_cc, f"get_argsort_expect_result_{d}d")})
    with open(os.path.join(here, "argsort_cc.json"), "w") as f:
        json.dump(arg_golden, f, indent=1)
    print("wrote sort_cc.json, argsort_cc.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference/checkout")
    main(sys.argv[1])
