"""Shared helpers of the parity tests: golden-case decoding, key sorting, column comparison."""
from __future__ import annotations

import json
import math
import os
from typing import List, Sequence

import numpy as np

from cudf_b200.types import HostColumn, Kind, NullPolicy, STORAGE_DTYPE, TypeId, is_floating, result_type

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_known_answers.json")

# north_star tolerances: float sum/mean/var within 1e-12 (fp64 sources) or 1e-5 (fp32 sources)
RTOL_F64 = 1e-12
RTOL_F32 = 1e-5


def load_golden() -> list:
    with open(GOLDEN, encoding="utf-8") as f:
        return json.load(f)["cases"]


def _num(x):
    if isinstance(x, str):
        return {"inf": math.inf, "-inf": -math.inf, "nan": math.nan}[x]
    return x


def make_column(values: Sequence, type_name: str, offset: int = 0) -> HostColumn:
    """Column of the named type from a Python list where ``None`` is a null element."""
    t = TypeId[type_name]
    valid = np.array([v is not None for v in values], dtype=bool)
    if t == TypeId.STRING:
        return HostColumn.from_strings(list(values))
    filled = [0 if v is None else _num(v) for v in values]
    arr = np.array(filled, dtype=np.float64 if is_floating(t) else np.int64).astype(STORAGE_DTYPE[t])
    return HostColumn.from_numpy(arr, None if valid.all() and len(values) else (valid if len(values) else None),
                                 type_id=t, offset=offset)


def sort_order(keys: List[HostColumn]) -> np.ndarray:
    """Permutation that sorts the groups by key (nulls first), the way the reference's tests sort
    a result before comparing it (cpp/tests/groupby/groupby_test_util.cpp:83-90)."""
    n = keys[0].size if keys else 0
    if n == 0:
        return np.zeros(0, dtype=np.int64)
    cols = []
    for k in reversed(keys):
        v = k.valid()
        if k.type_id == TypeId.STRING:
            py = k.to_pylist()
            ranks = {s: i for i, s in enumerate(sorted(set(x for x in py if x is not None)))}
            vals = np.array([ranks[x] if x is not None else -1 for x in py], dtype=np.int64)
        else:
            vals = k.values().copy()
            if is_floating(k.type_id):
                vals = np.where(np.isnan(vals), np.inf, vals) + 0.0  # -0 -> +0, NaN last
        vals = np.where(v, vals, vals.dtype.type(0))
        cols.append(vals)
        cols.append(v.astype(np.int8))
    return np.lexsort(cols)


def take(col: HostColumn, order: np.ndarray) -> list:
    py = col.to_pylist()
    return [py[i] for i in order]


def assert_column_equal(got: HostColumn, exp: HostColumn, order_got, order_exp, rtol: float, what: str,
                        check_nullable: bool = False):
    assert TypeId(got.type_id) == TypeId(exp.type_id), f"{what}: type {got.type_id!r} != {exp.type_id!r}"
    assert got.size == exp.size, f"{what}: size {got.size} != {exp.size}"
    if check_nullable:
        assert (got.mask is None) == (exp.mask is None), f"{what}: nullability differs"
    g, e = take(got, order_got), take(exp, order_exp)
    if is_floating(got.type_id):
        for i, (a, b) in enumerate(zip(g, e)):
            if a is None or b is None:
                assert a is None and b is None, f"{what}[{i}]: {a} vs {b}"
            elif math.isnan(b) or math.isnan(a):
                assert math.isnan(a) and math.isnan(b), f"{what}[{i}]: {a} vs {b}"
            elif math.isinf(b) or math.isinf(a):
                assert a == b, f"{what}[{i}]: {a} vs {b}"
            else:
                assert abs(a - b) <= rtol * max(abs(b), abs(a)) + 1e-300, f"{what}[{i}]: {a} vs {b} (rtol {rtol})"
    else:
        assert g == e, f"{what}: {g[:16]} vs {e[:16]}"


def assert_keys_equal(got: List[HostColumn], exp: List[HostColumn], order_got, order_exp):
    assert len(got) == len(exp)
    for i, (a, b) in enumerate(zip(got, exp)):
        assert TypeId(a.type_id) == TypeId(b.type_id)
        ga, gb = take(a, order_got), take(b, order_exp)
        if is_floating(a.type_id):
            # +0 == -0 and NaN == NaN as keys
            norm = lambda x: None if x is None else ("nan" if math.isnan(x) else x + 0.0)
            ga, gb = [norm(x) for x in ga], [norm(x) for x in gb]
        assert ga == gb, f"key column {i}: {ga[:16]} vs {gb[:16]}"


def rtol_for(source_type: int) -> float:
    return RTOL_F32 if TypeId(source_type) == TypeId.FLOAT32 else RTOL_F64


def golden_instances(case: dict):
    """Expands a golden case into (id, keys column, values column, kind, ddof, policy,
    expected keys column, expected values column)."""
    kind = Kind[case["agg"]]
    policy = NullPolicy[case["null_policy"]]
    for vt in case["value_types"]:
        if vt != "STRING" and any(isinstance(v, (int, float)) and v < 0 for v in case["vals"] if v is not None) \
                and vt.startswith("UINT"):
            continue
        keys = make_column(case["keys"], case["key_type"])
        vals = make_column(case["vals"], vt)
        rt = TypeId.INT32 if vt == "STRING" else result_type(TypeId[vt], kind)
        ekeys = make_column(case["expect_keys"], case["key_type"])
        evals = make_column(case["expect_vals"], rt.name)
        yield f'{case["name"]}[{vt}]', keys, vals, kind, case["ddof"], policy, ekeys, evals
