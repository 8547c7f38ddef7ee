"""Writes tests/golden/reference_known_answers.json.

The cases are the known-answer vectors of the reference's own groupby unit tests
(NVIDIA/cudf, cpp/tests/groupby/*.cpp), transcribed by reading those test files: the literal
input columns, the null policy, the aggregation and the expected (key-sorted) output.  ``ref``
gives the test file and line each case comes from.  ``None`` stands for a null element.
A case with ``value_types`` is a TYPED_TEST: it is run once per listed value type, the
expected values cast to the aggregation's result type for that source type.

Run:  python tests/golden/make_known_answers.py
"""
import json
import math
import os

INF = "inf"
NINF = "-inf"
NAN = "nan"

K10 = [1, 2, 3, 1, 2, 2, 1, 3, 3, 2]
V10 = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9]
# keys {1,2,3,1,2,2,1,3,3,2,4} with row 7 null
K11N = [1, 2, 3, 1, 2, 2, 1, None, 3, 2, 4]


def nulls(vals, valid):
    return [v if ok else None for v, ok in zip(vals, valid)]


V11_A = nulls([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 4], [0, 1, 1, 1, 1, 0, 1, 1, 1, 1, 0])
V11_B = nulls([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 3], [0, 1, 1, 1, 1, 0, 1, 1, 1, 1, 1])
V11_C = nulls([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 4], [1, 1, 1, 1, 1, 1, 0, 1, 1, 0, 0])
V11_D = nulls([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 3], [0, 1, 1, 1, 1, 0, 1, 1, 1, 1, 0])

NUMERIC = ["INT8", "INT16", "INT32", "INT64", "FLOAT32", "FLOAT64"]
ALL_FIXED = NUMERIC + ["UINT8", "UINT16", "UINT32", "UINT64"]

cases = []


def case(name, ref, keys, vals, agg, expect_keys, expect_vals, value_types=None, key_type="INT32",
         null_policy="EXCLUDE", ddof=1, value_type=None, scale=0, expect_overflow=None):
    c = dict(name=name, ref=ref, key_type=key_type, keys=keys, vals=vals, agg=agg, ddof=ddof,
             null_policy=null_policy, expect_keys=expect_keys, expect_vals=expect_vals,
             value_types=value_types or [value_type or "INT32"], scale=scale)
    if expect_overflow is not None:
        # SUM_OVERFLOW: the struct's children are expect_vals (None = null struct, "?" = a sum the test does
        # not look at) and these flags
        c["expect_overflow"] = expect_overflow
    cases.append(c)


def family(agg, file, lines, basic, nullcase, nullvals, value_types, zero_valid_values=None):
    """The five-case pattern every per-aggregation test file repeats."""
    case(f"{agg}.basic", f"{file}:{lines[0]}", K10, V10, agg, [1, 2, 3], basic, value_types)
    case(f"{agg}.empty_cols", f"{file}:{lines[1]}", [], [], agg, [], [], value_types)
    case(f"{agg}.zero_valid_keys", f"{file}:{lines[2]}", [None, None, None], [3, 4, 5], agg, [], [], value_types)
    case(f"{agg}.zero_valid_values", f"{file}:{lines[3]}", [1, 1, 1], [None, None, None], agg, [1],
         [None] if zero_valid_values is None else zero_valid_values, value_types)
    case(f"{agg}.null_keys_and_values", f"{file}:{lines[4]}", K11N, nullvals, agg, [1, 2, 3, 4], nullcase, value_types)


family("SUM", "cpp/tests/groupby/sum_tests.cpp", [68, 82, 96, 110, 124], [9, 19, 17], [9, 14, 10, None], V11_A, NUMERIC)
case("SUM.overflow_integer", "cpp/tests/groupby/sum_tests.cpp:167", [0, 0], [-2147483648, -2147483648], "SUM",
     [0], [-4294967296], value_type="INT32")
family("COUNT_VALID", "cpp/tests/groupby/count_tests.cpp", [21, 42, 60, 81, 103], [3, 4, 3], [2, 3, 2, 0], V11_A,
       ALL_FIXED, zero_valid_values=[0])
case("COUNT_ALL.basic", "cpp/tests/groupby/count_tests.cpp:37", K10, V10, "COUNT_ALL", [1, 2, 3], [3, 4, 3], ALL_FIXED)
case("COUNT_ALL.zero_valid_values", "cpp/tests/groupby/count_tests.cpp:98", [1, 1, 1], [None, None, None],
     "COUNT_ALL", [1], [3], ALL_FIXED)
case("COUNT_ALL.null_keys_and_values", "cpp/tests/groupby/count_tests.cpp:128", K11N, V11_A, "COUNT_ALL",
     [1, 2, 3, 4], [3, 4, 2, 1], ALL_FIXED)
# ARGMIN / ARGMAX: the row index of the extreme value (values are distinct in the reference's vectors)
V10_DESC = [9, 8, 7, 6, 5, 4, 3, 2, 1, 0]
ARG_TYPES = ["INT8", "INT16", "INT32", "INT64", "FLOAT32", "FLOAT64", "UINT8", "UINT16", "UINT32", "UINT64"]
case("ARGMIN.basic", "cpp/tests/groupby/argmin_tests.cpp:23", K10, V10_DESC, "ARGMIN", [1, 2, 3], [6, 9, 8], ARG_TYPES)
case("ARGMIN.zero_valid_keys", "cpp/tests/groupby/argmin_tests.cpp:43", [None, None, None], [3, 4, 5], "ARGMIN", [], [], ARG_TYPES)
case("ARGMIN.zero_valid_values", "cpp/tests/groupby/argmin_tests.cpp:63", [1, 1, 1], [None, None, None], "ARGMIN", [1], [None], ARG_TYPES)
case("ARGMIN.null_keys_and_values", "cpp/tests/groupby/argmin_tests.cpp:83", K11N,
     nulls([9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 4], [1, 1, 1, 1, 1, 0, 0, 1, 1, 1, 0]), "ARGMIN", [1, 2, 3, 4], [3, 9, 8, None], ARG_TYPES)
case("ARGMAX.basic", "cpp/tests/groupby/argmax_tests.cpp:22", K10, V10_DESC, "ARGMAX", [1, 2, 3], [0, 1, 2], ARG_TYPES)
case("ARGMAX.zero_valid_keys", "cpp/tests/groupby/argmax_tests.cpp:42", [None, None, None], [3, 4, 5], "ARGMAX", [], [], ARG_TYPES)
case("ARGMAX.zero_valid_values", "cpp/tests/groupby/argmax_tests.cpp:62", [1, 1, 1], [None, None, None], "ARGMAX", [1], [None], ARG_TYPES)
case("ARGMAX.null_keys_and_values", "cpp/tests/groupby/argmax_tests.cpp:82",
     [1, 2, None, 1, 2, 2, 1, 3, 3, 2, 4], nulls([9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 4], [0, 0, 1, 1, 1, 1, 1, 1, 1, 1, 0]),
     "ARGMAX", [1, 2, 3, 4], [3, 4, 7, None], ARG_TYPES)
STR10 = ["año", "bit", "₹1", "aaa", "zit", "bat", "aab", "$1", "€1", "wut"]
case("ARGMIN.string_basic", "cpp/tests/groupby/argmin_tests.cpp:111", K10, STR10, "ARGMIN", [1, 2, 3], [3, 5, 7], value_type="STRING")
case("ARGMIN.string_zero_valid_values", "cpp/tests/groupby/argmin_tests.cpp:129", [1, 1, 1], [None, None, None], "ARGMIN",
     [1], [None], value_type="STRING")
case("ARGMAX.string_basic", "cpp/tests/groupby/argmax_tests.cpp:110", K10, STR10, "ARGMAX", [1, 2, 3], [0, 4, 2], value_type="STRING")
case("ARGMAX.string_zero_valid_values", "cpp/tests/groupby/argmax_tests.cpp:128", [1, 1, 1], [None, None, None], "ARGMAX",
     [1], [None], value_type="STRING")
# MIN / MAX of strings (ARGMIN / ARGMAX + gather in the hash path)
STR10B = ["año", "bit", "₹1", "aaa", "zit", "bat", "aaa", "$1", "₹1", "wut"]
case("MIN.string_basic", "cpp/tests/groupby/min_tests.cpp:123", K10, STR10B, "MIN", [1, 2, 3], ["aaa", "bat", "$1"], value_type="STRING")
case("MIN.string_zero_valid_values", "cpp/tests/groupby/min_tests.cpp:139", [1, 1, 1], [None, None, None], "MIN", [1], [None],
     value_type="STRING")
case("MAX.string_basic", "cpp/tests/groupby/max_tests.cpp:127", K10, STR10B, "MAX", [1, 2, 3], ["año", "zit", "₹1"], value_type="STRING")
case("MAX.string_zero_valid_values", "cpp/tests/groupby/max_tests.cpp:143", [1, 1, 1], [None, None, None], "MAX", [1], [None],
     value_type="STRING")
family("MEAN", "cpp/tests/groupby/mean_tests.cpp", [37, 57, 72, 87, 102], [3.0, 19.0 / 4, 17.0 / 3],
       [4.5, 14.0 / 3, 5.0, None], V11_A, NUMERIC)
family("VARIANCE", "cpp/tests/groupby/var_tests.cpp", [24, 44, 60, 76, 92], [9.0, 131.0 / 12, 31.0 / 3],
       [4.5, 49.0 / 3, 18.0, None], V11_B, NUMERIC)
case("VARIANCE.ddof_non_default", "cpp/tests/groupby/var_tests.cpp:115", K11N, V11_B, "VARIANCE", [1, 2, 3, 4],
     [None, 98.0 / 3, None, None], NUMERIC, ddof=2)
family("STD", "cpp/tests/groupby/std_tests.cpp", [24, 44, 60, 76, 92],
       [3.0, math.sqrt(131.0 / 12), math.sqrt(31.0 / 3)],
       [3 / math.sqrt(2), 7 / math.sqrt(3), 3 * math.sqrt(2), None], V11_B, NUMERIC)
case("STD.ddof_non_default", "cpp/tests/groupby/std_tests.cpp:114", K11N, V11_B, "STD", [1, 2, 3, 4],
     [None, 7 * math.sqrt(2.0 / 3), None, None], NUMERIC, ddof=2)
family("MIN", "cpp/tests/groupby/min_tests.cpp", [26, 44, 62, 80, 98], [0, 1, 2], [3, 1, 2, None], V11_A, ALL_FIXED)
family("MAX", "cpp/tests/groupby/max_tests.cpp", [30, 48, 66, 84, 102], [6, 9, 8], [3, 5, 8, None], V11_C, ALL_FIXED)
case("MIN.values_with_infinity", "cpp/tests/groupby/min_tests.cpp:497", [1, 2, 1, 2], [1, 1, NINF, 2], "MIN",
     [1, 2], [NINF, 1], ["FLOAT32", "FLOAT64"])
case("MAX.values_with_infinity", "cpp/tests/groupby/max_tests.cpp:505", [1, 2, 1, 2], [1, 1, INF, 2], "MAX",
     [1, 2], [INF, 2], ["FLOAT32", "FLOAT64"])
family("SUM_OF_SQUARES", "cpp/tests/groupby/sum_of_squares_tests.cpp", [26, 44, 60, 76, 92], [45, 123, 117],
       [45, 98, 68, None], V11_D, NUMERIC)
family("PRODUCT", "cpp/tests/groupby/product_tests.cpp", [24, 47, 66, 85, 104], [0, 180, 112],
       [18, 36, 16, None], V11_D, NUMERIC)

# fixed point values on the hash path: the representation is aggregated, type and scale are kept
# (TYPED over decimal32/64/128 and scales 2..-2 in the reference; of the 128-bit instances the SUM runs on the
# reference's hash path, cpp/src/groupby/hash/groupby.cu:82-85, MIN and MAX on its sort path)
DECIMALS = ["DECIMAL32", "DECIMAL64"]
for sc in (2, 1, 0, -1, -2):
    case(f"SUM.decimal_hash[scale={sc}]", "cpp/tests/groupby/sum_tests.cpp:220", K10, V10, "SUM", [1, 2, 3],
         [9, 19, 17], DECIMALS + ["DECIMAL128"], scale=sc)
    case(f"MIN.decimal_hash[scale={sc}]", "cpp/tests/groupby/min_tests.cpp:271", K10, V10, "MIN", [1, 2, 3],
         [0, 1, 2], DECIMALS, scale=sc)
    case(f"MAX.decimal_hash[scale={sc}]", "cpp/tests/groupby/max_tests.cpp:279", K10, V10, "MAX", [1, 2, 3],
         [6, 9, 8], DECIMALS, scale=sc)

# M2: cpp/tests/groupby/m2_tests.cpp (keys are typed like the values there; int32 keys here, the
# key type is covered by the KEYS cases)
case("M2.AllNullValuesInput", "cpp/tests/groupby/m2_tests.cpp:107", [1, 2, 3], [None, None, None], "M2",
     [1, 2, 3], [0.0, 0.0, 0.0], NUMERIC)
case("M2.SimpleInput", "cpp/tests/groupby/m2_tests.cpp:122", K10, V10, "M2", [1, 2, 3],
     [18.0, 32.75, 20.0 + 2.0 / 3.0], NUMERIC)
case("M2.SimpleInputHavingNegativeValues", "cpp/tests/groupby/m2_tests.cpp:141", K10,
     [0, 1, -2, 3, -4, -5, -6, 7, -8, 9], "M2", [1, 2, 3], [42.0, 122.75, 114.0], NUMERIC)
case("M2.ValuesHaveNulls", "cpp/tests/groupby/m2_tests.cpp:160", [1, 2, 3, 4, 5, 2, 3, 2],
     [0, None, 2, 3, None, 5, 6, 7], "M2", [1, 2, 3, 4, 5], [0.0, 2.0, 8.0, 0.0, 0.0], NUMERIC)
case("M2.KeysAndValuesHaveNulls", "cpp/tests/groupby/m2_tests.cpp:176", K11N,
     [None, 1, 2, 3, 4, None, 6, 7, 8, 9, None], "M2", [1, 2, 3, 4], [4.5, 32.0 + 2.0 / 3.0, 18.0, 0.0], NUMERIC)
case("M2.InputHaveNullsAndNaNs", "cpp/tests/groupby/m2_tests.cpp:196",
     [4, 3, 1, 2, 3, 1, 2, 2, 1, None, 3, 2, 4, 4],
     [None, None, 0.0, 1.0, 2.0, 3.0, 4.0, NAN, 6.0, 7.0, 8.0, 9.0, 10.0, NAN], "M2", [1, 2, 3, 4],
     [18.0, NAN, 18.0, NAN], value_type="FLOAT64")

# keys: cpp/tests/groupby/keys_tests.cpp (TYPED over key types)
KEY_TYPES = ["INT8", "INT16", "INT32", "INT64", "FLOAT32", "FLOAT64"]
for kt in KEY_TYPES:
    case(f"KEYS.basic[{kt}]", "cpp/tests/groupby/keys_tests.cpp:25", K10, V10, "COUNT_VALID", [1, 2, 3], [3, 4, 3],
         key_type=kt)
    case(f"KEYS.zero_valid_keys[{kt}]", "cpp/tests/groupby/keys_tests.cpp:43", [None, None, None], [3, 4, 5],
         "COUNT_VALID", [], [], key_type=kt)
    case(f"KEYS.some_null_keys[{kt}]", "cpp/tests/groupby/keys_tests.cpp:61", K11N,
         [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 4], "COUNT_VALID", [1, 2, 3, 4], [3, 4, 2, 1], key_type=kt)
    case(f"KEYS.include_null_keys[{kt}]", "cpp/tests/groupby/keys_tests.cpp:82", K11N,
         [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 4], "SUM", [1, 2, 3, 4, None], [9, 19, 10, 4, 7], key_type=kt,
         null_policy="INCLUDE")
case("KEYS.string_basic", "cpp/tests/groupby/keys_tests.cpp:306",
     ["aaa", "año", "₹1", "aaa", "año", "año", "aaa", "₹1", "₹1", "año"], V10, "SUM",
     ["aaa", "año", "₹1"], [9, 19, 17], key_type="STRING")
case("COUNT_VALID.string_values", "cpp/tests/groupby/count_tests.cpp:134", [1, 3, 3, 5, 5, 0],
     ["1", "1", "1", "1", "1", "1"], "COUNT_VALID", [0, 1, 3, 5], [1, 1, 2, 2], value_type="STRING")

# SUM_OVERFLOW: a struct {sum in the source type, overflow flag} per group
SOVF = "cpp/tests/groupby/sum_overflow_tests.cpp"
SOVF_TYPES = ["INT8", "INT16", "INT32", "INT64", "DECIMAL32", "DECIMAL64", "DECIMAL128"]
case("SUM_OVERFLOW.basic", f"{SOVF}:42", K10, V10, "SUM_OVERFLOW", [1, 2, 3], [9, 19, 17], SOVF_TYPES,
     expect_overflow=[False, False, False])
case("SUM_OVERFLOW.empty_cols", f"{SOVF}:145", [], [], "SUM_OVERFLOW", [], [], SOVF_TYPES, expect_overflow=[])
case("SUM_OVERFLOW.zero_valid_keys", f"{SOVF}:167", [None, None, None], [3, 4, 5], "SUM_OVERFLOW", [], [], SOVF_TYPES,
     expect_overflow=[])
case("SUM_OVERFLOW.zero_valid_values", f"{SOVF}:190", [1, 1, 1], [None, None, None], "SUM_OVERFLOW", [1], [None],
     SOVF_TYPES, expect_overflow=[False])
case("SUM_OVERFLOW.null_keys_and_values", f"{SOVF}:222", K11N, V11_A, "SUM_OVERFLOW", [1, 2, 3, 4], [9, 14, 10, None],
     SOVF_TYPES, expect_overflow=[False, False, False, False])
for vt, bits in (("INT8", 8), ("INT16", 16), ("INT32", 32), ("INT64", 64), ("DECIMAL32", 32), ("DECIMAL64", 64),
                 ("DECIMAL128", 128)):
    # type_max - 5, + 10 (group 1); type_max - 5 twice (group 3); type_min + 5, - 10 (group 4): only the flags
    # are compared there
    mx, mn = 2 ** (bits - 1) - 1, -(2 ** (bits - 1))
    case(f"SUM_OVERFLOW.overflow_detection[{vt}]", f"{SOVF}:260", [1, 2, 3, 4, 1, 2, 2, 1, 3, 3, 2, 4, 4],
         [mx - 5, 10, 20, mn + 5, 10, 20, 30, mx - 5, mx - 5, 1, 40, -10, mn + 5], "SUM_OVERFLOW", [1, 2, 3, 4],
         ["?", 100, "?", "?"], value_type=vt, expect_overflow=[True, False, True, True])

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_known_answers.json")
with open(out, "w", encoding="utf-8") as f:
    json.dump(dict(source="NVIDIA/cudf cpp/tests/groupby (version 26.10.00)", cases=cases), f, indent=1,
              ensure_ascii=False)
print(f"{len(cases)} cases -> {out}")
