"""Writes tests/golden/reference_streaming_cases.json.

The cases are the literal batches of the reference's streaming_groupby unit tests
(NVIDIA/cudf, cpp/tests/groupby/streaming_groupby_test.cpp), transcribed by reading that file:
the batch tables, the requests, the null policy, which worker sees which batch (merge tests) and,
where the test states one, the expected key-sorted output.  Most of those tests compare against a
one-shot groupby over the concatenated batches (``verify_against_groupby``); cases without
``expect`` carry that rule.  ``None`` stands for a null element.  ``ref`` = file:line.

Run:  python tests/golden/make_streaming_cases.py
"""
import json
import os

F = "cpp/tests/groupby/streaming_groupby_test.cpp"
NUMERIC = ["INT8", "INT16", "INT32", "INT64", "FLOAT32", "FLOAT64"]
DURATIONS = ["DURATION_DAYS", "DURATION_SECONDS", "DURATION_MILLISECONDS", "DURATION_MICROSECONDS",
             "DURATION_NANOSECONDS"]
cases = []


def case(name, line, batches, requests, value_types=("INT32",), key_types=("INT32",), policy="EXCLUDE",
         workers=None, finalize_after=(), expect=None, max_keys=1024, typed=None):
    """batches: list of batches, each a list of columns (keys first, then value columns)."""
    cases.append(dict(name=name, ref=f"{F}:{line}", key_types=list(key_types), value_types=list(value_types),
                      batches=batches, requests=[list(r) for r in requests], null_policy=policy,
                      workers=workers, finalize_after=list(finalize_after), expect=expect, max_keys=max_keys,
                      typed=typed))


def nulls(vals, valid):
    return [v if ok else None for v, ok in zip(vals, valid)]


SUM1 = [(1, "SUM", 1)]
case("SumTwoBatches", 152, [[[1, 2, 3, 1], [10, 20, 30, 40]], [[2, 3, 1, 4], [5, 15, 25, 35]]], SUM1)
case("MinMaxTwoBatches", 176, [[[1, 2, 1], [5.0, 2.0, 8.0]], [[1, 2, 3], [3.0, 9.0, 1.0]]],
     [(1, "MIN", 1), (1, "MAX", 1)], ["FLOAT64"])
case("CountValidTwoBatches", 202, [[[1, 2, 1, 2], nulls([10, 20, 30, 40], [1, 0, 1, 1])],
                                   [[1, 2], nulls([50, 60], [0, 1])]], [(1, "COUNT_VALID", 1)])
case("MeanTwoBatches", 227, [[[1, 2, 1], [10.0, 20.0, 30.0]], [[1, 2], [50.0, 40.0]]], [(1, "MEAN", 1)], ["FLOAT64"])
case("ProductTwoBatches", 251, [[[1, 2], [3, 5]], [[1, 2], [4, 2]]], [(1, "PRODUCT", 1)])
case("MaxMinOnIntegers", 275, [[[1, 2], [0, 1]], [[1, 2], [1, 1]]], [(1, "MAX", 1), (1, "MIN", 1)])
case("MergeTwoObjects", 300, [[[1, 2, 1], [10, 20, 30]], [[2, 3], [40, 50]]], SUM1, workers=[0, 1],
     expect=dict(keys=[[1, 2, 3]], vals=[[40, 60, 50]]))
case("EmptyBatch", 328, [[[], []], [[1, 2], [10, 20]]], SUM1, expect=dict(keys=[[1, 2]], vals=[[10, 20]]))
case("SingleBatch", 352, [[[1, 2, 1, 3, 2], [10, 20, 30, 40, 50]]], SUM1)
case("NewKeysInLaterBatches", 371, [[[1, 2], [10, 20]], [[3, 4], [30, 40]], [[1, 4], [50, 60]]], SUM1)
case("MultipleRequestsOnDifferentColumns", 400,
     [[[1, 2, 1], [10, 20, 30], [1.0, 2.0, 3.0]], [[2, 1], [40, 50], [4.0, 5.0]]],
     [(1, "SUM", 1), (2, "MIN", 1)], ["INT32", "FLOAT64"])
case("FinalizeDoesNotModifyState", 427, [[[1, 2], [10, 20]], [[1], [30]]], SUM1, finalize_after=[0],
     expect=dict(keys=[[1, 2]], vals=[[40, 20]]))
case("NullKeysExcluded", 456, [[nulls([1, 2, 3], [1, 0, 1]), [10, 20, 30]], [nulls([1, 2], [1, 0]), [40, 50]]], SUM1)
case("NullKeysIncluded", 482, [[nulls([1, 2, 3], [1, 0, 1]), [10, 20, 30]], [nulls([1, 2], [1, 0]), [40, 50]]], SUM1,
     policy="INCLUDE", expect=dict(keys=[[None, 1, 3]], vals=[[70, 50, 30]]))
case("AllNullKeysExcluded", 514, [[nulls([1, 2], [0, 0]), [10, 20]]], SUM1, expect=dict(keys=[[]], vals=[[]]))
case("SumTyped.TwoBatches", 542, [[[1, 2, 3, 1, 2, 2, 1, 3, 3, 2], [0, 1, 2, 3, 4, 5, 6, 7, 8, 9]],
                                  [[1, 2, 3], [10, 20, 30]]], SUM1, typed=NUMERIC + DURATIONS)
case("MinTyped.TwoBatches", 575, [[[1, 2, 1], [5, 2, 8]], [[1, 2], [3, 9]]], [(1, "MIN", 1)],
     typed=NUMERIC + DURATIONS)
VB = [[[1, 2, 3, 1, 2], [0, 1, 2, 3, 4]], [[2, 1, 3, 3, 2], [5, 6, 7, 8, 9]]]
case("VarianceBasic", 599, VB, [(1, "VARIANCE", 1)], ["FLOAT64"])
case("StdBasic", 623, VB, [(1, "STD", 1)], ["FLOAT64"])
case("DisjointKeysAcrossBatches", 668, [[[1, 2], [10, 20]], [[3, 4], [30, 40]]], SUM1)
case("AllDuplicateKeysAcrossBatches", 692, [[[1, 2], [10, 20]], [[1, 2], [30, 40]], [[1, 2], [50, 60]]], SUM1)
case("SingleRowBatches", 721, [[[i % 3], [i * 10]] for i in range(10)], SUM1)
case("InternalDuplicatesDoNotCorruptStaging", 750, [[[1, 1, 2, 3], [10, 10, 20, 30]], [[4, 5], [40, 50]]], SUM1)
case("SumAndMeanOnSameColumn", 777, [[[1, 2, 1], [10.0, 20.0, 30.0]], [[2, 1], [40.0, 50.0]]],
     [(1, "SUM", 1), (1, "MEAN", 1)], ["FLOAT64"])
case("ManySmallBatches", 804, [[[b % 8, (b + 1) % 8, (b + 2) % 8, (b + 3) % 8],
                                [b * 10, b * 10 + 1, b * 10 + 2, b * 10 + 3]] for b in range(10)], SUM1, max_keys=40)
case("MergeMeanTwoBatches", 884, [[[1, 2, 1], [10.0, 20.0, 30.0]], [[2, 1, 3], [40.0, 50.0, 60.0]]],
     [(1, "MEAN", 1)], ["FLOAT64"], workers=[0, 1])
case("MergeCountTwoBatches", 912, [[[1, 2, 1, 1], [10, 20, 30, 40]], [[2, 1, 2], [50, 60, 70]]],
     [(1, "COUNT_VALID", 1)], workers=[0, 1])
case("MergeVarianceTwoBatches", 942, VB, [(1, "VARIANCE", 1)], ["FLOAT64"], workers=[0, 1])
case("SumOfSquaresBasic", 969, [[[1, 2, 1], [3.0, 4.0, 5.0]], [[2, 1], [6.0, 7.0]]], [(1, "SUM_OF_SQUARES", 1)],
     ["FLOAT64"])
case("M2Basic", 993, [[[1, 2, 1, 2], [1.0, 2.0, 3.0, 4.0]], [[1, 2], [5.0, 6.0]]], [(1, "M2", 1)], ["FLOAT64"])
case("StdWithNullValues", 1017, [[[1, 2, 1, 2], nulls([1.0, 2.0, 3.0, 4.0], [1, 1, 0, 1])],
                                 [[1, 2, 1], nulls([5.0, 6.0, 7.0], [1, 0, 1])]], [(1, "STD", 1)], ["FLOAT64"])
case("CountAllTwoBatches", 1224, [[[1, 2, 1], nulls([10, 20, 30], [1, 0, 1])], [[2, 1], nulls([40, 50], [0, 1])]],
     [(1, "COUNT_ALL", 1)])
case("MultiColumnKeys", 1248, [[[1, 1, 2], [10, 20, 10], [100, 200, 300]], [[1, 2], [10, 10], [400, 500]]],
     [(2, "SUM", 1)], key_types=["INT32", "INT32"])
case("CumulativeRowsCanExceedMaxDistinctKeys", 1293, [[[0, 1, 2], [10, 20, 30]]] * 5, SUM1, max_keys=3)

# string keys (kept as a table of partial aggregates that is reduced batch by batch)
STR = ["STRING"]
case("StringKeySumTwoBatches", 1043, [[["a", "b", "c", "a"], [10, 20, 30, 40]], [["b", "c", "a", "d"], [5, 15, 25, 35]]],
     SUM1, key_types=STR)
case("StringKeyNonAsciiUtf8", 1066, [[["αλφα", "βητα", "γαμμα", "αλφα"], [10, 20, 30, 40]],
                                     [["βητα", "δελτα", "αλφα", "🙂"], [5, 15, 25, 35]]], SUM1, key_types=STR)
case("StringKeyMinMaxTwoBatches", 1089, [[["cat", "dog", "cat"], [5.0, 2.0, 8.0]], [["cat", "dog", "bird"], [3.0, 9.0, 1.0]]],
     [(1, "MIN", 1), (1, "MAX", 1)], ["FLOAT64"], key_types=STR)
UNIVERSE = ["alpha", "beta", "gamma", "delta"]
case("StringKeyManySmallBatches", 1112, [[[UNIVERSE[b % 4], UNIVERSE[(b + 1) % 4]], [b * 10, b * 10 + 1]] for b in range(8)],
     SUM1, key_types=STR)
case("StringKeyDisjointBatches", 1141, [[["x", "y"], [10, 20]], [["z", "w"], [30, 40]], [["x", "w"], [50, 60]]], SUM1,
     key_types=STR)
case("StringKeyNullKeysExcluded", 1169, [[nulls(["a", "b", "c"], [1, 0, 1]), [10, 20, 30]], [nulls(["a", "b"], [1, 0]), [40, 50]]],
     SUM1, key_types=STR)
case("StringKeyMerge", 1196, [[["a", "b"], [10, 20]], [["b", "c"], [30, 40]]], SUM1, key_types=STR, workers=[0, 1])

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_streaming_cases.json")
with open(out, "w", encoding="utf-8") as f:
    json.dump(dict(source="NVIDIA/cudf " + F, cases=cases), f, indent=1)
print(f"{len(cases)} cases -> {out}")
