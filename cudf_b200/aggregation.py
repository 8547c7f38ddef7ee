"""Aggregation descriptors, mirroring the factories of pylibcudf.aggregation / cudf::make_*_aggregation
(cpp/include/cudf/aggregation.hpp:262-322)."""
from __future__ import annotations

from dataclasses import dataclass

from .types import Kind, NullPolicy


@dataclass(frozen=True)
class Aggregation:
    kind: Kind
    ddof: int = 1


def sum() -> Aggregation:  # noqa: A001 - mirrors the reference's name
    return Aggregation(Kind.SUM)


def sum_overflow() -> Aggregation:
    """cudf::make_sum_overflow_aggregation (cpp/include/cudf/aggregation.hpp:214-217): a struct
    {sum in the source type, overflow flag} per group; signed integers and decimals only."""
    return Aggregation(Kind.SUM_OVERFLOW)


def product() -> Aggregation:
    return Aggregation(Kind.PRODUCT)


def min() -> Aggregation:  # noqa: A001
    return Aggregation(Kind.MIN)


def max() -> Aggregation:  # noqa: A001
    return Aggregation(Kind.MAX)


def count(null_handling: NullPolicy = NullPolicy.EXCLUDE) -> Aggregation:
    """COUNT_VALID for EXCLUDE, COUNT_ALL for INCLUDE (cpp/include/cudf/aggregation.hpp:275-280)."""
    return Aggregation(Kind.COUNT_VALID if null_handling == NullPolicy.EXCLUDE else Kind.COUNT_ALL)


def sum_of_squares() -> Aggregation:
    return Aggregation(Kind.SUM_OF_SQUARES)


def mean() -> Aggregation:
    return Aggregation(Kind.MEAN)


def m2() -> Aggregation:
    return Aggregation(Kind.M2)


def variance(ddof: int = 1) -> Aggregation:
    return Aggregation(Kind.VARIANCE, ddof)


def std(ddof: int = 1) -> Aggregation:
    return Aggregation(Kind.STD, ddof)


def argmax() -> Aggregation:
    """Row index of the largest valid value of every group (the first such row on ties)."""
    return Aggregation(Kind.ARGMAX)


def argmin() -> Aggregation:
    """Row index of the smallest valid value of every group (the first such row on ties)."""
    return Aggregation(Kind.ARGMIN)


def median() -> Aggregation:
    """Served by the reference's sort path only; this engine reports it as unsupported."""
    return Aggregation(Kind.MEDIAN)


def nth_element(n: int = 0) -> Aggregation:
    """Served by the reference's sort path only; this engine reports it as unsupported."""
    return Aggregation(Kind.NTH_ELEMENT)
