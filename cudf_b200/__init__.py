"""cudf_b200 — B200-native hash groupby-aggregate engine behind the reference's groupby API.

Public surface (mirrors pylibcudf.groupby / pylibcudf.aggregation for this one path):
    Column, Table, GroupBy, GroupByRequest, GroupByState, StreamingGroupBy, aggregation, TypeId, Kind, NullPolicy
The compute path is the CUDA library cudf_b200/libb2groupby.so (C ABI: include/b2_groupby.h).
"""
from .types import HostColumn, Kind, NullPolicy, TypeId  # noqa: F401


def __getattr__(name):
    # torch-dependent modules load lazily so that the type tables import without torch
    if name in ("Column", "Table"):
        from . import column
        return getattr(column, name)
    if name in ("GroupBy", "GroupByRequest", "GroupByState", "last_call_stats", "LogicError", "DataTypeError",
                "UnsupportedError", "CudaError"):
        from . import groupby
        return getattr(groupby, name)
    if name in ("StreamingGroupBy", "StreamingAggregationRequest"):
        from . import streaming
        return getattr(streaming, name)
    if name == "aggregation":
        import importlib
        return importlib.import_module(".aggregation", __name__)
    raise AttributeError(name)
