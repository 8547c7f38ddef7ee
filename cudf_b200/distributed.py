"""Multi-GPU groupby: one process per GPU, hash partition + all-to-all + local aggregation.

The reference has no NCCL path; its multi-GPU groupby is the cudf-polars streaming executor:
local aggregation, hash shuffle of the PARTIAL aggregates keyed on the group keys, then a reduction
groupby on each owner (python/cudf_polars/cudf_polars/streaming/actor_graph/groupby.py:339-456),
with the shuffle built on cudf::hash_partition (cpp/libcudf_streaming/src/partition_utils.cpp:72-100).
For keys that pack into 64 bits the whole plan is ONE call into the CUDA library per rank
(``b2_groupby_aggregate_multi``: local aggregate, partition of the partial records by owner, NCCL
send / recv on the caller's stream, merge, finalise) over a communicator the library creates from
an id that ``torch.distributed`` broadcasts once per process group (``Communicator``).  For the
other shapes (string / float / wide keys, the rows strategy) the exchange is
``torch.distributed.all_to_all_single`` (NCCL over NVLink/NVSwitch on GPUs, gloo on CPU for tests)
between calls into the library.

Two strategies:
  * ``partials``: aggregate locally, partition the partial records {key, n, Σx, Σx², min, max …} by
    owner = hash(key) % world, exchange, merge, finalise.  Wire bytes ∝ local groups.
  * ``rows``: partition the raw rows by owner, exchange the columns, aggregate locally.  Wire bytes
    ∝ rows; used when almost every row is its own group.
Each rank ends up with the complete results of the groups it owns (disjoint across ranks).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def plan_exchange(send_counts: Sequence[int], recv_counts: Sequence[int], unit_bytes: int):
    """Split sizes (bytes) of a variable all-to-all and the receive offsets (in units)."""
    in_splits = [int(c) * unit_bytes for c in send_counts]
    out_splits = [int(c) * unit_bytes for c in recv_counts]
    recv_offsets = [0]
    for c in recv_counts:
        recv_offsets.append(recv_offsets[-1] + int(c))
    return in_splits, out_splits, recv_offsets


def exchange_counts(send_counts: Sequence[int], device, group=None) -> List[int]:
    """Every rank tells every other rank how many units it will send (the count matrix column)."""
    t = torch.tensor(list(send_counts), dtype=torch.int64, device=device)
    r = torch.empty_like(t)
    dist.all_to_all_single(r, t, group=group)
    return [int(x) for x in r.tolist()]


def exchange_buffer(buf: torch.Tensor, send_counts: Sequence[int], recv_counts: Sequence[int], unit_bytes: int,
                    group=None) -> torch.Tensor:
    """Variable-size all-to-all of a destination-major uint8 buffer; returns the source-major buffer."""
    in_splits, out_splits, _ = plan_exchange(send_counts, recv_counts, unit_bytes)
    buf = buf.contiguous().view(torch.uint8).reshape(-1)
    assert buf.numel() >= sum(in_splits)
    out = torch.empty(max(sum(out_splits), 0), dtype=torch.uint8, device=buf.device)
    dist.all_to_all_single(out, buf[: sum(in_splits)], output_split_sizes=out_splits, input_split_sizes=in_splits,
                           group=group)
    return out


def agree_on_status(ok: bool, device, group=None) -> bool:
    """True iff every rank reports ``ok``.  A rank whose local step failed must still reach the next
    collective, or its peers wait there for ever: it reports the failure here and all ranks raise."""
    t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item()) == 0


def exchange_records(records: torch.Tensor, counts: Sequence[int], record_bytes: int, group=None
                     ) -> Tuple[torch.Tensor, int]:
    """Exchange of packed partial records: returns (received records, number received)."""
    recv_counts = exchange_counts(counts, records.device, group)
    out = exchange_buffer(records, counts, recv_counts, record_bytes, group)
    return out, sum(recv_counts)


class Communicator:
    """``b2_comm``: the NCCL communicator ``b2_groupby_aggregate_multi`` exchanges over, one per
    (process group, device).  Rank 0 draws the NCCL unique id, ``torch.distributed`` broadcasts it."""

    _cache = {}

    def __init__(self, device, group=None):
        import ctypes as C
        from . import _lib
        from .groupby import _check
        lib = _lib.load()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            _check(lib.b2_comm_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        ident = ident.to(device)
        dist.broadcast(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        raw = (C.c_uint8 * 128)(*ident.cpu().tolist())
        handle = C.c_void_p()
        with torch.cuda.device(device):
            _check(lib.b2_comm_create(raw, rank, world, C.byref(handle)))
        self._handle = handle
        self.rank, self.world = rank, world

    @classmethod
    def for_group(cls, device, group=None) -> "Communicator":
        key = (id(group), str(device))
        if key not in cls._cache:
            cls._cache[key] = cls(device, group)
        return cls._cache[key]

    def close(self):
        from . import _lib
        if self._handle:
            _lib.load().b2_comm_destroy(self._handle)
            self._handle = None


class DistributedGroupBy:
    """``GroupBy`` over row-sharded inputs: every rank passes its own rows; every rank receives the
    finished groups it owns."""

    def __init__(self, keys, null_handling=0, *, strategy: str = "partials", group=None, python_exchange: bool = False,
                 **options):
        """``python_exchange`` keeps the partials strategy on ``torch.distributed`` collectives between
        library calls (the only form on CPU/gloo) instead of the single native call."""
        from .groupby import GroupBy
        self._python_exchange = bool(python_exchange)
        if strategy not in ("partials", "rows"):
            raise ValueError("strategy must be 'partials' or 'rows'")
        self._keys = keys
        self._null_handling = null_handling
        self._options = options
        self._strategy = strategy
        self._group = group
        self._gb = GroupBy(keys, null_handling, **options)
        self._chunks_overflowed = False   # the fixed-size exchange overflowed before (same on every rank)
        self._local_groups_hint = 0       # local groups of the previous variable-size call
        self._owned_groups_hint = 0       # groups this rank owned after the previous variable-size call

    def aggregate(self, requests):
        world = dist.get_world_size(self._group) if dist.is_initialized() else 1
        if world == 1:
            return self._gb.aggregate(requests)
        if self._strategy == "partials":
            from .partials import keys_are_row_keyed
            if keys_are_row_keyed(self._keys.columns(), self._null_handling):
                # string / float / wide keys: their table slots reference local rows and cannot travel;
                # the partial aggregates travel as a table instead
                return self._aggregate_partial_table(requests, world)
            if self._keys.columns()[0].data is not None and self._keys.columns()[0].data.is_cuda and not self._python_exchange:
                return self._aggregate_partials_native(requests)
            return self._aggregate_partials(requests, world)
        return self._aggregate_rows(requests, world)

    def _aggregate_partials_native(self, requests):
        """Packed keys on GPUs: the whole plan inside the library (``b2_groupby_aggregate_multi``)."""
        import ctypes as C
        from . import _lib
        from .column import allocator_for
        from .groupby import _adopt_result, _check, _requests_to_c
        lib = _lib.load()
        device = self._gb._device
        comm = Communicator.for_group(device, self._group)
        keep: list = []
        creqs = _requests_to_c(requests, keep)
        alloc = allocator_for(device)
        res = _lib.GroupbyResult()
        stream = torch.cuda.current_stream(device).cuda_stream
        _check(lib.b2_groupby_aggregate_multi(comm._handle, self._gb._handle, creqs, len(requests), C.c_void_p(stream),
                                              C.byref(alloc.struct), C.byref(res)))
        return _adopt_result(res, alloc)

    # records per destination of the fixed-size exchange (one all-to-all, no host round trip)
    CHUNK_RECORDS = 16384

    def _aggregate_partials(self, requests, world):
        from .groupby import GroupByState, LogicError
        st = GroupByState(self._gb, requests)
        # table sizing from the previous call on this object (a stream of similar batches): skips the
        # speculative table and the cardinality estimate; a wrong hint only costs a regrowth
        if self._local_groups_hint > 0 and "expected_groups" not in self._options:
            st.reset(expected_groups=self._local_groups_hint + self._local_groups_hint // 8)
        device = self._keys.columns()[0].data.device
        error = None
        try:
            st.update()
        except Exception as e:   # reported to every rank before anyone enters the exchange
            error = e
        if not agree_on_status(error is None, device, self._group):
            raise error if error is not None else RuntimeError("the local aggregate failed on another rank")
        if not self._chunks_overflowed and st.chunk_bytes(self.CHUNK_RECORDS) * world <= (64 << 20):
            # small states: equal-split all-to-all of fixed chunks; a sender with too many records
            # marks every chunk it sends, so all ranks take the fallback below together — and, having
            # all seen the same flag, all skip the fixed-size attempt on their next calls
            certain = st.num_groups() > world * self.CHUNK_RECORDS  # cannot fit whatever the split
            if certain:
                # still take part in the collective (the other ranks cannot know), with empty flagged chunks
                words = st.chunk_bytes(self.CHUNK_RECORDS) // 8
                flagged = torch.zeros(world * words, dtype=torch.int64, device=self._keys.columns()[0].data.device)
                flagged[1::words] = 1
                send = flagged.view(torch.uint8)
            else:
                send = st.pack_chunks(world, self.CHUNK_RECORDS)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self._group)
            if certain:
                self._chunks_overflowed = True
            else:
                merged = GroupByState(self._gb, requests)
                merged.merge_chunks(recv, world, self.CHUNK_RECORDS)
                try:
                    return merged.finalize()
                except LogicError as e:
                    if "chunk overflow" not in str(e):
                        raise
                    self._chunks_overflowed = True
        records, counts = st.pack(world)
        self._local_groups_hint = int(sum(counts))
        recv, nrecv = exchange_records(records, counts, st.record_bytes, self._group)
        # the merged table is sized from the number of groups this rank owned last time, if known
        # (a too small estimate costs a second merge pass, never a wrong result)
        own = self._owned_groups_hint
        st.reset(expected_groups=max(own + own // 8 if own > 0 else nrecv, 1))
        st.merge(recv, nrecv)
        out = st.finalize()
        self._owned_groups_hint = out[0].num_rows()
        return out

    def _aggregate_partial_table(self, requests, world):
        """Partials strategy for keys that do not pack into 64 bits: local aggregate into a TABLE of partial
        aggregates (keys, n, Σx, Σx², min, max ... per value column), hash partition of that table by key,
        all-to-all of its columns, reduction groupby on the owner, finalisers — the reference's
        multi-partition plan (python/cudf_polars/cudf_polars/streaming/actor_graph/groupby.py:339-456).
        Wire bytes ∝ local groups, as for packed keys."""
        from .column import Table
        from .partials import PartialTable
        from .partition import hash_partition
        specs, sources = [], {}
        for r in requests:
            sources[id(r._values)] = r._values
            specs += [(id(r._values), a.kind, a.ddof) for a in r._aggregations]
        nkeys = self._keys.num_columns()
        local = PartialTable(specs, self._null_handling, batch_options=self._options)
        local.add_batch(self._keys.columns(), sources)
        parts, offsets = hash_partition(Table(local.keys + local.columns()), nkeys, world)
        recv = exchange_rows(parts, offsets, world, self._group)
        local.reduce_rows(recv[:nkeys], recv[nkeys:])
        okeys, flat = local.finalize(detect_nulls=True)
        results, i = [], 0
        for r in requests:
            results.append(Table(flat[i:i + len(r._aggregations)]))
            i += len(r._aggregations)
        return Table(okeys), results

    def _aggregate_rows(self, requests, world):
        from .column import Table
        from .groupby import GroupBy, GroupByRequest
        from .partition import hash_partition
        nkeys = self._keys.num_columns()
        vals, seen = [], {}
        for r in requests:
            if id(r._values) not in seen:
                seen[id(r._values)] = len(vals)
                vals.append(r._values)
        cols = self._keys.columns() + vals
        parts, offsets = hash_partition(Table(cols), nkeys, world)
        new_cols = exchange_rows(parts, offsets, world, self._group)
        gb = GroupBy(Table(new_cols[:nkeys]), self._null_handling, **self._options)
        new_reqs = [GroupByRequest(new_cols[nkeys + seen[id(r._values)]], r._aggregations) for r in requests]
        return gb.aggregate(new_reqs)


def exchange_rows(parts, offsets, world, group=None):
    """All-to-all of a hash-partitioned table (partition p goes to rank p): data as bytes, validity
    as one byte per row (a partition starts at an arbitrary bit of its mask), strings as offsets +
    chars with the received offsets rebased segment by segment.  Returns the received columns."""
    from .column import Column
    from .partition import bytes_to_mask, mask_to_bytes
    from .types import TypeId, type_width
    device = parts.columns()[0].data.device
    send_counts = [offsets[p + 1] - offsets[p] for p in range(world)]
    recv_counts = exchange_counts(send_counts, device, group)
    nrecv = sum(recv_counts)
    out = []
    for c in parts.columns():
        mask, nulls = None, 0
        if c.mask is not None:
            vb = exchange_buffer(mask_to_bytes(c), send_counts, recv_counts, 1, group)
            mask, nulls = bytes_to_mask(vb)
        if c.type_id == TypeId.STRING:
            odt = torch.int64 if c.offsets_type == TypeId.INT64 else torch.int32
            offs = c.offsets.view(odt)[: c.size + 1].to(torch.int64)
            bounds = offs[torch.tensor(offsets, device=device)].tolist()          # char range of every partition
            send_chars = [bounds[p + 1] - bounds[p] for p in range(world)]
            recv_chars = exchange_counts(send_chars, device, group)
            chars = exchange_buffer(c.data if c.data is not None else torch.zeros(0, dtype=torch.uint8, device=device),
                                    send_chars, recv_chars, 1, group)
            roffs = exchange_buffer(offs[: c.size].contiguous().view(torch.uint8), send_counts, recv_counts, 8,
                                    group).view(torch.int64)
            new_offs = torch.empty(nrecv + 1, dtype=torch.int64, device=device)
            row0, char0 = 0, 0
            for s in range(world):                                                   # rebase each sender's segment
                if recv_counts[s]:
                    seg = roffs[row0:row0 + recv_counts[s]]
                    new_offs[row0:row0 + recv_counts[s]] = seg - seg[0] + char0
                row0 += recv_counts[s]
                char0 += recv_chars[s]
            new_offs[nrecv] = char0
            out.append(Column(TypeId.STRING, nrecv, chars, mask, 0, nulls, new_offs.view(torch.uint8), TypeId.INT64))
        else:
            buf = exchange_buffer(c.data, send_counts, recv_counts, type_width(c.type_id), group)
            out.append(Column(c.type_id, nrecv, buf, mask, 0, nulls, None, TypeId.INT32, c.scale))
    return out
