/*
 * b2_groupby.h — C ABI of the B200-native hash groupby-aggregate engine.
 *
 * The library is a drop-in for ONE path of NVIDIA/cudf:
 *     cudf::groupby::groupby(keys, null_policy).aggregate(requests)
 * (reference: cpp/include/cudf/groupby.hpp:54-57 aggregation_request, :81-84
 * aggregation_result, :121-125 constructor, :181-184 aggregate;
 * cpp/src/groupby/groupby.cu:39-50,219-236; hash back end cpp/src/groupby/hash/).
 *
 * Everything crossing this boundary is a plain pointer, an integer or a POD
 * struct.  All `data`, `null_mask` and child pointers are DEVICE pointers on the
 * current CUDA device unless a comment says "host".  Inputs are non-owning views
 * (the caller keeps them alive until the stream work has finished, like
 * cudf::column_view); outputs are owning buffers obtained from the caller's
 * allocator (the stand-in for rmm::device_async_resource_ref).
 *
 * Error model: every entry point returns a b2_status.  The codes map 1:1 onto
 * the exception classes the reference throws (cpp/include/cudf/utilities/error.hpp:35-97);
 * b2_last_error() returns the message of the calling thread's last failure.
 */
#ifndef B2_GROUPBY_H
#define B2_GROUPBY_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
typedef enum b2_status {
  B2_SUCCESS          = 0,
  B2_LOGIC_ERROR      = 1, /* cudf::logic_error      (precondition violated, e.g. size mismatch) */
  B2_INVALID_ARGUMENT = 2, /* std::invalid_argument                                              */
  B2_DATA_TYPE_ERROR  = 3, /* cudf::data_type_error  (a column of a type the call cannot read)    */
  B2_CUDA_ERROR       = 4, /* cudf::cuda_error                                                   */
  B2_UNSUPPORTED      = 5, /* valid for the reference's sort path, not handled by this hash path;
                              an adapter falls through to the reference for these               */
  B2_OUT_OF_MEMORY    = 6, /* std::bad_alloc / rmm::out_of_memory                                */
  B2_INTERNAL_ERROR   = 7
} b2_status;

/* ---- element types: numeric values of cudf::type_id (cpp/include/cudf/types.hpp:185-217).
 *      Served as keys: integers, BOOL8, floats, timestamps, durations, DECIMAL32/64, STRING, and
 *      DICTIONARY32 over any of these (one-shot aggregate; the key column comes back as a dictionary).
 *      Served as values: the same fixed-width types (which aggregation on which type follows
 *      cudf::detail::is_valid_aggregation; DECIMAL32/64: SUM, SUM_OVERFLOW, MIN, MAX, COUNT on the
 *      integer representation, result type and `scale` of the source kept; DECIMAL128 (16-byte
 *      little-endian elements): SUM, SUM_OVERFLOW, COUNT, like the reference's hash path), STRING
 *      values for MIN / MAX / ARGMIN / ARGMAX / COUNT, and DICTIONARY32 values (children {indices,
 *      keys}, keys sorted and unique as cudf::dictionary guarantees; one-shot aggregate only):
 *      fixed-width keys with every aggregation of the keys' type, STRING keys with MIN / MAX (results
 *      are DICTIONARY32 columns over a copy of the keys), ARGMIN / ARGMAX and COUNT.  LIST and STRUCT
 *      values and the other aggregations of DECIMAL128 return B2_UNSUPPORTED. */
typedef enum b2_type_id {
  B2_EMPTY = 0, B2_INT8 = 1, B2_INT16 = 2, B2_INT32 = 3, B2_INT64 = 4,
  B2_UINT8 = 5, B2_UINT16 = 6, B2_UINT32 = 7, B2_UINT64 = 8,
  B2_FLOAT32 = 9, B2_FLOAT64 = 10, B2_BOOL8 = 11,
  B2_TIMESTAMP_DAYS = 12, B2_TIMESTAMP_SECONDS = 13, B2_TIMESTAMP_MILLISECONDS = 14,
  B2_TIMESTAMP_MICROSECONDS = 15, B2_TIMESTAMP_NANOSECONDS = 16,
  B2_DURATION_DAYS = 17, B2_DURATION_SECONDS = 18, B2_DURATION_MILLISECONDS = 19,
  B2_DURATION_MICROSECONDS = 20, B2_DURATION_NANOSECONDS = 21,
  B2_DICTIONARY32 = 22, B2_STRING = 23, B2_LIST = 24,
  B2_DECIMAL32 = 25, B2_DECIMAL64 = 26, B2_DECIMAL128 = 27, B2_STRUCT = 28
} b2_type_id;

/* ---- aggregation kinds: numeric values of cudf::aggregation::Kind
 *      (cpp/include/cudf/aggregation.hpp:78-121).  Only the kinds the reference's
 *      hash path serves are listed (cpp/src/groupby/hash/groupby.cu:63-131). */
typedef enum b2_agg_kind {
  B2_AGG_SUM = 0, B2_AGG_SUM_OVERFLOW = 1, B2_AGG_PRODUCT = 2, B2_AGG_MIN = 3, B2_AGG_MAX = 4,
  B2_AGG_COUNT_VALID = 5, B2_AGG_COUNT_ALL = 6, B2_AGG_SUM_OF_SQUARES = 9,
  B2_AGG_MEAN = 10, B2_AGG_M2 = 11, B2_AGG_VARIANCE = 12, B2_AGG_STD = 13,
  B2_AGG_ARGMAX = 16, B2_AGG_ARGMIN = 17
} b2_agg_kind;

/* cudf::null_policy (cpp/include/cudf/types.hpp:115-118) */
typedef enum b2_null_policy { B2_NULL_EXCLUDE = 0, B2_NULL_INCLUDE = 1 } b2_null_policy;

/* ---- non-owning column view: field-for-field cudf::column_view
 *      (cpp/include/cudf/column/column_view.hpp:236-243 base fields, :469 children).
 *      Element i lives at data[(offset+i)] and its validity bit is bit (offset+i)%32 of
 *      null_mask[(offset+i)/32], 1 = valid (cpp/include/cudf/utilities/bit.hpp:47-104);
 *      null_mask == NULL means all valid.  STRING: data = chars, children[0] = offsets
 *      column of size+1 entries typed INT32 or INT64
 *      (cpp/include/cudf/strings/strings_column_view.hpp:53). */
typedef struct b2_column_view {
  int32_t type_id;                        /* b2_type_id                                */
  int32_t scale;                          /* decimal scale; 0 otherwise                */
  int32_t size;                           /* number of elements (cudf::size_type)      */
  int32_t null_count;                     /* number of nulls, or -1 if unknown         */
  const void* data;                       /* device                                    */
  const uint32_t* null_mask;              /* device; NULL = no nulls                   */
  int32_t offset;                         /* element offset of a sliced view           */
  int32_t num_children;
  const struct b2_column_view* children;  /* host array                                */
} b2_column_view;

/* One aggregation to compute on a values column: stands for
 * std::unique_ptr<cudf::groupby_aggregation> (kind + the one parameter the
 * supported kinds carry: ddof of VARIANCE/STD, cpp/include/cudf/aggregation.hpp:293,305). */
typedef struct b2_aggregation {
  int32_t kind; /* b2_agg_kind                            */
  int32_t ddof; /* VARIANCE / STD only; reference default 1 */
} b2_aggregation;

/* cudf::groupby::aggregation_request (cpp/include/cudf/groupby.hpp:54-57) */
typedef struct b2_aggregation_request {
  b2_column_view values;
  int32_t num_aggregations;
  const b2_aggregation* aggregations; /* host array */
} b2_aggregation_request;

/* ---- allocator: stands for rmm::device_async_resource_ref.  Stream-ordered on
 *      `stream` (a cudaStream_t).  NULL allocator ⇒ the library's own stream-ordered pool. */
typedef struct b2_allocator {
  void* (*allocate)(size_t bytes, void* stream, void* ctx);
  void (*deallocate)(void* ptr, size_t bytes, void* stream, void* ctx);
  void* ctx;
} b2_allocator;

/* ---- owning output column: stands for cudf::column
 *      (cpp/include/cudf/column/column.hpp:37,249-270).  `data`, `null_mask` come from the
 *      allocator passed to the producing call and are released by b2_result_free (or adopted
 *      by the caller, who then sets them to NULL first). */
typedef struct b2_owned_column {
  int32_t type_id;
  int32_t scale;
  int32_t size;
  int32_t null_count;
  void* data;
  size_t data_bytes;
  uint32_t* null_mask; /* NULL when the column is not nullable */
  size_t null_mask_bytes;
  int32_t num_children;
  struct b2_owned_column* children; /* host array (STRING: children[0] = offsets; STRUCT, the result of
                                       SUM_OVERFLOW: children[0] = the sum in the source type, children[1] =
                                       the BOOL8 overflow flag, the null mask on the struct) */
} b2_owned_column;

/* Return value of aggregate: std::pair<std::unique_ptr<table>, std::vector<aggregation_result>>
 * (cpp/include/cudf/groupby.hpp:181-184).  results[r][a] is the column for aggregation a of
 * request r, in request order (groupby.hpp:139-146).  Group order is unspecified (:148-150). */
typedef struct b2_groupby_result {
  int32_t num_groups;
  int32_t num_keys;
  b2_owned_column* keys; /* host array, num_keys */
  int32_t num_requests;
  int32_t* num_results;       /* host array, per request */
  b2_owned_column** results;  /* host array of host arrays */
  b2_allocator allocator;     /* the allocator that owns the device buffers */
  void* stream;
} b2_groupby_result;

/* ---- tuning knobs (the reference keeps these as compile-time constants,
 *      cpp/src/groupby/hash/helpers.cuh:19-40, cpp/include/cudf/detail/cuco_helpers.hpp:16) */
typedef struct b2_groupby_options {
  int64_t expected_groups;  /* hint; <= 0 = unknown (engine speculates, then estimates)        */
  int32_t table_variant;    /* 0 auto; 1 global-memory table only; 2 = auto, but the partitioned
                               path folds no hot keys and keeps fp64 cells (no fixed-point limbs); 3 shared-memory table with
                               hashing only (no dense key box); 4 / 5 = auto, but the lean
                               float-mean kernel reads its tiles through registers (4) or
                               through the cp.async.bulk shared-memory ring (5); 6 = always
                               take the radix-partitioned path when the keys allow it (auto
                               takes it from about half a million groups), 7 = never; 8 =
                               auto, and STRING key columns are replaced by dictionary ids
                               first whatever the row count (auto does so from 2M rows)       */
  int32_t shared_table_bytes; /* <= 0 = auto                                                   */
  /* Fused drop_nulls pre-filter (cpp/src/stream_compaction/drop_nulls.cu:56-96): a row takes
   * part only if it is valid in every one of these masks (bit i = row i, same bit layout and
   * the same `offset` convention as a column sliced at `row_filter_offsets[j]`). */
  int32_t num_row_filters;
  const uint32_t* const* row_filter_masks; /* host array of device pointers */
  const int32_t* row_filter_offsets;       /* host array or NULL (all zero) */
} b2_groupby_options;

typedef struct b2_groupby b2_groupby;             /* cudf::groupby::groupby          */
typedef struct b2_groupby_state b2_groupby_state; /* partial-aggregate state, below */

/* ---- the drop-in path -------------------------------------------------- */

/* groupby::groupby(table_view const& keys, null_policy) — cpp/include/cudf/groupby.hpp:121-125,
 * cpp/src/groupby/groupby.cu:39-50.  The views are copied; the device data is not. */
b2_status b2_groupby_create(const b2_column_view* keys, int32_t num_keys, int32_t null_policy,
                            const b2_groupby_options* options /* may be NULL */, b2_groupby** out);

/* groupby::aggregate(requests, stream, mr) — cpp/include/cudf/groupby.hpp:181-184,
 * cpp/src/groupby/groupby.cu:219-236 → detail::hash::groupby (cpp/src/groupby/hash/groupby.cu:134-147).
 * Work is enqueued on `stream`; the call synchronises the stream once to learn the group count.
 * Errors: B2_LOGIC_ERROR "Size mismatch between request values and groupby keys."
 * (groupby.cu:225-229); B2_LOGIC_ERROR "Invalid type/aggregation combination."
 * (groupby.cu:185-201, a CUDF_EXPECTS with the default exception type); B2_UNSUPPORTED for requests only the reference's sort path serves. */
b2_status b2_groupby_aggregate(b2_groupby* gb, const b2_aggregation_request* requests,
                               int32_t num_requests, void* stream, const b2_allocator* allocator,
                               b2_groupby_result* out);

/* ~groupby() */
void b2_groupby_destroy(b2_groupby* gb);

/* Releases every device buffer and host array of a result (what ~table / ~column do). */
void b2_result_free(b2_groupby_result* result);

/* ---- partial-aggregate state: the multi-GPU / batch-wise decomposition ---
 * The reference ships partial aggregates between GPUs and merges them
 * (python/cudf_polars/cudf_polars/streaming/actor_graph/groupby.py:339-456; stateful form
 * cudf::groupby::streaming_groupby, cpp/include/cudf/groupby.hpp:478-598,
 * cpp/src/groupby/streaming_groupby/merge.cu:91-142).  A state holds one hash table of
 * {key, n, Σx, Σx², min, max …} cells for a fixed (key schema, request list). */

/* Creates an empty state for the key schema of `gb` and the given requests (values pointers
 * are read at update time from `requests` passed to b2_state_update). */
b2_status b2_state_create(const b2_groupby* gb, const b2_aggregation_request* requests,
                          int32_t num_requests, b2_groupby_state** out);

/* Aggregates the rows of (gb keys, requests values) into the state: the local pass of a
 * multi-GPU groupby, or one batch of streaming_groupby::aggregate (groupby.hpp:539-541). */
b2_status b2_state_update(b2_groupby_state* st, const b2_groupby* gb,
                          const b2_aggregation_request* requests, int32_t num_requests,
                          void* stream);

/* Size in bytes of one packed partial record ({key cell, accumulator cells…}, 8-byte cells). */
int32_t b2_state_record_bytes(const b2_groupby_state* st);

/* Hash-partitions the state's groups by owner = hash(key) % num_parts (the role of
 * cudf::hash_partition on the partial table, cpp/src/partitioning/partitioning.cu:569-750):
 * writes the records destination-major into ONE device buffer obtained from `allocator` (owned by
 * the caller: *records_out, *records_bytes) and the per-destination record counts into `counts`
 * (host array, num_parts).  Synchronises `stream`. */
b2_status b2_state_pack(b2_groupby_state* st, int32_t num_parts, void* stream,
                        const b2_allocator* allocator, void** records_out, size_t* records_bytes,
                        int64_t* counts);

/* Fixed-size form of the same partition for small states: no host round trip.  The records of
 * destination d go to chunk d of `out` (device memory, num_parts * b2_state_chunk_bytes()):
 * chunk = { uint64 count, uint64 overflow, records[chunk_records] }.  If any destination holds more
 * than `chunk_records` records, every chunk carries overflow = 1 and no records, so that all
 * receivers of an all-to-all with equal splits learn it and the caller falls back to
 * b2_state_pack.  Enqueues on `stream` without synchronising it. */
int64_t b2_state_chunk_bytes(const b2_groupby_state* st, int64_t chunk_records);
b2_status b2_state_pack_chunks(b2_groupby_state* st, int32_t num_parts, int64_t chunk_records,
                               void* stream, void* out);

/* Merges `num_chunks` received chunks into an EMPTY state.  Does not synchronise; a sender's
 * overflow mark surfaces as B2_LOGIC_ERROR "partial-record chunk overflow" from the next
 * b2_state_finalize / b2_state_num_groups on this state. */
b2_status b2_state_merge_chunks(b2_groupby_state* st, const void* chunks, int32_t num_chunks,
                                int64_t chunk_records, void* stream);

/* Merges `num_records` packed records (device memory, any origin with the same schema) into
 * the state: streaming_groupby::merge (groupby.hpp:548-556). */
b2_status b2_state_merge(b2_groupby_state* st, const void* records, int64_t num_records,
                         void* stream);

/* Drops all groups but keeps the schema; `expected_groups` sizes the next table (<=0 unknown). */
b2_status b2_state_reset(b2_groupby_state* st, int64_t expected_groups, void* stream);

/* Number of groups currently held (synchronises `stream`). */
b2_status b2_state_num_groups(b2_groupby_state* st, void* stream, int64_t* out);

/* Compacts keys and finalises the compound aggregations (mean = Σx/n; M2 = Σx² − (Σx)²/n;
 * var = M2/(n−ddof); std = sqrt(var)) — cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:93-186,
 * cpp/src/groupby/common/m2_var_std.cu:49-59,160-187; streaming_groupby::finalize
 * (groupby.hpp:566-568).  The state stays valid. */
b2_status b2_state_finalize(b2_groupby_state* st, void* stream, const b2_allocator* allocator,
                            b2_groupby_result* out);

void b2_state_destroy(b2_groupby_state* st);

/* ---- row-level hash partition: the multi-GPU pre-step for high-cardinality inputs ---
 * cudf::hash_partition(input, columns_to_hash, num_partitions, hash_function, seed)
 * (cpp/include/cudf/partitioning.hpp:97-108; cpp/src/partitioning/partitioning.cu:876-975):
 * reorders the rows of `columns` (fixed-width and STRING columns, nullable or not; the first
 * `num_key_columns` are hashed) so that partition p occupies rows [offsets[p], offsets[p+1]).
 * The partition of a row is the reference's: row hash % num_parts with
 *   B2_HASH_MURMUR3  MurmurHash3_x86_32(element bytes, seed) per column, a null element hashing to
 *                    UINT32_MAX, columns folded left to right with hash_combine
 *                    (hashing/detail/murmurhash3_x86_32.cuh:22-76, row_operator/hashing.cuh:52-134,
 *                    hashing/detail/hashing.hpp:83-86; floats: -0 as +0, one NaN);
 *   B2_HASH_IDENTITY the numeric element cast to uint32 (partitioning.cu:856-874); hashing a
 *                    non-numeric column is B2_LOGIC_ERROR "IdentityHash does not support this data type".
 * Output columns come from the allocator; `offsets` is a host array of num_parts+1 entries.  Up to
 * 2^20 partitions (beyond 4096 the per-CTA counters move from shared to global memory).
 * num_key_columns == 0, num_parts == 0, num_columns == 0 or zero rows give empty columns of the
 * input types and all-zero offsets (partitioning.cu:885-888,
 * cpp/tests/partitioning/hash_partition_test.cpp:72-142); columns of different sizes are
 * B2_INVALID_ARGUMENT (std::invalid_argument in the reference, :934-937).  The order of rows inside a
 * partition is unspecified.  Synchronises `stream`. */
enum { B2_HASH_IDENTITY = 0, B2_HASH_MURMUR3 = 1 };  /* cudf::hash_id, partitioning.hpp:32-35 */
b2_status b2_hash_partition(const b2_column_view* columns, int32_t num_columns,
                            int32_t num_key_columns, int32_t num_parts, int32_t hash_function,
                            uint32_t seed, void* stream, const b2_allocator* allocator,
                            b2_owned_column* out_columns, int64_t* offsets);

/* Validity bitmask <-> one byte per row (1 = valid).  A row exchange between ranks moves validity
 * as bytes because a partition starts at an arbitrary bit of its mask
 * (the reference copies bitmask ranges with cudf::copy_bitmask / concatenate_masks,
 * cpp/include/cudf/null_mask.hpp).  b2_bytes_to_mask writes ceil(size/32) words and the number of
 * nulls to *null_count_device (device memory).  Both enqueue on `stream` without synchronising. */
b2_status b2_mask_to_bytes(const uint32_t* mask, int64_t offset, int64_t size, void* stream, uint8_t* out);
b2_status b2_bytes_to_mask(const uint8_t* bytes, int64_t size, void* stream, uint32_t* mask,
                           int32_t* null_count_device);

/* Finishes partial aggregates that travel as columns (what string / float / wide keys exchange between ranks
 * and batches: Σx, n and Σx² per group): the finalizers of the hash path over such columns
 * (cpp/src/groupby/hash/hash_compound_agg_finalizer.cu:93-186, cpp/src/groupby/common/m2_var_std.cu:57).
 * `kind` is B2_AGG_COUNT_VALID (n as INT32), B2_AGG_MEAN (Σx / n as `result_type_id`: FLOAT64, or a duration type
 * by integer division), B2_AGG_M2, B2_AGG_VARIANCE, B2_AGG_STD (FLOAT64), or -1: no values, only the validity of
 * a result from n.  `sum` / `sum_sq` are fixed-width numeric columns (NULL where the kind does not need them),
 * `count` is an integer column (INT32 from one aggregate, INT64 once counts were summed).  `nullable` != 0 gives the result a validity mask (valid where n > 0; variance and standard
 * deviation: where n - ddof > 0) and its null count; variance and standard deviation always carry one.
 * Synchronises `stream` once. */
b2_status b2_finish_partial(int32_t kind, int32_t ddof, int32_t result_type_id, const b2_column_view* sum,
                            const b2_column_view* count, const b2_column_view* sum_sq, int32_t nullable,
                            void* stream, const b2_allocator* allocator, b2_owned_column* out);

/* Releases the buffers of one owned column obtained from b2_hash_partition. */
void b2_column_free(b2_owned_column* col, const b2_allocator* allocator, void* stream);

/* ---- multi-GPU: one process per GPU, NCCL over NVLink / NVSwitch ----------
 * The reference's distributed groupby aggregates locally, hash-partitions the PARTIAL aggregates by
 * key, shuffles them and reduces on the owner (python/cudf_polars/cudf_polars/streaming/actor_graph/
 * groupby.py:339-456 over partition_and_pack / unpack_and_concat,
 * cpp/libcudf_streaming/src/partition_utils.cpp:72-185).  b2_groupby_aggregate_multi is that plan as
 * one call per rank: local fused aggregate -> partial records partitioned by owner = hash(key) mod
 * ranks -> ONE exchange (ncclSend / ncclRecv pairs inside an ncclGroup, on `stream`) -> merge ->
 * finalize.  Every rank receives the finished groups it owns; the key sets of the ranks are disjoint.
 *
 * A b2_comm wraps an NCCL communicator.  The NCCL library is resolved at run time (the copy
 * already loaded into the process, else libnccl.so.2 from the loader path; B2_NCCL_LIB overrides),
 * so the library has no link-time dependency on it.  b2_comm_unique_id (rank 0) + b2_comm_create
 * (every rank, with its GPU current) follow ncclGetUniqueId / ncclCommInitRank; b2_comm_adopt wraps a
 * communicator the caller already owns (it is not destroyed by b2_comm_destroy).
 *
 * Small states travel as fixed-size chunks (no host round trip: b2_state_pack_chunks); a rank with
 * more records than a chunk holds marks every chunk it sends, and all ranks repeat the exchange with
 * exact sizes (one all-gather of the count matrix, then variable send / recv).  Keys that do not
 * pack into 64 bits (strings, floats, wide composites) return B2_UNSUPPORTED on EVERY rank before
 * any communication (the key types are the same everywhere): partition the rows with
 * b2_hash_partition instead.  All ranks must make the same sequence of calls. */
typedef struct b2_comm b2_comm;
#define B2_COMM_ID_BYTES 128
b2_status b2_comm_unique_id(uint8_t id[B2_COMM_ID_BYTES]);
b2_status b2_comm_create(const uint8_t id[B2_COMM_ID_BYTES], int32_t rank, int32_t num_ranks, b2_comm** out);
b2_status b2_comm_adopt(void* nccl_comm, int32_t rank, int32_t num_ranks, b2_comm** out);
void b2_comm_destroy(b2_comm* comm);
b2_status b2_groupby_aggregate_multi(b2_comm* comm, b2_groupby* gb, const b2_aggregation_request* requests,
                                     int32_t num_requests, void* stream, const b2_allocator* allocator,
                                     b2_groupby_result* out);

/* ---- aggregate without any device allocation -----------------------------
 * No counterpart in the reference (libcudf always allocates through an rmm resource).
 *
 * For callers that must not allocate device memory while they run: code inside a latency-critical
 * serving loop or a real-time pipeline where a cudaMalloc (an implicit device-wide
 * synchronisation) is not acceptable, plug-ins that run under a host framework owning all device
 * memory and handing out fixed buffers, and processes whose memory pool has been frozen.  The
 * whole aggregate runs inside buffers the caller passes plus ONE fixed scratch array that lives in
 * the library image: a file-scope __device__ array of B2_NOALLOC_SCRATCH_BYTES that every GPU
 * loading the library holds until the process exits.  The hash table, the control block and the
 * null counters are carved out of it.
 *
 * Same semantics and result types as b2_groupby_aggregate, with these limits:
 *   - keys must be packable into 64 bits (fixed-width, non-float key columns; no strings);
 *   - the table needs 2*max_groups+1 slots of (1 + number of accumulator cells) * 8 bytes; a call
 *     whose table would not fit the scratch array is rejected with B2_INVALID_ARGUMENT and a
 *     message that names both sizes (e.g. one SUM+COUNT request: up to 174,000 groups);
 *   - if the input holds more than max_groups groups the call fails with B2_LOGIC_ERROR and the
 *     output buffers hold garbage.
 * Outputs: key_data[k] and result_data[i] are device buffers of max_groups elements of the
 * column's result type (result i = aggregations in request order, request after request);
 * key_masks[k] / result_masks[i] are device buffers of ceil(max_groups/32) words, required where
 * the column is nullable (key: INCLUDE policy and a masked key column; result: see
 * b2_groupby_aggregate), otherwise they may be NULL.  *num_groups_out (host) receives the group
 * count; null_counts_out (host, may be NULL) receives num_keys + total-aggregations null counts.
 *
 * The first call on each device looks up the scratch array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before any stream
 * capture begins.  The call uses no cudaMalloc / cudaFree / cudaMallocAsync, and neither reads nor
 * configures any memory pool.
 * Every call reuses the same scratch array and re-initialises the parts it reads, so the previous
 * call's contents never leak into a result — but two calls that overlap in time on one GPU (other
 * streams, other host threads) race on it: serialise them.  Synchronises `stream` twice when the
 * input has rows (once for the group count, once after the results are written), once otherwise. */
#define B2_NOALLOC_SCRATCH_BYTES (8u << 20)
b2_status b2_groupby_aggregate_noalloc(b2_groupby* gb, const b2_aggregation_request* requests,
                                       int32_t num_requests, void* stream, int32_t max_groups,
                                       void* const* key_data, uint32_t* const* key_masks,
                                       void* const* result_data, uint32_t* const* result_masks,
                                       int32_t* num_groups_out, int32_t* null_counts_out);

/* ---- introspection ------------------------------------------------------ */
const char* b2_last_error(void);   /* message of this thread's last failure */
const char* b2_version(void);
/* Counters of the calling thread's last aggregate/update call: kernels launched, table
 * attempts (1 = first table size was enough), bytes of scratch used. */
typedef struct b2_call_stats {
  int32_t kernel_launches;
  int32_t table_attempts;
  int64_t table_capacity;
  int64_t scratch_bytes;
  int32_t used_shared_table;
  float aggregate_kernel_ms; /* device time of the fused aggregate kernel(s), CUDA events on the
                                call's stream, read after the call's own synchronisation */
} b2_call_stats;
void b2_get_last_stats(b2_call_stats* out);

#ifdef __cplusplus
}
#endif
#endif /* B2_GROUPBY_H */
