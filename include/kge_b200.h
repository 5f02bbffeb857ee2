/*
 * kge_b200.h — C ABI of libkge_b200.so: knowledge-graph-embedding scoring on NVIDIA B200 (sm_100a).
 *
 * This is the boundary that replaces cuke's "emit CUDA text, JIT-compile it, call module.run(*args)"
 * step (reference: pycuke1/run/gpu.py:4-19 and the generated host wrapper
 * pycuke1/codegen/gpu_template.cu:8-17) and its hand-written inspector module
 * (reference: apps/kge/kge.py:249-271, apps/kge/inspection/inspector.cu:139-146).
 *
 * Conventions
 *   - C linkage, POD structs, raw DEVICE pointers (e.g. torch `tensor.data_ptr()`), row-major contiguous
 *     tensors, every base pointer 16-byte aligned (id arrays: aligned to their element size).  Pointers are
 *     never retained after a call returns.
 *   - The library never allocates or frees device memory that the caller can see: outputs and scratch
 *     ("workspace") are caller-provided; `*_workspace_bytes` says how much is needed.
 *   - Every launch goes to the `cudaStream_t` passed in; calls are asynchronous with respect to the host
 *     unless stated otherwise.  Re-entrant per (device, stream).
 *   - Return value: 0 = success; negative = argument error (KGE_E_*), nothing was launched;
 *     positive = a cudaError_t reported by the runtime for this call's launches.  `kge_last_error()`
 *     returns a thread-local, human-readable description of the last non-zero return.
 *   - Entity / relation ids are int64 (the reference's GPU convention, pycuke1/codegen/gpu.py:200-201)
 *     or int32 (`id_bits`).  Ids are trusted to lie inside the tables, exactly as in the reference
 *     (its generated kernels do no bounds checks either), unless KGE_FLAG_CHECK_IDS / kge_validate_ids is used.
 *   - Relation matrices use the orientation of the reference's CPU path: for `'i,ij->j'`
 *     (apps/kge/kge.py:21-23) out[j] = sum_i x[i] * Proj[r][i][j].
 */
#ifndef KGE_B200_H
#define KGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque stand-in so that this header needs no CUDA include; pass a cudaStream_t. */
typedef struct CUstream_st* kge_stream_t;

#define KGE_ABI_VERSION 1

#if defined(__GNUC__)
#define KGE_API __attribute__((visibility("default")))
#else
#define KGE_API
#endif

enum kge_status {
    KGE_OK = 0,
    KGE_E_NULL = -1,         /* a required pointer is NULL */
    KGE_E_ALIGN = -2,        /* a pointer is not 16-byte aligned */
    KGE_E_UNSUPPORTED = -3,  /* model / dtype / mode / dim combination not supported */
    KGE_E_SHAPE = -4,        /* inconsistent sizes (e.g. batch not a multiple of chunk) */
    KGE_E_WORKSPACE = -5,    /* workspace too small */
    KGE_E_RANGE = -6,        /* size beyond a stated maximum */
    KGE_E_DEVICE = -7        /* no usable sm_100 device / kernel image missing */
};

/* Score functions.  TransE/TransH/TransR/TransF/RESCAL follow apps/kge/kge.py:273-390; DistMult and
 * ComplEx are absent from the reference and written with the same operators (bvv over elementwise
 * products). */
enum kge_model {
    KGE_TRANSE = 0,   /* v = E[h] - E[t] + R[r]                         score = -||v||_2 */
    KGE_TRANSH = 1,   /* u = E[h]-E[t]; v = u + R[r] - (W[r].u) W[r]    score = -||v||_2 */
    KGE_TRANSR = 2,   /* v = (E[h]-E[t]) . P[r] + R[r]                  score = -||v||_2 */
    KGE_TRANSF = 3,   /* score = (E[h]+R[r]).E[t] + (E[t]-R[r]).E[h]                     */
    KGE_DISTMULT = 4, /* score = sum_k E[h][k] R[r][k] E[t][k]                           */
    KGE_RESCAL = 5,   /* score = sum_j (sum_i E[h][i] P[r][i][j]) E[t][j]                */
    KGE_COMPLEX = 6   /* rows interleaved re,im; score = Re(sum_k h_k r_k conj(t_k))     */
};

enum kge_dtype { KGE_F32 = 0, KGE_BF16 = 1 };   /* storage type of the tables; accumulation is fp32 */

enum kge_precision {
    KGE_PREC_FP32 = 0,    /* fp32 CUDA-core arithmetic throughout (default) */
    KGE_PREC_TENSOR = 1,  /* contractions on the tensor cores where a kernel exists.  fp32 operands are split in two bf16
                             terms, v ~ hi + lo (16 mantissa bits), and a product is three bf16 MMAs (lo.hi + hi.lo + hi.hi)
                             accumulated in fp32: relative product error ~2^-16, inside the 1e-4 tolerance, at the full
                             tensor rate and 4 operand bytes per element; bf16 tables as one bf16 MMA; everything else as
                             KGE_PREC_FP32 */
    KGE_PREC_TENSOR_TF32 = 2  /* as KGE_PREC_TENSOR with fp32 operands split in two tf32 terms ("3xTF32": product error
                             ~2^-20, half the tensor rate, 8 operand bytes per element) */
};

enum kge_neg_mode {
    KGE_NEG_NONE = 0,         /* positives only */
    KGE_NEG_PER_TRIPLE = 1,   /* neg is (batch, n_neg): triple i is scored against its own n_neg rows */
    KGE_NEG_CHUNK_SHARED = 2  /* neg is (batch/chunk, n_neg): all triples of a chunk share n_neg rows
                                 (the layout of apps/examples/examples.py:1434-1441) */
};

typedef struct kge_problem {
    int32_t model;       /* enum kge_model */
    int32_t dtype;       /* enum kge_dtype */
    int32_t neg_mode;    /* enum kge_neg_mode */
    int32_t id_bits;     /* 32 or 64: width of h, r, t, neg */
    int32_t dim;         /* floats per entity row (ComplEx: 2 x complex dimension) */
    int32_t n_neg;       /* negatives per triple (per-triple) or per chunk (chunk-shared); 0 if none */
    int32_t n_neg_head;  /* the first n_neg_head negatives replace the head, the others the tail */
    int32_t chunk;       /* triples per chunk (chunk-shared), else 0 */
    int64_t batch;       /* number of positive triples */
    int64_t n_ent;       /* rows of `ent` */
    int64_t n_rel;       /* rows of `rel` / `rel2` */
    int32_t precision;   /* enum kge_precision */
    int32_t reserved;    /* flags: 0 or KGE_FLAG_CHECK_IDS */
} kge_problem;

/* kge_problem.reserved flag for kge_score_forward / kge_score_backward / kge_score_loss_backward: h, t, neg are checked
 * against n_ent and r against n_rel before anything is gathered; an id outside sets KGE_ERR_ID_RANGE and row 0 is used
 * in its place (that triple's outputs are meaningless, nothing outside the tables is touched).  Costs one pass over the
 * ids and a copy of them in the workspace (kge_score_workspace_bytes accounts for it).  The rel_* grouping of the
 * relation-matrix models is not re-checked: build it with kge_inspect over relation ids that went through
 * kge_validate_ids. */
#define KGE_FLAG_CHECK_IDS 1

typedef struct kge_tensors {
    const void* ent;   /* (n_ent, dim) entity table, or a compact staging buffer addressed by slot ids */
    const void* rel;   /* (n_rel, dim) relation vectors; NULL for RESCAL */
    const void* rel2;  /* TransH: hyperplane normals (n_rel, dim); TransR/RESCAL: (n_rel, dim, dim); else NULL */
    const void* h;     /* (batch,) head ids */
    const void* r;     /* (batch,) relation ids */
    const void* t;     /* (batch,) tail ids */
    const void* neg;   /* negative entity ids, shape per neg_mode; NULL if none */
    /* Relation grouping produced by kge_inspect over `r`; required by TransR/RESCAL scoring, else NULL. */
    const int32_t* rel_perm;    /* (batch,) triples ordered by relation id (stable) */
    const int32_t* rel_seg;     /* (>= n_rel_groups+1,) start of each group in rel_perm */
    const int64_t* rel_uniq;    /* (n_rel_groups,) relation id of each group */
    const int64_t* n_rel_groups;/* device scalar */
} kge_tensors;

/* Per-slot gradient rows written by kge_score_backward ("slot" = one id occurrence).  g_head, g_tail and
 * g_neg are normally three consecutive regions of one buffer laid out like the id list [h | t | neg] given
 * to kge_inspect, so that a single kge_segment_reduce turns them into one gradient row per distinct entity. */
typedef struct kge_grads {
    float* g_head;   /* (batch, dim) */
    float* g_tail;   /* (batch, dim) */
    float* g_neg;    /* (number of negative ids, dim); NULL if no negatives */
    float* g_rel;    /* (batch, dim) gradient of R[r] per triple; NULL for RESCAL */
    float* g_rel2;   /* TransH: (batch, dim) gradient of W[r] per triple.
                        TransR/RESCAL: (n_rel_groups, dim, dim) gradient of P[rel_uniq[g]], already summed
                        over the triples of group g.  Else NULL. */
} kge_grads;

/* ---- library ------------------------------------------------------------------------------------ */

KGE_API int kge_version(void);                 /* KGE_ABI_VERSION of the loaded library */
KGE_API const char* kge_last_error(void);      /* thread-local message for the last non-zero return */
KGE_API long long kge_launch_count(void);      /* kernels launched by this library in this process so far */

/* Values OR-ed into the device error word by kernels of this library. */
#define KGE_ERR_WAIT_TIMEOUT 2  /* a bounded wait inside a kernel ran out and the kernel gave up: its outputs are invalid */
#define KGE_ERR_ID_RANGE 8      /* an id outside its table was met by kge_validate_ids / a call with KGE_FLAG_CHECK_IDS */

/* Reads (and clears) the device error word of the current device: 0 = clean, else an OR of KGE_ERR_*.
 * Synchronises `stream`. */
KGE_API int kge_check(kge_stream_t stream, int32_t* flags_out);

/* Range check of an id array: every ids[i] outside [0, id_space) sets KGE_ERR_ID_RANGE in the device error word, and,
 * if `sanitized` is not NULL, sanitized[i] (same width; may be `ids` itself) receives the id or 0 in its place, so
 * that a later gather never touches memory outside the table.  The reference's generated kernels trust their ids
 * (pycuke1/codegen/gpu.py:9-123 emits no bounds checks); this is the opt-in check for ids that come from outside. */
KGE_API int kge_validate_ids(const void* ids, int32_t id_bits, int64_t n, int64_t id_space, void* sanitized,
                             kge_stream_t stream);

/* Self-test of the bounded waits used inside the tensor-core kernels: one warp waits on a shared-memory barrier that
 * nothing ever completes, with a limit of `polls` polls (1..65536), gives up, sets KGE_ERR_WAIT_TIMEOUT and returns.
 * Shows that a wait that runs out ends the kernel normally and is reported through kge_check.  No reference
 * counterpart. */
KGE_API int kge_selftest_wait_timeout(int32_t polls, kge_stream_t stream);

/* ---- reference-compatible forward ---------------------------------------------------------------
 * Replaces `module.run(*args)` of the code the reference generates for apps/kge/kge.py:273-390
 * (launch site pycuke1/codegen/gpu_template.cu:11).  Output exactly as the reference returns it:
 * TransE/TransH/TransR -> the per-triple VECTOR v, (batch, dim) fp32, no norm;
 * TransF/RESCAL/DistMult/ComplEx -> the scalar score, (batch,) fp32.
 * neg_mode must be KGE_NEG_NONE (the reference flattens negatives into a longer batch,
 * apps/kge/data/data_init.py:55-61).  TransR/RESCAL do not need the rel_* grouping here. */
KGE_API int kge_ref_forward(const kge_problem* p, const kge_tensors* t, float* out, kge_stream_t stream);

/* ---- inspector ----------------------------------------------------------------------------------
 * GPU inspector: LSD radix sort + unique over n ids in [0, id_space).  Supersedes the per-16-id
 * `build_index` kernel (apps/kge/inspection/inspector.cu:68-136) and the host-side
 * `torch.argsort(rel_ids)` (apps/kge/test_cuke.py:93-96).  All outputs are bit-exact with
 *   uniq, inverse = numpy.unique(ids, return_inverse=True);  perm = numpy.argsort(ids, kind="stable");
 *   seg[u] = first sorted position of uniq[u];  seg[U..n] = n.
 *   uniq     (n,)   int64  sorted distinct ids in [0, U); entries >= U are left untouched
 *   inverse  (n,)   int32  ids[i] == uniq[inverse[i]]
 *   perm     (n,)   int32  sorted position -> original position
 *   seg      (n+1,) int32
 *   n_unique (1,)   int64  U, on the device
 * id_space must be <= 2^31.  n <= 2^31 - 1. */
KGE_API size_t kge_inspect_workspace_bytes(int64_t n);
KGE_API int kge_inspect(const void* ids, int32_t id_bits, int64_t n, int64_t id_space,
                void* workspace, size_t workspace_bytes,
                int64_t* uniq, int32_t* inverse, int32_t* perm, int32_t* seg, int64_t* n_unique,
                kge_stream_t stream);

/* Legacy inspector with the reference's exact outputs (apps/kge/kge.py:249-271,
 * apps/kge/inspection/inspector.cu:68-143): for every chunk of 16 consecutive relation ids the two most
 * frequent ids (count >= 2) go to uniq[b][0..1] (other entries = rel_num), buf[b][i] is the cache slot
 * (0/1) or id+16, cnt[b] the number of cached ids.  rel (n,) int64, n a multiple of 16;
 * uniq, buf (n/16, 16) int64 and cnt (n/16,) int64 must be zero-initialised by the caller as the
 * reference does.  Chunks whose 16 ids are all distinct are handled without the reference's
 * out-of-bounds shared-memory write (inspector.cu:90) and give the result that write-free code gives. */
KGE_API int kge_legacy_inspect(const int64_t* rel, int64_t n, int64_t rel_num,
                       int64_t* uniq, int64_t* buf, int64_t* cnt, kge_stream_t stream);

/* Copies the rows ids[0..n) of `table` (n_rows x dim, dtype) into out (n x dim, same dtype): the
 * dedup staging step (each distinct row leaves HBM once per batch).  If n_dev is not NULL the row
 * count is min(n, *n_dev) read on the device.  `first_row` is subtracted from every id (row-partitioned
 * tables: the local shard starts at global row first_row). */
KGE_API int kge_gather_rows(const void* table, int32_t dtype, int32_t dim, const int64_t* ids, int64_t n,
                    const int64_t* n_dev, int64_t first_row, void* out, kge_stream_t stream);

/* Inverse of kge_gather_rows for fp32 rows: out[ids[i] - first_row][:] = rows[i][:] for i < min(n, *n_dev).
 * ids must be distinct (the inspector's `uniq`); used to place compact gradient rows into a dense table.
 * No counterpart in the reference, which never aggregates gradients (apps/kge/kge.py:393-515). */
KGE_API int kge_scatter_rows(const float* rows, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                             int64_t first_row, float* out, kge_stream_t stream);

/* Segmented sum: out[u][:] = sum over sorted positions p in [seg[u], seg[u+1]) of rows[perm[p]][:],
 * added in a fixed order (deterministic, no atomics).  rows (n, dim) fp32; out fp32 with room for
 * max(U, n_out) rows (n rows always suffice); rows u in [U, n_out) are zero-filled, n_out = 0 skips that.  The backward "scatter-add" of per-slot gradient rows
 * into one row per distinct id (replaces the un-aggregated outputs of apps/kge/kge.py:393-515). */
KGE_API size_t kge_segment_reduce_workspace_bytes(int64_t n, int32_t dim);
KGE_API int kge_segment_reduce(const float* rows, int32_t dim, int64_t n, const int32_t* perm, const int32_t* seg,
                       const int64_t* n_unique, float* out, int64_t n_out,
                       void* workspace, size_t workspace_bytes, kge_stream_t stream);

/* Same result as kge_segment_reduce, for hosts that may not allocate device memory: the partial-row scratch
 * lives in a fixed array inside the library (8 MiB of device memory per GPU, held from library load to process
 * exit) instead of a caller-provided workspace, and this call performs no allocation of any kind.
 * It has no counterpart in the reference.  Typical callers: a serving or training loop that was handed its
 * buffers up front and runs under a "no allocation after start-up" rule (allocator calls synchronise the device
 * and can fail late), or an FFI host that can pass its own input/output buffers but has no device allocator to
 * size a workspace with.  Inputs and outputs are still the caller's.
 * Limit: ceil(n / 32) * dim <= 1,048,576 (e.g. n = 131,072 slots at dim = 256); larger problems are rejected
 * with KGE_E_RANGE and a message, nothing is launched.
 * The first call on each device looks up the scratch address (a host-side, non-stream operation); make that
 * first call before any stream capture begins on that device.
 * All calls on a device share the one scratch array: two calls that overlap on the GPU (different streams, or
 * different host threads without ordering) race on it and corrupt each other's sums.  The array keeps the
 * previous call's contents; nothing in it needs to start at zero, because every partial row is written before
 * it is read within a call. */
KGE_API int kge_segment_reduce_static(const float* rows, int32_t dim, int64_t n, const int32_t* perm, const int32_t* seg,
                                      const int64_t* n_unique, float* out, int64_t n_out, kge_stream_t stream);

/* ---- scoring ------------------------------------------------------------------------------------
 * Fused gather + score.  pos_score (batch,) ; neg_score (batch, n_neg) per-triple or
 * (batch/chunk, chunk, n_neg) chunk-shared.  Scores as in enum kge_model.  Ids index `ent` directly; to
 * score against a compact staging buffer pass that buffer as `ent` and slot numbers (the inspector's
 * `inverse`, id_bits = 32) as h, t, neg.  Replaces the generated kernels of apps/kge/kge.py:273-390 plus
 * the norm the reference leaves to the caller. */
KGE_API size_t kge_score_workspace_bytes(const kge_problem* p, int32_t backward);
KGE_API int kge_score_forward(const kge_problem* p, const kge_tensors* t, float* pos_score, float* neg_score,
                      void* workspace, size_t workspace_bytes, kge_stream_t stream);

/* Backward of kge_score_forward: given d(loss)/d(score) for every score, writes the per-slot gradient rows
 * of struct kge_grads.  pos_score / neg_score are the forward's outputs (the distance models reuse them).
 * True gradients of the forward above (the reference's backward_* demos, apps/kge/kge.py:393-515, are
 * per-triple pieces of these). */
KGE_API int kge_score_backward(const kge_problem* p, const kge_tensors* t,
                       const float* pos_score, const float* neg_score,
                       const float* dpos, const float* dneg, const kge_grads* g,
                       void* workspace, size_t workspace_bytes, kge_stream_t stream);

/* Forward, logistic ranking loss and backward of the chunk-shared scorers in one call, on the tensor-core path:
 * the same numbers as kge_score_forward -> kge_logistic_loss(neg_weight) -> kge_score_backward, but each score of a
 * negative is turned into its loss term and its gradient weight inside the tile that produced it, so the
 * (batch, n_neg) score matrix, its gradient and a second operand pack never reach memory.  Writes pos_score (batch,),
 * loss_out (1,) and the gradient rows of `g`; scores of the negatives are not returned.  Needs precision
 * KGE_PREC_TENSOR and either neg_mode KGE_NEG_CHUNK_SHARED, dim % 4 == 0 and TransE, DistMult or ComplEx, or TransR over
 * bf16 tables (any per-triple negatives; the relation-grouped difference rows are then packed once for the forward and
 * the three backward products, and the rel_* grouping of kge_tensors is required); KGE_E_UNSUPPORTED otherwise.
 * No reference counterpart: the reference stops at per-triple outputs
 * (apps/kge/kge.py:273-390) and leaves loss and gradients to the caller's framework. */
KGE_API size_t kge_score_loss_backward_workspace_bytes(const kge_problem* p);
KGE_API int kge_score_loss_backward(const kge_problem* p, const kge_tensors* t, float neg_weight,
                            float* pos_score, float* loss_out, const kge_grads* g,
                            void* workspace, size_t workspace_bytes, kge_stream_t stream);

/* Logistic ranking loss over the scores and its derivative, for driving fwd+bwd without a host round trip:
 * loss = sum softplus(-pos) + (1/n_neg_per_pos) sum softplus(neg);  dpos = -sigmoid(-pos),
 * dneg = sigmoid(neg)/n_neg_per_pos.  loss_out (1,) fp32 device, reduced in a fixed order.
 * workspace >= 4096 bytes. */
KGE_API int kge_logistic_loss(const float* pos, int64_t n_pos, const float* neg, int64_t n_neg_total,
                      float neg_weight, float* dpos, float* dneg, float* loss_out,
                      void* workspace, size_t workspace_bytes, kge_stream_t stream);

/* ---- row-partitioned tables (multi-GPU) ----------------------------------------------------------
 * counts[g] = number of ids in uniq[0..U) owned by rank g under the contiguous partition
 * owner(id) = id / rows_per_rank; uniq is sorted, so each rank's ids are one contiguous range.
 * counts (world,) int64 device. */
KGE_API int kge_owner_counts(const int64_t* uniq, const int64_t* n_unique, int64_t n_max, int64_t rows_per_rank,
                     int32_t world, int64_t* counts, kge_stream_t stream);

/* The row-partitioned table read in place by every GPU of a node (one process per GPU, NVLink / NVSwitch peer access).
 * kge_ipc_export: handle64 (64 bytes) identifies the device allocation that holds ptr, *offset is ptr's distance from
 *   its start; both travel to the other processes by any host channel.  The memory must come from cudaMalloc (the
 *   default of torch's caching allocator), not from a memory pool or a virtual-memory mapping.
 * kge_ipc_open: maps a peer's allocation into this process (peer access is enabled on first use) and returns the
 *   address that corresponds to the exported ptr.  kge_ipc_close unmaps it (same offset).
 * kge_gather_rows_peers: out[i][:] = row ids[i] of the partitioned table for i < min(n, *n_dev), where shards is a DEVICE
 *   array of `world` pointers, shards[g] = first row of rank g's shard (rows [g * rows_per_rank, ...)), this rank's own
 *   shard included; n_rows is the table's total row count.  One kernel: local rows come from HBM, remote rows through
 *   NVLink with plain 16-byte loads, and every row lands in this GPU's memory.  An id outside [0, n_rows) sets
 *   KGE_ERR_ID_RANGE and yields a zero row; nothing outside the table is read.  Ordering against the owners' updates of
 *   their rows is the caller's (a barrier among the ranks after the updates of a step, before the gathers of the next).
 * No counterpart in the reference (single GPU, apps/kge/data/data_init.py:6-15). */
/* kge_pull_reduce: the owner-side sum of gradient rows, read in place from the ranks' buffers (the counterpart of
 *   kge_gather_rows_peers for the way back).  The ids the ranks requested from this owner were concatenated in rank order
 *   (rank r: positions [src_start[r], src_start[r+1])) and inspected (perm, seg, n_unique as from kge_inspect).  bases is a
 *   DEVICE array of `world` pointers to the ranks' gradient-row buffers, rows in the order of each rank's own sorted
 *   distinct ids, of which this owner's start at row src_off[r].  out[u][:] = sum over the ranks that touched distinct id
 *   u, in rank order (fixed order, no atomics), for u < min(n_max, *n_unique).  src_off, src_start (world + 1) int64 device.
 *   With sgd_table (fp32, this owner's shard) the owner's plain SGD step is applied in the same pass:
 *   sgd_table[ids[u] - first_row][:] -= lr * out[u][:], ids = the sorted distinct ids of the inspection; NULL: no update.
 *   The caller orders it after every rank's rows are complete (a barrier among the ranks) and keeps the buffers
 *   unchanged until every owner has read them. */
KGE_API int kge_pull_reduce(const float* const* bases, const int64_t* src_off, const int64_t* src_start, int32_t world, int32_t dim,
                    const int32_t* perm, const int32_t* seg, const int64_t* n_unique, int64_t n_max, float* out,
                    float* sgd_table, const int64_t* ids, int64_t first_row, float lr, kge_stream_t stream);
KGE_API int kge_ipc_export(const void* ptr, void* handle64, uint64_t* offset);
KGE_API int kge_ipc_open(const void* handle64, uint64_t offset, void** ptr_out);
KGE_API int kge_ipc_close(void* ptr, uint64_t offset);
KGE_API int kge_gather_rows_peers(const void* const* shards, int32_t world, int64_t rows_per_rank, int64_t n_rows, int32_t dtype,
                          int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev, void* out, kge_stream_t stream);

/* ---- general expressions ----------------------------------------------------------------------------------------
 * Evaluates, for every batch element i, a small register program over per-element VECTOR registers (dim floats) and
 * SCALAR registers: the target of the Python front-end for expressions of the reference's batched operators that are
 * not one of the seven score functions (what cuke's generator does for any composition of bvv / bsv / bvm / bov / bsm
 * over gathered rows, apps/kge/kge.py:13-84, pycuke1/codegen/gpu.py:182-236).  Instructions are (op, dst, a, b, c):
 *    0 GATHER  v[dst] = tables[a][ids[b][i]]           1..4 VADD VSUB VMUL VDIV  v[dst] = v[a] op v[b]
 *    5 SPLAT   v[dst][:] = s[a]                        6 DOT   s[dst] = v[a] . v[b]
 *    7..10 SADD SSUB SMUL SDIV  s[dst] = s[a] op s[b]  11 SCONST  s[dst] = float with bit pattern a
 *   12 VECMAT  v[dst][j] = sum_k v[a][k] M[k][j]       13 COLSUM  v[dst][j] = sum_k M[k][j] (M = tables[a][ids[b][i]])
 *   14 MATVEC  v[dst][k] = sum_j M[k][j] v[a][j]       (12, 14: M = tables[b][ids[c][i]], a (dim, dim) matrix per row id)
 *   15 ROW     v[dst] = tables[a][i]  ((batch, dim))   16 LOADS  s[dst] = tables[a][i]  ((batch,) operand)
 * Result (out_kind): 0 vector v[out_a] -> out (batch, dim); 1 scalar s[out_a] -> out (batch,); 2 outer product
 * s[out_s] * v[out_a] (x) v[out_b] -> out (batch, dim, dim); 3 s[out_s] * tables[out_table][ids[out_ids][i]] -> out
 * (batch, dim, dim); out_s < 0 means no scalar factor.  Tables are fp32, row-major, (rows, dim) or (rows, dim, dim).
 * Limits: 64 instructions, 16 vector and 16 scalar registers, 8 tables, 4 id arrays, dim <= 1024 and
 * n_vreg * dim * 4 bytes <= 48 KB. */
typedef struct kge_program {
    int32_t n_ops, n_vreg, n_sreg;
    int32_t out_kind, out_a, out_b, out_s, out_table, out_ids;
    int32_t ops[64][5];
} kge_program;
KGE_API int kge_eval_program(const kge_program* prog, int32_t dim, int64_t batch, const float* const* tables, int32_t n_tables,
                             const void* const* ids, int32_t id_bits, int32_t n_ids, float* out, kge_stream_t stream);

/* ---- batch ids generated on the device ---------------------------------------------------------------------
 * Counter-based sampling (Philox4x32-10): element i of stream `stream_id` under `seed` is a pure function of
 * (seed, stream_id, i) - counter words (i low, i high, stream_id, 0), key words (seed low, seed high), output words
 * 0 and 1 joined into w = x0 * 2^32 + x1 - so a batch can be regenerated anywhere, bit for bit.  Takes the place of the
 * host-side batch assembly of apps/kge/data/data_init.py:47-63 (ids drawn by CPU workers and copied to the GPU).
 *   kge_sample_uniform  out[i] = floor(w * id_space / 2^64)
 *   kge_sample_cdf      u = (w >> 11) * 2^-53; rank = first k with cdf[k] >= u, at most n_items - 1;
 *                       out[i] = perm[rank], or rank when perm is NULL.  cdf (n_items,) float64 non-decreasing with
 *                       cdf[n_items - 1] == 1; perm (n_items,) int64.  With cdf[k] = sum_{j<=k} (j+1)^-s / total this
 *                       is the bounded Zipf(s) law over a permuted id space.
 *   kge_sample_triples  row = floor(w * n_triples / 2^64); (h[i], r[i], t[i]) = triples[row][0..2], triples
 *                       (n_triples, 3) int64: positives drawn from a stored triple list (the train.txt of
 *                       apps/kge/data/preprocess.py:26-98 once mapped to ids).
 * `out`, h, r, t have id_bits-wide elements. */
KGE_API int kge_sample_uniform(void* out, int32_t id_bits, int64_t n, int64_t id_space, uint64_t seed, uint32_t stream_id,
                               kge_stream_t stream);
KGE_API int kge_sample_cdf(void* out, int32_t id_bits, int64_t n, const double* cdf, const int64_t* perm, int64_t n_items,
                           uint64_t seed, uint32_t stream_id, kge_stream_t stream);
KGE_API int kge_sample_triples(void* h, void* r, void* t, int32_t id_bits, int64_t n, const int64_t* triples, int64_t n_triples,
                               uint64_t seed, uint32_t stream_id, kge_stream_t stream);

/* ---- sparse optimizers ---------------------------------------------------------------------------------------
 * Update of exactly the rows a batch touched, from one gradient row per distinct id (the output of
 * kge_segment_reduce): for i < min(n, *n_dev) (n_dev may be NULL), row = ids[i] - first_row (row i when ids is NULL),
 *   kge_apply_sgd      table[row] -= lr * grad[i]
 *   kge_apply_adagrad  state[row] += grad[i]^2 (element-wise);  table[row] -= lr * grad[i] / (sqrt(state[row]) + eps)
 * table (rows, dim) fp32 or bf16 (updated in fp32, rounded to nearest even), state (rows, dim) fp32, grad (n, dim) fp32.
 * ids must be distinct.  No reference counterpart: the reference's backward_* functions (apps/kge/kge.py:393-515) stop
 * at per-triple gradient pieces. */
KGE_API int kge_apply_sgd(void* table, int32_t dtype, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                          int64_t first_row, const float* grad, float lr, kge_stream_t stream);
KGE_API int kge_apply_adagrad(void* table, int32_t dtype, float* state, int32_t dim, const int64_t* ids, int64_t n,
                              const int64_t* n_dev, int64_t first_row, const float* grad, float lr, float eps, kge_stream_t stream);

/* ---- measurement aid -----------------------------------------------------------------------------------
 * Launches `blocks` x 256 threads of independent fp32 FMA chains (iters x 128 FMAs per thread) and returns the
 * flop count (2 per FMA) in *flops_out; time it with CUDA events to get this GPU's attainable fp32 FMA rate,
 * the roofline denominator of the CUDA-core contraction kernels.  No counterpart in the reference. */
/* Live timing of the tensor-core tile kernel: after kge_profile_gemm(1) every launch of that kernel (up to 64 between
 * reads) is bracketed by CUDA events on its stream; kge_profile_gemm_read waits for them and returns the summed
 * duration, the number of launches and their useful flops (2 M N K per contraction), then resets the counters. */
KGE_API int kge_profile_gemm(int32_t enable);
KGE_API int kge_profile_gemm_read(double* ms, int64_t* launches, double* flops);

KGE_API int kge_probe_fma(float* out, int32_t blocks, int32_t iters, double* flops_out, kge_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KGE_B200_H */
