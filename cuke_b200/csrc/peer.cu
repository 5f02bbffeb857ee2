// Row-partitioned entity table across the GPUs of one node, read in place over NVLink.
//
// One process per GPU; rank g holds rows [g * rows_per_rank, (g + 1) * rows_per_rank).  Every rank exports its shard as a
// CUDA IPC handle once and maps the shards of the others, so a kernel on any GPU can address every row of the table:
// the staging gather of a batch (row uniq[u] -> row u of the compact buffer) then is ONE kernel that reads local rows
// from HBM and remote rows through NVSwitch with plain 16-byte loads, instead of an id exchange, a gather at each
// owner and an all-to-all of rows.  No TMA and no multicast: a remote row is fetched by the warp that owns the
// destination row and lands in local HBM, where every later kernel reads it.
//
// Ordering is the caller's: a rank may read a peer's rows only after that peer's last update of them has completed
// (a barrier among the ranks on the streams that carry the updates), and may update its own rows only after every
// peer's gather of the step has completed (implied when the update consumes gradients computed from gathered rows).
//
// The reference has no counterpart (single GPU, apps/kge/data/data_init.py:6-15).
#include <string.h>
#include "common.cuh"

namespace kge {

typedef int (*MemRangeFn)(unsigned long long* base, size_t* size, unsigned long long ptr);

static MemRangeFn mem_range_fn() {
    static MemRangeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<MemRangeFn>(p);
    }
    return fn;
}

// One warp per destination row; 16-byte units; four loads in flight per lane before the first store (a remote load takes
// a few microseconds, and the bytes in flight are what fills the link).
template <typename V>
__global__ void __launch_bounds__(256) gather_rows_peers_kernel(const void* const* shards, int world, long long rows_per_rank,
                                                                long long n_rows_total, long long row_units, const long long* ids,
                                                                long long n, const long long* n_dev, V* out, int32_t* err) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long cnt = n_dev ? min(n, *n_dev) : n;
    if (i >= cnt) return;
    const long long id = ids[i];
    if (id < 0 || id >= n_rows_total) {            // never dereference a row outside the table: flag and leave the row zero
        if (lane == 0) atomicOr(err, KGE_ERR_ID_RANGE);
        V* dst = out + i * row_units;
        const V z{};
        for (long long k = lane; k < row_units; k += 32) dst[k] = z;
        return;
    }
    const int owner = (int)(id / rows_per_rank);
    const V* src = static_cast<const V*>(shards[owner]) + (id - owner * rows_per_rank) * row_units;
    V* dst = out + i * row_units;
    for (long long k = lane; k < row_units; k += 128) {
        const bool pb = k + 32 < row_units, pc = k + 64 < row_units, pd = k + 96 < row_units;
        V a = src[k], b{}, c{}, d{};
        if (pb) b = src[k + 32];
        if (pc) c = src[k + 64];
        if (pd) d = src[k + 96];
        dst[k] = a;
        if (pb) dst[k + 32] = b;
        if (pc) dst[k + 64] = c;
        if (pd) dst[k + 96] = d;
    }
}

int launch_gather_rows_peers(const void* const* shards, int world, long long rows_per_rank, long long n_rows_total, int dtype, int dim,
                             const long long* ids, long long n, const long long* n_dev, void* out, cudaStream_t s) {
    if (n <= 0) return 0;
    const size_t row_bytes = (size_t)dim * (dtype == KGE_F32 ? 4 : 2);
    int32_t* err = device_error_word();
    if (!err) { set_error("no device error word"); return KGE_E_DEVICE; }
    const int wpb = 8;
    const unsigned blocks = (unsigned)((n + wpb - 1) / wpb);
    if (row_bytes % 16 == 0)
        gather_rows_peers_kernel<uint4><<<blocks, wpb * 32, 0, s>>>(shards, world, rows_per_rank, n_rows_total, (long long)(row_bytes / 16), ids, n, n_dev, static_cast<uint4*>(out), err);
    else if (row_bytes % 4 == 0)
        gather_rows_peers_kernel<unsigned><<<blocks, wpb * 32, 0, s>>>(shards, world, rows_per_rank, n_rows_total, (long long)(row_bytes / 4), ids, n, n_dev, static_cast<unsigned*>(out), err);
    else
        gather_rows_peers_kernel<unsigned short><<<blocks, wpb * 32, 0, s>>>(shards, world, rows_per_rank, n_rows_total, (long long)(row_bytes / 2), ids, n, n_dev, static_cast<unsigned short*>(out), err);
    KGE_LAUNCH_CHECK("gather_rows_peers_kernel");
    return 0;
}

// Owner-side sum of the gradient rows that the ranks hold for this rank's rows, read in place from their buffers.
// The ids requested by the ranks were concatenated in rank order (position pos of rank r: src_start[r] <= pos <
// src_start[r + 1]) and inspected: distinct id u owns the sorted positions [seg[u], seg[u + 1]) of perm.  Rank r keeps its
// gradient rows in the order of ITS sorted distinct ids, of which this owner's are the range starting at src_off[r]; so the
// row for position pos lives at bases[r] + (src_off[r] + pos - src_start[r]) * dim.  One warp per distinct id; at most one
// row per rank and id, added in rank order (perm is a stable sort): a fixed order, no atomics.  With sgd_table set the
// plain SGD step of the owner follows in the same pass: sgd_table[ids[u] - first_row] -= lr * sum (fp32 table).
__global__ void __launch_bounds__(256) pull_reduce_kernel(const float* const* bases, const long long* src_off, const long long* src_start,
                                                          int world, int dim, const int* perm, const int* seg, const long long* n_unique,
                                                          long long n_max, float* out, float* sgd_table, const long long* ids,
                                                          long long first_row, float lr) {
    const int lane = threadIdx.x & 31;
    const long long u = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (u >= min(n_max, *n_unique)) return;
    const int p0 = seg[u], p1 = seg[u + 1];
    float* dst = out + u * dim;
    float* trow = sgd_table ? sgd_table + (ids[u] - first_row) * dim : nullptr;
    const bool vec = (dim & 3) == 0;
    for (int k0 = 0; k0 < dim; k0 += 128) {                 // 128 floats per pass: one float4 per lane
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const int k = k0 + 4 * lane;
        for (int p = p0; p < p1; ++p) {
            const long long pos = perm[p];
            int r = 0;
            while (r + 1 < world && pos >= src_start[r + 1]) ++r;
            const float* row = bases[r] + (src_off[r] + pos - src_start[r]) * dim;
            if (vec) {
                if (k < dim) { const float4 x = *reinterpret_cast<const float4*>(row + k); acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w; }
            } else {
                if (k < dim) acc.x += row[k];
                if (k + 1 < dim) acc.y += row[k + 1];
                if (k + 2 < dim) acc.z += row[k + 2];
                if (k + 3 < dim) acc.w += row[k + 3];
            }
        }
        if (vec) {
            if (k < dim) {
                *reinterpret_cast<float4*>(dst + k) = acc;
                if (trow) {
                    float4 w = *reinterpret_cast<float4*>(trow + k);
                    w.x -= lr * acc.x; w.y -= lr * acc.y; w.z -= lr * acc.z; w.w -= lr * acc.w;
                    *reinterpret_cast<float4*>(trow + k) = w;
                }
            }
        } else {
            const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int e = 0; e < 4; ++e)
                if (k + e < dim) { dst[k + e] = a4[e]; if (trow) trow[k + e] -= lr * a4[e]; }
        }
    }
}

int launch_pull_reduce(const float* const* bases, const long long* src_off, const long long* src_start, int world, int dim,
                       const int* perm, const int* seg, const long long* n_unique, long long n_max, float* out, float* sgd_table,
                       const long long* ids, long long first_row, float lr, cudaStream_t s) {
    if (n_max <= 0) return 0;
    const int wpb = 8;
    pull_reduce_kernel<<<(unsigned)((n_max + wpb - 1) / wpb), wpb * 32, 0, s>>>(bases, src_off, src_start, world, dim, perm, seg, n_unique, n_max, out,
                                                                                sgd_table, ids, first_row, lr);
    KGE_LAUNCH_CHECK("pull_reduce_kernel");
    return 0;
}

// handle: 64 bytes (cudaIpcMemHandle_t) of the allocation that holds ptr; *offset: ptr's distance from its start.
int ipc_export(const void* ptr, void* handle, unsigned long long* offset) {
    MemRangeFn range = mem_range_fn();
    if (!range) { set_error("cuMemGetAddressRange is not available from this driver"); return KGE_E_DEVICE; }
    unsigned long long base = 0;
    size_t size = 0;
    const int r = range(&base, &size, (unsigned long long)(uintptr_t)ptr);
    if (r != 0) { set_error("cuMemGetAddressRange failed with CUresult %d", r); return KGE_E_DEVICE; }
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base));
    if (e != cudaSuccess) return cuda_status(e, "cudaIpcGetMemHandle");
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle, &h, 64);
    *offset = (unsigned long long)(uintptr_t)ptr - base;
    return 0;
}

int ipc_open(const void* handle, unsigned long long offset, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_status(e, "cudaIpcOpenMemHandle");
    *out = static_cast<char*>(base) + offset;
    return 0;
}

int ipc_close(void* ptr, unsigned long long offset) {
    cudaError_t e = cudaIpcCloseMemHandle(static_cast<char*>(ptr) - offset);
    if (e != cudaSuccess) return cuda_status(e, "cudaIpcCloseMemHandle");
    return 0;
}

}  // namespace kge
