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
    long long k = lane;
    for (; k + 96 < row_units; k += 128) {
        const V a = src[k], b = src[k + 32], c = src[k + 64], d = src[k + 96];
        dst[k] = a; dst[k + 32] = b; dst[k + 64] = c; dst[k + 96] = d;
    }
    for (; k < row_units; k += 32) dst[k] = src[k];
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
