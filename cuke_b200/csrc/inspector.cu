// GPU inspector and the kernels driven by its output.
//
// The reference's inspector (apps/kge/inspection/inspector.cu:68-136) sorts each chunk of 16 relation ids
// with a bitonic network and caches the two most frequent ids; the global order comes from a host-side
// torch.argsort (apps/kge/test_cuke.py:93-96).  Here one pass over ALL ids of a batch produces the sorted
// distinct ids, the inverse map, the stable sort permutation and segment offsets:
//   - LSD radix sort, 8 bits per pass, three kernels per pass (histogram, scan, stable scatter).  No CTA
//     ever waits on another CTA: ordering between the phases is the kernel boundary.
//   - adjacent-difference flags + two-level scan -> uniq / seg / inverse.
// The segmented reduction turns per-slot gradient rows into one row per distinct id in a fixed order
// (no atomics), and gather_rows stages each distinct row once.
#include "rows.cuh"

namespace kge {

constexpr int RS_THREADS = 256;
constexpr int RS_MAX_BLOCKS = 2048;

struct Tiling { int ipt; int tile; int blocks; };
static inline Tiling tiling_for(long long n) {
    Tiling t;
    long long ipt = 8;
    long long need = (n + (long long)RS_MAX_BLOCKS * RS_THREADS - 1) / ((long long)RS_MAX_BLOCKS * RS_THREADS);
    if (need > ipt) ipt = need;
    t.ipt = (int)ipt;
    t.tile = t.ipt * RS_THREADS;
    t.blocks = (int)((n + t.tile - 1) / t.tile);
    if (t.blocks < 1) t.blocks = 1;
    return t;
}

// ---- block-wide inclusive scan (blockDim.x <= 1024, multiple of 32) ------------------------------------
__device__ __forceinline__ int block_inclusive_scan(int v, int* warp_tot /* smem[33] */, int& block_total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(kFull, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();                      // protects warp_tot reuse across calls
    if (lane == 31) warp_tot[w] = v;
    __syncthreads();
    if (w == 0) {
        int t = lane < nw ? warp_tot[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int u = __shfl_up_sync(kFull, t, o);
            if (lane >= o) t += u;
        }
        warp_tot[lane] = t;               // inclusive totals of warps
        if (lane == 31) warp_tot[32] = t;
    }
    __syncthreads();
    block_total = warp_tot[32];
    return v + (w > 0 ? warp_tot[w - 1] : 0);
}

// ---- radix sort -------------------------------------------------------------------------------------
template <typename I>
__global__ void ids_to_keys_kernel(const void* ids, long long n, unsigned* keys) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) keys[i] = (unsigned)load_id<I>(ids, i);
}

// Range check with an optional sanitised copy (ids outside [0, limit) become 0).
template <typename I>
__global__ void validate_ids_kernel(const void* ids, long long n, long long limit, void* out, int32_t* err) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    long long v = static_cast<long long>(reinterpret_cast<const I*>(ids)[i]);
    if (v < 0 || v >= limit) { atomicOr(err, KGE_ERR_ID_RANGE); v = 0; }
    if (out) reinterpret_cast<I*>(out)[i] = static_cast<I>(v);
}
int launch_validate_ids(const void* ids, int id_bits, long long n, long long limit, void* out, cudaStream_t s) {
    if (n <= 0) return 0;
    int32_t* err = device_error_word();
    if (!err) { set_error("no device error word"); return KGE_E_DEVICE; }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (id_bits == 64) validate_ids_kernel<int64_t><<<blocks, 256, 0, s>>>(ids, n, limit, out, err);
    else validate_ids_kernel<int32_t><<<blocks, 256, 0, s>>>(ids, n, limit, out, err);
    KGE_LAUNCH_CHECK("validate_ids_kernel");
    return 0;
}

__global__ void __launch_bounds__(RS_THREADS) radix_hist_kernel(const unsigned* keys, long long n, int shift, int ipt,
                                                                unsigned* hist, int nblocks) {
    __shared__ unsigned h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * ipt * RS_THREADS;
    for (int r = 0; r < ipt; ++r) {
        long long i = base + (long long)r * RS_THREADS + threadIdx.x;
        if (i < n) atomicAdd(&h[(keys[i] >> shift) & 255u], 1u);
    }
    __syncthreads();
    hist[(long long)threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];
}

// Exclusive scan of `total` unsigned counters by ONE block of 1024 threads (total <= 256 * 2048).  Each warp owns a
// contiguous span (a multiple of 32 counters) and reads it 32 counters at a time, lane = consecutive counter: pass 1 sums
// the spans, the 32 span totals are scanned, pass 2 rewrites each span with its running prefix.  Four groups are
// requested before the first is used, so a span costs a few memory round trips instead of one per counter.
__global__ void __launch_bounds__(1024) scan_exclusive_kernel(unsigned* data, int total, long long* total_out) {
    __shared__ int span_tot[32];
    __shared__ int span_off[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int groups = (total + 31) / 32;                         // groups of 32 counters
    const int gpw = (groups + 31) / 32;                           // groups per warp
    const int g0 = w * gpw, g1 = min(groups, g0 + gpw);
    int s = 0;
    for (int g = g0; g < g1; g += 4) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const int i = (g + u) * 32 + lane; v[u] = (g + u < g1 && i < total) ? (int)data[i] : 0; }
        s += (v[0] + v[1]) + (v[2] + v[3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
    if (lane == 0) span_tot[w] = s;
    __syncthreads();
    if (w == 0) {
        const int t = span_tot[lane];
        int incl = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += y; }
        span_off[lane] = incl - t;
        if (lane == 31 && total_out) *total_out = incl;
    }
    __syncthreads();
    int run = span_off[w];
    for (int g = g0; g < g1; g += 4) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const int i = (g + u) * 32 + lane; v[u] = (g + u < g1 && i < total) ? (int)data[i] : 0; }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            int incl = v[u];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += y; }
            const int i = (g + u) * 32 + lane;
            if (g + u < g1 && i < total) data[i] = (unsigned)(run + incl - v[u]);
            run += __shfl_sync(kFull, incl, 31);
        }
    }
}

__global__ void __launch_bounds__(RS_THREADS) radix_scatter_kernel(const unsigned* keys_in, const int* vals_in,
                                                                   unsigned* keys_out, int* vals_out, long long n,
                                                                   int shift, int ipt, const unsigned* hist, int nblocks) {
    __shared__ unsigned base[256];
    __shared__ unsigned running[256];
    __shared__ unsigned short warp_cnt[RS_THREADS / 32][256];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    base[tid] = hist[(long long)tid * nblocks + blockIdx.x];
    running[tid] = 0;
#pragma unroll
    for (int q = 0; q < RS_THREADS / 32; ++q) warp_cnt[q][tid] = 0;
    __syncthreads();
    const long long tile0 = (long long)blockIdx.x * ipt * RS_THREADS;
    for (int r = 0; r < ipt; ++r) {
        const long long i = tile0 + (long long)r * RS_THREADS + tid;
        const bool valid = i < n;
        unsigned key = 0; int val = 0; unsigned d = 256u;          // 256 = "no item" group
        if (valid) { key = keys_in[i]; val = vals_in ? vals_in[i] : (int)i; d = (key >> shift) & 255u; }
        const unsigned peers = __match_any_sync(kFull, d);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (valid && rank == 0) warp_cnt[w][d] = (unsigned short)__popc(peers);
        __syncthreads();
        if (valid) {
            unsigned off = running[d] + rank;
            for (int q = 0; q < w; ++q) off += warp_cnt[q][d];
            const long long pos = (long long)base[d] + off;
            keys_out[pos] = key;
            vals_out[pos] = val;
        }
        __syncthreads();
        {   // thread `tid` owns digit `tid`: fold this pass's counts into the running offset and clear them
            unsigned t = 0;
#pragma unroll
            for (int q = 0; q < RS_THREADS / 32; ++q) { t += warp_cnt[q][tid]; warp_cnt[q][tid] = 0; }
            running[tid] += t;
        }
        __syncthreads();
    }
}

// ---- unique -------------------------------------------------------------------------------------------
// Pass A: per tile, inclusive scan of "starts a new run" flags; tile totals to bsum.
__global__ void __launch_bounds__(RS_THREADS) unique_flags_kernel(const unsigned* keys, long long n, int ipt,
                                                                  int* local_incl, unsigned* bsum) {
    __shared__ int warp_tot[33];
    const long long tile0 = (long long)blockIdx.x * ipt * RS_THREADS;
    int carry = 0;
    for (int r = 0; r < ipt; ++r) {
        const long long i = tile0 + (long long)r * RS_THREADS + threadIdx.x;
        int f = 0;
        if (i < n) f = (i == 0) ? 1 : (keys[i] != keys[i - 1]);
        int tot;
        int incl = block_inclusive_scan(f, warp_tot, tot);
        if (i < n) local_incl[i] = carry + incl;
        carry += tot;
    }
    if (threadIdx.x == 0) bsum[blockIdx.x] = (unsigned)carry;
}
// Pass B (after scan_exclusive_kernel over bsum): write uniq / seg / inverse.
__global__ void __launch_bounds__(RS_THREADS) unique_apply_kernel(const unsigned* keys, const int* perm, long long n, int ipt,
                                                                  const int* local_incl, const unsigned* bsum_excl,
                                                                  const long long* n_unique,
                                                                  long long* uniq, int* inverse, int* seg) {
    const long long tile0 = (long long)blockIdx.x * ipt * RS_THREADS;
    const int off = (int)bsum_excl[blockIdx.x];
    const long long U = *n_unique;
    for (int r = 0; r < ipt; ++r) {
        const long long i = tile0 + (long long)r * RS_THREADS + threadIdx.x;
        if (i >= n) break;
        const int g = off + local_incl[i] - 1;
        const bool first = (i == 0) || (keys[i] != keys[i - 1]);
        if (first) { uniq[g] = (long long)keys[i]; seg[g] = (int)i; }
        inverse[perm[i]] = g;
        if (i >= U) seg[i] = (int)n;
        if (i == n - 1) seg[n] = (int)n;
    }
}

// ---- segmented reduction -------------------------------------------------------------------------------
// Window = 32 consecutive sorted positions, one warp per window.  A segment that lies inside one window is
// finished there; a segment that crosses window boundaries leaves one partial row per window ("trail" in
// its first window, "lead" in every later one), summed in window order by segred_span_kernel.
// Largest u in [0, U) with seg[u] <= p, found by the whole warp: every round the 32 lanes probe 32 evenly spaced
// entries at once, so the search is log32(U) dependent loads deep instead of log2(U).  seg[0] == 0 <= p always holds.
__device__ __forceinline__ int seg_of_position(const int* seg, int U, int p, int lane) {
    int lo = 0, hi = U - 1;
    while (hi - lo >= 32) {
        const int step = (hi - lo + 32) >> 5;                  // ceil((hi - lo + 1) / 32)
        const int idx = lo + lane * step;
        const bool ok = idx <= hi && seg[idx] <= p;            // true for lanes 0 .. k, false above
        const int k = __popc(__ballot_sync(kFull, ok)) - 1;
        lo += k * step;
        hi = min(hi, lo + step - 1);
    }
    const int idx = lo + lane;
    const bool ok = idx <= hi && seg[idx] <= p;
    return lo + __popc(__ballot_sync(kFull, ok)) - 1;
}

template <int NV, bool VEC>
__global__ void __launch_bounds__(256) segred_window_kernel(const float* rows, int dim, long long n, const int* perm,
                                                            const int* seg, const long long* n_unique, float* out,
                                                            float* lead, float* trail) {
    const int lane = threadIdx.x & 31;
    const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long p0 = wi * 32;
    if (p0 >= n) return;
    const int p1 = (int)min(n, p0 + 32);
    const int U = (int)*n_unique;
    int cur = seg_of_position(seg, U, (int)p0, lane);
    int cur_end = seg[cur + 1];
    const int my = (p0 + lane < n) ? perm[p0 + lane] : 0;
    Row<NV> acc;
    row_zero<NV>(acc);
    // four rows are requested before the first of them is added: the adds (and the stores at segment ends) stay in
    // position order, the memory latency of the gathered rows overlaps
    for (int pb = (int)p0; pb < p1; pb += 4) {
        Row<NV> x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int src = __shfl_sync(kFull, my, min(pb + u, p1 - 1) - (int)p0);
            if (pb + u < p1) load_row_f32<NV, VEC>(x[u], rows + (long long)src * dim, dim, lane);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int p = pb + u;
            if (p >= p1) break;
#pragma unroll
            for (int q = 0; q < NV; ++q) acc.v[q] = acc.v[q] + x[u].v[q];
            if (p + 1 == cur_end || p + 1 == p1) {
                const int s = seg[cur];
                float* dst;
                if (s >= (int)p0 && cur_end <= p1) dst = out + (long long)cur * dim;       // whole segment in this window
                else if (s < (int)p0) dst = lead + wi * dim;                              // continues from the left
                else dst = trail + wi * dim;                                              // continues to the right
                store_row<NV, VEC>(dst, acc, dim, lane);
                row_zero<NV>(acc);
                if (p + 1 == cur_end && p + 1 < p1) { ++cur; cur_end = seg[cur + 1]; }
            }
        }
    }
}

// One CTA per window boundary b (between windows b and b+1): if a segment crosses it and starts in window b, the
// CTA sums trail[b] + lead[b+1] + ... + lead[last].  Warp w takes parts w, w+8, ... in order, then warp 0 adds the
// eight partial rows in order: a fixed summation order, and the hottest row of a Zipf batch (hundreds of windows)
// is spread over eight warps instead of one.
template <int NV, bool VEC>
__global__ void __launch_bounds__(256) segred_span_kernel(int dim, long long n, const int* seg, const long long* n_unique,
                                                          float* out, const float* lead, const float* trail) {
    extern __shared__ __align__(16) float part[];          // 8 x dim
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const long long b = blockIdx.x;
    const long long edge = (b + 1) * 32;            // first position of window b+1
    if (edge >= n) return;
    const int U = (int)*n_unique;
    const int u = seg_of_position(seg, U, (int)edge - 1, lane);
    const int s = seg[u], e = seg[u + 1];
    if (e <= edge || s < b * 32) return;            // does not cross here, or started in an earlier window (block-uniform)
    const long long parts = (e - 1) / 32 - b + 1;   // part 0 = trail[b], part k = lead[b + k]
    Row<NV> acc;
    row_zero<NV>(acc);
    // four parts are requested before the first is added (same order of additions): the hottest row of a Zipf batch has
    // hundreds of parts, and its chain of dependent loads would otherwise set the duration of the whole launch
    for (long long k = w; k < parts; k += 32) {
        Row<NV> x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long kk = k + 8 * u;
            if (kk < parts) load_row_f32<NV, VEC>(x[u], (kk == 0 ? trail + b * dim : lead + (b + kk) * dim), dim, lane);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (k + 8 * u < parts) {
#pragma unroll
                for (int q = 0; q < NV; ++q) acc.v[q] = acc.v[q] + x[u].v[q];
            }
        }
    }
    store_row<NV, VEC>(part + w * dim, acc, dim, lane);
    __syncthreads();
    if (w == 0) {      // shared-memory reads: plain loads (the row helpers use the read-only global path)
        row_zero<NV>(acc);
        for (int k = 0; k < 8; ++k) {
            const float* pr = part + k * dim;
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                const int e0 = 4 * (lane + 32 * q);
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e0 + 0 < dim) v.x = pr[e0 + 0];
                if (e0 + 1 < dim) v.y = pr[e0 + 1];
                if (e0 + 2 < dim) v.z = pr[e0 + 2];
                if (e0 + 3 < dim) v.w = pr[e0 + 3];
                acc.v[q] = acc.v[q] + v;
            }
        }
        store_row<NV, VEC>(out + (long long)u * dim, acc, dim, lane);
    }
}

__global__ void zero_tail_rows_kernel(float* out, int dim, const long long* n_unique, long long n_out) {
    const long long U = *n_unique;
    const long long total = (n_out - U) * dim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        out[U * dim + i] = 0.f;
}

// ---- gather rows ------------------------------------------------------------------------------------------
template <typename V>
__global__ void __launch_bounds__(256) gather_rows_kernel(const V* table, long long row_units, const long long* ids,
                                                          long long n, const long long* n_dev, long long first_row, V* out) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long cnt = n_dev ? min(n, *n_dev) : n;
    if (i >= cnt) return;
    const V* src = table + (ids[i] - first_row) * row_units;
    V* dst = out + i * row_units;
    for (long long k = lane; k < row_units; k += 32) dst[k] = __ldg(src + k);
}

// out[ids[i] - first_row][:] = rows[i][:] for i < min(n, *n_dev): places compact rows into a dense table.
__global__ void __launch_bounds__(256) scatter_rows_kernel(const float* rows, int dim, const long long* ids, long long n,
                                                           const long long* n_dev, long long first_row, float* out) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long cnt = n_dev ? min(n, *n_dev) : n;
    if (i >= cnt) return;
    const float* src = rows + i * dim;
    float* dst = out + (ids[i] - first_row) * dim;
    for (int k = lane; k < dim; k += 32) dst[k] = src[k];
}

// Measurement aid: dependent-free FMA chains, 8 accumulators per thread; reports nothing but keeps the result live.
__global__ void __launch_bounds__(256) fma_probe_kernel(float* out, int iters) {
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = threadIdx.x * 1e-3f + i;
    const float x = 1.0000001f, y = 1e-7f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < 16; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = fmaf(a[i], x, y);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += a[i];
    if (s == 12345.678f) out[0] = s;
}

__global__ void owner_counts_kernel(const long long* uniq, const long long* n_unique, long long n_max,
                                    long long rows_per_rank, int world, long long* counts) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= world) return;
    const long long U = min(*n_unique, n_max);
    auto lower = [&](long long key) {   // first index with uniq[idx] >= key
        long long lo = 0, hi = U;
        while (lo < hi) { long long mid = (lo + hi) >> 1; if (uniq[mid] < key) lo = mid + 1; else hi = mid; }
        return lo;
    };
    const long long a = lower((long long)g * rows_per_rank);
    const long long b = (g == world - 1) ? U : lower((long long)(g + 1) * rows_per_rank);
    counts[g] = b - a;
}

// ---- legacy per-16 inspector ------------------------------------------------------------------------------
// Same outputs as build_index (apps/kge/inspection/inspector.cu:68-136); one thread per chunk, everything in
// registers/local memory, so none of the reference's unsynchronised shared-memory steps exist here.
__global__ void legacy_inspect_kernel(const long long* rel, long long nchunks, long long rel_num,
                                      long long* uniq, long long* buf, long long* cnt) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nchunks) return;
    constexpr int C = 16, T = 2;
    int idx[C], src[C];
    for (int i = 0; i < C; ++i) { idx[i] = (int)rel[b * C + i]; src[i] = i; }
    for (int i = 1; i < C; ++i) {                      // insertion sort (ascending), carrying origins
        int k = idx[i], s = src[i], j = i - 1;
        while (j >= 0 && idx[j] > k) { idx[j + 1] = idx[j]; src[j + 1] = src[j]; --j; }
        idx[j + 1] = k; src[j + 1] = s;
    }
    int grp[C], pcount[C + 1], count[C], idx_count[C], ord_uniq[C];
    for (int i = 0; i <= C; ++i) pcount[i] = 0;
    grp[0] = 0;
    for (int i = 1; i < C; ++i) grp[i] = grp[i - 1] + (idx[i] > idx[i - 1] ? 1 : 0);
    pcount[grp[C - 1] + 1] = C;
    for (int i = 1; i < C; ++i) if (idx[i] > idx[i - 1]) pcount[grp[i]] = i;
    for (int i = 0; i < C; ++i) { count[i] = -1; idx_count[i] = -1; ord_uniq[i] = i; }
    for (int i = 1; i < C; ++i)
        if (pcount[i] - pcount[i - 1] > 0) { count[i - 1] = pcount[i] - pcount[i - 1]; idx_count[i - 1] = pcount[i] - 1; }
    auto swp = [&](int x, int y) {
        int t = count[x]; count[x] = count[y]; count[y] = t;
        t = idx_count[x]; idx_count[x] = idx_count[y]; idx_count[y] = t;
        t = ord_uniq[x]; ord_uniq[x] = ord_uniq[y]; ord_uniq[y] = t;
    };
    for (int s = C / 2; s > 0; s >>= 1)
        for (int i = 0; i < s; ++i) if (count[i] < count[i + s]) swp(i, i + s);
    if (count[1] < count[2]) swp(1, 2);
    long long iuniq[C];
    for (int i = 0; i < C; ++i) iuniq[i] = rel_num;
    for (int i = 0; i < T; ++i) if (count[i] > T - 1) iuniq[i] = idx[idx_count[i]];
    long long slot[C];
    for (int i = 0; i < C; ++i) {
        if (grp[i] == ord_uniq[0] && iuniq[0] < rel_num) slot[i] = 0;
        else if (grp[i] == ord_uniq[1] && iuniq[1] < rel_num) slot[i] = 1;
        else slot[i] = (long long)idx[i] + C;
    }
    for (int i = 0; i + 1 < C; ++i) if (iuniq[i] < rel_num && iuniq[i + 1] == rel_num) cnt[b] = i + 1;
    for (int i = 0; i < C; ++i) { buf[b * C + src[i]] = slot[i]; uniq[b * C + i] = iuniq[i]; }
}

// ---- logistic loss ------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(256) loss_partial_kernel(const float* pos, long long n_pos, const float* neg, long long n_neg,
                                                           float neg_w, float* dpos, float* dneg, float* partial) {
    __shared__ float red[256];
    // each block owns a contiguous slice of quads of `neg` (and of `pos`), so the partial sums have a fixed order
    const bool vec = (n_neg % 4 == 0) && ((reinterpret_cast<uintptr_t>(neg) | reinterpret_cast<uintptr_t>(dneg)) & 15u) == 0;
    float s = 0.f;
    {
        const long long per = (n_pos + gridDim.x - 1) / gridDim.x;
        const long long lo = (long long)blockIdx.x * per, hi = min(n_pos, lo + per);
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) { const float x = pos[i]; s += softplusf(-x); dpos[i] = -sigmoidf(-x); }
    }
    if (vec) {
        const long long nq = n_neg / 4;
        const long long per = (nq + gridDim.x - 1) / gridDim.x;
        const long long lo = (long long)blockIdx.x * per, hi = min(nq, lo + per);
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(neg) + i);
            s += neg_w * ((softplusf(x.x) + softplusf(x.y)) + (softplusf(x.z) + softplusf(x.w)));
            reinterpret_cast<float4*>(dneg)[i] = make_float4(neg_w * sigmoidf(x.x), neg_w * sigmoidf(x.y), neg_w * sigmoidf(x.z), neg_w * sigmoidf(x.w));
        }
    } else {
        const long long per = (n_neg + gridDim.x - 1) / gridDim.x;
        const long long lo = (long long)blockIdx.x * per, hi = min(n_neg, lo + per);
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) { const float x = neg[i]; s += neg_w * softplusf(x); dneg[i] = neg_w * sigmoidf(x); }
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}
__global__ void __launch_bounds__(256) loss_final_kernel(const float* partial, int n, float* loss) {
    __shared__ float red[256];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) *loss = red[0];
}

// ======================================================================================================
// host side
// ======================================================================================================
static inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

struct InspectLayout {
    size_t keys_a, keys_b, vals_a, vals_b, hist, local, bsum, total;
};
static InspectLayout inspect_layout(long long n) {
    Tiling t = tiling_for(n);
    InspectLayout L;
    size_t off = 0;
    L.keys_a = off; off += align_up((size_t)n * 4);
    L.keys_b = off; off += align_up((size_t)n * 4);
    L.vals_a = off; off += align_up((size_t)n * 4);
    L.vals_b = off; off += align_up((size_t)n * 4);
    L.hist = off; off += align_up((size_t)256 * t.blocks * 4);
    L.local = off; off += align_up((size_t)n * 4);
    L.bsum = off; off += align_up((size_t)(t.blocks + 1) * 4);
    L.total = off;
    return L;
}

size_t inspect_workspace_bytes(long long n) { return inspect_layout(n < 1 ? 1 : n).total; }

int launch_inspect(const void* ids, int id_bits, long long n, long long id_space, void* ws, size_t ws_bytes,
                   long long* uniq, int* inverse, int* perm, int* seg, long long* n_unique, cudaStream_t s) {
    if (n == 0) {
        cudaError_t e = cudaMemsetAsync(n_unique, 0, sizeof(long long), s);
        if (e == cudaSuccess) e = cudaMemsetAsync(seg, 0, sizeof(int), s);
        return cuda_status(e, "inspect(n=0)");
    }
    InspectLayout L = inspect_layout(n);
    if (ws_bytes < L.total) { set_error("inspect workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* base = static_cast<char*>(ws);
    unsigned* keys[2] = {reinterpret_cast<unsigned*>(base + L.keys_a), reinterpret_cast<unsigned*>(base + L.keys_b)};
    int* vals[2] = {reinterpret_cast<int*>(base + L.vals_a), reinterpret_cast<int*>(base + L.vals_b)};
    unsigned* hist = reinterpret_cast<unsigned*>(base + L.hist);
    int* local = reinterpret_cast<int*>(base + L.local);
    unsigned* bsum = reinterpret_cast<unsigned*>(base + L.bsum);
    const Tiling t = tiling_for(n);

    const unsigned cb = (unsigned)((n + 255) / 256);
    if (id_bits == 64) ids_to_keys_kernel<int64_t><<<cb, 256, 0, s>>>(ids, n, keys[0]);
    else ids_to_keys_kernel<int32_t><<<cb, 256, 0, s>>>(ids, n, keys[0]);
    KGE_LAUNCH_CHECK("ids_to_keys_kernel");

    int bits = 1;
    while (bits < 32 && ((long long)1 << bits) < id_space) ++bits;
    const int passes = (bits + 7) / 8;
    int cur = 0;
    for (int p = 0; p < passes; ++p) {
        const int shift = 8 * p;
        const bool last = (p == passes - 1);
        radix_hist_kernel<<<t.blocks, RS_THREADS, 0, s>>>(keys[cur], n, shift, t.ipt, hist, t.blocks);
        KGE_LAUNCH_CHECK("radix_hist_kernel");
        scan_exclusive_kernel<<<1, 1024, 0, s>>>(hist, 256 * t.blocks, nullptr);
        KGE_LAUNCH_CHECK("scan_exclusive_kernel");
        int* vout = last ? perm : vals[cur ^ 1];
        const int* vin = (p == 0) ? nullptr : vals[cur];
        radix_scatter_kernel<<<t.blocks, RS_THREADS, 0, s>>>(keys[cur], vin, keys[cur ^ 1], vout, n, shift, t.ipt, hist, t.blocks);
        KGE_LAUNCH_CHECK("radix_scatter_kernel");
        cur ^= 1;
    }
    unique_flags_kernel<<<t.blocks, RS_THREADS, 0, s>>>(keys[cur], n, t.ipt, local, bsum);
    KGE_LAUNCH_CHECK("unique_flags_kernel");
    scan_exclusive_kernel<<<1, 1024, 0, s>>>(bsum, t.blocks, n_unique);
    KGE_LAUNCH_CHECK("scan_exclusive_kernel(bsum)");
    unique_apply_kernel<<<t.blocks, RS_THREADS, 0, s>>>(keys[cur], perm, n, t.ipt, local, bsum, n_unique, uniq, inverse, seg);
    KGE_LAUNCH_CHECK("unique_apply_kernel");
    return 0;
}

size_t segment_reduce_workspace_bytes(long long n, int dim) {
    const long long nwin = (n + 31) / 32;
    return align_up((size_t)nwin * dim * 4) * 2;
}

template <int NV, bool VEC>
static int segred_go(const float* rows, int dim, long long n, const int* perm, const int* seg, const long long* n_unique,
                     float* out, long long n_out, float* lead, float* trail, cudaStream_t s) {
    const long long nwin = (n + 31) / 32;
    const int wpb = 8;
    const unsigned blocks = (unsigned)((nwin + wpb - 1) / wpb);
    segred_window_kernel<NV, VEC><<<blocks, wpb * 32, 0, s>>>(rows, dim, n, perm, seg, n_unique, out, lead, trail);
    KGE_LAUNCH_CHECK("segred_window_kernel");
    if (nwin > 1) {
        segred_span_kernel<NV, VEC><<<(unsigned)(nwin - 1), 256, 8 * dim * sizeof(float), s>>>(dim, n, seg, n_unique, out, lead, trail);
        KGE_LAUNCH_CHECK("segred_span_kernel");
    }
    if (n_out > 0) {
        zero_tail_rows_kernel<<<296, 256, 0, s>>>(out, dim, n_unique, n_out);
        KGE_LAUNCH_CHECK("zero_tail_rows_kernel");
    }
    return 0;
}

int launch_segment_reduce(const float* rows, int dim, long long n, const int* perm, const int* seg,
                          const long long* n_unique, float* out, long long n_out, void* ws, size_t ws_bytes,
                          cudaStream_t s) {
    if (n == 0) {
        if (n_out > 0) return cuda_status(cudaMemsetAsync(out, 0, (size_t)n_out * dim * 4, s), "segment_reduce(n=0)");
        return 0;
    }
    const size_t need = segment_reduce_workspace_bytes(n, dim);
    if (ws_bytes < need) { set_error("segment_reduce workspace: need %zu bytes, got %zu", need, ws_bytes); return KGE_E_WORKSPACE; }
    float* lead = static_cast<float*>(ws);
    float* trail = reinterpret_cast<float*>(static_cast<char*>(ws) + need / 2);
    const bool vec = dim % 4 == 0;
    const int nv = quads_per_lane(dim);
    if (nv == 0) { set_error("dim %d > 1024 is not supported", dim); return KGE_E_UNSUPPORTED; }
#define KGE_SR(N) case N: return vec ? segred_go<N, true>(rows, dim, n, perm, seg, n_unique, out, n_out, lead, trail, s) \
                                     : segred_go<N, false>(rows, dim, n, perm, seg, n_unique, out, n_out, lead, trail, s);
    switch (nv) { KGE_SR(1) KGE_SR(2) KGE_SR(4) KGE_SR(8) }
#undef KGE_SR
    return KGE_E_UNSUPPORTED;
}

int launch_gather_rows(const void* table, int dtype, int dim, const long long* ids, long long n, const long long* n_dev,
                       long long first_row, void* out, cudaStream_t s) {
    if (n <= 0) return 0;
    const size_t row_bytes = (size_t)dim * (dtype == KGE_F32 ? 4 : 2);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((n + wpb - 1) / wpb);
    if (row_bytes % 16 == 0)
        gather_rows_kernel<uint4><<<blocks, wpb * 32, 0, s>>>(static_cast<const uint4*>(table), (long long)(row_bytes / 16), ids, n, n_dev, first_row, static_cast<uint4*>(out));
    else if (row_bytes % 4 == 0)
        gather_rows_kernel<unsigned><<<blocks, wpb * 32, 0, s>>>(static_cast<const unsigned*>(table), (long long)(row_bytes / 4), ids, n, n_dev, first_row, static_cast<unsigned*>(out));
    else
        gather_rows_kernel<unsigned short><<<blocks, wpb * 32, 0, s>>>(static_cast<const unsigned short*>(table), (long long)(row_bytes / 2), ids, n, n_dev, first_row, static_cast<unsigned short*>(out));
    KGE_LAUNCH_CHECK("gather_rows_kernel");
    return 0;
}

int launch_scatter_rows(const float* rows, int dim, const long long* ids, long long n, const long long* n_dev,
                        long long first_row, float* out, cudaStream_t s) {
    if (n <= 0) return 0;
    const int wpb = 8;
    scatter_rows_kernel<<<(unsigned)((n + wpb - 1) / wpb), wpb * 32, 0, s>>>(rows, dim, ids, n, n_dev, first_row, out);
    KGE_LAUNCH_CHECK("scatter_rows_kernel");
    return 0;
}

int launch_fma_probe(float* out, int blocks, int iters, cudaStream_t s) {
    fma_probe_kernel<<<blocks, 256, 0, s>>>(out, iters);
    KGE_LAUNCH_CHECK("fma_probe_kernel");
    return 0;
}

int launch_owner_counts(const long long* uniq, const long long* n_unique, long long n_max, long long rows_per_rank,
                        int world, long long* counts, cudaStream_t s) {
    owner_counts_kernel<<<(world + 63) / 64, 64, 0, s>>>(uniq, n_unique, n_max, rows_per_rank, world, counts);
    KGE_LAUNCH_CHECK("owner_counts_kernel");
    return 0;
}

int launch_legacy_inspect(const long long* rel, long long n, long long rel_num, long long* uniq, long long* buf,
                          long long* cnt, cudaStream_t s) {
    const long long nchunks = n / 16;
    if (nchunks <= 0) return 0;
    legacy_inspect_kernel<<<(unsigned)((nchunks + 127) / 128), 128, 0, s>>>(rel, nchunks, rel_num, uniq, buf, cnt);
    KGE_LAUNCH_CHECK("legacy_inspect_kernel");
    return 0;
}

int launch_logistic_loss(const float* pos, long long n_pos, const float* neg, long long n_neg, float neg_w, float* dpos,
                         float* dneg, float* loss, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (ws_bytes < 4096) { set_error("logistic_loss workspace: need 4096 bytes, got %zu", ws_bytes); return KGE_E_WORKSPACE; }
    float* partial = static_cast<float*>(ws);
    const int blocks = 1024;
    loss_partial_kernel<<<blocks, 256, 0, s>>>(pos, n_pos, neg, n_neg, neg_w, dpos, dneg, partial);
    KGE_LAUNCH_CHECK("loss_partial_kernel");
    loss_final_kernel<<<1, 256, 0, s>>>(partial, blocks, loss);
    KGE_LAUNCH_CHECK("loss_final_kernel");
    return 0;
}


// ---- segmented reduction with library-owned scratch -----------------------------------------------------------
// Scratch of kge_segment_reduce_static: two halves (lead / trail partial rows), resident on every GPU that loads
// the library for the life of the process.
constexpr long long kStaticHalfFloats = 1LL << 20;            // 4 MiB per half, 8 MiB in total
static __device__ __align__(256) float g_segred_static[2 * kStaticHalfFloats];

// In host code `g_segred_static` is only a handle for the runtime, not a device address: the address the
// kernels need is looked up once per device (with that device current) and remembered.
static float* g_static_base[128] = {nullptr};

static int static_scratch(float** base) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "kge_segment_reduce_static: cudaGetDevice");
    if (dev < 0 || dev >= 128) { set_error("kge_segment_reduce_static: device ordinal %d outside [0, 128)", dev); return KGE_E_DEVICE; }
    if (g_static_base[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_segred_static);
        if (e != cudaSuccess) return cuda_status(e, "kge_segment_reduce_static: cudaGetSymbolAddress");
        g_static_base[dev] = p;
    }
    *base = g_static_base[dev];
    return 0;
}

}  // namespace kge

extern "C" int kge_segment_reduce_static(const float* rows, int32_t dim, int64_t n, const int32_t* perm, const int32_t* seg,
                                         const int64_t* n_unique, float* out, int64_t n_out, kge_stream_t stream) {
    using namespace kge;
    const char* fn = "kge_segment_reduce_static";
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (n < 0 || n > 2147483647LL || n_out < 0) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (dim <= 0 || dim > 1024) { set_error("%s: dim %d outside [1, 1024]", fn, dim); return KGE_E_UNSUPPORTED; }
    const long long nwin = (n + 31) / 32;
    if (nwin * dim > kStaticHalfFloats) {
        set_error("%s: ceil(n/32) * dim = %lld exceeds the built-in scratch of %lld floats per half "
                  "(n = %lld, dim = %d); use kge_segment_reduce with a caller-provided workspace",
                  fn, nwin * dim, kStaticHalfFloats, (long long)n, dim);
        return KGE_E_RANGE;
    }
    // `out` receives rows whenever there is anything to reduce (n > 0) or to zero-fill (n_out > 0)
    const void* ptrs[] = {(n_out > 0 || n > 0) ? out : (float*)16, n > 0 ? (const void*)rows : (const void*)16,
                          n > 0 ? (const void*)perm : (const void*)16, n > 0 ? (const void*)seg : (const void*)16,
                          n > 0 ? (const void*)n_unique : (const void*)16};
    const char* names[] = {"out", "rows", "perm", "seg", "n_unique"};
    for (int i = 0; i < 5; ++i) {
        if (ptrs[i] == nullptr) { set_error("%s: %s is NULL", fn, names[i]); return KGE_E_NULL; }
        if (!aligned16(ptrs[i])) { set_error("%s: %s is not 16-byte aligned", fn, names[i]); return KGE_E_ALIGN; }
    }
    float* base = nullptr;
    int rc = static_scratch(&base);
    if (rc) return rc;
    if (n == 0) {
        if (n_out > 0) return cuda_status(cudaMemsetAsync(out, 0, (size_t)n_out * dim * 4, s), fn);
        return 0;
    }
    float* lead = base;
    float* trail = base + kStaticHalfFloats;
    const bool vec = dim % 4 == 0;
    switch (quads_per_lane(dim)) {
        case 1: return vec ? segred_go<1, true>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s)
                           : segred_go<1, false>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s);
        case 2: return vec ? segred_go<2, true>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s)
                           : segred_go<2, false>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s);
        case 4: return vec ? segred_go<4, true>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s)
                           : segred_go<4, false>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s);
        case 8: return vec ? segred_go<8, true>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s)
                           : segred_go<8, false>(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, lead, trail, s);
    }
    return KGE_E_UNSUPPORTED;
}
