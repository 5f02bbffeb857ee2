// The steps either side of the scoring path: where a batch's ids come from, and where its gradients go.
//
//   * id sampler: counter-based (Philox4x32-10) uniform and bounded-Zipf entity / relation ids generated on the GPU,
//     straight into the id list the inspector sorts.  Takes the place of the host-side batch assembly of the reference
//     (apps/kge/data/data_init.py:47-63: positives from a DGL EdgeSampler, negatives flattened with repeat_interleave);
//     element i of stream s is a pure function of (seed, s, i), so any process - or a numpy restatement - reproduces it
//     bit for bit.
//   * sparse optimizers: SGD and Adagrad applied to exactly the rows a batch touched, from the one-row-per-distinct-id
//     gradients the segmented reduction produces.  The reference stops at un-aggregated per-triple gradient pieces
//     (apps/kge/kge.py:393-515) and has no update step.
#include "rows.cuh"

namespace kge {

// ---- Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) ----------------------------
struct Philox4 { uint32_t x[4]; };
__host__ __device__ inline Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = static_cast<uint64_t>(M0) * c0, p1 = static_cast<uint64_t>(M1) * c2;
        const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
        const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += W0; k1 += W1;
    }
    Philox4 r;
    r.x[0] = c0; r.x[1] = c1; r.x[2] = c2; r.x[3] = c3;
    return r;
}

// Element i of stream `stream`: counter (i low, i high, stream, 0), key (seed low, seed high); words 0 and 1 are used.
__device__ __forceinline__ void draw2(unsigned long long seed, uint32_t stream, long long i, uint32_t& a, uint32_t& b) {
    const Philox4 r = philox4x32_10(static_cast<uint32_t>(i), static_cast<uint32_t>(static_cast<unsigned long long>(i) >> 32), stream, 0u,
                                    static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
    a = r.x[0]; b = r.x[1];
}

// uniform: id = floor(w * id_space / 2^64) with w the 64-bit word (a << 32 | b): exact integer arithmetic
template <typename I>
__global__ void __launch_bounds__(256) sample_uniform_kernel(void* out, long long n, unsigned long long id_space, unsigned long long seed,
                                                             uint32_t stream) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t a, b;
    draw2(seed, stream, i, a, b);
    const unsigned long long w = (static_cast<unsigned long long>(a) << 32) | b;
    reinterpret_cast<I*>(out)[i] = static_cast<I>(__umul64hi(w, id_space));
}

// bounded Zipf (or any discrete law) by inverse CDF: u = top 53 bits of the 64-bit word as a double in [0, 1), rank =
// first k with cdf[k] >= u (clamped to n_items - 1), id = perm[rank] (or the rank itself without a permutation)
template <typename I>
__global__ void __launch_bounds__(256) sample_cdf_kernel(void* out, long long n, const double* __restrict__ cdf, const long long* __restrict__ perm,
                                                         long long n_items, unsigned long long seed, uint32_t stream) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t a, b;
    draw2(seed, stream, i, a, b);
    const unsigned long long w = (static_cast<unsigned long long>(a) << 32) | b;
    const double u = static_cast<double>(w >> 11) * (1.0 / 9007199254740992.0);
    long long lo = 0, hi = n_items;                     // first index with cdf[idx] >= u
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if (__ldg(cdf + mid) < u) lo = mid + 1; else hi = mid;
    }
    if (lo > n_items - 1) lo = n_items - 1;
    reinterpret_cast<I*>(out)[i] = static_cast<I>(perm ? __ldg(perm + lo) : lo);
}

// positives drawn from a stored triple list: row = floor(w * n_triples / 2^64); h, r, t of that row
template <typename I>
__global__ void __launch_bounds__(256) sample_triples_kernel(void* h, void* r, void* t, long long n, const long long* __restrict__ triples,
                                                             unsigned long long n_triples, unsigned long long seed, uint32_t stream) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t a, b;
    draw2(seed, stream, i, a, b);
    const unsigned long long w = (static_cast<unsigned long long>(a) << 32) | b;
    const unsigned long long row = __umul64hi(w, n_triples);
    reinterpret_cast<I*>(h)[i] = static_cast<I>(__ldg(triples + 3 * row + 0));
    reinterpret_cast<I*>(r)[i] = static_cast<I>(__ldg(triples + 3 * row + 1));
    reinterpret_cast<I*>(t)[i] = static_cast<I>(__ldg(triples + 3 * row + 2));
}

int launch_sample_uniform(void* out, int id_bits, long long n, long long id_space, unsigned long long seed, unsigned stream_id, cudaStream_t s) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (id_bits == 64) sample_uniform_kernel<int64_t><<<blocks, 256, 0, s>>>(out, n, (unsigned long long)id_space, seed, stream_id);
    else sample_uniform_kernel<int32_t><<<blocks, 256, 0, s>>>(out, n, (unsigned long long)id_space, seed, stream_id);
    KGE_LAUNCH_CHECK("sample_uniform_kernel");
    return 0;
}
int launch_sample_cdf(void* out, int id_bits, long long n, const double* cdf, const long long* perm, long long n_items,
                      unsigned long long seed, unsigned stream_id, cudaStream_t s) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (id_bits == 64) sample_cdf_kernel<int64_t><<<blocks, 256, 0, s>>>(out, n, cdf, perm, n_items, seed, stream_id);
    else sample_cdf_kernel<int32_t><<<blocks, 256, 0, s>>>(out, n, cdf, perm, n_items, seed, stream_id);
    KGE_LAUNCH_CHECK("sample_cdf_kernel");
    return 0;
}
int launch_sample_triples(void* h, void* r, void* t, int id_bits, long long n, const long long* triples, long long n_triples,
                          unsigned long long seed, unsigned stream_id, cudaStream_t s) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (id_bits == 64) sample_triples_kernel<int64_t><<<blocks, 256, 0, s>>>(h, r, t, n, triples, (unsigned long long)n_triples, seed, stream_id);
    else sample_triples_kernel<int32_t><<<blocks, 256, 0, s>>>(h, r, t, n, triples, (unsigned long long)n_triples, seed, stream_id);
    KGE_LAUNCH_CHECK("sample_triples_kernel");
    return 0;
}

// ---- sparse optimizers ----------------------------------------------------------------------------------------------
// One warp per gradient row i < min(n, *n_dev): table row ids[i] - first_row (or row i when ids == NULL).  The ids are
// distinct (the inspector's `uniq`), so no two warps touch the same row.  bf16 tables are updated in fp32 and rounded
// to nearest even on the way back.
__device__ __forceinline__ float tbl_get(const float* p) { return *p; }
__device__ __forceinline__ float tbl_get(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void tbl_put(float* p, float v) { *p = v; }
__device__ __forceinline__ void tbl_put(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T, bool ADAGRAD>
__global__ void __launch_bounds__(256) apply_rows_kernel(T* table, float* state, int dim, const long long* ids, long long n,
                                                         const long long* n_dev, long long first_row, const float* grad,
                                                         float lr, float eps) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long cnt = n_dev ? min(n, *n_dev) : n;
    if (i >= cnt) return;
    const long long row = (ids ? ids[i] : i) - first_row;
    T* w = table + row * dim;
    const float* g = grad + i * dim;
    float* st = ADAGRAD ? state + row * dim : nullptr;
    for (int k = lane; k < dim; k += 32) {
        const float gk = g[k];
        float step = lr * gk;
        if (ADAGRAD) {
            const float acc = st[k] + gk * gk;
            st[k] = acc;
            step = lr * gk / (sqrtf(acc) + eps);
        }
        tbl_put(w + k, tbl_get(w + k) - step);
    }
}

int launch_apply_rows(void* table, int dtype, float* state, int dim, const long long* ids, long long n, const long long* n_dev,
                      long long first_row, const float* grad, float lr, float eps, bool adagrad, cudaStream_t s) {
    if (n <= 0) return 0;
    const int wpb = 8;
    const unsigned blocks = (unsigned)((n + wpb - 1) / wpb);
#define KGE_AP(T, A) apply_rows_kernel<T, A><<<blocks, wpb * 32, 0, s>>>(static_cast<T*>(table), state, dim, ids, n, n_dev, first_row, grad, lr, eps)
    if (dtype == KGE_F32) { if (adagrad) KGE_AP(float, true); else KGE_AP(float, false); }
    else { if (adagrad) KGE_AP(__nv_bfloat16, true); else KGE_AP(__nv_bfloat16, false); }
#undef KGE_AP
    KGE_LAUNCH_CHECK("apply_rows_kernel");
    return 0;
}

}  // namespace kge

using namespace kge;

extern "C" {

int kge_sample_uniform(void* out, int32_t id_bits, int64_t n, int64_t id_space, uint64_t seed, uint32_t stream_id, kge_stream_t stream) {
    const char* fn = "kge_sample_uniform";
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    if (n < 0 || id_space < 1 || (id_bits == 32 && id_space > (1LL << 31))) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (n == 0) return 0;
    if (!out) { set_error("%s: out is NULL", fn); return KGE_E_NULL; }
    if (reinterpret_cast<uintptr_t>(out) & (id_bits / 8 - 1)) { set_error("%s: out is not aligned to its element size", fn); return KGE_E_ALIGN; }
    return launch_sample_uniform(out, id_bits, n, id_space, seed, stream_id, reinterpret_cast<cudaStream_t>(stream));
}

int kge_sample_cdf(void* out, int32_t id_bits, int64_t n, const double* cdf, const int64_t* perm, int64_t n_items, uint64_t seed,
                   uint32_t stream_id, kge_stream_t stream) {
    const char* fn = "kge_sample_cdf";
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    if (n < 0 || n_items < 1) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (n == 0) return 0;
    if (!out || !cdf) { set_error("%s: out / cdf is NULL", fn); return KGE_E_NULL; }
    if ((reinterpret_cast<uintptr_t>(out) & (id_bits / 8 - 1)) || (reinterpret_cast<uintptr_t>(cdf) & 7) || (reinterpret_cast<uintptr_t>(perm) & 7)) {
        set_error("%s: a pointer is not aligned to its element size", fn); return KGE_E_ALIGN;
    }
    return launch_sample_cdf(out, id_bits, n, cdf, (const long long*)perm, n_items, seed, stream_id, reinterpret_cast<cudaStream_t>(stream));
}

int kge_sample_triples(void* h, void* r, void* t, int32_t id_bits, int64_t n, const int64_t* triples, int64_t n_triples, uint64_t seed,
                       uint32_t stream_id, kge_stream_t stream) {
    const char* fn = "kge_sample_triples";
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    if (n < 0 || n_triples < 1) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (n == 0) return 0;
    if (!h || !r || !t || !triples) { set_error("%s: a pointer is NULL", fn); return KGE_E_NULL; }
    const uintptr_t m = id_bits / 8 - 1;
    if ((reinterpret_cast<uintptr_t>(h) & m) || (reinterpret_cast<uintptr_t>(r) & m) || (reinterpret_cast<uintptr_t>(t) & m) ||
        (reinterpret_cast<uintptr_t>(triples) & 7)) { set_error("%s: a pointer is not aligned to its element size", fn); return KGE_E_ALIGN; }
    return launch_sample_triples(h, r, t, id_bits, n, (const long long*)triples, n_triples, seed, stream_id, reinterpret_cast<cudaStream_t>(stream));
}

static int apply_common(const char* fn, void* table, int32_t dtype, float* state, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                        int64_t first_row, const float* grad, float lr, float eps, bool adagrad, kge_stream_t stream) {
    if (n < 0 || dim <= 0) { set_error("%s: bad sizes", fn); return KGE_E_SHAPE; }
    if (dtype != KGE_F32 && dtype != KGE_BF16) { set_error("%s: unknown dtype %d", fn, dtype); return KGE_E_UNSUPPORTED; }
    if (n == 0) return 0;
    if (!table || !grad || (adagrad && !state)) { set_error("%s: table / grad / state is NULL", fn); return KGE_E_NULL; }
    if ((reinterpret_cast<uintptr_t>(table) & (dtype == KGE_F32 ? 3 : 1)) || (reinterpret_cast<uintptr_t>(grad) & 3) ||
        (reinterpret_cast<uintptr_t>(state) & 3) || (reinterpret_cast<uintptr_t>(ids) & 7) || (reinterpret_cast<uintptr_t>(n_dev) & 7)) {
        set_error("%s: a pointer is not aligned to its element size", fn); return KGE_E_ALIGN;
    }
    return launch_apply_rows(table, dtype, state, dim, (const long long*)ids, n, (const long long*)n_dev, first_row, grad, lr, eps, adagrad,
                             reinterpret_cast<cudaStream_t>(stream));
}

int kge_apply_sgd(void* table, int32_t dtype, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev, int64_t first_row,
                  const float* grad, float lr, kge_stream_t stream) {
    return apply_common("kge_apply_sgd", table, dtype, nullptr, dim, ids, n, n_dev, first_row, grad, lr, 0.f, false, stream);
}

int kge_apply_adagrad(void* table, int32_t dtype, float* state, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                      int64_t first_row, const float* grad, float lr, float eps, kge_stream_t stream) {
    return apply_common("kge_apply_adagrad", table, dtype, state, dim, ids, n, n_dev, first_row, grad, lr, eps, true, stream);
}

}  // extern "C"
