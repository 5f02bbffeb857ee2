// Relation-grouped projections for the relation-matrix models (fp32 CUDA-core path).
//
// cuke's generated TransR / RESCAL kernels (apps/kge/kge.py:321-343, 370-390) multiply every triple's vector
// with its relation's dim x dim matrix, caching at most the two most frequent matrices per 16 triples
// (pycuke1/transform/cuda_smem.py:401-590).  Here the inspector groups ALL triples of a batch by relation
// and each group becomes one dense (rows x dim) . (dim x dim) product, so P[r] is read once per 128-row tile.
// Orientation is the reference CPU path's:  y[j] = sum_i x[i] P[r][i][j].
//
//   RESCAL  anchors[i]  = E[h_i] . P[r_i]                                (rescal_anchor_kernel)
//           g_head[i]   = GA[i] . P[r_i]^T                               (rescal_ghead_kernel)
//           dP[g]       = sum_{i in group g} E[h_i] (x) GA[i]            (rescal_dproj_kernel)
//   TransR  score(i,j)  = -|| (a - b) . P[r_i] + R[r_i] ||  for the positive (j = 0) and every negative
//                                                                        (transr_fwd_kernel)
#include "tile_gemm.cuh"

namespace kge {

// Dense rows of a (.., dim) matrix in storage type T as a B operand: B(k, n) = base[k][n0 + n].
template <typename T, bool VEC>
struct MatRowsDirect {
    static constexpr bool K_CONTIG = false;
    const T* base; int n_rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= n_rows) return f4(0.f);
        return load_quad<T, VEC>(base + (long long)k * dim, (n0 + r4) >> 2, dim);
    }
};
// Rows n0.. of a matrix read along k: B(k, n) = base[n0 + n][k]  (the transposed use of P[r]).
template <typename T, bool VEC>
struct MatRowsK {
    static constexpr bool K_CONTIG = true;
    const T* base; int n_rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r, int k) const {
        if (n0 + r >= n_rows) return f4(0.f);
        return load_quad<T, VEC>(base + (long long)(n0 + r) * dim, k >> 2, dim);
    }
};
// Gathered rows (K_CONTIG), up to two rows per thread.
template <typename T, bool VEC>
struct GatherK {
    static constexpr bool K_CONTIG = true;
    const T* row[2]; int dim;
    __device__ __forceinline__ float4 get(int r, int k) const {
        const int u = r >> 6;
        return row[u] ? load_quad<T, VEC>(row[u], k >> 2, dim) : f4(0.f);
    }
};
// Difference of two gathered rows (K_CONTIG): a - b.
template <typename T, bool VEC>
struct DiffK {
    static constexpr bool K_CONTIG = true;
    const T* a[2]; const T* b[2]; int dim;
    __device__ __forceinline__ float4 get(int r, int k) const {
        const int u = r >> 6;
        if (a[u] == nullptr) return f4(0.f);
        return load_quad<T, VEC>(a[u], k >> 2, dim) - load_quad<T, VEC>(b[u], k >> 2, dim);
    }
};
// Columns of gathered rows as an A operand: A(m, k) = row(k)[m0 + m]; rows addressed through a list.
template <typename T, typename I, bool VEC>
struct GatherColsDirect {
    static constexpr bool K_CONTIG = false;
    const T* table; const void* ids; const int* list; int n_rows; int dim; int m0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= n_rows) return f4(0.f);
        const long long id = load_id<I>(ids, list[k]);
        return load_quad<T, VEC>(table + id * dim, (m0 + r4) >> 2, dim);
    }
};
// fp32 rows addressed through a list as a B operand: B(k, n) = rows[list[k]][n0 + n].
template <bool VEC>
struct ListRowsDirect {
    static constexpr bool K_CONTIG = false;
    const float* rows; const int* list; int n_rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= n_rows) return f4(0.f);
        return load_quad<float, VEC>(rows + (long long)list[k] * dim, (n0 + r4) >> 2, dim);
    }
};

struct GroupArgs {
    const void* ent; const void* rel; const void* proj;
    const void* h; const void* t; const void* neg;
    const int* rel_perm; const int* rel_seg; const long long* rel_uniq; const long long* n_groups;
    int dim; int n_neg; int n_neg_head; long long batch;
};

// ---- RESCAL: anchors = E[h] . P[r] ---------------------------------------------------------------------
template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) rescal_anchor_kernel(GroupArgs a, float* anchors) {
    __shared__ __align__(16) TileSmem sm;
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int tid = threadIdx.x, n0 = blockIdx.y * TG_BN, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const long long rid = a.rel_uniq[g];
    const T* E = reinterpret_cast<const T*>(a.ent);
    MatRowsDirect<T, VEC> bl;
    bl.base = reinterpret_cast<const T*>(a.proj) + rid * (long long)dim * dim; bl.n_rows = dim; bl.dim = dim; bl.n0 = n0;
    for (int m0 = s; m0 < e; m0 += TG_BM) {
        GatherK<T, VEC> al;
        al.dim = dim;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int p = m0 + (tid >> 2) + 64 * u;
            al.row[u] = (p < e) ? E + load_id<I>(a.h, a.rel_perm[p]) * dim : nullptr;
        }
        float acc[8][8];
        tile_mainloop<OP_DOT>(al, bl, dim, sm, acc);
        auto ep = [&](int row, int col4, float4 v) {
            const int p = m0 + row, n = n0 + col4;
            if (p >= e || n >= dim) return;
            store_quad<VEC>(anchors + (long long)a.rel_perm[p] * dim, n >> 2, dim, v);
        };
        tile_epilogue(acc, ep);
    }
}

// ---- RESCAL backward: g_head = GA . P[r]^T -------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) rescal_ghead_kernel(GroupArgs a, const float* ga, float* g_head) {
    __shared__ __align__(16) TileSmem sm;
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int tid = threadIdx.x, n0 = blockIdx.y * TG_BN, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const long long rid = a.rel_uniq[g];
    MatRowsK<T, VEC> bl;
    bl.base = reinterpret_cast<const T*>(a.proj) + rid * (long long)dim * dim; bl.n_rows = dim; bl.dim = dim; bl.n0 = n0;
    for (int m0 = s; m0 < e; m0 += TG_BM) {
        GatherK<float, VEC> al;
        al.dim = dim;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int p = m0 + (tid >> 2) + 64 * u;
            al.row[u] = (p < e) ? ga + (long long)a.rel_perm[p] * dim : nullptr;
        }
        float acc[8][8];
        tile_mainloop<OP_DOT>(al, bl, dim, sm, acc);
        auto ep = [&](int row, int col4, float4 v) {
            const int p = m0 + row, n = n0 + col4;
            if (p >= e || n >= dim) return;
            store_quad<VEC>(g_head + (long long)a.rel_perm[p] * dim, n >> 2, dim, v);
        };
        tile_epilogue(acc, ep);
    }
}

// ---- RESCAL backward: dP[g] = sum_i E[h_i] (x) GA[i] -------------------------------------------------------------
template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) rescal_dproj_kernel(GroupArgs a, const float* ga, float* dproj) {
    __shared__ __align__(16) TileSmem sm;
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int m0 = blockIdx.y * TG_BM, n0 = blockIdx.z * TG_BN, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    GatherColsDirect<T, I, VEC> al;
    al.table = reinterpret_cast<const T*>(a.ent); al.ids = a.h; al.list = a.rel_perm + s; al.n_rows = e - s; al.dim = dim; al.m0 = m0;
    ListRowsDirect<VEC> bl;
    bl.rows = ga; bl.list = a.rel_perm + s; bl.n_rows = e - s; bl.dim = dim; bl.n0 = n0;
    float acc[8][8];
    tile_mainloop<OP_DOT>(al, bl, e - s, sm, acc);
    float* out = dproj + (long long)g * dim * dim;
    auto ep = [&](int row, int col4, float4 v) {
        const int m = m0 + row, n = n0 + col4;
        if (m >= dim || n >= dim) return;
        store_quad<VEC>(out + (long long)m * dim, n >> 2, dim, v);
    };
    tile_epilogue(acc, ep);
}

// ---- TransR forward ---------------------------------------------------------------------------------------------
// Rows of group g: for each of its triples, 1 + n_neg differences (positive first).  One CTA owns a 128-row
// tile and walks all column tiles, accumulating the squared norm of (diff . P + R[r]) per row.
template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) transr_fwd_kernel(GroupArgs a, float* pos, float* negs) {
    __shared__ __align__(16) TileSmem sm;
    __shared__ float rownorm[TG_BM];
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int tid = threadIdx.x, tx = tid & 15, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const long long rid = a.rel_uniq[g];
    const int per = 1 + a.n_neg;
    const long long rows = (long long)(e - s) * per;
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* Rv = reinterpret_cast<const T*>(a.rel) + rid * dim;
    const T* P = reinterpret_cast<const T*>(a.proj) + rid * (long long)dim * dim;

    for (long long m0 = (long long)blockIdx.y * TG_BM; m0 < rows; m0 += (long long)gridDim.y * TG_BM) {
        DiffK<T, VEC> al;
        al.dim = dim;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const long long row = m0 + (tid >> 2) + 64 * u;
            al.a[u] = nullptr; al.b[u] = nullptr;
            if (row < rows) {
                const int i = a.rel_perm[s + (int)(row / per)];
                const int j = (int)(row % per);
                const T* hrow = E + load_id<I>(a.h, i) * dim;
                const T* trow = E + load_id<I>(a.t, i) * dim;
                if (j == 0) { al.a[u] = hrow; al.b[u] = trow; }
                else {
                    const T* x = E + load_id<I>(a.neg, (long long)i * a.n_neg + (j - 1)) * dim;
                    if (j - 1 < a.n_neg_head) { al.a[u] = x; al.b[u] = trow; } else { al.a[u] = hrow; al.b[u] = x; }
                }
            }
        }
        if (tid < TG_BM) rownorm[tid] = 0.f;
        __syncthreads();
        for (int n0 = 0; n0 < dim; n0 += TG_BN) {
            MatRowsDirect<T, VEC> bl;
            bl.base = P; bl.n_rows = dim; bl.dim = dim; bl.n0 = n0;
            float acc[8][8];
            tile_mainloop<OP_DOT>(al, bl, dim, sm, acc);
            // add R[r], square, sum over this thread's 8 columns, then over the 16 threads sharing the row
            float4 r0 = load_quad<T, VEC>(Rv, (n0 + tx * 4) >> 2, dim);
            float4 r1 = load_quad<T, VEC>(Rv, (n0 + 64 + tx * 4) >> 2, dim);
            const float rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float ssq = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = n0 + ((j < 4) ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                    const float v = (col < dim) ? acc[i][j] + rr[j] : 0.f;
                    ssq = fmaf(v, v, ssq);
                }
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ssq += __shfl_xor_sync(kFull, ssq, o);
                if (tx == 0) {
                    const int row = (i < 4) ? (tid >> 4) * 4 + i : 64 + (tid >> 4) * 4 + (i - 4);
                    rownorm[row] += ssq;          // one writer per row
                }
            }
            __syncthreads();
        }
        if (tid < TG_BM) {
            const long long row = m0 + tid;
            if (row < rows) {
                const int i = a.rel_perm[s + (int)(row / per)];
                const int j = (int)(row % per);
                const float sc = -sqrtf(rownorm[tid]);
                if (j == 0) pos[i] = sc; else negs[(long long)i * a.n_neg + (j - 1)] = sc;
            }
        }
        __syncthreads();
    }
}

// ---- host ---------------------------------------------------------------------------------------------------------
static GroupArgs group_args(const kge_problem* p, const kge_tensors* t) {
    GroupArgs a;
    a.ent = t->ent; a.rel = t->rel; a.proj = t->rel2; a.h = t->h; a.t = t->t; a.neg = t->neg;
    a.rel_perm = t->rel_perm; a.rel_seg = t->rel_seg; a.rel_uniq = (const long long*)t->rel_uniq;
    a.n_groups = (const long long*)t->n_rel_groups;
    a.dim = p->dim; a.n_neg = p->n_neg; a.n_neg_head = p->n_neg_head; a.batch = p->batch;
    return a;
}
static inline unsigned group_bound(const kge_problem* p) {
    return (unsigned)(p->n_rel < p->batch ? p->n_rel : p->batch);
}

#define KGE_TI_DISPATCH(KERNEL_CALL)                                                       \
    do {                                                                                   \
        const bool vec = p->dim % 4 == 0;                                                  \
        if (p->dtype == KGE_F32) {                                                         \
            if (p->id_bits == 64) { if (vec) { KERNEL_CALL(float, int64_t, true); } else { KERNEL_CALL(float, int64_t, false); } } \
            else { if (vec) { KERNEL_CALL(float, int32_t, true); } else { KERNEL_CALL(float, int32_t, false); } }                  \
        } else {                                                                           \
            if (p->id_bits == 64) { if (vec) { KERNEL_CALL(__nv_bfloat16, int64_t, true); } else { KERNEL_CALL(__nv_bfloat16, int64_t, false); } } \
            else { if (vec) { KERNEL_CALL(__nv_bfloat16, int32_t, true); } else { KERNEL_CALL(__nv_bfloat16, int32_t, false); } }  \
        }                                                                                  \
    } while (0)

int launch_rescal_anchors(const kge_problem* p, const kge_tensors* t, float* anchors, cudaStream_t s) {
    if (p->batch <= 0) return 0;
    const GroupArgs a = group_args(p, t);
    const dim3 grid(group_bound(p), (p->dim + TG_BN - 1) / TG_BN);
#define KGE_CALL(T, I, V) rescal_anchor_kernel<T, I, V><<<grid, 256, 0, s>>>(a, anchors)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("rescal_anchor_kernel");
    return 0;
}

int launch_rescal_backward(const kge_problem* p, const kge_tensors* t, const float* ga, float* g_head, float* dproj,
                           cudaStream_t s) {
    if (p->batch <= 0) return 0;
    const GroupArgs a = group_args(p, t);
    const unsigned nt = (p->dim + TG_BN - 1) / TG_BN;
    const dim3 grid1(group_bound(p), nt);
    const dim3 grid2(group_bound(p), nt, nt);
#define KGE_CALL(T, I, V) rescal_ghead_kernel<T, V><<<grid1, 256, 0, s>>>(a, ga, g_head)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("rescal_ghead_kernel");
#define KGE_CALL(T, I, V) rescal_dproj_kernel<T, I, V><<<grid2, 256, 0, s>>>(a, ga, dproj)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("rescal_dproj_kernel");
    return 0;
}

int launch_transr_forward(const kge_problem* p, const kge_tensors* t, float* pos, float* negs, cudaStream_t s) {
    if (p->batch <= 0) return 0;
    const GroupArgs a = group_args(p, t);
    // rows per group are unknown on the host; 8 row-tile walkers per group keep the GPU busy without a sync
    const dim3 grid(group_bound(p), 8);
#define KGE_CALL(T, I, V) transr_fwd_kernel<T, I, V><<<grid, 256, 0, s>>>(a, pos, negs)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("transr_fwd_kernel");
    return 0;
}

}  // namespace kge
