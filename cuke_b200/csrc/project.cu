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
//                                                                        (transr_fwd_kernel; backward: transr_gv/gd/dproj/reduce)
#include <atomic>
#include "tile_gemm.cuh"
#include "rows.cuh"

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

// =====================================================================================================================
// Small groups: relation-grouped projections for tens of rows per relation (tens of rows per relation), fp32 CUDA cores.
//
// With ~33 triples per relation (RESCAL at 16,384 triples over 500 relations) a relation's dim x dim matrix is used by
// so few rows that the products are bound by READING the matrices (131 MB at dim 256), not by arithmetic: a 128-row tile
// engine would spend three quarters of its work on padding.  Here one CTA owns one relation group and streams P[r]
// through once per block of 32 rows; the group's rows sit transposed in shared memory (Xs[k][m], so that four rows are
// one 128-bit broadcast read) and thread t owns output column t (dim <= 256):
//
//   small_fwd    Y[m][j]  = sum_i X[m][i] P[r][i][j]      X = E[h] gathered        -> anchors          (RESCAL forward)
//   small_bwd_x  Y[m][i]  = sum_j G[m][j] P[r][i][j]      G = anchor gradients     -> g_head           (thread t streams row P[t][:])
//   small_dproj  dP[i][j] = sum_m X[m][i] G[m][j]         one (dim x dim) gradient per group, up to 64 rows per pass
//
// Orientation is the reference CPU path's (out[j] = sum_i x[i] P[r][i][j], apps/kge/kge.py:21-23,370-390).
struct SmallGroupArgs {
    const void* ent; const void* proj; const void* h;
    const int* rel_perm; const int* rel_seg; const long long* rel_uniq; const long long* n_groups;
    int dim;
};

// Register tile of a thread: 16 rows x 4 columns.  256 threads = 4 row groups (two warps each) x 64 column groups, so a
// pass covers 64 rows x 256 columns; per k a thread reads its 16 row values as four 128-bit shared-memory BROADCASTS (the
// whole warp shares the row group) and its 4 matrix values as one 128-bit load: 5 memory instructions per 64 FMAs.
// (One row per thread-register and one column per thread would need a shared-memory instruction per 4 FMAs and is bound
// by the shared-memory pipe, not by arithmetic.)
constexpr int SG_ROWS = 64;        // rows per pass
constexpr int SG_LD = 68;          // pitch of the transposed row block Xs[k][m] (floats; multiple of 4)
constexpr int SG_DP_ROWS = 32;     // rows per pass of small_dproj (X and G rows side by side in shared memory)

__device__ __forceinline__ float sg_get(const float* p) { return __ldg(p); }
__device__ __forceinline__ float sg_get(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Rows [m0, m0 + rows) of the group -> Xs[k * SG_LD + m], transposed (zero for m >= rows).  Warp w takes rows w, w + 8, ...;
// a lane reads consecutive elements of the row.  SRC: 0 = entity rows gathered through h (type T), 1 = fp32 rows `frows`
// indexed by triple.
template <typename T, typename I, int SRC>
__device__ __forceinline__ void sg_stage_transposed(const SmallGroupArgs& a, const float* frows, int m0, int rows, float* Xs) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, dim = a.dim;
    for (int m = w; m < SG_ROWS; m += 8) {
        const bool ok = m < rows;
        const int tri = ok ? a.rel_perm[m0 + m] : 0;
        if (SRC == 0) {
            const T* row = reinterpret_cast<const T*>(a.ent) + (ok ? load_id<I>(a.h, tri) : 0) * dim;
            for (int k = lane; k < dim; k += 32) Xs[k * SG_LD + m] = ok ? sg_get(row + k) : 0.f;
        } else {
            const float* row = frows + (long long)tri * dim;
            for (int k = lane; k < dim; k += 32) Xs[k * SG_LD + m] = ok ? __ldg(row + k) : 0.f;
        }
    }
}

// acc[r][c] += x[r] * p[c] for the first 4 * nq of the thread's 16 rows
__device__ __forceinline__ void sg_fma_tile(float (&acc)[16][4], const float* xk, const float4 p, int nq) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q < nq) {
            const float4 x = *reinterpret_cast<const float4*>(xk + 4 * q);
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                acc[4 * q + r][0] = fmaf(xs[r], p.x, acc[4 * q + r][0]);
                acc[4 * q + r][1] = fmaf(xs[r], p.y, acc[4 * q + r][1]);
                acc[4 * q + r][2] = fmaf(xs[r], p.z, acc[4 * q + r][2]);
                acc[4 * q + r][3] = fmaf(xs[r], p.w, acc[4 * q + r][3]);
            }
        }
    }
}

// TRANS = false: Y = X . P      thread columns j = 4cg..4cg+3: P[k][4cg..] is one 128-bit load, a warp reads 512 B of a row of P
// TRANS = true : Y = G . P^T    thread outputs i = 4cg..4cg+3: the thread streams four rows of P, 4 k-values at a time
template <typename T, typename I, int SRC, bool TRANS>
__global__ void __launch_bounds__(256, 2) small_proj_kernel(SmallGroupArgs a, const float* frows, float* out) {
    extern __shared__ __align__(16) float Xs[];                 // dim * SG_LD floats
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int dim = a.dim;
    const int cg = threadIdx.x & 63, rg = threadIdx.x >> 6;     // column group, row group (uniform within a warp)
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const T* P = reinterpret_cast<const T*>(a.proj) + a.rel_uniq[g] * (long long)dim * dim;
    const bool col_ok = 4 * cg < dim;                           // dim % 4 == 0
    for (int m0 = s; m0 < e; m0 += SG_ROWS) {
        const int rows = min(SG_ROWS, e - m0);
        const int my_rows = min(16, rows - 16 * rg);            // rows of this thread's row group that exist (may be <= 0)
        const int nq = (my_rows + 3) >> 2;
        __syncthreads();                                        // the previous pass's reads of Xs are done
        sg_stage_transposed<T, I, SRC>(a, frows, m0, rows, Xs);
        __syncthreads();
        if (!col_ok || my_rows <= 0) continue;                  // no barrier below this point inside the pass
        float acc[16][4];
#pragma unroll
        for (int r = 0; r < 16; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; acc[r][2] = 0.f; acc[r][3] = 0.f; }
        const float* xr = Xs + 16 * rg;
        // The matrix comes straight from HBM (each element is used by this group only).  Loads run three batches (twelve
        // 16-byte loads per thread) ahead of their use: a batch of four is re-requested right after it has been consumed,
        // so every load has two batches of arithmetic (512 FMAs per thread) to arrive.
        float4 pv[3][4];
        if (!TRANS) {
            const T* pc = P + 4 * cg;
            auto fetch = [&](int b, int k) {
#pragma unroll
                for (int u = 0; u < 4; ++u) pv[b][u] = k + u < dim ? load_quad<T, true>(pc + (long long)(k + u) * dim, 0, 4) : f4(0.f);
            };
#pragma unroll
            for (int b = 0; b < 3; ++b) fetch(b, 4 * b);
            for (int k0 = 0; k0 < dim; k0 += 12) {
#pragma unroll
                for (int b = 0; b < 3; ++b) {
                    const int k = k0 + 4 * b;
#pragma unroll
                    for (int u = 0; u < 4; ++u) if (k + u < dim) sg_fma_tile(acc, xr + (k + u) * SG_LD, pv[b][u], nq);
                    fetch(b, k + 12);
                }
            }
        } else {
            const T* pr = P + (long long)(4 * cg) * dim;
            auto fetch = [&](int b, int k) {          // four k-values of the thread's four rows of P; zero past dim
#pragma unroll
                for (int c = 0; c < 4; ++c) pv[b][c] = load_quad<T, true>(pr + (long long)c * dim, k >> 2, dim);
            };
#pragma unroll
            for (int b = 0; b < 3; ++b) fetch(b, 4 * b);
            for (int k0 = 0; k0 < dim; k0 += 12) {
#pragma unroll
                for (int b = 0; b < 3; ++b) {
                    const int k = k0 + 4 * b;
                    if (k < dim) {
                        sg_fma_tile(acc, xr + (k + 0) * SG_LD, make_float4(pv[b][0].x, pv[b][1].x, pv[b][2].x, pv[b][3].x), nq);
                        sg_fma_tile(acc, xr + (k + 1) * SG_LD, make_float4(pv[b][0].y, pv[b][1].y, pv[b][2].y, pv[b][3].y), nq);
                        sg_fma_tile(acc, xr + (k + 2) * SG_LD, make_float4(pv[b][0].z, pv[b][1].z, pv[b][2].z, pv[b][3].z), nq);
                        sg_fma_tile(acc, xr + (k + 3) * SG_LD, make_float4(pv[b][0].w, pv[b][1].w, pv[b][2].w, pv[b][3].w), nq);
                    }
                    fetch(b, k + 12);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 16; ++r)
            if (r < my_rows)
                *reinterpret_cast<float4*>(out + (long long)a.rel_perm[m0 + 16 * rg + r] * dim + 4 * cg) =
                    make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
}

// dP[g][i][j] = sum over the group's rows m of X[m][i] * G[m][j].  Up to 32 rows of X and of G sit row-major in shared
// memory; the output is produced in four blocks of 64 i-values, a thread owning 16 i x 4 j of a block: per row m four
// 128-bit broadcasts of X[m][i0..i0+15] and one 128-bit read of G[m][4cg..].  Groups with more than 32 rows take further
// passes that add to what the earlier ones stored.
template <typename T, typename I>
__global__ void __launch_bounds__(256) small_dproj_kernel(SmallGroupArgs a, const float* grows, float* dproj) {
    extern __shared__ __align__(16) float sm[];                 // X rows: SG_DP_ROWS * dim, then G rows: SG_DP_ROWS * dim
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int dim = a.dim;
    const int cg = threadIdx.x & 63, ig = threadIdx.x >> 6;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    float* Xr = sm;
    float* Gr = sm + SG_DP_ROWS * dim;
    float* out = dproj + (long long)g * dim * dim;
    const bool col_ok = 4 * cg < dim;
    for (int m0 = s; m0 < e; m0 += SG_DP_ROWS) {
        const int rows = min(SG_DP_ROWS, e - m0);
        __syncthreads();
        for (int m = w; m < rows; m += 8) {
            const int tri = a.rel_perm[m0 + m];
            const T* xrow = reinterpret_cast<const T*>(a.ent) + load_id<I>(a.h, tri) * dim;
            const float* grow = grows + (long long)tri * dim;
            for (int k = lane; k < dim; k += 32) { Xr[m * dim + k] = sg_get(xrow + k); Gr[m * dim + k] = __ldg(grow + k); }
        }
        __syncthreads();
        if (!col_ok) continue;
        for (int ib = 0; ib < dim; ib += 64) {
            const int i0 = ib + 16 * ig;
            if (i0 >= dim) continue;
            float acc[16][4];
#pragma unroll
            for (int r = 0; r < 16; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; acc[r][2] = 0.f; acc[r][3] = 0.f; }
            for (int m = 0; m < rows; ++m)
                sg_fma_tile(acc, Xr + m * dim + i0, *reinterpret_cast<const float4*>(Gr + m * dim + 4 * cg), 4);
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                if (i0 + r < dim) {
                    float4* o = reinterpret_cast<float4*>(out + (long long)(i0 + r) * dim + 4 * cg);
                    float4 v = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
                    if (m0 != s) { const float4 old = *o; v = v + old; }
                    *o = v;
                }
            }
        }
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

// The small-group kernels give each thread one output column: dim <= 256, vector rows.
static bool small_groups(const kge_problem* p) { return p->dim <= 256 && p->dim % 4 == 0; }
static SmallGroupArgs small_args(const kge_problem* p, const kge_tensors* t) {
    SmallGroupArgs a;
    a.ent = t->ent; a.proj = t->rel2; a.h = t->h; a.rel_perm = t->rel_perm; a.rel_seg = t->rel_seg;
    a.rel_uniq = (const long long*)t->rel_uniq; a.n_groups = (const long long*)t->n_rel_groups; a.dim = p->dim;
    return a;
}
// Dynamic shared memory of the small-group kernels at dim 256: 68 KB (projections), 64 KB (matrix gradient) - above the
// 48 KB default, so every instantiation is opted in once per device.
static int small_opt_in() {
    static std::atomic<bool> opted[128];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cuda_status(cudaGetLastError(), "cudaGetDevice");
    if (dev >= 0 && dev < 128 && opted[dev].load(std::memory_order_acquire)) return 0;
    const int bytes = 256 * SG_LD * (int)sizeof(float);
    cudaError_t e = cudaSuccess;
#define KGE_OPT(T, I)                                                                                                              \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(small_proj_kernel<T, I, 0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(small_proj_kernel<T, I, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);  \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(small_dproj_kernel<T, I>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    KGE_OPT(float, int64_t) KGE_OPT(float, int32_t) KGE_OPT(__nv_bfloat16, int64_t) KGE_OPT(__nv_bfloat16, int32_t)
#undef KGE_OPT
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(small-group kernels)");
    if (dev >= 0 && dev < 128) opted[dev].store(true, std::memory_order_release);
    return 0;
}
#define KGE_SMALL_DISPATCH(CALL)                                                                  \
    do {                                                                                          \
        if (p->dtype == KGE_F32) { if (p->id_bits == 64) { CALL(float, int64_t); } else { CALL(float, int32_t); } }            \
        else { if (p->id_bits == 64) { CALL(__nv_bfloat16, int64_t); } else { CALL(__nv_bfloat16, int32_t); } }                \
    } while (0)

int launch_rescal_anchors(const kge_problem* p, const kge_tensors* t, float* anchors, cudaStream_t s) {
    if (p->batch <= 0) return 0;
    if (small_groups(p)) {
        const SmallGroupArgs sa = small_args(p, t);
        const size_t smem = (size_t)p->dim * SG_LD * sizeof(float);
        if (int rc = small_opt_in()) return rc;
#define KGE_CALL(T, I) small_proj_kernel<T, I, 0, false><<<group_bound(p), 256, smem, s>>>(sa, nullptr, anchors)
        KGE_SMALL_DISPATCH(KGE_CALL);
#undef KGE_CALL
        KGE_LAUNCH_CHECK("small_proj_kernel(anchors)");
        return 0;
    }
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
    if (small_groups(p)) {
        const SmallGroupArgs sa = small_args(p, t);
        const size_t smem = (size_t)p->dim * SG_LD * sizeof(float), smem2 = (size_t)2 * SG_DP_ROWS * p->dim * sizeof(float);
        if (int rc = small_opt_in()) return rc;
#define KGE_CALL(T, I) small_proj_kernel<T, I, 1, true><<<group_bound(p), 256, smem, s>>>(sa, ga, g_head)
        KGE_SMALL_DISPATCH(KGE_CALL);
#undef KGE_CALL
        KGE_LAUNCH_CHECK("small_proj_kernel(g_head)");
#define KGE_CALL(T, I) small_dproj_kernel<T, I><<<group_bound(p), 256, smem2, s>>>(sa, ga, dproj)
        KGE_SMALL_DISPATCH(KGE_CALL);
#undef KGE_CALL
        KGE_LAUNCH_CHECK("small_dproj_kernel");
        return 0;
    }
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


// ---- TransR backward ---------------------------------------------------------------------------------------------
// With v = diff . P + R and score = -||v||, dL/dv = (dS / S) v.  Four launches:
//   transr_gv_kernel      GV[row]  = (dS/S) (diff . P[r] + R[r])                       (recomputes the forward product)
//   transr_gd_kernel      GD[row]  = GV[row] . P[r]^T ; negatives' rows go to g_neg with their sign, positives' to GD0
//   transr_dproj_kernel   dP[g]    = sum_rows diff^T (x) GV[row]
//   transr_reduce_kernel  per triple: g_head, g_tail from GD0 and its g_neg rows, g_rel = sum of its GV rows
// Rows are numbered as in the forward: row = triple_in_group * (1 + n_neg) + j, GV is stored triple-major
// (global row i * (1 + n_neg) + j) so that the per-triple pass reads contiguous rows.
struct TransRBwd {
    const float* pos; const float* negs; const float* dpos; const float* dneg;
    float* gv; float* gd0; float* g_neg; float* g_head; float* g_tail; float* g_rel; float* dproj;
};

template <typename T, typename I>
__device__ __forceinline__ void transr_row(const GroupArgs& a, int s, int per, long long row, int& i, int& j,
                                           const T*& pa, const T*& pb) {
    const T* E = reinterpret_cast<const T*>(a.ent);
    i = a.rel_perm[s + (int)(row / per)];
    j = (int)(row % per);
    const T* hrow = E + load_id<I>(a.h, i) * a.dim;
    const T* trow = E + load_id<I>(a.t, i) * a.dim;
    if (j == 0) { pa = hrow; pb = trow; }
    else {
        const T* x = E + load_id<I>(a.neg, (long long)i * a.n_neg + (j - 1)) * a.dim;
        if (j - 1 < a.n_neg_head) { pa = x; pb = trow; } else { pa = hrow; pb = x; }
    }
}

template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) transr_gv_kernel(GroupArgs a, TransRBwd w) {
    __shared__ __align__(16) TileSmem sm;
    __shared__ float coef[TG_BM];
    __shared__ long long grow[TG_BM];
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int tid = threadIdx.x, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const long long rid = a.rel_uniq[g];
    const int per = 1 + a.n_neg;
    const long long rows = (long long)(e - s) * per;
    const T* Rv = reinterpret_cast<const T*>(a.rel) + rid * dim;
    const T* P = reinterpret_cast<const T*>(a.proj) + rid * (long long)dim * dim;
    for (long long m0 = (long long)blockIdx.y * TG_BM; m0 < rows; m0 += (long long)gridDim.y * TG_BM) {
        DiffK<T, VEC> al;
        al.dim = dim;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const long long row = m0 + (tid >> 2) + 64 * u;
            al.a[u] = nullptr; al.b[u] = nullptr;
            if (row < rows) { int i, j; transr_row<T, I>(a, s, per, row, i, j, al.a[u], al.b[u]); }
        }
        if (tid < TG_BM) {
            const long long row = m0 + tid;
            float c = 0.f; long long gr = -1;
            if (row < rows) {
                const int i = a.rel_perm[s + (int)(row / per)];
                const int j = (int)(row % per);
                const float sc = j == 0 ? w.pos[i] : w.negs[(long long)i * a.n_neg + (j - 1)];
                const float ds = j == 0 ? w.dpos[i] : w.dneg[(long long)i * a.n_neg + (j - 1)];
                c = sc != 0.f ? ds / sc : 0.f;
                gr = (long long)i * per + j;
            }
            coef[tid] = c; grow[tid] = gr;
        }
        __syncthreads();
        for (int n0 = 0; n0 < dim; n0 += TG_BN) {
            MatRowsDirect<T, VEC> bl;
            bl.base = P; bl.n_rows = dim; bl.dim = dim; bl.n0 = n0;
            float acc[8][8];
            tile_mainloop<OP_DOT>(al, bl, dim, sm, acc);
            auto ep = [&](int row, int col4, float4 v) {
                const int n = n0 + col4;
                if (grow[row] < 0 || n >= dim) return;
                const float4 r = load_quad<T, VEC>(Rv, n >> 2, dim);
                const float c = coef[row];
                store_quad<VEC>(w.gv + grow[row] * dim, n >> 2, dim,
                                make_float4(c * (v.x + r.x), c * (v.y + r.y), c * (v.z + r.z), c * (v.w + r.w)));
            };
            tile_epilogue(acc, ep);
        }
        __syncthreads();
    }
}

template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) transr_gd_kernel(GroupArgs a, TransRBwd w) {
    __shared__ __align__(16) TileSmem sm;
    __shared__ int row_i[TG_BM], row_j[TG_BM];
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int tid = threadIdx.x, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const long long rid = a.rel_uniq[g];
    const int per = 1 + a.n_neg;
    const long long rows = (long long)(e - s) * per;
    const T* P = reinterpret_cast<const T*>(a.proj) + rid * (long long)dim * dim;
    for (long long m0 = (long long)blockIdx.y * TG_BM; m0 < rows; m0 += (long long)gridDim.y * TG_BM) {
        GatherK<float, VEC> al;
        al.dim = dim;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const long long row = m0 + (tid >> 2) + 64 * u;
            al.row[u] = nullptr;
            if (row < rows) {
                const int i = a.rel_perm[s + (int)(row / per)];
                al.row[u] = w.gv + ((long long)i * per + (row % per)) * dim;
            }
        }
        if (tid < TG_BM) {
            const long long row = m0 + tid;
            row_i[tid] = row < rows ? a.rel_perm[s + (int)(row / per)] : -1;
            row_j[tid] = (int)(row % per);
        }
        __syncthreads();
        for (int n0 = 0; n0 < dim; n0 += TG_BN) {
            MatRowsK<T, VEC> bl;
            bl.base = P; bl.n_rows = dim; bl.dim = dim; bl.n0 = n0;
            float acc[8][8];
            tile_mainloop<OP_DOT>(al, bl, dim, sm, acc);
            auto ep = [&](int row, int col4, float4 v) {
                const int n = n0 + col4, i = row_i[row], j = row_j[row];
                if (i < 0 || n >= dim) return;
                if (j == 0) store_quad<VEC>(w.gd0 + (long long)i * dim, n >> 2, dim, v);
                else {
                    if (j - 1 >= a.n_neg_head) v = make_float4(-v.x, -v.y, -v.z, -v.w);     // diff = h - x: dL/dx = -GD
                    store_quad<VEC>(w.g_neg + ((long long)i * a.n_neg + (j - 1)) * dim, n >> 2, dim, v);
                }
            };
            tile_epilogue(acc, ep);
        }
        __syncthreads();
    }
}

// A(m, k) = diff(row k)[m0 + m]; rows of one relation group, numbered as in the forward.
template <typename T, typename I, bool VEC>
struct DiffColsDirect {
    static constexpr bool K_CONTIG = false;
    GroupArgs a; int s; int per; long long rows; int m0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= rows) return f4(0.f);
        int i, j; const T* pa; const T* pb;
        transr_row<T, I>(a, s, per, k, i, j, pa, pb);
        return load_quad<T, VEC>(pa, (m0 + r4) >> 2, a.dim) - load_quad<T, VEC>(pb, (m0 + r4) >> 2, a.dim);
    }
};
// B(k, n) = GV[global row of group row k][n0 + n]
template <bool VEC>
struct GvRowsDirect {
    static constexpr bool K_CONTIG = false;
    const float* gv; const int* perm; int per; long long rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= rows) return f4(0.f);
        const long long gr = (long long)perm[k / per] * per + (k % per);
        return load_quad<float, VEC>(gv + gr * dim, (n0 + r4) >> 2, dim);
    }
};

template <typename T, typename I, bool VEC>
__global__ void __launch_bounds__(256) transr_dproj_kernel(GroupArgs a, TransRBwd w) {
    __shared__ __align__(16) TileSmem sm;
    const int g = blockIdx.x;
    if (g >= *a.n_groups) return;
    const int m0 = blockIdx.y * TG_BM, n0 = blockIdx.z * TG_BN, dim = a.dim;
    const int s = a.rel_seg[g], e = a.rel_seg[g + 1];
    const int per = 1 + a.n_neg;
    const long long rows = (long long)(e - s) * per;
    DiffColsDirect<T, I, VEC> al;
    al.a = a; al.s = s; al.per = per; al.rows = rows; al.m0 = m0;
    GvRowsDirect<VEC> bl;
    bl.gv = w.gv; bl.perm = a.rel_perm + s; bl.per = per; bl.rows = rows; bl.dim = dim; bl.n0 = n0;
    float acc[8][8];
    tile_mainloop<OP_DOT>(al, bl, (int)rows, sm, acc);
    float* out = w.dproj + (long long)g * dim * dim;
    auto ep = [&](int row, int col4, float4 v) {
        const int m = m0 + row, n = n0 + col4;
        if (m >= dim || n >= dim) return;
        store_quad<VEC>(out + (long long)m * dim, n >> 2, dim, v);
    };
    tile_epilogue(acc, ep);
}

// One warp per triple: g_head = GD0 - sum of its tail-replaced g_neg rows, g_tail = -GD0 - sum of its head-replaced
// g_neg rows, g_rel = sum of its GV rows; all in ascending j.
__global__ void __launch_bounds__(256) transr_reduce_kernel(long long batch, int dim, int n_neg, int n_neg_head, TransRBwd w) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= batch) return;
    const int per = 1 + n_neg;
    for (int k = lane; k < dim; k += 32) {
        const float g0 = w.gd0[i * dim + k];
        float gh = g0, gt = -g0, gr = w.gv[(i * per) * dim + k];
        for (int j = 0; j < n_neg; ++j) {
            const float gx = w.g_neg[(i * n_neg + j) * dim + k];
            if (j < n_neg_head) gt -= gx; else gh -= gx;
            gr += w.gv[(i * per + 1 + j) * dim + k];
        }
        w.g_head[i * dim + k] = gh;
        w.g_tail[i * dim + k] = gt;
        w.g_rel[i * dim + k] = gr;
    }
}

size_t transr_backward_workspace_bytes(const kge_problem* p) {
    const size_t rows = (size_t)p->batch * (1 + (p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg));
    return (rows * p->dim * 4 + 255) / 256 * 256 + ((size_t)p->batch * p->dim * 4 + 255) / 256 * 256;
}

int launch_transr_backward(const kge_problem* p, const kge_tensors* t, const float* pos, const float* negs, const float* dpos,
                           const float* dneg, const kge_grads* g, void* ws, cudaStream_t s) {
    if (p->batch <= 0) return 0;
    GroupArgs a = group_args(p, t);
    if (p->neg_mode == KGE_NEG_NONE) { a.n_neg = 0; a.n_neg_head = 0; }
    const size_t rows = (size_t)p->batch * (1 + a.n_neg);
    TransRBwd w;
    w.pos = pos; w.negs = negs; w.dpos = dpos; w.dneg = dneg;
    w.gv = static_cast<float*>(ws);
    w.gd0 = reinterpret_cast<float*>(static_cast<char*>(ws) + (rows * p->dim * 4 + 255) / 256 * 256);
    w.g_neg = g->g_neg; w.g_head = g->g_head; w.g_tail = g->g_tail; w.g_rel = g->g_rel; w.dproj = g->g_rel2;
    const unsigned nt = (p->dim + TG_BN - 1) / TG_BN;
    const dim3 grid_rows(group_bound(p), 8);
    const dim3 grid_dp(group_bound(p), nt, nt);
#define KGE_CALL(T, I, V) transr_gv_kernel<T, I, V><<<grid_rows, 256, 0, s>>>(a, w)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("transr_gv_kernel");
#define KGE_CALL(T, I, V) transr_gd_kernel<T, I, V><<<grid_rows, 256, 0, s>>>(a, w)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("transr_gd_kernel");
#define KGE_CALL(T, I, V) transr_dproj_kernel<T, I, V><<<grid_dp, 256, 0, s>>>(a, w)
    KGE_TI_DISPATCH(KGE_CALL);
#undef KGE_CALL
    KGE_LAUNCH_CHECK("transr_dproj_kernel");
    const int wpb = 8;
    transr_reduce_kernel<<<(unsigned)((p->batch + wpb - 1) / wpb), wpb * 32, 0, s>>>(p->batch, p->dim, a.n_neg, a.n_neg_head, w);
    KGE_LAUNCH_CHECK("transr_reduce_kernel");
    return 0;
}
}  // namespace kge
