// Chunk-shared negatives: every triple of a chunk is scored against the same n_neg replacement rows
// (the layout of the reference's view-based negative example, apps/examples/examples.py:1434-1441),
// which turns the scorer into a (chunk x n_neg x dim) contraction per chunk.
//
//   forward   S[c][i][j] = score(anchor_i, x_j)                 pair_fwd_kernel   (OP_DIST / OP_DOT)
//   backward  GA[i]  = sum_j W_ij x_j   (+ rank-1 term, DIST)   pair_bwd_anchor_kernel
//             GX[j]  = sum_i W_ij a_i   (+ rank-1 term, DIST)   pair_bwd_neg_kernel
//   with W = dS for the dot-product models and W = dS / S for the distance models
//   (S = -||a_i - x_j||, so dS/dx_j = W (x_j - a_i) ... summed: GA_i = (sum_j W_ij) a_i - sum_j W_ij x_j,
//    GX_j = (sum_i W_ij) x_j - sum_i W_ij a_i).  Row / column sums of W are accumulated by the operand
//   loaders on the side, so W is never written to memory.
#include "tile_gemm.cuh"

namespace kge {

template <int MODEL> struct PairOp { static constexpr int value = OP_DOT; };
template <> struct PairOp<KGE_TRANSE> { static constexpr int value = OP_DIST; };

// ---- operand loaders ---------------------------------------------------------------------------------
// Anchor rows of the tile's triples, computed on the fly from the gathered h (or t) and r rows.
template <int MODEL, typename T, bool VEC>
struct AnchorLoader {
    static constexpr bool K_CONTIG = true;
    const T* own[2]; const T* rel[2]; const float* pre[2]; int dim; bool head;
    __device__ __forceinline__ float4 get(int row, int k) const {
        const int u = row >> 6;
        if (MODEL == KGE_RESCAL) {
            return pre[u] ? load_quad<float, VEC>(pre[u], k >> 2, dim) : f4(0.f);
        } else {
            if (own[u] == nullptr) return f4(0.f);
            const float4 o = load_quad<T, VEC>(own[u], k >> 2, dim);
            const float4 r = load_quad<T, VEC>(rel[u], k >> 2, dim);
            if (MODEL == KGE_TRANSE) return head ? o - r : o + r;
            if (MODEL == KGE_DISTMULT) return o * r;
            return head ? cmul_conj(o, r) : cmul(o, r);     // ComplEx
        }
    }
};
// Gathered table rows, quads along the row (k).
template <typename T, bool VEC>
struct RowLoaderK {
    static constexpr bool K_CONTIG = true;
    const T* row[2]; int dim;
    __device__ __forceinline__ float4 get(int r, int k) const {
        const int u = r >> 6;
        return row[u] ? load_quad<T, VEC>(row[u], k >> 2, dim) : f4(0.f);
    }
};

__device__ __forceinline__ float4 w_from(float4 ds, float4 s) {   // W = dS / S, 0 where S == 0
    return make_float4(s.x != 0.f ? ds.x / s.x : 0.f, s.y != 0.f ? ds.y / s.y : 0.f,
                       s.z != 0.f ? ds.z / s.z : 0.f, s.w != 0.f ? ds.w / s.w : 0.f);
}

// W rows of one chunk, quads along j (the reduction index of GA); accumulates row sums on the side.
template <bool DIST, bool VEC>
struct WRowLoader {
    static constexpr bool K_CONTIG = true;
    const float* ds[2]; const float* sc[2]; int n_neg; mutable float rs[2];
    __device__ __forceinline__ float4 get(int row, int k) const {
        const int u = row >> 6;
        if (ds[u] == nullptr) return f4(0.f);
        float4 w = load_quad<float, VEC>(ds[u], k >> 2, n_neg);
        if (DIST) { w = w_from(w, load_quad<float, VEC>(sc[u], k >> 2, n_neg)); rs[u] += hsum4(w); }
        return w;
    }
};
// W^T of one chunk: A(m = j, k = i) = W[i][j], quads along j; accumulates column sums on the side.
template <bool DIST, bool VEC>
struct WColLoader {
    static constexpr bool K_CONTIG = false;
    const float* ds; const float* sc; int n_neg; int chunk_rows; int j0; mutable float4 cs;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= chunk_rows) return f4(0.f);
        const long long off = (long long)k * n_neg;
        // quad index relative to the row start; rows start 16-byte aligned only if n_neg % 4 == 0 (VEC)
        float4 w = load_quad<float, VEC>(ds + off, (j0 + r4) >> 2, n_neg);
        if (DIST) { w = w_from(w, load_quad<float, VEC>(sc + off, (j0 + r4) >> 2, n_neg)); cs = cs + w; }
        return w;
    }
};
// Gathered table rows as the B operand of GA: B(k = j, n) = x_j[n0 + n], quads along n.
template <typename T, typename I, bool VEC>
struct NegRowsDirect {
    static constexpr bool K_CONTIG = false;
    const T* table; const void* ids; long long id0; int n_rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= n_rows) return f4(0.f);
        const long long id = load_id<I>(ids, id0 + k);
        return load_quad<T, VEC>(table + id * dim, (n0 + r4) >> 2, dim);
    }
};
// Dense fp32 rows as the B operand of GX: B(k = i, n) = anchors[i0 + k][n0 + n].
template <bool VEC>
struct DenseRowsDirect {
    static constexpr bool K_CONTIG = false;
    const float* base; int n_rows; int dim; int n0;
    __device__ __forceinline__ float4 get(int r4, int k) const {
        if (k >= n_rows) return f4(0.f);
        return load_quad<float, VEC>(base + (long long)k * dim, (n0 + r4) >> 2, dim);
    }
};

// ---- forward -----------------------------------------------------------------------------------------
template <int MODEL, typename T, typename I, bool VEC, bool VECOUT>
__global__ void __launch_bounds__(256, 2) pair_fwd_kernel(ScoreArgs a, int head) {
    __shared__ __align__(16) TileSmem sm;
    constexpr int OP = PairOp<MODEL>::value;
    if (a.guard != nullptr && *a.guard <= a.guard_cap) return;      // exact recomputation not needed
    const int tid = threadIdx.x;
    const int c = blockIdx.z, m0 = blockIdx.y * TG_BM, n0 = blockIdx.x * TG_BN;
    const long long i0 = (long long)c * a.chunk;
    const int rows = (int)min((long long)a.chunk, a.batch - i0);      // triples in this chunk
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* R = reinterpret_cast<const T*>(a.rel);

    AnchorLoader<MODEL, T, VEC> al;
    RowLoaderK<T, VEC> bl;
    al.dim = bl.dim = a.dim; al.head = head != 0;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int m = m0 + (tid >> 2) + 64 * u;
        al.own[u] = nullptr; al.rel[u] = nullptr; al.pre[u] = nullptr;
        if (m < rows) {
            const long long i = i0 + m;
            if (MODEL == KGE_RESCAL) al.pre[u] = a.anchors + i * a.dim;
            else {
                al.own[u] = E + load_id<I>(head ? a.t : a.h, i) * a.dim;
                al.rel[u] = R + load_id<I>(a.r, i) * a.dim;
            }
        }
        const int n = n0 + (tid >> 2) + 64 * u;
        bl.row[u] = (n < a.n_neg) ? E + load_id<I>(a.neg, (long long)c * a.n_neg + n) * a.dim : nullptr;
    }

    float acc[8][8];
    tile_mainloop<OP>(al, bl, a.dim, sm, acc);

    float* out = a.negs + (i0 + m0) * (long long)a.n_neg + n0;
    const int n_neg = a.n_neg;
    auto ep = [&](int row, int col4, float4 v) {
        if (m0 + row >= rows) return;
        if (OP == OP_DIST) v = make_float4(-sqrtf(v.x), -sqrtf(v.y), -sqrtf(v.z), -sqrtf(v.w));
        float* p = out + (long long)row * n_neg + col4;
        const int n = n0 + col4;
        if (VECOUT) { if (n < n_neg) *reinterpret_cast<float4*>(p) = v; }
        else {
            if (n + 0 < n_neg) p[0] = v.x;
            if (n + 1 < n_neg) p[1] = v.y;
            if (n + 2 < n_neg) p[2] = v.z;
            if (n + 3 < n_neg) p[3] = v.w;
        }
    };
    tile_epilogue(acc, ep);
}

// ---- backward: anchor gradients  GA[i][:] = sum_j W_ij x_j  (DIST: rowsum_i a_i - that) -------------------
template <bool DIST, typename T, typename I, bool VEC, bool VECW>
__global__ void __launch_bounds__(256, 2) pair_bwd_anchor_kernel(ScoreArgs a, const float* anchors, float* ga) {
    __shared__ __align__(16) TileSmem sm;
    __shared__ float rowsum[TG_BM];
    const int tid = threadIdx.x;
    const int c = blockIdx.z, m0 = blockIdx.y * TG_BM, n0 = blockIdx.x * TG_BN;
    const long long i0 = (long long)c * a.chunk;
    const int rows = (int)min((long long)a.chunk, a.batch - i0);

    WRowLoader<DIST, VECW> al;
    al.n_neg = a.n_neg;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int m = m0 + (tid >> 2) + 64 * u;
        al.rs[u] = 0.f;
        if (m < rows) { al.ds[u] = a.dneg + (i0 + m) * (long long)a.n_neg; al.sc[u] = a.negs + (i0 + m) * (long long)a.n_neg; }
        else { al.ds[u] = nullptr; al.sc[u] = nullptr; }
    }
    NegRowsDirect<T, I, VEC> bl;
    bl.table = reinterpret_cast<const T*>(a.ent); bl.ids = a.neg; bl.id0 = (long long)c * a.n_neg;
    bl.n_rows = a.n_neg; bl.dim = a.dim; bl.n0 = n0;

    float acc[8][8];
    tile_mainloop<OP_DOT>(al, bl, a.n_neg, sm, acc);

    if (DIST) {   // the 4 threads sharing a row each saw a quarter of its k-quads
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            float v = al.rs[u];
            v += __shfl_xor_sync(kFull, v, 1);
            v += __shfl_xor_sync(kFull, v, 2);
            if ((tid & 3) == 0) rowsum[(tid >> 2) + 64 * u] = v;
        }
        __syncthreads();
    }
    const int dim = a.dim;
    auto ep = [&](int row, int col4, float4 v) {
        const int n = n0 + col4;
        if (m0 + row >= rows || n >= dim) return;
        const long long i = i0 + m0 + row;
        if (DIST) {
            const float rs = rowsum[row];
            const float4 an = load_quad<float, VEC>(anchors + i * dim, n >> 2, dim);
            v = make_float4(fmaf(rs, an.x, -v.x), fmaf(rs, an.y, -v.y), fmaf(rs, an.z, -v.z), fmaf(rs, an.w, -v.w));
        }
        store_quad<VEC>(ga + i * dim, n >> 2, dim, v);
    };
    tile_epilogue(acc, ep);
}

// ---- backward: negative-row gradients  GX[j][:] = sum_i W_ij a_i  (DIST: colsum_j x_j - that) ----------------
template <bool DIST, typename T, typename I, bool VEC, bool VECW>
__global__ void __launch_bounds__(256, 2) pair_bwd_neg_kernel(ScoreArgs a, const float* anchors) {
    __shared__ __align__(16) TileSmem sm;
    __shared__ float colpart[8][TG_BM];
    const int tid = threadIdx.x;
    const int c = blockIdx.z, m0 = blockIdx.y * TG_BM, n0 = blockIdx.x * TG_BN;   // m = negative j
    const long long i0 = (long long)c * a.chunk;
    const int rows = (int)min((long long)a.chunk, a.batch - i0);

    WColLoader<DIST, VECW> al;
    al.ds = a.dneg + i0 * (long long)a.n_neg; al.sc = a.negs + i0 * (long long)a.n_neg;
    al.n_neg = a.n_neg; al.chunk_rows = rows; al.j0 = m0; al.cs = f4(0.f);
    DenseRowsDirect<VEC> bl;
    bl.base = anchors + i0 * a.dim; bl.n_rows = rows; bl.dim = a.dim; bl.n0 = n0;

    float acc[8][8];
    tile_mainloop<OP_DOT>(al, bl, rows, sm, acc);

    if (DIST) {   // thread (warp w, lane l) summed W over k == w (mod 8) for columns 4l..4l+3
        const int w = tid >> 5, l = tid & 31;
        colpart[w][4 * l + 0] = al.cs.x; colpart[w][4 * l + 1] = al.cs.y;
        colpart[w][4 * l + 2] = al.cs.z; colpart[w][4 * l + 3] = al.cs.w;
        __syncthreads();
        if (tid < TG_BM) {
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) s += colpart[q][tid];
            colpart[0][tid] = s;
        }
        __syncthreads();
    }
    const int dim = a.dim;
    const T* E = reinterpret_cast<const T*>(a.ent);
    auto ep = [&](int row, int col4, float4 v) {
        const int n = n0 + col4;
        const int j = m0 + row;
        if (j >= a.n_neg || n >= dim) return;
        const long long slot = (long long)c * a.n_neg + j;
        if (DIST) {
            const float cs = colpart[0][row];
            const long long id = load_id<I>(a.neg, slot);
            const float4 x = load_quad<T, VEC>(E + id * dim, n >> 2, dim);
            v = make_float4(fmaf(cs, x.x, -v.x), fmaf(cs, x.y, -v.y), fmaf(cs, x.z, -v.z), fmaf(cs, x.w, -v.w));
        }
        store_quad<VEC>(a.g_neg + slot * dim, n >> 2, dim, v);
    };
    tile_epilogue(acc, ep);
}

// ---- host dispatch ---------------------------------------------------------------------------------
static inline dim3 pair_grid(int mrows, int ncols, long long nchunks) {
    return dim3((unsigned)((ncols + TG_BN - 1) / TG_BN), (unsigned)((mrows + TG_BM - 1) / TG_BM), (unsigned)nchunks);
}

template <int MODEL, typename T, typename I>
static int pair_fwd_go(const ScoreArgs& a, int head, cudaStream_t s) {
    const long long nchunks = (a.batch + a.chunk - 1) / a.chunk;
    const dim3 grid = pair_grid(a.chunk, a.n_neg, nchunks);
    const bool vec = a.dim % 4 == 0, vout = a.n_neg % 4 == 0;
    if (vec && vout) pair_fwd_kernel<MODEL, T, I, true, true><<<grid, 256, 0, s>>>(a, head);
    else if (vec) pair_fwd_kernel<MODEL, T, I, true, false><<<grid, 256, 0, s>>>(a, head);
    else if (vout) pair_fwd_kernel<MODEL, T, I, false, true><<<grid, 256, 0, s>>>(a, head);
    else pair_fwd_kernel<MODEL, T, I, false, false><<<grid, 256, 0, s>>>(a, head);
    KGE_LAUNCH_CHECK("pair_fwd_kernel");
    return 0;
}
template <int MODEL>
static int pair_fwd_types(const ScoreArgs& a, int head, cudaStream_t s) {
    if (a.dtype == KGE_F32)
        return a.id_bits == 64 ? pair_fwd_go<MODEL, float, int64_t>(a, head, s) : pair_fwd_go<MODEL, float, int32_t>(a, head, s);
    return a.id_bits == 64 ? pair_fwd_go<MODEL, __nv_bfloat16, int64_t>(a, head, s)
                           : pair_fwd_go<MODEL, __nv_bfloat16, int32_t>(a, head, s);
}
int launch_pair_forward(const ScoreArgs& a, int head, cudaStream_t s) {
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    switch (a.model) {
        case KGE_TRANSE: return pair_fwd_types<KGE_TRANSE>(a, head, s);
        case KGE_DISTMULT: return pair_fwd_types<KGE_DISTMULT>(a, head, s);
        case KGE_COMPLEX: return pair_fwd_types<KGE_COMPLEX>(a, head, s);
        case KGE_RESCAL: return pair_fwd_types<KGE_RESCAL>(a, head, s);
        default: break;
    }
    set_error("model %d is not supported with chunk-shared negatives", a.model);
    return KGE_E_UNSUPPORTED;
}

template <bool DIST, typename T, typename I>
static int pair_bwd_go(const ScoreArgs& a, const float* anchors, float* ga, cudaStream_t s) {
    const long long nchunks = (a.batch + a.chunk - 1) / a.chunk;
    const bool vec = a.dim % 4 == 0, vw = a.n_neg % 4 == 0;
    const dim3 g1 = pair_grid(a.chunk, a.dim, nchunks);
    const dim3 g2 = pair_grid(a.n_neg, a.dim, nchunks);
#define KGE_PB(V, VW)                                                                                   \
    do {                                                                                                \
        pair_bwd_anchor_kernel<DIST, T, I, V, VW><<<g1, 256, 0, s>>>(a, anchors, ga);                   \
        KGE_LAUNCH_CHECK("pair_bwd_anchor_kernel");                                                     \
        pair_bwd_neg_kernel<DIST, T, I, V, VW><<<g2, 256, 0, s>>>(a, anchors);                          \
        KGE_LAUNCH_CHECK("pair_bwd_neg_kernel");                                                        \
    } while (0)
    if (vec && vw) KGE_PB(true, true);
    else if (vec) KGE_PB(true, false);
    else if (vw) KGE_PB(false, true);
    else KGE_PB(false, false);
#undef KGE_PB
    return 0;
}
// anchors: (batch, dim) fp32 anchors of the replaced side; ga: (batch, dim) output.
int launch_pair_backward(const ScoreArgs& a, const float* anchors, float* ga, cudaStream_t s) {
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    const bool dist = a.model == KGE_TRANSE;
    if (a.model != KGE_TRANSE && a.model != KGE_DISTMULT && a.model != KGE_COMPLEX && a.model != KGE_RESCAL) {
        set_error("model %d is not supported with chunk-shared negatives", a.model);
        return KGE_E_UNSUPPORTED;
    }
#define KGE_PT(D)                                                                                          \
    if (a.dtype == KGE_F32)                                                                                \
        return a.id_bits == 64 ? pair_bwd_go<D, float, int64_t>(a, anchors, ga, s)                         \
                               : pair_bwd_go<D, float, int32_t>(a, anchors, ga, s);                        \
    return a.id_bits == 64 ? pair_bwd_go<D, __nv_bfloat16, int64_t>(a, anchors, ga, s)                     \
                           : pair_bwd_go<D, __nv_bfloat16, int32_t>(a, anchors, ga, s);
    if (dist) { KGE_PT(true) } else { KGE_PT(false) }
#undef KGE_PT
}

}  // namespace kge
