// Tensor-core path of the chunk-shared scorers (fp32 tables, "3xTF32").  Per chunk c the work is three contractions
//
//   forward   S[i][j]   = sum_k a_i[k] x_j[k]                       (anchors x negative rows, K = dim)
//   backward  GA[i][:]  = sum_j W_ij x_j          (K = n_neg)       W = dS (dot-product scorers) or dS / S (TransE)
//             GX[j][:]  = sum_i W_ij a_i          (K = chunk)
//
// all run by ONE kernel, umma_gemm_kernel, on the 5th-generation tensor cores:
//   * operands are dense fp32 matrices split into hi = top 19 bits (exact in tf32) and lo = tf32(v - hi), written
//     once by pack kernels (anchors are computed there from the gathered h/t and r rows; W from dS and S);
//   * TMA (3-D tensor maps: batch, rows, cols; 128-byte swizzle; out-of-range reads as zero) feeds a shared-memory
//     ring; an operand is used K-major (rows of 32 k-values) or MN-major (32 m/n-values per k-row) as it lies in
//     memory, so W, X and A are never transposed;
//   * one elected thread issues tcgen05.mma kind::tf32 for lo*hi + hi*lo + hi*hi into an fp32 accumulator in tensor
//     memory; eight epilogue warps read it back with tcgen05.ld and apply the scorer's epilogue; the kernel is
//     persistent with two accumulators, so that epilogue overlaps the next tile's main loop.
//   The split makes products exact to ~2^-20 relative, inside the 1e-4 tolerance of the fp32 path (a single tf32
//   pass, 2^-11, would not be).  TransE's distance uses |a|^2 + |x|^2 - 2 a.x; entries where that form cancels
//   (d^2 < 2^-6 (|a|^2 + |x|^2)) are listed by the epilogue and recomputed exactly from the rows by a fix-up kernel;
//   if the list overflows, the exact CUDA-core kernel recomputes the whole matrix (device-side guard, no host sync).
//
// Replaces the scalar-FMA inner loops that cuke generates for bvv over gathered rows
// (apps/kge/kge.py:13-15, pycuke1/codegen/gpu.py:43-51).
#include <string.h>
#include <atomic>
#include "rows.cuh"
#include "umma.cuh"

namespace kge {

int launch_pair_forward(const ScoreArgs& a, int head, cudaStream_t s);     // pairwise.cu (exact CUDA-core kernel)

// ---- host: tensor maps -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tensor_map_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t batch, uint64_t rows, uint64_t cols,
                       uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_rows, uint32_t box_cols, bool atom32) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return KGE_E_DEVICE; }
    cuuint64_t gdim[3] = {cols, rows, batch};
    cuuint64_t gstride[2] = {row_stride_bytes, batch_stride_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                    const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return KGE_E_DEVICE; }
    return 0;
}
int make_tensor_map_slabs(CUtensorMap* out, const void* base, int elem_bytes, uint64_t batch, uint64_t krows, uint64_t cols_padded,
                          uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_krows, uint32_t box_slabs) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return KGE_E_DEVICE; }
    const uint32_t slab_cols = 128 / elem_bytes;
    if (cols_padded % slab_cols != 0) { set_error("slab tensor map: %llu columns are not whole slabs", (unsigned long long)cols_padded); return KGE_E_SHAPE; }
    cuuint64_t gdim[4] = {slab_cols, krows, cols_padded / slab_cols, batch};
    cuuint64_t gstride[3] = {row_stride_bytes, 128, batch_stride_bytes};
    cuuint32_t box[4] = {slab_cols, box_krows, box_slabs, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                    const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    elem_bytes == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (slabs) failed with CUresult %d", (int)r); return KGE_E_DEVICE; }
    return 0;
}
int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
    return make_tensor_map_3d(out, base, elem_bytes, 1, rows, cols, row_stride_bytes, rows * row_stride_bytes, box_rows, box_cols);
}

// ---- operand split ----------------------------------------------------------------------------------------------
// A contraction of fp32 operands runs on the tensor cores as three MMAs over a two-term split of each operand,
// v ~ hi + lo:  lo*hi + hi*lo + hi*hi  (the lo*lo term is below the target accuracy).  Two element formats:
//   ES = 2  bf16 split (default): hi = bf16(v), lo = bf16(v - hi); hi + lo carries 16 mantissa bits, products are exact to
//           ~2^-16 relative, and the MMAs are kind::f16 at the full tensor rate with 4 bytes of operands per element.
//   ES = 4  tf32 split in fp32 storage: hi = top 19 bits of v (exact in tf32), lo = v - hi exactly; products exact to
//           ~2^-20, kind::tf32 at half the rate with 8 bytes per element ("3xTF32").
// Both stay inside the 1e-4 tolerance of the fp32 path (a single bf16 or tf32 pass, 2^-9 / 2^-11, would not).
__device__ __forceinline__ float tf32_trunc(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }
template <int ES> struct Split;
template <> struct Split<4> {
    using T = float;
    __device__ static __forceinline__ void put(T* hi, T* lo, float v) { const float h = tf32_trunc(v); *hi = h; *lo = v - h; }
    __device__ static __forceinline__ float get(const T* hi, const T* lo) { return __ldg(hi) + __ldg(lo); }
};
template <> struct Split<2> {
    using T = __nv_bfloat16;
    __device__ static __forceinline__ void put(T* hi, T* lo, float v) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        *hi = h; *lo = __float2bfloat16_rn(v - __bfloat162float(h));
    }
    __device__ static __forceinline__ float get(const T* hi, const T* lo) { return __bfloat162float(*hi) + __bfloat162float(*lo); }
};
// quad (4 consecutive elements) forms for the row kernels; `b2` (bf16 split only, may be NULL) receives the third term
// v - hi - lo, which makes hi + lo + b2 == v exactly for the rows an epilogue has to rebuild
__device__ __forceinline__ void put_quad(float* hi, float* lo, float* /*b2*/, float4 v) {
    const float4 h = make_float4(tf32_trunc(v.x), tf32_trunc(v.y), tf32_trunc(v.z), tf32_trunc(v.w));
    *reinterpret_cast<float4*>(hi) = h;
    *reinterpret_cast<float4*>(lo) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
}
__device__ __forceinline__ uint2 bf16x4(float4 v, float4& back) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x, v.y), p1 = __floats2bfloat162_rn(v.z, v.w);
    const float2 f0 = __bfloat1622float2(p0), f1 = __bfloat1622float2(p1);
    back = make_float4(f0.x, f0.y, f1.x, f1.y);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&p0); u.y = *reinterpret_cast<unsigned*>(&p1);
    return u;
}
__device__ __forceinline__ void put_quad(__nv_bfloat16* hi, __nv_bfloat16* lo, __nv_bfloat16* b2, float4 v) {
    float4 h, l, t;
    *reinterpret_cast<uint2*>(hi) = bf16x4(v, h);
    const float4 r1 = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
    *reinterpret_cast<uint2*>(lo) = bf16x4(r1, l);
    if (b2) *reinterpret_cast<uint2*>(b2) = bf16x4(make_float4(r1.x - l.x, r1.y - l.y, r1.z - l.z, r1.w - l.w), t);
}

// ---- pack kernels --------------------------------------------------------------------------------------------
// Rows [0, n_a): anchors of the triples; rows [n_a, n_a + n_x): the negative rows, in id-list order.
// One warp per row; hi / lo (/ b2) are (n_a + n_x) rows of split elements with a pitch of ldp elements (dim rounded up to
// whole 128-byte slabs, the padding written as zero), sq (n_a + n_x) the squared norms of the unsplit rows.
template <int MODEL, typename T, typename I, int NV, int ES>
__global__ void __launch_bounds__(256) tc_pack_kernel(ScoreArgs a, int head, long long n_a, long long n_x, int ldp,
                                                      void* hi_v, void* lo_v, void* b2_v, float* sq) {
    using S = typename Split<ES>::T;
    S* hi = static_cast<S*>(hi_v); S* lo = static_cast<S*>(lo_v); S* b2 = static_cast<S*>(b2_v);
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_a + n_x) return;
    const int dim = a.dim;
    const T* E = reinterpret_cast<const T*>(a.ent);
    Row<NV> v;
    if (row < n_a) {
        if (MODEL == KGE_RESCAL) {
            load_row_f32<NV, true>(v, a.anchors + row * dim, dim, lane);
        } else {
            const T* R = reinterpret_cast<const T*>(a.rel);
            Row<NV> o, r;
            load_row<T, NV, true>(o, E + load_id<I>(head ? a.t : a.h, row) * dim, dim, lane);
            load_row<T, NV, true>(r, R + load_id<I>(a.r, row) * dim, dim, lane);
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                if (MODEL == KGE_TRANSE) v.v[q] = head ? o.v[q] - r.v[q] : o.v[q] + r.v[q];
                else if (MODEL == KGE_DISTMULT) v.v[q] = o.v[q] * r.v[q];
                else v.v[q] = head ? cmul_conj(o.v[q], r.v[q]) : cmul(o.v[q], r.v[q]);
            }
        }
    } else {
        load_row<T, NV, true>(v, E + load_id<I>(a.neg, row - n_a) * dim, dim, lane);
    }
    float s = 0.f;
    const long long base = row * ldp;
#pragma unroll
    for (int q = 0; q < NV; ++q) {
        s = dot4(v.v[q], v.v[q], s);
        const int k = 4 * (lane + 32 * q);
        if (k < dim) put_quad(hi + base + k, lo + base + k, b2 ? b2 + base + k : nullptr, v.v[q]);
    }
    for (int k = dim + 4 * lane; k < ldp; k += 128)       // zero padding up to the slab boundary
        put_quad(hi + base + k, lo + base + k, b2 ? b2 + base + k : nullptr, make_float4(0.f, 0.f, 0.f, 0.f));
    s = warp_sum(s);
    if (lane == 0 && sq) sq[row] = s;
}

// W = dS split into hi / lo (dot-product scorers).  One warp per row of the (batch, n_neg) matrix; hi / lo have a pitch
// of ldw floats (n_neg rounded up to whole slabs, padding zero).
template <int ES>
__global__ void __launch_bounds__(256) tc_pack_w_kernel(const float* ds, long long rows, int n_neg, int ldw, void* hi_v, void* lo_v) {
    using S = typename Split<ES>::T;
    S* hi = static_cast<S*>(hi_v); S* lo = static_cast<S*>(lo_v);
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* d = ds + row * n_neg;
    for (int j = lane; j < ldw; j += 32) Split<ES>::put(hi + row * ldw + j, lo + row * ldw + j, j < n_neg ? d[j] : 0.f);
}
// TransE: W = dS / S (0 where S == 0) split into hi / lo, with its row sums and per-block column sums in the same pass.
// A block takes TW_ROWS consecutive rows of one chunk; thread t owns columns t, t + 256, ...: for a fixed row the block
// reads consecutive columns (coalesced), a thread's column sum stays in a register across the rows, and the row sums are
// reduced once per block.  colpart[(chunk * blocks_per_chunk + block)][j] holds the block's column sums; all sums are
// added in a fixed order, so the result does not depend on scheduling.
constexpr int TW_ROWS = 32;
template <int ES>
__global__ void __launch_bounds__(256) tc_pack_w_sums_kernel(const float* __restrict__ ds, const float* __restrict__ sc, int chunk, int n_neg,
                                                             int ldw, void* hi_v, void* lo_v,
                                                             float* __restrict__ rowsum, float* __restrict__ colpart) {
    using S = typename Split<ES>::T;
    S* hi = static_cast<S*>(hi_v); S* lo = static_cast<S*>(lo_v);
    __shared__ float row_part[8][TW_ROWS];
    const int c = blockIdx.y, r0 = blockIdx.x * TW_ROWS;
    const int rows = min(TW_ROWS, chunk - r0);
    const long long row0 = (long long)c * chunk + r0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float rs[TW_ROWS];
#pragma unroll
    for (int i = 0; i < TW_ROWS; ++i) rs[i] = 0.f;
    float* cp = colpart + ((long long)c * gridDim.x + blockIdx.x) * n_neg;
    for (int j = threadIdx.x; j < ldw; j += 256) {
        float cs = 0.f;
        const bool in = j < n_neg;
        float dv[TW_ROWS], sv[TW_ROWS];
#pragma unroll
        for (int i = 0; i < TW_ROWS; ++i) {          // all loads of the column strip first
            const bool ok = in && i < rows;
            const long long o = (row0 + i) * n_neg + j;
            dv[i] = ok ? __ldg(ds + o) : 0.f;
            sv[i] = ok ? __ldg(sc + o) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < TW_ROWS; ++i) {
            if (i < rows) {
                const float w = sv[i] != 0.f ? dv[i] / sv[i] : 0.f;
                Split<ES>::put(hi + (row0 + i) * ldw + j, lo + (row0 + i) * ldw + j, w);
                cs += w;
                rs[i] += w;
            }
        }
        if (in) cp[j] = cs;
    }
#pragma unroll
    for (int i = 0; i < TW_ROWS; ++i) {
        const float v = warp_sum(rs[i]);
        if (lane == 0) row_part[warp][i] = v;
    }
    __syncthreads();
    if (threadIdx.x < rows) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += row_part[w][threadIdx.x];
        rowsum[row0 + threadIdx.x] = v;
    }
}
// Column sums of W per chunk from the per-block sums: colsum[c][j] = sum_b colpart[c][b][j], ascending b.
__global__ void __launch_bounds__(256) tc_colsum_kernel(const float* colpart, int blocks_per_chunk, int n_neg, float* colsum) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    const int c = blockIdx.y;
    if (j >= n_neg) return;
    const float* cp = colpart + (long long)c * blocks_per_chunk * n_neg + j;
    float s = 0.f;
    for (int b = 0; b < blocks_per_chunk; ++b) s += cp[(long long)b * n_neg];
    colsum[(long long)c * n_neg + j] = s;
}

// ---- the tensor-core tile kernels ------------------------------------------------------------------------------
constexpr int UM_BM = 128, UM_BK = 32;                       // 32 fp32 = one 128-byte swizzle row
constexpr int UM_A_BYTES = UM_BM * UM_BK * 4;                // 16 KiB per A tile (either major)
constexpr int UM_SLAB_BYTES = UM_BK * 128;                   // one MN-major slab: 32 k-rows x 128 bytes
constexpr int UM_EPI_BYTES = 8 * 32 * 32 * 4 + 8 * 32 * 4;   // per epilogue warp: one 32x32 fp32 square, then one 32-float strip
constexpr int UM_TAIL_BYTES = 256 + UM_EPI_BYTES;            // barriers and tensor-memory slot, then the staging squares
constexpr int UM_MAX_SMEM = 227 * 1024;                     // opt-in shared memory per CTA on sm_100

constexpr long long kTailSide = 1LL << 40;      // added to a slot number in row_dst: the row's gradient enters with a minus sign
enum { EP_STORE = 0, EP_DIST = 1, EP_RANK1 = 2, EP_NORM = 3, EP_GV = 4, EP_SCATTER = 5, EP_LOSS = 6 };

struct GemmTc {
    int m_rows, n_cols, k_len;        // extents per batch
    int batch;
    int bn;                           // tile width (multiple of 16, <= 256)
    int a_mn, b_mn;                   // operand majors: 0 K-major, 1 MN-major
    int stages;
    int ep;                           // epilogue
    float* out; long long out_ld; long long out_batch_rows;      // out[(b * out_batch_rows + m) * out_ld + n]
    // EP_DIST
    const float* sq_a; const float* sq_b;                        // (batch * m_rows), (batch * n_cols)
    unsigned long long* fix_count; unsigned long long* fix_list; unsigned long long fix_cap;
    // EP_RANK1: out = scale[b * m_rows + m] * (y_hi + y_lo)[(b * m_rows + m) * out_ld + n] - acc
    const float* scale; const void* y_hi; const void* y_lo;      // y in the operands' split format
    // element type and split: elem_bytes 4 (tf32) or 2 (bf16); passes 3 (hi/lo split) or 1 (hi only)
    int elem_bytes; int passes;
    // grouped mode (relation-grouped projections): tile list in device memory, one n-tile
    const int4* tile_tab; const long long* n_tiles_dev; long long tile_cap;       // (first row, z, group, valid rows)
    // EP_NORM: score = -|| acc + rel_vec[z] ||, scattered through row_dst
    const long long* row_dst; float* pos_out; float* neg_out; const void* rel_vec; int rel_is_bf16;
    // grouped-K mode (sum over the rows of a relation group): tile = (first k-row, k-rows, m0, output batch)
    int group_k;
    // EP_GV: gv_out[row] = bf16(coef[row] * (acc + rel_vec[z]));  EP_SCATTER: rows go to neg_out (signed by side) / pos_out
    const float* coef; __nv_bfloat16* gv_out; int sc_n_neg; int sc_n_neg_head;
    // EP_LOSS: the score never leaves the tile.  loss += neg_w * softplus(S), dS = neg_w * sigmoid(S), and
    // W = dS (dot-product scorers) or dS / S (loss_dist: S = -sqrt(sq_a + sq_b - 2 acc), exact where that cancels) is
    // stored split into w_hi / w_lo (pitch ldw) for the backward products, with partial row sums
    // rowpart[(n_tile * 2 + half)][row], partial column sums colpart[(batch * ceil(m_rows / 32) + row block)][col]
    // and one loss partial per epilogue warp and tile, loss_part[slot].
    void* w_hi; void* w_lo; long long ldw; float neg_w; int loss_dist;      // W in the operands' split format, pitch in elements
    float* rowpart; float* colpart; float* loss_part;
    const void* ex_a_hi; const void* ex_a_lo; const void* ex_x_hi; const void* ex_x_lo; long long ex_ld;   // exact rows: hi + lo
    const void* ex_a_b2; const void* ex_x_b2;                     // (+ b2 for the bf16 split)
    int pair;                         // 1: CTA pairs (256-row tiles, umma_pair_kernel)
    int a_slabs4d, b_slabs4d;         // MN-major operand read through a 4-D slab map: one copy per stage instead of one per slab
    long long y_ld;                   // EP_RANK1: row pitch of y_hi / y_lo
    int32_t* err;
};

// One special-function instruction each (flush-to-zero forms: no denormal fix-up code around them); relative error ~2^-22.
__device__ __forceinline__ float sqrt_approx(float x) { float r; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float ex2_approx(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float lg2_approx(float x) { float r; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float rcp_approx(float x) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
// log1p(e) for e in [0, 1]: lg2(1 + e) ln 2, or e - e^2/2 where 1 + e would round the small term away
__device__ __forceinline__ float log1p_unit(float e) {
    const float big = lg2_approx(1.f + e) * 0.69314718f;
    return e < 0.00024414062f ? e * fmaf(-0.5f, e, 1.f) : big;
}

constexpr int UM_THREADS = 320;      // warp 0: TMA, warp 1: MMA + tensor-memory owner, warps 2..9: epilogue
// The relation-grouped instantiation runs TWO sets of eight epilogue warps (warps 2..9 and 10..17), one per accumulator
// buffer: its tiles are small (one k-pass of <= 256) and an epilogue is a chain of dependent latencies (tile record, per-row
// operands, tensor-memory reads), so two tiles are drained at the same time.  Its epilogues need 90 registers, which
// leaves room for 576 threads; the dense epilogues (168 registers) stay with one set.
constexpr int UM_THREADS_GROUPED = 64 + 2 * 256;
constexpr int UM_EPI_WARPS = 8;

// Epilogue of one 128-row x bn_tile accumulator, run by the eight epilogue warps of a CTA.  A warp may only read the
// tensor-memory lane quarter (warp % 4); the two warps of a quarter take alternate 32-column chunks.  m0 is the first
// row of THIS CTA's 128 rows.  `drained` is the (shared::cluster) address of the barrier that hands the accumulator
// back to the MMA thread; every warp arrives on it once its tensor-memory reads are done.
//
// tcgen05.ld hands each thread one ROW of the chunk (32 consecutive columns), and the epilogues work in that layout:
// a thread's 32 values are one contiguous 128-byte (fp32) or 64-byte (bf16) piece of its destination row, written with
// 16-byte stores; everything per ROW (squared norm, scale, destination pointers) is a register of the owning thread
// computed once per tile; a per-COLUMN operand (the squared norms of the distance forms) sits in a 32-float strip of the
// warp, refilled per chunk and read as 128-bit broadcasts; the 32 elements of a thread are 32 independent dependency
// chains, which is what keeps the special-function pipe busy with two warps per scheduler.  Only the column sums of the
// fused distance form cross rows: they go through the warp's XOR-swizzled 32x32 square once per chunk.
// GROUP selects which epilogues an instantiation of the one-CTA kernel carries: G_DENSE the dense chunk-shared products
// (store, distance, rank-1, fused loss; epilogue_tile below), G_GROUPED the relation-grouped products (store, norm, dL/dv
// rows, scatter; epilogue_grouped).  Two instantiations keep the register allocation of each set independent of the other.
enum { G_DENSE = 0, G_GROUPED = 1 };

// One 32-byte global store (sm_100: 256-bit vector accesses).  A thread-per-row epilogue issues one store request per
// lane - the lanes of a warp write 32 different rows - and the L1 / L2 path takes requests, not bytes: a request that
// fills a whole 32-byte sector moves twice the data of a 16-byte one at the same cost.  p must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4, uint32_t a5,
                                             uint32_t a6, uint32_t a7) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :: "l"(p), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7) : "memory");
}
// 32 fp32 values of one row -> out[0..lim): vector stores when the row is 16-byte aligned and lim a multiple of 4
// (32-byte stores where the address allows, else 16-byte ones)
__device__ __forceinline__ void store_row32(float* out, const float (&v)[32], int lim, bool vec) {
    if (vec && (reinterpret_cast<uintptr_t>(out) & 31) == 0 && (lim & 7) == 0) {
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8)
            if (8 * j8 < lim)
                st_global_v8(out + 8 * j8, __float_as_uint(v[8 * j8]), __float_as_uint(v[8 * j8 + 1]), __float_as_uint(v[8 * j8 + 2]),
                             __float_as_uint(v[8 * j8 + 3]), __float_as_uint(v[8 * j8 + 4]), __float_as_uint(v[8 * j8 + 5]),
                             __float_as_uint(v[8 * j8 + 6]), __float_as_uint(v[8 * j8 + 7]));
    } else if (vec) {
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4)
            if (4 * j4 < lim) *reinterpret_cast<float4*>(out + 4 * j4) = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < lim) out[j] = v[j];
    }
}
// 32 values of one row as split elements: columns [0, wlim) of hi / lo, wlim a multiple of 16
__device__ __forceinline__ void put_row32(float* hi, float* lo, const float (&v)[32], int wlim) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4)
        if (4 * j4 < wlim) put_quad(hi + 4 * j4, lo + 4 * j4, nullptr, make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]));
}
// (wlim is a multiple of 16 and the row pieces start on 32-byte boundaries: 16 elements = one 32-byte store per part)
__device__ __forceinline__ void put_row32(__nv_bfloat16* hi, __nv_bfloat16* lo, const float (&v)[32], int wlim) {
#pragma unroll
    for (int j16 = 0; j16 < 2; ++j16) {
        if (16 * j16 < wlim) {
            uint32_t hw[8], lw[8];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int j = 16 * j16 + 4 * q4;
                float4 h, t;
                const uint2 a = bf16x4(make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]), h);
                const uint2 l = bf16x4(make_float4(v[j] - h.x, v[j + 1] - h.y, v[j + 2] - h.z, v[j + 3] - h.w), t);
                hw[2 * q4] = a.x; hw[2 * q4 + 1] = a.y; lw[2 * q4] = l.x; lw[2 * q4 + 1] = l.y;
            }
            st_global_v8(hi + 16 * j16, hw[0], hw[1], hw[2], hw[3], hw[4], hw[5], hw[6], hw[7]);
            st_global_v8(lo + 16 * j16, lw[0], lw[1], lw[2], lw[3], lw[4], lw[5], lw[6], lw[7]);
        }
    }
}
// y[0..32) = hi + lo of 32 consecutive split elements (16-byte aligned; the pitch padding makes the whole read legal)
__device__ __forceinline__ void get_row32(const float* hi, const float* lo, float (&y)[32]) {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
        const float4 h = __ldg(reinterpret_cast<const float4*>(hi) + j4), l = __ldg(reinterpret_cast<const float4*>(lo) + j4);
        y[4 * j4] = h.x + l.x; y[4 * j4 + 1] = h.y + l.y; y[4 * j4 + 2] = h.z + l.z; y[4 * j4 + 3] = h.w + l.w;
    }
}
__device__ __forceinline__ void get_row32(const __nv_bfloat16* hi, const __nv_bfloat16* lo, float (&y)[32]) {
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
        const uint4 h = __ldg(reinterpret_cast<const uint4*>(hi) + j8), l = __ldg(reinterpret_cast<const uint4*>(lo) + j8);
        const uint32_t hw[4] = {h.x, h.y, h.z, h.w}, lw[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {      // a 32-bit word holds two bf16: the low half is the even element
            y[8 * j8 + 2 * i] = __uint_as_float(hw[i] << 16) + __uint_as_float(lw[i] << 16);
            y[8 * j8 + 2 * i + 1] = __uint_as_float(hw[i] & 0xFFFF0000u) + __uint_as_float(lw[i] & 0xFFFF0000u);
        }
    }
}

// `acc_full` / `aph`: barrier and phase that announce the finished accumulator.  The epilogue waits on it itself, after it
// has requested everything that does not depend on the accumulator (per-row operands, the first chunk's per-column
// operands): the accumulator buffer is then held only for the tensor-memory reads and the arithmetic, not for the
// latency of those loads.  Returns false if the wait ran out (nothing was read or written for this tile).
template <int GROUP, int ES>
__device__ __forceinline__ bool epilogue_tile(const GemmTc& p, uint32_t tmem_d, int warp, int lane, int m0, int n0, int b,
                                              int bn_tile, int buf, uint32_t drained, float* epi_smem, long long slot,
                                              uint64_t* acc_full, uint32_t aph) {
    using S = typename Split<ES>::T;
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int n_chunks32 = (bn_tile + 31) / 32;
    const int mq = m0 + q * 32;                                  // first row of this warp's quarter
    const int m = mq + lane;                                     // this thread's row of the batch
    const bool row_ok = m < p.m_rows;
    const int rows_here = min(32, p.m_rows - mq);               // rows of the quarter that exist (may be <= 0)
    const uint32_t t_row = tmem_d + (static_cast<uint32_t>(q * 32) << 16);
    float* stg = epi_smem + (warp - 2) * 1024;                  // this warp's 32x32 square (column sums of W)
    float* strip = epi_smem + UM_EPI_WARPS * 1024 + (warp - 2) * 32;      // this chunk's per-column operand
    const long long grow0 = static_cast<long long>(b) * p.m_rows + mq;        // first row of the quarter in per-row vectors
    const long long grow = grow0 + lane;
    const float inf = __int_as_float(0x7f800000);
    const bool dist_form = p.ep == EP_DIST || (p.ep == EP_LOSS && p.loss_dist);
    // per-row operands of the owning thread.  Distance forms: rows past the end carry a squared norm of +inf, which turns
    // each of their entries into an exact zero without a test per element.
    float row_op = 0.f;
    if (dist_form) row_op = row_ok ? p.sq_a[grow] : inf;
    else if (p.ep == EP_RANK1 && row_ok) row_op = p.scale[grow];
    float* orow = (row_ok && p.ep != EP_LOSS) ? p.out + (static_cast<long long>(b) * p.out_batch_rows + m) * p.out_ld : nullptr;
    const bool vec_out = (p.out_ld & 3) == 0;
    S* wh = nullptr; S* wl = nullptr;
    if (p.ep == EP_LOSS && row_ok) { wh = static_cast<S*>(p.w_hi) + grow * p.ldw; wl = static_cast<S*>(p.w_lo) + grow * p.ldw; }
    const S* yh = nullptr; const S* yl = nullptr;
    if (p.ep == EP_RANK1 && row_ok) { yh = static_cast<const S*>(p.y_hi) + grow * p.y_ld; yl = static_cast<const S*>(p.y_lo) + grow * p.y_ld; }
    const float nw = p.neg_w;
    float lsum = 0.f, row_acc = 0.f;             // EP_LOSS: this thread's loss terms (unscaled); this row's sum of W
    // distance forms: this lane's per-column operand of chunk c (+inf past the last column), requested one chunk ahead
    auto col_operand = [&](int c) -> float {
        const int nb = n0 + c * 32;
        const int lm = min(32, min(bn_tile - c * 32, p.n_cols - nb));
        return (c < n_chunks32 && lane < lm) ? p.sq_b[static_cast<long long>(b) * p.n_cols + nb + lane] : inf;
    };
    float sb_cur = dist_form ? col_operand(half) : 0.f;
    bool acc_ready = false;
#pragma unroll 1
    for (int c = half; c < n_chunks32; c += 2) {
        const int nbase = n0 + c * 32;
        const int lim = min(32, min(bn_tile - c * 32, p.n_cols - nbase));                 // valid columns of this chunk
        const float sb_next = dist_form ? col_operand(c + 2) : 0.f;
        float y[32];
        if (p.ep == EP_RANK1) {                  // the y row comes from memory: requested before the accumulator is read
            if (yh != nullptr && lim > 0) get_row32(yh + nbase, yl + nbase, y);
            else {
#pragma unroll
                for (int j = 0; j < 32; ++j) y[j] = 0.f;
            }
        }
        if (!acc_ready) {
            if (!umma::mbar_wait(acc_full, aph)) return false;          // warp-uniform
            umma::tc_fence_after();
            acc_ready = true;
        }
        float v[32];
        umma::tmem_ld32(t_row + c * 32, v);         // warp-collective
        const float sb_mine = sb_cur;
        sb_cur = sb_next;
        if (rows_here <= 0 || lim <= 0) continue;    // warp-uniform
        if (dist_form) {
            __syncwarp();                            // the previous chunk's reads of the strip are done
            strip[lane] = sb_mine;
            __syncwarp();
        }
        if (p.ep == EP_LOSS) {
            // columns this chunk writes: its own, and - in the chunk that holds the last column - the zero padding of the pitch
            const int wlim = nbase + lim >= p.n_cols ? static_cast<int>(min(32LL, p.ldw - nbase)) : lim;
            if (p.loss_dist) {
                // S = -dd, dd = sqrt(d2) >= 0: softplus(S) = log1p(e), sigmoid(S) = e / (1 + e) with e = exp(-dd), and
                // W = dS / S = -neg_w e / ((1 + e) dd).  No branches: columns past the end carry sq_b = +inf and entries
                // whose d2 cancels are set to +inf too - both then contribute exact zeros - and the cancelling entries
                // are redone from the rows themselves below.
                uint32_t bad = 0;
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 sb4 = *reinterpret_cast<const float4*>(strip + 4 * j4);
                    const float sbv[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = 4 * j4 + i;
                        const float nn = row_op + sbv[i];
                        float d2 = fmaf(-2.f, v[j], nn);
                        const bool flag = d2 < 0.015625f * nn;
                        bad |= (flag ? 1u : 0u) << j;
                        d2 = flag ? inf : fmaxf(d2, 0.f);
                        const float dd = sqrt_approx(d2);
                        const float e = ex2_approx(dd * -1.44269504f);
                        const float qq = rcp_approx((1.f + e) * dd);         // dd = inf: qq = 0 and e = 0; dd = 0: masked below
                        const float w = dd > 0.f ? (-nw * e) * qq : 0.f;
                        lsum += log1p_unit(e);
                        row_acc += w;
                        v[j] = w;
                    }
                }
                if (wh != nullptr) put_row32(wh + nbase, wl + nbase, v, wlim);
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 32 + (j ^ lane)] = v[j];
                __syncwarp();
                if (__any_sync(0xffffffffu, bad != 0)) {
                    for (int r = 0; r < rows_here; ++r) {
                        unsigned todo = __shfl_sync(0xffffffffu, bad, r);
                        while (todo) {
                            const int cl = __ffs(todo) - 1;
                            todo &= todo - 1;
                            const long long ao = (grow0 + r) * p.ex_ld, xo = (static_cast<long long>(b) * p.n_cols + nbase + cl) * p.ex_ld;
                            float e2 = 0.f;
                            for (int k = lane; k < p.k_len; k += 32) {
                                float av = Split<ES>::get(static_cast<const S*>(p.ex_a_hi) + ao + k, static_cast<const S*>(p.ex_a_lo) + ao + k);
                                float xv = Split<ES>::get(static_cast<const S*>(p.ex_x_hi) + xo + k, static_cast<const S*>(p.ex_x_lo) + xo + k);
                                if (ES == 2) {        // third term of the bf16 split: hi + lo + b2 is the row itself
                                    av += static_cast<float>(static_cast<const S*>(p.ex_a_b2)[ao + k]);
                                    xv += static_cast<float>(static_cast<const S*>(p.ex_x_b2)[xo + k]);
                                }
                                const float df = av - xv;
                                e2 = fmaf(df, df, e2);
                            }
                            e2 = warp_sum(e2);
                            if (lane == r) {           // the row's owner patches the one entry (after its own vector stores)
                                const float dd = sqrtf(e2);
                                const float e = __expf(-dd);
                                const float w = dd > 0.f ? -nw * e / ((1.f + e) * dd) : 0.f;
                                lsum += log1pf(e);
                                row_acc += w;
                                stg[r * 32 + (cl ^ r)] = w;
                                Split<ES>::put(wh + nbase + cl, wl + nbase + cl, w);
                            }
                        }
                    }
                    __syncwarp();
                }
                float cs = 0.f;                       // lane = column: this quarter's part of the column sum of W
#pragma unroll
                for (int r = 0; r < 32; ++r) cs += stg[r * 32 + (lane ^ r)];
                if (lane < lim) p.colpart[(static_cast<long long>(b) * ((p.m_rows + 31) / 32) + (mq >> 5)) * p.n_cols + nbase + lane] = cs;
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    // softplus(sc) and sigmoid(sc) from one exponential: e = exp(-|sc|) in (0, 1]
                    const float sc = v[j];
                    const float e = ex2_approx(fabsf(sc) * -1.44269504f);
                    const float l1p = log1p_unit(e);
                    const float inv = rcp_approx(1.f + e);
                    const bool ok = row_ok && j < lim;
                    v[j] = ok ? nw * (sc >= 0.f ? inv : e * inv) : 0.f;
                    lsum += ok ? fmaxf(sc, 0.f) + l1p : 0.f;
                }
                if (wh != nullptr) put_row32(wh + nbase, wl + nbase, v, wlim);
            }
        } else if (p.ep == EP_DIST) {
            uint32_t bad = 0;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                const float4 sb4 = *reinterpret_cast<const float4*>(strip + 4 * j4);
                const float sbv[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = 4 * j4 + i;
                    const float nn = row_op + sbv[i];
                    const float d2 = fmaf(-2.f, v[j], nn);
                    bad |= (d2 < 0.015625f * nn ? 1u : 0u) << j;       // cancellation: listed for exact recomputation
                    v[j] = -sqrt_approx(fmaxf(d2, 0.f));
                }
            }
            if (orow != nullptr) {
                store_row32(orow + nbase, v, lim, vec_out && (lim & 3) == 0);
                while (bad) {
                    const int j = __ffs(bad) - 1;
                    bad &= bad - 1;
                    const unsigned long long at = atomicAdd(p.fix_count, 1ULL);
                    if (at < p.fix_cap) p.fix_list[at] = static_cast<unsigned long long>(grow) * p.n_cols + nbase + j;
                }
            }
        } else if (p.ep == EP_RANK1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaf(row_op, y[j], -v[j]);
            if (orow != nullptr) store_row32(orow + nbase, v, lim, vec_out && (lim & 3) == 0);
        } else {                             // EP_STORE
            if (orow != nullptr) store_row32(orow + nbase, v, lim, vec_out && (lim & 3) == 0);
        }
    }
    if (!acc_ready && !umma::mbar_wait(acc_full, aph)) return false;      // a warp without chunks still takes part in the hand-over
    // this warp is done reading the accumulator: hand it back to the MMA thread
    umma::tc_fence_before();
    __syncwarp();
    if (lane == 0) umma::mbar_arrive_cluster(drained);
    if (p.ep == EP_LOSS) {
        const long long total_rows = static_cast<long long>(p.batch) * p.m_rows;
        if (row_ok && p.loss_dist) p.rowpart[(static_cast<long long>(n0 / p.bn) * 2 + half) * total_rows + grow] = row_acc;
        const float l = warp_sum(nw * lsum);
        if (lane == 0) p.loss_part[slot * UM_EPI_WARPS + (warp - 2)] = l;
    }
    return true;
}

// Epilogues of the relation-grouped products (norm, dL/dv rows, scatter, plain store), in the layout tcgen05.ld delivers:
// thread = row, 32 consecutive columns per chunk.  Everything that is per ROW (destination, coefficient, sign) is then a
// register of the owning thread, computed once per tile, and a thread's 32 values are one contiguous 128-byte (fp32) or
// 64-byte (bf16) piece of its destination row, written with 16-byte stores; the per-COLUMN vector R[z] sits in a
// shared-memory strip of the warp and is read as 128-bit broadcasts.  (The dense epilogues go through a transposing
// staging square instead, because their per-column operands and row-contiguous destinations favour lane = column.)
__device__ __forceinline__ bool epilogue_grouped(const GemmTc& p, uint32_t tmem_d, int warp, int lane, int m0, int n0, int b,
                                                 int bn_tile, int buf, int par, uint32_t drained, float* epi_smem,
                                                 uint64_t* acc_full, uint32_t aph, volatile uint32_t* epi_fail) {
    const int q = warp & 3;
    const int half = ((warp - 2) & 7) >> 2;
    const int row = q * 32 + lane;
    const int n_chunks32 = (bn_tile + 31) / 32;
    const int m = m0 + row;
    const bool row_ok = m < p.m_rows;
    const uint32_t t_row = tmem_d + (static_cast<uint32_t>(q * 32) << 16);
    float* rs = epi_smem + 1024 + (warp - 2) * 256;            // this warp's copy of R[z] (n_cols <= 256), zero padded; 16 warps
    if (p.ep == EP_NORM || p.ep == EP_GV) {
        for (int c = lane; c < 256; c += 32) {
            float rv = 0.f;
            if (c < p.n_cols) {
                const long long ri = static_cast<long long>(b) * p.n_cols + c;
                rv = p.rel_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.rel_vec)[ri])
                                   : reinterpret_cast<const float*>(p.rel_vec)[ri];
            }
            rs[c] = rv;
        }
        __syncwarp();
    }
    // per-row operands of the owning thread
    float coef = 0.f, sign = 1.f;
    float* orow = nullptr;                                     // fp32 destination row (scatter, store)
    __nv_bfloat16* grow = nullptr;                             // bf16 destination row (dL/dv)
    if (row_ok) {
        if (p.ep == EP_GV) { coef = p.coef[m]; grow = p.gv_out + static_cast<long long>(m) * p.n_cols; }
        else if (p.ep == EP_SCATTER) {
            const long long dst = p.row_dst[m];                // >= kTailSide: slot, minus sign; >= 0: slot; <= -2: positive -2-i; -1: padding
            if (dst >= kTailSide) { orow = p.neg_out + (dst - kTailSide) * p.n_cols; sign = -1.f; }
            else if (dst >= 0) orow = p.neg_out + dst * p.n_cols;
            else if (dst <= -2) orow = p.pos_out + (-2 - dst) * p.n_cols;
        } else if (p.ep == EP_STORE) {
            orow = p.out + (static_cast<long long>(b) * p.out_batch_rows + m) * p.out_ld;
        }
    }
    float ssq = 0.f;
    // The accumulator is waited for only now, after the per-tile operands above have been requested (see epilogue_tile).
    bool ok = umma::mbar_wait(acc_full, aph);                                                   // warp-uniform result
    if (p.ep == EP_NORM) {
        // the eight epilogue warps of a set meet at a named barrier inside this epilogue: they give up together or not at all
        if (!ok && lane == 0) *epi_fail = 1u;
        asm volatile("bar.sync %0, 256;" :: "r"(1 + buf) : "memory");
        ok = *epi_fail == 0u;
    }
    if (!ok) return false;
    umma::tc_fence_after();
#pragma unroll 1
    for (int c = half; c < n_chunks32; c += 2) {
        float v[32];
        umma::tmem_ld32(t_row + c * 32, v);                     // warp-collective
        const int nbase = n0 + c * 32;
        const int lim = min(32, min(bn_tile - c * 32, p.n_cols - nbase));      // valid columns of this chunk (a multiple of 4)
        if (p.ep == EP_NORM) {
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                const float4 r4 = *reinterpret_cast<const float4*>(rs + c * 32 + 4 * j4);
                if (4 * j4 < lim) {
                    const float t0 = v[4 * j4 + 0] + r4.x, t1 = v[4 * j4 + 1] + r4.y, t2 = v[4 * j4 + 2] + r4.z, t3 = v[4 * j4 + 3] + r4.w;
                    ssq = fmaf(t0, t0, fmaf(t1, t1, fmaf(t2, t2, fmaf(t3, t3, ssq))));
                }
            }
        } else if (p.ep == EP_GV) {
            if (grow != nullptr) {
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                    if (8 * j8 < lim) {
                        const float4 ra = *reinterpret_cast<const float4*>(rs + c * 32 + 8 * j8);
                        const float4 rb = *reinterpret_cast<const float4*>(rs + c * 32 + 8 * j8 + 4);
                        __nv_bfloat162 o0 = __floats2bfloat162_rn(coef * (v[8 * j8 + 0] + ra.x), coef * (v[8 * j8 + 1] + ra.y));
                        __nv_bfloat162 o1 = __floats2bfloat162_rn(coef * (v[8 * j8 + 2] + ra.z), coef * (v[8 * j8 + 3] + ra.w));
                        __nv_bfloat162 o2 = __floats2bfloat162_rn(coef * (v[8 * j8 + 4] + rb.x), coef * (v[8 * j8 + 5] + rb.y));
                        __nv_bfloat162 o3 = __floats2bfloat162_rn(coef * (v[8 * j8 + 6] + rb.z), coef * (v[8 * j8 + 7] + rb.w));
                        uint4 u;
                        u.x = *reinterpret_cast<unsigned*>(&o0); u.y = *reinterpret_cast<unsigned*>(&o1);
                        u.z = *reinterpret_cast<unsigned*>(&o2); u.w = *reinterpret_cast<unsigned*>(&o3);
                        *reinterpret_cast<uint4*>(grow + nbase + 8 * j8) = u;
                    }
                }
            }
        } else {                                               // EP_SCATTER (signed) and EP_STORE
            if (orow != nullptr) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] *= sign;
                store_row32(orow + nbase, v, lim, true);       // n_cols % 8 == 0 on this path: rows are 32-byte aligned
            }
        }
    }
    // this warp is done reading the accumulator: hand it back to the MMA thread
    umma::tc_fence_before();
    __syncwarp();
    if (lane == 0) umma::mbar_arrive_cluster(drained);
    if (p.ep == EP_NORM) {
        // [2 accumulators = warp sets][2 tile parities][2 halves][128 rows]: a set's next tile writes the other parity, so
        // its faster warps cannot overwrite sums that the slower ones have not read yet
        float* ssq_part = epi_smem + (buf * 2 + par) * 2 * UM_BM;
        ssq_part[half * UM_BM + row] = ssq;
        asm volatile("bar.sync %0, 256;" :: "r"(1 + buf) : "memory");         // the eight epilogue warps of this buffer's set
        if (half == 0) {
            long long dst = p.row_dst[m];                      // >= 0: negative score index (+ kTailSide), <= -2: positive -2-i, -1: padding
            if (dst >= kTailSide) dst -= kTailSide;
            const float sc = -sqrt_approx(ssq_part[row] + ssq_part[UM_BM + row]);
            if (dst >= 0) p.neg_out[dst] = sc; else if (dst <= -2) p.pos_out[-2 - dst] = sc;
        }
    }
    return true;
}

// Persistent: each CTA walks the tile list (tile = blockIdx.x, += gridDim.x; the n-tile index runs fastest so that CTAs
// working at the same time share A rows in L2).  Two accumulators in tensor memory alternate, so the epilogue of tile i
// (tcgen05.ld, scorer epilogue, global stores) overlaps the TMA/MMA main loop of tile i+1.
template <int GROUP, int ES>
__global__ void __launch_bounds__(GROUP == G_GROUPED ? UM_THREADS_GROUPED : UM_THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo, GemmTc p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    // element size 4: tf32 (fp32 storage), 2: bf16.  A shared-memory row is always 128 bytes of K (K-major) or of M/N (MN-major).
    const int bk = 128 / ES;                  // k-values per stage
    const int slab_cols = 128 / ES;           // M/N-columns per MN-major slab
    const int slab_bytes = bk * 128;                    // MN-major slab: bk k-rows x 128 bytes
    const int a_slabs = UM_BM / slab_cols;
    const int b_slabs = (p.bn + slab_cols - 1) / slab_cols;
    const int b_bytes = p.b_mn ? b_slabs * slab_bytes : p.bn * 128;       // one B tile (hi or lo)
    const int n_parts = p.passes == 1 ? 1 : 2;          // hi only, or hi and lo
    const int stage_bytes = n_parts * (UM_A_BYTES + b_bytes);
    const int tx_bytes = stage_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
    uint64_t* empty = full + p.stages;
    uint64_t* acc_full = empty + p.stages;          // [2] accumulator written  (MMA -> epilogue)
    uint64_t* acc_empty = acc_full + 2;             // [2] accumulator drained  (epilogue -> MMA)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* epi_fail = tmem_slot + 1;    // set by an epilogue warp whose wait ran out (EP_NORM)
    float* epi_smem = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(full) + 256);      // staging squares (EP_NORM: partial sums)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.k_len + bk - 1) / bk;
    const uint32_t acc_cols = p.bn <= 32 ? 32u : p.bn <= 64 ? 64u : p.bn <= 128 ? 128u : 256u;
    const uint32_t tmem_cols = 2 * acc_cols;        // <= 512, the whole tensor memory at bn > 128
    const int tiles_n = (p.n_cols + p.bn - 1) / p.bn;
    const int tiles_m = (p.m_rows + UM_BM - 1) / UM_BM;
    // grouped mode: the tile list comes from device memory (one n-tile; rows of A are absolute; z selects the B matrix).
    // The host keeps the tile count below 2^31, so 32-bit tile arithmetic is exact.
    const int n_tiles = static_cast<int>(p.tile_tab ? min(*p.n_tiles_dev, p.tile_cap)
                                                    : static_cast<long long>(tiles_n) * tiles_m * p.batch);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { umma::mbar_init(&full[s], 1); umma::mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { umma::mbar_init(&acc_full[s], 1); umma::mbar_init(&acc_empty[s], UM_EPI_WARPS); }
        *epi_fail = 0u;
        umma::fence_barrier_init();
    }
    if (warp == 1) { umma::tmem_alloc(tmem_slot, tmem_cols); umma::tmem_relinquish(); }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------------------------------------
        if (lane == 0) {
            umma::prefetch_tensormap(&map_a_hi); umma::prefetch_tensormap(&map_a_lo);
            umma::prefetch_tensormap(&map_b_hi); umma::prefetch_tensormap(&map_b_lo);
            int s = 0; uint32_t ph = 0;            // ring position: stage and its phase bit
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int tq = tile / tiles_n;
                int n0 = (tile - tq * tiles_n) * p.bn;
                int b = tq / tiles_m;
                int m0 = (tq - b * tiles_m) * UM_BM;
                int za = b;
                int kbase = 0, nkb = num_kb;
                if (p.tile_tab) {
                    const int4 tt = p.tile_tab[tile];
                    n0 = 0; za = 0;
                    if (p.group_k) { kbase = tt.x; nkb = tt.y / bk; m0 = tt.z; b = 0; } else { m0 = tt.x; b = tt.y; }
                }
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!umma::mbar_wait(&empty[s], ph ^ 1)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }
                    uint8_t* st = smem + s * stage_bytes;
                    uint8_t* a_hi = st, *a_lo = st + UM_A_BYTES, *b_hi = st + n_parts * UM_A_BYTES, *b_lo = b_hi + b_bytes;
                    umma::mbar_expect_tx(&full[s], tx_bytes);
                    const int k0 = kbase + kb * bk;
                    const bool lo = p.passes != 1;
                    if (!p.a_mn) {
                        umma::tma_load_3d(a_hi, &map_a_hi, k0, m0, za, &full[s]);
                        if (lo) umma::tma_load_3d(a_lo, &map_a_lo, k0, m0, za, &full[s]);
                    } else if (p.a_slabs4d) {
                        umma::tma_load_4d(a_hi, &map_a_hi, 0, k0, m0 / slab_cols, za, &full[s]);
                        if (lo) umma::tma_load_4d(a_lo, &map_a_lo, 0, k0, m0 / slab_cols, za, &full[s]);
                    } else {
                        for (int sl = 0; sl < a_slabs; ++sl) {
                            umma::tma_load_3d(a_hi + sl * slab_bytes, &map_a_hi, m0 + slab_cols * sl, k0, za, &full[s]);
                            if (lo) umma::tma_load_3d(a_lo + sl * slab_bytes, &map_a_lo, m0 + slab_cols * sl, k0, za, &full[s]);
                        }
                    }
                    if (!p.b_mn) {
                        umma::tma_load_3d(b_hi, &map_b_hi, k0, n0, b, &full[s]);
                        if (lo) umma::tma_load_3d(b_lo, &map_b_lo, k0, n0, b, &full[s]);
                    } else if (p.b_slabs4d) {
                        umma::tma_load_4d(b_hi, &map_b_hi, 0, k0, n0 / slab_cols, b, &full[s]);
                        if (lo) umma::tma_load_4d(b_lo, &map_b_lo, 0, k0, n0 / slab_cols, b, &full[s]);
                    } else {
                        for (int sl = 0; sl < b_slabs; ++sl) {
                            umma::tma_load_3d(b_hi + sl * slab_bytes, &map_b_hi, n0 + slab_cols * sl, k0, b, &full[s]);
                            if (lo) umma::tma_load_3d(b_lo + sl * slab_bytes, &map_b_lo, n0 + slab_cols * sl, k0, b, &full[s]);
                        }
                    }
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------------------------------------
        if (lane == 0) {
            const bool f16 = ES == 2;
            const uint32_t idesc = umma::instr_desc(f16 ? 1u /* bf16 */ : 2u /* tf32 */, UM_BM, (uint32_t)p.bn, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
            // Descriptor templates: everything but the start address is fixed for the whole kernel, so the issuing thread
            // only adds an address per MMA (it is the one thread feeding the tensor core; its instruction count matters).
            const uint32_t mn_sbo = f16 ? 1024u : 512u, mn_layout = f16 ? 2u : 1u;
            const uint64_t a_tmpl = p.a_mn ? umma::smem_desc_mn(0, slab_bytes, mn_sbo, mn_layout) : umma::smem_desc_k_sw128(0);
            const uint64_t b_tmpl = p.b_mn ? umma::smem_desc_mn(0, slab_bytes, mn_sbo, mn_layout) : umma::smem_desc_k_sw128(0);
            // per MMA step (32 bytes of K): K-major moves 32 bytes along the swizzled row, MN-major 8 (tf32) / 16 (bf16) k-rows
            const uint32_t a_step = (p.a_mn ? (f16 ? 2048u : 1024u) : 32u) >> 4;
            const uint32_t b_step = (p.b_mn ? (f16 ? 2048u : 1024u) : 32u) >> 4;
            const uint32_t a_lo_off = UM_A_BYTES >> 4, b_hi_off = (n_parts * UM_A_BYTES) >> 4, b_lo_off = b_hi_off + (b_bytes >> 4);
            const bool single = p.passes == 1;
            const int kstep_elems = 32 / ES;      // k-values per MMA step
            int s = 0; uint32_t ph = 0;
            int lt = 0;                            // tiles done by this CTA
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = static_cast<uint32_t>(lt >> 1) & 1;
                if (!umma::mbar_wait(&acc_empty[buf], aph ^ 1)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }   // drained?
                umma::tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * acc_cols;
                const int nkb = (p.tile_tab && p.group_k) ? p.tile_tab[tile].y / bk : num_kb;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!umma::mbar_wait(&full[s], ph)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }
                    umma::tc_fence_after();
                    const uint32_t st = (umma::smem_u32(smem + s * stage_bytes) & 0x3FFFFu) >> 4;     // start address field
                    uint64_t dah = a_tmpl | st, dbh = b_tmpl | (st + b_hi_off);
                    // a stage holds four MMA steps of K (32 bytes each); the last k-block of a product only issues the
                    // steps that hold data (the rest of the stage is the zero fill of the TMA box)
                    const int ksteps = p.group_k ? 4 : min(4, (p.k_len - kb * bk + kstep_elems - 1) / kstep_elems);
                    if (single) {
                        if (f16) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step)
                                if (k8 < ksteps) umma::mma_f16(tmem_d, dah, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                        } else {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step)
                                if (k8 < ksteps) umma::mma_tf32(tmem_d, dah, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                        }
                    } else {
                        uint64_t dal = a_tmpl | (st + a_lo_off), dbl = b_tmpl | (st + b_lo_off);
#pragma unroll
                        for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step, dal += a_step, dbl += b_step) {
                            if (k8 < ksteps) {
                                if (ES == 2) {
                                    umma::mma_f16(tmem_d, dal, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);  // small terms first
                                    umma::mma_f16(tmem_d, dah, dbl, idesc, 1u);
                                    umma::mma_f16(tmem_d, dah, dbh, idesc, 1u);
                                } else {
                                    umma::mma_tf32(tmem_d, dal, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                                    umma::mma_tf32(tmem_d, dah, dbl, idesc, 1u);
                                    umma::mma_tf32(tmem_d, dah, dbh, idesc, 1u);
                                }
                            }
                        }
                    }
                    umma::mma_commit(&empty[s]);          // frees the stage once these MMAs have read it
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                umma::mma_commit(&acc_full[buf]);         // accumulator complete (or abandoned)
            }
        }
    } else {
        // ---- epilogue ---------------------------------------------------------------------------------------------
        // grouped instantiation: the set of this warp (warps 2..9: 0, 10..17: 1) drains the tiles of its own buffer
        const int set = (warp - 2) >> 3;
        int lt = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
            if (GROUP == G_GROUPED && (lt & 1) != set) continue;
            const int tq = tile / tiles_n;
            int n0 = (tile - tq * tiles_n) * p.bn;
            int b = tq / tiles_m;
            int m0 = (tq - b * tiles_m) * UM_BM;
            if (p.tile_tab) {
                const int4 tt = p.tile_tab[tile];
                n0 = 0;
                if (p.group_k) { m0 = tt.z; b = tt.w; } else { m0 = tt.x; b = tt.y; }
            }
            const int buf = lt & 1;
            const uint32_t aph = static_cast<uint32_t>(lt >> 1) & 1;
            bool ok;                                   // false: the wait for the accumulator ran out (warp-uniform)
            if (GROUP == G_GROUPED) ok = epilogue_grouped(p, tmem_base + buf * acc_cols, warp, lane, m0, n0, b, p.bn, buf, (lt >> 1) & 1,
                                                          umma::smem_u32(&acc_empty[buf]), epi_smem, &acc_full[buf], aph, epi_fail);
            else ok = epilogue_tile<G_DENSE, ES>(p, tmem_base + buf * acc_cols, warp, lane, m0, n0, b, p.bn, buf,
                                                 umma::smem_u32(&acc_empty[buf]), epi_smem, tile, &acc_full[buf], aph);
            if (!ok) { if (lane == 0) atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); break; }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) { umma::tc_fence_after(); umma::tmem_dealloc(tmem_base, tmem_cols); }
}

// CTA-pair variant (cluster of two, tcgen05 cta_group::2): one 256-row x bn tile per pair.  Each CTA stages its own 128
// rows of A and its own half of the bn columns of B, so a stage carries half the operand bytes per flop of the one-CTA
// kernel; the one-CTA kernel is bound by shared-memory bandwidth (TMA writes + operand reads of three MMAs per k-step),
// this one by the tensor pipe.  The even CTA issues the MMAs for both and commits to the barriers of both; each CTA
// drains its own 128 accumulator rows.  Dense (non-grouped) products only.  With an MN-major B the last n-tile is
// narrowed to the columns that exist (in units of two slabs), so a width like 400 costs 448 columns, not 512.
template <int ES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(UM_THREADS, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo, GemmTc p) {
    extern __shared__ uint8_t smem_raw[];
    // the same offset in both CTAs: the dynamic shared-memory window starts at the same address in every CTA of a launch
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int bk = 128 / ES;
    const int slab_cols = 128 / ES;
    const int slab_bytes = bk * 128;
    const int a_slabs = UM_BM / slab_cols;
    const int half_n = p.bn / 2;                                          // B columns staged by each CTA (full-width tile)
    const int b_bytes = p.b_mn ? (half_n / slab_cols) * slab_bytes : half_n * 128;
    const int n_parts = p.passes == 1 ? 1 : 2;
    const int stage_bytes = n_parts * (UM_A_BYTES + b_bytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
    uint64_t* empty = full + p.stages;
    uint64_t* acc_full = empty + p.stages;
    uint64_t* acc_empty = acc_full + 2;             // only the leader's are waited on; both CTAs' epilogue warps arrive there
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    float* epi_smem = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(full) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = umma::cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int num_kb = (p.k_len + bk - 1) / bk;
    const uint32_t acc_cols = p.bn <= 32 ? 32u : p.bn <= 64 ? 64u : p.bn <= 128 ? 128u : 256u;
    const uint32_t tmem_cols = 2 * acc_cols;
    const int tiles_n = (p.n_cols + p.bn - 1) / p.bn;
    const int tiles_m = (p.m_rows + 2 * UM_BM - 1) / (2 * UM_BM);
    const int n_tiles = tiles_n * tiles_m * p.batch;          // the host keeps this below 2^31
    const int unit = 2 * slab_cols;                          // MN-major B: a tile is a whole number of slabs per CTA

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { umma::mbar_init(&full[s], 1); umma::mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { umma::mbar_init(&acc_full[s], 1); umma::mbar_init(&acc_empty[s], 2 * UM_EPI_WARPS); }
        umma::fence_barrier_init();
    }
    if (warp == 1) { umma::tmem_alloc_pair(tmem_slot, tmem_cols); umma::tmem_relinquish_pair(); }
    umma::tc_fence_before();
    __syncthreads();
    umma::cluster_sync();          // the peer's barriers exist before anything is signalled across the pair
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer (both CTAs; all bytes are counted on the leader's `full` barrier) -------------------------
        if (lane == 0) {
            umma::prefetch_tensormap(&map_a_hi); umma::prefetch_tensormap(&map_a_lo);
            umma::prefetch_tensormap(&map_b_hi); umma::prefetch_tensormap(&map_b_lo);
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            const bool lo = p.passes != 1;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int tq = tile / tiles_n;
                const int n0 = (tile - tq * tiles_n) * p.bn;
                const int b = tq / tiles_m;
                const int m0 = (tq - b * tiles_m) * (2 * UM_BM) + static_cast<int>(rank) * UM_BM;      // this CTA's rows
                const int bnt = p.b_mn ? min(p.bn, (p.n_cols - n0 + unit - 1) / unit * unit) : p.bn;
                const int hn = bnt / 2;
                const int nb0 = n0 + static_cast<int>(rank) * hn;                                      // this CTA's columns
                const int b_slabs = hn / slab_cols;
                const uint32_t tx_pair = 2u * n_parts * (UM_A_BYTES + (p.b_slabs4d ? b_bytes : p.b_mn ? b_slabs * slab_bytes : hn * 128));
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!umma::mbar_wait(&empty[s], ph ^ 1)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }
                    uint8_t* st = smem + s * stage_bytes;
                    uint8_t* a_hi = st, *a_lo = st + UM_A_BYTES, *b_hi = st + n_parts * UM_A_BYTES, *b_lo = b_hi + b_bytes;
                    const uint32_t lead_full = umma::map_to_cta(umma::smem_u32(&full[s]), 0);
                    if (rank == 0) umma::mbar_expect_tx(&full[s], tx_pair);
                    const int k0 = kb * bk;
                    if (!p.a_mn) {
                        umma::tma_load_3d_pair(a_hi, &map_a_hi, k0, m0, b, lead_full);
                        if (lo) umma::tma_load_3d_pair(a_lo, &map_a_lo, k0, m0, b, lead_full);
                    } else if (p.a_slabs4d) {
                        umma::tma_load_4d_pair(a_hi, &map_a_hi, 0, k0, m0 / slab_cols, b, lead_full);
                        if (lo) umma::tma_load_4d_pair(a_lo, &map_a_lo, 0, k0, m0 / slab_cols, b, lead_full);
                    } else {
                        for (int sl = 0; sl < a_slabs; ++sl) {
                            umma::tma_load_3d_pair(a_hi + sl * slab_bytes, &map_a_hi, m0 + slab_cols * sl, k0, b, lead_full);
                            if (lo) umma::tma_load_3d_pair(a_lo + sl * slab_bytes, &map_a_lo, m0 + slab_cols * sl, k0, b, lead_full);
                        }
                    }
                    if (!p.b_mn) {
                        umma::tma_load_3d_pair(b_hi, &map_b_hi, k0, nb0, b, lead_full);
                        if (lo) umma::tma_load_3d_pair(b_lo, &map_b_lo, k0, nb0, b, lead_full);
                    } else if (p.b_slabs4d) {         // the box is the full half-tile: slabs past the narrowed tile read as zero
                        umma::tma_load_4d_pair(b_hi, &map_b_hi, 0, k0, nb0 / slab_cols, b, lead_full);
                        if (lo) umma::tma_load_4d_pair(b_lo, &map_b_lo, 0, k0, nb0 / slab_cols, b, lead_full);
                    } else {
                        for (int sl = 0; sl < b_slabs; ++sl) {
                            umma::tma_load_3d_pair(b_hi + sl * slab_bytes, &map_b_hi, nb0 + slab_cols * sl, k0, b, lead_full);
                            if (lo) umma::tma_load_3d_pair(b_lo + sl * slab_bytes, &map_b_lo, nb0 + slab_cols * sl, k0, b, lead_full);
                        }
                    }
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
            // tail: every commit aimed at this CTA's `empty` barriers has landed before the CTA may exit
            for (int i = 0; i < p.stages && ok; ++i) {
                if (!umma::mbar_wait(&empty[s], ph ^ 1)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; }
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the leader only --------------------------------------------------------------------------------
        if (lane == 0 && rank == 0) {
            const bool f16 = ES == 2;
            const uint32_t mn_sbo = f16 ? 1024u : 512u, mn_layout = f16 ? 2u : 1u;
            const uint64_t a_tmpl = p.a_mn ? umma::smem_desc_mn(0, slab_bytes, mn_sbo, mn_layout) : umma::smem_desc_k_sw128(0);
            const uint64_t b_tmpl = p.b_mn ? umma::smem_desc_mn(0, slab_bytes, mn_sbo, mn_layout) : umma::smem_desc_k_sw128(0);
            const uint32_t a_step = (p.a_mn ? (f16 ? 2048u : 1024u) : 32u) >> 4;
            const uint32_t b_step = (p.b_mn ? (f16 ? 2048u : 1024u) : 32u) >> 4;
            const uint32_t a_lo_off = UM_A_BYTES >> 4, b_hi_off = (n_parts * UM_A_BYTES) >> 4, b_lo_off = b_hi_off + (b_bytes >> 4);
            const bool single = p.passes == 1;
            const int kstep_elems = 32 / ES;
            int s = 0; uint32_t ph = 0;
            int lt = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++lt) {
                const int n0 = (tile % tiles_n) * p.bn;
                const int bnt = p.b_mn ? min(p.bn, (p.n_cols - n0 + unit - 1) / unit * unit) : p.bn;
                const uint32_t idesc = umma::instr_desc(f16 ? 1u : 2u, 2 * UM_BM, (uint32_t)bnt, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
                const int buf = lt & 1;
                const uint32_t aph = static_cast<uint32_t>(lt >> 1) & 1;
                if (!umma::mbar_wait(&acc_empty[buf], aph ^ 1)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }
                umma::tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * acc_cols;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!umma::mbar_wait(&full[s], ph)) { atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT); ok = false; break; }
                    umma::tc_fence_after();
                    const uint32_t st = (umma::smem_u32(smem + s * stage_bytes) & 0x3FFFFu) >> 4;
                    uint64_t dah = a_tmpl | st, dbh = b_tmpl | (st + b_hi_off);
                    const int ksteps = min(4, (p.k_len - kb * bk + kstep_elems - 1) / kstep_elems);     // steps of this stage that hold data
                    if (single) {
                        if (f16) {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step)
                                if (k8 < ksteps) umma::mma_f16_pair(tmem_d, dah, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                        } else {
#pragma unroll
                            for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step)
                                if (k8 < ksteps) umma::mma_tf32_pair(tmem_d, dah, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                        }
                    } else {
                        uint64_t dal = a_tmpl | (st + a_lo_off), dbl = b_tmpl | (st + b_lo_off);
#pragma unroll
                        for (int k8 = 0; k8 < 4; ++k8, dah += a_step, dbh += b_step, dal += a_step, dbl += b_step) {
                            if (k8 < ksteps) {
                                if (ES == 2) {
                                    umma::mma_f16_pair(tmem_d, dal, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);  // small terms first
                                    umma::mma_f16_pair(tmem_d, dah, dbl, idesc, 1u);
                                    umma::mma_f16_pair(tmem_d, dah, dbh, idesc, 1u);
                                } else {
                                    umma::mma_tf32_pair(tmem_d, dal, dbh, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                                    umma::mma_tf32_pair(tmem_d, dah, dbl, idesc, 1u);
                                    umma::mma_tf32_pair(tmem_d, dah, dbh, idesc, 1u);
                                }
                            }
                        }
                    }
                    const uint32_t e0 = umma::smem_u32(&empty[s]);
                    umma::mma_commit_pair(e0);                              // frees the stage in this CTA ...
                    umma::mma_commit_pair(umma::map_to_cta(e0, 1));         // ... and in the peer
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                const uint32_t f0 = umma::smem_u32(&acc_full[buf]);
                umma::mma_commit_pair(f0);
                umma::mma_commit_pair(umma::map_to_cta(f0, 1));
            }
        }
    } else {
        // ---- epilogue (both CTAs, each its own 128 rows) -------------------------------------------------------------------
        int lt = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++lt) {
            const int tq = tile / tiles_n;
            const int n0 = (tile - tq * tiles_n) * p.bn;
            const int b = tq / tiles_m;
            const int m0 = (tq - b * tiles_m) * (2 * UM_BM) + static_cast<int>(rank) * UM_BM;
            const int bnt = p.b_mn ? min(p.bn, (p.n_cols - n0 + unit - 1) / unit * unit) : p.bn;
            const int buf = lt & 1;
            const uint32_t aph = static_cast<uint32_t>(lt >> 1) & 1;
            if (!epilogue_tile<G_DENSE, ES>(p, tmem_base + buf * acc_cols, warp, lane, m0, n0, b, bnt, buf,
                                            umma::map_to_cta(umma::smem_u32(&acc_empty[buf]), 0), epi_smem, 2LL * tile + rank,
                                            &acc_full[buf], aph)) {
                if (lane == 0) atomicOr(p.err, KGE_ERR_WAIT_TIMEOUT);
                break;
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::cluster_sync();          // neither CTA frees tensor memory or exits while the other may still signal it
    if (warp == 1) { umma::tc_fence_after(); umma::tmem_dealloc_pair(tmem_base, tmem_cols); }
}

// Exact recomputation of the listed TransE scores from the table rows (one warp per entry).
template <typename T, typename I, int NV>
__global__ void __launch_bounds__(256) tc_fixup_kernel(ScoreArgs a, int head, const unsigned long long* count,
                                                       const unsigned long long* list, unsigned long long cap) {
    const int lane = threadIdx.x & 31;
    const unsigned long long n = min(*count, cap);
    if (*count > cap) return;                           // overflow: the exact kernel recomputes everything
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* R = reinterpret_cast<const T*>(a.rel);
    const int dim = a.dim;
    for (unsigned long long e = (unsigned long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < n;
         e += (unsigned long long)gridDim.x * (blockDim.x >> 5)) {
        const unsigned long long pair = list[e];
        const long long i = (long long)(pair / a.n_neg);           // triple
        const int j = (int)(pair % a.n_neg);
        const long long c = i / a.chunk;
        Row<NV> o, r, x;
        load_row<T, NV, true>(o, E + load_id<I>(head ? a.t : a.h, i) * dim, dim, lane);
        load_row<T, NV, true>(r, R + load_id<I>(a.r, i) * dim, dim, lane);
        load_row<T, NV, true>(x, E + load_id<I>(a.neg, c * a.n_neg + j) * dim, dim, lane);
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            const float4 anc = head ? o.v[q] - r.v[q] : o.v[q] + r.v[q];
            const float4 d = anc - x.v[q];
            s = dot4(d, d, s);
        }
        s = warp_sum(s);
        if (lane == 0) a.negs[pair] = -sqrtf(s);
    }
}

// ---- host launchers ---------------------------------------------------------------------------------------------------
static inline size_t al256(size_t x) { return (x + 255) / 256 * 256; }

struct TcLayout {        // carving of the tensor-core workspace
    size_t mat;          // bytes of one (n_a + n_x, dim) split matrix
    size_t w;            // bytes of one (batch, n_neg) split matrix (backward only)
    size_t off_hi, off_lo, off_b2, off_sq, off_fixc, off_fixl, off_whi, off_wlo, off_rowsum, off_colsum, off_colpart, off_rowpart, off_losspart, total;
    long long loss_parts;    // fused mode: loss partials (one per epilogue warp and 128-row tile)
    int fwd_bn, fwd_pair;    // tiling of the forward product
    unsigned long long fix_cap;
    int es;              // bytes per split element: 2 (bf16 split) or 4 (tf32 split in fp32 storage)
    int ldp, ldw;        // row pitches in elements: dim and n_neg rounded up to whole 128-byte slabs
    bool third;          // a third split term is kept (bf16 split, fused distance epilogue: rows rebuilt exactly)
};
// CTA pairs pay off once a product has more than one 128-row tile per batch; narrow outputs stay on the one-CTA kernel.
static bool want_pair(int m_rows, int n_cols) { return m_rows > UM_BM && n_cols >= 64; }
static int pick_bn(int n);

// mode 0: forward, 1: backward, 2: fused forward + loss + backward; es: split element size; dist: TransE
static TcLayout tc_layout(long long batch, int chunk, int n_neg, int dim, int mode, int es, bool dist) {
    const bool backward = mode != 0;
    TcLayout L;
    const long long n_chunks = batch / chunk;
    const size_t rows = static_cast<size_t>(batch + n_chunks * n_neg);
    const size_t pairs = static_cast<size_t>(batch) * n_neg;
    const int slab = 128 / es;
    L.es = es;
    L.ldp = (dim + slab - 1) / slab * slab;
    L.ldw = (n_neg + slab - 1) / slab * slab;
    L.mat = al256(rows * L.ldp * es);
    L.w = backward ? al256(static_cast<size_t>(batch) * L.ldw * es) : 0;
    L.third = es == 2 && mode == 2 && dist;
    L.fix_cap = backward ? 0 : (pairs / 64 > 4096 ? pairs / 64 : 4096);
    L.fwd_pair = want_pair(chunk, n_neg) ? 1 : 0;
    L.fwd_bn = L.fwd_pair ? pick_bn(n_neg) : (n_neg >= 128 ? 128 : pick_bn(n_neg));
    const long long tiles_n = (n_neg + L.fwd_bn - 1) / L.fwd_bn;
    L.loss_parts = tiles_n * ((chunk + UM_BM - 1) / UM_BM + 1) * n_chunks * UM_EPI_WARPS;
    size_t o = 0;
    L.off_hi = o; o += L.mat;
    L.off_lo = o; o += L.mat;
    L.off_b2 = o; o += L.third ? L.mat : 0;
    L.off_sq = o; o += al256(rows * 4);
    L.off_fixc = o; o += 256;
    L.off_fixl = o; o += al256(L.fix_cap * 8);
    L.off_whi = o; o += L.w;
    L.off_wlo = o; o += L.w;
    L.off_rowsum = o; o += backward ? al256(static_cast<size_t>(batch) * 4) : 0;
    L.off_colsum = o; o += backward ? al256(static_cast<size_t>(n_chunks) * n_neg * 4) : 0;
    L.off_colpart = o; o += backward ? al256(static_cast<size_t>(n_chunks) * ((chunk + TW_ROWS - 1) / TW_ROWS) * n_neg * 4) : 0;
    L.off_rowpart = o; o += mode == 2 ? al256(static_cast<size_t>(2 * tiles_n) * batch * 4) : 0;
    L.off_losspart = o; o += mode == 2 ? al256(static_cast<size_t>(L.loss_parts) * 4) : 0;
    L.total = o;
    return L;
}
// Upper bound over the scorers (the distance scorer's fused call keeps a third split term).
size_t tc_pair_workspace_bytes(long long batch, int chunk, int n_neg, int dim, int mode, int es) {
    return tc_layout(batch, chunk, n_neg, dim, mode, es, true).total;
}

template <int MODEL, typename T, typename I, int ES>
static int tc_pack_go(const ScoreArgs& a, int head, long long n_a, long long n_x, int ldp, void* hi, void* lo, void* b2, float* sq, cudaStream_t s) {
    const int nv = quads_per_lane(a.dim);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((n_a + n_x + wpb - 1) / wpb);
    switch (nv) {
        case 1: tc_pack_kernel<MODEL, T, I, 1, ES><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, ldp, hi, lo, b2, sq); break;
        case 2: tc_pack_kernel<MODEL, T, I, 2, ES><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, ldp, hi, lo, b2, sq); break;
        case 4: tc_pack_kernel<MODEL, T, I, 4, ES><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, ldp, hi, lo, b2, sq); break;
        case 8: tc_pack_kernel<MODEL, T, I, 8, ES><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, ldp, hi, lo, b2, sq); break;
        default: set_error("dim %d > 1024 is not supported", a.dim); return KGE_E_UNSUPPORTED;
    }
    KGE_LAUNCH_CHECK("tc_pack_kernel");
    return 0;
}
template <int MODEL, int ES>
static int tc_pack_types(const ScoreArgs& a, int head, long long n_a, long long n_x, int ldp, void* hi, void* lo, void* b2, float* sq, cudaStream_t s) {
    if (a.dtype == KGE_F32)
        return a.id_bits == 64 ? tc_pack_go<MODEL, float, int64_t, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s)
                               : tc_pack_go<MODEL, float, int32_t, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
    return a.id_bits == 64 ? tc_pack_go<MODEL, __nv_bfloat16, int64_t, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s)
                           : tc_pack_go<MODEL, __nv_bfloat16, int32_t, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
}
template <int ES>
static int tc_pack_es(const ScoreArgs& a, int head, long long n_a, long long n_x, int ldp, void* hi, void* lo, void* b2, float* sq, cudaStream_t s) {
    switch (a.model) {
        case KGE_TRANSE: return tc_pack_types<KGE_TRANSE, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
        case KGE_DISTMULT: return tc_pack_types<KGE_DISTMULT, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
        case KGE_COMPLEX: return tc_pack_types<KGE_COMPLEX, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
        case KGE_RESCAL: return tc_pack_types<KGE_RESCAL, ES>(a, head, n_a, n_x, ldp, hi, lo, b2, sq, s);
        default: break;
    }
    set_error("model %d is not supported with chunk-shared negatives", a.model);
    return KGE_E_UNSUPPORTED;
}
static int tc_pack(const ScoreArgs& a, int head, long long n_a, long long n_x, const TcLayout& L, char* w, float* sq, cudaStream_t s) {
    void* hi = w + L.off_hi; void* lo = w + L.off_lo; void* b2 = L.third ? w + L.off_b2 : nullptr;
    return L.es == 2 ? tc_pack_es<2>(a, head, n_a, n_x, L.ldp, hi, lo, b2, sq, s) : tc_pack_es<4>(a, head, n_a, n_x, L.ldp, hi, lo, b2, sq, s);
}

template <typename T, typename I>
static int tc_fixup_go(const ScoreArgs& a, int head, const unsigned long long* cnt, const unsigned long long* list,
                       unsigned long long cap, cudaStream_t s) {
    switch (quads_per_lane(a.dim)) {
        case 1: tc_fixup_kernel<T, I, 1><<<296, 256, 0, s>>>(a, head, cnt, list, cap); break;
        case 2: tc_fixup_kernel<T, I, 2><<<296, 256, 0, s>>>(a, head, cnt, list, cap); break;
        case 4: tc_fixup_kernel<T, I, 4><<<296, 256, 0, s>>>(a, head, cnt, list, cap); break;
        case 8: tc_fixup_kernel<T, I, 8><<<296, 256, 0, s>>>(a, head, cnt, list, cap); break;
        default: return KGE_E_UNSUPPORTED;
    }
    KGE_LAUNCH_CHECK("tc_fixup_kernel");
    return 0;
}

// Tile width over `n` columns: one tile if it fits 256, else equal tiles, multiples of 16.
static int pick_bn(int n) {
    const int tiles = (n + 255) / 256;
    int bn = ((n + tiles - 1) / tiles + 15) / 16 * 16;
    return bn < 16 ? 16 : bn;
}

// ---- optional live timing of the tile kernel (CUDA events on the launching stream) ---------------------------------
static bool g_prof_on = false;
static double g_prof_flops = 0.0;
static long long g_prof_launches = 0;
static cudaEvent_t g_prof_ev[2 * 64];
static int g_prof_n = 0;                 // events pairs recorded and not yet read
static bool g_prof_events_made = false;

void gemm_profile_enable(int on) { g_prof_on = on != 0; g_prof_n = 0; g_prof_flops = 0.0; g_prof_launches = 0; }
int gemm_profile_read(double* ms, long long* launches, double* flops) {
    double total = 0.0;
    for (int i = 0; i < g_prof_n; ++i) {
        cudaError_t e = cudaEventSynchronize(g_prof_ev[2 * i + 1]);
        float t = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, g_prof_ev[2 * i], g_prof_ev[2 * i + 1]);
        if (e != cudaSuccess) return cuda_status(e, "gemm_profile_read");
        total += t;
    }
    if (ms) *ms = total;
    if (launches) *launches = g_prof_launches;
    if (flops) *flops = g_prof_flops;
    g_prof_n = 0; g_prof_flops = 0.0; g_prof_launches = 0;
    return 0;
}

static int run_gemm(const CUtensorMap& ah, const CUtensorMap& al, const CUtensorMap& bh, const CUtensorMap& bl, GemmTc& p,
                    long long batch, cudaStream_t s) {
    if ((p.elem_bytes != 2 && p.elem_bytes != 4) || (p.passes != 1 && p.passes != 3) || (p.tile_tab && p.elem_bytes != 2) || (p.pair && p.passes != 3)) {
        set_error("tile kernel: element size %d with %d passes is not built", p.elem_bytes, p.passes);
        return KGE_E_UNSUPPORTED;
    }
    p.err = device_error_word();
    if (!p.err) { set_error("no device error word"); return KGE_E_DEVICE; }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        return cuda_status(cudaGetLastError(), "cudaDeviceGetAttribute(multiprocessor count)");
    // the shared-memory opt-in is a per-device attribute of the kernel: remembered per device ordinal
    static std::atomic<bool> attr_set[128];
    if (dev < 0 || dev >= 128 || !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(umma_gemm_kernel<G_DENSE, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_MAX_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_gemm_kernel<G_DENSE, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_MAX_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_gemm_kernel<G_GROUPED, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_MAX_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_pair_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_MAX_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_MAX_SMEM);
        if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(tile kernels)");
        if (dev >= 0 && dev < 128) attr_set[dev].store(true, std::memory_order_release);
    }
    const int slab_cols = 128 / p.elem_bytes;
    const int b_cols = p.pair ? p.bn / 2 : p.bn;                     // B columns staged per CTA
    const int b_bytes = p.b_mn ? ((b_cols + slab_cols - 1) / slab_cols) * (slab_cols * 128) : b_cols * 128;
    const int stage_bytes = (p.passes == 1 ? 1 : 2) * (UM_A_BYTES + b_bytes);
    p.stages = (UM_MAX_SMEM - 1024 - UM_TAIL_BYTES) / stage_bytes;
    if (p.stages > 6) p.stages = 6;
    const size_t smem = static_cast<size_t>(p.stages) * stage_bytes + 1024 + UM_TAIL_BYTES;
    p.batch = (int)batch;
    const int tile_rows = p.pair ? 2 * UM_BM : UM_BM;
    const long long n_tiles = (long long)((p.n_cols + p.bn - 1) / p.bn) * ((p.m_rows + tile_rows - 1) / tile_rows) * batch;
    const long long bound = p.tile_tab ? p.tile_cap : n_tiles;      // grouped mode: the tile count is only known on the device
    if (bound >= (1LL << 31)) { set_error("tile kernel: %lld tiles exceed the 32-bit tile index", bound); return KGE_E_SHAPE; }
    const int slots = p.pair ? sms / 2 : sms;                       // persistent: one CTA (or CTA pair) per SM (pair of SMs)
    const unsigned ctas = (unsigned)(bound < slots ? bound : slots) * (p.pair ? 2u : 1u);
    const bool prof = g_prof_on && g_prof_n < 64;
    if (prof) {
        if (!g_prof_events_made) {
            for (int i = 0; i < 128; ++i)
                if (cudaEventCreate(&g_prof_ev[i]) != cudaSuccess) return cuda_status(cudaGetLastError(), "cudaEventCreate");
            g_prof_events_made = true;
        }
        cudaEventRecord(g_prof_ev[2 * g_prof_n], s);
    }
    if (p.pair) {
        if (p.elem_bytes == 2) umma_pair_kernel<2><<<ctas, UM_THREADS, smem, s>>>(ah, al, bh, bl, p);
        else umma_pair_kernel<4><<<ctas, UM_THREADS, smem, s>>>(ah, al, bh, bl, p);
        KGE_LAUNCH_CHECK("umma_pair_kernel");
    } else {
        if (p.tile_tab) umma_gemm_kernel<G_GROUPED, 2><<<ctas, UM_THREADS_GROUPED, smem, s>>>(ah, al, bh, bl, p);
        else if (p.elem_bytes == 2) umma_gemm_kernel<G_DENSE, 2><<<ctas, UM_THREADS, smem, s>>>(ah, al, bh, bl, p);
        else umma_gemm_kernel<G_DENSE, 4><<<ctas, UM_THREADS, smem, s>>>(ah, al, bh, bl, p);
        KGE_LAUNCH_CHECK("umma_gemm_kernel");
    }
    if (prof) {
        cudaEventRecord(g_prof_ev[2 * g_prof_n + 1], s);
        ++g_prof_n; ++g_prof_launches;
        g_prof_flops += 2.0 * p.m_rows * (double)p.n_cols * p.k_len * (double)batch;
    }
    return 0;
}

// Forward scores of the chunk's negatives.  ws: tc_pair_workspace_bytes(batch, chunk, n_neg, dim, 0).
int launch_pair_forward_tc(const ScoreArgs& a, int head, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    if (a.dim % 4 != 0) { set_error("the tensor-core path needs dim %% 4 == 0 (16-byte rows), got %d", a.dim); return KGE_E_UNSUPPORTED; }
    const long long n_chunks = a.batch / a.chunk;
    const long long n_a = a.batch, n_x = n_chunks * a.n_neg;
    const bool dist = a.model == KGE_TRANSE;
    const int es = a.tc_es == 4 ? 4 : 2, bk = 128 / es;
    const TcLayout L = tc_layout(a.batch, a.chunk, a.n_neg, a.dim, 0, es, dist);
    if (ws_bytes < L.total) { set_error("tensor-core workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* w = static_cast<char*>(ws);
    char* hi = w + L.off_hi;
    char* lo = w + L.off_lo;
    float* sq = reinterpret_cast<float*>(w + L.off_sq);
    unsigned long long* fixc = reinterpret_cast<unsigned long long*>(w + L.off_fixc);
    unsigned long long* fixl = reinterpret_cast<unsigned long long*>(w + L.off_fixl);
    int rc = tc_pack(a, head, n_a, n_x, L, w, sq, s);
    if (rc) return rc;
    if (dist) {
        cudaError_t e = cudaMemsetAsync(fixc, 0, 8, s);
        if (e != cudaSuccess) return cuda_status(e, "cudaMemsetAsync(fix counter)");
    }
    // n_neg rows need 16-byte row pitch in the output only for vector stores; tensor maps need dim % 4 == 0 (checked)
    CUtensorMap mah, mal, mbh, mbl;
    const uint64_t ld = static_cast<uint64_t>(L.ldp) * es;
    const bool pair = L.fwd_pair != 0;
    const int bn = L.fwd_bn;
    const int b_box = pair ? bn / 2 : bn;           // a CTA of a pair stages half of the tile's columns
    if ((rc = make_tensor_map_3d(&mah, hi, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, UM_BM, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mal, lo, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, UM_BM, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mbh, hi + n_a * ld, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, b_box, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mbl, lo + n_a * ld, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, b_box, bk))) return rc;
    GemmTc p;
    memset(&p, 0, sizeof(p));
    p.m_rows = a.chunk; p.n_cols = a.n_neg; p.k_len = a.dim; p.bn = bn; p.a_mn = 0; p.b_mn = 0; p.pair = pair;
    p.elem_bytes = es; p.passes = 3;
    p.ep = dist ? EP_DIST : EP_STORE;
    p.out = a.negs; p.out_ld = a.n_neg; p.out_batch_rows = a.chunk;
    p.sq_a = sq; p.sq_b = sq + n_a; p.fix_count = fixc; p.fix_list = fixl; p.fix_cap = L.fix_cap;
    if ((rc = run_gemm(mah, mal, mbh, mbl, p, n_chunks, s))) return rc;
    if (dist) {
        if (a.dtype == KGE_F32) rc = a.id_bits == 64 ? tc_fixup_go<float, int64_t>(a, head, fixc, fixl, L.fix_cap, s)
                                                     : tc_fixup_go<float, int32_t>(a, head, fixc, fixl, L.fix_cap, s);
        else rc = a.id_bits == 64 ? tc_fixup_go<__nv_bfloat16, int64_t>(a, head, fixc, fixl, L.fix_cap, s)
                                  : tc_fixup_go<__nv_bfloat16, int32_t>(a, head, fixc, fixl, L.fix_cap, s);
        if (rc) return rc;
        ScoreArgs g = a;                    // exact kernel behind a device-side guard: runs only if the list overflowed
        g.guard = fixc; g.guard_cap = L.fix_cap;
        rc = launch_pair_forward(g, head, s);
    }
    return rc;
}

// The two backward products from W (split, in the workspace) and the packed operands: GA = W . X and GX = W^T . A, with
// the rank-1 terms of the distance scorer (row / column sums of W).
static int tc_backward_products(const ScoreArgs& a, const TcLayout& L, char* w, bool dist, float* ga, const float** ga_scale,
                                cudaStream_t s) {
    const long long n_chunks = a.batch / a.chunk;
    const long long n_a = a.batch;
    const int es = L.es, bk = 128 / es, slab = 128 / es;
    char* hi = w + L.off_hi;
    char* lo = w + L.off_lo;
    char* whi = w + L.off_whi;
    char* wlo = w + L.off_wlo;
    float* rowsum = reinterpret_cast<float*>(w + L.off_rowsum);
    float* colsum = reinterpret_cast<float*>(w + L.off_colsum);
    int rc = 0;
    const uint64_t ld = static_cast<uint64_t>(L.ldp) * es, lw = static_cast<uint64_t>(L.ldw) * es;
    // Pairs with an MN-major B: tiles are whole slabs per CTA (multiples of two slabs), the last one narrowed by the kernel.
    // The packed matrices have whole-slab pitches, so MN-major operands are read through 4-D slab maps (one copy per stage);
    // the one-CTA kernel keeps per-slab copies for B because its tile width need not be a whole number of slabs.
    const bool pair_ga = want_pair(a.chunk, a.dim), pair_gx = want_pair(a.n_neg, a.dim);
    const int unit = 2 * slab;
    const int bnp = a.dim >= 256 ? 256 : (a.dim + unit - 1) / unit * unit;
    const char* xhi = hi + n_a * ld;
    const char* xlo = lo + n_a * ld;
    CUtensorMap mah, mal, mbh, mbl;
    GemmTc p;
    // GA = W . X : A = W K-major (rows i, K = j), B = X MN-major (N = dim, K rows = j)
    memset(&p, 0, sizeof(p));
    p.m_rows = a.chunk; p.n_cols = a.dim; p.k_len = a.n_neg; p.bn = pair_ga ? bnp : pick_bn(a.dim); p.a_mn = 0; p.b_mn = 1; p.pair = pair_ga;
    p.elem_bytes = es; p.passes = 3;
    if ((rc = make_tensor_map_3d(&mah, whi, es, n_chunks, a.chunk, a.n_neg, lw, lw * a.chunk, UM_BM, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mal, wlo, es, n_chunks, a.chunk, a.n_neg, lw, lw * a.chunk, UM_BM, bk))) return rc;
    if (pair_ga) {
        p.b_slabs4d = 1;
        if ((rc = make_tensor_map_slabs(&mbh, xhi, es, n_chunks, a.n_neg, L.ldp, ld, ld * a.n_neg, bk, bnp / unit))) return rc;
        if ((rc = make_tensor_map_slabs(&mbl, xlo, es, n_chunks, a.n_neg, L.ldp, ld, ld * a.n_neg, bk, bnp / unit))) return rc;
    } else {
        if ((rc = make_tensor_map_3d(&mbh, xhi, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, bk, slab, es == 4))) return rc;
        if ((rc = make_tensor_map_3d(&mbl, xlo, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, bk, slab, es == 4))) return rc;
    }
    p.ep = EP_STORE;
    p.out = ga; p.out_ld = a.dim; p.out_batch_rows = a.chunk;
    if (dist) *ga_scale = rowsum;
    if ((rc = run_gemm(mah, mal, mbh, mbl, p, n_chunks, s))) return rc;
    // GX = W^T . A : A-operand = W MN-major (M = j, K rows = i), B = anchors MN-major (N = dim, K rows = i)
    memset(&p, 0, sizeof(p));
    p.m_rows = a.n_neg; p.n_cols = a.dim; p.k_len = a.chunk; p.bn = pair_gx ? bnp : pick_bn(a.dim); p.a_mn = 1; p.b_mn = 1; p.pair = pair_gx;
    p.elem_bytes = es; p.passes = 3;
    p.a_slabs4d = 1;
    if ((rc = make_tensor_map_slabs(&mah, whi, es, n_chunks, a.chunk, L.ldw, lw, lw * a.chunk, bk, UM_BM / slab))) return rc;
    if ((rc = make_tensor_map_slabs(&mal, wlo, es, n_chunks, a.chunk, L.ldw, lw, lw * a.chunk, bk, UM_BM / slab))) return rc;
    if (pair_gx) {
        p.b_slabs4d = 1;
        if ((rc = make_tensor_map_slabs(&mbh, hi, es, n_chunks, a.chunk, L.ldp, ld, ld * a.chunk, bk, bnp / unit))) return rc;
        if ((rc = make_tensor_map_slabs(&mbl, lo, es, n_chunks, a.chunk, L.ldp, ld, ld * a.chunk, bk, bnp / unit))) return rc;
    } else {
        if ((rc = make_tensor_map_3d(&mbh, hi, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, bk, slab, es == 4))) return rc;
        if ((rc = make_tensor_map_3d(&mbl, lo, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, bk, slab, es == 4))) return rc;
    }
    p.ep = dist ? EP_RANK1 : EP_STORE;
    p.out = a.g_neg; p.out_ld = a.dim; p.out_batch_rows = a.n_neg;
    p.scale = colsum; p.y_hi = xhi; p.y_lo = xlo; p.y_ld = L.ldp;
    return run_gemm(mah, mal, mbh, mbl, p, n_chunks, s);
}

// Backward contractions.  ga: (batch, dim) fp32 anchor-gradient rows; g_neg rows are written to a.g_neg.  For the distance
// scorer ga holds only sum_j W_ij x_j and *ga_scale the row sums of W: the anchor gradient is ga_scale[i] * anchor_i - ga_i,
// applied by the per-triple backward kernel, which has the anchor row in registers anyway (else *ga_scale is NULL).
// ws: tc_pair_workspace_bytes(batch, chunk, n_neg, dim, 1).
int launch_pair_backward_tc(const ScoreArgs& a, int head, float* ga, const float** ga_scale, void* ws, size_t ws_bytes, cudaStream_t s) {
    *ga_scale = nullptr;
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    if (a.dim % 4 != 0) { set_error("the tensor-core path needs dim %% 4 == 0 (16-byte rows), got %d", a.dim); return KGE_E_UNSUPPORTED; }
    const long long n_chunks = a.batch / a.chunk;
    const long long n_a = a.batch, n_x = n_chunks * a.n_neg;
    const bool dist = a.model == KGE_TRANSE;
    const int es = a.tc_es == 4 ? 4 : 2;
    const TcLayout L = tc_layout(a.batch, a.chunk, a.n_neg, a.dim, 1, es, dist);
    if (ws_bytes < L.total) { set_error("tensor-core workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* w = static_cast<char*>(ws);
    void* whi = w + L.off_whi;
    void* wlo = w + L.off_wlo;
    float* rowsum = reinterpret_cast<float*>(w + L.off_rowsum);
    float* colsum = reinterpret_cast<float*>(w + L.off_colsum);
    float* colpart = reinterpret_cast<float*>(w + L.off_colpart);
    int rc = tc_pack(a, head, n_a, n_x, L, w, nullptr, s);
    if (rc) return rc;
    if (dist) {
        const int bpc = (a.chunk + TW_ROWS - 1) / TW_ROWS;
        const dim3 grid(bpc, (unsigned)n_chunks);
        if (es == 2) tc_pack_w_sums_kernel<2><<<grid, 256, 0, s>>>(a.dneg, a.negs, a.chunk, a.n_neg, L.ldw, whi, wlo, rowsum, colpart);
        else tc_pack_w_sums_kernel<4><<<grid, 256, 0, s>>>(a.dneg, a.negs, a.chunk, a.n_neg, L.ldw, whi, wlo, rowsum, colpart);
        KGE_LAUNCH_CHECK("tc_pack_w_sums_kernel");
        tc_colsum_kernel<<<dim3((a.n_neg + 255) / 256, (unsigned)n_chunks), 256, 0, s>>>(colpart, bpc, a.n_neg, colsum);
        KGE_LAUNCH_CHECK("tc_colsum_kernel");
    } else {
        const int wpb = 8;
        const unsigned blocks = (unsigned)((a.batch + wpb - 1) / wpb);
        if (es == 2) tc_pack_w_kernel<2><<<blocks, wpb * 32, 0, s>>>(a.dneg, a.batch, a.n_neg, L.ldw, whi, wlo);
        else tc_pack_w_kernel<4><<<blocks, wpb * 32, 0, s>>>(a.dneg, a.batch, a.n_neg, L.ldw, whi, wlo);
        KGE_LAUNCH_CHECK("tc_pack_w_kernel");
    }
    return tc_backward_products(a, L, w, dist, ga, ga_scale, s);
}


// ---- fused forward + logistic loss + backward (chunk-shared negatives) -----------------------------------------------
// rowsum[i] = sum_t rowpart[t][i], t ascending.
__global__ void __launch_bounds__(256) tc_rowsum_kernel(const float* rowpart, int parts, long long rows, float* rowsum) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows) return;
    float s = 0.f;
    for (int t = 0; t < parts; ++t) s += rowpart[(long long)t * rows + i];
    rowsum[i] = s;
}
// loss[0] += sum of the partials, in a fixed order (thread-strided, then a tree).
__global__ void __launch_bounds__(1024) tc_loss_add_kernel(const float* part, long long n, float* loss) {
    __shared__ float red[1024];
    float s = 0.f;
    for (long long i = threadIdx.x; i < n; i += 1024) s += part[i];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) { if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) *loss += red[0];
}

// loss[0] += sum of part[0..n), in the fixed order of tc_loss_add_kernel.
int launch_loss_add(const float* part, long long n, float* loss, cudaStream_t s) {
    tc_loss_add_kernel<<<1, 1024, 0, s>>>(part, n, loss);
    KGE_LAUNCH_CHECK("tc_loss_add_kernel");
    return 0;
}

// Scores of the negatives, their logistic loss and the backward products in one pass: the forward tile kernel turns each
// score into its loss term and its W entry in the epilogue (EP_LOSS), so the (batch x n_neg) score matrix, its gradient
// and a second operand pack are never written or read.  loss[0] must be initialised by the caller; the
// negatives' part is added to it.  ga / *ga_scale as in launch_pair_backward_tc; g_neg rows go to a.g_neg.
// ws: tc_pair_workspace_bytes(batch, chunk, n_neg, dim, 2).
int launch_pair_loss_backward_tc(const ScoreArgs& a, int head, float neg_w, float* loss, float* ga, const float** ga_scale,
                                 void* ws, size_t ws_bytes, cudaStream_t s) {
    *ga_scale = nullptr;
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    if (a.dim % 4 != 0) { set_error("the tensor-core path needs dim %% 4 == 0 (16-byte rows), got %d", a.dim); return KGE_E_UNSUPPORTED; }
    const long long n_chunks = a.batch / a.chunk;
    const long long n_a = a.batch, n_x = n_chunks * a.n_neg;
    const bool dist = a.model == KGE_TRANSE;
    const int es = a.tc_es == 4 ? 4 : 2, bk = 128 / es;
    const TcLayout L = tc_layout(a.batch, a.chunk, a.n_neg, a.dim, 2, es, dist);
    if (ws_bytes < L.total) { set_error("tensor-core workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* w = static_cast<char*>(ws);
    char* hi = w + L.off_hi;
    char* lo = w + L.off_lo;
    float* sq = reinterpret_cast<float*>(w + L.off_sq);
    float* rowsum = reinterpret_cast<float*>(w + L.off_rowsum);
    float* colsum = reinterpret_cast<float*>(w + L.off_colsum);
    float* colpart = reinterpret_cast<float*>(w + L.off_colpart);
    float* rowpart = reinterpret_cast<float*>(w + L.off_rowpart);
    float* losspart = reinterpret_cast<float*>(w + L.off_losspart);
    int rc = tc_pack(a, head, n_a, n_x, L, w, sq, s);
    if (rc) return rc;
    CUtensorMap mah, mal, mbh, mbl;
    const uint64_t ld = static_cast<uint64_t>(L.ldp) * es;
    const bool pair = L.fwd_pair != 0;
    const int bn = L.fwd_bn;
    const int b_box = pair ? bn / 2 : bn;
    if ((rc = make_tensor_map_3d(&mah, hi, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, UM_BM, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mal, lo, es, n_chunks, a.chunk, a.dim, ld, ld * a.chunk, UM_BM, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mbh, hi + n_a * ld, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, b_box, bk))) return rc;
    if ((rc = make_tensor_map_3d(&mbl, lo + n_a * ld, es, n_chunks, a.n_neg, a.dim, ld, ld * a.n_neg, b_box, bk))) return rc;
    GemmTc p;
    memset(&p, 0, sizeof(p));
    p.m_rows = a.chunk; p.n_cols = a.n_neg; p.k_len = a.dim; p.bn = bn; p.a_mn = 0; p.b_mn = 0; p.pair = pair;
    p.elem_bytes = es; p.passes = 3;
    p.ep = EP_LOSS;
    p.sq_a = sq; p.sq_b = sq + n_a; p.loss_dist = dist ? 1 : 0; p.neg_w = neg_w;
    p.w_hi = w + L.off_whi; p.w_lo = w + L.off_wlo; p.ldw = L.ldw;
    p.rowpart = rowpart; p.colpart = colpart; p.loss_part = losspart;
    p.ex_a_hi = hi; p.ex_a_lo = lo; p.ex_x_hi = hi + n_a * ld; p.ex_x_lo = lo + n_a * ld; p.ex_ld = L.ldp;
    if (L.third) { p.ex_a_b2 = w + L.off_b2; p.ex_x_b2 = w + L.off_b2 + n_a * ld; }
    if ((rc = run_gemm(mah, mal, mbh, mbl, p, n_chunks, s))) return rc;
    const long long tiles_n = (a.n_neg + bn - 1) / bn;
    const long long tiles = tiles_n * ((a.chunk + (pair ? 2 : 1) * UM_BM - 1) / ((pair ? 2 : 1) * UM_BM)) * n_chunks;
    tc_loss_add_kernel<<<1, 1024, 0, s>>>(losspart, tiles * (pair ? 2 : 1) * UM_EPI_WARPS, loss);
    KGE_LAUNCH_CHECK("tc_loss_add_kernel");
    if (dist) {
        tc_rowsum_kernel<<<(unsigned)((a.batch + 255) / 256), 256, 0, s>>>(rowpart, (int)(2 * tiles_n), a.batch, rowsum);
        KGE_LAUNCH_CHECK("tc_rowsum_kernel");
        tc_colsum_kernel<<<dim3((a.n_neg + 255) / 256, (unsigned)n_chunks), 256, 0, s>>>(colpart, (a.chunk + 31) / 32, a.n_neg, colsum);
        KGE_LAUNCH_CHECK("tc_colsum_kernel");
    }
    return tc_backward_products(a, L, w, dist, ga, ga_scale, s);
}

// ---- TransR forward on the tensor cores (bf16 tables) ---------------------------------------------------------------
// score(i, j) = -|| (a - b) . P[r_i] + R[r_i] ||.  The inspector has grouped the triples by relation; every group's
// difference rows (1 + n_neg per triple, positive first) are packed as bf16 into one matrix, each group padded to a
// multiple of 128 rows, so a 128-row tile never mixes relations.  The tile list (row offset, relation id) is built on the
// device; umma_gemm_kernel runs it in grouped mode with B = P[relation] read straight from the table by TMA (MN-major:
// out[j] = sum_i x[i] P[r][i][j] needs no transpose) and the EP_NORM epilogue.  Needs dim <= 256 (one n-tile per row).
struct TransRPlan {
    const int* rel_perm; const int* rel_seg; const long long* rel_uniq; const long long* n_groups;
    int per;                    // rows per triple: 1 + n_neg
    int4* tile_tab; long long* n_tiles;
    long long tile_cap;
    int4* tile_tab2; long long* n_tiles2; int tiles_m2;     // grouped-K tiles of the dP product (backward), or NULL
    int z_is_group;             // the B matrices are packed per GROUP (RESCAL over fp32 tables): z = group index, not relation id
};

// One block: tiles per group, exclusive scan, tile table (first padded row, relation id, group, valid rows).
__global__ void __launch_bounds__(1024) transr_plan_kernel(TransRPlan pl) {
    __shared__ long long part[1024];
    const int G = (int)*pl.n_groups;
    const int tid = threadIdx.x;
    const int chunk = (G + 1023) / 1024;
    const int g0 = min(G, tid * chunk), g1 = min(G, g0 + chunk);
    long long mine = 0;
    for (int g = g0; g < g1; ++g) mine += ((long long)(pl.rel_seg[g + 1] - pl.rel_seg[g]) * pl.per + UM_BM - 1) / UM_BM;
    part[tid] = mine;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {            // Hillis-Steele inclusive scan, double-synchronised
        const long long v = tid >= o ? part[tid - o] : 0;
        __syncthreads();
        part[tid] += v;
        __syncthreads();
    }
    long long t0 = part[tid] - mine;
    if (tid == 1023) *pl.n_tiles = part[1023] < pl.tile_cap ? part[1023] : pl.tile_cap;
    for (int g = g0; g < g1; ++g) {
        const long long rows = (long long)(pl.rel_seg[g + 1] - pl.rel_seg[g]) * pl.per;
        const long long nt = (rows + UM_BM - 1) / UM_BM;
        const int z = pl.z_is_group ? g : (int)pl.rel_uniq[g];
        for (long long t = 0; t < nt && t0 + t < pl.tile_cap; ++t)
            pl.tile_tab[t0 + t] = make_int4((int)((t0 + t) * UM_BM), z, g, (int)min((long long)UM_BM, rows - t * UM_BM));
        if (pl.tile_tab2)
            for (int mt = 0; mt < pl.tiles_m2; ++mt)
                pl.tile_tab2[(long long)g * pl.tiles_m2 + mt] = make_int4((int)(t0 * UM_BM), (int)(nt * UM_BM), mt * UM_BM, g);
        t0 += nt;
    }
    if (pl.tile_tab2 && tid == 0) *pl.n_tiles2 = (long long)G * pl.tiles_m2;
}

// One CTA per tile (8 warps x 16 rows): difference rows of the tile's group as bf16, and where each row's score goes.
template <typename I, int NV>
__global__ void __launch_bounds__(256) transr_pack_kernel(ScoreArgs a, TransRPlan pl, __nv_bfloat16* rows_out, long long* row_dst,
                                                          float* coef, int* trow0) {
    const long long tile = blockIdx.x;
    if (tile >= *pl.n_tiles) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int4 tt = pl.tile_tab[tile];
    const int g = tt.z, valid = tt.w;
    // first group-local row of this tile: tiles of a group are consecutive, the group's first tile starts at its first row
    long long first = tt.x;
    {   // walk back to the group's first tile (a group has few tiles)
        long long t = tile;
        while (t > 0 && pl.tile_tab[t - 1].z == g) --t;
        first = (long long)tt.x - pl.tile_tab[t].x;
    }
    const int dim = a.dim;
    const __nv_bfloat16* E = reinterpret_cast<const __nv_bfloat16*>(a.ent);
    for (int rr = warp; rr < UM_BM; rr += 8) {
        const long long prow = (long long)tt.x + rr;
        if (rr >= valid) {                                                       // padding row: zeros, no score, no gradient
            for (int k = lane * 4; k < dim; k += 128) *reinterpret_cast<uint2*>(rows_out + prow * dim + k) = make_uint2(0u, 0u);
            if (lane == 0) { row_dst[prow] = -1; if (coef) coef[prow] = 0.f; }
            continue;
        }
        const long long rho = first + rr;                                        // row within the group
        const int p = pl.rel_seg[g] + (int)(rho / pl.per), j = (int)(rho % pl.per);
        const int i = pl.rel_perm[p];
        const __nv_bfloat16* hrow = E + load_id<I>(a.h, i) * dim;
        const __nv_bfloat16* trow = E + load_id<I>(a.t, i) * dim;
        const __nv_bfloat16 *pa = hrow, *pb = trow;
        if (j > 0) {
            const __nv_bfloat16* x = E + load_id<I>(a.neg, (long long)i * a.n_neg + (j - 1)) * dim;
            if (j - 1 < a.n_neg_head) pa = x; else pb = x;
        }
        Row<NV> ra, rb;
        load_row<__nv_bfloat16, NV, true>(ra, pa, dim, lane);
        load_row<__nv_bfloat16, NV, true>(rb, pb, dim, lane);
        __nv_bfloat16* out = rows_out + prow * dim;
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            const int k = 4 * (lane + 32 * q);
            if (k < dim) {
                const float4 d = ra.v[q] - rb.v[q];
                __nv_bfloat162 p0 = __floats2bfloat162_rn(d.x, d.y), p1 = __floats2bfloat162_rn(d.z, d.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&p0); u.y = *reinterpret_cast<unsigned*>(&p1);
                *reinterpret_cast<uint2*>(out + k) = u;
            }
        }
        if (lane == 0) {
            // a tail-replaced negative receives minus the row gradient in the backward; the side is folded into the slot
            // number here (+ kTailSide) so that the scatter epilogue needs no division per row (the norm epilogue strips it)
            const bool tail_side = j > 0 && j - 1 >= a.n_neg_head;
            row_dst[prow] = j == 0 ? -2 - (long long)i : (long long)i * a.n_neg + (j - 1) + (tail_side ? kTailSide : 0);
            if (coef) {      // dL/dv = (dS / S) v
                const float sc = j == 0 ? a.pos[i] : a.negs[(long long)i * a.n_neg + (j - 1)];
                const float ds = j == 0 ? a.dpos[i] : a.dneg[(long long)i * a.n_neg + (j - 1)];
                coef[prow] = sc != 0.f ? ds / sc : 0.f;
                if (j == 0) trow0[i] = (int)prow;
            }
        }
    }
}

// dL/dv coefficients of the packed rows from the scores and their gradients (fused step: the rows were packed before the
// scores existed): coef[row] = dS / S, and trow0[i] = packed row of triple i's positive.
__global__ void __launch_bounds__(256) transr_coef_kernel(ScoreArgs a, const long long* row_dst, const long long* n_tiles, float* coef, int* trow0) {
    const long long prow = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (prow >= *n_tiles * UM_BM) return;
    long long dst = row_dst[prow];
    if (dst == -1) { coef[prow] = 0.f; return; }
    float sc, ds;
    if (dst <= -2) { const long long i = -2 - dst; sc = a.pos[i]; ds = a.dpos[i]; trow0[i] = (int)prow; }
    else { if (dst >= kTailSide) dst -= kTailSide; sc = a.negs[dst]; ds = a.dneg[dst]; }
    coef[prow] = sc != 0.f ? ds / sc : 0.f;
}

// Per triple: g_head = GD0 - sum of its tail-replaced g_neg rows, g_tail = -GD0 - sum of its head-replaced g_neg rows,
// g_rel = sum of its dL/dv rows (bf16, consecutive in the packed order), all in ascending j.  One warp per triple, lane L
// owns quads L and L + 32 of a row (dim <= 256); four rows are requested before the first is added.
__global__ void __launch_bounds__(256) transr_reduce_tc_kernel(ScoreArgs a, const __nv_bfloat16* gv, const float* gd0, const int* trow0) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= a.batch) return;
    const int dim = a.dim, n_neg = a.n_neg;
    const long long r0 = trow0[i];
    Row<2> g0, gh, gt, gr;
    load_row_f32<2, true>(g0, gd0 + i * dim, dim, lane);
    load_row<__nv_bfloat16, 2, true>(gr, gv + r0 * dim, dim, lane);
#pragma unroll
    for (int q = 0; q < 2; ++q) { gh.v[q] = g0.v[q]; gt.v[q] = -1.f * g0.v[q]; }
    for (int j0 = 0; j0 < n_neg; j0 += 4) {
        Row<2> gx[4], gvr[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (j0 + u < n_neg) {
                load_row_f32<2, true>(gx[u], a.g_neg + (i * n_neg + j0 + u) * dim, dim, lane);
                load_row<__nv_bfloat16, 2, true>(gvr[u], gv + (r0 + 1 + j0 + u) * dim, dim, lane);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (j0 + u < n_neg) {
                const bool head_side = j0 + u < a.n_neg_head;
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    if (head_side) gt.v[q] = gt.v[q] - gx[u].v[q]; else gh.v[q] = gh.v[q] - gx[u].v[q];
                    gr.v[q] = gr.v[q] + gvr[u].v[q];
                }
            }
        }
    }
    store_row<2, true>(a.g_head + i * dim, gh, dim, lane);
    store_row<2, true>(a.g_tail + i * dim, gt, dim, lane);
    store_row<2, true>(a.g_rel + i * dim, gr, dim, lane);
}

struct TransRLayout { size_t off_rows, off_dst, off_tab, off_nt, off_tab2, off_coef, off_trow0, off_gv, off_gd0, off_negs, off_dpos, off_dneg, off_loss, total;
                      long long rows_cap, tile_cap, gmax; int tiles_m2; };
// mode 0: forward, 1: backward, 2: fused forward + loss + backward (scores of the negatives and the score gradients live in the workspace)
static TransRLayout transr_layout(long long batch, int n_neg, int dim, long long n_rel, int mode = 0) {
    const bool backward = mode != 0;
    TransRLayout L;
    const long long gmax = n_rel < batch ? n_rel : batch;
    L.rows_cap = batch * (1 + n_neg) + gmax * UM_BM;
    L.tile_cap = L.rows_cap / UM_BM + 1;
    size_t o = 0;
    L.off_rows = o; o += al256((size_t)L.rows_cap * dim * 2);
    L.off_dst = o; o += al256((size_t)L.rows_cap * 8);
    L.off_tab = o; o += al256((size_t)L.tile_cap * 16);
    L.off_nt = o; o += 256;
    L.gmax = gmax; L.tiles_m2 = (dim + UM_BM - 1) / UM_BM;
    L.off_tab2 = o; o += backward ? al256((size_t)gmax * L.tiles_m2 * 16) : 0;
    L.off_coef = o; o += backward ? al256((size_t)L.rows_cap * 4) : 0;
    L.off_trow0 = o; o += backward ? al256((size_t)batch * 4) : 0;
    L.off_gv = o; o += backward ? al256((size_t)L.rows_cap * dim * 2) : 0;
    L.off_gd0 = o; o += backward ? al256((size_t)batch * dim * 4) : 0;
    const size_t nneg = (size_t)batch * (n_neg > 0 ? n_neg : 0);
    L.off_negs = o; o += mode == 2 ? al256(nneg * 4 + 16) : 0;
    L.off_dpos = o; o += mode == 2 ? al256((size_t)batch * 4) : 0;
    L.off_dneg = o; o += mode == 2 ? al256(nneg * 4 + 16) : 0;
    L.off_loss = o; o += mode == 2 ? 4096 : 0;
    L.total = o;
    return L;
}
size_t tc_transr_workspace_bytes(long long batch, int n_neg, int dim, long long n_rel, int mode) {
    return transr_layout(batch, n_neg, dim, n_rel, mode).total;
}
int launch_logistic_loss(const float* pos, long long n_pos, const float* neg, long long n_neg, float neg_w, float* dpos,
                         float* dneg, float* loss, void* ws, size_t ws_bytes, cudaStream_t s);      // inspector.cu

// a: ScoreArgs of the problem (bf16 tables); rel grouping from the inspector over r.  backward == false: scores into
// a.pos / a.negs.  backward == true: a.pos/a.negs/a.dpos/a.dneg are inputs, gradients go to a.g_head, a.g_tail, a.g_neg,
// a.g_rel and dproj (n_groups, dim, dim).
// mode 0: scores into a.pos / a.negs.  mode 1: a.pos / a.negs / a.dpos / a.dneg are inputs, gradients go to a.g_head, a.g_tail,
// a.g_neg, a.g_rel and dproj (n_groups, dim, dim).  mode 2: both in one pass over ONE pack of the difference rows, with the
// logistic loss in between (a.pos and `loss` are outputs; negative scores and score gradients stay in the workspace).
static int transr_tc(const ScoreArgs& a_in, int mode, float neg_w, float* loss, float* dproj, const int* rel_perm, const int* rel_seg,
                     const long long* rel_uniq, const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes, cudaStream_t s) {
    ScoreArgs a = a_in;
    if (a.batch <= 0) return 0;
    const bool backward = mode != 0;
    const TransRLayout L = transr_layout(a.batch, a.n_neg, a.dim, n_rel, mode);
    if (ws_bytes < L.total) { set_error("TransR tensor-core workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* w = static_cast<char*>(ws);
    __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(w + L.off_rows);
    long long* dst = reinterpret_cast<long long*>(w + L.off_dst);
    float* coef = backward ? reinterpret_cast<float*>(w + L.off_coef) : nullptr;
    int* trow0 = backward ? reinterpret_cast<int*>(w + L.off_trow0) : nullptr;
    if (mode == 2) {
        a.negs = reinterpret_cast<float*>(w + L.off_negs);
        a.dpos = reinterpret_cast<float*>(w + L.off_dpos);
        a.dneg = reinterpret_cast<float*>(w + L.off_dneg);
    }
    float* pack_coef = mode == 1 ? coef : nullptr;          // the fused step packs before the scores exist
    __nv_bfloat16* gv = reinterpret_cast<__nv_bfloat16*>(w + L.off_gv);
    float* gd0 = reinterpret_cast<float*>(w + L.off_gd0);
    TransRPlan pl;
    pl.rel_perm = rel_perm; pl.rel_seg = rel_seg; pl.rel_uniq = rel_uniq; pl.n_groups = n_groups; pl.per = 1 + a.n_neg;
    pl.tile_tab = reinterpret_cast<int4*>(w + L.off_tab); pl.n_tiles = reinterpret_cast<long long*>(w + L.off_nt);
    pl.tile_cap = L.tile_cap;
    pl.tile_tab2 = backward ? reinterpret_cast<int4*>(w + L.off_tab2) : nullptr;
    pl.n_tiles2 = pl.n_tiles + 1; pl.tiles_m2 = L.tiles_m2; pl.z_is_group = 0;
    transr_plan_kernel<<<1, 1024, 0, s>>>(pl);
    KGE_LAUNCH_CHECK("transr_plan_kernel");
    {
        const unsigned blocks = (unsigned)L.tile_cap;            // one CTA per tile; CTAs past the device-side tile count exit
        const int nv = quads_per_lane(a.dim);
#define KGE_TP(N)                                                                                          \
        case N: if (a.id_bits == 64) transr_pack_kernel<int64_t, N><<<blocks, 256, 0, s>>>(a, pl, rows, dst, pack_coef, trow0);  \
                else transr_pack_kernel<int32_t, N><<<blocks, 256, 0, s>>>(a, pl, rows, dst, pack_coef, trow0); break;
        switch (nv) { KGE_TP(1) KGE_TP(2) default: set_error("TransR tensor-core path needs dim <= 256"); return KGE_E_UNSUPPORTED; }
#undef KGE_TP
        KGE_LAUNCH_CHECK("transr_pack_kernel");
    }
    CUtensorMap ma, mb;
    int rc;
    const uint64_t lda = (uint64_t)a.dim * 2;
    const int bn = (a.dim + 15) / 16 * 16;
    // v = diff . P[r]: A = packed rows (K-major), B = P[r] as stored (MN-major)
    if ((rc = make_tensor_map_3d(&ma, rows, 2, 1, L.rows_cap, a.dim, lda, lda * L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mb, a.rel2, 2, n_rel, a.dim, a.dim, lda, lda * a.dim, 64, 64))) return rc;
    GemmTc p;
    memset(&p, 0, sizeof(p));
    p.m_rows = (int)L.rows_cap; p.n_cols = a.dim; p.k_len = a.dim; p.bn = bn;
    p.a_mn = 0; p.b_mn = 1; p.elem_bytes = 2; p.passes = 1;
    p.tile_tab = pl.tile_tab; p.n_tiles_dev = pl.n_tiles; p.tile_cap = L.tile_cap;
    p.row_dst = dst; p.rel_vec = a.rel; p.rel_is_bf16 = 1;
    if (mode != 1) {
        p.ep = EP_NORM; p.pos_out = a.pos; p.neg_out = a.negs;
        if ((rc = run_gemm(ma, ma, mb, mb, p, 1, s))) return rc;
        if (mode == 0) return 0;
        const long long nneg = a.batch * (long long)a.n_neg;
        if ((rc = launch_logistic_loss(a.pos, a.batch, a.negs, nneg, neg_w, const_cast<float*>(a.dpos), const_cast<float*>(a.dneg), loss,
                                       w + L.off_loss, 4096, s))) return rc;
        transr_coef_kernel<<<(unsigned)((L.tile_cap * UM_BM + 255) / 256), 256, 0, s>>>(a, dst, pl.n_tiles, coef, trow0);
        KGE_LAUNCH_CHECK("transr_coef_kernel");
    }
    p.ep = EP_GV; p.coef = coef; p.gv_out = gv;
    if ((rc = run_gemm(ma, ma, mb, mb, p, 1, s))) return rc;
    // GD = GV . P[r]^T: A = GV rows (K-major over j), B[n = i'][k = j] = P[r][i'][j] (K-major as stored); rows scatter to slots
    CUtensorMap mg, mp;
    if ((rc = make_tensor_map_3d(&mg, gv, 2, 1, L.rows_cap, a.dim, lda, lda * L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mp, a.rel2, 2, n_rel, a.dim, a.dim, lda, lda * a.dim, bn, 64))) return rc;
    p.b_mn = 0; p.ep = EP_SCATTER; p.neg_out = a.g_neg; p.pos_out = gd0; p.sc_n_neg = a.n_neg > 0 ? a.n_neg : 1; p.sc_n_neg_head = a.n_neg_head;
    if ((rc = run_gemm(mg, mg, mp, mp, p, 1, s))) return rc;
    // dP[g] = sum over the group's rows of diff^T (x) GV: both operands MN-major, K runs over the (zero-padded) rows
    CUtensorMap md, mv;
    if ((rc = make_tensor_map_3d(&md, rows, 2, 1, L.rows_cap, a.dim, lda, lda * L.rows_cap, 64, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mv, gv, 2, 1, L.rows_cap, a.dim, lda, lda * L.rows_cap, 64, 64))) return rc;
    GemmTc q;
    memset(&q, 0, sizeof(q));
    q.m_rows = a.dim; q.n_cols = a.dim; q.k_len = UM_BM; q.bn = bn; q.a_mn = 1; q.b_mn = 1; q.elem_bytes = 2; q.passes = 1;
    q.tile_tab = pl.tile_tab2; q.n_tiles_dev = pl.n_tiles2; q.tile_cap = L.gmax * L.tiles_m2; q.group_k = 1;
    q.ep = EP_STORE; q.out = dproj; q.out_ld = a.dim; q.out_batch_rows = a.dim;
    if ((rc = run_gemm(md, md, mv, mv, q, 1, s))) return rc;
    const int wpb = 8;
    transr_reduce_tc_kernel<<<(unsigned)((a.batch + wpb - 1) / wpb), wpb * 32, 0, s>>>(a, gv, gd0, trow0);
    KGE_LAUNCH_CHECK("transr_reduce_tc_kernel");
    return 0;
}

// One warp, one barrier that nobody completes: the bounded wait runs out after `polls` polls and the kernel leaves normally.
__global__ void wait_timeout_selftest_kernel(int polls, int32_t* err) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { umma::mbar_init(&bar, 1); umma::fence_barrier_init(); }
    __syncwarp();
    if (threadIdx.x == 0 && !umma::mbar_wait(&bar, 0, (uint32_t)polls)) atomicOr(err, KGE_ERR_WAIT_TIMEOUT);
}
int launch_wait_timeout_selftest(int polls, cudaStream_t s) {
    int32_t* err = device_error_word();
    if (!err) { set_error("no device error word"); return KGE_E_DEVICE; }
    wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(polls, err);
    KGE_LAUNCH_CHECK("wait_timeout_selftest_kernel");
    return 0;
}

int launch_transr_forward_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                             const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes, cudaStream_t s) {
    return transr_tc(a, 0, 0.f, nullptr, nullptr, rel_perm, rel_seg, rel_uniq, n_groups, n_rel, ws, ws_bytes, s);
}
int launch_transr_backward_tc(const ScoreArgs& a, float* dproj, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                              const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes, cudaStream_t s) {
    return transr_tc(a, 1, 0.f, nullptr, dproj, rel_perm, rel_seg, rel_uniq, n_groups, n_rel, ws, ws_bytes, s);
}
// Forward, logistic loss and backward of TransR over bf16 tables with ONE pack of the difference rows: a.pos (batch) and
// loss (1,) are written, gradients as in launch_transr_backward_tc.  ws: tc_transr_workspace_bytes(..., 2).
int launch_transr_loss_backward_tc(const ScoreArgs& a, float neg_w, float* loss, float* dproj, const int* rel_perm, const int* rel_seg,
                                   const long long* rel_uniq, const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes,
                                   cudaStream_t s) {
    return transr_tc(a, 2, neg_w, loss, dproj, rel_perm, rel_seg, rel_uniq, n_groups, n_rel, ws, ws_bytes, s);
}

// ---- RESCAL projections on the tensor cores (fp32 tables: bf16 operand split; bf16 tables: one pass) ---------------------
// anchors[i] = E[h_i] . P[r_i], g_head[i] = ga[i] . P[r_i]^T and dP[g] = sum over the group of E[h]^T (x) ga are the same
// relation-grouped products as TransR's, over fp32 tables: rows and the matrices of the relations that occur in the batch
// are split into bf16 pairs (v ~ hi + lo) by two pack kernels, and umma_gemm_kernel<G_GROUPED> runs them with three MMAs per
// k-step.  A group of ~33 rows fills a quarter of a 128-row tile, but the tensor pipe has the room (the products are bound by
// reading the matrices): what counts is that a matrix is read from HBM once, split once, and then read by TMA.  Over bf16
// tables nothing is split: rows are copied, P[r] is read by TMA straight from the table, gradient rows are rounded to bf16
// (the 2e-2 tolerance of bf16 tables), one MMA per k-step.
struct RescalTcLayout { size_t off_xhi, off_xlo, off_phi, off_plo, off_dst, off_tab, off_nt, off_tab2, off_ghi, off_glo, total;
                        long long rows_cap, tile_cap, gmax; int tiles_m2; };
static RescalTcLayout rescal_tc_layout(long long batch, int dim, long long n_rel, bool backward) {
    RescalTcLayout L;
    L.gmax = n_rel < batch ? n_rel : batch;
    L.rows_cap = batch + L.gmax * UM_BM;
    L.tile_cap = L.rows_cap / UM_BM + 1;
    L.tiles_m2 = (dim + UM_BM - 1) / UM_BM;
    size_t o = 0;
    L.off_xhi = o; o += al256((size_t)L.rows_cap * dim * 2);
    L.off_xlo = o; o += al256((size_t)L.rows_cap * dim * 2);
    L.off_phi = o; o += al256((size_t)L.gmax * dim * dim * 2);
    L.off_plo = o; o += al256((size_t)L.gmax * dim * dim * 2);
    L.off_dst = o; o += al256((size_t)L.rows_cap * 8);
    L.off_tab = o; o += al256((size_t)L.tile_cap * 16);
    L.off_nt = o; o += 256;
    L.off_tab2 = o; o += backward ? al256((size_t)L.gmax * L.tiles_m2 * 16) : 0;
    L.off_ghi = o; o += backward ? al256((size_t)L.rows_cap * dim * 2) : 0;
    L.off_glo = o; o += backward ? al256((size_t)L.rows_cap * dim * 2) : 0;
    L.total = o;
    return L;
}
size_t tc_rescal_workspace_bytes(long long batch, int dim, long long n_rel, int backward) {
    return rescal_tc_layout(batch, dim, n_rel, backward != 0).total;
}

// One CTA per tile (8 warps x 16 rows): the group's rows as bf16 pairs.  SRC 0: entity rows E[h] (fp32), 1: fp32 rows
// `frows` in triple order.  row_dst (if given): -2 - triple for the valid rows (the scatter epilogue's "positive" slot:
// output row = triple), -1 for padding.
// lo == NULL (bf16 tables): one bf16 term per element - entity rows are copied, fp32 rows rounded.
template <typename T, typename I, int SRC>
__global__ void __launch_bounds__(256) rescal_pack_rows_kernel(ScoreArgs a, TransRPlan pl, const float* frows, __nv_bfloat16* hi,
                                                               __nv_bfloat16* lo, long long* row_dst) {
    const long long tile = blockIdx.x;
    if (tile >= *pl.n_tiles) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int4 tt = pl.tile_tab[tile];
    const int g = tt.z, valid = tt.w;
    long long t0 = tile;
    while (t0 > 0 && pl.tile_tab[t0 - 1].z == g) --t0;              // the group's first tile (a group has few tiles)
    const long long first = (long long)tt.x - pl.tile_tab[t0].x;    // group-local index of this tile's first row
    const int dim = a.dim;
    for (int rr = warp; rr < UM_BM; rr += 8) {
        const long long prow = (long long)tt.x + rr;
        __nv_bfloat16* oh = hi + prow * dim;
        __nv_bfloat16* ol = lo + prow * dim;
        if (rr >= valid) {
            for (int k = lane * 4; k < dim; k += 128) {
                *reinterpret_cast<uint2*>(oh + k) = make_uint2(0u, 0u);
                if (lo) *reinterpret_cast<uint2*>(ol + k) = make_uint2(0u, 0u);
            }
            if (row_dst && lane == 0) row_dst[prow] = -1;
            continue;
        }
        const int tri = pl.rel_perm[pl.rel_seg[g] + (int)(first + rr)];
        for (int k = lane * 4; k < dim; k += 128) {
            float4 v;
            if (SRC == 0) v = ldg4(reinterpret_cast<const T*>(a.ent) + load_id<I>(a.h, tri) * dim + k);
            else v = __ldg(reinterpret_cast<const float4*>(frows + (long long)tri * dim + k));
            if (lo) put_quad(oh + k, ol + k, nullptr, v);
            else { float4 back; *reinterpret_cast<uint2*>(oh + k) = bf16x4(v, back); }
        }
        if (row_dst && lane == 0) row_dst[prow] = -2 - (long long)tri;
    }
}

// P[rel_uniq[g]] (dim x dim fp32) -> bf16 pairs at packed matrix g, for g < n_groups.  grid (blocks per matrix, gmax).
__global__ void __launch_bounds__(256) rescal_pack_p_kernel(const float* proj, const long long* rel_uniq, const long long* n_groups,
                                                            int dim, __nv_bfloat16* hi, __nv_bfloat16* lo) {
    const long long g = blockIdx.y;
    if (g >= *n_groups) return;
    const long long quads = (long long)dim * dim / 4;
    const float4* src = reinterpret_cast<const float4*>(proj + rel_uniq[g] * (long long)dim * dim);
    __nv_bfloat16* oh = hi + g * (long long)dim * dim;
    __nv_bfloat16* ol = lo + g * (long long)dim * dim;
    for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += (long long)gridDim.x * blockDim.x)
        put_quad(oh + 4 * q, ol + 4 * q, nullptr, __ldg(src + q));
}

struct RescalTc {
    RescalTcLayout L; TransRPlan pl; char* w;
    __nv_bfloat16 *xhi, *xlo, *phi, *plo, *ghi, *glo; long long* dst;
    bool single;               // bf16 tables: one term per operand, the matrices read straight from the table
    long long p_batch;         // matrices behind phi / plo: the batch's groups (packed) or all relations (the table)
    int passes;
};

// Plan (tile list), X rows and the batch's matrices as bf16 pairs.  a: fp32 tables, dim % 8 == 0, dim <= 256.
// launch == false: the workspace already holds all of that from an earlier call with the same arguments on this stream
// (the anchors of a backward call): only the pointers are rebuilt.
static int rescal_tc_prepare(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                             const long long* n_groups, long long n_rel, bool backward, void* ws, size_t ws_bytes, RescalTc& r,
                             cudaStream_t s, bool launch = true) {
    r.L = rescal_tc_layout(a.batch, a.dim, n_rel, backward);
    const RescalTcLayout& L = r.L;
    if (ws_bytes < L.total) { set_error("RESCAL tensor-core workspace: need %zu bytes, got %zu", L.total, ws_bytes); return KGE_E_WORKSPACE; }
    char* w = r.w = static_cast<char*>(ws);
    r.xhi = reinterpret_cast<__nv_bfloat16*>(w + L.off_xhi); r.xlo = reinterpret_cast<__nv_bfloat16*>(w + L.off_xlo);
    r.phi = reinterpret_cast<__nv_bfloat16*>(w + L.off_phi); r.plo = reinterpret_cast<__nv_bfloat16*>(w + L.off_plo);
    r.ghi = backward ? reinterpret_cast<__nv_bfloat16*>(w + L.off_ghi) : nullptr;
    r.glo = backward ? reinterpret_cast<__nv_bfloat16*>(w + L.off_glo) : nullptr;
    r.dst = reinterpret_cast<long long*>(w + L.off_dst);
    r.single = a.dtype == KGE_BF16;
    r.passes = r.single ? 1 : 3;
    r.p_batch = r.single ? n_rel : L.gmax;
    if (r.single) {            // every "lo" aliases its "hi": run_gemm reads one map per operand in a single pass
        r.xlo = r.xhi; r.glo = r.ghi;
        r.phi = r.plo = const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(a.rel2));
    }
    TransRPlan& pl = r.pl;
    pl.rel_perm = rel_perm; pl.rel_seg = rel_seg; pl.rel_uniq = rel_uniq; pl.n_groups = n_groups; pl.per = 1;
    pl.tile_tab = reinterpret_cast<int4*>(w + L.off_tab); pl.n_tiles = reinterpret_cast<long long*>(w + L.off_nt);
    pl.tile_cap = L.tile_cap;
    pl.tile_tab2 = backward ? reinterpret_cast<int4*>(w + L.off_tab2) : nullptr;
    pl.n_tiles2 = pl.n_tiles + 1; pl.tiles_m2 = L.tiles_m2; pl.z_is_group = r.single ? 0 : 1;
    if (!launch) return 0;
    transr_plan_kernel<<<1, 1024, 0, s>>>(pl);
    KGE_LAUNCH_CHECK("transr_plan_kernel");
    const unsigned blocks = (unsigned)L.tile_cap;
    __nv_bfloat16* xlo = r.single ? nullptr : r.xlo;
    if (r.single) {
        if (a.id_bits == 64) rescal_pack_rows_kernel<__nv_bfloat16, int64_t, 0><<<blocks, 256, 0, s>>>(a, pl, nullptr, r.xhi, xlo, r.dst);
        else rescal_pack_rows_kernel<__nv_bfloat16, int32_t, 0><<<blocks, 256, 0, s>>>(a, pl, nullptr, r.xhi, xlo, r.dst);
    } else {
        if (a.id_bits == 64) rescal_pack_rows_kernel<float, int64_t, 0><<<blocks, 256, 0, s>>>(a, pl, nullptr, r.xhi, xlo, r.dst);
        else rescal_pack_rows_kernel<float, int32_t, 0><<<blocks, 256, 0, s>>>(a, pl, nullptr, r.xhi, xlo, r.dst);
    }
    KGE_LAUNCH_CHECK("rescal_pack_rows_kernel");
    if (r.single) return 0;
    const unsigned per_matrix = (unsigned)(((long long)a.dim * a.dim / 4 + 1023) / 1024);
    rescal_pack_p_kernel<<<dim3(per_matrix, (unsigned)L.gmax), 256, 0, s>>>(reinterpret_cast<const float*>(a.rel2), rel_uniq, n_groups, a.dim,
                                                                          r.phi, r.plo);
    KGE_LAUNCH_CHECK("rescal_pack_p_kernel");
    return 0;
}

static void rescal_tc_params(GemmTc& p, const ScoreArgs& a, const RescalTc& r) {
    memset(&p, 0, sizeof(p));
    p.m_rows = (int)r.L.rows_cap; p.n_cols = a.dim; p.k_len = a.dim; p.bn = (a.dim + 15) / 16 * 16;
    p.elem_bytes = 2; p.passes = r.passes;
    p.tile_tab = r.pl.tile_tab; p.n_tiles_dev = r.pl.n_tiles; p.tile_cap = r.L.tile_cap;
    p.row_dst = r.dst; p.ep = EP_SCATTER; p.sc_n_neg = 1;
}

// anchors (batch, dim) fp32 in triple order.  ws: tc_rescal_workspace_bytes(batch, dim, n_rel, backward); with backward != 0 the
// workspace is laid out (and the tile lists built) for a launch_rescal_backward_tc(..., prepared = true) that follows.
int launch_rescal_anchors_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                             const long long* n_groups, long long n_rel, float* anchors, int backward, void* ws, size_t ws_bytes,
                             cudaStream_t s) {
    if (a.batch <= 0) return 0;
    RescalTc r;
    int rc = rescal_tc_prepare(a, rel_perm, rel_seg, rel_uniq, n_groups, n_rel, backward != 0, ws, ws_bytes, r, s);
    if (rc) return rc;
    const uint64_t lda = (uint64_t)a.dim * 2;
    CUtensorMap mah, mal, mbh, mbl;
    // Y = X . P[g]: A = packed rows (K-major), B = packed matrix of the group as stored (MN-major: out[j] = sum_i x[i] P[i][j])
    if ((rc = make_tensor_map_3d(&mah, r.xhi, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mal, r.xlo, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mbh, r.phi, 2, r.p_batch, a.dim, a.dim, lda, lda * a.dim, 64, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mbl, r.plo, 2, r.p_batch, a.dim, a.dim, lda, lda * a.dim, 64, 64))) return rc;
    GemmTc p;
    rescal_tc_params(p, a, r);
    p.a_mn = 0; p.b_mn = 1;
    p.pos_out = anchors; p.neg_out = anchors;
    return run_gemm(mah, mal, mbh, mbl, p, 1, s);
}

// g_head[i] = ga[i] . P[r_i]^T (rows of g_head in triple order) and dproj[g] = sum over group g of E[h]^T (x) ga.
// ws: tc_rescal_workspace_bytes(batch, dim, n_rel, 1); prepared: see launch_rescal_anchors_tc.
int launch_rescal_backward_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                              const long long* n_groups, long long n_rel, const float* ga, float* g_head, float* dproj,
                              bool prepared, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (a.batch <= 0) return 0;
    RescalTc r;
    int rc = rescal_tc_prepare(a, rel_perm, rel_seg, rel_uniq, n_groups, n_rel, true, ws, ws_bytes, r, s, !prepared);
    if (rc) return rc;
    const unsigned blocks = (unsigned)r.L.tile_cap;
    // (the source type of the SRC = 1 form is fp32 whatever the tables are)
    if (a.id_bits == 64) rescal_pack_rows_kernel<float, int64_t, 1><<<blocks, 256, 0, s>>>(a, r.pl, ga, r.ghi, r.single ? nullptr : r.glo, nullptr);
    else rescal_pack_rows_kernel<float, int32_t, 1><<<blocks, 256, 0, s>>>(a, r.pl, ga, r.ghi, r.single ? nullptr : r.glo, nullptr);
    KGE_LAUNCH_CHECK("rescal_pack_rows_kernel(ga)");
    const uint64_t lda = (uint64_t)a.dim * 2;
    const int bn = (a.dim + 15) / 16 * 16;
    CUtensorMap mgh, mgl, mph, mpl;
    // GH = GA . P[g]^T: A = packed gradient rows (K-major over j), B[n = i][k = j] = P[g][i][j] (K-major as stored)
    if ((rc = make_tensor_map_3d(&mgh, r.ghi, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mgl, r.glo, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, UM_BM, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mph, r.phi, 2, r.p_batch, a.dim, a.dim, lda, lda * a.dim, bn, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mpl, r.plo, 2, r.p_batch, a.dim, a.dim, lda, lda * a.dim, bn, 64))) return rc;
    GemmTc p;
    rescal_tc_params(p, a, r);
    p.a_mn = 0; p.b_mn = 0;
    p.pos_out = g_head; p.neg_out = g_head;
    if ((rc = run_gemm(mgh, mgl, mph, mpl, p, 1, s))) return rc;
    // dP[g] = X^T . GA over the group's (zero-padded) rows: both operands MN-major, K runs over the rows
    CUtensorMap mxh, mxl, mvh, mvl;
    if ((rc = make_tensor_map_3d(&mxh, r.xhi, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, 64, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mxl, r.xlo, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, 64, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mvh, r.ghi, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, 64, 64))) return rc;
    if ((rc = make_tensor_map_3d(&mvl, r.glo, 2, 1, r.L.rows_cap, a.dim, lda, lda * r.L.rows_cap, 64, 64))) return rc;
    GemmTc q;
    memset(&q, 0, sizeof(q));
    q.m_rows = a.dim; q.n_cols = a.dim; q.k_len = UM_BM; q.bn = bn; q.a_mn = 1; q.b_mn = 1; q.elem_bytes = 2; q.passes = r.passes;
    q.tile_tab = r.pl.tile_tab2; q.n_tiles_dev = r.pl.n_tiles2; q.tile_cap = r.L.gmax * r.L.tiles_m2; q.group_k = 1;
    q.ep = EP_STORE; q.out = dproj; q.out_ld = a.dim; q.out_batch_rows = a.dim;
    return run_gemm(mxh, mxl, mvh, mvl, q, 1, s);
}

}  // namespace kge
