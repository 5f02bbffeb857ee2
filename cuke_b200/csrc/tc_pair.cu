// Tensor-core path of the chunk-shared scorers (fp32 tables, "3xTF32"): per chunk the score matrix is the
// contraction  S[i][j] = sum_k a_i[k] x_j[k]  (DistMult / ComplEx / RESCAL anchors against the chunk's negative rows),
// which runs on the 5th-generation tensor cores:
//
//   pack kernels   a_i (anchor, computed from the gathered h/t and r rows) and x_j (gathered negative rows) are
//                  written once as dense K-major matrices split into hi = top 19 bits (exactly representable in
//                  tf32) and lo = tf32(a - hi); also |a_i|^2 and |x_j|^2 for the distance form.
//   umma kernel    per 128 x 128 output tile: TMA (128-byte swizzle) feeds a 3-stage shared-memory ring, one
//                  elected thread issues tcgen05.mma kind::tf32 for hi*hi + hi*lo + lo*hi into one fp32
//                  accumulator in tensor memory, four epilogue warps read it back with tcgen05.ld and store.
//   The split makes the products exact to ~2^-20 relative, inside the 1e-4 tolerance of the fp32 path
//   (a single tf32 pass, 2^-11, would not be).
//
// Replaces the scalar-FMA inner loops that cuke generates for bvv over gathered rows
// (apps/kge/kge.py:13-15, pycuke1/codegen/gpu.py:43-51).
#include "rows.cuh"
#include "umma.cuh"

namespace kge {

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

int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return KGE_E_DEVICE; }
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return KGE_E_DEVICE; }
    return 0;
}

// ---- pack kernels --------------------------------------------------------------------------------------------
__device__ __forceinline__ float tf32_trunc(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }
__device__ __forceinline__ void split4(float4 v, float4& hi, float4& lo) {
    hi = make_float4(tf32_trunc(v.x), tf32_trunc(v.y), tf32_trunc(v.z), tf32_trunc(v.w));
    lo = make_float4(tf32_trunc(v.x - hi.x), tf32_trunc(v.y - hi.y), tf32_trunc(v.z - hi.z), tf32_trunc(v.w - hi.w));
}

// Rows [0, n_a): anchors of the triples; rows [n_a, n_a + n_x): the negative rows, in id-list order.
// One warp per row; hi / lo are (n_a + n_x, dim) fp32, sq (n_a + n_x) the squared norms of the unsplit rows.
template <int MODEL, typename T, typename I, int NV>
__global__ void __launch_bounds__(256) tc_pack_kernel(ScoreArgs a, int head, long long n_a, long long n_x,
                                                      float* hi, float* lo, float* sq) {
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
    Row<NV> h, l;
#pragma unroll
    for (int q = 0; q < NV; ++q) { s = dot4(v.v[q], v.v[q], s); split4(v.v[q], h.v[q], l.v[q]); }
    store_row<NV, true>(hi + row * dim, h, dim, lane);
    store_row<NV, true>(lo + row * dim, l, dim, lane);
    s = warp_sum(s);
    if (lane == 0 && sq) sq[row] = s;
}

// ---- the tensor-core tile kernel -------------------------------------------------------------------------------
constexpr int UM_BM = 128, UM_BN = 128, UM_BK = 32;         // 32 fp32 = one 128-byte swizzle row
constexpr int UM_STAGES = 3;
constexpr int UM_TILE_BYTES = UM_BM * UM_BK * 4;             // 16 KiB per operand tile
constexpr int UM_STAGE_BYTES = 4 * UM_TILE_BYTES;            // A_hi, A_lo, B_hi, B_lo
constexpr int UM_SMEM_BYTES = UM_STAGES * UM_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

struct UmmaParams {
    int rows_a;            // rows of A per batch (chunk)
    int rows_b;            // rows of B per batch (n_neg)
    int k;                 // reduction length (dim)
    float* out;            // (batch, rows_a, rows_b)
    const float* sq_a;     // squared norms, distance form only
    const float* sq_b;
    int dist;              // 0: out = acc;  1: out = -sqrt(max(sq_a + sq_b - 2 acc, 0))
    int32_t* err;          // device error word
};

__global__ void __launch_bounds__(192, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo, UmmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + UM_STAGES * UM_STAGE_BYTES);
    uint64_t* empty = full + UM_STAGES;
    uint64_t* acc_ready = empty + UM_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * UM_BN, m0 = blockIdx.y * UM_BM, b = blockIdx.z;
    const int num_kb = (p.k + UM_BK - 1) / UM_BK;
    const int row_a0 = b * p.rows_a + m0;        // first row of this tile in the flattened (batch * rows) operand
    const int row_b0 = b * p.rows_b + n0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < UM_STAGES; ++s) { umma::mbar_init(&full[s], 1); umma::mbar_init(&empty[s], 1); }
        umma::mbar_init(acc_ready, 1);
        umma::fence_barrier_init();
    }
    if (warp == 1) { umma::tmem_alloc(tmem_slot, UM_BN); umma::tmem_relinquish(); }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------------------------------------
        if (lane == 0) {
            umma::prefetch_tensormap(&map_a_hi); umma::prefetch_tensormap(&map_a_lo);
            umma::prefetch_tensormap(&map_b_hi); umma::prefetch_tensormap(&map_b_lo);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % UM_STAGES;
                const uint32_t ph = (kb / UM_STAGES) & 1;
                if (!umma::mbar_wait(&empty[s], ph ^ 1)) { atomicOr(p.err, 2); break; }
                uint8_t* st = smem + s * UM_STAGE_BYTES;
                umma::mbar_expect_tx(&full[s], UM_STAGE_BYTES);
                umma::tma_load_2d(st + 0 * UM_TILE_BYTES, &map_a_hi, kb * UM_BK, row_a0, &full[s]);
                umma::tma_load_2d(st + 1 * UM_TILE_BYTES, &map_a_lo, kb * UM_BK, row_a0, &full[s]);
                umma::tma_load_2d(st + 2 * UM_TILE_BYTES, &map_b_hi, kb * UM_BK, row_b0, &full[s]);
                umma::tma_load_2d(st + 3 * UM_TILE_BYTES, &map_b_lo, kb * UM_BK, row_b0, &full[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma::instr_desc(2 /* tf32 */, UM_BM, UM_BN);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % UM_STAGES;
                const uint32_t ph = (kb / UM_STAGES) & 1;
                if (!umma::mbar_wait(&full[s], ph)) { atomicOr(p.err, 2); ok = false; break; }
                umma::tc_fence_after();
                const uint32_t st = umma::smem_u32(smem + s * UM_STAGE_BYTES);
                const uint64_t a_hi = umma::smem_desc_k_sw128(st + 0 * UM_TILE_BYTES);
                const uint64_t a_lo = umma::smem_desc_k_sw128(st + 1 * UM_TILE_BYTES);
                const uint64_t b_hi = umma::smem_desc_k_sw128(st + 2 * UM_TILE_BYTES);
                const uint64_t b_lo = umma::smem_desc_k_sw128(st + 3 * UM_TILE_BYTES);
#pragma unroll
                for (int k8 = 0; k8 < UM_BK / 8; ++k8) {
                    const uint64_t adv = static_cast<uint64_t>((k8 * 8 * 4) >> 4);   // 32 bytes per K=8 step, in 16-byte units
                    umma::mma_tf32(tmem_base, a_lo + adv, b_hi + adv, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);   // small terms first
                    umma::mma_tf32(tmem_base, a_hi + adv, b_lo + adv, idesc, 1u);
                    umma::mma_tf32(tmem_base, a_hi + adv, b_hi + adv, idesc, 1u);
                }
                umma::mma_commit(&empty[s]);          // frees the stage once these MMAs have read it
            }
            umma::mma_commit(acc_ready);              // accumulator complete (or abandoned)
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lane quarters (warp % 4) ----------------------------------------------------
        const int q = warp & 3;
        const int row = q * 32 + lane;                 // row of the tile held by this thread
        const bool ok = umma::mbar_wait(acc_ready, 0);
        if (!ok && lane == 0) atomicOr(p.err, 2);
        umma::tc_fence_after();
        const int m = m0 + row;
        const bool row_ok = ok && (m < p.rows_a);
        float* orow = p.out + (static_cast<long long>(b) * p.rows_a + m) * p.rows_b + n0;
        const float sa = (p.dist && row_ok) ? p.sq_a[static_cast<long long>(b) * p.rows_a + m] : 0.f;
#pragma unroll 1
        for (int c = 0; c < UM_BN / 32; ++c) {
            float v[32];
            umma::tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c * 32, v);   // warp-collective
            if (!row_ok) continue;
            const int nbase = n0 + c * 32;
            if (p.dist) {
                const float* sb = p.sq_b + static_cast<long long>(b) * p.rows_b + nbase;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float nb = (nbase + j < p.rows_b) ? sb[j] : 0.f;
                    v[j] = -sqrtf(fmaxf(fmaf(-2.f, v[j], sa + nb), 0.f));
                }
            }
            if (nbase + 32 <= p.rows_b && (p.rows_b & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(orow + c * 32 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (nbase + j < p.rows_b) orow[c * 32 + j] = v[j];
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1) { umma::tc_fence_after(); umma::tmem_dealloc(tmem_base, UM_BN); }
}

// ---- host launcher ---------------------------------------------------------------------------------------------------
size_t tc_pair_workspace_bytes(long long n_a, long long n_x, int dim) {
    const size_t rows = static_cast<size_t>(n_a + n_x);
    return 2 * ((rows * dim * 4 + 255) / 256 * 256) + (rows * 4 + 255) / 256 * 256;
}

template <int MODEL, typename T, typename I>
static int tc_pack_go(const ScoreArgs& a, int head, long long n_a, long long n_x, float* hi, float* lo, float* sq, cudaStream_t s) {
    const int nv = quads_per_lane(a.dim);
    const int wpb = 8;
    const unsigned blocks = (unsigned)((n_a + n_x + wpb - 1) / wpb);
    switch (nv) {
        case 1: tc_pack_kernel<MODEL, T, I, 1><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, hi, lo, sq); break;
        case 2: tc_pack_kernel<MODEL, T, I, 2><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, hi, lo, sq); break;
        case 4: tc_pack_kernel<MODEL, T, I, 4><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, hi, lo, sq); break;
        case 8: tc_pack_kernel<MODEL, T, I, 8><<<blocks, wpb * 32, 0, s>>>(a, head, n_a, n_x, hi, lo, sq); break;
        default: set_error("dim %d > 1024 is not supported", a.dim); return KGE_E_UNSUPPORTED;
    }
    KGE_LAUNCH_CHECK("tc_pack_kernel");
    return 0;
}
template <int MODEL>
static int tc_pack_types(const ScoreArgs& a, int head, long long n_a, long long n_x, float* hi, float* lo, float* sq, cudaStream_t s) {
    if (a.dtype == KGE_F32)
        return a.id_bits == 64 ? tc_pack_go<MODEL, float, int64_t>(a, head, n_a, n_x, hi, lo, sq, s)
                               : tc_pack_go<MODEL, float, int32_t>(a, head, n_a, n_x, hi, lo, sq, s);
    return a.id_bits == 64 ? tc_pack_go<MODEL, __nv_bfloat16, int64_t>(a, head, n_a, n_x, hi, lo, sq, s)
                           : tc_pack_go<MODEL, __nv_bfloat16, int32_t>(a, head, n_a, n_x, hi, lo, sq, s);
}

// Forward scores of the chunk's negatives on the tensor cores.  ws: tc_pair_workspace_bytes(batch, n_chunks * n_neg, dim).
int launch_pair_forward_tc(const ScoreArgs& a, int head, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (a.batch <= 0 || a.n_neg <= 0) return 0;
    if (a.dim % 4 != 0) { set_error("the tensor-core path needs dim %% 4 == 0 (16-byte rows), got %d", a.dim); return KGE_E_UNSUPPORTED; }
    const long long n_chunks = a.batch / a.chunk;
    const long long n_a = a.batch, n_x = n_chunks * a.n_neg;
    const size_t need = tc_pair_workspace_bytes(n_a, n_x, a.dim);
    if (ws_bytes < need) { set_error("tensor-core workspace: need %zu bytes, got %zu", need, ws_bytes); return KGE_E_WORKSPACE; }
    const size_t mat = (static_cast<size_t>(n_a + n_x) * a.dim * 4 + 255) / 256 * 256;
    float* hi = static_cast<float*>(ws);
    float* lo = reinterpret_cast<float*>(static_cast<char*>(ws) + mat);
    float* sq = reinterpret_cast<float*>(static_cast<char*>(ws) + 2 * mat);
    int rc;
    switch (a.model) {
        case KGE_TRANSE: rc = tc_pack_types<KGE_TRANSE>(a, head, n_a, n_x, hi, lo, sq, s); break;
        case KGE_DISTMULT: rc = tc_pack_types<KGE_DISTMULT>(a, head, n_a, n_x, hi, lo, sq, s); break;
        case KGE_COMPLEX: rc = tc_pack_types<KGE_COMPLEX>(a, head, n_a, n_x, hi, lo, sq, s); break;
        case KGE_RESCAL: rc = tc_pack_types<KGE_RESCAL>(a, head, n_a, n_x, hi, lo, sq, s); break;
        default: set_error("model %d is not supported with chunk-shared negatives", a.model); return KGE_E_UNSUPPORTED;
    }
    if (rc) return rc;

    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    const uint64_t ld = static_cast<uint64_t>(a.dim) * 4;
    if ((rc = make_tensor_map_2d(&ma_hi, hi, 4, n_a, a.dim, ld, UM_BM, UM_BK))) return rc;
    if ((rc = make_tensor_map_2d(&ma_lo, lo, 4, n_a, a.dim, ld, UM_BM, UM_BK))) return rc;
    if ((rc = make_tensor_map_2d(&mb_hi, hi + n_a * a.dim, 4, n_x, a.dim, ld, UM_BN, UM_BK))) return rc;
    if ((rc = make_tensor_map_2d(&mb_lo, lo + n_a * a.dim, 4, n_x, a.dim, ld, UM_BN, UM_BK))) return rc;

    cudaError_t e = cudaFuncSetAttribute(umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(umma_pair_kernel)");
    UmmaParams p;
    p.rows_a = a.chunk; p.rows_b = a.n_neg; p.k = a.dim; p.out = a.negs;
    p.sq_a = sq; p.sq_b = sq + n_a; p.dist = (a.model == KGE_TRANSE) ? 1 : 0;
    p.err = device_error_word();
    if (!p.err) { set_error("no device error word"); return KGE_E_DEVICE; }
    const dim3 grid((a.n_neg + UM_BN - 1) / UM_BN, (a.chunk + UM_BM - 1) / UM_BM, (unsigned)n_chunks);
    umma_pair_kernel<<<grid, 192, UM_SMEM_BYTES, s>>>(ma_hi, ma_lo, mb_hi, mb_lo, p);
    KGE_LAUNCH_CHECK("umma_pair_kernel");
    return 0;
}

}  // namespace kge
