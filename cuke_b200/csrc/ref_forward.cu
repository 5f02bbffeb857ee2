// Reference-compatible forward: returns exactly what the code cuke generates for the score functions of
// apps/kge/kge.py:273-390 returns from `module.run(*args)` (pycuke1/codegen/gpu_template.cu:8-13):
//   TransE  out[b][:] = E[h]-E[t]+R[r]                                  (batch, dim)   kge.py:293
//   TransH  out[b][:] = E[h]-E[t]+R[r] - (W[r].(E[h]-E[t])) W[r]         (batch, dim)   kge.py:317
//   TransR  out[b][j] = sum_i (E[h][i]-E[t][i]) P[r][i][j] + R[r][j]    (batch, dim)   kge.py:342
//   TransF  out[b] = (E[h]+R[r]).E[t] + (E[t]-R[r]).E[h]                (batch,)       kge.py:363
//   RESCAL  out[b] = sum_j (sum_i E[h][i] P[r][i][j]) E[t][j]           (batch,)       kge.py:389
//   DistMult / ComplEx (not in the reference): the scalar score          (batch,)
// One warp per triple; rows are read with 128-bit loads and never re-read; the relation-matrix models
// stream P[r] once per triple with lanes along the contiguous j index (the reference CPU orientation).
#include "rows.cuh"

namespace kge {

template <int MODEL, typename T, typename I, int NV, bool VEC>
__global__ void __launch_bounds__(256) ref_vec_kernel(const void* ent, const void* rel, const void* rel2,
                                                      const void* hh, const void* rr, const void* tt,
                                                      float* out, long long batch, int dim) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= batch) return;
    const T* E = reinterpret_cast<const T*>(ent);
    const T* R = reinterpret_cast<const T*>(rel);
    const T* W = reinterpret_cast<const T*>(rel2);
    const long long hid = load_id<I>(hh, i), tid = load_id<I>(tt, i), rid = load_id<I>(rr, i);
    Row<NV> h, t, r;
    load_row<T, NV, VEC>(h, E + hid * dim, dim, lane);
    load_row<T, NV, VEC>(t, E + tid * dim, dim, lane);
    load_row<T, NV, VEC>(r, R + rid * dim, dim, lane);
    if (MODEL == KGE_TRANSE) {
#pragma unroll
        for (int q = 0; q < NV; ++q) h.v[q] = (h.v[q] - t.v[q]) + r.v[q];
        store_row<NV, VEC>(out + i * dim, h, dim, lane);
    } else if (MODEL == KGE_TRANSH) {
        Row<NV> w;
        load_row<T, NV, VEC>(w, W + rid * dim, dim, lane);
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { h.v[q] = h.v[q] - t.v[q]; s = dot4(w.v[q], h.v[q], s); }
        s = warp_sum(s);
#pragma unroll
        for (int q = 0; q < NV; ++q) h.v[q] = (h.v[q] + r.v[q]) - s * w.v[q];
        store_row<NV, VEC>(out + i * dim, h, dim, lane);
    } else {
        float s = 0.f;
        if (MODEL == KGE_TRANSF) {
            float s2 = 0.f;
#pragma unroll
            for (int q = 0; q < NV; ++q) { s = dot4(h.v[q] + r.v[q], t.v[q], s); s2 = dot4(t.v[q] - r.v[q], h.v[q], s2); }
            s = warp_sum(s) + warp_sum(s2);
        } else if (MODEL == KGE_DISTMULT) {
#pragma unroll
            for (int q = 0; q < NV; ++q) s = dot4(h.v[q] * r.v[q], t.v[q], s);
            s = warp_sum(s);
        } else {   // ComplEx, interleaved re/im
#pragma unroll
            for (int q = 0; q < NV; ++q) s = dot4(cmul(h.v[q], r.v[q]), t.v[q], s);
            s = warp_sum(s);
        }
        if (lane == 0) out[i] = s;
    }
}

// Relation-matrix models.  The warp parks x = E[h]-E[t] (TransR) or E[h] (RESCAL) in shared memory and
// sweeps P[r] row by row; lane L accumulates output columns L, L+32, ...
template <int MODEL, typename T, typename I, int NJ>
__global__ void __launch_bounds__(256) ref_mat_kernel(const void* ent, const void* rel, const void* proj,
                                                      const void* hh, const void* rr, const void* tt,
                                                      float* out, long long batch, int dim) {
    extern __shared__ float xs[];   // 8 warps x dim
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
    if (i >= batch) return;
    const T* E = reinterpret_cast<const T*>(ent);
    const T* R = reinterpret_cast<const T*>(rel);
    const T* P = reinterpret_cast<const T*>(proj);
    const long long hid = load_id<I>(hh, i), tid = load_id<I>(tt, i), rid = load_id<I>(rr, i);
    float* x = xs + wib * dim;
    for (int k = lane; k < dim; k += 32) {
        float v = ldg1(E + hid * dim + k);
        if (MODEL == KGE_TRANSR) v -= ldg1(E + tid * dim + k);
        x[k] = v;
    }
    __syncwarp();
    float acc[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j] = 0.f;
    const T* M = P + rid * (long long)dim * dim;
    for (int k = 0; k < dim; ++k) {
        const float xk = x[k];
        const T* mrow = M + (long long)k * dim;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int col = lane + 32 * j;
            if (col < dim) acc[j] = fmaf(xk, ldg1(mrow + col), acc[j]);
        }
    }
    if (MODEL == KGE_TRANSR) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int col = lane + 32 * j;
            if (col < dim) out[i * dim + col] = acc[j] + ldg1(R + rid * dim + col);
        }
    } else {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int col = lane + 32 * j;
            if (col < dim) s = fmaf(acc[j], ldg1(E + tid * dim + col), s);
        }
        s = warp_sum(s);
        if (lane == 0) out[i] = s;
    }
}

template <int MODEL, typename T, typename I>
static int ref_go(const kge_problem* p, const kge_tensors* t, float* out, cudaStream_t s) {
    const int wpb = 8;
    const unsigned blocks = (unsigned)((p->batch + wpb - 1) / wpb);
    if (MODEL == KGE_TRANSR || MODEL == KGE_RESCAL) {
        const int nj = (p->dim + 31) / 32;
        const size_t smem = (size_t)wpb * p->dim * sizeof(float);
#define KGE_MAT(N) ref_mat_kernel<MODEL, T, I, N><<<blocks, wpb * 32, smem, s>>>(t->ent, t->rel, t->rel2, t->h, t->r, t->t, out, p->batch, p->dim)
        if (nj <= 4) KGE_MAT(4); else if (nj <= 8) KGE_MAT(8); else if (nj <= 16) KGE_MAT(16); else if (nj <= 32) KGE_MAT(32);
        else { set_error("dim %d > 1024 is not supported", p->dim); return KGE_E_UNSUPPORTED; }
#undef KGE_MAT
        KGE_LAUNCH_CHECK("ref_mat_kernel");
        return 0;
    } else {
        const bool vec = p->dim % 4 == 0;
        const int nv = quads_per_lane(p->dim);
        if (nv == 0) { set_error("dim %d > 1024 is not supported", p->dim); return KGE_E_UNSUPPORTED; }
#define KGE_VEC(N, V) ref_vec_kernel<MODEL, T, I, N, V><<<blocks, wpb * 32, 0, s>>>(t->ent, t->rel, t->rel2, t->h, t->r, t->t, out, p->batch, p->dim)
#define KGE_VEC_CASE(N) case N: if (vec) KGE_VEC(N, true); else KGE_VEC(N, false); break;
        switch (nv) { KGE_VEC_CASE(1) KGE_VEC_CASE(2) KGE_VEC_CASE(4) KGE_VEC_CASE(8) }
#undef KGE_VEC_CASE
#undef KGE_VEC
        KGE_LAUNCH_CHECK("ref_vec_kernel");
        return 0;
    }
}

template <int MODEL>
static int ref_types(const kge_problem* p, const kge_tensors* t, float* out, cudaStream_t s) {
    if (p->dtype == KGE_F32)
        return p->id_bits == 64 ? ref_go<MODEL, float, int64_t>(p, t, out, s) : ref_go<MODEL, float, int32_t>(p, t, out, s);
    return p->id_bits == 64 ? ref_go<MODEL, __nv_bfloat16, int64_t>(p, t, out, s)
                            : ref_go<MODEL, __nv_bfloat16, int32_t>(p, t, out, s);
}

int launch_ref_forward(const kge_problem* p, const kge_tensors* t, float* out, cudaStream_t s) {
    if (p->batch <= 0) return 0;
    switch (p->model) {
        case KGE_TRANSE: return ref_types<KGE_TRANSE>(p, t, out, s);
        case KGE_TRANSH: return ref_types<KGE_TRANSH>(p, t, out, s);
        case KGE_TRANSR: return ref_types<KGE_TRANSR>(p, t, out, s);
        case KGE_TRANSF: return ref_types<KGE_TRANSF>(p, t, out, s);
        case KGE_DISTMULT: return ref_types<KGE_DISTMULT>(p, t, out, s);
        case KGE_RESCAL: return ref_types<KGE_RESCAL>(p, t, out, s);
        case KGE_COMPLEX: return ref_types<KGE_COMPLEX>(p, t, out, s);
        default: break;
    }
    set_error("unknown model %d", p->model);
    return KGE_E_UNSUPPORTED;
}

}  // namespace kge
