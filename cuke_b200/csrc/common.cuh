// Shared device/host helpers of libkge_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/kge_b200.h"

namespace kge {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// ---- host-side error plumbing -------------------------------------------------------------------
void set_error(const char* fmt, ...);          // thread-local message (capi.cu)
int cuda_status(cudaError_t e, const char* what);  // 0 or positive cudaError_t, records message
int32_t* device_error_word();                  // per-device error word (capi.cu)
void note_launch();                            // counts kernel launches issued by this library (capi.cu)

#define KGE_LAUNCH_CHECK(what)                                   \
    do {                                                         \
        cudaError_t e__ = cudaGetLastError();                    \
        if (e__ != cudaSuccess) return kge::cuda_status(e__, what); \
        kge::note_launch();                                      \
    } while (0)

// ---- element access --------------------------------------------------------------------------------
// A "quad" is 4 consecutive elements of a row; every row-wise kernel gives lane L the quads
// L, L+32, L+64, ... so that a warp reads 512 B (fp32) / 256 B (bf16) contiguous per pass.
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ldg4(const __nv_bfloat16* p) {
    uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&u.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ float ldg1(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldg1(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Loads quad q (elements 4q..4q+3) of a row of `dim` elements; elements >= dim read as 0.
template <typename T, bool VEC>
__device__ __forceinline__ float4 load_quad(const T* row, int q, int dim) {
    if (VEC) {
        return (4 * q < dim) ? ldg4(row + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        int k = 4 * q;
        if (k + 0 < dim) v.x = ldg1(row + k + 0);
        if (k + 1 < dim) v.y = ldg1(row + k + 1);
        if (k + 2 < dim) v.z = ldg1(row + k + 2);
        if (k + 3 < dim) v.w = ldg1(row + k + 3);
        return v;
    }
}
template <bool VEC>
__device__ __forceinline__ void store_quad(float* row, int q, int dim, float4 v) {
    int k = 4 * q;
    if (VEC) {
        if (k < dim) *reinterpret_cast<float4*>(row + k) = v;
    } else {
        if (k + 0 < dim) row[k + 0] = v.x;
        if (k + 1 < dim) row[k + 1] = v.y;
        if (k + 2 < dim) row[k + 2] = v.z;
        if (k + 3 < dim) row[k + 3] = v.w;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// float4 arithmetic
__device__ __forceinline__ float4 f4(float a) { return make_float4(a, a, a, a); }
__device__ __forceinline__ float4 operator+(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 operator-(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 operator*(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 operator*(float s, float4 a) { return make_float4(s * a.x, s * a.y, s * a.z, s * a.w); }
__device__ __forceinline__ float4 fma4(float s, float4 a, float4 c) { return make_float4(fmaf(s, a.x, c.x), fmaf(s, a.y, c.y), fmaf(s, a.z, c.z), fmaf(s, a.w, c.w)); }
__device__ __forceinline__ float4 fma4(float4 a, float4 b, float4 c) { return make_float4(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y), fmaf(a.z, b.z, c.z), fmaf(a.w, b.w, c.w)); }
__device__ __forceinline__ float dot4(float4 a, float4 b, float acc) { return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc)))); }
__device__ __forceinline__ float hsum4(float4 a) { return (a.x + a.y) + (a.z + a.w); }

// Complex products on quads holding two interleaved complex numbers (re0, im0, re1, im1).
__device__ __forceinline__ float4 cmul(float4 a, float4 b) {        // a * b
    return make_float4(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x, a.z * b.z - a.w * b.w, a.z * b.w + a.w * b.z);
}
__device__ __forceinline__ float4 cmul_conj(float4 a, float4 b) {   // a * conj(b)
    return make_float4(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y, a.z * b.z + a.w * b.w, a.w * b.z - a.z * b.w);
}

template <typename I>
__device__ __forceinline__ long long load_id(const void* ids, long long i) {
    return static_cast<long long>(__ldg(reinterpret_cast<const I*>(ids) + i));
}

// Host: dispatch helpers -----------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int quads_per_lane(int dim) {   // NV template value: quads each lane owns
    int q = (dim + 3) / 4;
    int nv = (q + 31) / 32;
    if (nv <= 1) return 1;
    if (nv <= 2) return 2;
    if (nv <= 4) return 4;
    if (nv <= 8) return 8;
    return 0;                          // dim > 1024 unsupported by the row-per-warp kernels
}
inline bool can_vec(int dim, int dtype) { return dtype == KGE_F32 ? (dim % 4 == 0) : (dim % 4 == 0); }

// Entry points implemented across the .cu files (all return kge_status / cudaError_t) ----------------
struct ScoreArgs {
    const void* ent; const void* rel; const void* rel2;
    const void* h; const void* r; const void* t; const void* neg;
    float* pos; float* negs;                 // forward outputs / backward inputs (saved scores)
    const float* dpos; const float* dneg;    // backward
    float* pos_loss;                         // optional (batch): the per-triple backward kernel forms the positive's score
                                             // (-> pos), its logistic loss term (-> pos_loss) and dS itself; dpos is unused
    float* g_head; float* g_tail; float* g_neg; float* g_rel; float* g_rel2;
    const float* ga_tail_init;               // (batch, dim) anchor gradients accumulated elsewhere (chunk-shared)
    const float* ga_head_init;
    const float* ga_init_scale;              // optional (batch): the initial anchor gradient is scale[i] * anchor_i - init_i
    const float* anchors;                    // (batch, dim) precomputed anchors (RESCAL), or NULL
    const unsigned long long* guard;         // if set, pair_fwd_kernel only runs when *guard > guard_cap (tensor-core overflow path)
    unsigned long long guard_cap;
    long long batch; int dim; int n_neg; int n_neg_head; int chunk;
    int model; int dtype; int id_bits;
    int tc_es;                               // tensor-core split of fp32 operands: 2 = bf16 pairs, 4 = tf32 pairs
};

int launch_ref_forward(const kge_problem* p, const kge_tensors* t, float* out, cudaStream_t s);
int launch_triple_forward(const ScoreArgs& a, cudaStream_t s);
int launch_triple_backward(const ScoreArgs& a, cudaStream_t s);
int launch_anchor(const ScoreArgs& a, float* anchors_tail, float* anchors_head, cudaStream_t s);

}  // namespace kge
