// Register-resident embedding rows: lane L of a warp owns quads L, L+32, ... of a row.
#pragma once
#include "common.cuh"

namespace kge {

template <int NV> struct Row { float4 v[NV]; };

template <typename T, int NV, bool VEC>
__device__ __forceinline__ void load_row(Row<NV>& x, const T* row, int dim, int lane) {
#pragma unroll
    for (int q = 0; q < NV; ++q) x.v[q] = load_quad<T, VEC>(row, lane + 32 * q, dim);
}
template <int NV, bool VEC>
__device__ __forceinline__ void load_row_f32(Row<NV>& x, const float* row, int dim, int lane) {
#pragma unroll
    for (int q = 0; q < NV; ++q) x.v[q] = load_quad<float, VEC>(row, lane + 32 * q, dim);
}
template <int NV, bool VEC>
__device__ __forceinline__ void store_row(float* row, const Row<NV>& x, int dim, int lane) {
#pragma unroll
    for (int q = 0; q < NV; ++q) store_quad<VEC>(row, lane + 32 * q, dim, x.v[q]);
}
template <int NV, bool VEC>
__device__ __forceinline__ void add_row(float* row, const Row<NV>& x, int dim, int lane) {
    // read-modify-write of a row this warp wrote earlier in the same kernel: coherent (plain) loads, not the read-only path
#pragma unroll
    for (int q = 0; q < NV; ++q) {
        const int k = 4 * (lane + 32 * q);
        if (VEC) {
            if (k < dim) {
                float4* p = reinterpret_cast<float4*>(row + k);
                *p = *p + x.v[q];
            }
        } else {
            if (k + 0 < dim) row[k + 0] += x.v[q].x;
            if (k + 1 < dim) row[k + 1] += x.v[q].y;
            if (k + 2 < dim) row[k + 2] += x.v[q].z;
            if (k + 3 < dim) row[k + 3] += x.v[q].w;
        }
    }
}
template <int NV> __device__ __forceinline__ float row_dot(const Row<NV>& a, const Row<NV>& b) {
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < NV; ++q) s = dot4(a.v[q], b.v[q], s);
    return warp_sum(s);
}
template <int NV> __device__ __forceinline__ void row_zero(Row<NV>& a) {
#pragma unroll
    for (int q = 0; q < NV; ++q) a.v[q] = f4(0.f);
}

}  // namespace kge
