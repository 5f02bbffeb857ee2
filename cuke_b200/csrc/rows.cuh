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
#pragma unroll
    for (int q = 0; q < NV; ++q) {
        float4 o = load_quad<float, VEC>(row, lane + 32 * q, dim);   // own row, written earlier by this warp
        store_quad<VEC>(row, lane + 32 * q, dim, o + x.v[q]);
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
