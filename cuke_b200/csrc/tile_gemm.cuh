// fp32 CUDA-core tile engine shared by the chunk-shared scorers and the relation-grouped projections.
//
// One CTA of 256 threads produces a 128 x 128 tile of  acc[m][n] = sum_k f(A(m,k), B(k,n))  with
// f = a*b (OP_DOT) or (a-b)^2 (OP_DIST: squared distance for TransE, which cannot go through the
// ||a||^2+||b||^2-2ab GEMM form without losing the 1e-4 tolerance to cancellation).
// Operands are fetched through loader functors, so gathers through id lists (the indirect index
// Eemb[h] of pycuke1/asg.py:154-156) and on-the-fly anchor arithmetic fuse into the operand fetch.
// k advances in steps of 16; the next k-slab is prefetched into registers while the current one is
// consumed from shared memory (double buffered).  Each thread owns an 8 x 8 micro-tile laid out as
// rows {4ty..4ty+3, 64+4ty..} x cols {4tx..4tx+3, 64+4tx..} so that all shared-memory reads are
// conflict-free 128-bit loads and all global stores are 256 B contiguous per half-warp.
#pragma once
#include "common.cuh"

namespace kge {

constexpr int TG_BM = 128, TG_BN = 128, TG_BK = 16, TG_LD = 132;   // LD: padded row length (floats)
enum { OP_DOT = 0, OP_DIST = 1 };

struct TileSmem {
    float A[2][TG_BK][TG_LD];
    float B[2][TG_BK][TG_LD];
};

// Loader concept:
//   static constexpr bool K_CONTIG;
//   K_CONTIG  : float4 get(int row, int k)   -> elements (row, k..k+3)        row in [0,128) of the tile
//   otherwise : float4 get(int row4, int k)  -> elements (row4..row4+3, k)    row4 multiple of 4
//   Out-of-range elements must read as 0.

template <class L>
__device__ __forceinline__ void tg_fetch(const L& l, int k0, int tid, float4 (&reg)[2]) {
    if (L::K_CONTIG) {
        const int kq = (tid & 3) * 4;
        reg[0] = l.get(tid >> 2, k0 + kq);
        reg[1] = l.get(64 + (tid >> 2), k0 + kq);
    } else {
        const int r4 = (tid & 31) * 4;
        reg[0] = l.get(r4, k0 + (tid >> 5));
        reg[1] = l.get(r4, k0 + 8 + (tid >> 5));
    }
}
template <class L>
__device__ __forceinline__ void tg_stash(float (*S)[TG_LD], int tid, const float4 (&reg)[2]) {
    if (L::K_CONTIG) {
        const int kq = (tid & 3) * 4;
        const int r0 = tid >> 2;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int r = r0 + 64 * u;
            S[kq + 0][r] = reg[u].x; S[kq + 1][r] = reg[u].y; S[kq + 2][r] = reg[u].z; S[kq + 3][r] = reg[u].w;
        }
    } else {
        const int r4 = (tid & 31) * 4;
        *reinterpret_cast<float4*>(&S[tid >> 5][r4]) = reg[0];
        *reinterpret_cast<float4*>(&S[8 + (tid >> 5)][r4]) = reg[1];
    }
}

template <int OP, class AL, class BL>
__device__ __forceinline__ void tile_mainloop(const AL& al, const BL& bl, int K, TileSmem& sm, float (&acc)[8][8]) {
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 ra[2], rb[2];
    const int KT = (K + TG_BK - 1) / TG_BK;
    if (KT == 0) return;
    tg_fetch<AL>(al, 0, tid, ra);
    tg_fetch<BL>(bl, 0, tid, rb);
    tg_stash<AL>(sm.A[0], tid, ra);
    tg_stash<BL>(sm.B[0], tid, rb);
    __syncthreads();
    for (int kt = 0; kt < KT; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < KT) {
            tg_fetch<AL>(al, (kt + 1) * TG_BK, tid, ra);
            tg_fetch<BL>(bl, (kt + 1) * TG_BK, tid, rb);
        }
#pragma unroll
        for (int k = 0; k < TG_BK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&sm.A[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&sm.A[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&sm.B[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&sm.B[buf][k][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (OP == OP_DOT) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    else { const float d = av[i] - bv[j]; acc[i][j] = fmaf(d, d, acc[i][j]); }
                }
        }
        if (kt + 1 < KT) {
            tg_stash<AL>(sm.A[buf ^ 1], tid, ra);
            tg_stash<BL>(sm.B[buf ^ 1], tid, rb);
        }
        __syncthreads();
    }
}

// Hands the micro-tile to an epilogue functor:  ep(row, col4, float4 v)  with tile-relative row in
// [0,128) and col4 in {0,4,...,124}; v holds columns col4..col4+3 of that row.
template <class EP>
__device__ __forceinline__ void tile_epilogue(const float (&acc)[8][8], EP& ep) {
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = (i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4);
        ep(row, tx * 4, make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]));
        ep(row, 64 + tx * 4, make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]));
    }
}

}  // namespace kge
