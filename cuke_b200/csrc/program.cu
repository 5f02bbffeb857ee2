// General fused gather-compute evaluator: runs a small register program over every triple of a batch.
//
// cuke lowers ANY composition of its batched operators (bvv, bsv, bvm, bov, bsm over gathered rows; the cases its
// fusion rule handles are listed in apps/kge/kge.py:36-84) to a generated kernel.  The seven score functions have
// hand-written kernels here; every other expression of the same operators is compiled by the Python front-end
// (cuke_b200/program.py) into a linear program over per-triple vector and scalar registers, and this ONE kernel evaluates
// it: one warp per batch element, vector registers in shared memory (lane L owns elements L, L + 32, ...), scalar
// registers replicated in the lanes' own registers through shared memory, gathers straight from the tables.  No new
// kernel is needed for a new score function; the price is that nothing is specialised (a vector-matrix product is a
// per-triple loop over the relation's matrix, as in the reference's generated code).
#include <string.h>
#include "common.cuh"

namespace kge {

enum {
    PG_GATHER = 0,     // v[dst] = T[a][ ids[b][i] ]                          (a: table, b: id array)
    PG_VADD = 1, PG_VSUB = 2, PG_VMUL = 3, PG_VDIV = 4,   // v[dst] = v[a] (op) v[b]
    PG_SPLAT = 5,      // v[dst][:] = s[a]
    PG_DOT = 6,        // s[dst] = sum_k v[a][k] * v[b][k]
    PG_SADD = 7, PG_SSUB = 8, PG_SMUL = 9, PG_SDIV = 10,  // s[dst] = s[a] (op) s[b]
    PG_SCONST = 11,    // s[dst] = bit pattern a
    PG_VECMAT = 12,    // v[dst][j] = sum_k v[a][k] * M[k][j],  M = T[b][ ids[c][i] ]  (dim x dim)
    PG_COLSUM = 13,    // v[dst][j] = sum_k M[k][j],             M = T[a][ ids[b][i] ]
    PG_MATVEC = 14,    // v[dst][k] = sum_j M[k][j] * v[a][j],   M = T[b][ ids[c][i] ]
    PG_ROW = 15,       // v[dst] = T[a][i]        (a (batch, dim) operand used element by element, no index)
    PG_LOADS = 16      // s[dst] = T[a][i]        (a (batch,) operand)
};
enum { PG_OUT_VECTOR = 0, PG_OUT_SCALAR = 1, PG_OUT_OUTER = 2, PG_OUT_MATRIX = 3 };

constexpr int PG_MAX_OPS = 64, PG_MAX_TABLES = 8, PG_MAX_IDS = 4, PG_MAX_SREG = 16, PG_MAX_VREG = 16;

struct ProgramArgs {
    int n_ops, n_vreg, dim, id_bits;
    int ops[PG_MAX_OPS][5];                 // op, dst, a, b, c
    const float* tables[PG_MAX_TABLES];
    const void* ids[PG_MAX_IDS];
    int out_kind, out_a, out_b, out_s;      // VECTOR: v[out_a]; SCALAR: s[out_a]; OUTER: s[out_s] * v[out_a] (x) v[out_b] (out_s < 0: no
    int out_table, out_ids;                 // scale); MATRIX: s[out_s] * T[out_table][ids[out_ids][i]]
    long long batch;
    float* out;
};

__device__ __forceinline__ long long pg_id(const ProgramArgs& p, int which, long long i) {
    return p.id_bits == 64 ? static_cast<long long>(reinterpret_cast<const long long*>(p.ids[which])[i])
                           : static_cast<long long>(reinterpret_cast<const int*>(p.ids[which])[i]);
}

__global__ void __launch_bounds__(256) program_kernel(const __grid_constant__ ProgramArgs p) {
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const long long i = static_cast<long long>(blockIdx.x) * wpb + w;
    if (i >= p.batch) return;
    const int dim = p.dim;
    float* vr = smem + static_cast<size_t>(w) * p.n_vreg * dim;      // this warp's vector registers
    float sr[PG_MAX_SREG];                                           // scalar registers: the same value in every lane
#pragma unroll
    for (int k = 0; k < PG_MAX_SREG; ++k) sr[k] = 0.f;
    auto sget = [&](int k) {
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < PG_MAX_SREG; ++q) if (q == k) v = sr[q];
        return v;
    };
    auto sset = [&](int k, float v) {
#pragma unroll
        for (int q = 0; q < PG_MAX_SREG; ++q) if (q == k) sr[q] = v;
    };
    for (int pc = 0; pc < p.n_ops; ++pc) {
        const int op = p.ops[pc][0], dst = p.ops[pc][1], a = p.ops[pc][2], b = p.ops[pc][3], c = p.ops[pc][4];
        switch (op) {
            case PG_GATHER: {
                const float* row = p.tables[a] + pg_id(p, b, i) * dim;
                for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = __ldg(row + k);
                break;
            }
            case PG_ROW: {
                const float* row = p.tables[a] + i * dim;
                for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = __ldg(row + k);
                break;
            }
            case PG_LOADS: sset(dst, __ldg(p.tables[a] + i)); break;
            case PG_VADD: for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = vr[a * dim + k] + vr[b * dim + k]; break;
            case PG_VSUB: for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = vr[a * dim + k] - vr[b * dim + k]; break;
            case PG_VMUL: for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = vr[a * dim + k] * vr[b * dim + k]; break;
            case PG_VDIV: for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = vr[a * dim + k] / vr[b * dim + k]; break;
            case PG_SPLAT: { const float s = sget(a); for (int k = lane; k < dim; k += 32) vr[dst * dim + k] = s; break; }
            case PG_DOT: {
                float s = 0.f;
                for (int k = lane; k < dim; k += 32) s = fmaf(vr[a * dim + k], vr[b * dim + k], s);
                sset(dst, warp_sum(s));
                break;
            }
            case PG_SADD: sset(dst, sget(a) + sget(b)); break;
            case PG_SSUB: sset(dst, sget(a) - sget(b)); break;
            case PG_SMUL: sset(dst, sget(a) * sget(b)); break;
            case PG_SDIV: sset(dst, sget(a) / sget(b)); break;
            case PG_SCONST: sset(dst, __int_as_float(a)); break;
            case PG_VECMAT: {         // lane owns output columns j: coalesced rows of M, the vector read as a broadcast
                __syncwarp();
                const float* M = p.tables[b] + pg_id(p, c, i) * static_cast<long long>(dim) * dim;
                for (int j = lane; j < dim; j += 32) {
                    float s = 0.f;
                    for (int k = 0; k < dim; ++k) s = fmaf(vr[a * dim + k], __ldg(M + static_cast<long long>(k) * dim + j), s);
                    vr[dst * dim + j] = s;
                }
                break;
            }
            case PG_COLSUM: {
                const float* M = p.tables[a] + pg_id(p, b, i) * static_cast<long long>(dim) * dim;
                for (int j = lane; j < dim; j += 32) {
                    float s = 0.f;
                    for (int k = 0; k < dim; ++k) s += __ldg(M + static_cast<long long>(k) * dim + j);
                    vr[dst * dim + j] = s;
                }
                break;
            }
            case PG_MATVEC: {         // one output row at a time: lanes stride along the row, then a warp sum
                __syncwarp();
                const float* M = p.tables[b] + pg_id(p, c, i) * static_cast<long long>(dim) * dim;
                for (int k = 0; k < dim; ++k) {
                    float s = 0.f;
                    for (int j = lane; j < dim; j += 32) s = fmaf(__ldg(M + static_cast<long long>(k) * dim + j), vr[a * dim + j], s);
                    s = warp_sum(s);
                    if (lane == 0) vr[dst * dim + k] = s;
                }
                break;
            }
            default: break;
        }
        __syncwarp();                 // a register written by some lanes is read by others in the next instruction
    }
    if (p.out_kind == PG_OUT_VECTOR) {
        for (int k = lane; k < dim; k += 32) p.out[i * dim + k] = vr[p.out_a * dim + k];
    } else if (p.out_kind == PG_OUT_SCALAR) {
        if (lane == 0) p.out[i] = sget(p.out_a);
    } else if (p.out_kind == PG_OUT_OUTER) {
        const float s = p.out_s >= 0 ? sget(p.out_s) : 1.f;
        float* o = p.out + i * static_cast<long long>(dim) * dim;
        for (int r = 0; r < dim; ++r) {
            const float ar = s * vr[p.out_a * dim + r];
            for (int k = lane; k < dim; k += 32) o[static_cast<long long>(r) * dim + k] = ar * vr[p.out_b * dim + k];
        }
    } else {
        const float s = p.out_s >= 0 ? sget(p.out_s) : 1.f;
        const float* M = p.tables[p.out_table] + pg_id(p, p.out_ids, i) * static_cast<long long>(dim) * dim;
        float* o = p.out + i * static_cast<long long>(dim) * dim;
        for (long long k = lane; k < static_cast<long long>(dim) * dim; k += 32) o[k] = s * __ldg(M + k);
    }
}

}  // namespace kge

using namespace kge;

extern "C" int kge_eval_program(const kge_program* prog, int32_t dim, int64_t batch, const float* const* tables, int32_t n_tables,
                                const void* const* ids, int32_t id_bits, int32_t n_ids, float* out, kge_stream_t stream) {
    const char* fn = "kge_eval_program";
    if (!prog) { set_error("%s: program is NULL", fn); return KGE_E_NULL; }
    if (dim <= 0 || dim > 1024 || batch < 0) { set_error("%s: bad sizes", fn); return KGE_E_SHAPE; }
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    if (prog->n_ops < 0 || prog->n_ops > PG_MAX_OPS || prog->n_vreg < 0 || prog->n_vreg > PG_MAX_VREG || prog->n_sreg < 0 ||
        prog->n_sreg > PG_MAX_SREG || n_tables < 0 || n_tables > PG_MAX_TABLES || n_ids < 0 || n_ids > PG_MAX_IDS) {
        set_error("%s: program outside the limits (%d ops, %d vector / %d scalar registers, %d tables, %d id arrays)", fn, PG_MAX_OPS,
                  PG_MAX_VREG, PG_MAX_SREG, PG_MAX_TABLES, PG_MAX_IDS);
        return KGE_E_RANGE;
    }
    if (batch == 0) return 0;
    if (!out) { set_error("%s: out is NULL", fn); return KGE_E_NULL; }
    ProgramArgs a;
    memset(&a, 0, sizeof(a));
    a.n_ops = prog->n_ops; a.n_vreg = prog->n_vreg; a.dim = dim; a.id_bits = id_bits; a.batch = batch; a.out = out;
    for (int t = 0; t < n_tables; ++t) {
        if (!tables || !tables[t]) { set_error("%s: table %d is NULL", fn, t); return KGE_E_NULL; }
        a.tables[t] = tables[t];
    }
    for (int t = 0; t < n_ids; ++t) {
        if (!ids || !ids[t]) { set_error("%s: id array %d is NULL", fn, t); return KGE_E_NULL; }
        a.ids[t] = ids[t];
    }
    auto vreg = [&](int r) { return r >= 0 && r < prog->n_vreg; };
    auto sreg = [&](int r) { return r >= 0 && r < prog->n_sreg; };
    auto tab = [&](int t) { return t >= 0 && t < n_tables; };
    auto idx = [&](int t) { return t >= 0 && t < n_ids; };
    for (int k = 0; k < prog->n_ops; ++k) {
        const int32_t* o = prog->ops[k];
        bool ok = false;
        switch (o[0]) {
            case PG_GATHER: ok = vreg(o[1]) && tab(o[2]) && idx(o[3]); break;
            case PG_VADD: case PG_VSUB: case PG_VMUL: case PG_VDIV: ok = vreg(o[1]) && vreg(o[2]) && vreg(o[3]); break;
            case PG_SPLAT: ok = vreg(o[1]) && sreg(o[2]); break;
            case PG_DOT: ok = sreg(o[1]) && vreg(o[2]) && vreg(o[3]); break;
            case PG_SADD: case PG_SSUB: case PG_SMUL: case PG_SDIV: ok = sreg(o[1]) && sreg(o[2]) && sreg(o[3]); break;
            case PG_SCONST: ok = sreg(o[1]); break;
            case PG_VECMAT: case PG_MATVEC: ok = vreg(o[1]) && vreg(o[2]) && o[1] != o[2] && tab(o[3]) && idx(o[4]); break;
            case PG_COLSUM: ok = vreg(o[1]) && tab(o[2]) && idx(o[3]); break;
            case PG_ROW: ok = vreg(o[1]) && tab(o[2]); break;
            case PG_LOADS: ok = sreg(o[1]) && tab(o[2]); break;
            default: ok = false;
        }
        if (!ok) { set_error("%s: instruction %d (op %d) is malformed", fn, k, o[0]); return KGE_E_UNSUPPORTED; }
        for (int q = 0; q < 5; ++q) a.ops[k][q] = o[q];
    }
    a.out_kind = prog->out_kind; a.out_a = prog->out_a; a.out_b = prog->out_b; a.out_s = prog->out_s;
    a.out_table = prog->out_table; a.out_ids = prog->out_ids;
    bool ok = false;
    switch (prog->out_kind) {
        case PG_OUT_VECTOR: ok = vreg(prog->out_a); break;
        case PG_OUT_SCALAR: ok = sreg(prog->out_a); break;
        case PG_OUT_OUTER: ok = vreg(prog->out_a) && vreg(prog->out_b) && (prog->out_s < 0 || sreg(prog->out_s)); break;
        case PG_OUT_MATRIX: ok = tab(prog->out_table) && idx(prog->out_ids) && (prog->out_s < 0 || sreg(prog->out_s)); break;
        default: ok = false;
    }
    if (!ok) { set_error("%s: the program's result is malformed", fn); return KGE_E_UNSUPPORTED; }
    const size_t per_warp = static_cast<size_t>(prog->n_vreg > 0 ? prog->n_vreg : 1) * dim * sizeof(float);
    int wpb = static_cast<int>((48 * 1024) / per_warp);
    if (wpb < 1) { set_error("%s: %d vector registers of %d floats do not fit the shared memory of one warp", fn, prog->n_vreg, dim); return KGE_E_RANGE; }
    if (wpb > 8) wpb = 8;
    const unsigned blocks = static_cast<unsigned>((batch + wpb - 1) / wpb);
    program_kernel<<<blocks, wpb * 32, per_warp * wpb, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    KGE_LAUNCH_CHECK("program_kernel");
    return 0;
}
