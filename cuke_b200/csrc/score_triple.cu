// Row-per-warp scoring kernels: one warp owns one triple, holds its anchor vector in registers and
// streams that triple's negative rows past it (fused gather + score, no (batch, dim) intermediate).
//
// Replaces the kernels cuke generates for apps/kge/kge.py:273-390 (one warp per triple, scalar loads,
// vector written back to HBM) plus the norm the reference leaves to its caller, and gives the true
// gradients in place of the per-triple demo pieces of apps/kge/kge.py:393-515.
//
// "Anchor" formulation: for a triple (h, r, t) and a replacement row x,
//   tail replaced:  TransE  c = h + r            score = -||c - x||
//                   TransH  c = h - (w.h)w + d   score = -||c - x + (w.x) w||
//                   DistMult c = h*r, ComplEx c = h r (complex), TransF c = 2h + r (+ c0 = -r.h),
//                   RESCAL  c = h P_r (precomputed)                 score = c . x (+ c0)
//   head replaced:  TransE  c = t - r,  TransH c = t - (w.t)w - d,  DistMult c = t*r,
//                   ComplEx c = t conj(r),  TransF c = 2t - r (+ c0 = r.t)       (same score forms)
#include "rows.cuh"

namespace kge {

enum { FORM_DIST = 0, FORM_DIST_H = 1, FORM_DOT = 2 };
template <int MODEL> struct Form { static constexpr int value = FORM_DOT; };
template <> struct Form<KGE_TRANSE> { static constexpr int value = FORM_DIST; };
template <> struct Form<KGE_TRANSH> { static constexpr int value = FORM_DIST_H; };

// Anchor of one triple for the tail-replaced (head == false) or head-replaced (head == true) negatives.
// own = h (tail phase) or t (head phase); c0 is the additive constant of TransF; wown = w.own (TransH).
template <int MODEL, int NV>
__device__ __forceinline__ void make_anchor(bool head, const Row<NV>& own, const Row<NV>& r, const Row<NV>& w,
                                            Row<NV>& c, float& c0, float& wown) {
    c0 = 0.f; wown = 0.f;
    if (MODEL == KGE_TRANSE) {
#pragma unroll
        for (int q = 0; q < NV; ++q) c.v[q] = head ? own.v[q] - r.v[q] : own.v[q] + r.v[q];
    } else if (MODEL == KGE_TRANSH) {
        wown = row_dot<NV>(w, own);
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            float4 p = own.v[q] - wown * w.v[q];
            c.v[q] = head ? p - r.v[q] : p + r.v[q];
        }
    } else if (MODEL == KGE_DISTMULT) {
#pragma unroll
        for (int q = 0; q < NV; ++q) c.v[q] = own.v[q] * r.v[q];
    } else if (MODEL == KGE_COMPLEX) {
#pragma unroll
        for (int q = 0; q < NV; ++q) c.v[q] = head ? cmul_conj(own.v[q], r.v[q]) : cmul(own.v[q], r.v[q]);
    } else if (MODEL == KGE_TRANSF) {
        float ro = row_dot<NV>(r, own);
        c0 = head ? ro : -ro;
#pragma unroll
        for (int q = 0; q < NV; ++q) c.v[q] = head ? 2.f * own.v[q] - r.v[q] : 2.f * own.v[q] + r.v[q];
    } else {   // RESCAL: anchors are precomputed, `own` already holds the anchor
#pragma unroll
        for (int q = 0; q < NV; ++q) c.v[q] = own.v[q];
    }
}

// Score of the positive triple, with the reference's operation order (apps/kge/kge.py:293,317,363,389).
template <int MODEL, int NV>
__device__ __forceinline__ float positive_score(const Row<NV>& h, const Row<NV>& t, const Row<NV>& r, const Row<NV>& w,
                                                const Row<NV>& anchor) {
    if (MODEL == KGE_TRANSE) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { float4 v = (h.v[q] - t.v[q]) + r.v[q]; s = dot4(v, v, s); }
        return -sqrtf(warp_sum(s));
    } else if (MODEL == KGE_TRANSH) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) s = dot4(w.v[q], h.v[q] - t.v[q], s);
        s = warp_sum(s);
        float n2 = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { float4 v = ((h.v[q] - t.v[q]) + r.v[q]) - s * w.v[q]; n2 = dot4(v, v, n2); }
        return -sqrtf(warp_sum(n2));
    } else if (MODEL == KGE_DISTMULT) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) s = dot4(h.v[q] * r.v[q], t.v[q], s);
        return warp_sum(s);
    } else if (MODEL == KGE_COMPLEX) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) s = dot4(cmul(h.v[q], r.v[q]), t.v[q], s);
        return warp_sum(s);
    } else if (MODEL == KGE_TRANSF) {
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { s1 = dot4(h.v[q] + r.v[q], t.v[q], s1); s2 = dot4(t.v[q] - r.v[q], h.v[q], s2); }
        return warp_sum(s1) + warp_sum(s2);
    } else {   // RESCAL: anchor = h P_r
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) s = dot4(anchor.v[q], t.v[q], s);
        return warp_sum(s);
    }
}

template <int MODEL, int NV>
__device__ __forceinline__ float negative_score(const Row<NV>& c, float c0, const Row<NV>& w, const Row<NV>& x) {
    constexpr int FORM = Form<MODEL>::value;
    if (FORM == FORM_DIST) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { float4 e = c.v[q] - x.v[q]; s = dot4(e, e, s); }
        return -sqrtf(warp_sum(s));
    } else if (FORM == FORM_DIST_H) {
        float sw = row_dot<NV>(w, x);
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < NV; ++q) { float4 v = fma4(sw, w.v[q], c.v[q] - x.v[q]); s = dot4(v, v, s); }
        return -sqrtf(warp_sum(s));
    } else {
        return row_dot<NV>(c, x) + c0;
    }
}

// ---------------------------------------------------------------------------------------------------
// Forward.  Work item = (triple i, slice sp of its negatives); nsplit slices per triple keep the GPU
// full when the batch is small.  Slice 0 also scores the positive.
// ---------------------------------------------------------------------------------------------------
template <int MODEL, typename T, typename I, int NV, bool VEC>
__global__ void __launch_bounds__(256) triple_fwd_kernel(ScoreArgs a, int nsplit, int slice) {
    constexpr int U = (NV <= 2) ? 4 : (NV <= 4 ? 2 : 1);
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long i = wid / nsplit;
    const int sp = (int)(wid % nsplit);
    if (i >= a.batch) return;
    const int dim = a.dim;
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* R = reinterpret_cast<const T*>(a.rel);
    const T* W = reinterpret_cast<const T*>(a.rel2);
    const long long hid = load_id<I>(a.h, i), tid = load_id<I>(a.t, i), rid = load_id<I>(a.r, i);

    Row<NV> h, t, r, w, c;
    row_zero<NV>(r); row_zero<NV>(w);
    load_row<T, NV, VEC>(h, E + hid * dim, dim, lane);
    load_row<T, NV, VEC>(t, E + tid * dim, dim, lane);
    if (MODEL != KGE_RESCAL) load_row<T, NV, VEC>(r, R + rid * dim, dim, lane);
    if (MODEL == KGE_TRANSH) load_row<T, NV, VEC>(w, W + rid * dim, dim, lane);
    if (MODEL == KGE_RESCAL) load_row_f32<NV, VEC>(c, a.anchors + i * dim, dim, lane);

    if (sp == 0 && a.pos != nullptr) {
        float ps = positive_score<MODEL, NV>(h, t, r, w, c);
        if (lane == 0) a.pos[i] = ps;
    }
    if (a.n_neg == 0) return;

    const int j_lo = sp * slice;
    const int j_hi = min(a.n_neg, j_lo + slice);
    float* out = a.negs + i * (long long)a.n_neg;
    const long long nbase = i * (long long)a.n_neg;

#pragma unroll 1
    for (int phase = 0; phase < 2; ++phase) {
        const bool head = (phase == 0);
        const int p_lo = head ? j_lo : max(j_lo, a.n_neg_head);
        const int p_hi = head ? min(j_hi, a.n_neg_head) : j_hi;
        if (p_lo >= p_hi) continue;
        float c0, wown;
        if (MODEL == KGE_RESCAL) { c0 = 0.f; }
        else make_anchor<MODEL, NV>(head, head ? t : h, r, w, c, c0, wown);

        float keep = 0.f;
        int j = p_lo;
        for (; j + U <= p_hi; j += U) {
            Row<NV> x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                long long nid = load_id<I>(a.neg, nbase + j + u);
                load_row<T, NV, VEC>(x[u], E + nid * dim, dim, lane);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float sc = negative_score<MODEL, NV>(c, c0, w, x[u]);
                int rel = j + u - p_lo;
                if ((rel & 31) == lane) keep = sc;
                if ((rel & 31) == 31) out[j + u - 31 + lane] = keep;
            }
        }
        for (; j < p_hi; ++j) {
            Row<NV> x;
            long long nid = load_id<I>(a.neg, nbase + j);
            load_row<T, NV, VEC>(x, E + nid * dim, dim, lane);
            float sc = negative_score<MODEL, NV>(c, c0, w, x);
            int rel = j - p_lo;
            if ((rel & 31) == lane) keep = sc;
            if ((rel & 31) == 31) out[j - 31 + lane] = keep;
        }
        const int rem = (p_hi - p_lo) & 31;            // scores still parked in lanes [0, rem)
        if (rem && lane < rem) out[p_hi - rem + lane] = keep;
    }
}

// ---------------------------------------------------------------------------------------------------
// Backward.  One warp per triple; writes one gradient row per id occurrence ("slot"):
//   g_head[i], g_tail[i], g_rel[i] (, g_rel2[i] for TransH), g_neg[i*n_neg + j].
// Phases: positive -> head-replaced negatives -> tail-replaced negatives; each phase adds into the
// triple's own rows (same warp, so plain read-modify-write).  In chunk-shared mode n_neg == 0 here and
// the anchor gradients summed over the chunk's negatives arrive through ga_tail_init / ga_head_init.
// RESCAL: writes the total anchor gradient to g_rel (consumed by the projection backward) and g_tail.
// ---------------------------------------------------------------------------------------------------
template <int MODEL, typename T, typename I, int NV, bool VEC>
__global__ void __launch_bounds__(128) triple_bwd_kernel(ScoreArgs a) {
    constexpr int FORM = Form<MODEL>::value;
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= a.batch) return;
    const int dim = a.dim;
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* R = reinterpret_cast<const T*>(a.rel);
    const T* W = reinterpret_cast<const T*>(a.rel2);
    const long long hid = load_id<I>(a.h, i), tid = load_id<I>(a.t, i), rid = load_id<I>(a.r, i);
    float* gH = a.g_head + i * dim;
    float* gT = a.g_tail + i * dim;
    float* gR = a.g_rel ? a.g_rel + i * dim : nullptr;
    float* gW = (MODEL == KGE_TRANSH) ? a.g_rel2 + i * dim : nullptr;

    Row<NV> w;
    row_zero<NV>(w);
    if (MODEL == KGE_TRANSH) load_row<T, NV, VEC>(w, W + rid * dim, dim, lane);

    // ---- positive ---------------------------------------------------------------------------------
    {
        Row<NV> h, t, r, o1, o2, o3;
        row_zero<NV>(r);
        load_row<T, NV, VEC>(h, E + hid * dim, dim, lane);
        load_row<T, NV, VEC>(t, E + tid * dim, dim, lane);
        if (MODEL != KGE_RESCAL) load_row<T, NV, VEC>(r, R + rid * dim, dim, lane);
        float ds = a.dpos ? a.dpos[i] : 0.f;
        if (a.pos_loss != nullptr) {          // fused step: same formulas as the logistic loss kernel
            const float ps = positive_score<MODEL, NV>(h, t, r, w, h);
            ds = -1.f / (1.f + __expf(ps));                                         // -sigmoid(-ps)
            if (lane == 0) {
                a.pos[i] = ps;
                a.pos_loss[i] = fmaxf(-ps, 0.f) + log1pf(__expf(-fabsf(ps)));      // softplus(-ps)
            }
        }
        if (MODEL == KGE_TRANSE) {
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < NV; ++q) { o1.v[q] = (h.v[q] - t.v[q]) + r.v[q]; s = dot4(o1.v[q], o1.v[q], s); }
            float n = sqrtf(warp_sum(s));
            float coef = n > 0.f ? -ds / n : 0.f;
#pragma unroll
            for (int q = 0; q < NV; ++q) { o1.v[q] = coef * o1.v[q]; o2.v[q] = -1.f * o1.v[q]; }
            store_row<NV, VEC>(gH, o1, dim, lane);
            store_row<NV, VEC>(gT, o2, dim, lane);
            store_row<NV, VEC>(gR, o1, dim, lane);
        } else if (MODEL == KGE_TRANSH) {
            Row<NV> u;
#pragma unroll
            for (int q = 0; q < NV; ++q) u.v[q] = h.v[q] - t.v[q];
            float s = row_dot<NV>(w, u);
            float n2 = 0.f;
#pragma unroll
            for (int q = 0; q < NV; ++q) { o1.v[q] = (u.v[q] + r.v[q]) - s * w.v[q]; n2 = dot4(o1.v[q], o1.v[q], n2); }
            float n = sqrtf(warp_sum(n2));
            float coef = n > 0.f ? -ds / n : 0.f;
#pragma unroll
            for (int q = 0; q < NV; ++q) o1.v[q] = coef * o1.v[q];          // gv
            float gvw = row_dot<NV>(o1, w);
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                o2.v[q] = o1.v[q] - gvw * w.v[q];                            // g_u
                o3.v[q] = -1.f * (gvw * u.v[q] + s * o1.v[q]);               // g_w
            }
            store_row<NV, VEC>(gH, o2, dim, lane);
            store_row<NV, VEC>(gR, o1, dim, lane);
            store_row<NV, VEC>(gW, o3, dim, lane);
#pragma unroll
            for (int q = 0; q < NV; ++q) o2.v[q] = -1.f * o2.v[q];
            store_row<NV, VEC>(gT, o2, dim, lane);
        } else if (MODEL == KGE_DISTMULT) {
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                o1.v[q] = ds * (r.v[q] * t.v[q]); o2.v[q] = ds * (h.v[q] * r.v[q]); o3.v[q] = ds * (h.v[q] * t.v[q]);
            }
            store_row<NV, VEC>(gH, o1, dim, lane);
            store_row<NV, VEC>(gT, o2, dim, lane);
            store_row<NV, VEC>(gR, o3, dim, lane);
        } else if (MODEL == KGE_COMPLEX) {
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                float4 ga = ds * t.v[q];
                o1.v[q] = cmul_conj(ga, r.v[q]);            // g_h = ga conj(r)
                o2.v[q] = ds * cmul(h.v[q], r.v[q]);        // g_t = ds * (h r)
                o3.v[q] = cmul_conj(ga, h.v[q]);            // g_r = ga conj(h)
            }
            store_row<NV, VEC>(gH, o1, dim, lane);
            store_row<NV, VEC>(gT, o2, dim, lane);
            store_row<NV, VEC>(gR, o3, dim, lane);
        } else if (MODEL == KGE_TRANSF) {
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                o1.v[q] = ds * (2.f * t.v[q] - r.v[q]);
                o2.v[q] = ds * (2.f * h.v[q] + r.v[q]);
                o3.v[q] = ds * (t.v[q] - h.v[q]);
            }
            store_row<NV, VEC>(gH, o1, dim, lane);
            store_row<NV, VEC>(gT, o2, dim, lane);
            store_row<NV, VEC>(gR, o3, dim, lane);
        } else {   // RESCAL: anchor c = h P_r;  ga = ds * t -> g_rel buffer; g_tail = ds * c
            Row<NV> c;
            load_row_f32<NV, VEC>(c, a.anchors + i * dim, dim, lane);
#pragma unroll
            for (int q = 0; q < NV; ++q) { o1.v[q] = ds * t.v[q]; o2.v[q] = ds * c.v[q]; }
            store_row<NV, VEC>(gR, o1, dim, lane);
            store_row<NV, VEC>(gT, o2, dim, lane);
        }
    }

    // ---- negatives -----------------------------------------------------------------------------------
    const long long nbase = i * (long long)a.n_neg;
#pragma unroll 1
    for (int phase = 0; phase < 2; ++phase) {
        const bool head = (phase == 0);
        const int p_lo = head ? 0 : a.n_neg_head;
        const int p_hi = head ? a.n_neg_head : a.n_neg;
        const float* init = head ? a.ga_head_init : a.ga_tail_init;
        if (p_lo >= p_hi && init == nullptr) continue;
        if (MODEL == KGE_RESCAL && head) continue;

        Row<NV> own, r, c, gc, gw;
        row_zero<NV>(r); row_zero<NV>(gw);
        float c0 = 0.f, wown = 0.f, cw = 0.f, ww = 0.f, sum_ds = 0.f;
        if (MODEL == KGE_RESCAL) {
            load_row_f32<NV, VEC>(c, a.anchors + i * dim, dim, lane);
        } else {
            load_row<T, NV, VEC>(own, E + (head ? tid : hid) * dim, dim, lane);
            load_row<T, NV, VEC>(r, R + rid * dim, dim, lane);
            make_anchor<MODEL, NV>(head, own, r, w, c, c0, wown);
        }
        if (FORM == FORM_DIST_H) { cw = row_dot<NV>(c, w); ww = row_dot<NV>(w, w); }
        if (init) load_row_f32<NV, VEC>(gc, init + i * dim, dim, lane); else row_zero<NV>(gc);
        if (init && a.ga_init_scale) {         // distance scorers on the tensor cores: init holds sum_j W_ij x_j only
            const float sc = a.ga_init_scale[i];
#pragma unroll
            for (int q = 0; q < NV; ++q) gc.v[q] = sc * c.v[q] - gc.v[q];
        }

        for (int j = p_lo; j < p_hi; ++j) {
            Row<NV> x, gx;
            const long long nid = load_id<I>(a.neg, nbase + j);
            load_row<T, NV, VEC>(x, E + nid * dim, dim, lane);
            const float ds = a.dneg[nbase + j];
            if (FORM == FORM_DIST) {
                float s = 0.f;
#pragma unroll
                for (int q = 0; q < NV; ++q) { x.v[q] = c.v[q] - x.v[q]; s = dot4(x.v[q], x.v[q], s); }
                float n = sqrtf(warp_sum(s));
                float coef = n > 0.f ? -ds / n : 0.f;
#pragma unroll
                for (int q = 0; q < NV; ++q) {
                    float4 gv = coef * x.v[q];
                    gc.v[q] = gc.v[q] + gv;
                    gx.v[q] = -1.f * gv;
                }
            } else if (FORM == FORM_DIST_H) {
                float sw = row_dot<NV>(w, x);
                float s = 0.f;
                Row<NV> v;
#pragma unroll
                for (int q = 0; q < NV; ++q) { v.v[q] = fma4(sw, w.v[q], c.v[q] - x.v[q]); s = dot4(v.v[q], v.v[q], s); }
                float n = sqrtf(warp_sum(s));
                float coef = n > 0.f ? -ds / n : 0.f;
                float gvw = coef * (cw - sw + sw * ww);          // gv . w, with v.w = c.w - (w.x)(1 - w.w)
#pragma unroll
                for (int q = 0; q < NV; ++q) {
                    float4 gv = coef * v.v[q];
                    gc.v[q] = gc.v[q] + gv;
                    gw.v[q] = fma4(gvw, x.v[q], fma4(sw, gv, gw.v[q]));
                    gx.v[q] = fma4(gvw, w.v[q], -1.f * gv);
                }
            } else {
                sum_ds += ds;
#pragma unroll
                for (int q = 0; q < NV; ++q) { gc.v[q] = fma4(ds, x.v[q], gc.v[q]); gx.v[q] = ds * c.v[q]; }
            }
            store_row<NV, VEC>(a.g_neg + (nbase + j) * dim, gx, dim, lane);
        }

        // anchor gradient -> gradients of the triple's own rows
        Row<NV> o;
        if (MODEL == KGE_TRANSE) {
            add_row<NV, VEC>(head ? gT : gH, gc, dim, lane);
            if (head) {
#pragma unroll
                for (int q = 0; q < NV; ++q) gc.v[q] = -1.f * gc.v[q];
            }
            add_row<NV, VEC>(gR, gc, dim, lane);
        } else if (MODEL == KGE_TRANSH) {
            float gcw = row_dot<NV>(gc, w);
#pragma unroll
            for (int q = 0; q < NV; ++q) {
                o.v[q] = gc.v[q] - gcw * w.v[q];
                gw.v[q] = gw.v[q] - (gcw * own.v[q] + wown * gc.v[q]);
            }
            add_row<NV, VEC>(head ? gT : gH, o, dim, lane);
            add_row<NV, VEC>(gW, gw, dim, lane);
            if (head) {
#pragma unroll
                for (int q = 0; q < NV; ++q) gc.v[q] = -1.f * gc.v[q];
            }
            add_row<NV, VEC>(gR, gc, dim, lane);
        } else if (MODEL == KGE_DISTMULT) {
#pragma unroll
            for (int q = 0; q < NV; ++q) o.v[q] = gc.v[q] * r.v[q];
            add_row<NV, VEC>(head ? gT : gH, o, dim, lane);
#pragma unroll
            for (int q = 0; q < NV; ++q) o.v[q] = gc.v[q] * own.v[q];
            add_row<NV, VEC>(gR, o, dim, lane);
        } else if (MODEL == KGE_COMPLEX) {
            if (!head) {   // c = h r : g_h = gc conj(r), g_r = gc conj(h)
#pragma unroll
                for (int q = 0; q < NV; ++q) o.v[q] = cmul_conj(gc.v[q], r.v[q]);
                add_row<NV, VEC>(gH, o, dim, lane);
#pragma unroll
                for (int q = 0; q < NV; ++q) o.v[q] = cmul_conj(gc.v[q], own.v[q]);
                add_row<NV, VEC>(gR, o, dim, lane);
            } else {       // c = t conj(r) : g_t = gc r, g_r = t conj(gc)
#pragma unroll
                for (int q = 0; q < NV; ++q) o.v[q] = cmul(gc.v[q], r.v[q]);
                add_row<NV, VEC>(gT, o, dim, lane);
#pragma unroll
                for (int q = 0; q < NV; ++q) o.v[q] = cmul_conj(own.v[q], gc.v[q]);
                add_row<NV, VEC>(gR, o, dim, lane);
            }
        } else if (MODEL == KGE_TRANSF) {
            const float sg = head ? sum_ds : -sum_ds;
#pragma unroll
            for (int q = 0; q < NV; ++q) o.v[q] = fma4(sg, r.v[q], 2.f * gc.v[q]);       // 2gc -/+ sum_ds r
            add_row<NV, VEC>(head ? gT : gH, o, dim, lane);
#pragma unroll
            for (int q = 0; q < NV; ++q) o.v[q] = fma4(sg, own.v[q], head ? -1.f * gc.v[q] : gc.v[q]);
            add_row<NV, VEC>(gR, o, dim, lane);
        } else {           // RESCAL: accumulate the anchor gradient for the projection backward
            add_row<NV, VEC>(gR, gc, dim, lane);
        }
    }
}

// Anchors of every triple as fp32 rows (operands of the chunk-shared backward contractions).
template <int MODEL, typename T, typename I, int NV, bool VEC>
__global__ void __launch_bounds__(256) anchor_kernel(ScoreArgs a, float* anchors_tail, float* anchors_head) {
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= a.batch) return;
    const int dim = a.dim;
    const T* E = reinterpret_cast<const T*>(a.ent);
    const T* R = reinterpret_cast<const T*>(a.rel);
    const T* W = reinterpret_cast<const T*>(a.rel2);
    const long long rid = load_id<I>(a.r, i);
    Row<NV> own, r, w, c;
    row_zero<NV>(w);
    load_row<T, NV, VEC>(r, R + rid * dim, dim, lane);
    if (MODEL == KGE_TRANSH) load_row<T, NV, VEC>(w, W + rid * dim, dim, lane);
    float c0, wown;
    if (anchors_tail) {
        load_row<T, NV, VEC>(own, E + load_id<I>(a.h, i) * dim, dim, lane);
        make_anchor<MODEL, NV>(false, own, r, w, c, c0, wown);
        store_row<NV, VEC>(anchors_tail + i * dim, c, dim, lane);
    }
    if (anchors_head) {
        load_row<T, NV, VEC>(own, E + load_id<I>(a.t, i) * dim, dim, lane);
        make_anchor<MODEL, NV>(true, own, r, w, c, c0, wown);
        store_row<NV, VEC>(anchors_head + i * dim, c, dim, lane);
    }
}

// ---------------------------------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------------------------------
enum { K_FWD = 0, K_BWD = 1, K_ANCHOR = 2 };

template <int MODEL, typename T, typename I, int NV, bool VEC>
static int run_kernel(int which, const ScoreArgs& a, float* at, float* ah, cudaStream_t s) {
    if (which == K_FWD) {
        // split a triple's negatives over several warps until ~4 warps per SM-slot are in flight
        int nsplit = 1;
        if (a.n_neg > 0) {
            long long target = 148LL * 64;
            while ((long long)a.batch * nsplit < target && a.n_neg / (nsplit * 2) >= 8) nsplit *= 2;
        }
        int slice = a.n_neg > 0 ? (a.n_neg + nsplit - 1) / nsplit : 0;
        long long warps = a.batch * nsplit;
        const int wpb = 8;
        long long blocks = (warps + wpb - 1) / wpb;
        triple_fwd_kernel<MODEL, T, I, NV, VEC><<<(unsigned)blocks, wpb * 32, 0, s>>>(a, nsplit, slice);
        KGE_LAUNCH_CHECK("triple_fwd_kernel");
    } else if (which == K_BWD) {
        const int wpb = 4;
        long long blocks = (a.batch + wpb - 1) / wpb;
        triple_bwd_kernel<MODEL, T, I, NV, VEC><<<(unsigned)blocks, wpb * 32, 0, s>>>(a);
        KGE_LAUNCH_CHECK("triple_bwd_kernel");
    } else {
        const int wpb = 8;
        long long blocks = (a.batch + wpb - 1) / wpb;
        anchor_kernel<MODEL, T, I, NV, VEC><<<(unsigned)blocks, wpb * 32, 0, s>>>(a, at, ah);
        KGE_LAUNCH_CHECK("anchor_kernel");
    }
    return 0;
}

template <int MODEL, typename T, typename I>
static int dispatch_nv(int which, const ScoreArgs& a, float* at, float* ah, cudaStream_t s) {
    const bool vec = (a.dim % 4 == 0);
    const int nv = quads_per_lane(a.dim);
    if (nv == 0) { set_error("dim %d > 1024 is not supported by the row-per-warp scorers", a.dim); return KGE_E_UNSUPPORTED; }
#define KGE_NV_CASE(N)                                                                            \
    case N: return vec ? run_kernel<MODEL, T, I, N, true>(which, a, at, ah, s)                    \
                       : run_kernel<MODEL, T, I, N, false>(which, a, at, ah, s);
    switch (nv) {
        KGE_NV_CASE(1) KGE_NV_CASE(2) KGE_NV_CASE(4) KGE_NV_CASE(8)
    }
#undef KGE_NV_CASE
    return KGE_E_UNSUPPORTED;
}

template <int MODEL>
static int dispatch_types(int which, const ScoreArgs& a, float* at, float* ah, cudaStream_t s) {
    if (a.dtype == KGE_F32) {
        return a.id_bits == 64 ? dispatch_nv<MODEL, float, int64_t>(which, a, at, ah, s)
                               : dispatch_nv<MODEL, float, int32_t>(which, a, at, ah, s);
    }
    return a.id_bits == 64 ? dispatch_nv<MODEL, __nv_bfloat16, int64_t>(which, a, at, ah, s)
                           : dispatch_nv<MODEL, __nv_bfloat16, int32_t>(which, a, at, ah, s);
}

static int dispatch_model(int which, const ScoreArgs& a, float* at, float* ah, cudaStream_t s) {
    if (a.batch <= 0) return 0;
    switch (a.model) {
        case KGE_TRANSE: return dispatch_types<KGE_TRANSE>(which, a, at, ah, s);
        case KGE_TRANSH: return dispatch_types<KGE_TRANSH>(which, a, at, ah, s);
        case KGE_TRANSF: return dispatch_types<KGE_TRANSF>(which, a, at, ah, s);
        case KGE_DISTMULT: return dispatch_types<KGE_DISTMULT>(which, a, at, ah, s);
        case KGE_COMPLEX: return dispatch_types<KGE_COMPLEX>(which, a, at, ah, s);
        case KGE_RESCAL:
            if (which == K_ANCHOR) break;
            return dispatch_types<KGE_RESCAL>(which, a, at, ah, s);
        default: break;
    }
    set_error("model %d has no row-per-warp scorer", a.model);
    return KGE_E_UNSUPPORTED;
}

int launch_triple_forward(const ScoreArgs& a, cudaStream_t s) { return dispatch_model(K_FWD, a, nullptr, nullptr, s); }
int launch_triple_backward(const ScoreArgs& a, cudaStream_t s) { return dispatch_model(K_BWD, a, nullptr, nullptr, s); }
int launch_anchor(const ScoreArgs& a, float* at, float* ah, cudaStream_t s) { return dispatch_model(K_ANCHOR, a, at, ah, s); }

}  // namespace kge
