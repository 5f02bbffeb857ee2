// extern "C" entry points of libkge_b200.so: argument validation, workspace carving, launch sequencing.
// Declarations and their reference counterparts are in include/kge_b200.h.
#include <stdarg.h>
#include <string.h>
#include <atomic>
#include "common.cuh"

namespace kge {

// ---- error plumbing ------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int cuda_status(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return (int)e;
}

static std::atomic<long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

__device__ int32_t g_error_word = 0;
int32_t* device_error_word() {
    int32_t* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_error_word) != cudaSuccess) return nullptr;
    return p;
}

// implemented in the other translation units
int launch_pair_forward(const ScoreArgs& a, int head, cudaStream_t s);
int launch_pair_backward(const ScoreArgs& a, const float* anchors, float* ga, cudaStream_t s);
size_t inspect_workspace_bytes(long long n);
int launch_inspect(const void* ids, int id_bits, long long n, long long id_space, void* ws, size_t ws_bytes,
                   long long* uniq, int* inverse, int* perm, int* seg, long long* n_unique, cudaStream_t s);
size_t segment_reduce_workspace_bytes(long long n, int dim);
int launch_segment_reduce(const float* rows, int dim, long long n, const int* perm, const int* seg,
                          const long long* n_unique, float* out, long long n_out, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_gather_rows(const void* table, int dtype, int dim, const long long* ids, long long n, const long long* n_dev,
                       long long first_row, void* out, cudaStream_t s);
int launch_scatter_rows(const float* rows, int dim, const long long* ids, long long n, const long long* n_dev,
                        long long first_row, float* out, cudaStream_t s);
int launch_fma_probe(float* out, int blocks, int iters, cudaStream_t s);
int launch_owner_counts(const long long* uniq, const long long* n_unique, long long n_max, long long rows_per_rank,
                        int world, long long* counts, cudaStream_t s);
int launch_legacy_inspect(const long long* rel, long long n, long long rel_num, long long* uniq, long long* buf,
                          long long* cnt, cudaStream_t s);
int launch_logistic_loss(const float* pos, long long n_pos, const float* neg, long long n_neg, float neg_w, float* dpos,
                         float* dneg, float* loss, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_rescal_anchors(const kge_problem* p, const kge_tensors* t, float* anchors, cudaStream_t s);
int launch_rescal_backward(const kge_problem* p, const kge_tensors* t, const float* ga, float* g_head, float* dproj,
                           cudaStream_t s);
int launch_transr_forward(const kge_problem* p, const kge_tensors* t, float* pos, float* negs, cudaStream_t s);
size_t tc_transr_workspace_bytes(long long batch, int n_neg, int dim, long long n_rel, int backward);
int launch_transr_backward_tc(const ScoreArgs& a, float* dproj, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                              const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_transr_forward_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                             const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes, cudaStream_t s);
size_t transr_backward_workspace_bytes(const kge_problem* p);
int launch_transr_backward(const kge_problem* p, const kge_tensors* t, const float* pos, const float* negs, const float* dpos,
                           const float* dneg, const kge_grads* g, void* ws, cudaStream_t s);
size_t tc_pair_workspace_bytes(long long batch, int chunk, int n_neg, int dim, int mode, int es);
size_t tc_rescal_workspace_bytes(long long batch, int dim, long long n_rel, int backward);
int launch_rescal_anchors_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                             const long long* n_groups, long long n_rel, float* anchors, int backward, void* ws, size_t ws_bytes,
                             cudaStream_t s);
int launch_rescal_backward_tc(const ScoreArgs& a, const int* rel_perm, const int* rel_seg, const long long* rel_uniq,
                              const long long* n_groups, long long n_rel, const float* ga, float* g_head, float* dproj,
                              bool prepared, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_pair_forward_tc(const ScoreArgs& a, int head, void* ws, size_t ws_bytes, cudaStream_t s);
void gemm_profile_enable(int on);
int gemm_profile_read(double* ms, long long* launches, double* flops);
int launch_pair_backward_tc(const ScoreArgs& a, int head, float* ga, const float** ga_scale, void* ws, size_t ws_bytes, cudaStream_t s);
int launch_pair_loss_backward_tc(const ScoreArgs& a, int head, float neg_w, float* loss, float* ga, const float** ga_scale,
                                 void* ws, size_t ws_bytes, cudaStream_t s);
int launch_loss_add(const float* part, long long n, float* loss, cudaStream_t s);
int launch_transr_loss_backward_tc(const ScoreArgs& a, float neg_w, float* loss, float* dproj, const int* rel_perm, const int* rel_seg,
                                   const long long* rel_uniq, const long long* n_groups, long long n_rel, void* ws, size_t ws_bytes,
                                   cudaStream_t s);
int launch_validate_ids(const void* ids, int id_bits, long long n, long long limit, void* out, cudaStream_t s);
int launch_gather_rows_peers(const void* const* shards, int world, long long rows_per_rank, long long n_rows_total, int dtype, int dim,
                             const long long* ids, long long n, const long long* n_dev, void* out, cudaStream_t s);
int launch_pull_reduce(const float* const* bases, const long long* src_off, const long long* src_start, int world, int dim,
                       const int* perm, const int* seg, const long long* n_unique, long long n_max, float* out, float* sgd_table,
                       const long long* ids, long long first_row, float lr, cudaStream_t s);
int ipc_export(const void* ptr, void* handle, unsigned long long* offset);
int ipc_open(const void* handle, unsigned long long offset, void** out);
int ipc_close(void* ptr, unsigned long long offset);
int launch_wait_timeout_selftest(int polls, cudaStream_t s);

// ---- validation -------------------------------------------------------------------------------------------
#define KGE_REQUIRE_PTR(ptr, name)                                                     \
    do {                                                                               \
        if ((ptr) == nullptr) { set_error("%s: %s is NULL", fn, name); return KGE_E_NULL; } \
        if (!aligned16(ptr)) { set_error("%s: %s is not 16-byte aligned", fn, name); return KGE_E_ALIGN; } \
    } while (0)
// id arrays are read element-wise: natural alignment is enough (slices of an inverse map start anywhere)
#define KGE_REQUIRE_IDS(ptr, name, bits)                                               \
    do {                                                                               \
        if ((ptr) == nullptr) { set_error("%s: %s is NULL", fn, name); return KGE_E_NULL; } \
        if (reinterpret_cast<uintptr_t>(ptr) & ((bits) / 8 - 1)) { set_error("%s: %s is not aligned to its element size", fn, name); return KGE_E_ALIGN; } \
    } while (0)
// gradient rows: vector (16-byte) stores only when dim % 4 == 0, element stores otherwise
#define KGE_REQUIRE_ROWS(ptr, name, dim)                                               \
    do {                                                                               \
        if ((ptr) == nullptr) { set_error("%s: %s is NULL", fn, name); return KGE_E_NULL; } \
        if (reinterpret_cast<uintptr_t>(ptr) & (((dim) % 4 == 0) ? 15u : 3u)) {        \
            set_error("%s: %s is not aligned (16 bytes when dim %% 4 == 0, else 4)", fn, name); return KGE_E_ALIGN; } \
    } while (0)
#define KGE_OPTIONAL_PTR(ptr, name)                                                    \
    do {                                                                               \
        if ((ptr) != nullptr && !aligned16(ptr)) { set_error("%s: %s is not 16-byte aligned", fn, name); return KGE_E_ALIGN; } \
    } while (0)

static bool uses_rel(int model) { return model != KGE_RESCAL; }
static bool uses_rel2(int model) { return model == KGE_TRANSH || model == KGE_TRANSR || model == KGE_RESCAL; }
static bool matrix_model(int model) { return model == KGE_TRANSR || model == KGE_RESCAL; }

static int check_problem(const char* fn, const kge_problem* p, const kge_tensors* t, bool scored) {
    if (!p || !t) { set_error("%s: problem/tensors is NULL", fn); return KGE_E_NULL; }
    if (p->model < KGE_TRANSE || p->model > KGE_COMPLEX) { set_error("%s: unknown model %d", fn, p->model); return KGE_E_UNSUPPORTED; }
    if (p->dtype != KGE_F32 && p->dtype != KGE_BF16) { set_error("%s: unknown dtype %d", fn, p->dtype); return KGE_E_UNSUPPORTED; }
    if (p->id_bits != 32 && p->id_bits != 64) { set_error("%s: id_bits must be 32 or 64, got %d", fn, p->id_bits); return KGE_E_UNSUPPORTED; }
    if (p->dim <= 0 || p->dim > 1024) { set_error("%s: dim %d outside [1, 1024]", fn, p->dim); return KGE_E_UNSUPPORTED; }
    if (p->model == KGE_COMPLEX && (p->dim & 1)) { set_error("%s: ComplEx needs an even dim (re,im interleaved), got %d", fn, p->dim); return KGE_E_SHAPE; }
    if (p->dtype == KGE_BF16 && (p->dim & 7)) { set_error("%s: bf16 tables need dim %% 8 == 0 (16-byte rows), got %d", fn, p->dim); return KGE_E_UNSUPPORTED; }
    if (p->batch < 0) { set_error("%s: negative batch", fn); return KGE_E_SHAPE; }
    if (p->precision != KGE_PREC_FP32 && p->precision != KGE_PREC_TENSOR && p->precision != KGE_PREC_TENSOR_TF32) { set_error("%s: unknown precision %d", fn, p->precision); return KGE_E_UNSUPPORTED; }
    if (p->reserved & ~KGE_FLAG_CHECK_IDS) { set_error("%s: unknown flags 0x%x in reserved", fn, p->reserved); return KGE_E_UNSUPPORTED; }
    if (!scored && p->reserved) { set_error("%s: KGE_FLAG_CHECK_IDS needs a workspace; check the ids with kge_validate_ids first", fn); return KGE_E_UNSUPPORTED; }
    if (p->batch == 0) return 0;
    KGE_REQUIRE_PTR(t->ent, "ent");
    if (uses_rel(p->model)) KGE_REQUIRE_PTR(t->rel, "rel");
    if (uses_rel2(p->model)) KGE_REQUIRE_PTR(t->rel2, "rel2");
    KGE_REQUIRE_IDS(t->h, "h", p->id_bits); KGE_REQUIRE_IDS(t->r, "r", p->id_bits); KGE_REQUIRE_IDS(t->t, "t", p->id_bits);
    if (!scored) {
        if (p->neg_mode != KGE_NEG_NONE) { set_error("%s: neg_mode must be KGE_NEG_NONE (flatten negatives into the batch)", fn); return KGE_E_UNSUPPORTED; }
        return 0;
    }
    if (p->neg_mode < KGE_NEG_NONE || p->neg_mode > KGE_NEG_CHUNK_SHARED) { set_error("%s: unknown neg_mode %d", fn, p->neg_mode); return KGE_E_UNSUPPORTED; }
    if (p->neg_mode != KGE_NEG_NONE) {
        if (p->n_neg <= 0) { set_error("%s: n_neg must be > 0 with negatives", fn); return KGE_E_SHAPE; }
        if (p->n_neg_head < 0 || p->n_neg_head > p->n_neg) { set_error("%s: n_neg_head %d outside [0, n_neg]", fn, p->n_neg_head); return KGE_E_SHAPE; }
        KGE_REQUIRE_IDS(t->neg, "neg", p->id_bits);
    }
    if (p->neg_mode == KGE_NEG_CHUNK_SHARED) {
        if (p->chunk <= 0 || p->batch % p->chunk != 0) { set_error("%s: batch %lld is not a multiple of chunk %d", fn, (long long)p->batch, p->chunk); return KGE_E_SHAPE; }
        if (p->n_neg_head != 0 && p->n_neg_head != p->n_neg) { set_error("%s: chunk-shared negatives replace one side only (n_neg_head must be 0 or n_neg)", fn); return KGE_E_UNSUPPORTED; }
        if (p->model == KGE_TRANSH || p->model == KGE_TRANSF || p->model == KGE_TRANSR) {
            set_error("%s: model %d supports per-triple negatives only", fn, p->model); return KGE_E_UNSUPPORTED;
        }
    }
    if (p->model == KGE_RESCAL && p->neg_mode != KGE_NEG_NONE && p->n_neg_head != 0) {
        set_error("%s: RESCAL negatives replace the tail only", fn); return KGE_E_UNSUPPORTED;
    }
    if (matrix_model(p->model)) {
        KGE_REQUIRE_PTR(t->rel_perm, "rel_perm"); KGE_REQUIRE_PTR(t->rel_seg, "rel_seg");
        KGE_REQUIRE_PTR(t->rel_uniq, "rel_uniq"); KGE_REQUIRE_PTR(t->n_rel_groups, "n_rel_groups");
        if (p->n_rel <= 0) { set_error("%s: n_rel must be given for relation-matrix models", fn); return KGE_E_SHAPE; }
    }
    return 0;
}

static ScoreArgs score_args(const kge_problem* p, const kge_tensors* t) {
    ScoreArgs a;
    memset(&a, 0, sizeof(a));
    a.ent = t->ent; a.rel = t->rel; a.rel2 = t->rel2; a.h = t->h; a.r = t->r; a.t = t->t; a.neg = t->neg;
    a.batch = p->batch; a.dim = p->dim; a.chunk = p->chunk;
    a.n_neg = p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg;
    a.n_neg_head = p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg_head;
    a.model = p->model; a.dtype = p->dtype; a.id_bits = p->id_bits;
    a.tc_es = p->precision == KGE_PREC_TENSOR_TF32 ? 4 : 2;
    return a;
}

static inline size_t rows_bytes(const kge_problem* p) { return ((size_t)p->batch * p->dim * 4 + 255) / 256 * 256; }

// The tensor-core contractions exist for the scorers that support chunk-shared negatives.
static bool tensor_precision(const kge_problem* p) { return p->precision == KGE_PREC_TENSOR || p->precision == KGE_PREC_TENSOR_TF32; }
static int tc_es(const kge_problem* p) { return p->precision == KGE_PREC_TENSOR_TF32 ? 4 : 2; }
static bool tc_forward(const kge_problem* p) {
    return tensor_precision(p) && p->neg_mode == KGE_NEG_CHUNK_SHARED && p->dim % 4 == 0 &&
           (p->model == KGE_TRANSE || p->model == KGE_DISTMULT || p->model == KGE_COMPLEX || p->model == KGE_RESCAL);
}
// TransR forward on the tensor cores: bf16 tables, one n-tile per row.
static bool tc_transr(const kge_problem* p) {
    return tensor_precision(p) && p->model == KGE_TRANSR && p->dtype == KGE_BF16 && p->dim % 8 == 0 && p->dim <= 256 &&
           p->neg_mode != KGE_NEG_CHUNK_SHARED;
}
// RESCAL projections on the tensor cores: fp32 tables split into bf16 pairs, one n-tile per row (dim <= 256)
static bool tc_rescal(const kge_problem* p) {
    return p->precision == KGE_PREC_TENSOR && p->model == KGE_RESCAL && p->dim % 8 == 0 && p->dim <= 256 && p->n_rel > 0;
}
static size_t tc_rescal_bytes(const kge_problem* p, int backward) {
    return tc_rescal(p) ? tc_rescal_workspace_bytes(p->batch, p->dim, p->n_rel, backward) : 0;
}
static bool tc_backward(const kge_problem* p) { return tc_forward(p); }
static size_t tc_bytes(const kge_problem* p, int backward) {
    if (backward ? !tc_backward(p) : !tc_forward(p)) return 0;
    return tc_pair_workspace_bytes(p->batch, p->chunk, p->n_neg, p->dim, backward, tc_es(p));
}
// Fused forward + loss + backward: the chunk-shared tensor-core scorers whose anchors are built from table rows alone.
static bool tc_fused(const kge_problem* p) { return tc_backward(p) && p->model != KGE_RESCAL; }

// ---- KGE_FLAG_CHECK_IDS: sanitised copies of h, r, t, neg in the tail of the workspace ------------------------------
static long long neg_id_count(const kge_problem* p) {
    if (p->neg_mode == KGE_NEG_PER_TRIPLE) return p->batch * p->n_neg;
    if (p->neg_mode == KGE_NEG_CHUNK_SHARED && p->chunk > 0) return (p->batch / p->chunk) * p->n_neg;
    return 0;
}
static inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
static size_t check_ids_bytes(const kge_problem* p) {
    if (!p || !(p->reserved & KGE_FLAG_CHECK_IDS) || p->batch <= 0) return 0;
    const size_t eb = p->id_bits == 64 ? 8 : 4;
    return 3 * up256((size_t)p->batch * eb) + up256((size_t)neg_id_count(p) * eb) + 256;
}
// `at` = first byte of the id area (the call's own scratch ends there).  Fills *ts with the sanitised id pointers.
static int sanitise_ids(const kge_problem* p, const kge_tensors* t, kge_tensors* ts, char* at, cudaStream_t s) {
    *ts = *t;
    const size_t eb = p->id_bits == 64 ? 8 : 4;
    at = reinterpret_cast<char*>(up256(reinterpret_cast<uintptr_t>(at)));
    const void* src[4] = {t->h, t->r, t->t, t->neg};
    const void** dst[4] = {&ts->h, &ts->r, &ts->t, &ts->neg};
    const long long cnt[4] = {p->batch, p->batch, p->batch, neg_id_count(p)};
    const long long lim[4] = {p->n_ent, p->n_rel, p->n_ent, p->n_ent};
    for (int k = 0; k < 4; ++k) {
        if (cnt[k] <= 0 || src[k] == nullptr) continue;
        int rc = launch_validate_ids(src[k], p->id_bits, cnt[k], lim[k], at, s);
        if (rc) return rc;
        *dst[k] = at;
        at += up256((size_t)cnt[k] * eb);
    }
    return 0;
}

}  // namespace kge

using namespace kge;

extern "C" {

int kge_version(void) { return KGE_ABI_VERSION; }
const char* kge_last_error(void) { return g_err; }
long long kge_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int kge_check(kge_stream_t stream, int32_t* flags_out) {
    const char* fn = "kge_check";
    if (!flags_out) { set_error("%s: flags_out is NULL", fn); return KGE_E_NULL; }
    int32_t* w = device_error_word();
    if (!w) { set_error("%s: no device error word (no usable device?)", fn); return KGE_E_DEVICE; }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(flags_out, w, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(w, 0, sizeof(int32_t), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return cuda_status(e, fn);
}

int kge_validate_ids(const void* ids, int32_t id_bits, int64_t n, int64_t id_space, void* sanitized, kge_stream_t stream) {
    const char* fn = "kge_validate_ids";
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    if (n < 0 || id_space < 1) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (n == 0) return 0;
    KGE_REQUIRE_IDS(ids, "ids", id_bits);
    if (sanitized) KGE_REQUIRE_IDS(sanitized, "sanitized", id_bits);
    return launch_validate_ids(ids, id_bits, n, id_space, sanitized, reinterpret_cast<cudaStream_t>(stream));
}

int kge_selftest_wait_timeout(int32_t polls, kge_stream_t stream) {
    const char* fn = "kge_selftest_wait_timeout";
    if (polls < 1 || polls > 65536) { set_error("%s: polls %d outside [1, 65536]", fn, polls); return KGE_E_RANGE; }
    return launch_wait_timeout_selftest(polls, reinterpret_cast<cudaStream_t>(stream));
}

int kge_ref_forward(const kge_problem* p, const kge_tensors* t, float* out, kge_stream_t stream) {
    const char* fn = "kge_ref_forward";
    int rc = check_problem(fn, p, t, false);
    if (rc) return rc;
    if (p->batch == 0) return 0;
    KGE_REQUIRE_PTR(out, "out");
    return launch_ref_forward(p, t, out, reinterpret_cast<cudaStream_t>(stream));
}

size_t kge_inspect_workspace_bytes(int64_t n) { return inspect_workspace_bytes(n); }

int kge_inspect(const void* ids, int32_t id_bits, int64_t n, int64_t id_space, void* workspace, size_t workspace_bytes,
                int64_t* uniq, int32_t* inverse, int32_t* perm, int32_t* seg, int64_t* n_unique, kge_stream_t stream) {
    const char* fn = "kge_inspect";
    if (n < 0 || n > 2147483647LL) { set_error("%s: n %lld outside [0, 2^31-1]", fn, (long long)n); return KGE_E_RANGE; }
    if (id_space < 1 || id_space > (1LL << 31)) { set_error("%s: id_space %lld outside [1, 2^31]", fn, (long long)id_space); return KGE_E_RANGE; }
    if (id_bits != 32 && id_bits != 64) { set_error("%s: id_bits must be 32 or 64", fn); return KGE_E_UNSUPPORTED; }
    KGE_REQUIRE_PTR(seg, "seg"); KGE_REQUIRE_PTR(n_unique, "n_unique");
    if (n > 0) {
        KGE_REQUIRE_PTR(ids, "ids"); KGE_REQUIRE_PTR(workspace, "workspace"); KGE_REQUIRE_PTR(uniq, "uniq");
        KGE_REQUIRE_PTR(inverse, "inverse"); KGE_REQUIRE_PTR(perm, "perm");
    }
    return launch_inspect(ids, id_bits, n, id_space, workspace, workspace_bytes, (long long*)uniq, inverse, perm, seg,
                          (long long*)n_unique, reinterpret_cast<cudaStream_t>(stream));
}

int kge_legacy_inspect(const int64_t* rel, int64_t n, int64_t rel_num, int64_t* uniq, int64_t* buf, int64_t* cnt,
                       kge_stream_t stream) {
    const char* fn = "kge_legacy_inspect";
    if (n < 0 || n % 16 != 0) { set_error("%s: n %lld is not a non-negative multiple of 16", fn, (long long)n); return KGE_E_SHAPE; }
    if (n == 0) return 0;
    KGE_REQUIRE_PTR(rel, "rel"); KGE_REQUIRE_PTR(uniq, "uniq"); KGE_REQUIRE_PTR(buf, "buf"); KGE_REQUIRE_PTR(cnt, "cnt");
    return launch_legacy_inspect((const long long*)rel, n, rel_num, (long long*)uniq, (long long*)buf, (long long*)cnt,
                                 reinterpret_cast<cudaStream_t>(stream));
}

int kge_gather_rows(const void* table, int32_t dtype, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                    int64_t first_row, void* out, kge_stream_t stream) {
    const char* fn = "kge_gather_rows";
    if (n <= 0) return 0;
    if (dim <= 0) { set_error("%s: dim must be positive", fn); return KGE_E_SHAPE; }
    if (dtype != KGE_F32 && dtype != KGE_BF16) { set_error("%s: unknown dtype %d", fn, dtype); return KGE_E_UNSUPPORTED; }
    KGE_REQUIRE_PTR(table, "table"); KGE_REQUIRE_PTR(ids, "ids"); KGE_REQUIRE_PTR(out, "out");
    return launch_gather_rows(table, dtype, dim, (const long long*)ids, n, (const long long*)n_dev, first_row, out,
                              reinterpret_cast<cudaStream_t>(stream));
}

int kge_gather_rows_peers(const void* const* shards, int32_t world, int64_t rows_per_rank, int64_t n_rows, int32_t dtype, int32_t dim,
                          const int64_t* ids, int64_t n, const int64_t* n_dev, void* out, kge_stream_t stream) {
    const char* fn = "kge_gather_rows_peers";
    if (n <= 0) return 0;
    if (dim <= 0 || world <= 0 || rows_per_rank <= 0 || n_rows <= 0 || n_rows > rows_per_rank * world) {
        set_error("%s: need dim, world, rows_per_rank > 0 and 0 < n_rows <= rows_per_rank * world", fn);
        return KGE_E_SHAPE;
    }
    if (dtype != KGE_F32 && dtype != KGE_BF16) { set_error("%s: unknown dtype %d", fn, dtype); return KGE_E_UNSUPPORTED; }
    if (shards == nullptr) { set_error("%s: shards is NULL", fn); return KGE_E_NULL; }
    KGE_REQUIRE_PTR(ids, "ids"); KGE_REQUIRE_PTR(out, "out");
    return launch_gather_rows_peers(shards, world, rows_per_rank, n_rows, dtype, dim, (const long long*)ids, n, (const long long*)n_dev, out,
                                    reinterpret_cast<cudaStream_t>(stream));
}

int kge_pull_reduce(const float* const* bases, const int64_t* src_off, const int64_t* src_start, int32_t world, int32_t dim,
                    const int32_t* perm, const int32_t* seg, const int64_t* n_unique, int64_t n_max, float* out, float* sgd_table,
                    const int64_t* ids, int64_t first_row, float lr, kge_stream_t stream) {
    const char* fn = "kge_pull_reduce";
    if (n_max <= 0) return 0;
    if (dim <= 0 || world <= 0) { set_error("%s: dim and world must be positive", fn); return KGE_E_SHAPE; }
    if (!bases || !src_off || !src_start || !perm || !seg || !n_unique) { set_error("%s: NULL argument", fn); return KGE_E_NULL; }
    KGE_REQUIRE_ROWS(out, "out", dim);
    if (sgd_table) {
        KGE_REQUIRE_ROWS(sgd_table, "sgd_table", dim);
        if (!ids) { set_error("%s: sgd_table without ids", fn); return KGE_E_NULL; }
    }
    return launch_pull_reduce(bases, (const long long*)src_off, (const long long*)src_start, world, dim, perm, seg,
                              (const long long*)n_unique, n_max, out, sgd_table, (const long long*)ids, first_row, lr,
                              reinterpret_cast<cudaStream_t>(stream));
}

int kge_ipc_export(const void* ptr, void* handle64, uint64_t* offset) {
    const char* fn = "kge_ipc_export";
    if (!ptr || !handle64 || !offset) { set_error("%s: NULL argument", fn); return KGE_E_NULL; }
    unsigned long long off = 0;
    const int rc = ipc_export(ptr, handle64, &off);
    *offset = off;
    return rc;
}

int kge_ipc_open(const void* handle64, uint64_t offset, void** ptr_out) {
    const char* fn = "kge_ipc_open";
    if (!handle64 || !ptr_out) { set_error("%s: NULL argument", fn); return KGE_E_NULL; }
    return ipc_open(handle64, offset, ptr_out);
}

int kge_ipc_close(void* ptr, uint64_t offset) {
    const char* fn = "kge_ipc_close";
    if (!ptr) { set_error("%s: NULL argument", fn); return KGE_E_NULL; }
    return ipc_close(ptr, offset);
}

int kge_scatter_rows(const float* rows, int32_t dim, const int64_t* ids, int64_t n, const int64_t* n_dev,
                     int64_t first_row, float* out, kge_stream_t stream) {
    const char* fn = "kge_scatter_rows";
    if (n <= 0) return 0;
    if (dim <= 0) { set_error("%s: dim must be positive", fn); return KGE_E_SHAPE; }
    KGE_REQUIRE_PTR(rows, "rows"); KGE_REQUIRE_PTR(ids, "ids"); KGE_REQUIRE_PTR(out, "out");
    return launch_scatter_rows(rows, dim, (const long long*)ids, n, (const long long*)n_dev, first_row, out,
                               reinterpret_cast<cudaStream_t>(stream));
}

int kge_probe_fma(float* out, int32_t blocks, int32_t iters, double* flops_out, kge_stream_t stream) {
    const char* fn = "kge_probe_fma";
    KGE_REQUIRE_PTR(out, "out");
    if (blocks <= 0 || iters <= 0) { set_error("%s: blocks and iters must be positive", fn); return KGE_E_SHAPE; }
    if (flops_out) *flops_out = 2.0 * 8 * 16 * (double)iters * 256.0 * (double)blocks;
    return launch_fma_probe(out, blocks, iters, reinterpret_cast<cudaStream_t>(stream));
}

size_t kge_segment_reduce_workspace_bytes(int64_t n, int32_t dim) { return segment_reduce_workspace_bytes(n < 1 ? 1 : n, dim); }

int kge_segment_reduce(const float* rows, int32_t dim, int64_t n, const int32_t* perm, const int32_t* seg,
                       const int64_t* n_unique, float* out, int64_t n_out, void* workspace, size_t workspace_bytes,
                       kge_stream_t stream) {
    const char* fn = "kge_segment_reduce";
    if (n < 0 || n > 2147483647LL || n_out < 0) { set_error("%s: bad sizes", fn); return KGE_E_RANGE; }
    if (dim <= 0 || dim > 1024) { set_error("%s: dim %d outside [1, 1024]", fn, dim); return KGE_E_UNSUPPORTED; }
    if (n_out > 0 || n > 0) KGE_REQUIRE_PTR(out, "out");
    if (n > 0) {
        KGE_REQUIRE_PTR(rows, "rows"); KGE_REQUIRE_PTR(perm, "perm"); KGE_REQUIRE_PTR(seg, "seg");
        KGE_REQUIRE_PTR(n_unique, "n_unique"); KGE_REQUIRE_PTR(workspace, "workspace");
    }
    return launch_segment_reduce(rows, dim, n, perm, seg, (const long long*)n_unique, out, n_out, workspace,
                                 workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

static size_t score_scratch_bytes(const kge_problem* p, int32_t backward);
size_t kge_score_workspace_bytes(const kge_problem* p, int32_t backward) {
    return score_scratch_bytes(p, backward) + check_ids_bytes(p);
}
static size_t score_scratch_bytes(const kge_problem* p, int32_t backward) {
    if (!p || p->batch <= 0) return 256;
    const size_t rb = rows_bytes(p);
    if (backward && tc_transr(p))
        return tc_transr_workspace_bytes(p->batch, p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg, p->dim, p->n_rel, 1) + 256;
    if (backward && p->model == KGE_TRANSR) return transr_backward_workspace_bytes(p) + 256;
    if (backward) return 3 * rb + tc_bytes(p, 1) + tc_rescal_bytes(p, 1) + 256;
    if (tc_transr(p)) return tc_transr_workspace_bytes(p->batch, p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg, p->dim, p->n_rel, 0) + 256;
    return (p->model == KGE_RESCAL ? rb : 0) + tc_bytes(p, 0) + tc_rescal_bytes(p, 0) + 256;
}

// RESCAL anchors by the tensor-core route where it applies (its scratch at `tcw`), else by the CUDA-core kernels
static int rescal_anchors(const kge_problem* p, const kge_tensors* t, const ScoreArgs& a, float* anchors, char* tcw, int backward,
                          cudaStream_t s) {
    if (tc_rescal(p) && t->rel_perm && t->rel_seg && t->rel_uniq && t->n_rel_groups)
        return launch_rescal_anchors_tc(a, t->rel_perm, t->rel_seg, (const long long*)t->rel_uniq, (const long long*)t->n_rel_groups,
                                        p->n_rel, anchors, backward, tcw, tc_rescal_bytes(p, backward), s);
    return launch_rescal_anchors(p, t, anchors, s);
}

int kge_score_forward(const kge_problem* p, const kge_tensors* t, float* pos_score, float* neg_score, void* workspace,
                      size_t workspace_bytes, kge_stream_t stream) {
    const char* fn = "kge_score_forward";
    int rc = check_problem(fn, p, t, true);
    if (rc) return rc;
    if (p->batch == 0) return 0;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    KGE_REQUIRE_PTR(pos_score, "pos_score");
    if (p->neg_mode != KGE_NEG_NONE) KGE_REQUIRE_PTR(neg_score, "neg_score");
    const size_t need = kge_score_workspace_bytes(p, 0);
    if (need > 256 || p->reserved) {
        KGE_REQUIRE_PTR(workspace, "workspace");
        if (workspace_bytes < need) { set_error("%s: workspace needs %zu bytes, got %zu", fn, need, workspace_bytes); return KGE_E_WORKSPACE; }
    }
    kge_tensors ts;
    if (p->reserved & KGE_FLAG_CHECK_IDS) {
        if (p->n_ent <= 0 || p->n_rel <= 0) { set_error("%s: KGE_FLAG_CHECK_IDS needs n_ent and n_rel", fn); return KGE_E_SHAPE; }
        rc = sanitise_ids(p, t, &ts, static_cast<char*>(workspace) + score_scratch_bytes(p, 0), s);
        if (rc) return rc;
        t = &ts;
    }
    ScoreArgs a = score_args(p, t);
    a.pos = pos_score; a.negs = neg_score;
    if (tc_transr(p))
        return launch_transr_forward_tc(a, t->rel_perm, t->rel_seg, (const long long*)t->rel_uniq, (const long long*)t->n_rel_groups,
                                        p->n_rel, workspace, workspace_bytes, s);
    if (p->model == KGE_TRANSR) return launch_transr_forward(p, t, pos_score, neg_score, s);
    if (p->model == KGE_RESCAL) {
        float* anchors = static_cast<float*>(workspace);
        rc = rescal_anchors(p, t, a, anchors, static_cast<char*>(workspace) + rows_bytes(p) + tc_bytes(p, 0), 0, s);
        if (rc) return rc;
        a.anchors = anchors;
    }
    if (p->neg_mode != KGE_NEG_CHUNK_SHARED) return launch_triple_forward(a, s);
    ScoreArgs apos = a;
    apos.n_neg = 0; apos.n_neg_head = 0;
    rc = launch_triple_forward(apos, s);
    if (rc) return rc;
    if (tc_forward(p)) {
        char* tcw = static_cast<char*>(workspace) + (p->model == KGE_RESCAL ? rows_bytes(p) : 0);
        return launch_pair_forward_tc(a, p->n_neg_head > 0 ? 1 : 0, tcw, tc_bytes(p, 0), s);
    }
    return launch_pair_forward(a, p->n_neg_head > 0 ? 1 : 0, s);
}

int kge_score_backward(const kge_problem* p, const kge_tensors* t, const float* pos_score, const float* neg_score,
                       const float* dpos, const float* dneg, const kge_grads* g, void* workspace, size_t workspace_bytes,
                       kge_stream_t stream) {
    const char* fn = "kge_score_backward";
    int rc = check_problem(fn, p, t, true);
    if (rc) return rc;
    if (p->batch == 0) return 0;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!g) { set_error("%s: grads is NULL", fn); return KGE_E_NULL; }
    KGE_REQUIRE_PTR(dpos, "dpos");
    KGE_REQUIRE_ROWS(g->g_head, "g_head", p->dim); KGE_REQUIRE_ROWS(g->g_tail, "g_tail", p->dim);
    if (p->model != KGE_RESCAL) KGE_REQUIRE_ROWS(g->g_rel, "g_rel", p->dim);
    if (p->model == KGE_TRANSH || p->model == KGE_RESCAL || p->model == KGE_TRANSR) KGE_REQUIRE_ROWS(g->g_rel2, "g_rel2", p->dim);
    if (p->model == KGE_TRANSR) { KGE_REQUIRE_PTR(pos_score, "pos_score"); if (p->neg_mode != KGE_NEG_NONE) KGE_REQUIRE_PTR(neg_score, "neg_score"); }
    if (p->neg_mode != KGE_NEG_NONE) {
        KGE_REQUIRE_PTR(dneg, "dneg"); KGE_REQUIRE_ROWS(g->g_neg, "g_neg", p->dim);
        if (p->neg_mode == KGE_NEG_CHUNK_SHARED && p->model == KGE_TRANSE) KGE_REQUIRE_PTR(neg_score, "neg_score");
    }
    (void)pos_score;
    const size_t need = kge_score_workspace_bytes(p, 1);
    KGE_REQUIRE_PTR(workspace, "workspace");
    if (workspace_bytes < need) { set_error("%s: workspace needs %zu bytes, got %zu", fn, need, workspace_bytes); return KGE_E_WORKSPACE; }
    kge_tensors ts;
    if (p->reserved & KGE_FLAG_CHECK_IDS) {
        if (p->n_ent <= 0 || p->n_rel <= 0) { set_error("%s: KGE_FLAG_CHECK_IDS needs n_ent and n_rel", fn); return KGE_E_SHAPE; }
        rc = sanitise_ids(p, t, &ts, static_cast<char*>(workspace) + score_scratch_bytes(p, 1), s);
        if (rc) return rc;
        t = &ts;
    }
    if (tc_transr(p)) {
        ScoreArgs a = score_args(p, t);
        a.pos = const_cast<float*>(pos_score); a.negs = const_cast<float*>(neg_score); a.dpos = dpos; a.dneg = dneg;
        a.g_head = g->g_head; a.g_tail = g->g_tail; a.g_neg = g->g_neg; a.g_rel = g->g_rel;
        return launch_transr_backward_tc(a, g->g_rel2, t->rel_perm, t->rel_seg, (const long long*)t->rel_uniq,
                                         (const long long*)t->n_rel_groups, p->n_rel, workspace, workspace_bytes, s);
    }
    if (p->model == KGE_TRANSR)
        return launch_transr_backward(p, t, pos_score, neg_score, dpos, dneg, g, workspace, s);
    const size_t rb = rows_bytes(p);
    float* ws0 = static_cast<float*>(workspace);                                          // anchors
    float* ws1 = reinterpret_cast<float*>(static_cast<char*>(workspace) + rb);            // chunk-shared anchor gradients
    float* ws2 = reinterpret_cast<float*>(static_cast<char*>(workspace) + 2 * rb);        // RESCAL total anchor gradient

    ScoreArgs a = score_args(p, t);
    a.negs = const_cast<float*>(neg_score);
    a.dpos = dpos; a.dneg = dneg;
    a.g_head = g->g_head; a.g_tail = g->g_tail; a.g_neg = g->g_neg; a.g_rel = g->g_rel; a.g_rel2 = g->g_rel2;
    char* rescal_tcw = static_cast<char*>(workspace) + 3 * rb + tc_bytes(p, 1);
    if (p->model == KGE_RESCAL) {
        rc = rescal_anchors(p, t, a, ws0, rescal_tcw, 1, s);
        if (rc) return rc;
        a.anchors = ws0; a.g_rel = ws2; a.g_rel2 = nullptr;
    }
    if (p->neg_mode == KGE_NEG_CHUNK_SHARED) {
        const bool head = p->n_neg_head > 0;
        const float* ga_scale = nullptr;
        if (tc_backward(p)) {
            rc = launch_pair_backward_tc(a, head ? 1 : 0, ws1, &ga_scale, static_cast<char*>(workspace) + 3 * rb, tc_bytes(p, 1), s);
        } else {
            if (p->model != KGE_RESCAL) {
                rc = launch_anchor(a, head ? nullptr : ws0, head ? ws0 : nullptr, s);
                if (rc) return rc;
            }
            rc = launch_pair_backward(a, ws0, ws1, s);
        }
        if (rc) return rc;
        ScoreArgs b = a;
        b.n_neg = 0; b.n_neg_head = 0;
        if (head) b.ga_head_init = ws1; else b.ga_tail_init = ws1;
        b.ga_init_scale = ga_scale;
        rc = launch_triple_backward(b, s);
    } else {
        rc = launch_triple_backward(a, s);
    }
    if (rc) return rc;
    if (p->model == KGE_RESCAL) {
        if (tc_rescal(p) && t->rel_perm && t->rel_seg && t->rel_uniq && t->n_rel_groups)
            rc = launch_rescal_backward_tc(a, t->rel_perm, t->rel_seg, (const long long*)t->rel_uniq, (const long long*)t->n_rel_groups,
                                           p->n_rel, ws2, g->g_head, g->g_rel2, true, rescal_tcw, tc_rescal_bytes(p, 1), s);
        else
            rc = launch_rescal_backward(p, t, ws2, g->g_head, g->g_rel2, s);
    }
    return rc;
}

size_t kge_score_loss_backward_workspace_bytes(const kge_problem* p) {
    if (p && p->batch > 0 && tc_transr(p))
        return tc_transr_workspace_bytes(p->batch, p->neg_mode == KGE_NEG_NONE ? 0 : p->n_neg, p->dim, p->n_rel, 2) + 256 + check_ids_bytes(p);
    if (!p || p->batch <= 0 || !tc_fused(p)) return 256;
    const size_t dpos_bytes = ((size_t)p->batch * 4 + 255) / 256 * 256;
    return rows_bytes(p) + dpos_bytes + 4096 + tc_pair_workspace_bytes(p->batch, p->chunk, p->n_neg, p->dim, 2, tc_es(p)) + 256 + check_ids_bytes(p);
}

int kge_score_loss_backward(const kge_problem* p, const kge_tensors* t, float neg_weight, float* pos_score, float* loss_out,
                            const kge_grads* g, void* workspace, size_t workspace_bytes, kge_stream_t stream) {
    const char* fn = "kge_score_loss_backward";
    int rc = check_problem(fn, p, t, true);
    if (rc) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (tc_transr(p)) {
        // TransR over bf16 tables: forward, loss and backward share ONE pack of the difference rows
        KGE_REQUIRE_PTR(loss_out, "loss_out");
        if (p->batch == 0) return cuda_status(cudaMemsetAsync(loss_out, 0, 4, s), "kge_score_loss_backward(batch=0)");
        if (!g) { set_error("%s: grads is NULL", fn); return KGE_E_NULL; }
        KGE_REQUIRE_PTR(pos_score, "pos_score");
        KGE_REQUIRE_ROWS(g->g_head, "g_head", p->dim); KGE_REQUIRE_ROWS(g->g_tail, "g_tail", p->dim);
        KGE_REQUIRE_ROWS(g->g_rel, "g_rel", p->dim); KGE_REQUIRE_ROWS(g->g_rel2, "g_rel2", p->dim);
        if (p->neg_mode != KGE_NEG_NONE) KGE_REQUIRE_ROWS(g->g_neg, "g_neg", p->dim);
        const size_t need = kge_score_loss_backward_workspace_bytes(p);
        KGE_REQUIRE_PTR(workspace, "workspace");
        if (workspace_bytes < need) { set_error("%s: workspace needs %zu bytes, got %zu", fn, need, workspace_bytes); return KGE_E_WORKSPACE; }
        kge_tensors ts;
        if (p->reserved & KGE_FLAG_CHECK_IDS) {
            if (p->n_ent <= 0 || p->n_rel <= 0) { set_error("%s: KGE_FLAG_CHECK_IDS needs n_ent and n_rel", fn); return KGE_E_SHAPE; }
            rc = sanitise_ids(p, t, &ts, static_cast<char*>(workspace) + need - check_ids_bytes(p), s);
            if (rc) return rc;
            t = &ts;
        }
        ScoreArgs a = score_args(p, t);
        a.pos = pos_score;
        a.g_head = g->g_head; a.g_tail = g->g_tail; a.g_neg = g->g_neg; a.g_rel = g->g_rel;
        return launch_transr_loss_backward_tc(a, neg_weight, loss_out, g->g_rel2, t->rel_perm, t->rel_seg, (const long long*)t->rel_uniq,
                                              (const long long*)t->n_rel_groups, p->n_rel, workspace, workspace_bytes, s);
    }
    if (!tc_fused(p)) {
        set_error("%s: needs precision KGE_PREC_TENSOR and either chunk-shared negatives with dim %% 4 == 0 and TransE, DistMult or "
                  "ComplEx, or TransR over bf16 tables; use kge_score_forward / kge_logistic_loss / kge_score_backward otherwise", fn);
        return KGE_E_UNSUPPORTED;
    }
    KGE_REQUIRE_PTR(loss_out, "loss_out");
    if (p->batch == 0) return cuda_status(cudaMemsetAsync(loss_out, 0, 4, s), "kge_score_loss_backward(batch=0)");
    if (!g) { set_error("%s: grads is NULL", fn); return KGE_E_NULL; }
    KGE_REQUIRE_PTR(pos_score, "pos_score");
    KGE_REQUIRE_PTR(g->g_head, "g_head"); KGE_REQUIRE_PTR(g->g_tail, "g_tail"); KGE_REQUIRE_PTR(g->g_rel, "g_rel");
    KGE_REQUIRE_PTR(g->g_neg, "g_neg");
    const size_t need = kge_score_loss_backward_workspace_bytes(p);
    KGE_REQUIRE_PTR(workspace, "workspace");
    if (workspace_bytes < need) { set_error("%s: workspace needs %zu bytes, got %zu", fn, need, workspace_bytes); return KGE_E_WORKSPACE; }
    const size_t rb = rows_bytes(p), dpos_bytes = ((size_t)p->batch * 4 + 255) / 256 * 256;
    char* wsb = static_cast<char*>(workspace);
    float* ga = reinterpret_cast<float*>(wsb);                       // anchor gradients summed over the chunk's negatives
    float* pos_loss = reinterpret_cast<float*>(wsb + rb);            // loss term of every positive
    char* tcw = wsb + rb + dpos_bytes + 4096;

    cudaError_t ce = cudaMemsetAsync(loss_out, 0, 4, s);
    if (ce != cudaSuccess) return cuda_status(ce, "kge_score_loss_backward(loss)");
    kge_tensors ts;
    if (p->reserved & KGE_FLAG_CHECK_IDS) {
        if (p->n_ent <= 0 || p->n_rel <= 0) { set_error("%s: KGE_FLAG_CHECK_IDS needs n_ent and n_rel", fn); return KGE_E_SHAPE; }
        rc = sanitise_ids(p, t, &ts, wsb + need - check_ids_bytes(p), s);
        if (rc) return rc;
        t = &ts;
    }
    ScoreArgs a = score_args(p, t);
    a.pos = pos_score;
    a.g_head = g->g_head; a.g_tail = g->g_tail; a.g_neg = g->g_neg; a.g_rel = g->g_rel; a.g_rel2 = g->g_rel2;
    const bool head = p->n_neg_head > 0;
    const float* ga_scale = nullptr;
    rc = launch_pair_loss_backward_tc(a, head ? 1 : 0, neg_weight, loss_out, ga, &ga_scale, tcw,
                                      tc_pair_workspace_bytes(p->batch, p->chunk, p->n_neg, p->dim, 2, tc_es(p)), s);
    if (rc) return rc;
    // positives: score, loss term, dS and their gradient rows in the per-triple kernel, on top of the anchor gradients
    ScoreArgs b = a;
    b.pos_loss = pos_loss; b.n_neg = 0; b.n_neg_head = 0;
    if (head) b.ga_head_init = ga; else b.ga_tail_init = ga;
    b.ga_init_scale = ga_scale;
    rc = launch_triple_backward(b, s);
    if (rc) return rc;
    return launch_loss_add(pos_loss, p->batch, loss_out, s);
}

int kge_logistic_loss(const float* pos, int64_t n_pos, const float* neg, int64_t n_neg_total, float neg_weight,
                      float* dpos, float* dneg, float* loss_out, void* workspace, size_t workspace_bytes,
                      kge_stream_t stream) {
    const char* fn = "kge_logistic_loss";
    if (n_pos < 0 || n_neg_total < 0) { set_error("%s: negative size", fn); return KGE_E_SHAPE; }
    KGE_REQUIRE_PTR(loss_out, "loss_out"); KGE_REQUIRE_PTR(workspace, "workspace");
    if (n_pos > 0) { KGE_REQUIRE_PTR(pos, "pos"); KGE_REQUIRE_PTR(dpos, "dpos"); }
    if (n_neg_total > 0) { KGE_REQUIRE_PTR(neg, "neg"); KGE_REQUIRE_PTR(dneg, "dneg"); }
    return launch_logistic_loss(pos, n_pos, neg, n_neg_total, neg_weight, dpos, dneg, loss_out, workspace, workspace_bytes,
                                reinterpret_cast<cudaStream_t>(stream));
}

int kge_profile_gemm(int32_t enable) { gemm_profile_enable(enable); return 0; }
int kge_profile_gemm_read(double* ms, int64_t* launches, double* flops) {
    long long n = 0;
    int rc = gemm_profile_read(ms, &n, flops);
    if (launches) *launches = n;
    return rc;
}

int kge_owner_counts(const int64_t* uniq, const int64_t* n_unique, int64_t n_max, int64_t rows_per_rank, int32_t world,
                     int64_t* counts, kge_stream_t stream) {
    const char* fn = "kge_owner_counts";
    if (world <= 0 || rows_per_rank <= 0) { set_error("%s: world and rows_per_rank must be positive", fn); return KGE_E_SHAPE; }
    KGE_REQUIRE_PTR(n_unique, "n_unique"); KGE_REQUIRE_PTR(counts, "counts");
    if (n_max > 0) KGE_REQUIRE_PTR(uniq, "uniq");
    return launch_owner_counts((const long long*)uniq, (const long long*)n_unique, n_max, rows_per_rank, world,
                               (long long*)counts, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
