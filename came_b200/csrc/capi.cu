// C ABI of libcame_b200: descriptor validation, workspace layout, work lists, step scheduling.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <tuple>
#include <vector>

#include "came_b200.h"
#include "launch.h"

using namespace came;

namespace {

constexpr int MAX_GROUPS = 64;
constexpr size_t ALIGN = 256;

thread_local char g_err[512] = "";
// CAME_B200_DISABLE_FAST=1 in the environment routes every tensor through the generic kernels (used by the
// tests to compare the two implementations of a pass against each other).  Read whenever a plan is sized or created,
// so that it must not change between came_b200_workspace_bytes and came_b200_plan_create of one plan.
inline bool disable_fast() { const char* e = getenv("CAME_B200_DISABLE_FAST"); return e && e[0] == '1'; }

// CAME_B200_WAVE_MB=n: run the momentum / apply passes in waves of tensors holding at most n MB of momentum state
const size_t g_wave_bytes = [] { const char* e = getenv("CAME_B200_WAVE_MB"); return e ? (size_t)atol(e) << 20 : (size_t)0; }();

// The fused momentum / apply kernel (fused_ma.cu).  CAME_B200_FUSED_MA=0 runs the three passes as separate launches.
// CAME_B200_MA_LAG: momentum items of later tensors placed between a tensor's last momentum item and its apply items
// (default: 5 per CTA; measured on Llama-7B shapes: 2 per CTA leaves the apply items waiting for the residual
// finalize, from 5 on the kernel runs at the DRAM limit).
// Read when a plan is created.
bool fused_ma_enabled() { const char* e = getenv("CAME_B200_FUSED_MA"); return !(e && e[0] == '0'); }
int env_int(const char* name, int dflt) { const char* e = getenv(name); return e ? atoi(e) : dflt; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

inline size_t align_up(size_t x, size_t a = ALIGN) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

struct LaunchItem {
    int kernel;
    KernelKey key;
    size_t work_off;   // in Work units from the start of the work region
    int n;
    size_t work2_off;  // fused momentum / apply kernel: its F items
    int n2;
};

inline int elem_bytes(int dt) { return dt == CAME_DT_F32 ? 4 : 2; }
inline bool is_nd(const CameTensorDesc& d) { return d.cols != 0 && d.batch > 1; }

// vector-path eligibility of a tensor for each kernel family
struct VecFlags {
    int k;      // gradient reductions: 1 = runs of 8
    int p2;     // momentum pass: 1 = runs of 16 over g and m, 2 = staged fast path (tile / fp32 layout: cols % 64 == 0)
    int p3;     // apply pass: same over m and p
    int flat;   // flat apply: 1 = runs of 8 over g, m, p
    bool operator==(const VecFlags& o) const { return k == o.k && p2 == o.p2 && p3 == o.p3 && flat == o.flat; }
};

VecFlags vec_flags(const CameTensorDesc& d) {
    VecFlags v{0, 0, 0, 0};
    if (d.cols == 0 || is_nd(d)) return v;      // 1-D and N-D tensors have kernels of their own
    const bool c8 = d.cols % 8 == 0, c16 = d.cols % 16 == 0;
    // staged fast path of the momentum / apply passes: both or neither, as they share the tile geometry
    const bool all_aligned = aligned16(d.g) && aligned16(d.m) && aligned16(d.p);
    const bool fast = !disable_fast() && all_aligned &&
                      ((d.mode == CAME_MODE_TILE8 && d.cols % 64 == 0) ||
                       (d.mode == CAME_MODE_FP32 && d.cols % 64 == 0) ||
                       (d.mode == CAME_MODE_FLAT8 && d.cols % 256 == 0 && d.g_dtype == d.p_dtype));
    v.k = c8 && aligned16(d.g);
    // (tensors with the 1e-30 clamps take the fused first pass too: its closed form for the clip sum holds whenever no
    // clamp binds, which the finalize checks; if one does, the two-pass sum runs for that tensor)
    if (v.k && !disable_fast() && fused_sq_eligible(d.cols, elem_bytes(d.g_dtype))) v.k = 2;
    v.p2 = (c16 && aligned16(d.g) && aligned16(d.m)) ? (fast ? 2 : 1) : 0;
    v.p3 = (c16 && aligned16(d.p) && aligned16(d.m)) ? (fast ? 2 : 1) : 0;
    v.flat = c8 && aligned16(d.g) && aligned16(d.p) && (reinterpret_cast<uintptr_t>(d.m) & 7u) == 0;
    if (fast && d.mode == CAME_MODE_FLAT8) v.flat = 2;
    return v;
}

struct Geometry {
    int64_t R, C;
    int tiles_r, tiles_c, ptiles_r, ptiles_c, nbR, nbC;
    int64_t flat_chunks;
    size_t floats;   // scratch floats of this tensor
};

Geometry geometry(const CameTensorDesc& d) {
    Geometry g{};
    g.R = d.rows;
    g.C = d.cols;
    g.nbR = (int)cdiv(g.R, QBLOCK);
    if (d.cols == 0) {
        g.floats = align_up((size_t)g.nbR + 1, 4);
        return g;
    }
    if (is_nd(d)) {      // nbR / nbC: blocks of the flattened row / column vectors; flat_chunks: flat blocks of 256 elements
        g.nbR = (int)cdiv((int64_t)d.batch * g.R, QBLOCK);
        g.nbC = (int)cdiv((int64_t)d.batch * g.C, QBLOCK);
        g.flat_chunks = cdiv((int64_t)d.batch * g.R * g.C, QBLOCK);
        return g;
    }
    g.nbC = (int)cdiv(g.C, QBLOCK);
    g.tiles_r = (int)cdiv(g.R, K_TR);
    g.tiles_c = (int)cdiv(g.C, K_TC);
    const bool wide = vec_flags(d).p2 == 2;
    g.ptiles_r = (int)cdiv(g.R, wide ? W_TR : P_TR);
    g.ptiles_c = (int)cdiv(g.C, wide ? W_TC : P_TC);
    g.flat_chunks = cdiv(cdiv(g.R * g.C, QBLOCK), FLAT_BLOCKS_PER_CTA);
    return g;
}

// carve the per-tensor float scratch; base == nullptr computes sizes only
size_t carve(const CameTensorDesc& d, const Geometry& g, float* base, Scratch* out) {
    size_t off = 0;
    auto take = [&](size_t n) -> float* {
        float* p = base ? base + off : nullptr;
        off += align_up(n, 4);
        return p;
    };
    Scratch s{};
    s.nbR = g.nbR;
    if (d.cols == 0) {
        s.spart = take((size_t)g.nbR + 1);      // block partials of sum u^2, then their sum
    } else if (is_nd(d)) {
        const size_t B = d.batch;
        s.nbC = g.nbC;
        s.vr = take(B * (size_t)g.R); s.vc = take(B * (size_t)g.C);
        s.Rr = take(B * (size_t)g.R); s.Rc = take(B * (size_t)g.C);
        s.rowblk = take(B); s.rowblk2 = take(B);      // per matrix: guarded mean of the fresh row vectors
        s.scal = take(4);
        s.spart = take((size_t)g.flat_chunks);
    } else {
        s.nbC = g.nbC;
        s.tiles_r = g.tiles_r; s.tiles_c = g.tiles_c;
        s.ptiles_r = g.ptiles_r; s.ptiles_c = g.ptiles_c;
        s.vr = take((size_t)g.R); s.vc = take((size_t)g.C);
        s.Rr = take((size_t)g.R); s.Rc = take((size_t)g.C);
        s.rowblk = take((size_t)g.nbR); s.rowblk2 = take((size_t)g.nbR);
        s.scal = take(4);
        s.rowpart = take((size_t)std::max(g.tiles_c, g.ptiles_c) * (size_t)g.R);
        s.sq_col_parts = g.tiles_r;
        int fa_groups = 1, fa_ng = 1, fa_rb = 1, fa_slot_kb = 64;
        if (vec_flags(d).k == 2) {
            fused_sq_geometry(g.C, elem_bytes(d.g_dtype), &fa_groups, &fa_ng, &fa_rb, &fa_slot_kb);
            s.sq_col_parts = g.tiles_r * fa_groups;
        }
        s.colpart = take((size_t)std::max(s.sq_col_parts, g.ptiles_r) * (size_t)g.C);
        s.spart = take(std::max((size_t)g.tiles_r * (size_t)g.tiles_c, (size_t)g.nbC));
        s.fac = (d.mode == CAME_MODE_FLAT8 && vec_flags(d).flat != 2) ? take(2 * (size_t)(g.R + g.C)) : nullptr;
        if (vec_flags(d).p2 == 2) {
            s.res_eps_deferred = 1;
            s.mfac = take((size_t)g.R);
            s.mfac_c = take((size_t)g.C);
            s.mfac_c2 = d.mode == CAME_MODE_FLAT8 ? take((size_t)g.C) : nullptr;
        }
        if (vec_flags(d).k == 2) {
            s.fused_a = 1;
            s.fa_rb = fa_rb;
            s.tpart = take((size_t)s.sq_col_parts * (size_t)g.C);
        }
    }
    if (out) *out = s;
    return off;
}

int validate(const CameTensorDesc& d, int i) {
    if (!d.p || !d.g || !d.m) return fail(CAME_E_INVALID, "tensor %d: p, g and m must be non-null", i);
    if (d.rows <= 0 || d.cols < 0) return fail(CAME_E_INVALID, "tensor %d: bad shape [%lld, %lld]", i, (long long)d.rows, (long long)d.cols);
    if (d.rows > 0x7fffffffLL || d.cols > 0x7fffffffLL) return fail(CAME_E_UNSUPPORTED, "tensor %d: dimension above 2^31-1", i);
    if (d.mode < CAME_MODE_FP32 || d.mode > CAME_MODE_FLAT8) return fail(CAME_E_INVALID, "tensor %d: bad mode %d", i, d.mode);
    if (d.p_dtype < CAME_DT_F32 || d.p_dtype > CAME_DT_BF16 || d.g_dtype < CAME_DT_F32 || d.g_dtype > CAME_DT_BF16)
        return fail(CAME_E_INVALID, "tensor %d: bad dtype", i);
    if (d.group < 0 || d.group >= MAX_GROUPS) return fail(CAME_E_INVALID, "tensor %d: group %d outside [0, %d)", i, d.group, MAX_GROUPS);
    const bool quant = d.mode != CAME_MODE_FP32;
    if (quant && !d.m_absmax) return fail(CAME_E_INVALID, "tensor %d: 8-bit exp_avg needs m_absmax", i);
    if (!d.sq_row || (quant && !d.sq_row_absmax)) return fail(CAME_E_INVALID, "tensor %d: missing exp_avg_sq state", i);
    if (d.cols == 0) {
        if (d.mode == CAME_MODE_TILE8) return fail(CAME_E_INVALID, "tensor %d: 1-D tensors use CAME_MODE_FLAT8 or CAME_MODE_FP32", i);
        return CAME_OK;
    }
    if (!d.sq_col || !d.res_row || !d.res_col) return fail(CAME_E_INVALID, "tensor %d: missing factored state", i);
    if (d.batch > 1) {
        if (d.mode == CAME_MODE_TILE8) return fail(CAME_E_INVALID, "tensor %d: the tile layout holds single matrices (batch %u)", i, d.batch);
        if ((double)d.batch * (double)d.rows * (double)d.cols > 9.0e18) return fail(CAME_E_UNSUPPORTED, "tensor %d: too many elements", i);
        if (cdiv((int64_t)d.batch * d.rows * d.cols, QBLOCK) > 0x7fffffffLL) return fail(CAME_E_UNSUPPORTED, "tensor %d: too many elements", i);
    }
    if (quant && (!d.sq_col_absmax || !d.res_row_absmax || !d.res_col_absmax))
        return fail(CAME_E_INVALID, "tensor %d: missing factored absmax", i);
    return CAME_OK;
}

struct Layout {
    size_t off_descs, off_scr, off_hyp, off_status, off_sync, off_work, off_float, total;
    size_t n_work;
};

size_t count_work(const CameTensorDesc* descs, int n) {
    size_t w = 0;
    for (int i = 0; i < n; ++i) {
        const Geometry g = geometry(descs[i]);
        if (descs[i].cols == 0) {
            w += 2 * (size_t)g.nbR + 1;      // partial, apply; one reduce CTA
            continue;
        }
        if (is_nd(descs[i])) {      // two vector passes, two mean passes (one item per matrix), S, two element passes
            w += 2 * (size_t)(g.nbR + g.nbC) + 2 * (size_t)descs[i].batch + 1 + 2 * (size_t)g.flat_chunks;
            continue;
        }
        w += 2 * (size_t)g.tiles_r * g.tiles_c;      // sq_partials, sumsq
        w += 2 * (size_t)(g.nbR + g.nbC);            // two vector finalizes
        // clip finalize: one CTA per S_FIN_CHUNK entries of the factor vectors on the staged momentum path
        w += vec_flags(descs[i]).p2 == 2 ? (size_t)std::max<int64_t>(1, cdiv(g.R + g.C, S_FIN_CHUNK)) : (size_t)1;
        w += (size_t)g.ptiles_r * g.ptiles_c;        // moment
        if (descs[i].mode == CAME_MODE_FLAT8)
            w += (size_t)(g.nbR + g.nbC) + std::max((size_t)g.flat_chunks, (size_t)g.ptiles_r * g.ptiles_c);
        else w += (size_t)g.ptiles_r * g.ptiles_c;   // apply
    }
    return w;
}

Layout layout(const CameTensorDesc* descs, int n) {
    Layout L{};
    size_t off = 0;
    L.off_descs = off; off = align_up(off + (size_t)n * sizeof(CameTensorDesc));
    L.off_scr = off;   off = align_up(off + (size_t)n * sizeof(Scratch));
    L.off_hyp = off;   off = align_up(off + (size_t)MAX_GROUPS * sizeof(CameHyper));
    L.off_status = off; off = align_up(off + sizeof(int));
    L.off_sync = off;  off = align_up(off + (2 * (size_t)n + 12) * sizeof(int));   // fused kernel: per-tensor item counters, list cursors
    L.n_work = count_work(descs, n);
    L.off_work = off;  off = align_up(off + L.n_work * sizeof(Work));
    L.off_float = off;
    size_t fl = 0;
    for (int i = 0; i < n; ++i) fl += align_up(carve(descs[i], geometry(descs[i]), nullptr, nullptr), 64);
    off = align_up(off + fl * sizeof(float));
    L.total = off;
    return L;
}

}  // namespace

namespace came {
// lets other translation units leave a message for came_b200_last_error()
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
int persistent_grid_limit() {
    static int limit = 0;
    if (limit == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        int reserved = 0;
        if (const char* e = getenv("CAME_B200_RESERVED_SMS")) reserved = atoi(e);
        if (reserved < 0) reserved = 0;
        if (reserved > sms - 1) reserved = sms - 1;
        limit = sms - reserved;
    }
    return limit;
}
}  // namespace came

struct came_plan {
    int n_tensors = 0;
    std::vector<CameTensorDesc> descs;
    std::vector<VecFlags> vflags;
    char* ws = nullptr;
    Layout L{};
    std::vector<LaunchItem> launches;
    int last_launches = 0;
    bool has_fused_ma = false;
    std::vector<char> fused;       // per tensor: stepped by the fused momentum / apply kernel
    int n_push = 0;                // push mode: peers that receive every parameter the fused kernel updates
    long long push_delta[MAX_PUSH_PEERS] = {};
    uintptr_t push_lo = 0, push_hi = 0;      // the local buffer the pushed parameters must lie in
    bool timing = false;
    struct Timed { int kernel; cudaEvent_t t0, t1; };
    std::vector<Timed> timed;
    // page-locked copy of the hyper-parameter records: the source of the upload when a step is captured into a
    // CUDA graph (the graph's copy node reads it again at every replay)
    CameHyper* graph_hyp = nullptr;
    int graph_groups = 0;
    ~came_plan() {
        for (auto& t : timed) { cudaEventDestroy(t.t0); cudaEventDestroy(t.t1); }
        if (graph_hyp) cudaFreeHost(graph_hyp);
    }
};

static int check_hypers(const char* who, const came_plan* plan, const CameHyper* hypers, int n_groups) {
    if (!plan || !hypers) return fail(CAME_E_INVALID, "%s: null argument", who);
    if (n_groups <= 0 || n_groups > MAX_GROUPS) return fail(CAME_E_INVALID, "%s: n_groups %d outside [1, %d]", who, n_groups, MAX_GROUPS);
    for (const auto& d : plan->descs)
        if (d.group >= n_groups) return fail(CAME_E_INVALID, "%s: a tensor refers to group %d, %d given", who, d.group, n_groups);
    for (int i = 0; i < n_groups; ++i) {
        if (!(hypers[i].clip_threshold > 0.0f)) return fail(CAME_E_INVALID, "%s: group %d: clip_threshold must be > 0", who, i);
    }
    return CAME_OK;
}

// (the buffer is allocated when the plan is created: page-locking memory is not allowed while a stream is captured)
// grad_scale == 0 (a zero-initialised record) means "no scaling"
static void normalise_hypers(CameHyper* h, int n_groups) {
    for (int i = 0; i < n_groups; ++i)
        if (h[i].grad_scale == 0.0f) h[i].grad_scale = 1.0f;
}

static int stage_graph_hypers(const char* who, came_plan* plan, const CameHyper* hypers, int n_groups) {
    if (!plan->graph_hyp) return fail(CAME_E_CUDA, "%s: the plan has no page-locked hyper-parameter buffer", who);
    std::memcpy(plan->graph_hyp, hypers, (size_t)n_groups * sizeof(CameHyper));
    normalise_hypers(plan->graph_hyp, n_groups);
    plan->graph_groups = n_groups;
    return CAME_OK;
}

extern "C" {

int came_b200_version(void) { return CAME_B200_VERSION; }
const char* came_b200_last_error(void) { return g_err; }

int came_b200_quantize_blockwise(const float* src, void* q, float* absmax, int64_t n, int is_signed, came_stream_t stream) {
    if (!q || !absmax || n < 0 || (n > 0 && !src)) return fail(CAME_E_INVALID, "quantize_blockwise: null pointer or negative size");
    const cudaError_t e = launch_quantize_blockwise(src, q, absmax, n, is_signed != 0, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "quantize_blockwise: %s", cudaGetErrorString(e));
}

int came_b200_dequantize_blockwise(const void* q, const float* absmax, float* dst, int64_t n, int is_signed, came_stream_t stream) {
    if (n < 0 || (n > 0 && (!q || !absmax || !dst))) return fail(CAME_E_INVALID, "dequantize_blockwise: null pointer or negative size");
    const cudaError_t e = launch_dequantize_blockwise(q, absmax, dst, n, is_signed != 0, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "dequantize_blockwise: %s", cudaGetErrorString(e));
}

int came_b200_quantize_tile16(const float* src, int8_t* q, float* absmax, int64_t rows, int64_t cols, came_stream_t stream) {
    if (!src || !q || !absmax || rows <= 0 || cols <= 0) return fail(CAME_E_INVALID, "quantize_tile16: bad argument");
    const cudaError_t e = launch_quantize_tile16(src, q, absmax, rows, cols, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "quantize_tile16: %s", cudaGetErrorString(e));
}

int came_b200_dequantize_tile16(const int8_t* q, const float* absmax, float* dst, int64_t rows, int64_t cols, came_stream_t stream) {
    if (!dst || !q || !absmax || rows <= 0 || cols <= 0) return fail(CAME_E_INVALID, "dequantize_tile16: bad argument");
    const cudaError_t e = launch_dequantize_tile16(q, absmax, dst, rows, cols, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "dequantize_tile16: %s", cudaGetErrorString(e));
}

size_t came_b200_workspace_bytes(const CameTensorDesc* descs, int n_tensors) {
    if (!descs || n_tensors <= 0) return 0;
    for (int i = 0; i < n_tensors; ++i)
        if (validate(descs[i], i) != CAME_OK) return 0;
    return layout(descs, n_tensors).total;
}

int came_b200_plan_create(const CameTensorDesc* descs, int n_tensors, void* workspace, size_t workspace_bytes,
                          came_stream_t stream, came_plan_t** out) {
    if (!out) return fail(CAME_E_INVALID, "plan_create: out is null");
    *out = nullptr;
    if (!descs || n_tensors <= 0) return fail(CAME_E_INVALID, "plan_create: no tensors");
    for (int i = 0; i < n_tensors; ++i) {
        const int rc = validate(descs[i], i);
        if (rc != CAME_OK) return rc;
    }
    const Layout L = layout(descs, n_tensors);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % ALIGN) != 0)
        return fail(CAME_E_WORKSPACE, "plan_create: workspace must be non-null and %zu-byte aligned", ALIGN);
    if (workspace_bytes < L.total)
        return fail(CAME_E_WORKSPACE, "plan_create: workspace of %zu bytes, %zu needed", workspace_bytes, L.total);

    came_plan* plan = new (std::nothrow) came_plan();
    if (!plan) return fail(CAME_E_INVALID, "plan_create: out of host memory");
    plan->n_tensors = n_tensors;
    plan->descs.assign(descs, descs + n_tensors);
    plan->ws = static_cast<char*>(workspace);
    plan->L = L;
    plan->vflags.resize(n_tensors);

    std::vector<Scratch> scr(n_tensors);
    std::vector<Geometry> geo(n_tensors);
    float* fbase = reinterpret_cast<float*>(plan->ws + L.off_float);
    size_t foff = 0;
    for (int i = 0; i < n_tensors; ++i) {
        geo[i] = geometry(descs[i]);
        plan->vflags[i] = vec_flags(descs[i]);
        foff += align_up(carve(descs[i], geo[i], fbase + foff, &scr[i]), 64);
    }

    // work lists, one per (kernel, template key), in execution order
    std::vector<Work> work;
    work.reserve(L.n_work);
    using Key = std::tuple<int, int, int, int>;   // g, p, mode, vec
    auto build = [&](int kernel, auto select, auto keyof, auto count) {
        std::map<Key, std::vector<int>> groups;
        for (int i = 0; i < n_tensors; ++i)
            if (select(i)) groups[keyof(i)].push_back(i);
        for (auto& kv : groups) {
            LaunchItem it{};
            it.kernel = kernel;
            it.key = KernelKey{std::get<0>(kv.first), std::get<1>(kv.first), std::get<2>(kv.first), std::get<3>(kv.first)};
            it.work_off = work.size();
            for (int i : kv.second) {
                const int64_t c = count(i);
                for (int64_t t = 0; t < c; ++t) work.push_back(Work{i, (int32_t)t});
            }
            it.n = (int)(work.size() - it.work_off);
            if (it.n > 0) plan->launches.push_back(it);
        }
    };
    const CameTensorDesc* D = descs;
    auto is1d = [&](int i) { return D[i].cols == 0; };
    auto is2d = [&](int i) { return D[i].cols != 0 && !is_nd(D[i]); };
    auto isnd = [&](int i) { return is_nd(D[i]); };
    auto isflat = [&](int i) { return is2d(i) && D[i].mode == CAME_MODE_FLAT8; };
    auto notflat = [&](int i) { return is2d(i) && D[i].mode != CAME_MODE_FLAT8; };
    auto nokey = [&](int) { return Key{0, 0, 0, 0}; };
    const auto& vf = plan->vflags;

    build(KID_NF_PARTIAL, is1d, [&](int i) { return Key{D[i].g_dtype, 0, 0, 0}; }, [&](int i) { return (int64_t)geo[i].nbR; });
    build(KID_NF_REDUCE, is1d, nokey, [&](int) { return (int64_t)1; });
    build(KID_NF_APPLY, is1d, [&](int i) { return Key{D[i].g_dtype, D[i].p_dtype, 0, 0}; }, [&](int i) { return (int64_t)geo[i].nbR; });
    // tensors of more than two dimensions
    auto nvec = [&](int i) { return (int64_t)geo[i].nbR + geo[i].nbC; };
    auto nmat = [&](int i) { return (int64_t)D[i].batch; };
    auto nblk = [&](int i) { return geo[i].flat_chunks; };
    build(KID_ND_SQ, isnd, nokey, nvec);
    build(KID_ND_MEAN, isnd, nokey, nmat);
    build(KID_ND_SUMSQ, isnd, nokey, nblk);
    build(KID_ND_S, isnd, nokey, [&](int) { return (int64_t)1; });
    build(KID_ND_RES, isnd, nokey, nvec);
    build(KID_ND_RESMEAN, isnd, nokey, nmat);
    build(KID_ND_APPLY, isnd, nokey, nblk);
    auto fusedA = [&](int i) { return is2d(i) && vf[i].k == 2; };
    auto twopass = [&](int i) { return is2d(i) && vf[i].k != 2; };
    auto fused_code = [&](int i) {      // column groups per thread | row sets << 4 | ring slot KB << 8
        int groups, ng, rb, slot_kb;
        fused_sq_geometry(D[i].cols, elem_bytes(D[i].g_dtype), &groups, &ng, &rb, &slot_kb);
        return ng | (groups << 4) | (slot_kb << 8);
    };
    build(KID_SQ_PARTIALS, fusedA, [&](int i) { return Key{D[i].g_dtype, 0, fused_code(i), 2}; },
          [&](int i) { return (int64_t)geo[i].tiles_r; });
    build(KID_SQ_PARTIALS, twopass, [&](int i) { return Key{D[i].g_dtype, 0, 0, vf[i].k}; },
          [&](int i) { return (int64_t)geo[i].tiles_r * geo[i].tiles_c; });
    build(KID_SQ_FINALIZE, is2d, nokey, [&](int i) { return (int64_t)geo[i].nbR + geo[i].nbC; });
    // (also for fused-first-pass tensors that carry the clamps: those CTAs return at once unless a clamp binds)
    auto needs_sumsq = [&](int i) { return twopass(i) || (fusedA(i) && (D[i].flags & CAME_F_SQ_CLAMP)); };
    build(KID_SUMSQ, needs_sumsq, [&](int i) { return Key{D[i].g_dtype, 0, 0, vf[i].k >= 1 ? 1 : 0}; },
          [&](int i) { return (int64_t)geo[i].tiles_r * geo[i].tiles_c; });
    // one CTA per tensor for the clip scalar; tensors of the staged momentum pass get one CTA per 2048 entries of
    // their factor vectors (each CTA repeats the cheap scalar part)
    build(KID_S_FINALIZE, is2d, nokey, [&](int i) {
        return vf[i].p2 == 2 ? std::max<int64_t>(1, cdiv(D[i].rows + D[i].cols, S_FIN_CHUNK)) : (int64_t)1;
    });
    // Tensors of the tile layout on the staged path (same element type for g and p) take the fused kernel: their M, F
    // and A items form one list, a tensor's F and A items delayed by `lag` momentum items of later tensors.
    std::vector<char> fused(n_tensors, 0);
    if (!disable_fast() && fused_ma_enabled()) {
        for (int i = 0; i < n_tensors; ++i)
            fused[i] = is2d(i) && D[i].g_dtype == D[i].p_dtype &&
                       ((D[i].mode == CAME_MODE_TILE8 && vf[i].p2 == 2 && vf[i].p3 == 2) ||
                        (D[i].mode == CAME_MODE_FLAT8 && vf[i].p2 == 2 && vf[i].flat == 2));
    }
    {
        const int grid = persistent_grid_limit();
        const size_t lag_a = (size_t)std::max(0, env_int("CAME_B200_MA_LAG", 5 * grid));
        const bool reverse_a = env_int("CAME_B200_MA_REVERSE", 1) != 0;
        const bool interleave = env_int("CAME_B200_MA_INTERLEAVE", 1) != 0;
        for (int dm = 0; dm < 6; ++dm) {
            const int dt = CAME_DT_F32 + dm % 3, md = dm < 3 ? CAME_MODE_TILE8 : CAME_MODE_FLAT8;
            LaunchItem it{};
            it.kernel = KID_MOMENT_APPLY;
            it.key = KernelKey{dt, dt, md, 2};
            it.work_off = work.size();
            struct Burst { size_t release; int tensor; };
            std::vector<Burst> pend;      // apply bursts waiting for their place in the list
            size_t next = 0, emitted = 0;
            auto burst = [&](const Burst& b) {
                const int64_t c = (int64_t)geo[b.tensor].ptiles_r * geo[b.tensor].ptiles_c;
                // the tiles written last are the likeliest to be still in L2: the apply items of a tensor run through its
                // tiles in the reverse order (CAME_B200_MA_REVERSE=0: same order as the momentum items)
                for (int64_t k = 0; k < c; ++k)
                    work.push_back(Work{b.tensor, (int32_t)(((uint32_t)MA_KIND_A << 28) | (uint32_t)(reverse_a ? c - 1 - k : k))});
            };
            // A released burst is dealt out one apply item per momentum item instead of all at once (CAME_B200_MA_INTERLEAVE=0:
            // all at once): DRAM-bound apply items and issue-bound momentum items then share the GPU at all times
            std::vector<Work> trickle;
            size_t tnext = 0;
            auto release = [&](const Burst& b) {
                if (!interleave) { burst(b); return; }
                const size_t before = work.size();
                burst(b);
                trickle.insert(trickle.end(), work.begin() + before, work.end());
                work.resize(before);
            };
            for (int i = 0; i < n_tensors; ++i) {
                if (!fused[i] || D[i].g_dtype != dt || D[i].mode != md) continue;
                const int64_t c = (int64_t)geo[i].ptiles_r * geo[i].ptiles_c;
                for (int64_t k = 0; k < c; ++k) {
                    work.push_back(Work{i, (int32_t)(((uint32_t)MA_KIND_M << 28) | (uint32_t)k)});
                    ++emitted;
                    while (next < pend.size() && pend[next].release <= emitted) release(pend[next++]);
                    if (tnext < trickle.size()) work.push_back(trickle[tnext++]);
                }
                pend.push_back(Burst{emitted + lag_a, i});
            }
            while (next < pend.size()) release(pend[next++]);
            while (tnext < trickle.size()) work.push_back(trickle[tnext++]);
            it.n = (int)(work.size() - it.work_off);
            it.work2_off = work.size();
            for (int i = 0; i < n_tensors; ++i) {
                if (!fused[i] || D[i].g_dtype != dt || D[i].mode != md) continue;
                for (int k = 0; k < geo[i].nbR + geo[i].nbC; ++k) work.push_back(Work{i, k});
            }
            it.n2 = (int)(work.size() - it.work2_off);
            if (it.n > 0) { plan->launches.push_back(it); plan->has_fused_ma = true; }
        }
    }
    plan->fused = fused;
    // The momentum pass, the residual finalize and the apply pass run wave by wave: a wave is a run of consecutive
    // tensors whose momentum state together stays below `wave_bytes`, so that the codes the momentum pass writes are
    // still in L2 when the apply pass reads them back (0: one wave, every pass covers all tensors).
    std::vector<int> wave(n_tensors, 0);
    int n_waves = 1;
    if (g_wave_bytes > 0) {
        size_t acc = 0;
        int w = 0;
        for (int i = 0; i < n_tensors; ++i) {
            if (D[i].cols == 0) { wave[i] = 0; continue; }
            const size_t mb = (size_t)D[i].rows * (size_t)D[i].cols * (D[i].mode == CAME_MODE_FP32 ? 4 : 1);
            if (acc > 0 && acc + mb > g_wave_bytes) { ++w; acc = 0; }
            wave[i] = w;
            acc += mb;
        }
        n_waves = w + 1;
    }
    for (int w = 0; w < n_waves; ++w) {
        auto in2d = [&](int i) { return is2d(i) && wave[i] == w && !fused[i]; };
        auto in_notflat = [&](int i) { return notflat(i) && wave[i] == w && !fused[i]; };
        build(KID_MOMENT, in2d, [&](int i) { return Key{D[i].g_dtype, 0, D[i].mode, vf[i].p2}; },
              [&](int i) { return (int64_t)geo[i].ptiles_r * geo[i].ptiles_c; });
        build(KID_RES_FINALIZE, in2d, nokey, [&](int i) { return (int64_t)geo[i].nbR + geo[i].nbC; });
        build(KID_APPLY, in_notflat, [&](int i) { return Key{0, D[i].p_dtype, D[i].mode, vf[i].p3}; },
              [&](int i) { return (int64_t)geo[i].ptiles_r * geo[i].ptiles_c; });
        auto flat_generic = [&](int i) { return isflat(i) && vf[i].flat != 2 && wave[i] == w; };
        auto flat_staged = [&](int i) { return isflat(i) && vf[i].flat == 2 && wave[i] == w && !fused[i]; };
        build(KID_FACTORS, flat_generic, nokey, [&](int i) { return (int64_t)geo[i].nbR + geo[i].nbC; });
        build(KID_APPLY_FLAT, flat_generic, [&](int i) { return Key{D[i].g_dtype, D[i].p_dtype, 0, vf[i].flat}; },
              [&](int i) { return geo[i].flat_chunks; });
        build(KID_APPLY_FLAT, flat_staged, [&](int i) { return Key{D[i].g_dtype, D[i].p_dtype, 0, 2}; },
              [&](int i) { return (int64_t)geo[i].ptiles_r * geo[i].ptiles_c; });
    }

    if (work.size() > L.n_work) {
        delete plan;
        return fail(CAME_E_INVALID, "plan_create: internal work-list overflow (%zu > %zu)", work.size(), L.n_work);
    }

    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(plan->ws + L.off_descs, plan->descs.data(), (size_t)n_tensors * sizeof(CameTensorDesc),
                                    cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(plan->ws + L.off_scr, scr.data(), (size_t)n_tensors * sizeof(Scratch), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(plan->ws + L.off_status, 0, sizeof(int), st);
    // the scratch starts at zero once (flags in it are reset by the kernels that use them)
    if (e == cudaSuccess) e = cudaMemsetAsync(plan->ws + L.off_float, 0, L.total - L.off_float, st);
    if (e == cudaSuccess && !work.empty())
        e = cudaMemcpyAsync(plan->ws + L.off_work, work.data(), work.size() * sizeof(Work), cudaMemcpyHostToDevice, st);
    // the host vectors above die at return: wait for the copies
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess)
        e = cudaHostAlloc(reinterpret_cast<void**>(&plan->graph_hyp), (size_t)MAX_GROUPS * sizeof(CameHyper), cudaHostAllocDefault);
    if (e != cudaSuccess) {
        delete plan;
        return fail(CAME_E_CUDA, "plan_create: %s", cudaGetErrorString(e));
    }
    *out = plan;
    return CAME_OK;
}

void came_b200_plan_destroy(came_plan_t* plan) { delete plan; }

// push mode: the whole parameter must lie inside the local buffer the peers mirror
static bool param_in_range(uintptr_t buf_lo, uintptr_t buf_hi, const CameTensorDesc& d) {
    const uintptr_t lo = reinterpret_cast<uintptr_t>(d.p);
    const uintptr_t bytes = (uintptr_t)d.rows * (uintptr_t)(d.cols ? d.cols : 1) * (uintptr_t)(d.batch > 1 ? d.batch : 1) *
                            (uintptr_t)elem_bytes(d.p_dtype);
    return lo >= buf_lo && lo + bytes <= buf_hi;
}
static bool pushed_param_in_range(const came_plan& plan, const CameTensorDesc& d) {
    return param_in_range(plan.push_lo, plan.push_hi, d);
}

int came_b200_plan_set_push(came_plan_t* plan, const void* local_base, size_t local_bytes, void* const* peer_bases, int n_peers) {
    if (!plan) return fail(CAME_E_INVALID, "plan_set_push: plan is null");
    if (n_peers == 0) { plan->n_push = 0; return CAME_OK; }
    if (n_peers < 0 || n_peers > MAX_PUSH_PEERS) return fail(CAME_E_INVALID, "plan_set_push: %d peers outside [0, %d]", n_peers, MAX_PUSH_PEERS);
    if (!local_base || !peer_bases || local_bytes == 0) return fail(CAME_E_INVALID, "plan_set_push: null argument");
    const uintptr_t buf_lo = reinterpret_cast<uintptr_t>(local_base), buf_hi = buf_lo + local_bytes;
    if (buf_lo % 16 != 0) return fail(CAME_E_INVALID, "plan_set_push: the local buffer is not 16-byte aligned");
    for (int i = 0; i < plan->n_tensors; ++i)
        if (plan->fused[i] && !param_in_range(buf_lo, buf_hi, plan->descs[i]))
            return fail(CAME_E_INVALID, "plan_set_push: tensor %d does not lie inside the local buffer", i);
    long long delta[MAX_PUSH_PEERS];
    for (int k = 0; k < n_peers; ++k) {
        const uintptr_t pb = reinterpret_cast<uintptr_t>(peer_bases[k]);
        if (!pb || pb % 16 != 0) return fail(CAME_E_INVALID, "plan_set_push: peer buffer %d is null or not 16-byte aligned", k);
        if (pb < buf_hi && pb + local_bytes > buf_lo) return fail(CAME_E_INVALID, "plan_set_push: peer buffer %d overlaps the local one", k);
        delta[k] = (long long)(pb - buf_lo);      // modular: the kernel adds it to a local address
    }
    plan->push_lo = buf_lo; plan->push_hi = buf_hi;
    for (int k = 0; k < n_peers; ++k) plan->push_delta[k] = delta[k];
    plan->n_push = n_peers;
    return CAME_OK;
}

int came_b200_plan_pushed(const came_plan_t* plan, int* flags, int n_tensors) {
    if (!plan || !flags) return fail(CAME_E_INVALID, "plan_pushed: null argument");
    if (n_tensors != plan->n_tensors) return fail(CAME_E_INVALID, "plan_pushed: %d tensors given, plan has %d", n_tensors, plan->n_tensors);
    for (int i = 0; i < n_tensors; ++i) flags[i] = plan->fused[i] ? 1 : 0;
    return CAME_OK;
}

int came_b200_plan_set_pointers(came_plan_t* plan, const void* const* g, void* const* p, int n_tensors, came_stream_t stream) {
    if (!plan) return fail(CAME_E_INVALID, "set_pointers: plan is null");
    if (n_tensors != plan->n_tensors) return fail(CAME_E_INVALID, "set_pointers: %d tensors given, plan has %d", n_tensors, plan->n_tensors);
    if (!g && !p) return CAME_OK;
    std::vector<CameTensorDesc> next = plan->descs;
    for (int i = 0; i < n_tensors; ++i) {
        if (g) next[i].g = g[i];
        if (p) next[i].p = p[i];
        if (!next[i].g || !next[i].p) return fail(CAME_E_INVALID, "set_pointers: tensor %d: null pointer", i);
        if (!(vec_flags(next[i]) == plan->vflags[i]))
            return fail(CAME_E_INVALID, "set_pointers: tensor %d changes 16-byte alignment class; create a new plan", i);
        if (plan->n_push > 0 && plan->fused[i] && !pushed_param_in_range(*plan, next[i]))
            return fail(CAME_E_INVALID, "set_pointers: tensor %d leaves the buffer the push mode was set up for", i);
    }
    plan->descs.swap(next);
    const cudaError_t e = cudaMemcpyAsync(plan->ws + plan->L.off_descs, plan->descs.data(),
                                          (size_t)n_tensors * sizeof(CameTensorDesc), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "set_pointers: %s", cudaGetErrorString(e));
}

int came_b200_plan_set_hyper(came_plan_t* plan, const CameHyper* hypers, int n_groups) {
    int rc = check_hypers("plan_set_hyper", plan, hypers, n_groups);
    if (rc != CAME_OK) return rc;
    if (plan->graph_groups && n_groups != plan->graph_groups)
        return fail(CAME_E_INVALID, "plan_set_hyper: %d groups given, the captured step has %d", n_groups, plan->graph_groups);
    return stage_graph_hypers("plan_set_hyper", plan, hypers, n_groups);
}

int came_b200_step(came_plan_t* plan, const CameHyper* hypers, int n_groups, came_stream_t stream) {
    int rc = check_hypers("step", plan, hypers, n_groups);
    if (rc != CAME_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // While the stream is being captured into a CUDA graph the upload must read memory that outlives the call:
    // the plan's page-locked copy, which came_b200_plan_set_hyper rewrites between replays.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) { cap = cudaStreamCaptureStatusNone; cudaGetLastError(); }
    const bool capturing = cap == cudaStreamCaptureStatusActive;
    std::vector<CameHyper> norm(hypers, hypers + n_groups);      // pageable source: read before the copy call returns
    normalise_hypers(norm.data(), n_groups);
    const CameHyper* src = norm.data();
    if (capturing) {
        rc = stage_graph_hypers("step", plan, hypers, n_groups);
        if (rc != CAME_OK) return rc;
        src = plan->graph_hyp;
    }
    cudaError_t e = cudaMemcpyAsync(plan->ws + plan->L.off_hyp, src, (size_t)n_groups * sizeof(CameHyper),
                                    cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(CAME_E_CUDA, "step: hyper-parameter upload: %s", cudaGetErrorString(e));
    const bool timing = plan->timing && !capturing;      // events are not recorded into a graph
    StepArgs a{reinterpret_cast<const CameTensorDesc*>(plan->ws + plan->L.off_descs),
               reinterpret_cast<const Scratch*>(plan->ws + plan->L.off_scr),
               reinterpret_cast<const CameHyper*>(plan->ws + plan->L.off_hyp),
               reinterpret_cast<int*>(plan->ws + plan->L.off_status), plan->n_push, 0, {}};
    for (int k = 0; k < plan->n_push; ++k) a.push_delta[k] = plan->push_delta[k];
    const Work* wbase = reinterpret_cast<const Work*>(plan->ws + plan->L.off_work);
    int* sync = reinterpret_cast<int*>(plan->ws + plan->L.off_sync);
    if (plan->has_fused_ma) {      // the per-tensor item counters start every step at zero
        e = cudaMemsetAsync(sync, 0, (2 * (size_t)plan->n_tensors + 12) * sizeof(int), st);
        if (e != cudaSuccess) return fail(CAME_E_CUDA, "step: counter reset: %s", cudaGetErrorString(e));
    }
    int launches = 0, fused_launches = 0;
    for (const LaunchItem& it : plan->launches) {
        came_plan::Timed tm{it.kernel, nullptr, nullptr};
        if (timing) {
            if (cudaEventCreate(&tm.t0) != cudaSuccess || cudaEventCreate(&tm.t1) != cudaSuccess)
                return fail(CAME_E_CUDA, "step: cudaEventCreate failed");
            cudaEventRecord(tm.t0, st);
        }
        if (it.kernel == KID_NF_PARTIAL || it.kernel == KID_NF_APPLY || it.kernel == KID_NF_REDUCE)
            e = launch_nonfactored(it.kernel, it.key, a, wbase + it.work_off, it.n, st);
        else if (it.kernel == KID_SQ_PARTIALS && it.key.variant == 2)
            e = launch_fused_sq(it.key, a, wbase + it.work_off, it.n, st);
        else if (it.kernel >= KID_ND_SQ && it.kernel <= KID_ND_APPLY)
            e = launch_nd(it.kernel, a, wbase + it.work_off, it.n, st);
        else if (it.kernel == KID_MOMENT_APPLY)
            e = launch_fused_ma(it.key, a, wbase + it.work_off, it.n, wbase + it.work2_off, it.n2, sync, sync + plan->n_tensors,
                                sync + 2 * plan->n_tensors + 2 * (fused_launches++ % 6), st);      // two list cursors per launch (at most 6)
        else
            e = launch_factored(it.kernel, it.key, a, wbase + it.work_off, it.n, st);
        if (timing) {
            cudaEventRecord(tm.t1, st);
            plan->timed.push_back(tm);
        }
        if (e != cudaSuccess) return fail(CAME_E_CUDA, "step: kernel %d: %s", it.kernel, cudaGetErrorString(e));
        ++launches;
    }
    plan->last_launches = launches;
    return CAME_OK;
}

int came_b200_peer_copy_async(void* dst, const void* src, size_t bytes, int src_device, came_stream_t stream) {
    if (!dst || !src) return fail(CAME_E_INVALID, "peer_copy_async: null pointer");
    if (bytes == 0) return CAME_OK;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(CAME_E_CUDA, "peer_copy_async: %s", cudaGetErrorString(e));
    if (src_device >= 0 && src_device != dev) {
        e = cudaDeviceEnablePeerAccess(src_device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
        if (e != cudaSuccess) return fail(CAME_E_CUDA, "peer_copy_async: enabling access to GPU %d: %s", src_device, cudaGetErrorString(e));
    }
    e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "peer_copy_async: %s", cudaGetErrorString(e));
}

int came_b200_ipc_export(const void* ptr, unsigned char handle[CAME_B200_IPC_HANDLE_BYTES], uint64_t* offset) {
    static_assert(sizeof(cudaIpcMemHandle_t) == CAME_B200_IPC_HANDLE_BYTES, "IPC handle size");
    if (!ptr || !handle || !offset) return fail(CAME_E_INVALID, "ipc_export: null argument");
    // base of the allocation that contains ptr (driver entry point: the runtime has no such query)
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn) return fail(CAME_E_CUDA, "ipc_export: cuMemGetAddressRange is not available");
    unsigned long long base = 0;
    size_t size = 0;
    if (reinterpret_cast<range_fn>(fn)(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0)
        return fail(CAME_E_CUDA, "ipc_export: the pointer is not inside a device allocation");
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base));
    if (e != cudaSuccess) return fail(CAME_E_CUDA, "ipc_export: %s", cudaGetErrorString(e));
    std::memcpy(handle, &h, sizeof(h));
    *offset = (uint64_t)((uintptr_t)ptr - (uintptr_t)base);
    return CAME_OK;
}

int came_b200_ipc_open(const unsigned char handle[CAME_B200_IPC_HANDLE_BYTES], void** base) {
    if (!handle || !base) return fail(CAME_E_INVALID, "ipc_open: null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    const cudaError_t e = cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "ipc_open: %s", cudaGetErrorString(e));
}

int came_b200_ipc_close(void* base) {
    if (!base) return CAME_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(base);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "ipc_close: %s", cudaGetErrorString(e));
}

int came_b200_selftest_bounded_wait(int* device_words, came_stream_t stream) {
    if (!device_words) return fail(CAME_E_INVALID, "selftest_bounded_wait: device_words is null");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(device_words, 0xff, 3 * sizeof(int), st);
    if (e == cudaSuccess) e = cudaMemsetAsync(device_words, 0, sizeof(int), st);
    if (e == cudaSuccess) e = launch_selftest_bounded_wait(device_words, device_words + 1, st);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "selftest_bounded_wait: %s", cudaGetErrorString(e));
}

int came_b200_plan_last_launches(const came_plan_t* plan) { return plan ? plan->last_launches : 0; }

int came_b200_plan_status(came_plan_t* plan, came_stream_t stream, int* status) {
    if (!plan || !status) return fail(CAME_E_INVALID, "plan_status: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(status, plan->ws + plan->L.off_status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? CAME_OK : fail(CAME_E_CUDA, "plan_status: %s", cudaGetErrorString(e));
}

int came_b200_plan_set_timing(came_plan_t* plan, int enable) {
    if (!plan) return fail(CAME_E_INVALID, "set_timing: plan is null");
    plan->timing = enable != 0;
    return CAME_OK;
}

int came_b200_plan_read_timing(came_plan_t* plan, float* ms, int* launches) {
    if (!plan || !ms || !launches) return fail(CAME_E_INVALID, "read_timing: null argument");
    static_assert(CAME_KERNEL_COUNT == KID_COUNT, "header and kernel table out of sync");
    for (int k = 0; k < CAME_KERNEL_COUNT; ++k) { ms[k] = 0.0f; launches[k] = 0; }
    int rc = CAME_OK;
    for (auto& t : plan->timed) {
        float dt = 0.0f;
        cudaError_t e = cudaEventSynchronize(t.t1);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&dt, t.t0, t.t1);
        if (e == cudaSuccess) { ms[t.kernel] += dt; launches[t.kernel] += 1; }
        else rc = fail(CAME_E_CUDA, "read_timing: %s", cudaGetErrorString(e));
        cudaEventDestroy(t.t0);
        cudaEventDestroy(t.t1);
    }
    plan->timed.clear();
    return rc;
}

const char* came_b200_kernel_name(int kernel) {
    static const char* names[CAME_KERNEL_COUNT] = {
        "sq_partials", "sq_finalize", "sumsq", "s_finalize", "moment", "res_finalize",
        "apply", "factors", "apply_flat", "nf_partial", "nf_apply", "nf_reduce", "nd_sq", "nd_mean", "nd_sumsq", "nd_s", "nd_res",
        "nd_resmean", "nd_apply", "moment_apply"};
    return (kernel >= 0 && kernel < CAME_KERNEL_COUNT) ? names[kernel] : "?";
}

}  // extern "C"
