// C-ABI entry points (include/ldn_b200.h): argument checks, choice of operand views (the caller's
// arrays where TMA can read them directly, canonical copies in scratch otherwise), tile-engine plans.
#include <math.h>
#include <string.h>

#include <mutex>

#include "ldn_b200.h"
#include "ldn_launch.cuh"
#include "ldn_prep.cuh"

namespace ldn {
int release_arenas();

namespace {

int g_max_ctas = 0;
int g_bound_one_pass_stages = kBoundBothMaxStages;  // longest reduction (in 32-channel stages) the one-pass kernel takes
// scratch the fused backward may use for its per-row-tile column sums (bytes); larger batches run in row chunks
size_t g_side_limit = size_t(1) << 30;

// A 3-D view of an operand for TMA: `inner` contiguous elements, `rows` rows, `groups` groups.
// row_coord tells which tensor-map coordinate carries the row (1: dims are (inner, rows, groups);
// 2: dims are (inner, groups, rows), used when the group stride is the smaller one).
struct View {
    const float* ptr;
    long long inner, rows, groups;
    long long stride_row, stride_group;
    int row_coord;
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int ceil4(int v) { return (v + 3) & ~3; }

inline View canonical_view(const float* ptr, long long inner, long long rows, long long groups) {
    const long long pitch = ceil4(static_cast<int>(inner));
    return View{ptr, inner, rows, groups, pitch, rows * pitch, 1};
}
inline size_t canonical_floats(long long inner, long long rows, long long groups) {
    return static_cast<size_t>(ceil4(static_cast<int>(inner))) * rows * groups;
}

// `span` = rows (RowMajor) or columns (KMajor) of the tile: 128, or 64 for the B operand of narrow tiles
int build_map(CUtensorMap* map, const View& v, Layout layout, int span = kTileM) {
    const unsigned bi = layout == Layout::RowMajor ? kTileK : span;
    const unsigned br = layout == Layout::RowMajor ? span : kTileK;
    unsigned long long dims[3], strides[2];
    unsigned box[3];
    dims[0] = v.inner;
    box[0] = bi;
    if (v.row_coord == 1) {
        dims[1] = v.rows; dims[2] = v.groups;
        strides[0] = v.stride_row; strides[1] = v.stride_group;
        box[1] = br; box[2] = 1;
    } else {
        dims[1] = v.groups; dims[2] = v.rows;
        strides[0] = v.stride_group; strides[1] = v.stride_row;
        box[1] = 1; box[2] = br;
    }
    return make_tensor_map(map, v.ptr, dims, strides, box, layout == Layout::RowMajor);
}

inline Operand as_operand(const View& v) { return Operand{v.ptr, v.stride_row, v.stride_group}; }

// internal: the batch (or the spatial extent) is empty -- nothing to compute, like the reference, whose
// kernels then run with every row masked off
constexpr int kEmptyBatch = -1;

int check_shape(int B, int CO, int CI, int G, int HW, Shape* s) {
    if (B < 0 || CO <= 0 || CI <= 0 || G <= 0 || HW < 0) return kBadArgument;
    if (CI % G != 0 || CO % G != 0) return kBadArgument;
    if (B == 0 || HW == 0) return kEmptyBatch;
    s->B = B; s->CO = CO; s->CI = CI; s->G = G; s->HW = HW;
    s->CIg = CI / G; s->COg = CO / G;
    s->co_src = CO; s->co_off = 0;
    s->M = static_cast<long long>(B) * HW;
    if (s->M > 0x7fffffffLL) return kBadArgument;
    return kOk;
}

// Result of a call on an empty batch: outputs with a batch dimension are empty; a weight gradient is a sum
// over no samples, i.e. zero.
int empty_result(float* grad_weight, int CO, int CI, int G, ldn_stream_t stream) {
    if (!grad_weight) return kOk;
    return cuda_status(cudaMemsetAsync(grad_weight, 0, sizeof(float) * static_cast<size_t>(CO) * (CI / G),
                                       reinterpret_cast<cudaStream_t>(stream)));
}

struct Call {
    const DeviceCtx* ctx;
    Arena* arena;
    Bump bump;
    cudaStream_t st;
    int cap;  // persistent CTAs
    const float* col_sub = nullptr;  // epilogue of the no-grad p = inf kernels (see TileParams)
    const float* col_add = nullptr;
    const float* norm_rows = nullptr;  // separable normaliser of FwdPowNorm and its guard word (see TileParams)
    const float* norm_cols = nullptr;
    int* guard = nullptr;
    const int* gate = nullptr;         // forward kernels launched while set return at once unless *gate != 0
    std::unique_lock<std::mutex> lock;  // the arena's call mutex, released when the entry point returns
};

int begin_call(Call* c, ldn_stream_t stream, size_t scratch_bytes) {
    int r = get_device_ctx(&c->ctx);
    if (r != kOk) return r;
    c->st = reinterpret_cast<cudaStream_t>(stream);
    c->cap = (g_max_ctas > 0 && g_max_ctas < c->ctx->sm_count) ? g_max_ctas : c->ctx->sm_count;
    r = find_arena(c->st, &c->arena);
    if (r != kOk) return r;
    c->lock = std::unique_lock<std::mutex>(*static_cast<std::mutex*>(c->arena->call_mutex));
    if ((r = ensure_arena(c->arena, c->st, scratch_bytes)) != kOk) return r;
    c->bump = Bump{c->arena->base, 0, c->arena->capacity};
    return kOk;
}

inline size_t partial_bytes(int cap, int arrays) {
    return pad256(static_cast<size_t>(cap) * 2 * arrays * kTileElems * sizeof(float));
}
inline int cap_for(const DeviceCtx* ctx) {
    return (g_max_ctas > 0 && g_max_ctas < ctx->sm_count) ? g_max_ctas : ctx->sm_count;
}

// The x operand as the engine reads it: the caller's array when it is fully connected (HW == 1) with a
// 16-byte aligned base and row length, else a canonical copy [g][m][pitch].
bool x_is_natural(const float* x, const Shape& s) { return s.HW == 1 && s.CIg % 4 == 0 && aligned16(x); }
View x_natural_view(const float* x, const Shape& s) {
    if (s.G == 1) return View{x, s.CIg, s.M, 1, s.CI, s.M * s.CI, 1};
    return View{x, s.CIg, s.M, s.G, s.CI, s.CIg, 2};
}
bool w_is_natural(const float* w, const Shape& s) { return s.CIg % 4 == 0 && aligned16(w); }
View w_natural_view(const float* w, const Shape& s) {
    return View{w, s.CIg, s.COg, s.G, s.CIg, static_cast<long long>(s.COg) * s.CIg, 1};
}

// Convolution-shaped inputs x[B, CI, HW] can be read in place as a k-major operand (positions contiguous, channels
// 32 per stage) when TMA can address them (HW a multiple of 4 floats, 16-byte aligned base) and a 128-position tile
// is mostly filled; every (sample, group) pair is then its own engine group.  Other shapes take the transposed copy.
bool x_inplace_kmajor(const float* x, const Shape& s) { return s.HW >= 96 && s.HW % 4 == 0 && aligned16(x); }
View x_kmajor_view(const float* x, const Shape& s) {
    return View{x, s.HW, s.CIg, static_cast<long long>(s.B) * s.G, s.HW, static_cast<long long>(s.CIg) * s.HW, 1};
}
// tile width (in units of 16 columns) for a layer with `cog` outputs per group
inline int narrow_reg_n(int cog) { return cog <= 32 ? 2 : (cog <= 64 ? 4 : 8); }

size_t x_scratch_bytes(const float* x, const Shape& s) {
    return x_is_natural(x, s) ? 0 : pad256(canonical_floats(s.CIg, s.M, s.G) * sizeof(float));
}
size_t w_scratch_bytes(const float* w, const Shape& s) {
    return w_is_natural(w, s) ? 0 : pad256(canonical_floats(s.CIg, s.COg, s.G) * sizeof(float));
}

int get_x_view(Call& c, const float* x, const Shape& s, View* v) {
    if (x_is_natural(x, s)) {
        *v = x_natural_view(x, s);
        return kOk;
    }
    float* xc = c.bump.take<float>(canonical_floats(s.CIg, s.M, s.G));
    if (!xc) return kWorkspace;
    *v = canonical_view(xc, s.CIg, s.M, s.G);
    return launch_canon_x(x, xc, s, static_cast<int>(v->stride_row), c.st);
}
int get_w_view(Call& c, const float* w, const Shape& s, View* v) {
    if (w_is_natural(w, s)) {
        *v = w_natural_view(w, s);
        return kOk;
    }
    float* wc = c.bump.take<float>(canonical_floats(s.CIg, s.COg, s.G));
    if (!wc) return kWorkspace;
    *v = canonical_view(wc, s.CIg, s.COg, s.G);
    return launch_canon_w(w, wc, s, static_cast<int>(v->stride_row), c.st);
}

// Common part of a tile-engine plan.
int fill_plan(Call& c, TileLaunch* L, long long M, int N, int K, int G, int arrays, OpGeom geom = OpGeom{kTileN, 1}) {
    memset(L, 0, sizeof(*L));
    TileParams& P = L->params;
    P.M = static_cast<int>(M); P.N = N; P.K = K; P.G = G;
    P.tiles_m = static_cast<int>((M + kTileM - 1) / kTileM);
    P.tiles_n = (N + geom.tile_n - 1) / geom.tile_n;
    P.kt = (K + kTileK - 1) / kTileK;
    P.total_iters = static_cast<long long>(G) * P.tiles_m * P.tiles_n * P.kt;
    const long long cap = static_cast<long long>(c.cap) * geom.ctas_per_sm;
    L->grid = static_cast<int>(P.total_iters < cap ? P.total_iters : cap);
    // (a narrow tile has half the outputs, and at most twice the CTAs: the slot size below is an upper bound)
    P.partials = c.bump.take<float>(static_cast<size_t>(L->grid) * 2 * arrays * (kTileM * geom.tile_n));
    if (!P.partials) return kWorkspace;
    P.status = c.arena->status;
    P.trace = trace_buffer();
    return kOk;
}

OutAddr y_addr(const Shape& s) {
    return OutAddr{static_cast<long long>(s.CO) * s.HW, 1, static_cast<long long>(s.COg) * s.HW, s.HW, s.HW};
}
OutAddr x_addr(const Shape& s) {
    return OutAddr{static_cast<long long>(s.CI) * s.HW, 1, static_cast<long long>(s.CIg) * s.HW, s.HW, s.HW};
}
OutAddr w_addr(const Shape& s) {
    return OutAddr{s.CIg, 0, static_cast<long long>(s.COg) * s.CIg, 1, 1};
}

// forward-type problem: out (m = (b, hw), n = o), k = c.  inplace: a0 is x_kmajor_view (HW > 1 read in place): one
// engine group per (sample, group), m = hw.
int run_forward(Call& c, FwdKind kind, int ip, const View& a0, const View* a1, const View& wv, const Shape& s,
                float* out0, float* out1, int* outi0, int* outi1, const float* pres, float p, bool inplace = false) {
    TileLaunch L;
    const int rn = fwd_variant_supported(kind, ip) ? narrow_reg_n(s.COg) : 8;
    const bool variant = inplace || rn != 8;
    if (inplace && !fwd_variant_supported(kind, ip)) return kBadArgument;
    OpGeom geom{16 * rn, 1};
    if (!variant) {
        if (kind == FwdKind::PowInt || kind == FwdKind::PowGen || kind == FwdKind::PowNorm) geom = fwd_pow_geom(kind, ip);
        else geom = fwd_inf_geom(kind);
    }
    const long long groups = inplace ? static_cast<long long>(s.B) * s.G : s.G;
    if (groups > 0x7fffffffLL) return kBadArgument;
    int r = fill_plan(c, &L, inplace ? s.HW : s.M, s.COg, s.CIg, static_cast<int>(groups), fwd_acc_arrays(kind), geom);
    if (r != kOk) return r;
    TileParams& P = L.params;
    P.a_row_coord = a0.row_coord;
    P.b_row_coord = wv.row_coord;
    P.b_group_mod = inplace ? s.G : 0;
    P.a0 = as_operand(a0);
    P.a1 = a1 ? as_operand(*a1) : P.a0;
    P.b = as_operand(wv);
    P.pres = Operand{pres, 0, 0};
    // y[((b G + g) COg + o) HW + hw]: with one engine group per (b, g) the row index is hw itself
    P.out = inplace ? OutAddr{1, 0, static_cast<long long>(s.COg) * s.HW, s.HW, 1} : y_addr(s);
    P.out_f0 = out0; P.out_f1 = out1; P.out_i0 = outi0; P.out_i1 = outi1;
    P.p = p; P.q = p - 1.0f;
    if (kind == FwdKind::Inf || kind == FwdKind::Bound) {
        P.col_sub = c.col_sub;
        P.col_add = c.col_add;
    }
    if (kind == FwdKind::PowNorm && pres == nullptr) {
        P.norm_rows = c.norm_rows;
        P.norm_cols = c.norm_cols;
        P.guard = c.guard;
    }
    P.gate = c.gate;
    const Layout la = inplace ? Layout::KMajor : Layout::RowMajor;
    if ((r = build_map(&L.map_a0, a0, la)) != kOk) return r;
    if ((r = build_map(&L.map_a1, a1 ? *a1 : a0, la)) != kOk) return r;
    if ((r = build_map(&L.map_b, wv, Layout::RowMajor, geom.tile_n)) != kOk) return r;
    if (inplace) return launch_fwd_variant_k(kind, rn, L, c.st);
    if (variant) return launch_fwd_variant_row(kind, rn, L, c.st);
    switch (kind) {
        case FwdKind::PowInt:
        case FwdKind::PowGen:
        case FwdKind::PowNorm: return launch_fwd_pow(kind, ip, L, c.st);
        default: return launch_fwd_inf(kind, L, c.st);
    }
}

// The folded general-p backward evaluates 2^(q lg2|t| - q lg2 y): the absolute error of the logarithm (~2e-7) is
// multiplied by q, so beyond this q the kernels take the logarithm of |t| / y (near 1 for the terms that matter).
constexpr float kFoldMaxQ = 64.0f;

// Largest p for which the forward pass normalises by the separable bound of the maximum (ldn_norm_dist_forward).
constexpr float kBoundNormMaxP = 100.0f;

// integer template value the reference dispatch would use for exponent e (norm_dist.cpp:17-35)
int int_power(float e) {
    if (e == static_cast<float>(static_cast<int>(e)) && static_cast<int>(e) >= 0 && static_cast<int>(e) <= 8)
        return static_cast<int>(e);
    return -1;
}

// One backward call on rows [0, s.B) of the given pointers.  accumulate_gw: add to grad_weight instead of
// overwriting it (only the fused path supports that; it is how the row chunks of one call combine).
//
// Integer p - 1 = q: the kernels multiply the per-(b, o) coefficient g / y^q by sgn(t) |t|^q, one instruction per
// pair fewer than the reference's g (|t| / y)^q (norm_dist_cuda.cu:238-243) but with less range: y^-q overflows or
// |t|^q goes denormal for very small outputs, the coefficient vanishes for very large ones.  The coefficient kernel
// therefore raises a device flag when some y^-q leaves [1e-30, 1e24], and the same gradients are then recomputed in
// the normalised form 2^(q lg2(|t| / y)) by the general-p kernels, launched behind the fast ones with that flag as a
// gate (they return at once when it is clear, which is always for networks' usual value ranges).
int norm_dist_backward_part(const float* go, const float* x, const float* w, const float* y, const Shape& s, float* gx,
                            float* gw, float p, ldn_stream_t stream, bool accumulate_gw, bool accumulate_gx = false) {
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    const int cap = cap_for(ctx);
    int iq = int_power(p - 1.0f);
    // general p: fold 1 / y into the exponent offset while q lg2|t| keeps the terms accurate to ~1e-5
    if (iq < 0 && p - 1.0f > kFoldMaxQ) iq = -2;
    const bool guarded = iq >= 1;  // integer form with a range guard (q = 0: the coefficient is g itself)
    // general p (and the guard's second form): coefficient arrays padded to whole tiles (see launch_coef_gen)
    const long long gen_rows = (s.M + kTileM - 1) / kTileM * kTileM;
    const long long gen_pitch = (s.COg + kTileK - 1) / kTileK * kTileK;
    const size_t gen_floats = static_cast<size_t>(gen_pitch) * gen_rows * s.G;
    const long long int_pitch = ceil4(s.COg);
    const size_t int_floats = static_cast<size_t>(int_pitch) * s.M * s.G;
    // Both gradients wanted: one fused kernel evaluates every term once (grad_input accumulators plus
    // per-row-tile column sums for grad_weight).  It needs tiles_m copies of grad_weight as scratch, so very
    // tall problems (conv layouts with many rows) keep the two-kernel path; so does p = 1 (constant terms).
    const long long tiles_m = (s.M + kTileM - 1) / kTileM;
    const size_t side_floats = static_cast<size_t>(tiles_m) * s.CO * s.CIg;
    const bool fused = gx && gw && iq != 0 && side_floats * sizeof(float) <= g_side_limit;
    if (accumulate_gw && !fused) return kBadArgument;
    size_t need = x_scratch_bytes(x, s) + w_scratch_bytes(w, s) + (iq >= 0 ? pad256(int_floats * sizeof(float)) : 0) +
                  ((iq < 0 || guarded) ? 2 * pad256(gen_floats * sizeof(float)) : 0) +
                  (guarded ? 4 : 2) * partial_bytes(cap, 1) + (fused ? pad256(side_floats * sizeof(float)) : 0);
    Call c;
    if ((r = begin_call(&c, stream, need)) != kOk) return r;
    View xv, wv;
    if ((r = get_x_view(c, x, s, &xv)) != kOk) return r;
    if ((r = get_w_view(c, w, s, &wv)) != kOk) return r;
    float* side = nullptr;
    if (fused && !(side = c.bump.take<float>(side_floats))) return kWorkspace;
    // the guard's flag: a word of the arena's status block, cleared in stream order before the coefficient kernel
    // may raise it (calls on one stream follow each other, so the previous call's gated kernels have read it by then)
    int* flag = nullptr;
    if (guarded) {
        flag = c.arena->status + 1;
        const cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int), c.st);
        if (e != cudaSuccess) return cuda_status(e);
    }

    // the kernels of one arithmetic form (fam: 0..8 integer q, -1 / -2 general p) on coefficient views cv0 / cv1.
    // gate: run only if *gate != 0 (the guard's second form); the weight-gradient reduction of the fast form is
    // gated the other way round, so exactly one of the two forms touches grad_weight.
    auto run_family = [&](int fam, const View& cv0, const View& cv1, const int* gate) -> int {
        auto plan_rows = [&](TileLaunch& L, const OpGeom geom) -> int {
            int e = fill_plan(c, &L, s.M, s.CIg, s.COg, s.G, 1, geom);
            if (e != kOk) return e;
            TileParams& P = L.params;
            P.a_row_coord = cv0.row_coord;
            P.b_row_coord = wv.row_coord;
            P.a0 = as_operand(cv0); P.a1 = as_operand(cv1); P.b = as_operand(wv);
            P.pres = as_operand(xv);
            P.out = x_addr(s);
            P.out_f0 = gx;
            P.p = p; P.q = p - 1.0f;
            P.gate = gate;
            P.accumulate_out = accumulate_gx ? 1 : 0;
            if (accumulate_gx && guarded && gate == nullptr) {
                // adding to grad_input: exactly one of the two forms may run (the fast one only while the flag is clear)
                P.gate = flag;
                P.gate_invert = 1;
            }
            if ((e = build_map(&L.map_a0, cv0, Layout::RowMajor)) != kOk) return e;
            if ((e = build_map(&L.map_a1, cv1, Layout::RowMajor)) != kOk) return e;
            return build_map(&L.map_b, wv, Layout::KMajor, geom.tile_n);
        };
        int e;
        if (fused) {
            TileLaunch L;
            if ((e = plan_rows(L, bwd_fused_geom(fam))) != kOk) return e;
            L.params.side_out = side;
            if ((e = launch_bwd_fused(fam, L, c.st)) != kOk) return e;
            return launch_side_reduce(side, gw, static_cast<long long>(s.CO) * s.CIg, static_cast<int>(tiles_m),
                                      accumulate_gw, gate ? gate : flag, gate != nullptr, c.st);
        }
        if (gx) {
            TileLaunch L;
            if ((e = plan_rows(L, bwd_x_geom(fam))) != kOk) return e;
            if ((e = launch_bwd_x(fam, L, c.st)) != kOk) return e;
        }
        if (gw) {
            // out (m = o, n = c), k = (b, hw)
            TileLaunch L;
            const OpGeom geom = bwd_w_geom(fam);
            if ((e = fill_plan(c, &L, s.COg, s.CIg, static_cast<int>(s.M), s.G, 1, geom)) != kOk) return e;
            TileParams& P = L.params;
            P.a_row_coord = cv0.row_coord;
            P.b_row_coord = xv.row_coord;
            P.a0 = as_operand(cv0); P.a1 = as_operand(cv1); P.b = as_operand(xv);
            P.pres = as_operand(wv);
            P.out = w_addr(s);
            P.out_f0 = gw;
            P.p = p; P.q = p - 1.0f;
            P.gate = gate;
            if ((e = build_map(&L.map_a0, cv0, Layout::KMajor)) != kOk) return e;
            if ((e = build_map(&L.map_a1, cv1, Layout::KMajor)) != kOk) return e;
            if ((e = build_map(&L.map_b, xv, Layout::KMajor, geom.tile_n)) != kOk) return e;
            if ((e = launch_bwd_w(fam, L, c.st)) != kOk) return e;
        }
        return kOk;
    };
    auto gen_views = [&](float* a, float* b, View* v0, View* v1) {
        *v0 = View{a, gen_pitch, gen_rows, s.G, gen_pitch, gen_rows * gen_pitch, 1};
        *v1 = View{b, gen_pitch, gen_rows, s.G, gen_pitch, gen_rows * gen_pitch, 1};
    };

    if (iq >= 0) {
        float* c0 = c.bump.take<float>(int_floats);
        if (!c0) return kWorkspace;
        const View cv = View{c0, s.COg, s.M, s.G, int_pitch, s.M * int_pitch, 1};
        if ((r = launch_coef_int(go, y, c0, s, static_cast<int>(int_pitch), iq, flag, c.st)) != kOk) return r;
        if ((r = run_family(iq, cv, cv, nullptr)) != kOk) return r;
        if (!guarded) return kOk;
        // second form, gated by the flag: 1 / y and g as coefficients, 2^(q lg2(|t| / y)) per pair
        float* r0 = c.bump.take<float>(gen_floats);
        float* r1 = c.bump.take<float>(gen_floats);
        if (!r0 || !r1) return kWorkspace;
        View v0, v1;
        gen_views(r0, r1, &v0, &v1);
        if ((r = launch_coef_gen(go, y, r0, r1, s, static_cast<int>(gen_pitch), gen_rows, p - 1.0f, false, flag, c.st)) != kOk)
            return r;
        return run_family(-2, v0, v1, flag);
    }
    float* c0 = c.bump.take<float>(gen_floats);
    float* c1 = c.bump.take<float>(gen_floats);
    if (!c0 || !c1) return kWorkspace;
    View v0, v1;
    gen_views(c0, c1, &v0, &v1);
    if ((r = launch_coef_gen(go, y, c0, c1, s, static_cast<int>(gen_pitch), gen_rows, p - 1.0f, iq == -1, nullptr, c.st)) != kOk)
        return r;
    return run_family(iq, v0, v1, nullptr);
}

int norm_dist_backward(const float* go, const float* x, const float* w, const float* y, const Shape& s, float* gx,
                       float* gw, float p, ldn_stream_t stream, bool accumulate_gx = false) {
    if (!go || !x || !w || !y || (!gx && !gw)) return kBadArgument;
    if (!(p > 0.0f) || isinf(p) || isnan(p)) return kBadArgument;
    // The fused kernel keeps one copy of grad_weight per 128-row tile as scratch.  A batch whose copies would
    // exceed the limit runs as chunks of whole samples, each within the limit; the chunks' weight gradients
    // add up in grad_weight (stream order), their input gradients are disjoint row ranges.
    if (gx && gw && int_power(p - 1.0f) != 0) {
        const size_t tile_bytes = static_cast<size_t>(s.CO) * s.CIg * sizeof(float);
        const long long max_tiles = static_cast<long long>(g_side_limit / tile_bytes);
        const long long tiles_m = (s.M + kTileM - 1) / kTileM;
        const long long chunk_b = max_tiles * kTileM / s.HW;
        if (tiles_m > max_tiles && chunk_b >= 1) {
            for (long long b0 = 0; b0 < s.B; b0 += chunk_b) {
                Shape sc = s;
                sc.B = static_cast<int>(s.B - b0 < chunk_b ? s.B - b0 : chunk_b);
                sc.M = static_cast<long long>(sc.B) * s.HW;
                const size_t oy = static_cast<size_t>(b0) * s.co_src * s.HW, ox = static_cast<size_t>(b0) * s.CI * s.HW;
                const int r = norm_dist_backward_part(go + oy, x + ox, w, y + oy, sc, gx + ox, gw, p, stream, b0 > 0,
                                                      accumulate_gx);
                if (r != kOk) return r;
            }
            return kOk;
        }
    }
    return norm_dist_backward_part(go, x, w, y, s, gx, gw, p, stream, false, accumulate_gx);
}

int inf_forward(const float* x, const float* w, const Shape& s, float* y, int* pos, ldn_stream_t stream,
                const float* col_sub = nullptr, const float* col_add = nullptr) {
    if (!x || !w || !y) return kBadArgument;
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    const FwdKind kind = pos ? FwdKind::InfPos : FwdKind::Inf;
    const bool inplace = x_inplace_kmajor(x, s);
    size_t need = (inplace ? 0 : x_scratch_bytes(x, s)) + w_scratch_bytes(w, s) +
                  partial_bytes(cap_for(ctx), fwd_acc_arrays(kind));
    Call c;
    if ((r = begin_call(&c, stream, need)) != kOk) return r;
    c.col_sub = col_sub;
    c.col_add = col_add;
    View xv, wv;
    if (inplace) xv = x_kmajor_view(x, s);
    else if ((r = get_x_view(c, x, s, &xv)) != kOk) return r;
    if ((r = get_w_view(c, w, s, &wv)) != kOk) return r;
    r = run_forward(c, kind, 0, xv, nullptr, wv, s, y, nullptr, pos, nullptr, nullptr, INFINITY, inplace);
    if (r != kOk || !pos) return r;
    if (inplace) {
        // the input as the index search addresses it: element (sample-group bg, position hw, channel k) at
        // bg * stride_group + hw * stride_row + k * HW
        const Operand xin{x, 1, static_cast<long long>(s.CIg) * s.HW};
        return launch_rescan(0, xin, xin, as_operand(wv), y, pos, s, c.st, s.HW);
    }
    return launch_rescan(0, as_operand(xv), as_operand(xv), as_operand(wv), y, pos, s, c.st, 1);
}

int bound_forward(const float* xl, const float* xu, const float* w, const Shape& s, float* yl, float* yu, int* pl,
                  int* pu, ldn_stream_t stream, const float* col_sub = nullptr, const float* col_add = nullptr) {
    if (!xl || !xu || !w || !yl || !yu || ((pl == nullptr) != (pu == nullptr))) return kBadArgument;
    const DeviceCtx* ctx;
    int r = get_device_ctx(&ctx);
    if (r != kOk) return r;
    const size_t xfloats = canonical_floats(s.CIg, s.M, s.G);
    size_t need = 2 * pad256(xfloats * sizeof(float)) + w_scratch_bytes(w, s) + 2 * partial_bytes(cap_for(ctx), 5);
    Call c;
    if ((r = begin_call(&c, stream, need)) != kOk) return r;
    c.col_sub = col_sub;
    c.col_add = col_add;
    float* lc = c.bump.take<float>(xfloats);
    float* uc = c.bump.take<float>(xfloats);
    if (!lc || !uc) return kWorkspace;
    const View lv = canonical_view(lc, s.CIg, s.M, s.G);
    const View uv = canonical_view(uc, s.CIg, s.M, s.G);
    if ((r = launch_canon_bounds(xl, xu, lc, uc, s, static_cast<int>(lv.stride_row), c.st)) != kOk) return r;
    View wv;
    if ((r = get_w_view(c, w, s, &wv)) != kOk) return r;
    if (!pl) return run_forward(c, FwdKind::Bound, 0, lv, &uv, wv, s, yl, yu, nullptr, nullptr, nullptr, INFINITY);
    if ((s.CIg + kTileK - 1) / kTileK <= g_bound_one_pass_stages) {
        // one pass: both bounds and the stage of each extremum, then the two index searches
        r = run_forward(c, FwdKind::BoundPosBoth, 0, lv, &uv, wv, s, yl, yu, pl, pu, nullptr, INFINITY);
        if (r != kOk) return r;
        if ((r = launch_rescan(1, as_operand(lv), as_operand(uv), as_operand(wv), yl, pl, s, c.st, 1)) != kOk) return r;
        return launch_rescan(2, as_operand(lv), as_operand(uv), as_operand(wv), yu, pu, s, c.st, 1);
    }
    r = run_forward(c, FwdKind::BoundPosLower, 0, lv, &uv, wv, s, yl, yu, pl, pu, nullptr, INFINITY);
    if (r != kOk) return r;
    if ((r = launch_rescan(1, as_operand(lv), as_operand(uv), as_operand(wv), yl, pl, s, c.st, 1)) != kOk) return r;
    r = run_forward(c, FwdKind::BoundPosUpper, 0, lv, &uv, wv, s, yl, yu, pl, pu, nullptr, INFINITY);
    if (r != kOk) return r;
    return launch_rescan(2, as_operand(lv), as_operand(uv), as_operand(wv), yu, pu, s, c.st, 1);
}

}  // namespace
}  // namespace ldn

using namespace ldn;

extern "C" {

LDN_API const char* ldn_status_string(int status) {
    switch (status) {
        case kOk: return "ok";
        case kBadArgument: return "bad argument (null pointer, non-positive size, CI or CO not divisible by G, or p not a positive finite number)";
        case kNoDevice: return "no usable CUDA device or driver entry point";
        case kWorkspace: return "scratch memory could not be provided";
        case kDeviceTimeout: return "a bounded wait inside a kernel gave up";
        case kTensorMap: return "the driver rejected a TMA descriptor";
        case kCaptureGrowth:
            return "the scratch arena would have to grow while its stream is being captured: issue the same call once "
                   "before the capture, or reserve the scratch with ldn_reserve_scratch";
        default: break;
    }
    if (status >= kCudaBase) return cudaGetErrorString(static_cast<cudaError_t>(status - kCudaBase));
    return "unknown status";
}

LDN_API const char* ldn_version(void) { return "ldn_b200 0.1 sm_100a"; }

LDN_API void ldn_set_max_ctas(int max_ctas) { g_max_ctas = max_ctas > 0 ? max_ctas : 0; }

LDN_API void ldn_set_bound_one_pass_limit(int stages) {
    g_bound_one_pass_stages = (stages >= 0 && stages < kBoundBothMaxStages) ? stages : kBoundBothMaxStages;
}

LDN_API void ldn_set_fused_scratch_limit(unsigned long long bytes) {
    g_side_limit = bytes > 0 ? static_cast<size_t>(bytes) : size_t(1) << 30;
}

LDN_API int ldn_release_scratch(void) { return release_arenas(); }

LDN_API int ldn_reserve_scratch(ldn_stream_t stream, unsigned long long bytes) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    Arena* arena;
    int r = find_arena(st, &arena);
    if (r != kOk) return r;
    std::lock_guard<std::mutex> lock(*static_cast<std::mutex*>(arena->call_mutex));
    return ensure_arena(arena, st, static_cast<size_t>(bytes));
}

LDN_API int ldn_check_status(ldn_stream_t stream) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    Arena* arena;
    int r = find_arena(st, &arena);
    if (r != kOk) return r;
    cudaError_t e = cudaMemcpyAsync(arena->status_host, arena->status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(arena->status, 0, sizeof(int), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_status(e);
    const int v = *arena->status_host;
    *arena->status_host = 0;
    return v;
}

LDN_API int ldn_norm_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                          float* output, float p, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!input || !weight || !output) return kBadArgument;
    if (!(p > 0.0f) || isinf(p) || isnan(p)) return kBadArgument;
    const DeviceCtx* ctx;
    if ((r = get_device_ctx(&ctx)) != kOk) return r;
    const bool normalised = p > 10.0f;  // MIN_NORMALIZED_P of the reference
    const int ip = normalised ? -1 : int_power(p);
    const FwdKind kind = normalised ? FwdKind::PowNorm : (ip >= 1 ? FwdKind::PowInt : FwdKind::PowGen);
    const bool inplace = x_inplace_kmajor(input, s) && fwd_variant_supported(kind, ip);
    // Up to this p the normaliser is the separable bound max|x| + max|w| of max|t| (two row reductions instead of a
    // full max pass); beyond, a bound a few per cent above the true maximum already underflows the sum, so the exact
    // maximum is computed first, as the reference does.
    const bool bound_norm = normalised && p <= kBoundNormMaxP;
    const long long xrows = inplace ? s.HW : s.M;
    const long long xgroups = inplace ? static_cast<long long>(s.B) * s.G : s.G;
    const size_t norm_floats = static_cast<size_t>(xrows * xgroups) + static_cast<size_t>(s.CO);
    const size_t ybytes = pad256(sizeof(float) * static_cast<size_t>(B) * CO * HW);
    size_t need = (inplace ? 0 : x_scratch_bytes(input, s)) + w_scratch_bytes(weight, s) +
                  (bound_norm ? 3 : 2) * partial_bytes(cap_for(ctx), 1) + (normalised ? ybytes : 0) +
                  (bound_norm ? 2 * pad256(norm_floats * sizeof(float)) : 0);
    Call c;
    if ((r = begin_call(&c, stream, need)) != kOk) return r;
    View xv, wv;
    if (inplace) xv = x_kmajor_view(input, s);
    else if ((r = get_x_view(c, input, s, &xv)) != kOk) return r;
    if ((r = get_w_view(c, weight, s, &wv)) != kOk) return r;
    if (!normalised)
        return run_forward(c, kind, ip >= 1 ? ip : -1, xv, nullptr, wv, s, output, nullptr, nullptr, nullptr, nullptr, p,
                           inplace);
    float* mbuf = c.bump.take<float>(static_cast<size_t>(B) * CO * HW);
    if (!mbuf) return kWorkspace;
    if (bound_norm) {
        float* xa = c.bump.take<float>(static_cast<size_t>(xrows * xgroups));
        float* wa = c.bump.take<float>(static_cast<size_t>(s.CO));
        if (!xa || !wa) return kWorkspace;
        // the guard word (a word of the arena's status block): cleared by the first row reduction, raised by the sum
        // kernel, read by the gated kernels behind it -- all in stream order
        int* flag = c.arena->status + 2;
        const Operand xop = inplace ? Operand{input, 1, static_cast<long long>(s.CIg) * s.HW} : as_operand(xv);
        if ((r = launch_row_absmax(xop, xrows, s.CIg, static_cast<int>(xgroups), inplace ? s.HW : 1, xa, flag,
                                   c.st)) != kOk)
            return r;
        if ((r = launch_row_absmax(as_operand(wv), s.COg, s.CIg, s.G, 1, wa, nullptr, c.st)) != kOk) return r;
        c.norm_rows = xa;
        c.norm_cols = wa;
        c.guard = flag;
        r = run_forward(c, FwdKind::PowNorm, -1, xv, nullptr, wv, s, output, nullptr, nullptr, nullptr, nullptr, p, inplace);
        if (r != kOk) return r;
        // the exact form behind it, gated by the guard word: runs only when some sum came out too small
        c.gate = flag;
    }
    r = run_forward(c, FwdKind::Inf, 0, xv, nullptr, wv, s, mbuf, nullptr, nullptr, nullptr, nullptr, INFINITY, inplace);
    if (r != kOk) return r;
    return run_forward(c, FwdKind::PowNorm, -1, xv, nullptr, wv, s, output, nullptr, nullptr, nullptr, mbuf, p, inplace);
}

LDN_API int ldn_norm_dist_forward_with_max(const float* input, const float* weight, const float* max_output,
                                   int B, int CO, int CI, int G, int HW, float* output, float p,
                                   ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!input || !weight || !max_output || !output) return kBadArgument;
    if (!(p > 0.0f) || isinf(p) || isnan(p)) return kBadArgument;
    const DeviceCtx* ctx;
    if ((r = get_device_ctx(&ctx)) != kOk) return r;
    size_t need = x_scratch_bytes(input, s) + w_scratch_bytes(weight, s) + partial_bytes(cap_for(ctx), 1);
    Call c;
    if ((r = begin_call(&c, stream, need)) != kOk) return r;
    View xv, wv;
    if ((r = get_x_view(c, input, s, &xv)) != kOk) return r;
    if ((r = get_w_view(c, weight, s, &wv)) != kOk) return r;
    return run_forward(c, FwdKind::PowNorm, -1, xv, nullptr, wv, s, output, nullptr, nullptr, nullptr, max_output, p);
}

LDN_API int ldn_norm_dist_backward_input(const float* grad_output, const float* input, const float* weight,
                                 const float* output, int B, int CO, int CI, int G, int HW,
                                 float* grad_input, float p, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_input) return kBadArgument;
    return norm_dist_backward(grad_output, input, weight, output, s, grad_input, nullptr, p, stream);
}

LDN_API int ldn_norm_dist_backward_input_weight(const float* grad_output, const float* input, const float* weight,
                                        const float* output, int B, int CO, int CI, int G, int HW,
                                        float* grad_input, float* grad_weight, float p, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(grad_weight, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_weight) return kBadArgument;
    return norm_dist_backward(grad_output, input, weight, output, s, grad_input, grad_weight, p, stream);
}

LDN_API int ldn_norm_dist_backward_channels(const float* grad_output, const float* input, const float* weight,
                                            const float* output, int B, int CO, int CI, int HW, int co_begin,
                                            int co_count, float* grad_input, float* grad_weight, float p,
                                            int accumulate_input, ldn_stream_t stream) {
    Shape s;
    if (co_begin < 0 || co_count <= 0 || co_begin > CO - co_count) return kBadArgument;
    int r = check_shape(B, co_count, CI, 1, HW, &s);
    if (r == kEmptyBatch) return empty_result(grad_weight ? grad_weight + static_cast<size_t>(co_begin) * CI : nullptr,
                                              co_count, CI, 1, stream);
    if (r != kOk) return r;
    if (!grad_input || !grad_weight || CO <= 0) return kBadArgument;
    s.co_src = CO;
    s.co_off = co_begin;
    const size_t woff = static_cast<size_t>(co_begin) * CI;
    return norm_dist_backward(grad_output, input, weight + woff, output, s, grad_input, grad_weight + woff, p, stream,
                              accumulate_input != 0);
}

LDN_API int ldn_inf_dist_forward_nograd(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                                float* output, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    return inf_forward(input, weight, s, output, nullptr, stream);
}

LDN_API int ldn_inf_dist_forward_nograd_shifted(const float* input, const float* weight, int B, int CO, int CI, int G,
                                                int HW, float* output, const float* sub, const float* add,
                                                ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    return inf_forward(input, weight, s, output, nullptr, stream, sub, add);
}

LDN_API int ldn_bound_inf_dist_forward_nograd_shifted(const float* inputL, const float* inputU, const float* weight,
                                                      int B, int CO, int CI, int G, int HW, float* outputL,
                                                      float* outputU, const float* sub, const float* add,
                                                      ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    return bound_forward(inputL, inputU, weight, s, outputL, outputU, nullptr, nullptr, stream, sub, add);
}

LDN_API int ldn_inf_dist_forward(const float* input, const float* weight, int B, int CO, int CI, int G, int HW,
                         float* output, int* pos, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!pos) return kBadArgument;
    return inf_forward(input, weight, s, output, pos, stream);
}

LDN_API int ldn_inf_dist_backward_input(const float* grad_output, const int* pos, int B, int CO, int CI, int G, int HW,
                                float* grad_input, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_output || !pos || !grad_input) return kBadArgument;
    return launch_inf_scatter(grad_output, pos, grad_input, nullptr, s, reinterpret_cast<cudaStream_t>(stream));
}

LDN_API int ldn_inf_dist_backward_input_weight(const float* grad_output, const int* pos, int B, int CO, int CI, int G,
                                       int HW, float* grad_input, float* grad_weight, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(grad_weight, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_output || !pos || !grad_weight) return kBadArgument;
    return launch_inf_scatter(grad_output, pos, grad_input, grad_weight, s, reinterpret_cast<cudaStream_t>(stream));
}

LDN_API int ldn_bound_inf_dist_forward_nograd(const float* inputL, const float* inputU, const float* weight,
                                      int B, int CO, int CI, int G, int HW, float* outputL, float* outputU,
                                      ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    return bound_forward(inputL, inputU, weight, s, outputL, outputU, nullptr, nullptr, stream);
}

LDN_API int ldn_bound_inf_dist_forward(const float* inputL, const float* inputU, const float* weight,
                               int B, int CO, int CI, int G, int HW, float* outputL, float* outputU,
                               int* posL, int* posU, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!posL || !posU) return kBadArgument;
    return bound_forward(inputL, inputU, weight, s, outputL, outputU, posL, posU, stream);
}

LDN_API int ldn_bound_inf_dist_backward_input(const float* grad_outputL, const float* grad_outputU,
                                      const int* posL, const int* posU, int B, int CO, int CI, int G, int HW,
                                      float* grad_inputL, float* grad_inputU, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_outputL || !grad_outputU || !posL || !posU || !grad_inputL || !grad_inputU) return kBadArgument;
    return launch_bound_scatter(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU, nullptr, s,
                                reinterpret_cast<cudaStream_t>(stream));
}

LDN_API int ldn_bound_inf_dist_backward_input_weight(const float* grad_outputL, const float* grad_outputU,
                                             const int* posL, const int* posU, int B, int CO, int CI, int G,
                                             int HW, float* grad_inputL, float* grad_inputU, float* grad_weight,
                                             ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(grad_weight, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!grad_outputL || !grad_outputU || !posL || !posU || !grad_inputL || !grad_inputU || !grad_weight)
        return kBadArgument;
    return launch_bound_scatter(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU, grad_weight, s,
                                reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the p = inf no-grad forward.
//
// Some hosts of this library must not allocate device memory once they are running: an inference
// server that hands its whole memory budget to its own pool at start-up, a caller that is about to
// record its launches into a CUDA graph or runs under a framework whose allocator must see every byte,
// a safety-certified runtime that forbids cudaMalloc after initialisation.  The regular entry points
// take their scratch from an arena that grows with cudaMalloc, so those callers get this one instead:
// its scratch is a fixed array in the library's own device image.
// ------------------------------------------------------------------------------------------------
namespace ldn {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(32) << 20;  // 32 MiB, resident on every GPU that loads the library
constexpr size_t kNoAllocStatusBytes = 256;                // the first bytes hold the device status word

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address; the address a
// kernel may use comes from cudaGetSymbolAddress, looked up once per device with that device current.
char* g_noalloc_ptr[64] = {};
std::mutex g_noalloc_mutex;

int noalloc_scratch_address(char** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kNoDevice;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_status(e);
        if (!p) return kWorkspace;
        g_noalloc_ptr[dev] = static_cast<char*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return kOk;
}

}  // namespace
}  // namespace ldn

extern "C" {

LDN_API int ldn_inf_dist_forward_nograd_noalloc(const float* input, const float* weight, int B, int CO, int CI,
                                                int G, int HW, float* output, ldn_stream_t stream) {
    Shape s;
    int r = check_shape(B, CO, CI, G, HW, &s);
    if (r == kEmptyBatch) return empty_result(nullptr, CO, CI, G, stream);
    if (r != kOk) return r;
    if (!input || !weight || !output) return kBadArgument;
    Call c;
    if ((r = get_device_ctx(&c.ctx)) != kOk) return r;
    c.st = reinterpret_cast<cudaStream_t>(stream);
    c.cap = cap_for(c.ctx);
    c.arena = nullptr;
    // everything this call needs must fit into the fixed array: refuse before anything is launched
    const size_t need = kNoAllocStatusBytes + x_scratch_bytes(input, s) + w_scratch_bytes(weight, s) +
                        partial_bytes(c.cap, fwd_acc_arrays(FwdKind::Inf));
    if (need > kNoAllocScratchBytes) return kWorkspace;
    char* base = nullptr;
    if ((r = noalloc_scratch_address(&base)) != kOk) return r;
    Arena fixed{base + kNoAllocStatusBytes, kNoAllocScratchBytes - kNoAllocStatusBytes,
                reinterpret_cast<int*>(base), nullptr, nullptr, false, nullptr};
    c.arena = &fixed;
    c.bump = Bump{fixed.base, 0, fixed.capacity};
    View xv, wv;
    if ((r = get_x_view(c, input, s, &xv)) != kOk) return r;
    if ((r = get_w_view(c, weight, s, &wv)) != kOk) return r;
    return run_forward(c, FwdKind::Inf, 0, xv, nullptr, wv, s, output, nullptr, nullptr, nullptr, nullptr, INFINITY);
}

LDN_API int ldn_noalloc_check_status(ldn_stream_t stream) {
    char* base = nullptr;
    int r = noalloc_scratch_address(&base);
    if (r != kOk) return r;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // a plain host int: the runtime stages the copy itself, nothing is allocated on the device
    int word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, base, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(base, 0, sizeof(int), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_status(e);
    return word;
}

}  // extern "C"

