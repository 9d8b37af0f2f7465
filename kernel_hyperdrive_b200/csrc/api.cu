// extern "C" entry points of the grouped-GEMM operators and of the fused layer path, argument checks,
// engine selection and the host-side error plumbing.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace b200moe {

static thread_local char g_detail[512] = "";
static std::atomic<int64_t> g_launches{0};
static std::atomic<int> g_engine{B200MOE_ENGINE_AUTO};
static std::atomic<int> g_options[B200MOE_OPT_COUNT] = {{0}, {2}, {-1}, {-1}, {0}};  // index = option id; [0] unused

void set_error_detail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_error_detail("%s: %s", what, cudaGetErrorString(err));
        return B200MOE_ERR_LAUNCH;
    }
    return B200MOE_OK;
}

int current_engine() { return g_engine.load(); }

int option_value(int option) { return (option > 0 && option < B200MOE_OPT_COUNT) ? g_options[option].load() : 0; }

// Per-shape tile table of the tensor-core engine, keyed on (operation, reduction extent K, output columns N, rows per
// expert); the first matching rule wins.  It stands where the reference has autotuner configurations keyed on N and K.
// The entries come from timing both tiles on a B200 with the benchmark's layer shapes (TFLOP/s of the whole step, two-CTA
// 256 x 256 tile vs one-CTA 128 x 256 tile): 8 experts x 4096 rows, hidden 4096, intermediate 14336: 1168-1190 vs 1122;
// 64 x 3072 rows, 2048 / 1408: 933-994 vs 891; 128 experts, Zipf-skewed, mean 4096 rows, 2048 / 768: 845-879 vs 791;
// 256 x 512 rows, 7168 / 2048: 847 vs 878, the one-CTA tile ahead in every one of the six launches (with four or five
// 128-row blocks per expert, half of the experts leave one CTA of a pair idle for a block, and a weight-gradient tile
// reduces over only eight 64-row steps).
struct TileRule {
    int op;                        // B200MOE_OP_* or -1 for every operation
    int k_min, k_max;              // reduction extent (weight gradients: output rows)
    int n_min, n_max;              // output columns
    int64_t rows_min, rows_max;    // rows per expert (padded capacity / experts)
    int tile;
};
constexpr int kAny = 1 << 30;
const TileRule kTileTable[] = {
    {-1, 0, kAny, 0, kAny, 0, 1023, B200MOE_TILE_CTA_128x256},
    {-1, 0, kAny, 0, kAny, 1024, (int64_t)1 << 40, B200MOE_TILE_PAIR_256x256},
};

int tile_table_lookup(int op, int K, int N, int64_t rows_per_expert) {
    for (const TileRule& r : kTileTable) {
        if ((r.op < 0 || r.op == op) && K >= r.k_min && K <= r.k_max && N >= r.n_min && N <= r.n_max && rows_per_expert >= r.rows_min &&
            rows_per_expert <= r.rows_max)
            return r.tile;
    }
    return B200MOE_TILE_PAIR_256x256;
}

int launch_offsets_from_sorted(const int64_t* sorted, int64_t M, int E, int64_t* offsets, cudaStream_t stream);
int launch_make_row_maps(const int64_t* idx, int64_t M, int fan_out, int32_t* src_map, int32_t* dst_map,
                         cudaStream_t stream);

namespace {

bool dtype_ok(int dtype) { return dtype == B200MOE_F32 || dtype == B200MOE_BF16 || dtype == B200MOE_F16; }

// Picks the engine for one problem; returns <0 on error, else 0 (SIMT) or 1 (UMMA).
template <typename G, typename F>
int pick_engine(const G& g, int dtype, F&& supported, const char* what) {
    int eng = current_engine();
    if (eng == B200MOE_ENGINE_SIMT) return 0;
    bool ok = dtype != B200MOE_F32 && supported(g, dtype);
    if (eng == B200MOE_ENGINE_UMMA || eng == B200MOE_ENGINE_UMMA_1CTA || eng == B200MOE_ENGINE_UMMA_GATHER4) {
        if (!ok) {
            set_error_detail("%s: shape/dtype not handled by the tcgen05 engine", what);
            return B200MOE_ERR_LAYOUT;
        }
        return 1;
    }
    return ok ? 1 : 0;
}

int run_row_gemm(const RowGemm& g, int dtype, int32_t* status, cudaStream_t stream, const char* what) {
    int eng = pick_engine(g, dtype, umma_row_gemm_supported, what);
    if (eng < 0) return eng;
    return eng ? umma_row_gemm(g, dtype, status, stream) : simt_row_gemm(g, dtype, stream);
}

int run_w_gemm(const WGemm& g, int dtype, int32_t* status, cudaStream_t stream, const char* what) {
    int eng = pick_engine(g, dtype, umma_w_gemm_supported, what);
    if (eng < 0) return eng;
    return eng ? umma_w_gemm(g, dtype, status, stream) : simt_w_gemm(g, dtype, stream);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_version(void) { return 200; }

extern "C" const char* b200moe_error_string(int code) {
    switch (code) {
        case B200MOE_OK:
            return "ok";
        case B200MOE_ERR_ARG:
            return "bad argument";
        case B200MOE_ERR_DTYPE:
            return "unknown dtype";
        case B200MOE_ERR_LAYOUT:
            return "unsupported stride or alignment";
        case B200MOE_ERR_WORKSPACE:
            return "workspace too small";
        case B200MOE_ERR_LAUNCH:
            return "CUDA launch error";
        case B200MOE_ERR_UNSUPPORTED:
            return "unsupported problem size";
        case B200MOE_ERR_DRIVER:
            return "CUDA driver entry point unavailable";
        case B200MOE_ERR_DEVICE:
            return "device-side failure (bounded wait expired or index out of range)";
        default:
            return "unknown error code";
    }
}

extern "C" const char* b200moe_last_error_detail(void) { return g_detail; }

extern "C" int b200moe_set_engine(int engine) {
    if (engine < B200MOE_ENGINE_AUTO || engine > B200MOE_ENGINE_UMMA_GATHER4) return B200MOE_ERR_ARG;
    return g_engine.exchange(engine);
}

extern "C" int b200moe_set_option(int option, int value) {
    if (option <= 0 || option >= B200MOE_OPT_COUNT) return B200MOE_ERR_ARG;
    if (option == B200MOE_OPT_DYNAMIC_TILES && (value < 0 || value > 3)) return B200MOE_ERR_ARG;
    if (option == B200MOE_OPT_TILE_VARIANT && (value < -1 || value >= B200MOE_TILE_COUNT)) return B200MOE_ERR_ARG;
    if (option == B200MOE_OPT_TILE_ORDER && (value < -1 || value > 2)) return B200MOE_ERR_ARG;
    if (option == B200MOE_OPT_SM_LIMIT && value < 0) return B200MOE_ERR_ARG;
    g_options[option].store(value);
    return B200MOE_OK;
}

extern "C" int b200moe_get_option(int option) { return option_value(option); }

extern "C" int b200moe_tile_table_lookup(int op, int K, int N, int64_t rows_per_expert) {
    if (op < 0 || op >= B200MOE_OP_COUNT || K <= 0 || N <= 0 || rows_per_expert < 0) return B200MOE_ERR_ARG;
    return tile_table_lookup(op, K, N, rows_per_expert);
}

extern "C" int64_t b200moe_launch_count(void) { return g_launches.load(); }

extern "C" int b200moe_check_status(int32_t* status_device, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(status_device != nullptr, B200MOE_ERR_ARG, "check_status: NULL status");
    int32_t v = 0;
    if (cudaMemcpyAsync(&v, status_device, sizeof(v), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return check_launch("check_status copy");
    if (v != 0) {
        cudaMemsetAsync(status_device, 0, sizeof(v), stream);
        set_error_detail("device status word = %d", v);
        return B200MOE_ERR_DEVICE;
    }
    return B200MOE_OK;
}

// ---- reference-signature operators ---------------------------------------------------------------

extern "C" int64_t b200moe_scatter2scatter_workspace_bytes(int64_t M, int E) {
    // offsets int64 (E) + two int32 row maps (M), each region 16-byte aligned
    int64_t off = ((int64_t)E * 8 + 15) / 16 * 16;
    int64_t map = (M * 4 + 15) / 16 * 16;
    return off + 2 * map;
}

extern "C" int b200moe_scatter2scatter(const void* X, int64_t ldx, const void* W, int64_t w_se, int64_t w_sk,
                                       int64_t w_sn, const int64_t* sorted_expert_idxs,
                                       const int64_t* sorted_scattered_idxs, void* out, int64_t ldo, int64_t M, int K,
                                       int N, int E, int fan_out, int x_grouped, int y_grouped, int dtype,
                                       void* workspace, int64_t workspace_bytes, int32_t* status,
                                       b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(dtype_ok(dtype), B200MOE_ERR_DTYPE, "scatter2scatter: dtype %d", dtype);
    B200MOE_REQUIRE(M >= 0 && K >= 0 && N >= 0 && fan_out > 0, B200MOE_ERR_ARG, "scatter2scatter: bad sizes");
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, "scatter2scatter: E=%d", E);
    if (M == 0 || N == 0) return B200MOE_OK;
    B200MOE_REQUIRE(X && W && out && sorted_expert_idxs && sorted_scattered_idxs, B200MOE_ERR_ARG,
                    "scatter2scatter: NULL pointer");
    B200MOE_REQUIRE(w_sk == 1 || w_sn == 1 || K == 1 || N == 1, B200MOE_ERR_LAYOUT,
                    "scatter2scatter: W needs unit stride along K or N");
    B200MOE_REQUIRE(workspace && workspace_bytes >= b200moe_scatter2scatter_workspace_bytes(M, E),
                    B200MOE_ERR_WORKSPACE, "scatter2scatter: workspace too small");
    char* ws = (char*)workspace;
    int64_t* offsets = (int64_t*)ws;
    int64_t off_bytes = ((int64_t)E * 8 + 15) / 16 * 16, map_bytes = (M * 4 + 15) / 16 * 16;
    int32_t* src_map = (int32_t*)(ws + off_bytes);
    int32_t* dst_map = (int32_t*)(ws + off_bytes + map_bytes);
    int rc = launch_offsets_from_sorted(sorted_expert_idxs, M, E, offsets, stream);
    if (rc) return rc;
    bool need_src = !x_grouped, need_dst = !y_grouped;
    if (need_src || need_dst) {
        rc = launch_make_row_maps(sorted_scattered_idxs, M, fan_out, need_src ? src_map : nullptr,
                                  need_dst ? dst_map : nullptr, stream);
        if (rc) return rc;
    }
    RowGemm g{};
    g.A = X;
    g.lda = ldx;
    g.a_map = need_src ? src_map : nullptr;
    g.a_rows = M;
    g.W = W;
    g.w_se = w_se;
    g.w_sk = w_sk;
    g.w_sn = w_sn;
    g.out = out;
    g.ldo = ldo;
    g.o_map = need_dst ? dst_map : nullptr;
    g.offsets = offsets;
    g.padded = 0;
    g.rows_cap = M;
    g.K = K;
    g.N = N;
    g.E = E;
    g.epi = EPI_STORE;
    return run_row_gemm(g, dtype, status, stream, "scatter2scatter");
}

extern "C" int b200moe_group_bwd_W(const void* DY, int64_t lddy, const void* X, int64_t ldx,
                                   const int64_t* expert_offsets, void* DW, int64_t d_se, int64_t d_sk, int64_t d_sn,
                                   int64_t M, int K, int N, int E, int dtype, int32_t* status,
                                   b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(dtype_ok(dtype), B200MOE_ERR_DTYPE, "group_bwd_W: dtype %d", dtype);
    B200MOE_REQUIRE(M >= 0 && K >= 0 && N >= 0, B200MOE_ERR_ARG, "group_bwd_W: bad sizes");
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, "group_bwd_W: E=%d", E);
    if (K == 0 || N == 0) return B200MOE_OK;
    B200MOE_REQUIRE(DW && expert_offsets && (M == 0 || (DY && X)), B200MOE_ERR_ARG, "group_bwd_W: NULL pointer");
    // DW[e][kk, n] = sum X[r, kk] * DY[r, n].  The operand whose feature index has unit stride in DW becomes
    // the column operand of the engine.
    WGemm g{};
    if (d_sk == 1 && d_sn != 1) {
        g.P = DY, g.ldp = lddy, g.Mout = N, g.d_sm = d_sn;
        g.Q = X, g.ldq = ldx, g.Nout = K, g.d_sn = d_sk;
    } else {
        g.P = X, g.ldp = ldx, g.Mout = K, g.d_sm = d_sk;
        g.Q = DY, g.ldq = lddy, g.Nout = N, g.d_sn = d_sn;
    }
    g.DW = DW;
    g.d_se = d_se;
    g.offsets = expert_offsets;
    g.padded = 0;
    g.rows_cap = M;
    g.E = E;
    return run_w_gemm(g, dtype, status, stream, "group_bwd_W");
}

// ---- fused layer path ----------------------------------------------------------------------------

#define REQUIRE_COMMON(name)                                                                       \
    B200MOE_REQUIRE(dtype_ok(dtype), B200MOE_ERR_DTYPE, name ": dtype %d", dtype);                  \
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, name ": E=%d", E);          \
    B200MOE_REQUIRE(H > 0 && I > 0 && m_cap >= 0 && m_cap % kPadRows == 0, B200MOE_ERR_ARG,         \
                    name ": bad H/I/m_cap (m_cap must be a multiple of 128)")

extern "C" int b200moe_up_forward(const void* x, int64_t ldx, const void* w_fc, const int64_t* expert_offsets,
                                  const int32_t* row_token, void* h, void* a, int64_t T, int H, int I, int E,
                                  int64_t m_cap, int activation, int dtype, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    REQUIRE_COMMON("up_forward");
    B200MOE_REQUIRE(activation == B200MOE_ACT_SWIGLU || activation == B200MOE_ACT_GLU || activation == B200MOE_ACT_GELU_TANH, B200MOE_ERR_ARG,
                    "up_forward: activation %d", activation);
    if (m_cap == 0) return B200MOE_OK;
    B200MOE_REQUIRE(x && w_fc && expert_offsets && h && a && T >= 0, B200MOE_ERR_ARG, "up_forward: NULL pointer");
    const bool gated = activation != B200MOE_ACT_GELU_TANH;
    const int F = gated ? 2 * I : I;  // output features of the up projection
    RowGemm g{};
    g.A = x;
    g.lda = ldx;
    g.a_map = row_token;
    g.a_rows = row_token ? T : m_cap;
    g.W = w_fc;  // (E, F, H): element (e, kk, n) at e*F*H + n*H + kk
    g.w_se = (int64_t)F * H;
    g.w_sk = 1;
    g.w_sn = H;
    g.out = h;
    g.ldo = F;
    g.o_map = nullptr;
    g.offsets = expert_offsets;
    g.padded = 1;
    g.rows_cap = m_cap;
    g.K = H;
    g.N = F;
    g.E = E;
    g.epi = gated ? EPI_SWIGLU : EPI_UNARY;
    g.act = activation;
    g.out2 = a;
    int eng = pick_engine(g, dtype, umma_row_gemm_supported, "up_forward");
    if (eng < 0) return eng;
    if (eng) return umma_row_gemm(g, dtype, status, stream);
    g.epi = EPI_STORE;
    int rc = simt_row_gemm(g, dtype, stream);
    if (rc) return rc;
    if (!gated) return launch_unary_forward(h, I, a, I, m_cap, I, dtype, stream);
    return launch_swiglu_forward(h, 2 * (int64_t)I, a, I, m_cap, I, dtype, stream, activation);
}

extern "C" int b200moe_down_forward(const void* a, const void* w_proj, const int64_t* expert_offsets,
                                    const int32_t* row_slot, const void* gates, void* y_expanded, int64_t ldy,
                                    int64_t M, int H, int I, int E, int64_t m_cap, int dtype, int32_t* status,
                                    b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    REQUIRE_COMMON("down_forward");
    if (m_cap == 0 || M == 0) return B200MOE_OK;
    B200MOE_REQUIRE(a && w_proj && expert_offsets && y_expanded, B200MOE_ERR_ARG, "down_forward: NULL pointer");
    B200MOE_REQUIRE(row_slot != nullptr || gates == nullptr, B200MOE_ERR_ARG,
                    "down_forward: gates are indexed by slot and need row_slot; the grouped output is unweighted");
    RowGemm g{};
    g.A = a;
    g.lda = I;
    g.a_map = nullptr;
    g.W = w_proj;  // (E, H, I): element (e, kk, n) at e*H*I + n*I + kk
    g.w_se = (int64_t)H * I;
    g.w_sk = 1;
    g.w_sn = I;
    g.out = y_expanded;
    g.ldo = ldy;
    g.o_map = row_slot;
    g.scale = gates;
    g.offsets = expert_offsets;
    g.padded = 1;
    g.rows_cap = m_cap;
    g.K = I;
    g.N = H;
    g.E = E;
    g.epi = EPI_STORE;
    return run_row_gemm(g, dtype, status, stream, "down_forward");
}

extern "C" int b200moe_down_dgrad(const void* grad_rows, int64_t ldg, const void* w_proj, const int64_t* expert_offsets,
                                  const int32_t* row_token, const void* h, void* dh, int64_t T, int H, int I, int E,
                                  int64_t m_cap, int activation, int dtype, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    REQUIRE_COMMON("down_dgrad");
    B200MOE_REQUIRE(activation == B200MOE_ACT_SWIGLU || activation == B200MOE_ACT_GLU || activation == B200MOE_ACT_GELU_TANH, B200MOE_ERR_ARG,
                    "down_dgrad: activation %d", activation);
    if (m_cap == 0) return B200MOE_OK;
    B200MOE_REQUIRE(grad_rows && w_proj && expert_offsets && h && dh && T >= 0, B200MOE_ERR_ARG, "down_dgrad: NULL pointer");
    const bool gated = activation != B200MOE_ACT_GELU_TANH;
    RowGemm g{};
    g.A = grad_rows;
    g.lda = ldg;
    g.a_map = row_token;
    g.a_rows = row_token ? T : m_cap;
    g.W = w_proj;  // reduction over H now: element (e, kk=h, n=i) at e*H*I + kk*I + n
    g.w_se = (int64_t)H * I;
    g.w_sk = I;
    g.w_sn = 1;
    g.out = dh;
    g.ldo = gated ? 2 * (int64_t)I : I;
    g.o_map = nullptr;
    g.offsets = expert_offsets;
    g.padded = 1;
    g.rows_cap = m_cap;
    g.K = H;
    g.N = I;
    g.E = E;
    g.epi = gated ? EPI_DGRAD_DOWN : EPI_DGRAD_UNARY;
    g.act = activation;
    g.h = h;
    int eng = pick_engine(g, dtype, umma_row_gemm_supported, "down_dgrad");
    if (eng < 0) return eng;
    if (eng) return umma_row_gemm(g, dtype, status, stream);
    // CUDA-core engine: d into (the first half of) every dh row, then the element-wise tail in place
    g.epi = EPI_STORE;
    int rc = simt_row_gemm(g, dtype, stream);
    if (rc) return rc;
    if (!gated) return launch_unary_backward(h, I, dh, I, m_cap, I, dtype, stream);
    return launch_dgrad_down_post(h, dh, m_cap, I, dtype, stream, activation);
}

extern "C" int b200moe_wgrad(const void* P, int64_t ldp, const int32_t* p_map, const void* Q, int64_t ldq,
                             const int32_t* q_map, const int64_t* expert_offsets, void* DW, int n_out, int n_in, int E,
                             int64_t m_cap, int dtype, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(dtype_ok(dtype), B200MOE_ERR_DTYPE, "wgrad: dtype %d", dtype);
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, "wgrad: E=%d", E);
    B200MOE_REQUIRE(n_out > 0 && n_in > 0 && m_cap >= 0, B200MOE_ERR_ARG, "wgrad: bad sizes");
    B200MOE_REQUIRE(P && Q && DW && expert_offsets, B200MOE_ERR_ARG, "wgrad: NULL pointer");
    WGemm g{};
    g.P = P;
    g.ldp = ldp;
    g.p_map = p_map;
    g.Q = Q;
    g.ldq = ldq;
    g.q_map = q_map;
    g.map_rows = m_cap;
    g.DW = DW;
    g.d_se = (int64_t)n_out * n_in;
    g.d_sm = n_in;
    g.d_sn = 1;
    g.offsets = expert_offsets;
    g.padded = 1;
    g.rows_cap = m_cap;
    g.Mout = n_out;
    g.Nout = n_in;
    g.E = E;
    return run_w_gemm(g, dtype, status, stream, "wgrad");
}

extern "C" int b200moe_up_dgrad(const void* dh, const void* w_fc, const int64_t* expert_offsets,
                                const int32_t* row_slot, void* dx_expanded, int64_t ldd, int64_t M, int H, int I,
                                int E, int64_t m_cap, int dtype, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    REQUIRE_COMMON("up_dgrad");
    if (m_cap == 0 || M == 0) return B200MOE_OK;
    B200MOE_REQUIRE(dh && w_fc && expert_offsets && dx_expanded, B200MOE_ERR_ARG, "up_dgrad: NULL pointer");
    RowGemm g{};
    g.A = dh;
    g.lda = 2 * (int64_t)I;
    g.a_map = nullptr;
    g.W = w_fc;  // reduction over 2I: element (e, kk, n=h) at e*2I*H + kk*H + n
    g.w_se = (int64_t)2 * I * H;
    g.w_sk = H;
    g.w_sn = 1;
    g.out = dx_expanded;
    g.ldo = ldd;
    g.o_map = row_slot;
    g.offsets = expert_offsets;
    g.padded = 1;
    g.rows_cap = m_cap;
    g.K = 2 * I;
    g.N = H;
    g.E = E;
    g.epi = EPI_STORE;
    return run_row_gemm(g, dtype, status, stream, "up_dgrad");
}

// ---- fused router ---------------------------------------------------------------------------------

extern "C" int b200moe_router_forward_scaled(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, const float* row_scale,
                                             int64_t T, int H, int E, int k, int scoring, void* logits, int64_t ldl, void* weights,
                                             int64_t* indices, int32_t* counts, int dtype, int32_t* status,
                                             b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(dtype == B200MOE_BF16 || dtype == B200MOE_F16, B200MOE_ERR_DTYPE,
                    "router_forward: 16-bit tensors only (dtype %d); route fp32 tensors with the eager router", dtype);
    B200MOE_REQUIRE(T >= 0 && T < ((int64_t)1 << 31) && H > 0 && E > 0, B200MOE_ERR_ARG, "router_forward: bad sizes");
    B200MOE_REQUIRE(E <= 256 && k >= 1 && k <= 8 && k <= E, B200MOE_ERR_UNSUPPORTED,
                    "router_forward: at most 256 experts and 8 experts per token (E=%d k=%d)", E, k);
    B200MOE_REQUIRE(scoring == 0 || scoring == 1, B200MOE_ERR_ARG, "router_forward: scoring must be 0 (softmax) or 1 (sigmoid)");
    B200MOE_REQUIRE(counts != nullptr, B200MOE_ERR_ARG, "router_forward: NULL pointer");
    cudaError_t err = cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, stream);
    B200MOE_REQUIRE(err == cudaSuccess, B200MOE_ERR_LAUNCH, "router_forward: memset: %s", cudaGetErrorString(err));
    if (T == 0) return B200MOE_OK;
    B200MOE_REQUIRE(x && gate_w && logits && weights && indices, B200MOE_ERR_ARG, "router_forward: NULL pointer");
    B200MOE_REQUIRE(H % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= H && ldw >= H && ldl >= E &&
                        ((uintptr_t)x & 15) == 0 && ((uintptr_t)gate_w & 15) == 0,
                    B200MOE_ERR_LAYOUT, "router_forward: rows of x and of the gate weight must be 16-byte aligned multiples of 16 bytes");
    return umma_router(x, ldx, gate_w, ldw, T, H, E, k, scoring, row_scale, logits, ldl, weights, indices, counts, dtype, status, stream);
}

extern "C" int b200moe_router_forward(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, int64_t T, int H, int E,
                                      int k, int scoring, void* logits, int64_t ldl, void* weights, int64_t* indices,
                                      int32_t* counts, int dtype, int32_t* status, b200moe_stream_t stream) {
    return b200moe_router_forward_scaled(x, ldx, gate_w, ldw, nullptr, T, H, E, k, scoring, logits, ldl, weights, indices, counts, dtype,
                                         status, stream);
}
