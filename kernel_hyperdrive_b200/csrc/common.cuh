// Shared definitions of the b200moe CUDA sources: element-type helpers, the two grouped-GEMM problem
// descriptions every engine consumes, and the host-side error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

constexpr int kMaxExperts = B200MOE_MAX_EXPERTS;
constexpr int kPadRows = 128;  // every expert segment of the padded grouped order starts at a multiple of this

// ---- host-side error plumbing -------------------------------------------------------------------
void set_error_detail(const char* fmt, ...);
void count_launch(int n = 1);
int check_launch(const char* what);  // cudaGetLastError -> B200MOE_ERR_LAUNCH with detail

#define B200MOE_REQUIRE(cond, code, ...)            \
    do {                                            \
        if (!(cond)) {                              \
            ::b200moe::set_error_detail(__VA_ARGS__); \
            return (code);                          \
        }                                           \
    } while (0)

// ---- element types ------------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

static inline int dtype_size(int dtype) { return dtype == B200MOE_F32 ? 4 : 2; }

// Logistic function split by sign so that exp never overflows.
__device__ __forceinline__ float sigmoidf_stable(float x) {
    if (x >= 0.f) {
        return 1.f / (1.f + __expf(-x));
    }
    float e = __expf(x);
    return e / (1.f + e);
}

// 16-bit tensors round the result to 8 or 11 mantissa bits anyway: the fast exponential and division are exact
// enough there and cut the instruction count of the element-wise kernels (the accurate form costs a branch and an
// IEEE division per element).  fp32 tensors keep the accurate form.
template <typename T>
__device__ __forceinline__ float sigmoid_for(float x) {
    return __fdividef(1.f, 1.f + __expf(-x));
}
template <>
__device__ __forceinline__ float sigmoid_for<float>(float x) {
    return sigmoidf_stable(x);
}

// Gated activations of the fused expert path: a = up * m(gate).  ACT_SILU: m(g) = g * sigmoid(g) (SwiGLU);
// ACT_SIGMOID: m(g) = sigmoid(g) (GLU).  `sg` is sigmoid(g).
enum { ACT_SILU = 0, ACT_SIGMOID = 1 };
__device__ __forceinline__ float gate_value(int act, float g, float sg) { return act == ACT_SIGMOID ? sg : g * sg; }
__device__ __forceinline__ float gate_slope(int act, float g, float sg) {
    return act == ACT_SIGMOID ? sg * (1.f - sg) : sg + g * sg * (1.f - sg);
}

// ---- segment layout -----------------------------------------------------------------------------
// Both problem descriptions address rows through a "segment layout": expert e owns layout rows
// [seg_start(e), seg_start(e) + count(e)), where count comes from the inclusive int64 offsets and
// seg_start(e) is offsets[e-1] (grouped order) or 128 * sum_{e'<e} ceil(count(e') / 128) (padded grouped).

// Family R: out[dst(p), n] = scale(p) * sum_k A[src(p), k] * W[e(p)][k, n]
struct RowGemm {
    const void* A;
    int64_t lda;
    const int32_t* a_map;  // layout row -> row of A (negative: zero row); NULL: identity
    int64_t a_rows;        // upper bound of the rows of A that a_map can name (tensor-map extent of the row gather)
    const void* W;
    int64_t w_se, w_sk, w_sn;  // element strides of W (E, K, N); one of w_sk, w_sn is 1
    void* out;
    int64_t ldo;
    const int32_t* o_map;  // layout row -> row of out (negative: skip); NULL: identity
    const void* scale;     // element type of the call; indexed by the out row; NULL: 1
    const int64_t* offsets;
    int padded;
    int64_t rows_cap;  // upper bound of layout rows (grid sizing)
    int K, N, E;
    // fused epilogues (tcgen05 engine only)
    int epi;               // EPI_STORE, EPI_SWIGLU (gated forward), EPI_DGRAD_DOWN (gated dgrad), EPI_UNARY, EPI_DGRAD_UNARY
    int act;               // gated activation of epilogues 1 and 2 (ACT_SILU, ACT_SIGMOID)
    void* out2;            // SwiGLU: activation output a (rows_cap, N/2)
    const void* h;         // dgrad: pre-activation (rows_cap, 2N) as the SwiGLU epilogue of the same engine stored it
};

// Family W: DW[e][m, n] = sum_{p in segment e} P[pmap(p), m] * Q[qmap(p), n]
struct WGemm {
    const void* P;
    int64_t ldp;
    const int32_t* p_map;
    const void* Q;
    int64_t ldq;
    const int32_t* q_map;
    int64_t map_rows;  // upper bound of the rows p_map / q_map can name
    void* DW;
    int64_t d_se, d_sm, d_sn;
    const int64_t* offsets;
    int padded;
    int64_t rows_cap;  // rows of P / Q when they are indexed by layout rows (tensor-map extent)
    int Mout, Nout, E;
};

// Un-gated activation of a plain (non-GLU) expert: a = f(h).  UNARY_GELU_TANH: the tanh form of GELU
// (torch.nn.GELU(approximate="tanh"), the activation of the reference's non-GLU layer test).  `th` is
// tanh(sqrt(2/pi) * (x + 0.044715 x^3)), supplied by the caller (hardware approximation for 16-bit tensors, tanhf for fp32).
enum { UNARY_GELU_TANH = 2 };
__device__ __forceinline__ float gelu_tanh_arg(float x) { return 0.7978845608028654f * (x + 0.044715f * x * x * x); }
__device__ __forceinline__ float gelu_tanh_value(float x, float th) { return 0.5f * x * (1.f + th); }
__device__ __forceinline__ float gelu_tanh_slope(float x, float th) {
    return 0.5f * (1.f + th) + 0.5f * x * (1.f - th * th) * 0.7978845608028654f * (1.f + 0.134145f * x * x);
}

// Epilogues of the tensor-core kernels (template arguments).  The two gated-activation epilogues exist once per gate
// function so that the choice costs nothing at run time; RowGemm names them as (EPI_SWIGLU or EPI_DGRAD_DOWN, act).
// EPI_UNARY / EPI_DGRAD_UNARY are the forward / input-gradient epilogues of a non-GLU expert (a = gelu_tanh(h)).
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_DGRAD_DOWN = 2, EPI_ROUTER = 3, EPI_GLU = 4, EPI_DGRAD_DOWN_GLU = 5, EPI_UNARY = 6, EPI_DGRAD_UNARY = 7 };
__host__ __device__ constexpr bool epi_gated_forward(int epi) { return epi == EPI_SWIGLU || epi == EPI_GLU; }
__host__ __device__ constexpr bool epi_gated_dgrad(int epi) { return epi == EPI_DGRAD_DOWN || epi == EPI_DGRAD_DOWN_GLU; }
__host__ __device__ constexpr int epi_act(int epi) { return (epi == EPI_GLU || epi == EPI_DGRAD_DOWN_GLU) ? 1 : 0; }

// engines
int simt_row_gemm(const RowGemm& g, int dtype, cudaStream_t stream);
int simt_w_gemm(const WGemm& g, int dtype, cudaStream_t stream);
bool umma_row_gemm_supported(const RowGemm& g, int dtype);
bool umma_w_gemm_supported(const WGemm& g, int dtype);
int umma_row_gemm(const RowGemm& g, int dtype, int32_t* status, cudaStream_t stream);
int umma_w_gemm(const WGemm& g, int dtype, int32_t* status, cudaStream_t stream);
int umma_router(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, int64_t T, int H, int E, int k, int scoring,
                const float* row_scale, void* logits, int64_t ldl, void* weights, int64_t* indices, int32_t* counts, int dtype,
                int32_t* status, cudaStream_t stream);

// row-wise kernels used by the API layer
int launch_swiglu_forward(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int h, int dtype,
                          cudaStream_t stream, int act = ACT_SILU);
int launch_swiglu_backward(const void* x, int64_t ldx, const void* dy, int64_t lddy, void* dx, int64_t lddx,
                           int64_t rows, int h, int dtype, cudaStream_t stream);
int launch_dgrad_down_post(const void* h, void* dh, int64_t rows, int I, int dtype, cudaStream_t stream, int act = ACT_SILU);
// a = gelu_tanh(h) on (rows, width) tensors, and dh = d * gelu_tanh'(h) in place on dh (which holds d on entry)
int launch_unary_forward(const void* h, int64_t ldh, void* a, int64_t lda, int64_t rows, int width, int dtype, cudaStream_t stream);
int launch_unary_backward(const void* h, int64_t ldh, void* dh, int64_t ldd, int64_t rows, int width, int dtype, cudaStream_t stream);

int current_engine();
int option_value(int option);
// The per-shape tile table: which tensor-core tile (B200MOE_TILE_*) a launch of `op` (B200MOE_OP_*) with reduction
// extent K, N output columns and about rows_per_expert rows per expert uses.
int tile_table_lookup(int op, int K, int N, int64_t rows_per_expert);

}  // namespace b200moe
