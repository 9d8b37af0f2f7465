// RMSNorm forward and backward (the normalisation that feeds the MoE layer's input in a transformer block).
//   y = x * rstd * w,  rstd = 1 / sqrt(mean(x^2) + eps)                       (w optional)
//   dx = rstd * (dy*w) - x * rstd^3 * mean((dy*w) * x),   dw = sum_rows dy * x * rstd
// HBM-bound row kernels.  Fast path (rows a multiple of 16 bytes wide, 16-byte aligned): a group of 32, 128 or 512
// threads owns a row and keeps it in registers as 16-byte vectors, so every element is read once; small groups with
// several vectors per thread keep many independent loads in flight and confine the reduction's barrier to four warps.
// Forward: one group per row.  Backward: groups walk the rows with a grid stride so that the weight vector and the
// weight-gradient partial sums stay in registers across rows; the partial sums (one fp32 row per group) go to a
// caller-provided workspace and a second kernel adds them up in a fixed order: no atomics, deterministic.
// Generic path (any width / alignment): one 128-thread block per row, scalar accesses, the row is read twice
// (the second read hits L1/L2); weight-gradient contributions are added with fp32 atomics into one workspace row.
#include "common.cuh"

namespace b200moe {
namespace umma {
int sm_count();
}

namespace {

template <typename T, int V>
struct alignas(sizeof(T) * V) Vec {
    T v[V];
};

__host__ __device__ constexpr int block_threads(int G) { return G < 128 ? 128 : G; }

// sum over the 128 threads of a block (generic path)
__device__ __forceinline__ float block_sum_128(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();  // smem may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    return smem[0] + smem[1] + smem[2] + smem[3];
}

// N sums at once, each over a group of G consecutive threads of the block (G = 32: shuffles only; otherwise one
// barrier round for the whole block, so every thread of the block must call it the same number of times)
template <int G, int N>
__device__ __forceinline__ void group_sum_n(float (&v)[N], float* smem) {
#pragma unroll
    for (int n = 0; n < N; ++n) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v[n] += __shfl_xor_sync(0xffffffffu, v[n], o);
    }
    if (G == 32) return;
    constexpr int WG = G / 32;  // warps per group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int n = 0; n < N; ++n) smem[warp * N + n] = v[n];
    }
    __syncthreads();
    const int w0 = (warp / WG) * WG;
#pragma unroll
    for (int n = 0; n < N; ++n) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < WG; ++i) t += smem[(w0 + i) * N + n];
        v[n] = t;
    }
}

// ---- fast path -------------------------------------------------------------------------------------
// A group of G threads owns a row (NV 16-byte vectors per thread); a block holds 128 / G groups (one when G >= 128).
// RP consecutive rows per group and iteration.  The loop is uniform over the block (rows past the end are masked),
// which the block-wide barrier of the reduction needs.
template <typename T, int NV, int RP, int G>
__global__ void __launch_bounds__(block_threads(G)) rmsnorm_fwd_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                                      T* __restrict__ y, int64_t ldy, float* __restrict__ rstd,
                                                                      int64_t rows, int H, float eps) {
    constexpr int V = 16 / sizeof(T);
    constexpr int GPB = block_threads(G) / G;
    using VT = Vec<T, V>;
    __shared__ float red[32 * RP];
    const int gid = threadIdx.x / G, gtid = threadIdx.x % G;
    VT wv[NV];
    if (w) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            int c = (gtid + i * G) * V;
            if (c < H) wv[i] = *reinterpret_cast<const VT*>(w + c);
        }
    }
    for (int64_t base = (int64_t)blockIdx.x * GPB * RP; base < rows; base += (int64_t)gridDim.x * GPB * RP) {
        const int64_t row0 = base + gid * RP;
        VT xv[RP][NV];
        float ss[RP];
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                int c = (gtid + i * G) * V;
                if (row0 + rp < rows && c < H) xv[rp][i] = *reinterpret_cast<const VT*>(x + (row0 + rp) * ldx + c);
            }
        }
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
            ss[rp] = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                int c = (gtid + i * G) * V;
                if (row0 + rp < rows && c < H) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        float f = Elem<T>::to_f(xv[rp][i].v[j]);
                        ss[rp] += f * f;
                    }
                }
            }
        }
        group_sum_n<G, RP>(ss, red);
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
            const int64_t row = row0 + rp;
            if (row < rows) {
                const float r = rsqrtf(ss[rp] / (float)H + eps);
                if (rstd && gtid == 0) rstd[row] = r;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    int c = (gtid + i * G) * V;
                    if (c < H) {
                        VT o;
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            float f = Elem<T>::to_f(xv[rp][i].v[j]) * r;
                            if (w) f *= Elem<T>::to_f(wv[i].v[j]);
                            o.v[j] = Elem<T>::from_f(f);
                        }
                        *reinterpret_cast<VT*>(y + row * ldy + c) = o;
                    }
                }
            }
        }
    }
}

// The weight-gradient partial sums of a thread's columns stay in registers across all rows the group handles and go to
// row (blockIdx.x * GPB + gid) of `partial` at the end.
template <typename T, int NV, int RP, int G>
__global__ void __launch_bounds__(block_threads(G)) rmsnorm_bwd_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                                      const T* __restrict__ dy, int64_t lddy,
                                                                      const float* __restrict__ rstd, T* __restrict__ dx,
                                                                      int64_t lddx, float* __restrict__ partial, int64_t rows,
                                                                      int H, float eps) {
    constexpr int V = 16 / sizeof(T);
    constexpr int GPB = block_threads(G) / G;
    using VT = Vec<T, V>;
    __shared__ float red[32 * 2 * RP];
    const int gid = threadIdx.x / G, gtid = threadIdx.x % G;
    VT wv[NV];
    float dw[NV][V];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        int c = (gtid + i * G) * V;
        if (w && c < H) wv[i] = *reinterpret_cast<const VT*>(w + c);
#pragma unroll
        for (int j = 0; j < V; ++j) dw[i][j] = 0.f;
    }
    for (int64_t base = (int64_t)blockIdx.x * GPB * RP; base < rows; base += (int64_t)gridDim.x * GPB * RP) {
        const int64_t row0 = base + gid * RP;
        VT xv[RP][NV], gv[RP][NV];
        float sums[2 * RP];  // [rp]: sum of squares, [RP + rp]: sum of (dy*w) * x
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                int c = (gtid + i * G) * V;
                if (row0 + rp < rows && c < H) {
                    xv[rp][i] = *reinterpret_cast<const VT*>(x + (row0 + rp) * ldx + c);
                    gv[rp][i] = *reinterpret_cast<const VT*>(dy + (row0 + rp) * lddy + c);
                }
            }
        }
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
            float ss = 0.f, dot = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                int c = (gtid + i * G) * V;
                if (row0 + rp < rows && c < H) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        float f = Elem<T>::to_f(xv[rp][i].v[j]), g = Elem<T>::to_f(gv[rp][i].v[j]);
                        if (w) g *= Elem<T>::to_f(wv[i].v[j]);
                        ss += f * f;
                        dot += f * g;
                    }
                }
            }
            sums[rp] = ss;
            sums[RP + rp] = dot;
        }
        group_sum_n<G, 2 * RP>(sums, red);
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
            const int64_t row = row0 + rp;
            if (row < rows) {
                const float r = rstd ? rstd[row] : rsqrtf(sums[rp] / (float)H + eps);
                const float coef = sums[RP + rp] * r * r * r / (float)H;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    int c = (gtid + i * G) * V;
                    if (c < H) {
                        VT o;
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            float f = Elem<T>::to_f(xv[rp][i].v[j]), g0 = Elem<T>::to_f(gv[rp][i].v[j]);
                            float g = w ? g0 * Elem<T>::to_f(wv[i].v[j]) : g0;
                            o.v[j] = Elem<T>::from_f(r * g - f * coef);
                            dw[i][j] += g0 * f * r;
                        }
                        *reinterpret_cast<VT*>(dx + row * lddx + c) = o;
                    }
                }
            }
        }
    }
    if (partial) {
        float* prow = partial + ((int64_t)blockIdx.x * GPB + gid) * H;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            int c = (gtid + i * G) * V;
            if (c < H) {
#pragma unroll
                for (int j = 0; j < V; j += 4) *reinterpret_cast<float4*>(prow + c + j) = make_float4(dw[i][j], dw[i][j + 1], dw[i][j + 2], dw[i][j + 3]);
            }
        }
    }
}

// dw[c] = sum over the partial rows, added in row order by 8 row lanes and then across the lanes: fixed order
template <typename T>
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, int64_t prows, T* __restrict__ dw, int H) {
    __shared__ float acc[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (c < H)
        for (int64_t p = threadIdx.y; p < prows; p += 8) s += partial[p * H + c];
    acc[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < H) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += acc[i][threadIdx.x];
        dw[c] = Elem<T>::from_f(t);
    }
}

// ---- generic path ------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_fwd_generic_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w, T* __restrict__ y,
                                           int64_t ldy, float* __restrict__ rstd, int64_t rows, int H, float eps) {
    __shared__ float red[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < H; c += 128) {
            float f = Elem<T>::to_f(x[row * ldx + c]);
            ss += f * f;
        }
        ss = block_sum_128(ss, red);
        const float r = rsqrtf(ss / (float)H + eps);
        if (rstd && threadIdx.x == 0) rstd[row] = r;
        for (int c = threadIdx.x; c < H; c += 128) {
            float f = Elem<T>::to_f(x[row * ldx + c]) * r;
            if (w) f *= Elem<T>::to_f(w[c]);
            y[row * ldy + c] = Elem<T>::from_f(f);
        }
    }
}

template <typename T>
__global__ void rmsnorm_bwd_generic_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                           const T* __restrict__ dy, int64_t lddy, const float* __restrict__ rstd,
                                           T* __restrict__ dx, int64_t lddx, float* __restrict__ partial, int64_t rows, int H,
                                           float eps) {
    __shared__ float red[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float ss = 0.f, dot = 0.f;
        for (int c = threadIdx.x; c < H; c += 128) {
            float f = Elem<T>::to_f(x[row * ldx + c]), g = Elem<T>::to_f(dy[row * lddy + c]);
            if (w) g *= Elem<T>::to_f(w[c]);
            ss += f * f;
            dot += f * g;
        }
        ss = block_sum_128(ss, red);
        dot = block_sum_128(dot, red);
        const float r = rstd ? rstd[row] : rsqrtf(ss / (float)H + eps);
        const float coef = dot * r * r * r / (float)H;
        for (int c = threadIdx.x; c < H; c += 128) {
            float f = Elem<T>::to_f(x[row * ldx + c]), g0 = Elem<T>::to_f(dy[row * lddy + c]);
            float g = w ? g0 * Elem<T>::to_f(w[c]) : g0;
            dx[row * lddx + c] = Elem<T>::from_f(r * g - f * coef);
            if (partial) atomicAdd(partial + c, g0 * f * r);
        }
    }
}

// ---- launch geometry ---------------------------------------------------------------------------------
struct Geometry {
    bool fast;
    int G, NV;  // threads per row, 16-byte vectors per thread and row
};

constexpr int RP = 1;  // rows per group and iteration

// Measured on B200 (bf16, 2048 to 8192 columns): 128 threads per row are fastest forward at every width and backward up
// to 512 vectors per row; wider rows run backward faster with 512 threads (fewer partial sums per thread, more threads
// resident).
Geometry geometry(int H, int dtype, bool aligned, bool backward) {
    Geometry g{};
    const int V = 16 / dtype_size(dtype);
    const int vecs = (H + V - 1) / V;
    g.fast = aligned && H % V == 0 && vecs <= 512 * 8;
    if (!g.fast) return g;
    g.G = vecs <= 128 ? 32 : (vecs <= (backward ? 512 : 1024) ? 128 : 512);
    const int per = (vecs + g.G - 1) / g.G;
    g.NV = g.G == 32 ? 1 : 2;
    while (g.NV < per) g.NV *= 2;
    return g;
}

// everything one call needs; `what` selects forward, backward, or only the sizing of the backward launch
enum { DO_FORWARD = 0, DO_BACKWARD = 1, DO_PLAN = 2 };
struct Call {
    const void* x;
    int64_t ldx;
    const void* w;
    void* y;  // forward: output; backward: dx
    int64_t ldy;
    const void* dy;
    int64_t lddy;
    float* rstd;
    float* partial;
    int64_t rows;
    int H;
    float eps;
    cudaStream_t stream;
    int grid;              // out (backward / plan)
    int64_t partial_rows;  // out (backward / plan)
};

int generic_grid(int64_t rows) {
    const int64_t cap = (int64_t)umma::sm_count() * 8;
    return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

template <typename T, int NV, int G>
int exec(Call& c, int what) {
    constexpr int threads = block_threads(G), gpb = threads / G;
    int64_t need = (c.rows + (int64_t)gpb * RP - 1) / ((int64_t)gpb * RP);
    if (need < 1) need = 1;
    if (what == DO_FORWARD) {
        // one group per row: the block scheduler keeps the SMs full
        const int grid = (int)(need < (1 << 30) ? need : (1 << 30));
        rmsnorm_fwd_kernel<T, NV, RP, G><<<grid, threads, 0, c.stream>>>((const T*)c.x, c.ldx, (const T*)c.w, (T*)c.y, c.ldy, c.rstd, c.rows, c.H, c.eps);
        return B200MOE_OK;
    }
    // backward: persistent grid of the blocks resident at once (occupancy of this instantiation)
    auto kern = rmsnorm_bwd_kernel<T, NV, RP, G>;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    const int64_t cap = (int64_t)umma::sm_count() * per_sm;
    c.grid = (int)(need < cap ? need : cap);
    c.partial_rows = (int64_t)c.grid * gpb;
    if (what == DO_BACKWARD)
        kern<<<c.grid, threads, 0, c.stream>>>((const T*)c.x, c.ldx, (const T*)c.w, (const T*)c.dy, c.lddy, c.rstd, (T*)c.y, c.ldy, c.partial, c.rows, c.H, c.eps);
    return B200MOE_OK;
}

template <typename T>
int dispatch(const Geometry& g, Call& c, int what) {
    if (!g.fast) {
        c.grid = generic_grid(c.rows);
        c.partial_rows = 1;
        if (what == DO_FORWARD)
            rmsnorm_fwd_generic_kernel<T><<<c.grid, 128, 0, c.stream>>>((const T*)c.x, c.ldx, (const T*)c.w, (T*)c.y, c.ldy, c.rstd, c.rows, c.H, c.eps);
        if (what == DO_BACKWARD)
            rmsnorm_bwd_generic_kernel<T><<<c.grid, 128, 0, c.stream>>>((const T*)c.x, c.ldx, (const T*)c.w, (const T*)c.dy, c.lddy, c.rstd, (T*)c.y, c.ldy, c.partial, c.rows, c.H, c.eps);
        return B200MOE_OK;
    }
    switch (g.G * 16 + g.NV) {  // the (G, NV) pairs `geometry` produces
        case 32 * 16 + 1: return exec<T, 1, 32>(c, what);
        case 32 * 16 + 2: return exec<T, 2, 32>(c, what);
        case 32 * 16 + 4: return exec<T, 4, 32>(c, what);
        case 128 * 16 + 2: return exec<T, 2, 128>(c, what);
        case 128 * 16 + 4: return exec<T, 4, 128>(c, what);
        case 128 * 16 + 8: return exec<T, 8, 128>(c, what);
        case 512 * 16 + 2: return exec<T, 2, 512>(c, what);
        case 512 * 16 + 4: return exec<T, 4, 512>(c, what);
        case 512 * 16 + 8: return exec<T, 8, 512>(c, what);
    }
    set_error_detail("rmsnorm: no kernel for G=%d NV=%d", g.G, g.NV);
    return B200MOE_ERR_UNSUPPORTED;
}

int dispatch_dtype(int dtype, const Geometry& g, Call& c, int what) {
    if (dtype == B200MOE_F32) return dispatch<float>(g, c, what);
    if (dtype == B200MOE_BF16) return dispatch<__nv_bfloat16>(g, c, what);
    return dispatch<__half>(g, c, what);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
bool dtype_known(int dtype) { return dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32; }

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int64_t b200moe_rmsnorm_workspace_bytes(int64_t rows, int H, int dtype) {
    if (rows < 0 || H <= 0 || !dtype_known(dtype)) return 0;
    Call c{};
    c.rows = rows;
    c.H = H;
    Geometry g = geometry(H, dtype, true, true);  // the 16-byte path writes the most partial rows; the generic path one
    if (dispatch_dtype(dtype, g, c, DO_PLAN) != B200MOE_OK || c.partial_rows < 1) c.partial_rows = 1;
    return c.partial_rows * H * (int64_t)sizeof(float);
}

extern "C" int b200moe_rmsnorm_forward(const void* x, int64_t ldx, const void* weight, void* y, int64_t ldy, float* rstd,
                                       int64_t rows, int H, float eps, int dtype, b200moe_stream_t stream_) {
    B200MOE_REQUIRE(dtype_known(dtype), B200MOE_ERR_DTYPE, "rmsnorm_forward: dtype %d", dtype);
    B200MOE_REQUIRE(rows >= 0 && H > 0, B200MOE_ERR_ARG, "rmsnorm_forward: bad sizes");
    if (rows == 0) return B200MOE_OK;
    B200MOE_REQUIRE(x && y && ldx >= H && ldy >= H, B200MOE_ERR_ARG, "rmsnorm_forward: NULL pointer or row stride below the width");
    const int V = 16 / dtype_size(dtype);
    const bool al = aligned16(x) && aligned16(y) && aligned16(weight) && ldx % V == 0 && ldy % V == 0;
    Call c{};
    c.x = x, c.ldx = ldx, c.w = weight, c.y = y, c.ldy = ldy, c.rstd = rstd, c.rows = rows, c.H = H, c.eps = eps;
    c.stream = (cudaStream_t)stream_;
    int rc = dispatch_dtype(dtype, geometry(H, dtype, al, false), c, DO_FORWARD);
    if (rc) return rc;
    count_launch();
    return check_launch("rmsnorm_forward");
}

extern "C" int b200moe_rmsnorm_backward(const void* x, int64_t ldx, const void* weight, const void* dy, int64_t lddy,
                                        const float* rstd, void* dx, int64_t lddx, void* dweight, void* workspace,
                                        int64_t workspace_bytes, int64_t rows, int H, float eps, int dtype,
                                        b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(dtype_known(dtype), B200MOE_ERR_DTYPE, "rmsnorm_backward: dtype %d", dtype);
    B200MOE_REQUIRE(rows >= 0 && H > 0, B200MOE_ERR_ARG, "rmsnorm_backward: bad sizes");
    B200MOE_REQUIRE(!dweight || weight, B200MOE_ERR_ARG, "rmsnorm_backward: a weight gradient needs the weight");
    const int esz = dtype_size(dtype);
    if (rows == 0) {  // no rows: the weight gradient is zero, nothing else to write
        if (dweight) {
            cudaError_t err = cudaMemsetAsync(dweight, 0, (size_t)H * esz, stream);
            B200MOE_REQUIRE(err == cudaSuccess, B200MOE_ERR_LAUNCH, "rmsnorm_backward: memset: %s", cudaGetErrorString(err));
        }
        return B200MOE_OK;
    }
    B200MOE_REQUIRE(x && dy && dx && ldx >= H && lddy >= H && lddx >= H, B200MOE_ERR_ARG,
                    "rmsnorm_backward: NULL pointer or row stride below the width");
    const int V = 16 / esz;
    const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(weight) && aligned16(workspace) && ldx % V == 0 &&
                    lddy % V == 0 && lddx % V == 0;
    Geometry g = geometry(H, dtype, al, true);
    Call c{};
    c.x = x, c.ldx = ldx, c.w = weight, c.y = dx, c.ldy = lddx, c.dy = dy, c.lddy = lddy, c.rstd = const_cast<float*>(rstd);
    c.rows = rows, c.H = H, c.eps = eps, c.stream = stream;
    if (dweight) {
        int rc = dispatch_dtype(dtype, g, c, DO_PLAN);
        if (rc) return rc;
        const int64_t need = c.partial_rows * H * (int64_t)sizeof(float);
        B200MOE_REQUIRE(workspace && workspace_bytes >= need, B200MOE_ERR_WORKSPACE, "rmsnorm_backward: workspace of %lld bytes needed",
                        (long long)need);
        c.partial = (float*)workspace;
        if (!g.fast) {  // the generic path accumulates with atomics
            cudaError_t err = cudaMemsetAsync(c.partial, 0, sizeof(float) * H, stream);
            B200MOE_REQUIRE(err == cudaSuccess, B200MOE_ERR_LAUNCH, "rmsnorm_backward: memset: %s", cudaGetErrorString(err));
        }
    }
    int rc = dispatch_dtype(dtype, g, c, DO_BACKWARD);
    if (rc) return rc;
    count_launch();
    rc = check_launch("rmsnorm_backward");
    if (rc || !dweight) return rc;
    dim3 block(32, 8);
    const int blocks = (H + 31) / 32;
    if (dtype == B200MOE_F32) {
        rmsnorm_dw_reduce_kernel<float><<<blocks, block, 0, stream>>>(c.partial, c.partial_rows, (float*)dweight, H);
    } else if (dtype == B200MOE_BF16) {
        rmsnorm_dw_reduce_kernel<__nv_bfloat16><<<blocks, block, 0, stream>>>(c.partial, c.partial_rows, (__nv_bfloat16*)dweight, H);
    } else {
        rmsnorm_dw_reduce_kernel<__half><<<blocks, block, 0, stream>>>(c.partial, c.partial_rows, (__half*)dweight, H);
    }
    count_launch();
    return check_launch("rmsnorm_dw_reduce");
}
