// Row-wise, HBM-bound kernels of the path: row gather with coefficient (`group`), the gathers into the padded grouped
// order (tokens; gate-scaled upstream gradient rows with the gate gradient), the sum over the k slots of a token
// (`combine`), SwiGLU forward / backward on a fused (rows, 2h) tensor, and the element-wise tail of the
// down-projection input gradient used by the CUDA-core engine.
// All of them move 16 bytes per thread access when pointers, row strides and widths allow it.
#include "common.cuh"

namespace b200moe {

namespace {

template <typename T, int V>
struct alignas(sizeof(T) * V) Pack {
    T v[V];
};

template <typename T>
constexpr int vec_elems() {
    return 16 / (int)sizeof(T);
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// ---- group ---------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void group_kernel(const T* __restrict__ A, int64_t lda, const int64_t* __restrict__ idx,
                             T* __restrict__ out, int64_t ldo, const T* __restrict__ coeff, int fan_out, int64_t M,
                             int K) {
    int64_t n = blockIdx.x;
    if (n >= M) return;
    int64_t s = idx[n];
    const T* src = A + (s / fan_out) * lda;
    T* dst = out + n * ldo;
    float c = coeff ? Elem<T>::to_f(coeff[s]) : 1.f;
    for (int col = threadIdx.x * V; col < K; col += blockDim.x * V) {
        Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(src + col);
        if (coeff) {
#pragma unroll
            for (int i = 0; i < V; ++i) p.v[i] = Elem<T>::from_f(Elem<T>::to_f(p.v[i]) * c);
        }
        *reinterpret_cast<Pack<T, V>*>(dst + col) = p;
    }
}

// ---- row passes of the padded grouped order: one warp per row ---------------------------------------
// The three kernels below give every row to one warp (eight rows per block, blocks stride over the rows): a lane keeps
// up to four 16-byte loads in flight, and a short row (4 KB at hidden 2048) no longer costs a whole block launch.
constexpr int kRowWarps = 8;
constexpr int kRowUnroll = 4;

static inline unsigned row_grid(int64_t rows) {
    int64_t blocks = (rows + kRowWarps - 1) / kRowWarps;
    const int64_t cap = 148 * 16;
    return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

template <typename T, int V>
__global__ void __launch_bounds__(kRowWarps * 32) gather_rows_kernel(const T* __restrict__ src, int64_t lds, const int32_t* __restrict__ row_map,
                                                                    T* __restrict__ out, int64_t ldo, int64_t rows, int width) {
    const int lane = threadIdx.x & 31;
    const int step = 32 * V;
    for (int64_t p = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5); p < rows; p += (int64_t)gridDim.x * kRowWarps) {
        const int r = row_map[p];
        T* dst = out + p * ldo;
        if (r < 0) {  // filler row: zeros
            Pack<T, V> z;
#pragma unroll
            for (int i = 0; i < V; ++i) z.v[i] = Elem<T>::from_f(0.f);
            for (int col = lane * V; col < width; col += step) *reinterpret_cast<Pack<T, V>*>(dst + col) = z;
            continue;
        }
        const T* s = src + (int64_t)r * lds;
        for (int col = lane * V; col < width; col += step * kRowUnroll) {
            Pack<T, V> v[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u)
                if (col + u * step < width) v[u] = *reinterpret_cast<const Pack<T, V>*>(s + col + u * step);
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u)
                if (col + u * step < width) *reinterpret_cast<Pack<T, V>*>(dst + col + u * step) = v[u];
        }
    }
}

// ---- combine -------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void combine_kernel(const T* __restrict__ in, int64_t ldi, const T* __restrict__ gates,
                               T* __restrict__ out, int64_t ldo, int64_t Tn, int k, int H) {
    int64_t t = blockIdx.x;
    if (t >= Tn) return;
    for (int col = threadIdx.x * V; col < H; col += blockDim.x * V) {
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
        for (int j = 0; j < k; ++j) {
            Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(in + (t * k + j) * ldi + col);
            float g = gates ? Elem<T>::to_f(gates[t * k + j]) : 1.f;
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += g * Elem<T>::to_f(p.v[i]);
        }
        Pack<T, V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.v[i] = Elem<T>::from_f(acc[i]);
        *reinterpret_cast<Pack<T, V>*>(out + t * ldo + col) = o;
    }
}

// out[t, :] = sum_j gates[t, j] * in[pos[t*k + j], :]: the combine pass reading rows of the padded grouped order.
// One warp per token; lane j < k looks up row j and its gate, the k rows are then read side by side.  k <= 32.
template <typename T, int V>
__global__ void __launch_bounds__(kRowWarps * 32) combine_rows_kernel(const T* __restrict__ in_rows, int64_t ldi, const int32_t* __restrict__ pos,
                                                                     const T* __restrict__ gates, T* __restrict__ out, int64_t ldo, int64_t Tn,
                                                                     int k, int H) {
    const int lane = threadIdx.x & 31;
    for (int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5); t < Tn; t += (int64_t)gridDim.x * kRowWarps) {
        int my_row = -1;
        float my_gate = 0.f;
        if (lane < k) {
            my_row = pos[t * k + lane];
            my_gate = gates ? Elem<T>::to_f(gates[t * k + lane]) : 1.f;
        }
        // every lane runs every sweep (the shuffles need the whole warp); a lane past the row's end only skips its accesses
        for (int col0 = 0; col0 < H; col0 += 32 * V) {
            const int col = col0 + lane * V;
            const bool in = col < H;
            float acc[V];
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.f;
#pragma unroll 4
            for (int j = 0; j < k; ++j) {
                const int row = __shfl_sync(0xffffffffu, my_row, j);
                const float g = __shfl_sync(0xffffffffu, my_gate, j);
                if (row < 0 || !in) continue;
                Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(in_rows + (int64_t)row * ldi + col);
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += g * Elem<T>::to_f(p.v[i]);
            }
            if (in) {
                Pack<T, V> o;
#pragma unroll
                for (int i = 0; i < V; ++i) o.v[i] = Elem<T>::from_f(acc[i]);
                *reinterpret_cast<Pack<T, V>*>(out + t * ldo + col) = o;
            }
        }
    }
}

// slot_row[row_slot[p]] = p for the real rows of the padded grouped order
__global__ void invert_row_map_kernel(const int32_t* __restrict__ row_slot, int64_t rows, int32_t* __restrict__ slot_row, int64_t M) {
    int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= rows) return;
    int s = row_slot[p];
    if (s >= 0 && s < M) slot_row[s] = (int32_t)p;
}

// ---- SwiGLU --------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t ldy,
                                  int64_t rows, int h, int act) {
    int64_t r = blockIdx.x;
    if (r >= rows) return;
    for (int col = threadIdx.x * V; col < h; col += blockDim.x * V) {
        Pack<T, V> up = *reinterpret_cast<const Pack<T, V>*>(x + r * ldx + col);
        Pack<T, V> gt = *reinterpret_cast<const Pack<T, V>*>(x + r * ldx + h + col);
        Pack<T, V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float g = Elem<T>::to_f(gt.v[i]);
            o.v[i] = Elem<T>::from_f(Elem<T>::to_f(up.v[i]) * gate_value(act, g, sigmoid_for<T>(g)));
        }
        *reinterpret_cast<Pack<T, V>*>(y + r * ldy + col) = o;
    }
}

template <typename T, int V>
__global__ void swiglu_bwd_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ dy, int64_t lddy,
                                  T* __restrict__ dx, int64_t lddx, int64_t rows, int h) {
    int64_t r = blockIdx.x;
    if (r >= rows) return;
    for (int col = threadIdx.x * V; col < h; col += blockDim.x * V) {
        Pack<T, V> up = *reinterpret_cast<const Pack<T, V>*>(x + r * ldx + col);
        Pack<T, V> gt = *reinterpret_cast<const Pack<T, V>*>(x + r * ldx + h + col);
        Pack<T, V> d = *reinterpret_cast<const Pack<T, V>*>(dy + r * lddy + col);
        Pack<T, V> du, dg;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float g = Elem<T>::to_f(gt.v[i]), u = Elem<T>::to_f(up.v[i]), dv = Elem<T>::to_f(d.v[i]);
            float sg = sigmoid_for<T>(g);
            du.v[i] = Elem<T>::from_f(dv * g * sg);
            dg.v[i] = Elem<T>::from_f(dv * u * (sg + g * sg * (1.f - sg)));
        }
        *reinterpret_cast<Pack<T, V>*>(dx + r * lddx + col) = du;
        *reinterpret_cast<Pack<T, V>*>(dx + r * lddx + h + col) = dg;
    }
}

// ---- tail of the down-projection input gradient (CUDA-core engine) --------------------------------
// On entry dh[p, :I] holds d[p, :] = (gate-scaled upstream gradient row) @ w_proj[e], rounded to T; h is in the plain
// (up | gate) layout the CUDA-core forward writes.  One block per padded grouped row; filler rows hold zeros already
// (their upstream rows are zero).
template <typename T>
__global__ void dgrad_down_post_kernel(const T* __restrict__ h, T* __restrict__ dh, int64_t rows, int I, int act_kind) {
    int64_t p = blockIdx.x;
    if (p >= rows) return;
    T* dh_row = dh + p * 2 * (int64_t)I;
    const T* h_row = h + p * 2 * (int64_t)I;
    for (int c = threadIdx.x; c < I; c += blockDim.x) {
        float up = Elem<T>::to_f(h_row[c]), gt = Elem<T>::to_f(h_row[I + c]);
        float d = Elem<T>::to_f(dh_row[c]);
        float sg = sigmoid_for<T>(gt);
        dh_row[c] = Elem<T>::from_f(d * gate_value(act_kind, gt, sg));
        dh_row[I + c] = Elem<T>::from_f(d * up * gate_slope(act_kind, gt, sg));
    }
}

// ---- upstream gradient rows of the backward pass ------------------------------------------------------
// One block per padded grouped row p (slot s = row_slot[p], token t = row_token[p]):
//   out[p, :]  = gates[s] * grad[t, :]            (zeros on filler rows)
//   d_gates[s] = <y_expanded[s or p, :], grad[t, :]>   (fp32; only when y_expanded is given; y_grouped: indexed by p)
// i.e. `group(grad_out, coeff=gates)` and the gate-gradient bmm of the reference's backward in one pass over grad.
template <typename T, int V>
__global__ void __launch_bounds__(kRowWarps * 32) gather_grad_rows_kernel(const T* __restrict__ grad, int64_t ldg, const int32_t* __restrict__ row_token,
                                                                         const int32_t* __restrict__ row_slot, const T* __restrict__ gates,
                                                                         const T* __restrict__ y_expanded, int64_t ldy, int y_grouped,
                                                                         T* __restrict__ out, int64_t ldo, float* __restrict__ d_gates, int64_t rows,
                                                                         int width) {
    const int lane = threadIdx.x & 31;
    const int step = 32 * V;
    for (int64_t p = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5); p < rows; p += (int64_t)gridDim.x * kRowWarps) {
        const int t = row_token[p];
        T* dst = out + p * ldo;
        if (t < 0) {
            Pack<T, V> z;
#pragma unroll
            for (int i = 0; i < V; ++i) z.v[i] = Elem<T>::from_f(0.f);
            for (int col = lane * V; col < width; col += step) *reinterpret_cast<Pack<T, V>*>(dst + col) = z;
            continue;
        }
        const int s = row_slot[p];
        const float g = gates ? Elem<T>::to_f(gates[s]) : 1.f;
        const T* src = grad + (int64_t)t * ldg;
        const T* yrow = y_expanded ? y_expanded + (y_grouped ? p : (int64_t)s) * ldy : nullptr;
        float dot = 0.f;
        for (int col = lane * V; col < width; col += step * 2) {
            Pack<T, V> v[2], y[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (col + u * step < width) {
                    v[u] = *reinterpret_cast<const Pack<T, V>*>(src + col + u * step);
                    if (yrow) y[u] = *reinterpret_cast<const Pack<T, V>*>(yrow + col + u * step);
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (col + u * step < width) {
                    if (yrow) {
#pragma unroll
                        for (int i = 0; i < V; ++i) dot += Elem<T>::to_f(y[u].v[i]) * Elem<T>::to_f(v[u].v[i]);
                    }
                    if (gates) {
#pragma unroll
                        for (int i = 0; i < V; ++i) v[u].v[i] = Elem<T>::from_f(g * Elem<T>::to_f(v[u].v[i]));
                    }
                    *reinterpret_cast<Pack<T, V>*>(dst + col + u * step) = v[u];
                }
            }
        }
        if (yrow) {
            // butterfly sum: the same order every run, so the gate gradient is reproducible
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) d_gates[s] = dot;
        }
    }
}

// ---- un-gated activation (CUDA-core engine of a non-GLU expert) -------------------------------------
template <typename T>
__device__ __forceinline__ float tanh_for(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}
template <>
__device__ __forceinline__ float tanh_for<float>(float x) {
    return tanhf(x);
}

template <typename T>
__global__ void unary_fwd_kernel(const T* __restrict__ h, int64_t ldh, T* __restrict__ a, int64_t lda, int64_t rows, int width) {
    const int64_t total = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / width;
        const int c = (int)(i - r * width);
        const float x = Elem<T>::to_f(h[r * ldh + c]);
        a[r * lda + c] = Elem<T>::from_f(gelu_tanh_value(x, tanh_for<T>(gelu_tanh_arg(x))));
    }
}

template <typename T>
__global__ void unary_bwd_kernel(const T* __restrict__ h, int64_t ldh, T* __restrict__ dh, int64_t ldd, int64_t rows, int width) {
    const int64_t total = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / width;
        const int c = (int)(i - r * width);
        const float x = Elem<T>::to_f(h[r * ldh + c]);
        const float d = Elem<T>::to_f(dh[r * ldd + c]);
        dh[r * ldd + c] = Elem<T>::from_f(d * gelu_tanh_slope(x, tanh_for<T>(gelu_tanh_arg(x))));
    }
}

template <typename F>
int dispatch_dtype(int dtype, F&& f) {
    switch (dtype) {
        case B200MOE_F32:
            return f(float{});
        case B200MOE_BF16:
            return f(__nv_bfloat16{});
        case B200MOE_F16:
            return f(__half{});
        default:
            set_error_detail("unknown dtype code %d", dtype);
            return B200MOE_ERR_DTYPE;
    }
}

static inline int row_threads(int width, int vec) {
    int t = (width / vec + 31) / 32 * 32;
    return t < 32 ? 32 : (t > 256 ? 256 : t);
}

}  // namespace

int launch_swiglu_forward(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int h, int dtype,
                          cudaStream_t stream, int act) {
    if (rows == 0 || h == 0) return B200MOE_OK;
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = h % V == 0 && ldx % V == 0 && ldy % V == 0 && aligned16(x) && aligned16(y);
        if (vec) {
            swiglu_fwd_kernel<T, V><<<(unsigned)rows, row_threads(h, V), 0, stream>>>((const T*)x, ldx, (T*)y, ldy, rows, h, act);
        } else {
            swiglu_fwd_kernel<T, 1><<<(unsigned)rows, row_threads(h, 1), 0, stream>>>((const T*)x, ldx, (T*)y, ldy, rows, h, act);
        }
        count_launch();
        return check_launch("swiglu_forward");
    });
}

int launch_swiglu_backward(const void* x, int64_t ldx, const void* dy, int64_t lddy, void* dx, int64_t lddx,
                           int64_t rows, int h, int dtype, cudaStream_t stream) {
    if (rows == 0 || h == 0) return B200MOE_OK;
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = h % V == 0 && ldx % V == 0 && lddy % V == 0 && lddx % V == 0 && aligned16(x) && aligned16(dy) &&
                   aligned16(dx);
        if (vec) {
            swiglu_bwd_kernel<T, V><<<(unsigned)rows, row_threads(h, V), 0, stream>>>((const T*)x, ldx, (const T*)dy, lddy,
                                                                                     (T*)dx, lddx, rows, h);
        } else {
            swiglu_bwd_kernel<T, 1><<<(unsigned)rows, row_threads(h, 1), 0, stream>>>((const T*)x, ldx, (const T*)dy, lddy,
                                                                                     (T*)dx, lddx, rows, h);
        }
        count_launch();
        return check_launch("swiglu_backward");
    });
}

int launch_dgrad_down_post(const void* h, void* dh, int64_t rows, int I, int dtype, cudaStream_t stream, int act) {
    if (rows == 0) return B200MOE_OK;
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        dgrad_down_post_kernel<T><<<(unsigned)rows, 256, 0, stream>>>((const T*)h, (T*)dh, rows, I, act);
        count_launch();
        return check_launch("dgrad_down_post");
    });
}

int launch_unary_forward(const void* h, int64_t ldh, void* a, int64_t lda, int64_t rows, int width, int dtype, cudaStream_t stream) {
    if (rows == 0 || width == 0) return B200MOE_OK;
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        int64_t blocks = (rows * width + 255) / 256;
        unary_fwd_kernel<T><<<(unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, stream>>>((const T*)h, ldh, (T*)a, lda, rows, width);
        count_launch();
        return check_launch("unary_forward");
    });
}

int launch_unary_backward(const void* h, int64_t ldh, void* dh, int64_t ldd, int64_t rows, int width, int dtype, cudaStream_t stream) {
    if (rows == 0 || width == 0) return B200MOE_OK;
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        int64_t blocks = (rows * width + 255) / 256;
        unary_bwd_kernel<T><<<(unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, stream>>>((const T*)h, ldh, (T*)dh, ldd, rows, width);
        count_launch();
        return check_launch("unary_backward");
    });
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_group(const void* A, int64_t lda, const int64_t* idx, void* out, int64_t ldo,
                             const void* coeff, int fan_out, int64_t M, int K, int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(M >= 0 && K >= 0 && fan_out > 0, B200MOE_ERR_ARG, "group: bad sizes");
    if (M == 0 || K == 0) return B200MOE_OK;
    B200MOE_REQUIRE(A && idx && out, B200MOE_ERR_ARG, "group: NULL pointer");
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = K % V == 0 && lda % V == 0 && ldo % V == 0 && aligned16(A) && aligned16(out);
        if (vec) {
            group_kernel<T, V><<<(unsigned)M, row_threads(K, V), 0, stream>>>((const T*)A, lda, idx, (T*)out, ldo,
                                                                             (const T*)coeff, fan_out, M, K);
        } else {
            group_kernel<T, 1><<<(unsigned)M, row_threads(K, 1), 0, stream>>>((const T*)A, lda, idx, (T*)out, ldo,
                                                                             (const T*)coeff, fan_out, M, K);
        }
        count_launch();
        return check_launch("group");
    });
}

extern "C" int b200moe_gather_rows(const void* src, int64_t lds, const int32_t* row_map, void* out, int64_t ldo,
                                   int64_t rows, int width, int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(rows >= 0 && width >= 0, B200MOE_ERR_ARG, "gather_rows: bad sizes");
    if (rows == 0 || width == 0) return B200MOE_OK;
    B200MOE_REQUIRE(src && row_map && out, B200MOE_ERR_ARG, "gather_rows: NULL pointer");
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = width % V == 0 && lds % V == 0 && ldo % V == 0 && aligned16(src) && aligned16(out);
        if (vec) {
            gather_rows_kernel<T, V><<<row_grid(rows), kRowWarps * 32, 0, stream>>>((const T*)src, lds, row_map, (T*)out, ldo, rows, width);
        } else {
            gather_rows_kernel<T, 1><<<row_grid(rows), kRowWarps * 32, 0, stream>>>((const T*)src, lds, row_map, (T*)out, ldo, rows, width);
        }
        count_launch();
        return check_launch("gather_rows");
    });
}

extern "C" int b200moe_gather_grad_rows(const void* grad, int64_t ldg, const int32_t* row_token, const int32_t* row_slot,
                                        const void* gates, const void* y_expanded, int64_t ldy, int y_grouped, void* out,
                                        int64_t ldo, float* d_gates, int64_t rows, int width, int dtype,
                                        b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(rows >= 0 && width >= 0, B200MOE_ERR_ARG, "gather_grad_rows: bad sizes");
    if (rows == 0 || width == 0) return B200MOE_OK;
    B200MOE_REQUIRE(grad && row_token && row_slot && out, B200MOE_ERR_ARG, "gather_grad_rows: NULL pointer");
    B200MOE_REQUIRE((y_expanded == nullptr) == (d_gates == nullptr), B200MOE_ERR_ARG,
                    "gather_grad_rows: y_expanded and d_gates are given together or not at all");
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = width % V == 0 && ldg % V == 0 && ldo % V == 0 && aligned16(grad) && aligned16(out) &&
                   (y_expanded == nullptr || (ldy % V == 0 && aligned16(y_expanded)));
        if (vec) {
            gather_grad_rows_kernel<T, V><<<row_grid(rows), kRowWarps * 32, 0, stream>>>(
                (const T*)grad, ldg, row_token, row_slot, (const T*)gates, (const T*)y_expanded, ldy, y_grouped, (T*)out, ldo, d_gates, rows, width);
        } else {
            gather_grad_rows_kernel<T, 1><<<row_grid(rows), kRowWarps * 32, 0, stream>>>(
                (const T*)grad, ldg, row_token, row_slot, (const T*)gates, (const T*)y_expanded, ldy, y_grouped, (T*)out, ldo, d_gates, rows, width);
        }
        count_launch();
        return check_launch("gather_grad_rows");
    });
}

extern "C" int b200moe_combine(const void* in, int64_t ldi, const void* gates, void* out, int64_t ldo, int64_t T_,
                               int k, int H, int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(T_ >= 0 && k > 0 && H >= 0, B200MOE_ERR_ARG, "combine: bad sizes");
    if (T_ == 0 || H == 0) return B200MOE_OK;
    B200MOE_REQUIRE(in && out, B200MOE_ERR_ARG, "combine: NULL pointer");
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = H % V == 0 && ldi % V == 0 && ldo % V == 0 && aligned16(in) && aligned16(out);
        if (vec) {
            combine_kernel<T, V><<<(unsigned)T_, row_threads(H, V), 0, stream>>>((const T*)in, ldi, (const T*)gates,
                                                                                (T*)out, ldo, T_, k, H);
        } else {
            combine_kernel<T, 1><<<(unsigned)T_, row_threads(H, 1), 0, stream>>>((const T*)in, ldi, (const T*)gates,
                                                                                (T*)out, ldo, T_, k, H);
        }
        count_launch();
        return check_launch("combine");
    });
}

extern "C" int b200moe_combine_rows(const void* in, int64_t ldi, const int32_t* pos, const void* gates, void* out, int64_t ldo,
                                    int64_t T_, int k, int H, int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(T_ >= 0 && k > 0 && k <= 32 && H >= 0, B200MOE_ERR_ARG, "combine_rows: bad sizes (k <= 32)");
    if (T_ == 0 || H == 0) return B200MOE_OK;
    B200MOE_REQUIRE(in && pos && out, B200MOE_ERR_ARG, "combine_rows: NULL pointer");
    return dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = vec_elems<T>();
        bool vec = H % V == 0 && ldi % V == 0 && ldo % V == 0 && aligned16(in) && aligned16(out);
        if (vec) {
            combine_rows_kernel<T, V><<<row_grid(T_), kRowWarps * 32, 0, stream>>>((const T*)in, ldi, pos, (const T*)gates, (T*)out, ldo, T_, k, H);
        } else {
            combine_rows_kernel<T, 1><<<row_grid(T_), kRowWarps * 32, 0, stream>>>((const T*)in, ldi, pos, (const T*)gates, (T*)out, ldo, T_, k, H);
        }
        count_launch();
        return check_launch("combine_rows");
    });
}

extern "C" int b200moe_invert_row_map(const int32_t* row_slot, int64_t rows, int32_t* slot_row, int64_t M, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(rows >= 0 && M >= 0, B200MOE_ERR_ARG, "invert_row_map: bad sizes");
    if (rows == 0 || M == 0) return B200MOE_OK;
    B200MOE_REQUIRE(row_slot && slot_row, B200MOE_ERR_ARG, "invert_row_map: NULL pointer");
    invert_row_map_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, stream>>>(row_slot, rows, slot_row, M);
    count_launch();
    return check_launch("invert_row_map");
}

extern "C" int b200moe_swiglu_unchunked_forward(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int h,
                                                int dtype, b200moe_stream_t stream) {
    B200MOE_REQUIRE(rows >= 0 && h >= 0, B200MOE_ERR_ARG, "swiglu_forward: bad sizes");
    B200MOE_REQUIRE(rows == 0 || h == 0 || (x && y), B200MOE_ERR_ARG, "swiglu_forward: NULL pointer");
    return launch_swiglu_forward(x, ldx, y, ldy, rows, h, dtype, (cudaStream_t)stream);
}

extern "C" int b200moe_swiglu_unchunked_backward(const void* x, int64_t ldx, const void* dy, int64_t lddy, void* dx,
                                                 int64_t lddx, int64_t rows, int h, int dtype,
                                                 b200moe_stream_t stream) {
    B200MOE_REQUIRE(rows >= 0 && h >= 0, B200MOE_ERR_ARG, "swiglu_backward: bad sizes");
    B200MOE_REQUIRE(rows == 0 || h == 0 || (x && dy && dx), B200MOE_ERR_ARG, "swiglu_backward: NULL pointer");
    return launch_swiglu_backward(x, ldx, dy, lddy, dx, lddx, rows, h, dtype, (cudaStream_t)stream);
}
