// Expert-parallel row exchange over peer memory (NVLink / NVSwitch): the token dispatch writes rows straight into
// the destination rank's receive buffer, the return path reads rows straight from the expert rank's output buffer
// and folds the gate-weighted sum over the k slots into the same pass.  Plain peer loads and stores of 16 bytes;
// no multimem, no TMA on peer memory.  Ordering between ranks (buffer free / data complete) is the caller's job
// (a barrier over the symmetric-memory signal pads before and after each kernel).
//
// Row placement.  Rank r sorts its routed rows by global expert, so the rows for destination rank d are the
// contiguous range [start[d], start[d+1]) of its sorted order, already ordered by d's local expert.  In d's buffer
// the rows of source rank r follow those of ranks 0..r-1: row n of the sorted order lands at base[d] + n - start[d].
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kMaxRanks = 64;

struct PeerTable {
    void* ptr[kMaxRanks];
};

template <typename T, int V>
struct alignas(sizeof(T) * V) Pack {
    T v[V];
};

__device__ __forceinline__ int find_dest(const int32_t* __restrict__ start, int R, int n) {
    int d = 0;
    while (d + 1 < R && n >= start[d + 1]) ++d;
    return d;
}

// Both exchange kernels give a row (push) or a token (pull) to one warp, six per block, blocks striding over the rows:
// a lane keeps several 16-byte accesses in flight, which is what a transfer over NVLink needs to approach the link rate.
// They are held to 40 registers per thread in blocks of 192 threads and use no shared memory, so that a block fits on an
// SM BESIDE a CTA of the persistent GEMM kernels (448 threads x 128 registers leave 8192 registers free; 192 x 40 = 7680):
// with the layer's tokens split into
// slices, the transfers of one slice then run while the expert GEMMs of another occupy every SM.
constexpr int kEpWarps = 6;
constexpr int kEpUnroll = 2;

template <typename T, int V>
__global__ void __launch_bounds__(kEpWarps * 32, 8) ep_push_kernel(const T* __restrict__ src, int64_t lds, const int64_t* __restrict__ idx, int fan_out,
                                                               const T* __restrict__ coeff, PeerTable peers, const int32_t* __restrict__ start,
                                                               const int32_t* __restrict__ base, const int32_t* __restrict__ dest_pos, int R,
                                                               int64_t M, int width, int64_t cap_rows, int32_t* status) {
    const int lane = threadIdx.x & 31;
    const int step = 32 * V;
    for (int64_t n = (int64_t)blockIdx.x * kEpWarps + (threadIdx.x >> 5); n < M; n += (int64_t)gridDim.x * kEpWarps) {
        const int d = find_dest(start, R, (int)n);
        // the row of the destination buffer: given explicitly (rows land in the receiver's padded grouped order), or the
        // rows of source rank r follow those of ranks 0..r-1 in the order they are sent
        const int64_t pos = dest_pos ? (int64_t)dest_pos[n] : (int64_t)base[d] + (n - start[d]);
        if (pos < 0 || pos >= cap_rows) {  // would overrun the peer's buffer: record and skip
            if (lane == 0 && status) atomicCAS(status, 0, 301);
            continue;
        }
        const int64_t s = idx ? idx[n] : n;
        const T* row = src + (s / fan_out) * lds;
        T* dst = (T*)peers.ptr[d] + pos * (int64_t)width;
        const float c = coeff ? Elem<T>::to_f(coeff[s]) : 1.f;
        for (int col = lane * V; col < width; col += step * kEpUnroll) {
            Pack<T, V> v[kEpUnroll];
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u)
                if (col + u * step < width) v[u] = *reinterpret_cast<const Pack<T, V>*>(row + col + u * step);
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u) {
                if (col + u * step < width) {
                    if (coeff) {
#pragma unroll
                        for (int i = 0; i < V; ++i) v[u].v[i] = Elem<T>::from_f(Elem<T>::to_f(v[u].v[i]) * c);
                    }
                    *reinterpret_cast<Pack<T, V>*>(dst + col + u * step) = v[u];
                }
            }
        }
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kEpWarps * 32, 8) ep_pull_combine_kernel(PeerTable peers, const int64_t* __restrict__ inv, const int32_t* __restrict__ start,
                                                                       const int32_t* __restrict__ base, const int32_t* __restrict__ dest_pos, int R,
                                                                       int64_t cap_rows, const T* __restrict__ gates,
                                                                       T* __restrict__ out, int64_t ldo, T* __restrict__ expanded, int64_t Tn, int k,
                                                                       int width) {
    const int lane = threadIdx.x & 31;
    for (int64_t t = (int64_t)blockIdx.x * kEpWarps + (threadIdx.x >> 5); t < Tn; t += (int64_t)gridDim.x * kEpWarps) {
        // lane j < k resolves where slot j of the token lives: the owning rank's buffer and the row in it
        const T* my_row = nullptr;
        float my_gate = 1.f;
        if (lane < k) {
            const int64_t n = inv[t * k + lane];
            const int d = find_dest(start, R, (int)n);
            const int64_t pos = dest_pos ? (int64_t)dest_pos[n] : (int64_t)base[d] + (n - start[d]);
            // a row that did not fit into the owner's buffer was never stored (the dispatch recorded status 301): it reads as zeros
            if (pos >= 0 && (cap_rows <= 0 || pos < cap_rows)) my_row = (const T*)peers.ptr[d] + pos * (int64_t)width;
            if (gates) my_gate = Elem<T>::to_f(gates[t * k + lane]);
        }
        // every lane runs every sweep (the shuffles need the whole warp); a lane past the row's end only skips its accesses
        for (int col0 = 0; col0 < width; col0 += 32 * V) {
            const int col = col0 + lane * V;
            const bool in = col < width;
            float acc[V];
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.f;
#pragma unroll 4
            for (int j = 0; j < k; ++j) {
                const T* row = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)my_row, j);
                const float g = __shfl_sync(0xffffffffu, my_gate, j);
                if (!in) continue;
                Pack<T, V> p;
                if (row != nullptr) {
                    p = *reinterpret_cast<const Pack<T, V>*>(row + col);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) p.v[i] = Elem<T>::from_f(0.f);
                }
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += g * Elem<T>::to_f(p.v[i]);
                if (expanded) *reinterpret_cast<Pack<T, V>*>(expanded + (t * k + j) * (int64_t)width + col) = p;
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

// d_gates[t, j] = <expanded[t*k + j, :], grad[t, :]> in fp32: the gate gradient of the return path, one block per token
// (the gradient row is read once for the k products).  Replaces the batched (k x H)(H x 1) products of
// cute_kernels/kernels/scattermoe/triton_implementation/ops.py:204, which run far below the HBM rate as a library bmm.
template <typename T, int V>
__global__ void gate_grad_kernel(const T* __restrict__ expanded, int64_t lde, const T* __restrict__ grad, int64_t ldg,
                                 T* __restrict__ d_gates, int64_t Tn, int k, int width) {
    int64_t t = blockIdx.x;
    if (t >= Tn) return;
    __shared__ float red[8];
    for (int j = 0; j < k; ++j) {
        const T* row = expanded + (t * k + j) * lde;
        float acc = 0.f;
        for (int col = threadIdx.x * V; col < width; col += blockDim.x * V) {
            Pack<T, V> a = *reinterpret_cast<const Pack<T, V>*>(row + col);
            Pack<T, V> g = *reinterpret_cast<const Pack<T, V>*>(grad + t * ldg + col);
#pragma unroll
            for (int i = 0; i < V; ++i) acc += Elem<T>::to_f(a.v[i]) * Elem<T>::to_f(g.v[i]);
        }
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        __syncthreads();  // red may still be read for the previous slot
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
            d_gates[t * k + j] = Elem<T>::from_f(s);
        }
    }
}

// Rank barrier over a symmetric int32 flag array (R words per rank, zero at start).  Thread d publishes `epoch` in word
// `rank` of rank d's array and then waits until word d of its own array has reached `epoch`.  Epochs only grow, so a
// peer that is already one barrier ahead is seen as arrived.  The wait is bounded: when a peer does not show up within
// the limit the kernel writes 302 to the status word and returns, so the host can read the failure and the context
// stays usable.
__global__ void ep_barrier_kernel(PeerTable flags, int rank, int R, int epoch, long long limit_cycles, int32_t* status) {
    const int d = threadIdx.x;
    if (d >= R) return;
    __threadfence_system();
    int* remote = (int*)flags.ptr[d] + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = (const int*)flags.ptr[rank] + d;
    const long long t0 = clock64();
    for (;;) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (v - epoch >= 0) break;
        if (clock64() - t0 > limit_cycles) {
            if (status) atomicCAS(status, 0, 302);
            break;
        }
        __nanosleep(200);
    }
}

// Rows of a padded grouped buffer that belong to no routed row: expert e owns rows [seg(e), seg(e) + count(e)) with
// seg(e) = 128 * sum_{e' < e} ceil(count(e') / 128); the rows from seg(e) + count(e) up to the next multiple of 128 are
// cleared (the weight-gradient GEMMs reduce over whole 64-row steps and must read zeros there).  One block per expert.
template <typename T, int V>
__global__ void zero_filler_rows_kernel(T* __restrict__ buf, int64_t ld, const int64_t* __restrict__ offsets, int E, int width, int64_t cap_rows) {
    const int e = blockIdx.x;
    if (e >= E) return;
    int64_t seg = 0;
    for (int i = 0; i < e; ++i) {
        const int64_t c = offsets[i] - (i ? offsets[i - 1] : 0);
        seg += (c + kPadRows - 1) / kPadRows * kPadRows;
    }
    const int64_t cnt = offsets[e] - (e ? offsets[e - 1] : 0);
    const int64_t first = seg + cnt, last = seg + (cnt + kPadRows - 1) / kPadRows * kPadRows;
    Pack<T, V> z;
#pragma unroll
    for (int i = 0; i < V; ++i) z.v[i] = Elem<T>::from_f(0.f);
    const int per_row = width / V;
    for (int64_t i = threadIdx.x; i < (last - first) * per_row; i += blockDim.x) {
        const int64_t r = first + i / per_row;
        if (r < cap_rows) *reinterpret_cast<Pack<T, V>*>(buf + r * ld + (i % per_row) * V) = z;
    }
}

int fill_peers(PeerTable& tab, const void* const* peer_ptrs, int R, const char* what) {
    B200MOE_REQUIRE(R >= 1 && R <= kMaxRanks && peer_ptrs, B200MOE_ERR_ARG, "%s: bad rank count or NULL peer table", what);
    for (int i = 0; i < R; ++i) {
        B200MOE_REQUIRE(peer_ptrs[i] != nullptr && ((uintptr_t)peer_ptrs[i] & 15) == 0, B200MOE_ERR_ARG,
                        "%s: peer buffer %d is NULL or not 16-byte aligned", what, i);
        tab.ptr[i] = const_cast<void*>(peer_ptrs[i]);
    }
    return B200MOE_OK;
}

// `max_blocks` > 0 caps the grid: with one block per SM at most, a transfer that runs beside the persistent GEMM kernels of
// another slice never takes the registers a GEMM CTA needs to become resident (blocks stride over the rows, so a block
// that got an SM keeps it until the whole transfer is done).
unsigned ep_grid(int64_t rows, int max_blocks = 0) {
    int64_t blocks = (rows + kEpWarps - 1) / kEpWarps;
    const int64_t cap = max_blocks > 0 ? max_blocks : 148 * 16;
    return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

int row_threads(int width, int vec) {
    int t = (width / vec + 31) / 32 * 32;
    return t < 64 ? 64 : (t > 256 ? 256 : t);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_ep_push_rows(const void* src, int64_t lds, const int64_t* idx, int fan_out, const void* coeff,
                                    const void* const* peer_ptrs, const int32_t* start, const int32_t* base, int R,
                                    int64_t M, int width, int64_t cap_rows, int dtype, int32_t* status,
                                    b200moe_stream_t stream_) {
    return b200moe_ep_push_rows_at(src, lds, idx, fan_out, coeff, peer_ptrs, start, base, nullptr, R, M, width, cap_rows, 0, dtype, status, stream_);
}

extern "C" int b200moe_ep_push_rows_at(const void* src, int64_t lds, const int64_t* idx, int fan_out, const void* coeff,
                                       const void* const* peer_ptrs, const int32_t* start, const int32_t* base,
                                       const int32_t* dest_pos, int R, int64_t M, int width, int64_t cap_rows, int max_blocks,
                                       int dtype, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(M >= 0 && width > 0 && fan_out > 0 && cap_rows >= 0, B200MOE_ERR_ARG, "ep_push_rows: bad sizes");
    if (M == 0) return B200MOE_OK;
    B200MOE_REQUIRE(src && start && (base || dest_pos), B200MOE_ERR_ARG, "ep_push_rows: NULL pointer");
    PeerTable tab{};
    int rc = fill_peers(tab, peer_ptrs, R, "ep_push_rows");
    if (rc) return rc;
    B200MOE_REQUIRE(dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32, B200MOE_ERR_DTYPE, "ep_push_rows: dtype");
    int esz = dtype == B200MOE_F32 ? 4 : 2, V = 16 / esz;
    B200MOE_REQUIRE(width % V == 0 && lds % V == 0 && ((uintptr_t)src & 15) == 0, B200MOE_ERR_LAYOUT,
                    "ep_push_rows: rows must be 16-byte aligned and a multiple of 16 bytes wide");
    if (dtype == B200MOE_F32) {
        ep_push_kernel<float, 4><<<ep_grid(M, max_blocks), kEpWarps * 32, 0, stream>>>((const float*)src, lds, idx, fan_out, (const float*)coeff, tab,
                                                                   start, base, dest_pos, R, M, width, cap_rows, status);
    } else if (dtype == B200MOE_BF16) {
        ep_push_kernel<__nv_bfloat16, 8><<<ep_grid(M, max_blocks), kEpWarps * 32, 0, stream>>>((const __nv_bfloat16*)src, lds, idx, fan_out,
                                                                           (const __nv_bfloat16*)coeff, tab, start, base, dest_pos, R, M,
                                                                           width, cap_rows, status);
    } else {
        ep_push_kernel<__half, 8><<<ep_grid(M, max_blocks), kEpWarps * 32, 0, stream>>>((const __half*)src, lds, idx, fan_out, (const __half*)coeff,
                                                                    tab, start, base, dest_pos, R, M, width, cap_rows, status);
    }
    count_launch();
    return check_launch("ep_push_rows");
}

extern "C" int b200moe_ep_pull_combine(const void* const* peer_ptrs, const int64_t* inv, const int32_t* start,
                                       const int32_t* base, int R, const void* gates, void* out, int64_t ldo,
                                       void* expanded, int64_t T_, int k, int width, int dtype,
                                       b200moe_stream_t stream_) {
    return b200moe_ep_pull_combine_at(peer_ptrs, inv, start, base, nullptr, R, 0, 0, gates, out, ldo, expanded, T_, k, width, dtype, stream_);
}

extern "C" int b200moe_ep_pull_combine_at(const void* const* peer_ptrs, const int64_t* inv, const int32_t* start,
                                          const int32_t* base, const int32_t* dest_pos, int R, int64_t cap_rows, int max_blocks,
                                          const void* gates, void* out, int64_t ldo, void* expanded, int64_t T_, int k, int width,
                                          int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(T_ >= 0 && width > 0 && k > 0 && k <= 32, B200MOE_ERR_ARG, "ep_pull_combine: bad sizes (k <= 32)");
    if (T_ == 0) return B200MOE_OK;
    B200MOE_REQUIRE(inv && start && (base || dest_pos) && out, B200MOE_ERR_ARG, "ep_pull_combine: NULL pointer");
    PeerTable tab{};
    int rc = fill_peers(tab, peer_ptrs, R, "ep_pull_combine");
    if (rc) return rc;
    B200MOE_REQUIRE(dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32, B200MOE_ERR_DTYPE, "ep_pull_combine: dtype");
    int esz = dtype == B200MOE_F32 ? 4 : 2, V = 16 / esz;
    B200MOE_REQUIRE(width % V == 0 && ldo % V == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)expanded & 15) == 0,
                    B200MOE_ERR_LAYOUT, "ep_pull_combine: rows must be 16-byte aligned and a multiple of 16 bytes wide");
    if (dtype == B200MOE_F32) {
        ep_pull_combine_kernel<float, 4><<<ep_grid(T_, max_blocks), kEpWarps * 32, 0, stream>>>(tab, inv, start, base, dest_pos, R, cap_rows, (const float*)gates, (float*)out,
                                                                            ldo, (float*)expanded, T_, k, width);
    } else if (dtype == B200MOE_BF16) {
        ep_pull_combine_kernel<__nv_bfloat16, 8><<<ep_grid(T_, max_blocks), kEpWarps * 32, 0, stream>>>(
            tab, inv, start, base, dest_pos, R, cap_rows, (const __nv_bfloat16*)gates, (__nv_bfloat16*)out, ldo, (__nv_bfloat16*)expanded, T_, k, width);
    } else {
        ep_pull_combine_kernel<__half, 8><<<ep_grid(T_, max_blocks), kEpWarps * 32, 0, stream>>>(tab, inv, start, base, dest_pos, R, cap_rows, (const __half*)gates,
                                                                             (__half*)out, ldo, (__half*)expanded, T_, k, width);
    }
    count_launch();
    return check_launch("ep_pull_combine");
}

extern "C" int b200moe_ep_gate_grad(const void* expanded, int64_t lde, const void* grad, int64_t ldg, void* d_gates, int64_t T_,
                                    int k, int width, int dtype, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(T_ >= 0 && width > 0 && k > 0, B200MOE_ERR_ARG, "ep_gate_grad: bad sizes");
    if (T_ == 0) return B200MOE_OK;
    B200MOE_REQUIRE(expanded && grad && d_gates, B200MOE_ERR_ARG, "ep_gate_grad: NULL pointer");
    B200MOE_REQUIRE(dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32, B200MOE_ERR_DTYPE, "ep_gate_grad: dtype");
    int esz = dtype == B200MOE_F32 ? 4 : 2, V = 16 / esz;
    B200MOE_REQUIRE(width % V == 0 && lde % V == 0 && ldg % V == 0 && ((uintptr_t)expanded & 15) == 0 && ((uintptr_t)grad & 15) == 0,
                    B200MOE_ERR_LAYOUT, "ep_gate_grad: rows must be 16-byte aligned and a multiple of 16 bytes wide");
    int threads = row_threads(width, V);
    if (dtype == B200MOE_F32) {
        gate_grad_kernel<float, 4><<<(unsigned)T_, threads, 0, stream>>>((const float*)expanded, lde, (const float*)grad, ldg, (float*)d_gates, T_, k, width);
    } else if (dtype == B200MOE_BF16) {
        gate_grad_kernel<__nv_bfloat16, 8><<<(unsigned)T_, threads, 0, stream>>>((const __nv_bfloat16*)expanded, lde, (const __nv_bfloat16*)grad, ldg,
                                                                            (__nv_bfloat16*)d_gates, T_, k, width);
    } else {
        gate_grad_kernel<__half, 8><<<(unsigned)T_, threads, 0, stream>>>((const __half*)expanded, lde, (const __half*)grad, ldg, (__half*)d_gates, T_, k, width);
    }
    count_launch();
    return check_launch("ep_gate_grad");
}

extern "C" int b200moe_ep_barrier(const void* const* flag_ptrs, int rank, int R, int epoch, int64_t limit_cycles, int32_t* status,
                                  b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(rank >= 0 && rank < R && limit_cycles > 0, B200MOE_ERR_ARG, "ep_barrier: bad rank or limit");
    PeerTable tab{};
    int rc = fill_peers(tab, flag_ptrs, R, "ep_barrier");
    if (rc) return rc;
    ep_barrier_kernel<<<1, 64, 0, stream>>>(tab, rank, R, epoch, (long long)limit_cycles, status);
    count_launch();
    return check_launch("ep_barrier");
}

extern "C" int b200moe_zero_filler_rows(void* buf, int64_t ld, const int64_t* expert_offsets, int E, int width, int64_t cap_rows, int dtype,
                                        b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts && width > 0 && cap_rows >= 0, B200MOE_ERR_ARG, "zero_filler_rows: bad sizes");
    B200MOE_REQUIRE(buf && expert_offsets, B200MOE_ERR_ARG, "zero_filler_rows: NULL pointer");
    B200MOE_REQUIRE(dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32, B200MOE_ERR_DTYPE, "zero_filler_rows: dtype");
    int esz = dtype == B200MOE_F32 ? 4 : 2, V = 16 / esz;
    B200MOE_REQUIRE(width % V == 0 && ld % V == 0 && ((uintptr_t)buf & 15) == 0, B200MOE_ERR_LAYOUT,
                    "zero_filler_rows: rows must be 16-byte aligned and a multiple of 16 bytes wide");
    if (dtype == B200MOE_F32) {
        zero_filler_rows_kernel<float, 4><<<E, 256, 0, stream>>>((float*)buf, ld, expert_offsets, E, width, cap_rows);
    } else if (dtype == B200MOE_BF16) {
        zero_filler_rows_kernel<__nv_bfloat16, 8><<<E, 256, 0, stream>>>((__nv_bfloat16*)buf, ld, expert_offsets, E, width, cap_rows);
    } else {
        zero_filler_rows_kernel<__half, 8><<<E, 256, 0, stream>>>((__half*)buf, ld, expert_offsets, E, width, cap_rows);
    }
    count_launch();
    return check_launch("zero_filler_rows");
}

// ---- placement plan of the direct exchange ------------------------------------------------------------
// Everything a rank derives from the all-gathered expert counts, in one launch (it replaces about twenty-five small
// tensor operations per pass, which weigh as much as the expert GEMMs when a rank holds only a few thousand tokens).
// counts_all[s * E + e]: rows that rank s routes to expert slot e.  Every block rebuilds the small tables in shared
// memory; the rows are spread over the grid.
constexpr int kPlanMaxCounts = 4096;  // world * E

__global__ void __launch_bounds__(256) ep_plan_kernel(const int32_t* __restrict__ counts_all, const int64_t* __restrict__ ss, int world,
                                                       int rank, int E, int64_t M, int32_t* __restrict__ start, int32_t* __restrict__ base,
                                                       int32_t* __restrict__ dest_pos, int64_t* __restrict__ local_offsets,
                                                       int64_t* __restrict__ summary, int64_t* __restrict__ inv) {
    __shared__ int cnt[kPlanMaxCounts];
    __shared__ int tot[kMaxExperts], before[kMaxExperts], pad_start[kMaxExperts], excl[kMaxExperts];
    __shared__ int padded_sum[64], to_own[64], base_s[64], recv_s[64];
    const int e_local = E / world;
    for (int i = threadIdx.x; i < world * E; i += blockDim.x) cnt[i] = counts_all[i];
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0, b = 0;
        for (int s = 0; s < world; ++s) {
            const int c = cnt[s * E + e];
            t += c;
            if (s < rank) b += c;
        }
        tot[e] = t;
        before[e] = b;
    }
    __syncthreads();
    if (threadIdx.x < world) {  // one thread per owner: the padded segments of its experts, and what this rank sends to it
        const int d = threadIdx.x;
        int run = 0, own = 0, bs = 0, rc = 0;
        for (int j = 0; j < e_local; ++j) {
            const int e = d * e_local + j;
            pad_start[e] = run;
            run += (tot[e] + kPadRows - 1) / kPadRows * kPadRows;
            own += cnt[rank * E + e];
            bs += before[e];
            rc += tot[e];
        }
        padded_sum[d] = run;
        to_own[d] = own;
        base_s[d] = bs;
        recv_s[d] = rc;
    }
    if (threadIdx.x == 32) {  // first sorted row of every expert on this rank
        int run = 0;
        for (int e = 0; e < E; ++e) {
            excl[e] = run;
            run += cnt[rank * E + e];
        }
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int run = 0, mx = 0;
        start[0] = 0;
        for (int d = 0; d < world; ++d) {
            run += to_own[d];
            start[d + 1] = run;
            base[d] = base_s[d];
            mx = padded_sum[d] > mx ? padded_sum[d] : mx;
        }
        int64_t off = 0;
        for (int j = 0; j < e_local; ++j) {
            off += tot[rank * e_local + j];
            local_offsets[j] = off;
        }
        summary[0] = recv_s[rank];  // real rows this rank receives
        summary[1] = mx;            // most padded rows any rank's buffers must hold
    }
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M; i += (int64_t)gridDim.x * blockDim.x) {
        int lo = 0, hi = E - 1;  // last expert whose first row is <= i (the experts after it that start there are empty)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (excl[mid] <= i) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        dest_pos[i] = pad_start[lo] + before[lo] + (int)(i - excl[lo]);
        inv[ss[i]] = i;
    }
}

extern "C" int b200moe_ep_plan(const int32_t* counts_all, const int64_t* sorted_scattered_idxs, int world, int rank, int E, int64_t M,
                               int32_t* start, int32_t* base, int32_t* dest_pos, int64_t* local_offsets, int64_t* summary, int64_t* inverse,
                               b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(world > 0 && world <= 64 && rank >= 0 && rank < world && E > 0 && E <= kMaxExperts && E % world == 0 &&
                        world * E <= kPlanMaxCounts && M >= 0 && M < ((int64_t)1 << 31),
                    B200MOE_ERR_ARG, "ep_plan: bad sizes");
    B200MOE_REQUIRE(counts_all && start && base && local_offsets && summary && (M == 0 || (sorted_scattered_idxs && dest_pos && inverse)),
                    B200MOE_ERR_ARG, "ep_plan: NULL pointer");
    int64_t blocks = (M + 255) / 256;
    blocks = blocks < 1 ? 1 : blocks > 592 ? 592 : blocks;
    ep_plan_kernel<<<(int)blocks, 256, 0, stream>>>(counts_all, sorted_scattered_idxs, world, rank, E, M, start, base, dest_pos, local_offsets,
                                                    summary, inverse);
    count_launch();
    return check_launch("ep_plan");
}
