// Routing kernels: histogram of expert ids, stable counting sort by expert, inclusive offsets and the
// row maps of the padded grouped order.  Integer work, bit-exact against torch.sort(stable=True),
// bincount and cumsum.  HBM-bound (8 bytes read per id, 16-24 bytes written per routed row).
#include <mutex>

#include "common.cuh"

namespace b200moe {

namespace {

constexpr int kSortThreads = 512;
constexpr int kSortItems = 8;
constexpr int kSortChunk = kSortThreads * kSortItems;  // ids per block

// ---- histogram -----------------------------------------------------------------------------------
template <typename IdT>
__global__ void histogram_kernel(const IdT* __restrict__ x, int64_t n, int32_t* __restrict__ out, int size,
                                 int use_smem) {
    extern __shared__ int32_t hist[];
    if (use_smem) {
        for (int i = threadIdx.x; i < size; i += blockDim.x) hist[i] = 0;
        __syncthreads();
    }
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t v = (int64_t)x[i];
        if (v >= 0 && v < size) {
            if (use_smem) {
                atomicAdd(&hist[v], 1);
            } else {
                atomicAdd(&out[v], 1);
            }
        }
    }
    if (use_smem) {
        __syncthreads();
        for (int i = threadIdx.x; i < size; i += blockDim.x) {
            int32_t c = hist[i];
            if (c) atomicAdd(&out[i], c);
        }
    }
}

// ---- sort, pass 1: per-block histogram -----------------------------------------------------------
__global__ void __launch_bounds__(kSortThreads) route_block_hist(const int64_t* __restrict__ ids, int64_t M,
                                                                 int E, int32_t* __restrict__ block_counts,
                                                                 int32_t* status) {
    __shared__ int32_t hist[kMaxExperts];
    for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    int64_t base = (int64_t)blockIdx.x * kSortChunk;
#pragma unroll
    for (int it = 0; it < kSortItems; ++it) {
        int64_t i = base + it * kSortThreads + threadIdx.x;
        if (i < M) {
            int64_t e = ids[i];
            if (e >= 0 && e < E) {
                atomicAdd(&hist[e], 1);
            } else if (e >= E && status) {
                atomicExch(status, 101);  // expert id out of range (a negative id is a slot without an expert: left out)
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += blockDim.x) block_counts[(int64_t)blockIdx.x * E + i] = hist[i];
}

// ---- sort, pass 2: scan over blocks per expert, then over experts --------------------------------
// In place: block_counts[b][e] becomes the number of ids of expert e in blocks before b.
__global__ void __launch_bounds__(kMaxExperts) route_scan(int32_t* __restrict__ block_counts, int nblocks, int E,
                                                           int32_t* __restrict__ counts,
                                                           int64_t* __restrict__ expert_offsets,
                                                           int32_t* __restrict__ excl_start,
                                                           int32_t* __restrict__ pad_start) {
    __shared__ int32_t total[kMaxExperts];
    int e = threadIdx.x;
    if (e < E) {
        int32_t run = 0;
        for (int b = 0; b < nblocks; ++b) {
            int32_t c = block_counts[(int64_t)b * E + e];
            block_counts[(int64_t)b * E + e] = run;
            run += c;
        }
        total[e] = run;
        if (counts) counts[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t incl = 0;
        int32_t excl = 0, pad = 0;
        for (int i = 0; i < E; ++i) {
            int32_t c = total[i];
            excl_start[i] = excl;
            pad_start[i] = pad;
            excl += c;
            incl += c;
            pad += (c + kPadRows - 1) / kPadRows * kPadRows;
            if (expert_offsets) expert_offsets[i] = incl;
        }
    }
}

// ---- sort, pass 3: stable placement --------------------------------------------------------------
__global__ void __launch_bounds__(kSortThreads) route_place(
    const int64_t* __restrict__ ids, int64_t M, int E, int k, const int32_t* __restrict__ block_base,
    const int32_t* __restrict__ excl_start, const int32_t* __restrict__ pad_start,
    int64_t* __restrict__ sorted_expert_idxs, int64_t* __restrict__ sorted_scattered_idxs,
    int32_t* __restrict__ row_token, int32_t* __restrict__ row_slot) {
    extern __shared__ int32_t smem[];
    constexpr int kWarps = kSortThreads / 32;
    int32_t* warp_cnt = smem;              // [kWarps][E]
    int32_t* running = smem + kWarps * E;  // [E] next free position of expert e for this block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    for (int i = threadIdx.x; i < E; i += blockDim.x)
        running[i] = excl_start[i] + block_base[(int64_t)blockIdx.x * E + i];
    int64_t base = (int64_t)blockIdx.x * kSortChunk;

    for (int it = 0; it < kSortItems; ++it) {
        for (int i = threadIdx.x; i < kWarps * E; i += blockDim.x) warp_cnt[i] = 0;
        __syncthreads();
        int64_t idx = base + it * kSortThreads + threadIdx.x;
        int64_t e64 = idx < M ? ids[idx] : -1;
        bool valid = e64 >= 0 && e64 < E;
        int e = valid ? (int)e64 : 0;
        // lanes without a valid id use a key no other lane has, so they only match themselves
        unsigned mask = __match_any_sync(0xffffffffu, valid ? e : (E + lane));
        int rank = __popc(mask & ((1u << lane) - 1));
        if (valid && rank == 0) warp_cnt[warp * E + e] = __popc(mask);
        __syncthreads();
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            int32_t acc = running[i];
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                int32_t c = warp_cnt[w * E + i];
                warp_cnt[w * E + i] = acc;
                acc += c;
            }
            running[i] = acc;
        }
        __syncthreads();
        if (valid) {
            int32_t pos = warp_cnt[warp * E + e] + rank;
            if (sorted_expert_idxs) sorted_expert_idxs[pos] = e;
            if (sorted_scattered_idxs) sorted_scattered_idxs[pos] = idx;
            if (row_slot) {
                int32_t pp = pad_start[e] + (pos - excl_start[e]);
                row_slot[pp] = (int32_t)idx;
                row_token[pp] = (int32_t)(idx / k);
            }
        }
        __syncthreads();
    }
}

// expert_offsets from an expert-sorted id list: offsets[e] = #{m : sorted[m] <= e}
__global__ void offsets_from_sorted_kernel(const int64_t* __restrict__ sorted, int64_t M, int E,
                                           int64_t* __restrict__ offsets) {
    int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    int64_t lo = 0, hi = M;  // first position with sorted[pos] > e
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (sorted[mid] <= e) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    offsets[e] = lo;
}

__global__ void make_row_maps_kernel(const int64_t* __restrict__ idx, int64_t M, int fan_out,
                                     int32_t* __restrict__ src_map, int32_t* __restrict__ dst_map) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M) return;
    int64_t s = idx[i];
    if (src_map) src_map[i] = (int32_t)(s / fan_out);
    if (dst_map) dst_map[i] = (int32_t)s;
}

}  // namespace

int launch_offsets_from_sorted(const int64_t* sorted, int64_t M, int E, int64_t* offsets, cudaStream_t stream) {
    offsets_from_sorted_kernel<<<(E + 127) / 128, 128, 0, stream>>>(sorted, M, E, offsets);
    count_launch();
    return check_launch("offsets_from_sorted");
}

int launch_make_row_maps(const int64_t* idx, int64_t M, int fan_out, int32_t* src_map, int32_t* dst_map,
                         cudaStream_t stream) {
    if (M == 0) return B200MOE_OK;
    make_row_maps_kernel<<<(unsigned)((M + 255) / 256), 256, 0, stream>>>(idx, M, fan_out, src_map, dst_map);
    count_launch();
    return check_launch("make_row_maps");
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_contiguous_count(const void* x, int x_is_int64, int64_t n, int32_t* out, int size,
                                        b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(out != nullptr && size > 0 && n >= 0, B200MOE_ERR_ARG, "contiguous_count: bad out/size/n");
    B200MOE_REQUIRE(n == 0 || x != nullptr, B200MOE_ERR_ARG, "contiguous_count: x is NULL");
    if (cudaMemsetAsync(out, 0, (size_t)size * sizeof(int32_t), stream) != cudaSuccess)
        return check_launch("contiguous_count memset");
    if (n == 0) return B200MOE_OK;
    int use_smem = size <= 8192;
    int threads = 256;
    int64_t want = (n + threads * 8 - 1) / (threads * 8);
    int blocks = (int)(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
    size_t smem = use_smem ? (size_t)size * sizeof(int32_t) : 0;
    if (x_is_int64) {
        histogram_kernel<int64_t><<<blocks, threads, smem, stream>>>((const int64_t*)x, n, out, size, use_smem);
    } else {
        histogram_kernel<int32_t><<<blocks, threads, smem, stream>>>((const int32_t*)x, n, out, size, use_smem);
    }
    count_launch();
    return check_launch("contiguous_count");
}

extern "C" int64_t b200moe_padded_rows_cap(int64_t M, int E) {
    // sum_e ceil(c_e / 128) <= floor(M / 128) + E
    return (M / kPadRows + E) * kPadRows;
}

extern "C" int64_t b200moe_route_workspace_bytes(int64_t M, int E) {
    int64_t nblocks = (M + kSortChunk - 1) / kSortChunk;
    if (nblocks < 1) nblocks = 1;
    return (nblocks * E + 2 * (int64_t)E) * (int64_t)sizeof(int32_t);
}

extern "C" int b200moe_route(const int64_t* expert_ids, int64_t M, int E, int k, int64_t* sorted_expert_idxs,
                             int64_t* sorted_scattered_idxs, int64_t* expert_offsets, int32_t* counts,
                             int32_t* row_token, int32_t* row_slot, int64_t m_cap, void* workspace,
                             int64_t workspace_bytes, int32_t* status, b200moe_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, "route: E=%d outside [1, %d]", E, kMaxExperts);
    B200MOE_REQUIRE(M >= 0 && M < (int64_t)1 << 31 && k > 0, B200MOE_ERR_ARG, "route: bad M or k");
    B200MOE_REQUIRE(M == 0 || expert_ids != nullptr, B200MOE_ERR_ARG, "route: expert_ids is NULL");
    B200MOE_REQUIRE((row_token == nullptr) == (row_slot == nullptr), B200MOE_ERR_ARG,
                    "route: row_token and row_slot go together");
    B200MOE_REQUIRE(workspace != nullptr && workspace_bytes >= b200moe_route_workspace_bytes(M, E),
                    B200MOE_ERR_WORKSPACE, "route: workspace too small");
    if (row_slot) {
        B200MOE_REQUIRE(m_cap >= b200moe_padded_rows_cap(M, E), B200MOE_ERR_ARG, "route: m_cap too small");
        if (cudaMemsetAsync(row_token, 0xFF, (size_t)m_cap * sizeof(int32_t), stream) != cudaSuccess ||
            cudaMemsetAsync(row_slot, 0xFF, (size_t)m_cap * sizeof(int32_t), stream) != cudaSuccess)
            return check_launch("route memset");
    }
    int nblocks = (int)((M + kSortChunk - 1) / kSortChunk);
    if (nblocks < 1) nblocks = 1;
    int32_t* block_counts = (int32_t*)workspace;
    int32_t* excl_start = block_counts + (int64_t)nblocks * E;
    int32_t* pad_start = excl_start + E;

    route_block_hist<<<nblocks, kSortThreads, 0, stream>>>(expert_ids, M, E, block_counts, status);
    route_scan<<<1, kMaxExperts, 0, stream>>>(block_counts, nblocks, E, counts, expert_offsets, excl_start, pad_start);
    count_launch(2);
    if (M > 0 && (sorted_expert_idxs || sorted_scattered_idxs || row_slot)) {
        size_t smem = (size_t)(kSortThreads / 32 + 1) * E * sizeof(int32_t);
        if (smem > 48 * 1024)  // per device, cheap enough to repeat
            cudaFuncSetAttribute(route_place, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        route_place<<<nblocks, kSortThreads, smem, stream>>>(expert_ids, M, E, k, block_counts, excl_start, pad_start,
                                                            sorted_expert_idxs, sorted_scattered_idxs, row_token,
                                                            row_slot);
        count_launch();
    }
    return check_launch("route");
}

// ---- routing for callers that cannot allocate ------------------------------------------------------
// Scratch of b200moe_route_static: lives in the library image, so every GPU that loads the library holds
// these bytes until the process exits.  In host code the array's name is only a stand-in; the device
// address comes from cudaGetSymbolAddress, looked up once per device below.
constexpr int64_t kStaticRouteScratchBytes = 256 * 1024;
static __device__ __align__(256) unsigned char g_route_static_scratch[kStaticRouteScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_route_static_mutex;
void* g_route_static_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int64_t b200moe_route_static_scratch_bytes(void) { return kStaticRouteScratchBytes; }

extern "C" int b200moe_route_static(const int64_t* expert_ids, int64_t M, int E, int k, int64_t* sorted_expert_idxs,
                                    int64_t* sorted_scattered_idxs, int64_t* expert_offsets, int32_t* counts,
                                    int32_t* row_token, int32_t* row_slot, int64_t m_cap, int32_t* status,
                                    b200moe_stream_t stream) {
    B200MOE_REQUIRE(E > 0 && E <= kMaxExperts, B200MOE_ERR_UNSUPPORTED, "route_static: E=%d outside [1, %d]", E, kMaxExperts);
    B200MOE_REQUIRE(M >= 0, B200MOE_ERR_ARG, "route_static: negative M");
    int64_t need = b200moe_route_workspace_bytes(M, E);
    B200MOE_REQUIRE(need <= kStaticRouteScratchBytes, B200MOE_ERR_UNSUPPORTED,
                    "route_static: M=%lld rows with E=%d experts need %lld bytes of scratch but the built-in array holds %lld; "
                    "use b200moe_route with a caller-owned workspace for this size",
                    (long long)M, E, (long long)need, (long long)kStaticRouteScratchBytes);
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        set_error_detail("route_static: cannot identify the current device");
        return B200MOE_ERR_LAUNCH;
    }
    void* scratch = nullptr;
    {
        // set-up, once per device, with that device current (first call on the device)
        std::lock_guard<std::mutex> lock(g_route_static_mutex);
        if (g_route_static_ptr[dev] == nullptr) {
            void* p = nullptr;
            cudaError_t err = cudaGetSymbolAddress(&p, g_route_static_scratch);
            if (err != cudaSuccess || p == nullptr) {
                cudaGetLastError();
                set_error_detail("route_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
                return B200MOE_ERR_LAUNCH;
            }
            g_route_static_ptr[dev] = p;
        }
        scratch = g_route_static_ptr[dev];
    }
    // Every scratch word the kernels read is written earlier in the same call (per-block histograms, then
    // the scans), so nothing needs clearing between calls.
    return b200moe_route(expert_ids, M, E, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, counts, row_token,
                         row_slot, m_cap, scratch, kStaticRouteScratchBytes, status, stream);
}
