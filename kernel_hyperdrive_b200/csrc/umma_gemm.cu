// Tensor-core engine (sm_100a) for the two grouped-GEMM families.
//
// One persistent CTA per SM, 128 x 256 output tiles, 64-deep k steps, 4-stage shared-memory ring,
// tcgen05.mma (cta_group::1, kind::f16, M=128, N=256, K=16) accumulating fp32 in tensor memory.  Two
// accumulators of 256 columns each fill the 512 TMEM columns, so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Warp roles (448 threads):
//   warp 0      TMA producer: operands that are plain 2-D tiles of a matrix (cp.async.bulk.tensor, SW128)
//   warp 1      allocates TMEM, then one lane issues every tcgen05.mma / tcgen05.commit
//   warps 2-5   gather producers: operands whose rows are picked by an index list (token gather) are
//               copied with 16-byte cp.async into the same 128-byte-swizzled layout TMA would write
//   warps 6-13  epilogue: tcgen05.ld of the accumulator, fused element-wise work, global stores; two warps
//               share each TMEM lane quarter and split the tile's columns
//
// Shared-memory tile layout (both operands): rows of 128 bytes (64 elements), 8-row groups of 1024 bytes,
// 16-byte chunk index XOR (row & 7).  For a K-major operand a row is one M/N index and holds 64
// consecutive k; for an MN-major operand a row is one k index and holds 64 consecutive M/N indices, and
// a 128- or 256-wide operand is 2 or 4 such [64 k][128 B] blocks one after the other.
//
// Every wait on an mbarrier is bounded: after about two seconds the waiting thread raises a CTA-wide
// abort flag, writes a code to the status word and every role leaves its loop; TMEM is freed on the way
// out.  Nothing here uses cluster multicast.
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "umma_common.cuh"

namespace b200moe {

namespace umma {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

}  // namespace

// Encoded tensor maps are a pure function of (base address, extents, strides, box, element type, swizzle): they are
// kept in a small cache so that a layer that calls with the same buffers and shapes step after step (weights always,
// activations whenever the allocator hands back the same blocks) does not pay the driver's encode call on every launch.
struct MapKey {
    const void* base;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    int rank, dtype, swizzle, promo;
    bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
        uint64_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
        return (size_t)h;
    }
};
static_assert(sizeof(MapKey) % 8 == 0, "MapKey is hashed in 8-byte words");

int encode_cached(CUtensorMap* map, const MapKey& key_in) {
    static std::mutex mtx;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key;
    memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
    key.base = key_in.base;
    for (int i = 0; i < 3; ++i) key.dims[i] = key_in.dims[i], key.box[i] = key_in.box[i];
    for (int i = 0; i < 2; ++i) key.strides[i] = key_in.strides[i];
    key.rank = key_in.rank, key.dtype = key_in.dtype, key.swizzle = key_in.swizzle, key.promo = key_in.promo;
    {
        std::lock_guard<std::mutex> lock(mtx);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return B200MOE_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    B200MOE_REQUIRE(fn != nullptr, B200MOE_ERR_DRIVER, "cuTensorMapEncodeTiled not available from the driver");
    cuuint64_t dims[3] = {key.dims[0], key.dims[1], key.dims[2]};
    cuuint64_t strides[2] = {key.strides[0], key.strides[1]};
    cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult rc = fn(map, key.dtype ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)key.rank, (void*)key.base, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, (CUtensorMapSwizzle)key.swizzle, (CUtensorMapL2promotion)key.promo,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200MOE_REQUIRE(rc == CUDA_SUCCESS, B200MOE_ERR_DRIVER, "cuTensorMapEncodeTiled failed with %d (rank=%d dims=%llu x %llu x %llu ld=%llu)", (int)rc,
                    key.rank, (unsigned long long)key.dims[0], (unsigned long long)key.dims[1], (unsigned long long)key.dims[2],
                    (unsigned long long)key.strides[0]);
    std::lock_guard<std::mutex> lock(mtx);
    if (cache.size() >= 4096) cache.clear();
    cache.emplace(key, *map);
    return B200MOE_OK;
}

// Output box of the epilogue: 32 columns x 32 rows (x 1 expert), 64-byte swizzle.  rank 2: [rows][cols] with row
// stride ld; rank 3: [experts][rows][cols] with expert stride se, so that a tile never spills into the next expert.
int make_store_map(CUtensorMap* map, const void* base, int64_t experts, int64_t rows, int64_t cols, int64_t ld, int64_t se,
                   int is_f16) {
    MapKey k{};
    k.base = base;
    k.rank = experts > 0 ? 3 : 2;
    k.dims[0] = (uint64_t)cols, k.dims[1] = (uint64_t)rows, k.dims[2] = (uint64_t)(experts > 0 ? experts : 1);
    k.strides[0] = (uint64_t)ld * 2, k.strides[1] = (uint64_t)se * 2;
    k.box[0] = 32u, k.box[1] = 32u, k.box[2] = 1u;
    k.dtype = is_f16 ? 1 : 0;
    k.swizzle = (int)CU_TENSOR_MAP_SWIZZLE_64B;
    k.promo = (int)CU_TENSOR_MAP_L2_PROMOTION_NONE;
    return encode_cached(map, k);
}

// 2-D row-major matrix [rows][cols] with row stride ld (elements), box of 64 columns x box_rows rows.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int is_f16) {
    MapKey k{};
    k.base = base;
    k.rank = 2;
    k.dims[0] = (uint64_t)cols, k.dims[1] = (uint64_t)rows, k.dims[2] = 1;
    k.strides[0] = (uint64_t)ld * 2, k.strides[1] = 0;
    k.box[0] = 64u, k.box[1] = (uint32_t)box_rows, k.box[2] = 1u;
    k.dtype = is_f16 ? 1 : 0;
    k.swizzle = (int)CU_TENSOR_MAP_SWIZZLE_128B;
    k.promo = (int)CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    return encode_cached(map, k);
}

// Row-gather map: [rows][cols] with row stride ld, box of 64 columns x 1 row (tile::gather4 fetches four such rows).
int make_gather_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int is_f16) {
    return make_map(map, base, rows, cols, ld, 1, is_f16);
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

// SMs a tensor-core GEMM launch may occupy: all of them unless the SM-limit option reserves some for other streams.
int gemm_sm_count() {
    const int all = sm_count(), limit = option_value(B200MOE_OPT_SM_LIMIT);
    return limit > 0 && limit < all ? limit : all;
}


uint32_t make_idesc(int a_mn, int b_mn, int is_f16, int m, int n) {
    uint32_t fmt = is_f16 ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

}  // namespace umma

using namespace umma;

namespace {

bool aligned16(const void* p) { return p != nullptr && ((uintptr_t)p & 15) == 0; }

// Which tile a launch uses.  The two-CTA kernel (256 x 256 cluster tile) needs every operand as a TMA tile; given that,
// the choice between it and the one-CTA kernel (128 x 256) comes from the per-shape table below unless the engine or the
// tile-variant option forces one.
bool use_pair_kernels(const UmmaParams& p, int epi, int64_t rows_cap) {
    if (!(p.a_tma && p.b_tma) || current_engine() == B200MOE_ENGINE_UMMA_1CTA) return false;
    if (current_engine() == B200MOE_ENGINE_UMMA_GATHER4 && (p.a_g4 || p.b_g4)) return true;
    int forced = option_value(B200MOE_OPT_TILE_VARIANT);
    if (forced == B200MOE_TILE_PAIR_256x256) return true;
    if (forced == B200MOE_TILE_CTA_128x256) return false;
    const int64_t rows_per_expert = p.E > 0 ? rows_cap / p.E : rows_cap;
    const int op = p.wfam ? B200MOE_OP_WGRAD
                          : ((epi_gated_forward(epi) || epi == EPI_UNARY) ? B200MOE_OP_UP_FORWARD
                                                                          : ((epi_gated_dgrad(epi) || epi == EPI_DGRAD_UNARY) ? B200MOE_OP_DOWN_DGRAD : B200MOE_OP_ROW_STORE));
    return tile_table_lookup(op, p.wfam ? p.Mout : p.K, p.N, rows_per_expert) == B200MOE_TILE_PAIR_256x256;
}

template <int EPI>
int launch(const UmmaParams& p, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mo2,
           const CUtensorMap& mo3, cudaStream_t stream);

template <int EPI>
int launch_any(UmmaParams& p, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mo2,
               const CUtensorMap& mo3, int64_t rows_cap, cudaStream_t stream) {
    if (use_pair_kernels(p, EPI, rows_cap)) {
        p.idesc = make_idesc(p.a_mn, p.b_mn, p.is_f16, 2 * BM);
        return launch_2cta(EPI, p, ma, mb, mo, mo2, mo3, rows_cap, stream);
    }
    return launch<EPI>(p, ma, mb, mo, mo2, mo3, stream);
}

#ifndef B200MOE_STAGES
#define B200MOE_STAGES 4
#endif
constexpr int STAGES = B200MOE_STAGES;
static_assert(STAGES == 4 && BK == 64, "the MMA lane writes out four slots and four MMAs per k step");
constexpr int B_STAGE_BYTES = BN * BK * 2;          // 32 KB
constexpr int NUM_THREADS = (6 + EPI_WARPS) * 32;   // 448
constexpr int GATHER_THREADS = 128;

// ---- the kernel ----------------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    umma_grouped_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_o,
                        const __grid_constant__ CUtensorMap tmap_o2, const __grid_constant__ CUtensorMap tmap_o3) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
    uint8_t* smem_stg = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);  // one 2 KB output box per epilogue warp
    uint64_t* bars = (uint64_t*)(smem_stg + EPI_WARPS * STG_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* tmem_full_bar = bars + 2 * STAGES;
    uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    Tables& tb = *(Tables*)(tmem_slot + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // segment tables
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
        if (p.offsets == nullptr) {  // one group of a size known to the host (router)
            tb.seg_cnt[e] = (int)p.rows_fixed;
        } else {
            int64_t prev = e ? p.offsets[e - 1] : 0;
            tb.seg_cnt[e] = (int)(p.offsets[e] - prev);
        }
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), p.full_count);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tmem_full_bar[a]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[a]), EPI_WARPS * 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (p.wfam) fill_expert_order(tb, p.E);
    if (threadIdx.x == 0) {
        int start = 0, tiles = 0;
        for (int e = 0; e < p.E; ++e) {
            int cnt = tb.seg_cnt[e];
            int cover = p.padded ? (cnt + kPadRows - 1) / kPadRows * kPadRows : cnt;
            tb.seg_start[e] = start;
            tb.tile_prefix[e] = tiles;
            start += cover;
            tiles += (cover + BM - 1) / BM;
        }
        tb.tile_prefix[p.E] = tiles;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int ntiles = total_tiles(p, tb);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && (p.a_tma || p.b_tma)) {
            // the router's weight matrix has at most 256 rows: one 128-row box when they fit, else two
            const uint32_t b_bytes = (EPI == EPI_ROUTER && p.N <= 128) ? B_STAGE_BYTES / 2 : B_STAGE_BYTES;
            const uint32_t tx_bytes = (p.a_tma ? A_STAGE_BYTES : 0) + (p.b_tma ? b_bytes : 0);
            int slot = 0;  // ring position; `phase` flips when it wraps
            uint32_t phase = 0;
            Tile ti;
            const uint32_t full0 = smem_u32(&full_bar[0]);
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            const uint32_t sa0 = smem_u32(smem_a), sb0 = smem_u32(smem_b);
            const bool a_tma = p.a_tma, b_tma = p.b_tma;
            const bool b_two = EPI != EPI_ROUTER || p.N > 128;
            // One tile's k loop, unrolled over the ring's slots like the MMA lane's.  MODE 0: K-major operands (one
            // 64 x 128 box of A, two of B); 1: weight-gradient family (token-major operands, 64 x 64 boxes: two of A,
            // four of B); 2: B stored MN-major (one box of A, four of B).  `ca`, `cb`, `cb2`: the tile's fixed coordinates;
            // the other coordinate advances by BK per k step from `ka` / `kb`.
            auto load_tile = [&](auto mode, const int nk, const int ca, const int cb, const int cb2, int ka, int kb) -> bool {
                constexpr int MODE = decltype(mode)::value;
                int ks = 0;
                for (;;) {
                    switch (slot) {
#define B200MOE_LOAD_STEP(S)                                                                                              \
    case S: {                                                                                                             \
        if (ks == nk) {                                                                                                   \
            slot = S;                                                                                                     \
            return true;                                                                                                  \
        }                                                                                                                 \
        if (!mbar_wait(empty0 + S * 8, phase ^ 1, abort_flag, p.status, 201)) return false;                               \
        constexpr uint32_t bar_off = S * 8, off_a = S * A_STAGE_BYTES, off_b = S * B_STAGE_BYTES;                         \
        mbar_arrive_expect_tx(full0 + bar_off, tx_bytes);                                                                 \
        if (MODE == 1) {                                                                                                  \
            if (a_tma) {                                                                                                  \
                tma_load_2d(sa0 + off_a, &tmap_a, full0 + bar_off, ca, ka);                                               \
                tma_load_2d(sa0 + off_a + 8192, &tmap_a, full0 + bar_off, ca + 64, ka);                                   \
            }                                                                                                             \
            if (b_tma) {                                                                                                  \
                tma_load_2d(sb0 + off_b, &tmap_b, full0 + bar_off, cb, kb);                                               \
                tma_load_2d(sb0 + off_b + 8192, &tmap_b, full0 + bar_off, cb + 64, kb);                                   \
                tma_load_2d(sb0 + off_b + 16384, &tmap_b, full0 + bar_off, cb + 128, kb);                                 \
                tma_load_2d(sb0 + off_b + 24576, &tmap_b, full0 + bar_off, cb + 192, kb);                                 \
            }                                                                                                             \
        } else if (MODE == 2) {                                                                                           \
            if (a_tma) tma_load_2d(sa0 + off_a, &tmap_a, full0 + bar_off, ka, ca);                                        \
            if (b_tma) {                                                                                                  \
                tma_load_2d(sb0 + off_b, &tmap_b, full0 + bar_off, cb, kb);                                               \
                tma_load_2d(sb0 + off_b + 8192, &tmap_b, full0 + bar_off, cb + 64, kb);                                   \
                tma_load_2d(sb0 + off_b + 16384, &tmap_b, full0 + bar_off, cb + 128, kb);                                 \
                tma_load_2d(sb0 + off_b + 24576, &tmap_b, full0 + bar_off, cb + 192, kb);                                 \
            }                                                                                                             \
        } else {                                                                                                          \
            if (a_tma) tma_load_2d(sa0 + off_a, &tmap_a, full0 + bar_off, ka, ca);                                        \
            if (b_tma) {                                                                                                  \
                tma_load_2d(sb0 + off_b, &tmap_b, full0 + bar_off, kb, cb);                                               \
                if (b_two) tma_load_2d(sb0 + off_b + 16384, &tmap_b, full0 + bar_off, kb, cb2);                           \
            }                                                                                                             \
        }                                                                                                                 \
        ka += BK;                                                                                                         \
        kb += BK;                                                                                                         \
        ++ks;                                                                                                             \
    }
                        B200MOE_LOAD_STEP(0) B200MOE_LOAD_STEP(1) B200MOE_LOAD_STEP(2) B200MOE_LOAD_STEP(3)
#undef B200MOE_LOAD_STEP
                    }
                    slot = 0;
                    phase ^= 1;
                }
            };
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
                decode_tile(p, tb, t, ti);
                bool ok;
                if (p.wfam) {
                    // both operands MN-major: boxes of 64 columns x 64 token rows
                    ok = load_tile(IntTag<1>{}, ti.ksteps, ti.mb * BM, ti.nb * BN, 0, ti.row0, ti.row0);
                } else if (p.b_mn) {
                    ok = load_tile(IntTag<2>{}, ti.ksteps, ti.row0, ti.nb * BN, 0, 0, ti.e * p.b_rows_per_expert);
                } else {
                    int r0, r1;
                    if (epi_gated_forward(EPI)) {
                        r0 = ti.e * p.b_rows_per_expert + ti.nb * 128;
                        r1 = r0 + p.swiglu_half;
                    } else {
                        r0 = ti.e * p.b_rows_per_expert + ti.nb * BN;
                        r1 = r0 + 128;
                    }
                    ok = load_tile(IntTag<0>{}, ti.ksteps, ti.row0, r0, r1, 0, 0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int slot = 0;  // ring position; `phase` flips when it wraps
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            Tile ti;
            const uint32_t a_step = p.a_mn ? 128u : 2u;  // descriptor address units (16 B) per 16-deep MMA
            const uint32_t b_step = p.b_mn ? 128u : 2u;
            const uint64_t adesc0 = make_desc(smem_u32(smem_a), p.a_mn);
            const uint64_t bdesc0 = make_desc(smem_u32(smem_b), p.b_mn);
            const uint32_t a_lo0 = (uint32_t)adesc0, a_hi = (uint32_t)(adesc0 >> 32);
            const uint32_t b_lo0 = (uint32_t)bdesc0, b_hi = (uint32_t)(bdesc0 >> 32);
            const uint32_t full0 = smem_u32(&full_bar[0]);
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            const uint32_t idesc = p.idesc;
            // One tile's k loop, unrolled over the ring's slots and entered at the ring position: one thread issues
            // everything, each of its instructions waits for the one before, and the tensor pipe queues only a few
            // MMAs, so whatever this lane executes per k step beyond four MMAs, one wait and one commit is idle time of
            // the pipe (the rolled loop needed about 610 clocks per k step against the pipe's 512).
            auto mma_tile = [&](const int nk, const uint32_t d_tmem) -> bool {
                int ks = 0;
                uint32_t accum = 0;
                for (;;) {
                    switch (slot) {
#define B200MOE_MMA_STEP(S)                                                                                               \
    case S: {                                                                                                             \
        if (ks == nk) {                                                                                                   \
            slot = S;                                                                                                     \
            return true;                                                                                                  \
        }                                                                                                                 \
        if (!mbar_wait(full0 + S * 8, phase, abort_flag, p.status, 203)) return false;                                    \
        if (p.full_count > 1) tc_fence_after(); /* operands written by the gather warps' cp.async */                     \
        constexpr uint32_t off_a = S * (A_STAGE_BYTES >> 4), off_b = S * (B_STAGE_BYTES >> 4);                            \
        tc_mma_lh(d_tmem, a_lo0 + off_a, a_hi, b_lo0 + off_b, b_hi, idesc, accum);                                        \
        tc_mma_lh(d_tmem, a_lo0 + off_a + a_step, a_hi, b_lo0 + off_b + b_step, b_hi, idesc, 1u);                         \
        tc_mma_lh(d_tmem, a_lo0 + off_a + 2 * a_step, a_hi, b_lo0 + off_b + 2 * b_step, b_hi, idesc, 1u);                 \
        tc_mma_lh(d_tmem, a_lo0 + off_a + 3 * a_step, a_hi, b_lo0 + off_b + 3 * b_step, b_hi, idesc, 1u);                 \
        tc_commit(empty0 + S * 8); /* frees the slot when these MMAs have read it */                                      \
        accum = 1u;                                                                                                       \
        ++ks;                                                                                                             \
    }
                        B200MOE_MMA_STEP(0) B200MOE_MMA_STEP(1) B200MOE_MMA_STEP(2) B200MOE_MMA_STEP(3)
#undef B200MOE_MMA_STEP
                    }
                    slot = 0;
                    phase ^= 1;
                }
            };
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
                decode_tile(p, tb, t, ti);
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, 202)) break;
                tc_fence_after();
                if (!mma_tile(ti.ksteps, tmem_base + acc * BN)) break;
                tc_commit(smem_u32(&tmem_full_bar[acc]));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
            }
        }
    } else if (warp < 6) {
        // ---------------- gather producers ----------------
        if (!p.a_tma || !p.b_tma) {
            const int g = threadIdx.x - 64;  // 0..127
            const int chunk = g & 7, rbase = g >> 3;  // this thread copies chunk `chunk` of rows rbase + 16 i
            const uint32_t swz = (uint32_t)((chunk ^ (rbase & 7)) << 4);
            const int esz = 2;
            int stage = 0;
            uint32_t phase = 0;
            Tile ti;
            bool ok = true;
            if (!p.wfam) {
                // K-major gather of operand A: the 128 source rows are fixed per tile; the next tile's rows are
                // fetched while the current tile streams so that the index latency stays off the critical path
                int src_r[8], src_n[8];
                auto load_rows = [&](int t, int (&dst)[8]) {
                    Tile tn;
                    if (t < ntiles) {
                        decode_tile(p, tb, t, tn);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            int r = rbase + 16 * i, src = -1;
                            if (r < tn.rows_valid) src = p.a_map ? p.a_map[tn.row0 + r] : tn.row0 + r;
                            dst[i] = src;
                        }
                    }
                };
                load_rows(blockIdx.x, src_n);
                for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                    decode_tile(p, tb, t, ti);
#pragma unroll
                    for (int i = 0; i < 8; ++i) src_r[i] = src_n[i];
                    load_rows(t + gridDim.x, src_n);
                    for (int ks = 0; ks < ti.ksteps; ++ks) {
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 204)) {
                            ok = false;
                            break;
                        }
                        const uint32_t sa = smem_u32(smem_a + stage * A_STAGE_BYTES) + rbase * 128 + swz;
                        const int kcol = ks * BK + chunk * 8;
                        const bool kin = kcol < p.K;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            int src = src_r[i];
                            bool v = kin && src >= 0;
                            const uint8_t* gp = (const uint8_t*)p.a_ptr + (v ? ((int64_t)src * p.a_ld + kcol) * esz : 0);
                            cp_async_16(sa + i * 2048, gp, v ? 16u : 0u);
                        }
                        cp_async_arrive_noinc(smem_u32(&full_bar[stage]));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            } else {
                // MN-major gather: 64 token rows per stage, 4 per thread; the row indices of step ks + 1 are
                // requested before the copies of step ks are issued
                const bool ga = !p.a_tma, gb = !p.b_tma;
                auto load_idx = [&](const Tile& tt, int ks, int (&ia)[4], int (&ib)[4]) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        int r = ks * BK + rbase + 16 * i;
                        int sa_ = -1, sb_ = -1;
                        if (r < tt.rows_valid) {
                            if (ga) sa_ = p.a_map ? p.a_map[tt.row0 + r] : tt.row0 + r;
                            if (gb) sb_ = p.b_map ? p.b_map[tt.row0 + r] : tt.row0 + r;
                        }
                        ia[i] = sa_;
                        ib[i] = sb_;
                    }
                };
                for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
                    decode_tile(p, tb, t, ti);
                    int cur_a[4], cur_b[4], nxt_a[4], nxt_b[4];
                    if (ti.ksteps > 0) load_idx(ti, 0, nxt_a, nxt_b);
                    for (int ks = 0; ks < ti.ksteps; ++ks) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            cur_a[i] = nxt_a[i];
                            cur_b[i] = nxt_b[i];
                        }
                        if (ks + 1 < ti.ksteps) load_idx(ti, ks + 1, nxt_a, nxt_b);
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 204)) {
                            ok = false;
                            break;
                        }
                        if (ga) {
                            const uint32_t sa = smem_u32(smem_a + stage * A_STAGE_BYTES) + rbase * 128 + swz;
#pragma unroll
                            for (int j = 0; j < BM / 64; ++j) {
                                int col = ti.mb * BM + j * 64 + chunk * 8;
                                bool cin = col < p.Mout;
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    bool v = cin && cur_a[i] >= 0;
                                    const uint8_t* gp =
                                        (const uint8_t*)p.a_ptr + (v ? ((int64_t)cur_a[i] * p.a_ld + col) * esz : 0);
                                    cp_async_16(sa + j * 8192 + i * 2048, gp, v ? 16u : 0u);
                                }
                            }
                        }
                        if (gb) {
                            const uint32_t sb = smem_u32(smem_b + stage * B_STAGE_BYTES) + rbase * 128 + swz;
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j) {
                                int col = ti.nb * BN + j * 64 + chunk * 8;
                                bool cin = col < p.N;
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    bool v = cin && cur_b[i] >= 0;
                                    const uint8_t* gp =
                                        (const uint8_t*)p.b_ptr + (v ? ((int64_t)cur_b[i] * p.b_ld + col) * esz : 0);
                                    cp_async_16(sb + j * 8192 + i * 2048, gp, v ? 16u : 0u);
                                }
                            }
                        }
                        cp_async_arrive_noinc(smem_u32(&full_bar[stage]));
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;               // TMEM lane quarter this warp may read
        const int half = (warp - 6) >> 2;     // which half of the tile's columns this warp handles
        // Outputs that are whole rows of a row-major matrix leave through shared memory: the warp writes its
        // 32 x 32 box (64-byte rows, 64-byte swizzle, conflict-free) and one lane hands it to TMA, which
        // stores full sectors.  The box is reused for every output, so the lane first waits until the
        // previous store has finished reading it.
        const uint32_t stg = smem_u32(smem_stg + (warp - 6) * STG_BYTES);
        const uint32_t stg_row = stg + lane * 64;
        const uint32_t stg_swz = (uint32_t)((lane >> 1) & 3);
        auto stage_store = [&](const CUtensorMap* map, int c0, int c1, int c2, const uint32_t (&pk)[16]) {
            if (lane == 0) bulk_wait_read0();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j)
                st_shared_v4(stg_row + ((j ^ stg_swz) << 4), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                if (p.o3d) {
                    tma_store_3d(map, stg, c0, c1, c2);
                } else {
                    tma_store_2d(map, stg, c0, c1);
                }
                bulk_commit();
            }
        };
        int acc = 0;
        uint32_t acc_phase = 0;
        Tile ti;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
            decode_tile(p, tb, t, ti);
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, 205, 200)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            epilogue_tile<EPI>(p, ti, taddr, q, half, lane, &tmap_o, &tmap_o2, &tmap_o3, stage_store);
            tc_fence_before();
            mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (lane == 0) bulk_wait0();  // every TMA store issued by this warp has been written
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        // give copies still in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

constexpr int SMEM_BYTES = 1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + EPI_WARPS * STG_BYTES + 128 + (int)sizeof(Tables) + 64;

template <int EPI>
int launch(const UmmaParams& p, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mo2,
           const CUtensorMap& mo3, cudaStream_t stream) {
    auto kern = umma_grouped_kernel<EPI>;
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (err != cudaSuccess) {
        set_error_detail("cudaFuncSetAttribute(smem=%d): %s", SMEM_BYTES, cudaGetErrorString(err));
        return B200MOE_ERR_LAUNCH;
    }
    kern<<<gemm_sm_count(), NUM_THREADS, SMEM_BYTES, stream>>>(p, ma, mb, mo, mo2, mo3);
    count_launch();
    return check_launch("umma_grouped_kernel");
}

}  // namespace

namespace {
// One CTA waits, with a short limit, on an mbarrier that nothing ever arrives on: the give-up path of the GEMM
// kernels (abort flag, status word, orderly return) exercised without touching anything that could fault.
__global__ void bounded_wait_selftest_kernel(int32_t* status, long long limit_cycles, int* finished) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait_slow(smem_u32(&bar), 0, &abort_flag, status, 299, 100, limit_cycles);
    __syncthreads();
    // every thread sees the abort flag, as the roles of the GEMM kernels do, and the kernel returns normally
    if (threadIdx.x == 0 && finished) *finished = (!ok && abort_flag) ? 1 : 2;
}
}  // namespace

bool umma_row_gemm_supported(const RowGemm& g, int dtype) {
    if (dtype != B200MOE_BF16 && dtype != B200MOE_F16) return false;
    if (g.E > kMaxExperts || g.K % 8 || g.N % 8 || g.lda % 8 || g.ldo % 8) return false;
    if (!aligned16(g.A) || !aligned16(g.W) || !aligned16(g.out)) return false;
    if (g.rows_cap >= ((int64_t)1 << 31) || (int64_t)g.E * (g.w_sk == 1 ? g.N : g.K) >= ((int64_t)1 << 31)) return false;
    if (g.w_sk == 1) {  // K-major weights: (E*N, K) matrix
        if (g.w_sn % 8 || g.w_sn < g.K || g.w_se != (int64_t)g.N * g.w_sn) return false;
    } else if (g.w_sn == 1) {  // MN-major: (E*K, N) matrix
        if (g.w_sk % 8 || g.w_sk < g.N || g.w_se != (int64_t)g.K * g.w_sk) return false;
    } else {
        return false;
    }
    if (g.epi == EPI_SWIGLU && (g.w_sk != 1 || (g.N / 2) % 8 || !aligned16(g.out2))) return false;
    if (g.epi == EPI_DGRAD_DOWN && !aligned16(g.h)) return false;
    if (g.epi == EPI_UNARY && !aligned16(g.out2)) return false;
    if (g.epi == EPI_DGRAD_UNARY && !aligned16(g.h)) return false;
    return true;
}

bool umma_w_gemm_supported(const WGemm& g, int dtype) {
    if (dtype != B200MOE_BF16 && dtype != B200MOE_F16) return false;
    if (g.E > kMaxExperts || g.Mout % 8 || g.Nout % 8 || g.ldp % 8 || g.ldq % 8) return false;
    if (g.d_sn != 1 || g.d_sm % 8 || g.d_se % 8) return false;
    if (!aligned16(g.P) || !aligned16(g.Q) || !aligned16(g.DW)) return false;
    return true;
}

int umma_row_gemm(const RowGemm& g, int dtype, int32_t* status, cudaStream_t stream) {
    if (g.rows_cap == 0 || g.N == 0) return B200MOE_OK;
    UmmaParams p{};
    p.wfam = 0;
    p.E = g.E;
    p.padded = g.padded;
    p.offsets = g.offsets;
    p.K = g.K;
    p.is_f16 = dtype == B200MOE_F16;
    p.a_mn = 0;
    // Rows picked by a row map: cp.async gather warps of the one-CTA kernel.  TMA row gather (tile::gather4) inside
    // the two-CTA kernel is built too but sustains only about a third of the rate (one gather instruction moves 512
    // bytes and the TMA unit issues them far slower than box loads), so it runs only when asked for.
    const bool gather4 = g.a_map != nullptr && current_engine() == B200MOE_ENGINE_UMMA_GATHER4 && g.a_rows > 0 &&
                         g.a_rows < ((int64_t)1 << 31);
    p.a_g4 = gather4;
    p.a_oob = (int)g.a_rows;
    p.a_tma = g.a_map == nullptr || gather4;
    p.a_ptr = g.A;
    p.a_ld = g.lda;
    p.a_map = g.a_map;
    p.b_tma = 1;
    p.b_mn = g.w_sn == 1 && g.w_sk != 1;
    p.b_ptr = g.W;
    p.out = g.out;
    p.ldo = g.ldo;
    p.o_map = g.o_map;
    p.scale = g.scale;
    p.out2 = g.out2;
    p.h = g.h;
    p.status = status;
    p.idesc = make_idesc(0, p.b_mn, p.is_f16, BM);
    p.full_count = 1 + (p.a_tma ? 0 : GATHER_THREADS);
    // Tile order inside an expert.  The tiles in flight at one time are consecutive in the list; what they share comes from
    // L2, what they do not share is streamed from HBM once per visit.  When one expert's weight matrix is small enough to stay
    // in L2 beside the activations in flight (K * N * 2 bytes up to 32 MB), the column blocks of a row tile are walked first, so
    // that every activation row is read from HBM once; with larger weight matrices (the Mixtral-shaped layer: 117 / 235 MB per
    // expert) the row tiles of a column block are walked first, so that the tiles in flight share the weight panel.
    // Option value 2 walks the experts of the pair kernel in blocks of 8 x 8 tiles instead (measured on the Mixtral-shaped
    // layer: 43.6 against 45.6 GB of DRAM traffic per step, no difference in time; not the default).
    {
        const int forced = option_value(B200MOE_OPT_TILE_ORDER);
        p.nb_inner = forced == 2 ? 0 : forced >= 0 ? forced : ((int64_t)g.K * g.N * 2 <= ((int64_t)32 << 20) ? 1 : 0);
        p.blocked_rows = forced == 2 ? 1 : 0;
    }

    CUtensorMap ma{}, mb{};
    int rc;
    if (p.a_g4) {
        rc = make_gather_map(&ma, g.A, g.a_rows, g.K, g.lda, p.is_f16);
        if (rc) return rc;
    } else if (p.a_tma) {
        rc = make_map(&ma, g.A, g.rows_cap, g.K, g.lda, 128, p.is_f16);
        if (rc) return rc;
    }
    if (p.b_mn) {
        p.b_rows_per_expert = g.K;
        rc = make_map(&mb, g.W, (int64_t)g.E * g.K, g.N, g.w_sk, 64, p.is_f16);
    } else {
        p.b_rows_per_expert = g.N;
        rc = make_map(&mb, g.W, (int64_t)g.E * g.N, g.K, g.w_sn, 128, p.is_f16);
    }
    if (rc) return rc;
    if (!p.a_tma) ma = mb;  // unused, but the parameter must hold a valid descriptor

    CUtensorMap mo = mb, mo2 = mb, mo3 = mb;  // placeholders when an output does not go through TMA
    p.o3d = 0;
    if (g.epi == EPI_SWIGLU) {
        B200MOE_REQUIRE(g.padded && g.o_map == nullptr, B200MOE_ERR_ARG, "SwiGLU epilogue needs the padded grouped order");
        p.swiglu_half = g.N / 2;
        p.N = g.N;
        p.nb_count = (p.swiglu_half + 127) / 128;
        // h is stored interleaved per 32-column chunk (up part, then gate part).  The up boxes get their own map whose
        // column extent ends where the gate part of a ragged last chunk begins, so that the box is clipped there; the
        // gate boxes are clipped by the row end.
        const int I_ = g.N / 2, ragged = I_ % 32;
        rc = make_store_map(&mo, g.out, 0, g.rows_cap, g.N - ragged, g.ldo, 0, p.is_f16);
        if (rc) return rc;
        rc = make_store_map(&mo3, g.out, 0, g.rows_cap, g.N, g.ldo, 0, p.is_f16);
        if (rc) return rc;
        rc = make_store_map(&mo2, g.out2, 0, g.rows_cap, g.N / 2, g.N / 2, 0, p.is_f16);
        if (rc) return rc;
        return g.act == ACT_SIGMOID ? launch_any<EPI_GLU>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream)
                                    : launch_any<EPI_SWIGLU>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream);
    }
    p.N = g.N;
    p.nb_count = (g.N + BN - 1) / BN;
    if (g.epi == EPI_UNARY || g.epi == EPI_DGRAD_UNARY) {
        B200MOE_REQUIRE(g.padded && g.o_map == nullptr, B200MOE_ERR_ARG, "activation epilogue needs the padded grouped order");
        rc = make_store_map(&mo, g.out, 0, g.rows_cap, g.N, g.ldo, 0, p.is_f16);
        if (rc) return rc;
        if (g.epi == EPI_UNARY) {
            rc = make_store_map(&mo2, g.out2, 0, g.rows_cap, g.N, g.N, 0, p.is_f16);
            if (rc) return rc;
            return launch_any<EPI_UNARY>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream);
        }
        return launch_any<EPI_DGRAD_UNARY>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream);
    }
    if (g.epi == EPI_DGRAD_DOWN) {
        B200MOE_REQUIRE(g.padded && g.o_map == nullptr, B200MOE_ERR_ARG, "dgrad epilogue needs the padded grouped order");
        rc = make_store_map(&mo, g.out, 0, g.rows_cap, g.N, 2 * (int64_t)g.N, 0, p.is_f16);
        if (rc) return rc;
        rc = make_store_map(&mo3, (const uint8_t*)g.out + (int64_t)g.N * 2, 0, g.rows_cap, g.N, 2 * (int64_t)g.N, 0, p.is_f16);
        if (rc) return rc;
        // one epilogue for both gate functions: the forward epilogue stored the derivative factors, not h
        return launch_any<EPI_DGRAD_DOWN>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream);
    }
    if (g.o_map == nullptr && g.scale == nullptr) {
        rc = make_store_map(&mo, g.out, 0, g.rows_cap, g.N, g.ldo, 0, p.is_f16);
        if (rc) return rc;
    }
    return launch_any<EPI_STORE>(p, ma, mb, mo, mo2, mo3, g.rows_cap, stream);
}

// Fused router: logits = x @ gate_wT on the tensor cores (one group of T rows, the experts are the tile's columns),
// top-k, scores and the per-expert counts in the epilogue.
int umma_router(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, int64_t T, int H, int E, int k, int scoring,
                const float* row_scale, void* logits, int64_t ldl, void* weights, int64_t* indices, int32_t* counts, int dtype,
                int32_t* status, cudaStream_t stream) {
    UmmaParams p{};
    p.wfam = 0;
    p.E = 1;
    p.padded = 0;
    p.offsets = nullptr;
    p.rows_fixed = T;
    p.K = H;
    p.N = E;
    p.nb_count = 1;
    p.is_f16 = dtype == B200MOE_F16;
    p.a_tma = p.b_tma = 1;
    p.a_ptr = x;
    p.a_ld = ldx;
    p.b_ptr = gate_w;
    p.b_rows_per_expert = E;
    p.out = logits;
    p.ldo = ldl;
    p.out2 = weights;
    p.r_indices = indices;
    p.r_counts = counts;
    p.r_rowscale = row_scale;
    p.r_k = k;
    p.r_scoring = scoring;
    p.r_vec = E % 8 == 0 && ldl % 8 == 0 && aligned16(logits);
    p.status = status;
    const int n_mma = E <= 16 ? 16 : (E + 15) / 16 * 16;
    p.idesc = make_idesc(0, 0, p.is_f16, BM, n_mma);
    p.full_count = 1;
    CUtensorMap ma{}, mb{};
    int rc = make_map(&ma, x, T, H, ldx, 128, p.is_f16);
    if (rc) return rc;
    rc = make_map(&mb, gate_w, E, H, ldw, 128, p.is_f16);  // rows past E read as zeros
    if (rc) return rc;
    return launch<EPI_ROUTER>(p, ma, mb, mb, mb, mb, stream);
}

int umma_w_gemm(const WGemm& g, int dtype, int32_t* status, cudaStream_t stream) {
    if (g.Mout == 0 || g.Nout == 0 || g.E == 0) return B200MOE_OK;
    UmmaParams p{};
    p.wfam = 1;
    p.E = g.E;
    p.padded = g.padded;
    p.offsets = g.offsets;
    p.is_f16 = dtype == B200MOE_F16;
    p.Mout = g.Mout;
    p.N = g.Nout;
    p.mb_count = (g.Mout + BM - 1) / BM;
    p.nb_count = (g.Nout + BN - 1) / BN;
    p.a_mn = 1;
    p.b_mn = 1;
    // An operand can come through TMA only when its rows are the layout rows themselves and filler rows are
    // known to be zero, i.e. in the padded order; everything else is gathered with zero fill.
    const bool pair_ok = current_engine() == B200MOE_ENGINE_UMMA_GATHER4 && g.map_rows > 0 && g.map_rows < ((int64_t)1 << 31);
    p.a_g4 = g.p_map != nullptr && pair_ok;
    p.b_g4 = g.q_map != nullptr && pair_ok;
    p.a_oob = p.b_oob = (int)g.map_rows;
    p.a_tma = (g.padded && g.p_map == nullptr && g.rows_cap > 0) || p.a_g4;
    p.b_tma = (g.padded && g.q_map == nullptr && g.rows_cap > 0) || p.b_g4;
    if (!(p.a_tma && p.b_tma)) {  // the one-CTA kernel gathers with cp.async: no row-gather maps there
        if (p.a_g4) p.a_tma = 0;
        if (p.b_g4) p.b_tma = 0;
        p.a_g4 = p.b_g4 = 0;
    }
    p.a_ptr = g.P;
    p.a_ld = g.ldp;
    p.a_map = g.p_map;
    p.b_ptr = g.Q;
    p.b_ld = g.ldq;
    p.b_map = g.q_map;
    p.out = g.DW;
    p.ldo = g.d_sm;
    p.d_se = g.d_se;
    p.status = status;
    p.idesc = make_idesc(1, 1, p.is_f16, BM);
    p.full_count = ((p.a_tma || p.b_tma) ? 1 : 0) + ((!p.a_tma || !p.b_tma) ? GATHER_THREADS : 0);

    CUtensorMap ma{}, mb{};
    int rc;
    bool have = false;
    if (p.a_tma) {
        rc = p.a_g4 ? make_gather_map(&ma, g.P, g.map_rows, g.Mout, g.ldp, p.is_f16) : make_map(&ma, g.P, g.rows_cap, g.Mout, g.ldp, 64, p.is_f16);
        if (rc) return rc;
        have = true;
    }
    if (p.b_tma) {
        rc = p.b_g4 ? make_gather_map(&mb, g.Q, g.map_rows, g.Nout, g.ldq, p.is_f16) : make_map(&mb, g.Q, g.rows_cap, g.Nout, g.ldq, 64, p.is_f16);
        if (rc) return rc;
        if (!have) ma = mb;
    } else if (have) {
        mb = ma;
    }
    CUtensorMap mo{};
    p.o3d = 1;
    rc = make_store_map(&mo, g.DW, g.E, g.Mout, g.Nout, g.d_sm, g.d_se, p.is_f16);
    if (rc) return rc;
    return launch_any<EPI_STORE>(p, ma, mb, mo, mo, mo, g.rows_cap, stream);
}

}  // namespace b200moe

extern "C" int b200moe_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, int32_t* finished, b200moe_stream_t stream_) {
    using namespace b200moe;
    B200MOE_REQUIRE(status != nullptr && limit_cycles > 0 && limit_cycles <= 4000000000LL, B200MOE_ERR_ARG,
                    "selftest_bounded_wait: status must be given and the limit must be at most 4e9 cycles");
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream_>>>(status, (long long)limit_cycles, finished);
    count_launch();
    return check_launch("bounded_wait_selftest");
}
