// Device and host pieces shared by the tensor-core (tcgen05) kernels: PTX wrappers, shared-memory and
// instruction descriptors, the tile bookkeeping derived from the expert offsets, and the epilogue of one tile.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200moe {
namespace umma {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int EPI_WARPS = 8;  // two warps per TMEM lane quarter, each takes half the columns
constexpr int STG_BYTES = 32 * 32 * 2;  // epilogue staging: 32 rows x 32 columns of 16-bit elements, 64-byte swizzle
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;
constexpr int ROUTER_KMAX = 8;  // most experts per token the fused router selects

struct UmmaParams {
    int wfam;    // 0: family R (row tiles), 1: family W (per-expert weight gradient)
    int E, padded;
    const int64_t* offsets;
    int K;          // R: reduction extent
    int N;          // columns of the output (R: N, W: Nout)
    int Mout;       // W: rows of the output
    int nb_count;   // column blocks
    int nb_inner;   // R: 1 = walk the column blocks of a row tile first (the expert's weight matrix fits L2), 0 = the row tiles of a column block first
    int blocked_rows;  // R, pair kernel, nb_inner == 0: experts with more rows than this walk their tiles in 8 x 8 blocks (0 = never)
    int mb_count;   // W: row blocks
    int swiglu_half;  // EPI_SWIGLU: I (columns of one half); tiles cover 128 columns of each half
    // operand A (R: activations; W: P)
    int a_tma, a_mn;
    int a_g4, a_oob;  // two-CTA kernel: rows of A come through TMA row gather by a_map; a_oob = index that reads as zeros
    const void* a_ptr;
    int64_t a_ld;
    const int32_t* a_map;
    // operand B (R: weights; W: Q)
    int b_tma, b_mn;
    int b_g4, b_oob;
    const void* b_ptr;
    int64_t b_ld;
    const int32_t* b_map;
    int b_rows_per_expert;  // R: rows of the 2-D weight matrix one expert owns
    // epilogue
    void* out;
    int64_t ldo;
    const int32_t* o_map;
    const void* scale;
    void* out2;
    const void* h;
    int64_t d_se;
    int32_t* status;
    unsigned int* tile_counter;  // two-CTA kernel: zeroed word the clusters draw tile indices from; NULL: static round-robin
    uint32_t idesc;
    int is_f16;
    int full_count;  // arrivals per full barrier
    int o3d;         // output tensor map is 3-D (expert, row, column): weight gradients
    // router (EPI_ROUTER, one-CTA kernel): one group of `rows_fixed` rows (offsets == nullptr), N = number of experts
    int64_t rows_fixed;
    int r_k, r_scoring, r_vec;  // experts per token; 0 softmax / 1 normalised sigmoid; logits rows allow 16-byte stores
    const float* r_rowscale;    // optional fp32 factor per row applied to the logits before rounding (RMSNorm's 1 / rms)
    int64_t* r_indices;         // (rows, k) selected experts
    int32_t* r_counts;          // (N) rows per expert, accumulated with atomics
};

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait.  Returns false when the CTA is aborting (this thread or another one gave up).
// `sleep_ns` > 0 puts the thread to sleep between polls: used where the wait is long and a wake-up delay of
// that order does not matter (epilogue warps waiting for a whole tile, producers that run stages ahead), so
// that idle warps do not spend issue slots and power on polling.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                                   int code, unsigned sleep_ns, long long limit_cycles = WAIT_LIMIT_CYCLES) {
    long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if (sleep_ns) __nanosleep(sleep_ns);
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int code, unsigned sleep_ns = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code, sleep_ns);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Arrives on the barrier once every cp.async this thread issued before has landed; the arrival is one
// of the barrier's expected arrivals (noinc), so the issuing thread never waits for its own copies.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((uint64_t)map), "r"(src),
                 "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"((uint64_t)map),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 1 / (1 + exp(-x)) with the fast exponential and division; exp overflow gives 1 / inf = 0, never NaN
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 with the hardware tanh: one special-function instruction instead of two
// (exponential and reciprocal).  Relative error about 2^-11, below the rounding of the 16-bit tensors it feeds.  Used in
// the forward epilogue; the down-dgrad epilogue measured slower with it and keeps sigmoid_fast.
__device__ __forceinline__ float sigmoid_tanh(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

__device__ __forceinline__ float tanh_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// The same instruction with the descriptors given as (low, high) words: along the k loop only the 14-bit start-address
// field in the low word changes (shared memory is below 256 KB, so the field never carries), which keeps the address
// arithmetic of the issuing lane at one 32-bit add per operand and MMA.
__device__ __forceinline__ void tc_mma_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
// K-major: 8-row groups 1024 B apart (SBO); LBO unused.  MN-major: 8-k groups 1024 B apart (SBO), 64-wide
// blocks along M/N 8192 B apart (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, int mn_major) {
    uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | ((mn_major ? (8192u >> 4) : 1u) << 16);
    uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

// ---- element helpers (bf16 / fp16 chosen at run time, uniform per launch) --------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b, int is_f16) {
    if (is_f16) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t u, int is_f16) {
    if (is_f16) return __half22float2(*reinterpret_cast<__half2*>(&u));
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ float load_scalar(const void* p, int64_t i, int is_f16) {
    if (is_f16) return __half2float(((const __half*)p)[i]);
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ float round_elem(float v, int is_f16) {
    if (is_f16) return __half2float(__float2half_rn(v));
    return __bfloat162float(__float2bfloat16_rn(v));
}

// Compile-time integer handed to a generic lambda (selects a code path without a run-time branch in its loop).
template <int V>
struct IntTag {
    static constexpr int value = V;
};

// ---- tile bookkeeping ----------------------------------------------------------------------------
struct Tables {
    int seg_start[kMaxExperts];    // first layout row of the expert's segment
    int seg_cnt[kMaxExperts];      // rows the expert really has
    int tile_prefix[kMaxExperts + 1];  // R: row tiles before the expert
    uint16_t order[kMaxExperts];   // W: experts by descending row count (the longest reductions are handed out first)
};

// Fills tb.order: position of expert e = number of experts with more rows (ties: lower index first).  Called by all
// threads of the CTA after seg_cnt is complete and before a barrier.
__device__ __forceinline__ void fill_expert_order(Tables& tb, int E) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = tb.seg_cnt[e];
        int pos = 0;
        for (int o = 0; o < E; ++o) {
            const int co = tb.seg_cnt[o];
            pos += (co > c || (co == c && o < e)) ? 1 : 0;
        }
        tb.order[pos] = (uint16_t)e;
    }
}

struct Tile {
    int e, row0, rows_valid, nb, mb, ksteps;
};

__device__ __forceinline__ int total_tiles(const UmmaParams& p, const Tables& tb) {
    return p.wfam ? p.E * p.mb_count * p.nb_count : tb.tile_prefix[p.E] * p.nb_count;
}

__device__ __forceinline__ void decode_tile(const UmmaParams& p, const Tables& tb, int t, Tile& ti) {
    if (p.wfam) {
        int per_e = p.mb_count * p.nb_count;
        const int ei = t / per_e;
        ti.e = tb.order[ei];
        int local = t - ei * per_e;
        if (p.mb_count <= p.nb_count) {  // walk the shorter side fastest: its operand panel stays L2-resident
            ti.mb = local % p.mb_count;
            ti.nb = local / p.mb_count;
        } else {
            ti.nb = local % p.nb_count;
            ti.mb = local / p.nb_count;
        }
        ti.row0 = tb.seg_start[ti.e];
        ti.rows_valid = tb.seg_cnt[ti.e];
        ti.ksteps = (ti.rows_valid + BK - 1) / BK;
    } else {
        int lo = 0, hi = p.E - 1;  // last e with tile_prefix[e] * nb <= t
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (tb.tile_prefix[mid] * p.nb_count <= t) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        ti.e = lo;
        int mt_e = tb.tile_prefix[lo + 1] - tb.tile_prefix[lo];
        int local = t - tb.tile_prefix[lo] * p.nb_count;
        int mt;
        if (p.nb_inner) {  // all column blocks of one row tile first: the rows are streamed once, the weights come from L2
            mt = local / p.nb_count;
            ti.nb = local - mt * p.nb_count;
        } else {  // all row tiles of one column block first: the weight panel is shared by the tiles in flight
            ti.nb = local / mt_e;
            mt = local - ti.nb * mt_e;
        }
        ti.mb = mt;
        ti.row0 = tb.seg_start[lo] + mt * BM;
        int cover = p.padded ? (tb.seg_cnt[lo] + kPadRows - 1) / kPadRows * kPadRows : tb.seg_cnt[lo];
        ti.rows_valid = min(BM, cover - mt * BM);
        ti.ksteps = (p.K + BK - 1) / BK;
    }
}


// ---- epilogue of one tile ------------------------------------------------------------------------
// Runs in the epilogue warps.  `taddr` addresses this warp's 32 TMEM lanes of the tile's accumulator, `q` is the
// lane quarter, `half` selects which half of the tile's columns this warp handles, `stage_store(map, c0, c1, c2,
// packed[16])` sends one 32 x 32 box of 16-bit values to the output through shared memory and TMA.
template <int EPI, class StageStore>
__device__ __forceinline__ void epilogue_tile(const UmmaParams& p, const Tile& ti, uint32_t taddr, int q, int half, int lane,
                                              const CUtensorMap* mo, const CUtensorMap* mo2, const CUtensorMap* mo3,
                                              StageStore& stage_store, int c_begin = -1, int c_end = -1) {
    // column range of this warp in BN-wide epilogues; the default is the half the warp's index names
    if (c_begin < 0) {
        c_begin = half * (BN / 2);
        c_end = c_begin + BN / 2;
    }
    const int r = q * 32 + lane;  // row of the tile this thread owns
    const int is_f16 = p.is_f16;
    const bool have_acc = ti.ksteps > 0;

    if (EPI == EPI_STORE) {
        const int n0 = ti.nb * BN;
        // whole-row output (weight gradients; grouped rows when this warp's 32 rows are all real)
        const bool via_tma = p.wfam || (p.o_map == nullptr && p.scale == nullptr && q * 32 + 32 <= ti.rows_valid);
        if (via_tma) {
            const int row_c = p.wfam ? ti.mb * BM + q * 32 : ti.row0 + q * 32;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                if (n0 + c >= p.N) break;
                uint32_t v[32], pk[16];
                if (have_acc) {
                    tc_ld32(taddr + c, v);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), is_f16);
                stage_store(mo, n0 + c, row_c, ti.e, pk);
            }
        } else {
            bool row_ok = r < ti.rows_valid;
            int d = -1;
            if (row_ok) d = p.o_map ? p.o_map[ti.row0 + r] : ti.row0 + r;
            row_ok = d >= 0;
            const int64_t dst = d;
            float sc = 1.f;
            if (row_ok && p.scale) sc = load_scalar(p.scale, dst, is_f16);
            uint8_t* orow = (uint8_t*)p.out + (dst * p.ldo + n0) * 2;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 32) {
                uint32_t v[32];
                if (have_acc) {
                    tc_ld32(taddr + c, v);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                if (row_ok) {
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {
                        if (n0 + c + qd * 8 < p.N) {
                            uint4 o;
                            o.x = pack2(__uint_as_float(v[qd * 8 + 0]) * sc, __uint_as_float(v[qd * 8 + 1]) * sc, is_f16);
                            o.y = pack2(__uint_as_float(v[qd * 8 + 2]) * sc, __uint_as_float(v[qd * 8 + 3]) * sc, is_f16);
                            o.z = pack2(__uint_as_float(v[qd * 8 + 4]) * sc, __uint_as_float(v[qd * 8 + 5]) * sc, is_f16);
                            o.w = pack2(__uint_as_float(v[qd * 8 + 6]) * sc, __uint_as_float(v[qd * 8 + 7]) * sc, is_f16);
                            *reinterpret_cast<uint4*>(orow + (c + qd * 8) * 2) = o;
                        }
                    }
                }
            }
        }
    } else if (epi_gated_forward(EPI)) {
        constexpr int ACT = epi_act(EPI);
        // accumulator columns [0,128) = up, [128,256) = gate, for output columns nb*128 .. +128 of each half;
        // the layout is the padded grouped order, so all 128 rows of the tile are written (fillers get zeros)
        const int I = p.swiglu_half;
        const int n0 = ti.nb * 128;
        const int row_c = ti.row0 + q * 32;
#pragma unroll 1
        for (int c = half * 64; c < (half + 1) * 64; c += 32) {
            if (n0 + c >= I) break;
            uint32_t u[32], gt[32], hu[16], hg[16], av[16];
            tc_ld32(taddr + c, u);
            tc_ld32(taddr + 128 + c, gt);
            tc_wait_ld();
            // What is kept for the backward pass are the two factors of the activation's derivative, not h itself: with
            // d the gradient of the activation output, d(up) = d * m(gate) and d(gate) = d * up * m'(gate).  All the
            // transcendental work thus happens here, where the epilogue has slack, and the down-dgrad epilogue is left with
            // two multiplications per element.  The factors are formed in fp32 from h rounded to the tensor type (what the
            // reference materialises) and rounded once more when stored.
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t ru = pack2(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]), is_f16);
                const uint32_t rg = pack2(__uint_as_float(gt[2 * i]), __uint_as_float(gt[2 * i + 1]), is_f16);
                const float2 fu = unpack2(ru, is_f16), fg = unpack2(rg, is_f16);
                const float s0 = sigmoid_tanh(fg.x), s1 = sigmoid_tanh(fg.y);
                const float m0 = gate_value(ACT, fg.x, s0), m1 = gate_value(ACT, fg.y, s1);
                av[i] = pack2(fu.x * m0, fu.y * m1, is_f16);
                hu[i] = pack2(m0, m1, is_f16);
                hg[i] = pack2(fu.x * gate_slope(ACT, fg.x, s0), fu.y * gate_slope(ACT, fg.y, s1), is_f16);
            }
            // stored interleaved per 32-column chunk: chunk j of a row holds the 32 (w in a ragged last chunk) first factors,
            // then the second factors of the same columns, so that the down-dgrad epilogue finds both in one 128-byte line.
            // The first box has its own map, clipped where the last chunk's second part begins.
            const int wch = min(32, I - (n0 + c));
            stage_store(mo, 2 * (n0 + c), row_c, 0, hu);
            stage_store(mo3, 2 * (n0 + c) + wch, row_c, 0, hg);
            stage_store(mo2, n0 + c, row_c, 0, av);   // activation
        }
    } else if (EPI == EPI_ROUTER) {
        // Router: the tile's columns are the experts.  One thread owns one token row: it rounds the logits to the
        // tensor type and stores them, keeps the ROUTER_KMAX largest (ties: lower expert first) in registers, turns
        // the first k into routing weights and counts the selected experts.  Only the first warp of each lane
        // quarter works; a row is never split between threads.
        if (half == 0) {
            const int E = p.N, k = p.r_k;
            const bool row_ok = r < ti.rows_valid;
            const int64_t row = ti.row0 + r;
            float tv[ROUTER_KMAX];
            int tix[ROUTER_KMAX];
#pragma unroll
            for (int j = 0; j < ROUTER_KMAX; ++j) {
                tv[j] = -INFINITY;
                tix[j] = 0;
            }
            uint8_t* lrow = (uint8_t*)p.out + row * p.ldo * 2;
            const float rs = (p.r_rowscale != nullptr && row_ok) ? p.r_rowscale[row] : 1.f;
#pragma unroll 1
            for (int c = 0; c < E; c += 32) {
                uint32_t v[32];
                tc_ld32(taddr + c, v);
                tc_wait_ld();
                float f[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) f[i] = round_elem(__uint_as_float(v[i]) * rs, is_f16);
                if (row_ok) {
                    if (p.r_vec) {
#pragma unroll
                        for (int qd = 0; qd < 4; ++qd) {
                            if (c + qd * 8 < E) {
                                uint4 o;
                                o.x = pack2(f[qd * 8 + 0], f[qd * 8 + 1], is_f16);
                                o.y = pack2(f[qd * 8 + 2], f[qd * 8 + 3], is_f16);
                                o.z = pack2(f[qd * 8 + 4], f[qd * 8 + 5], is_f16);
                                o.w = pack2(f[qd * 8 + 6], f[qd * 8 + 7], is_f16);
                                *reinterpret_cast<uint4*>(lrow + (c + qd * 8) * 2) = o;
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c + i < E) {
                                uint32_t pk = pack2(f[i], 0.f, is_f16);
                                *reinterpret_cast<uint16_t*>(lrow + (c + i) * 2) = (uint16_t)(pk & 0xFFFFu);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float val = f[i];
                    if (c + i < E && val > tv[ROUTER_KMAX - 1]) {
                        tv[ROUTER_KMAX - 1] = val;
                        tix[ROUTER_KMAX - 1] = c + i;
#pragma unroll
                        for (int j = ROUTER_KMAX - 1; j > 0; --j) {
                            if (tv[j] > tv[j - 1]) {
                                float a = tv[j];
                                tv[j] = tv[j - 1];
                                tv[j - 1] = a;
                                int b = tix[j];
                                tix[j] = tix[j - 1];
                                tix[j - 1] = b;
                            }
                        }
                    }
                }
            }
            // scores of the first k (fp32), as the eager router computes them from the rounded logits
            float sc[ROUTER_KMAX], sum = 0.f;
#pragma unroll
            for (int j = 0; j < ROUTER_KMAX; ++j) {
                float s = 0.f;
                if (j < k) s = p.r_scoring ? 1.f / (1.f + expf(-tv[j])) : expf(tv[j] - tv[0]);
                sc[j] = s;
                sum += s;
            }
            const float inv = 1.f / sum;
#pragma unroll
            for (int j = 0; j < ROUTER_KMAX; ++j) {
                if (j < k) {
                    if (row_ok) {
                        p.r_indices[row * k + j] = tix[j];
                        uint32_t pk = pack2(sc[j] * inv, 0.f, is_f16);
                        reinterpret_cast<uint16_t*>(p.out2)[row * k + j] = (uint16_t)(pk & 0xFFFFu);
                    }
                    // rows per expert: one atomic per distinct expert among the warp's rows
                    const int key = row_ok ? tix[j] : -1;
                    const unsigned same = __match_any_sync(0xFFFFFFFFu, key);
                    if (key >= 0 && lane == (__ffs(same) - 1)) atomicAdd(p.r_counts + key, __popc(same));
                }
            }
        }
    } else if (EPI == EPI_UNARY) {
        // Non-GLU expert, forward: the tile holds 256 columns of h = x @ w_fc^T.  h is rounded to the tensor type (the
        // reference materialises it); a = gelu_tanh(h) is stored for the down projection and gelu_tanh'(h) for the backward pass.
        const int n0 = ti.nb * BN;
        const int row_c = ti.row0 + q * 32;
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
            if (n0 + c >= p.N) break;
            uint32_t v[32], hv[16], av[16];
            tc_ld32(taddr + c, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float2 f = unpack2(pack2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), is_f16), is_f16);  // h as the reference stores it
                const float t0 = tanh_fast(gelu_tanh_arg(f.x)), t1 = tanh_fast(gelu_tanh_arg(f.y));
                av[i] = pack2(gelu_tanh_value(f.x, t0), gelu_tanh_value(f.y, t1), is_f16);
                hv[i] = pack2(gelu_tanh_slope(f.x, t0), gelu_tanh_slope(f.y, t1), is_f16);  // kept for the backward pass: the derivative
            }
            stage_store(mo, n0 + c, row_c, 0, hv);
            stage_store(mo2, n0 + c, row_c, 0, av);
        }
    } else if (EPI == EPI_DGRAD_UNARY) {
        // Non-GLU expert, input gradient of the down projection: dh = d * gelu_tanh'(h), d = the accumulator rounded to
        // the tensor type; p.h (rows, N) holds gelu_tanh'(h) as the forward epilogue stored it.
        const int n0 = ti.nb * BN;
        const int row_c = ti.row0 + q * 32;
        const uint8_t* hrow = (const uint8_t*)p.h + ((int64_t)(ti.row0 + r) * p.N + n0) * 2;
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
            if (n0 + c >= p.N) break;
            uint4 h4[4];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd)
                h4[qd] = (n0 + c + qd * 8 < p.N) ? *reinterpret_cast<const uint4*>(hrow + (c + qd * 8) * 2) : make_uint4(0, 0, 0, 0);
            uint32_t u[32], dv[16];
            tc_ld32(taddr + c, u);
            tc_wait_ld();
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const uint32_t ha[4] = {h4[qd].x, h4[qd].y, h4[qd].z, h4[qd].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 sl = unpack2(ha[i], is_f16);  // gelu_tanh'(h), stored by the forward epilogue
                    const float2 d = unpack2(pack2(__uint_as_float(u[qd * 8 + 2 * i]), __uint_as_float(u[qd * 8 + 2 * i + 1]), is_f16), is_f16);
                    dv[qd * 4 + i] = pack2(d.x * sl.x, d.y * sl.y, is_f16);
                }
            }
            stage_store(mo, n0 + c, row_c, 0, dv);
        }
    } else {  // EPI_DGRAD_DOWN, EPI_DGRAD_DOWN_GLU
        // The accumulator holds d[p, :] = (gate-scaled upstream gradient rows) @ w_proj[e]: the gradient with respect to
        // the activation output.  It is rounded to the tensor type (the reference materialises it) and multiplied by the two
        // derivative factors the forward epilogue stored (interleaved per 32-column chunk in p.h): d(up) = d * m(gate),
        // d(gate) = d * up * m'(gate).  The same code serves both gate functions.
        const int I = p.N;
        const int64_t prow = ti.row0 + r;
        const int n0 = ti.nb * BN;
        const int row_c = ti.row0 + q * 32;
        const uint8_t* hrow = (const uint8_t*)p.h + prow * 2 * (int64_t)I * 2;
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
            const int col = n0 + c;
            if (col >= I) break;
            const int wch = min(32, I - col);
            const uint8_t* hp = hrow + (int64_t)col * 4;  // chunk base: element 2 * col
            // the stored factors of this row: requested before the accumulator is read
            uint4 hu4[4], hg4[4];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const bool in = qd * 8 < wch;
                hu4[qd] = in ? *reinterpret_cast<const uint4*>(hp + qd * 16) : make_uint4(0, 0, 0, 0);
                hg4[qd] = in ? *reinterpret_cast<const uint4*>(hp + (wch + qd * 8) * 2) : make_uint4(0, 0, 0, 0);
            }
            uint32_t u[32], du[16], dg[16];
            tc_ld32(taddr + c, u);
            tc_wait_ld();
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const uint32_t hua[4] = {hu4[qd].x, hu4[qd].y, hu4[qd].z, hu4[qd].w};
                const uint32_t hga[4] = {hg4[qd].x, hg4[qd].y, hg4[qd].z, hg4[qd].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f1 = unpack2(hua[i], is_f16), f2 = unpack2(hga[i], is_f16);  // m(gate) and up * m'(gate)
                    const float2 d = unpack2(pack2(__uint_as_float(u[qd * 8 + 2 * i]), __uint_as_float(u[qd * 8 + 2 * i + 1]), is_f16), is_f16);
                    du[qd * 4 + i] = pack2(d.x * f1.x, d.y * f1.y, is_f16);
                    dg[qd * 4 + i] = pack2(d.x * f2.x, d.y * f2.y, is_f16);
                }
            }
            stage_store(mo, col, row_c, 0, du);    // up half of dh
            stage_store(mo3, col, row_c, 0, dg);   // gate half of dh
        }
    }
}

// ---- host helpers (defined in umma_gemm.cu) ---------------------------------------------------------
int make_store_map(CUtensorMap* map, const void* base, int64_t experts, int64_t rows, int64_t cols, int64_t ld, int64_t se,
                   int is_f16);
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int is_f16);
int make_gather_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int is_f16);
int sm_count();
int gemm_sm_count();
uint32_t make_idesc(int a_mn, int b_mn, int is_f16, int m, int n = BN);

// two-CTA kernels (umma2_gemm.cu); operands must all be TMA tiles
int launch_2cta(int epi, const UmmaParams& p, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo,
                const CUtensorMap& mo2, const CUtensorMap& mo3, int64_t rows_cap, cudaStream_t stream);

}  // namespace umma
}  // namespace b200moe
