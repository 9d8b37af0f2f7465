// Two-CTA variant of the tensor-core engine: a cluster of two CTAs (two SMs) works on one 256 x 256 output
// tile with tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16).
//
// Each CTA stages its own 128 rows of operand A and HALF of operand B (128 of the 256 B rows), so a CTA
// moves 32 KB per 64-deep k step instead of 48 KB: one third less L2 -> shared-memory traffic and
// shared-memory read bandwidth per FLOP than the one-CTA kernel, and six operand slots fit instead of four.
// The accumulator of a CTA's 128 rows lives in that CTA's tensor memory; each CTA runs its own epilogue.
//
// Protocol (rank 0 of the pair is the leader):
//   * both CTAs' producer lanes wait on their OWN empty barrier, then issue their TMA loads with the
//     completion bytes counted on the LEADER's full barrier (the leader arms it with the bytes of both CTAs);
//   * the leader's MMA lane waits on its full barrier, issues the MMAs, and commits to the empty barrier of
//     BOTH CTAs (one tcgen05.commit with a two-CTA mask) and, at the end of a tile, to both tmem_full barriers;
//   * every epilogue warp of both CTAs arrives on the LEADER's tmem_empty barrier when it has drained its part
//     of the accumulator.
// Tile scheduling.  With a tile counter (a zeroed word in global memory, one per launch) the clusters draw their tiles
// from it: the leader's producer lane takes the next index with atomicAdd while it streams the current tile, and
// hands every index to the other roles of both CTAs through a small ring in shared memory (one mbarrier pair per
// slot).  Tiles are therefore started in list order by whichever cluster is free: clusters that share a weight panel
// stay close together in the list, and the weight-gradient tiles, listed by descending reduction length, are balanced
// longest-first.  Without a counter every cluster walks the list with a fixed stride (its index, then + clusters).
// All operands must be plain TMA tiles (the layer path gathers rows beforehand).  No load uses cluster
// multicast.  Every wait is bounded like in the one-CTA kernel; a cluster barrier at the end keeps either CTA
// from exiting while its peer may still signal into its shared memory.
#include <atomic>
#include <mutex>

#include "umma_common.cuh"

namespace b200moe {
namespace umma {

namespace {

constexpr int STAGES2 = 6;
constexpr int SCHED_SLOTS = 8;  // tile indices in flight between the scheduling lane and the slowest role
constexpr int B_HALF_BYTES = (BN / 2) * BK * 2;  // 16 KB
// Epilogue warps per CTA: twelve (three per TMEM lane quarter with 96 / 96 / 64 columns) for the store and down-dgrad
// epilogues (latency-bound work: about a quarter of an instruction per cycle and scheduler with eight warps; exposed when
// the reduction loop of a tile is short), eight (two per lane quarter, 128 columns each) for the SwiGLU forward epilogue,
// whose register count does not fit twelve.
__host__ __device__ constexpr int epi_warps_of(int epi) { return epi_gated_forward(epi) ? 8 : 12; }
__host__ __device__ constexpr int threads_of(int epi) { return (2 + epi_warps_of(epi)) * 32; }  // + TMA warp, MMA warp

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Bounded wait whose acquire has cluster scope: used where the data guarded by the barrier was written by the peer CTA.
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
static __device__ __noinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                                      int code) {
    long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (mbar_try_wait_cluster(bar, parity)) return true;
            __nanosleep(100);
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of one CTA of the pair; `bar` is a shared::cluster address (the leader's full barrier).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// Row gather of one CTA of the pair: four rows (indices r[0..3]) of 64 columns starting at column c0 land as four
// consecutive 128-byte rows at dst; rows outside the tensor read as zeros.
__device__ __forceinline__ void tma_gather4_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, const int (&r)[4]) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
        : "memory");
}
// One commit that arrives on the barrier at the same offset in BOTH CTAs of the pair (`bar`: this CTA's address).  A
// single instruction with a two-CTA mask instead of one commit per CTA: measured 40-50 clocks less per k step.
__device__ __forceinline__ void tc_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((unsigned short)3)
                 : "memory");
}
// tcgen05.mma of the pair with the descriptors given as (low, high) words: along the k loop only the 14-bit start-address
// field in the low word changes (shared memory is below 256 KB, so the field never carries), which keeps the per-MMA
// address arithmetic of the issuing lane at one 32-bit add per operand.
__device__ __forceinline__ void tc_mma_pair_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// The k loops of the producer and MMA lanes are unrolled over the operand slots of the ring (entered at the ring's
// current position, Duff's-device style): one thread issues everything, each of its instructions waits for the one
// before, and with the slot a compile-time constant the barrier and buffer addresses are immediates.  Measured on a
// B200: the MMA lane of the rolled loop needed about 610 clocks per k step (340 of bookkeeping and hand-over, 70 per
// MMA) while the tensor pipe needs 512, i.e. the pipe idled a sixth of the time waiting for its next instruction.
#define B200MOE_SLOT_CASES(STEP) STEP(0) STEP(1) STEP(2) STEP(3) STEP(4) STEP(5)
static_assert(STAGES2 == 6 && BK == 64, "the slot cases and the four MMAs per k step are written out");

// Tile list of the pair kernels.  Family R: a cluster tile is two consecutive 128-row blocks of one expert
// (the second may not exist when the expert has an odd number of blocks: that CTA then idles through the tile);
// tile_prefix counts cluster tiles.  Family W: output blocks of 256 x 256, CTA `rank` owns rows 128*rank..+127.
__device__ __forceinline__ int total_tiles2(const UmmaParams& p, const Tables& tb) {
    return p.wfam ? p.E * ((p.mb_count + 1) / 2) * p.nb_count : tb.tile_prefix[p.E] * p.nb_count;
}

__device__ __forceinline__ void decode_tile2(const UmmaParams& p, const Tables& tb, int t, int rank, Tile& ti) {
    if (p.wfam) {
        const int mb2 = (p.mb_count + 1) / 2;
        int per_e = mb2 * p.nb_count;
        const int ei = t / per_e;
        ti.e = tb.order[ei];
        int local = t - ei * per_e;
        int pair;
        if (mb2 <= p.nb_count) {
            pair = local % mb2;
            ti.nb = local / mb2;
        } else {
            ti.nb = local % p.nb_count;
            pair = local / p.nb_count;
        }
        ti.mb = 2 * pair + rank;
        ti.row0 = tb.seg_start[ti.e];
        ti.rows_valid = tb.seg_cnt[ti.e];
        ti.ksteps = (ti.rows_valid + BK - 1) / BK;
    } else {
        int lo = 0, hi = p.E - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (tb.tile_prefix[mid] * p.nb_count <= t) {
                lo = mid;
            } else {
                hi = mid - 1;
            }
        }
        ti.e = lo;
        int pairs_e = tb.tile_prefix[lo + 1] - tb.tile_prefix[lo];
        int local = t - tb.tile_prefix[lo] * p.nb_count;
        int pair;
        if (p.nb_inner) {
            pair = local / p.nb_count;
            ti.nb = local - pair * p.nb_count;
        } else if (p.blocked_rows > 0 && pairs_e * 2 * BM > p.blocked_rows) {
            // Blocks of 8 row tiles x 8 column blocks, one block after the other: the 64 tiles of a block are handed out
            // together and share 8 + 8 operand panels (opt-in: tile-order option 2).
            const int per_brow = 8 * p.nb_count;
            int pb = local / per_brow;
            const int nbr = (pairs_e + 7) >> 3;
            if (pb > nbr - 1) pb = nbr - 1;
            const int rows_in = min(8, pairs_e - 8 * pb);
            const int local2 = local - pb * per_brow;
            const int nbc = (p.nb_count + 7) >> 3;
            int qb = local2 / (rows_in * 8);
            if (qb > nbc - 1) qb = nbc - 1;
            const int local3 = local2 - qb * rows_in * 8;
            const int q_in = local3 / rows_in;
            pair = 8 * pb + (local3 - q_in * rows_in);
            ti.nb = 8 * qb + q_in;
        } else {
            ti.nb = local / pairs_e;
            pair = local - ti.nb * pairs_e;
        }
        int blk = 2 * pair + rank;
        ti.mb = blk;
        ti.row0 = tb.seg_start[lo] + blk * BM;
        int cover = p.padded ? (tb.seg_cnt[lo] + kPadRows - 1) / kPadRows * kPadRows : tb.seg_cnt[lo];
        int left = cover - blk * BM;
        ti.rows_valid = left <= 0 ? 0 : (left < BM ? left : BM);
        ti.ksteps = (p.K + BK - 1) / BK;
    }
}

// Barriers and bookkeeping of one CTA; both CTAs of a pair use the same offsets, so a peer's word is this CTA's address
// mapped to the other rank.
struct Ctl2 {
    uint64_t full_bar[STAGES2];        // used in the leader only
    uint64_t empty_bar[STAGES2];       // one set per CTA
    uint64_t tmem_full_bar[2];         // one set per CTA
    uint64_t tmem_empty_bar[2];        // used in the leader only
    uint64_t sched_full[SCHED_SLOTS];  // one set per CTA: a tile index has been written to sched_tile[slot]
    uint64_t sched_empty[SCHED_SLOTS]; // used in the leader only: every role of both CTAs has read the slot
    int sched_tile[SCHED_SLOTS];
    uint32_t tmem_slot;
    int abort_flag;
    int use_counter;  // tiles come from the global counter (else: fixed stride)
    int pad[1];
    Tables tb;
};

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads_of(EPI), 1)
    umma2_grouped_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_o,
                         const __grid_constant__ CUtensorMap tmap_o2, const __grid_constant__ CUtensorMap tmap_o3) {
    extern __shared__ uint8_t smem_raw[];
    // identical layout in both CTAs of the pair: the peer's buffers and barriers sit at the same offsets
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES2 * A_STAGE_BYTES;
    uint8_t* smem_stg = smem + STAGES2 * (A_STAGE_BYTES + B_HALF_BYTES);
    constexpr int EW = epi_warps_of(EPI);
    Ctl2& ctl = *(Ctl2*)(smem_stg + EW * STG_BYTES);
    uint64_t* full_bar = ctl.full_bar;
    uint64_t* empty_bar = ctl.empty_bar;
    uint64_t* tmem_full_bar = ctl.tmem_full_bar;
    uint64_t* tmem_empty_bar = ctl.tmem_empty_bar;
    volatile int* abort_flag = (volatile int*)&ctl.abort_flag;
    Tables& tb = ctl.tb;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;

    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
        int64_t prev = e ? p.offsets[e - 1] : 0;
        tb.seg_cnt[e] = (int)(p.offsets[e] - prev);
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES2; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&tmem_full_bar[a]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[a]), 2 * EW);
        }
        for (int s = 0; s < SCHED_SLOTS; ++s) {
            mbar_init(smem_u32(&ctl.sched_full[s]), 1);
            // readers of a slot: the leader's MMA lane and epilogue warps, the peer's producer and epilogue warps
            mbar_init(smem_u32(&ctl.sched_empty[s]), 2 + 2 * EW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (p.wfam) fill_expert_order(tb, p.E);
    if (threadIdx.x == 0) {
        int start = 0, tiles = 0, maxc = 0;
        long long sum = 0;
        for (int e = 0; e < p.E; ++e) {
            int cnt = tb.seg_cnt[e];
            int cover = p.padded ? (cnt + kPadRows - 1) / kPadRows * kPadRows : cnt;
            tb.seg_start[e] = start;
            tb.tile_prefix[e] = tiles;
            start += cover;
            tiles += ((cover + BM - 1) / BM + 1) / 2;
            sum += cnt;
            maxc = cnt > maxc ? cnt : maxc;
        }
        tb.tile_prefix[p.E] = tiles;
        // Weight-gradient tiles are drawn from the counter only when the experts' row counts are uneven (the largest above
        // twice the mean): with even counts the fixed stride balances as well and needs no hand-over of indices.  Both
        // CTAs of every cluster see the same counts and so take the same decision.
        ctl.use_counter = p.tile_counter != nullptr && (!p.wfam || (long long)maxc * p.E > 2 * sum);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();  // barriers of both CTAs are initialised and visible before anyone signals the peer
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&ctl.tmem_slot;
    const int ntiles = total_tiles2(p, tb);
    const bool dyn = *(volatile int*)&ctl.use_counter != 0;

    // ---- tile feed ----
    // Readers (every role except the leader's producer): the next tile index of this cluster, or a value >= ntiles when
    // the list is exhausted or the kernel is aborting.  `whole_warp`: all 32 lanes call it together (one arrival).
    int f_slot = 0;
    uint32_t f_phase = 0;
    int f_static = cluster_id - nclusters;
    const uint32_t lead_sched_empty0 = map_to_cta(smem_u32(&ctl.sched_empty[0]), 0);
    auto next_tile = [&](bool whole_warp, int code) -> int {
        if (!dyn) {
            f_static += nclusters;
            return f_static;
        }
        const uint32_t bar = smem_u32(&ctl.sched_full[f_slot]);
        int t;
        if (rank == 0) {
            // the leader's own roles: index and barriers are local, CTA-scope ordering suffices (the cluster-scope
            // forms cost the MMA lane over a thousand clocks per tile)
            if (!mbar_wait(bar, f_phase, abort_flag, p.status, code)) return 0x7fffffff;
            t = *(volatile int*)&ctl.sched_tile[f_slot];
            if (whole_warp) __syncwarp();
            if (!whole_warp || lane == 0) mbar_arrive(smem_u32(&ctl.sched_empty[f_slot]));
        } else {
            if (!mbar_try_wait_cluster(bar, f_phase) && !mbar_wait_cluster(bar, f_phase, abort_flag, p.status, code)) return 0x7fffffff;
            t = *(volatile int*)&ctl.sched_tile[f_slot];
            if (whole_warp) __syncwarp();
            if (!whole_warp || lane == 0) mbar_arrive_cluster(lead_sched_empty0 + f_slot * 8);
        }
        if (++f_slot == SCHED_SLOTS) {
            f_slot = 0;
            f_phase ^= 1;
        }
        return t;
    };
    // The leader's producer lane: publishes tile index t to both CTAs.  Returns false when the kernel is aborting.
    auto publish_tile = [&](int t) -> bool {
        if (!mbar_wait(smem_u32(&ctl.sched_empty[f_slot]), f_phase ^ 1, abort_flag, p.status, 216)) return false;
        ctl.sched_tile[f_slot] = t;
        st_cluster_u32(map_to_cta(smem_u32(&ctl.sched_tile[f_slot]), 1), (uint32_t)t);
        mbar_arrive(smem_u32(&ctl.sched_full[f_slot]));
        mbar_arrive_cluster(map_to_cta(smem_u32(&ctl.sched_full[f_slot]), 1));
        if (++f_slot == SCHED_SLOTS) {
            f_slot = 0;
            f_phase ^= 1;
        }
        return true;
    };
    const bool scheduler = dyn && rank == 0;  // this CTA's producer lane draws the tiles

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (p.a_g4 || p.b_g4) {
            // Row-gather variant (opt-in engine): operands whose rows are picked by a row map come in through TMA row
            // gather (tile::gather4).  Every lane owns four rows of the stage and issues one gather per k step and
            // gathered operand; lane 0 also waits for the free stage, arms the barrier and issues the plain tile loads.
            // The row indices are read before the wait, so their latency hides behind it.
            int stage = 0;
            uint32_t phase = 0;
            Tile ti;
            int ok = 1;
            int t = cluster_id, nxt = cluster_id + nclusters;  // see the plain producer below for the scheduling scheme
            if (scheduler) {
                if (lane == 0) ok = publish_tile(t) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            while (ok) {
                int nxt2 = nxt + nclusters;
                if (scheduler) {
                    if (t >= ntiles) break;
                    if (lane == 0) {
                        ok = publish_tile(nxt) ? 1 : 0;
                        nxt2 = nxt < ntiles ? 2 * nclusters + (int)atomicAdd(p.tile_counter, 1u) : nxt;
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    nxt2 = __shfl_sync(0xffffffffu, nxt2, 0);
                    if (!ok) break;
                } else {
                    if (dyn) {
                        if (lane == 0) t = next_tile(false, 217);
                        t = __shfl_sync(0xffffffffu, t, 0);
                    }
                    if (t >= ntiles) break;
                }
                decode_tile2(p, tb, t, rank, ti);
                for (int ks = 0; ks < ti.ksteps; ++ks) {
                    const int k0 = ks * BK;
                    int ia[4], ib[4];
                    if (!p.wfam) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {  // K-major A: rows 4*lane .. 4*lane+3 of this CTA's 128 tile rows
                            int r = 4 * lane + i, v = -1;
                            if (r < ti.rows_valid) v = p.a_map[ti.row0 + r];
                            ia[i] = v < 0 ? p.a_oob : v;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {  // MN-major: token rows k0 + 4*(lane%16) .. +3, column block lane/16
                            int r = k0 + 4 * (lane & 15) + i, va = -1, vb = -1;
                            if (r < ti.rows_valid) {
                                if (p.a_g4) va = p.a_map[ti.row0 + r];
                                if (p.b_g4) vb = p.b_map[ti.row0 + r];
                            }
                            ia[i] = va < 0 ? p.a_oob : va;
                            ib[i] = vb < 0 ? p.b_oob : vb;
                        }
                    }
                    const uint32_t lead_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
                    const uint32_t sa = smem_u32(smem_a + stage * A_STAGE_BYTES);
                    const uint32_t sb = smem_u32(smem_b + stage * B_HALF_BYTES);
                    if (lane == 0) {
                        ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, 211) ? 1 : 0;
                        if (ok) {
                            if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * (A_STAGE_BYTES + B_HALF_BYTES));
                            if (p.wfam) {
                                int krow = ti.row0 + k0;
                                if (!p.a_g4)
                                    for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, lead_full, ti.mb * BM + j * 64, krow);
                                if (!p.b_g4)
                                    for (int j = 0; j < 2; ++j)
                                        tma_load_2d_pair(sb + j * 8192, &tmap_b, lead_full, ti.nb * BN + (int)rank * 128 + j * 64, krow);
                            } else if (p.b_mn) {
                                int krow = ti.e * p.b_rows_per_expert + k0;
                                for (int j = 0; j < 2; ++j)
                                    tma_load_2d_pair(sb + j * 8192, &tmap_b, lead_full, ti.nb * BN + (int)rank * 128 + j * 64, krow);
                            } else {
                                int r0 = epi_gated_forward(EPI) ? ti.e * p.b_rows_per_expert + ti.nb * 128 + (int)rank * p.swiglu_half
                                                           : ti.e * p.b_rows_per_expert + ti.nb * BN + (int)rank * 128;
                                tma_load_2d_pair(sb, &tmap_b, lead_full, k0, r0);
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    if (!p.wfam) {
                        tma_gather4_pair(sa + lane * 512, &tmap_a, lead_full, k0, ia);
                    } else {
                        const int j = lane >> 4;
                        const uint32_t off = (uint32_t)j * 8192u + (uint32_t)(lane & 15) * 512u;
                        if (p.a_g4) tma_gather4_pair(sa + off, &tmap_a, lead_full, ti.mb * BM + j * 64, ia);
                        if (p.b_g4) tma_gather4_pair(sb + off, &tmap_b, lead_full, ti.nb * BN + (int)rank * 128 + j * 64, ib);
                    }
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                t = nxt;
                nxt = nxt2;
            }
        } else if (lane == 0) {
            // plain tile loads: one lane per CTA
            int slot = 0;  // ring position; `phase` flips when it wraps
            uint32_t phase = 0;
            Tile ti;
            bool ok = true;
            const uint32_t lead_full0 = map_to_cta(smem_u32(&full_bar[0]), 0);
            const uint32_t full0 = smem_u32(&full_bar[0]);
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            const uint32_t sa0 = smem_u32(smem_a), sb0 = smem_u32(smem_b);
            // One tile's k loop.  MODE 0: both operands K-major (one 64 x 128 box each); 1: weight-gradient family
            // (both operands token-major, two 64 x 64 boxes each); 2: B stored MN-major (one box of A, two of B).
            // `ca` / `cb`: the tile's fixed coordinate of each operand; the other coordinate advances by BK per k step.
            auto load_tile = [&](auto mode, const int nk, const int ca, const int cb, const int kbase_a, const int kbase_b) -> bool {
                constexpr int MODE = decltype(mode)::value;
                int ka = kbase_a, kb = kbase_b;
                int ks = 0;
                for (;;) {
                    switch (slot) {
#define B200MOE_LOAD_STEP(S)                                                                                              \
    case S: {                                                                                                             \
        if (ks == nk) {                                                                                                   \
            slot = S;                                                                                                     \
            return true;                                                                                                  \
        }                                                                                                                 \
        if (!mbar_wait(empty0 + S * 8, phase ^ 1, abort_flag, p.status, 211)) return false;                               \
        if (rank == 0) mbar_arrive_expect_tx(full0 + S * 8, 2 * (A_STAGE_BYTES + B_HALF_BYTES));                          \
        constexpr uint32_t off_a = S * A_STAGE_BYTES, off_b = S * B_HALF_BYTES;                                           \
        if (MODE == 1) {                                                                                                  \
            tma_load_2d_pair(sa0 + off_a, &tmap_a, lead_full0 + S * 8, ca, ka);                                           \
            tma_load_2d_pair(sa0 + off_a + 8192, &tmap_a, lead_full0 + S * 8, ca + 64, ka);                               \
            tma_load_2d_pair(sb0 + off_b, &tmap_b, lead_full0 + S * 8, cb, kb);                                           \
            tma_load_2d_pair(sb0 + off_b + 8192, &tmap_b, lead_full0 + S * 8, cb + 64, kb);                               \
        } else if (MODE == 2) {                                                                                           \
            tma_load_2d_pair(sa0 + off_a, &tmap_a, lead_full0 + S * 8, ka, ca);                                           \
            tma_load_2d_pair(sb0 + off_b, &tmap_b, lead_full0 + S * 8, cb, kb);                                           \
            tma_load_2d_pair(sb0 + off_b + 8192, &tmap_b, lead_full0 + S * 8, cb + 64, kb);                               \
        } else {                                                                                                          \
            tma_load_2d_pair(sa0 + off_a, &tmap_a, lead_full0 + S * 8, ka, ca);                                           \
            tma_load_2d_pair(sb0 + off_b, &tmap_b, lead_full0 + S * 8, kb, cb);                                           \
        }                                                                                                                 \
        ka += BK;                                                                                                         \
        kb += BK;                                                                                                         \
        ++ks;                                                                                                             \
    }
                        B200MOE_SLOT_CASES(B200MOE_LOAD_STEP)
#undef B200MOE_LOAD_STEP
                    }
                    slot = 0;
                    phase ^= 1;
                }
            };
            // Scheduling lane: the first two tiles of a cluster are fixed (its index, then + clusters), the following ones
            // come from the counter.  An index is published a whole tile before it is needed (while tile i streams, the
            // other roles already hold the index of tile i + 1), and the counter is read two tiles ahead, so neither the
            // atomic nor the hand-over to the peer CTA is ever waited for.
            int t = cluster_id, nxt = cluster_id + nclusters;
            if (scheduler && !publish_tile(t)) ok = false;
            while (ok) {
                if (scheduler) {
                    if (t >= ntiles) break;
                    if (!publish_tile(nxt)) break;
                } else {
                    if (dyn) t = next_tile(false, 217);
                    if (t >= ntiles) break;
                }
                int nxt2 = nxt + nclusters;
                if (scheduler) nxt2 = nxt < ntiles ? 2 * nclusters + (int)atomicAdd(p.tile_counter, 1u) : nxt;
                decode_tile2(p, tb, t, rank, ti);
                if (p.wfam) {
                    ok = load_tile(IntTag<1>{}, ti.ksteps, ti.mb * BM, ti.nb * BN + (int)rank * 128, ti.row0, ti.row0);
                } else if (p.b_mn) {
                    ok = load_tile(IntTag<2>{}, ti.ksteps, ti.row0, ti.nb * BN + (int)rank * 128, 0, ti.e * p.b_rows_per_expert);
                } else {
                    // gated forward: the leader loads 128 "up" rows of W, the peer the matching 128 "gate" rows
                    const int r0 = epi_gated_forward(EPI) ? ti.e * p.b_rows_per_expert + ti.nb * 128 + (int)rank * p.swiglu_half
                                                          : ti.e * p.b_rows_per_expert + ti.nb * BN + (int)rank * 128;
                    ok = load_tile(IntTag<0>{}, ti.ksteps, ti.row0, r0, 0, 0);
                }
                t = nxt;
                nxt = nxt2;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            int slot = 0;  // ring position; `phase` flips when it wraps
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            Tile ti;
            const uint32_t a_step = p.a_mn ? 128u : 2u;
            const uint32_t b_step = p.b_mn ? 128u : 2u;
            const uint64_t adesc0 = make_desc(smem_u32(smem_a), p.a_mn);
            const uint64_t bdesc0 = make_desc(smem_u32(smem_b), p.b_mn);
            const uint32_t a_lo0 = (uint32_t)adesc0, a_hi = (uint32_t)(adesc0 >> 32);
            const uint32_t b_lo0 = (uint32_t)bdesc0, b_hi = (uint32_t)(bdesc0 >> 32);
            const uint32_t full0 = smem_u32(&full_bar[0]);
            const uint32_t empty0 = smem_u32(&empty_bar[0]);
            const uint32_t idesc = p.idesc;
            // One tile's k loop: per k step one wait for the operands, four MMAs, one commit that frees the slot in both
            // CTAs once the MMAs have read it.  Nothing else: the tensor pipe queues only a few instructions, so whatever
            // this lane executes between two MMAs beyond the pipe's 128 clocks per MMA is idle time of the pipe.
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
        if (!mbar_wait(full0 + S * 8, phase, abort_flag, p.status, 213)) return false;                                    \
        constexpr uint32_t off_a = S * (A_STAGE_BYTES >> 4), off_b = S * (B_HALF_BYTES >> 4);                             \
        tc_mma_pair_lh(d_tmem, a_lo0 + off_a, a_hi, b_lo0 + off_b, b_hi, idesc, accum);                                   \
        tc_mma_pair_lh(d_tmem, a_lo0 + off_a + a_step, a_hi, b_lo0 + off_b + b_step, b_hi, idesc, 1u);                    \
        tc_mma_pair_lh(d_tmem, a_lo0 + off_a + 2 * a_step, a_hi, b_lo0 + off_b + 2 * b_step, b_hi, idesc, 1u);            \
        tc_mma_pair_lh(d_tmem, a_lo0 + off_a + 3 * a_step, a_hi, b_lo0 + off_b + 3 * b_step, b_hi, idesc, 1u);            \
        tc_commit_both(empty0 + S * 8);                                                                                   \
        accum = 1u;                                                                                                       \
        ++ks;                                                                                                             \
    }
                        B200MOE_SLOT_CASES(B200MOE_MMA_STEP)
#undef B200MOE_MMA_STEP
                    }
                    slot = 0;
                    phase ^= 1;
                }
            };
            int t = next_tile(false, 218);
            while (t < ntiles) {
                decode_tile2(p, tb, t, 0, ti);
                if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, 212)) break;
                tc_fence_after();
                // the index of the following tile was published a whole tile ago
                const int t_next = next_tile(false, 218);
                if (!mma_tile(ti.ksteps, tmem_base + acc * BN)) break;
                tc_commit_both(smem_u32(&tmem_full_bar[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1;
                }
                t = t_next;
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, each on its own 128 rows) ----------------
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;  // which part of the tile's columns this warp handles
        // column range of a BN-wide epilogue: halves with eight warps; 96 / 96 / 64 columns with twelve
        const int c_begin = EW == 12 ? half * 96 : half * (BN / (EW / 4));
        const int c_end = EW == 12 ? (half == 2 ? BN : c_begin + 96) : c_begin + BN / (EW / 4);
        const uint32_t stg = smem_u32(smem_stg + (warp - 2) * STG_BYTES);
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
        for (int t = next_tile(true, 219), t_next; t < ntiles; t = t_next) {
            decode_tile2(p, tb, t, rank, ti);
            if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, 215, 200)) break;
            t_next = next_tile(true, 219);  // published a tile ago: no wait, and off the path between two accumulators
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            // a CTA whose half of the cluster tile does not exist (odd number of row blocks) has nothing to write
            const bool live = p.wfam || ti.rows_valid > 0;
            if (live) epilogue_tile<EPI>(p, ti, taddr, q, half, lane, &tmap_o, &tmap_o2, &tmap_o3, stage_store, c_begin, c_end);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1;
            }
        }
        if (lane == 0) bulk_wait0();
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

constexpr int smem_bytes2(int epi) {
    return 1024 + STAGES2 * (A_STAGE_BYTES + B_HALF_BYTES) + epi_warps_of(epi) * STG_BYTES + (int)sizeof(Ctl2) + 64;
}

// Tile counters: a ring of zero-initialised words in the library image.  Every launch that schedules its tiles
// dynamically takes the next word and clears it on the launch stream first, so launches in flight at the same time
// (different streams) never share a word unless more than kCounterSlots of them overlap.  In host code the array's
// name is only a stand-in; its device address is looked up once per device.
constexpr int kCounterSlots = 4096;
__device__ unsigned int g_tile_counters[kCounterSlots];
std::mutex g_counter_mutex;
unsigned int* g_counter_base[64] = {nullptr};
std::atomic<unsigned int> g_counter_next{0};

unsigned int* take_tile_counter(cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    unsigned int* base;
    {
        std::lock_guard<std::mutex> lock(g_counter_mutex);
        if (g_counter_base[dev] == nullptr) {
            void* ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_tile_counters) != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return nullptr;
            }
            g_counter_base[dev] = (unsigned int*)ptr;
        }
        base = g_counter_base[dev];
    }
    unsigned int* word = base + (g_counter_next.fetch_add(1, std::memory_order_relaxed) % kCounterSlots);
    if (cudaMemsetAsync(word, 0, sizeof(unsigned int), stream) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return word;
}

template <int EPI>
int launch2(const UmmaParams& p_in, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mo2,
            const CUtensorMap& mo3, int64_t tiles_bound, cudaStream_t stream) {
    auto kern = umma2_grouped_kernel<EPI>;
    constexpr int SMEM_BYTES2 = smem_bytes2(EPI);
    static_assert(SMEM_BYTES2 <= 232448, "shared memory of the two-CTA kernel exceeds 227 KB");
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES2);
    if (err != cudaSuccess) {
        set_error_detail("cudaFuncSetAttribute(smem=%d): %s", SMEM_BYTES2, cudaGetErrorString(err));
        return B200MOE_ERR_LAUNCH;
    }
    int grid = gemm_sm_count() & ~1;  // whole pairs
    UmmaParams p = p_in;
    // With no more tiles than clusters the fixed stride is already the best schedule; otherwise draw tiles dynamically
    // (a counter that cannot be had falls back to the fixed stride).
    p.tile_counter = nullptr;
    // Weight-gradient tiles differ in length by the experts' row counts, so they are always drawn dynamically (longest
    // first).  Row tiles are uniform; drawing them keeps the clusters that share a weight panel in step, which measured
    // equal or better with long reductions (K >= 4096) and slightly worse with short ones, where the hand-over of the
    // index is a larger part of a tile.
    const int mode = option_value(B200MOE_OPT_DYNAMIC_TILES);
    const bool dynamic = mode == 3 || (mode >= 1 && p.wfam) || (mode == 2 && !p.wfam && p.K >= 4096);
    if (dynamic && tiles_bound > grid / 2) p.tile_counter = take_tile_counter(stream);
    kern<<<grid, threads_of(EPI), SMEM_BYTES2, stream>>>(p, ma, mb, mo, mo2, mo3);
    count_launch();
    return check_launch("umma2_grouped_kernel");
}

}  // namespace

int launch_2cta(int epi, const UmmaParams& p, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo,
                const CUtensorMap& mo2, const CUtensorMap& mo3, int64_t rows_cap, cudaStream_t stream) {
    // upper bound of the cluster tiles (the exact number depends on the expert counts, which live on the device)
    const int64_t tiles_bound = p.wfam ? (int64_t)p.E * ((p.mb_count + 1) / 2) * p.nb_count
                                       : (rows_cap / (2 * BM) + p.E) * (int64_t)p.nb_count;
    switch (epi) {
        case EPI_STORE:
            return launch2<EPI_STORE>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        case EPI_SWIGLU:
            return launch2<EPI_SWIGLU>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        case EPI_DGRAD_DOWN:
            return launch2<EPI_DGRAD_DOWN>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        case EPI_GLU:
            return launch2<EPI_GLU>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        case EPI_UNARY:
            return launch2<EPI_UNARY>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        case EPI_DGRAD_UNARY:
            return launch2<EPI_DGRAD_UNARY>(p, ma, mb, mo, mo2, mo3, tiles_bound, stream);
        default:
            set_error_detail("unknown epilogue %d", epi);
            return B200MOE_ERR_ARG;
    }
}

}  // namespace umma
}  // namespace b200moe
