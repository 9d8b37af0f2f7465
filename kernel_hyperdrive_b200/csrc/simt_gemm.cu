// CUDA-core engine for the two grouped-GEMM families: 64x64 output tiles, 16-deep k steps, 4x4 register
// tiles, fp32 fused multiply-add accumulation.  It is the engine for fp32 tensors (true fp32 math, no
// TF32), for shapes the tensor-core engine does not take, and the cross-check of that engine in tests.
#include "common.cuh"

namespace b200moe {

namespace {

constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256;

// Finds which expert the `tile`-th row tile belongs to.  counts are staged in shared memory by the whole
// block, then one thread walks them.  info = {expert or -1, first layout row of the tile, rows to cover,
// layout row where the expert's segment starts, rows of the segment}.
__device__ void locate_row_tile(const int64_t* __restrict__ offsets, int E, int padded, int tile, int* s_cnt,
                                int* info) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int64_t prev = e ? offsets[e - 1] : 0;
        s_cnt[e] = (int)(offsets[e] - prev);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int start = 0, found = -1, row0 = 0, cover = 0, seg0 = 0, segn = 0;
        for (int e = 0; e < E; ++e) {
            int cnt = s_cnt[e];
            int seg_rows = padded ? (cnt + kPadRows - 1) / kPadRows * kPadRows : cnt;
            int nt = (seg_rows + TM - 1) / TM;
            if (tile < nt) {
                found = e;
                row0 = start + tile * TM;
                cover = min(TM, seg_rows - tile * TM);
                seg0 = start;
                segn = cnt;
                break;
            }
            tile -= nt;
            start += seg_rows;
        }
        info[0] = found;
        info[1] = row0;
        info[2] = cover;
        info[3] = seg0;
        info[4] = segn;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(THREADS) simt_row_gemm_kernel(RowGemm g) {
    __shared__ int s_cnt[kMaxExperts];
    __shared__ int info[5];
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    __shared__ int s_src[TM];

    locate_row_tile(g.offsets, g.E, g.padded, blockIdx.x, s_cnt, info);
    const int e = info[0];
    if (e < 0) return;
    const int row0 = info[1], cover = info[2];
    const int n0 = blockIdx.y * TN;
    const T* __restrict__ A = (const T*)g.A;
    const T* __restrict__ W = (const T*)g.W + (int64_t)e * g.w_se;

    if (threadIdx.x < TM) {
        int r = threadIdx.x, src = -1;
        if (r < cover) src = g.a_map ? g.a_map[row0 + r] : row0 + r;
        s_src[r] = src;
    }
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int a_r = threadIdx.x / 4, a_k = (threadIdx.x % 4) * 4;  // A: 64 rows x 16 k, 4 consecutive k per thread
    const bool w_n_contig = g.w_sn == 1;

    for (int k0 = 0; k0 < g.K; k0 += TK) {
        {
            int src = s_src[a_r];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int kk = k0 + a_k + i;
                float v = 0.f;
                if (src >= 0 && kk < g.K) v = Elem<T>::to_f(A[(int64_t)src * g.lda + kk]);
                As[a_k + i][a_r] = v;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int kk, nn;
            if (w_n_contig) {
                nn = threadIdx.x % TN;
                kk = threadIdx.x / TN + 4 * i;
            } else {
                kk = threadIdx.x % TK;
                nn = threadIdx.x / TK + 16 * i;
            }
            float v = 0.f;
            if (k0 + kk < g.K && n0 + nn < g.N) v = Elem<T>::to_f(W[(int64_t)(k0 + kk) * g.w_sk + (int64_t)(n0 + nn) * g.w_sn]);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    T* __restrict__ out = (T*)g.out;
    const T* __restrict__ scale = (const T*)g.scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = ty * 4 + i;
        if (r >= cover) continue;
        int dst = g.o_map ? g.o_map[row0 + r] : row0 + r;
        if (dst < 0) continue;
        float sc = scale ? Elem<T>::to_f(scale[dst]) : 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n < g.N) out[(int64_t)dst * g.ldo + n] = Elem<T>::from_f(acc[i][j] * sc);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) simt_w_gemm_kernel(WGemm g) {
    __shared__ int s_cnt[kMaxExperts];
    __shared__ int info[2];
    __shared__ float Ps[TK][TM + 1];
    __shared__ float Qs[TK][TN + 1];
    __shared__ int s_p[TK], s_q[TK];

    const int e = blockIdx.z;
    for (int i = threadIdx.x; i < g.E; i += blockDim.x) {
        int64_t prev = i ? g.offsets[i - 1] : 0;
        s_cnt[i] = (int)(g.offsets[i] - prev);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int start = 0;
        for (int i = 0; i < e; ++i) {
            int cnt = s_cnt[i];
            start += g.padded ? (cnt + kPadRows - 1) / kPadRows * kPadRows : cnt;
        }
        info[0] = start;
        info[1] = s_cnt[e];
    }
    __syncthreads();
    const int seg0 = info[0], cnt = info[1];
    const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    const T* __restrict__ P = (const T*)g.P;
    const T* __restrict__ Q = (const T*)g.Q;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;

    for (int r0 = 0; r0 < cnt; r0 += TK) {
        if (threadIdx.x < TK) {
            int r = r0 + threadIdx.x, sp = -1, sq = -1;
            if (r < cnt) {
                sp = g.p_map ? g.p_map[seg0 + r] : seg0 + r;
                sq = g.q_map ? g.q_map[seg0 + r] : seg0 + r;
            }
            s_p[threadIdx.x] = sp;
            s_q[threadIdx.x] = sq;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int c = threadIdx.x % TM, r = threadIdx.x / TM + 4 * i;
            float pv = 0.f, qv = 0.f;
            int sp = s_p[r], sq = s_q[r];
            if (sp >= 0 && m0 + c < g.Mout) pv = Elem<T>::to_f(P[(int64_t)sp * g.ldp + m0 + c]);
            if (sq >= 0 && n0 + c < g.Nout) qv = Elem<T>::to_f(Q[(int64_t)sq * g.ldq + n0 + c]);
            Ps[r][c] = pv;
            Qs[r][c] = qv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Ps[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Qs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    T* __restrict__ DW = (T*)g.DW + (int64_t)e * g.d_se;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= g.Mout) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n < g.Nout) DW[(int64_t)m * g.d_sm + (int64_t)n * g.d_sn] = Elem<T>::from_f(acc[i][j]);
        }
    }
}

}  // namespace

int simt_row_gemm(const RowGemm& g, int dtype, cudaStream_t stream) {
    if (g.rows_cap == 0 || g.N == 0) return B200MOE_OK;
    int64_t tiles = g.padded ? g.rows_cap / TM : (g.rows_cap + TM - 1) / TM + g.E;
    dim3 grid((unsigned)tiles, (unsigned)((g.N + TN - 1) / TN));
    switch (dtype) {
        case B200MOE_F32:
            simt_row_gemm_kernel<float><<<grid, THREADS, 0, stream>>>(g);
            break;
        case B200MOE_BF16:
            simt_row_gemm_kernel<__nv_bfloat16><<<grid, THREADS, 0, stream>>>(g);
            break;
        case B200MOE_F16:
            simt_row_gemm_kernel<__half><<<grid, THREADS, 0, stream>>>(g);
            break;
        default:
            set_error_detail("unknown dtype code %d", dtype);
            return B200MOE_ERR_DTYPE;
    }
    count_launch();
    return check_launch("simt_row_gemm");
}

int simt_w_gemm(const WGemm& g, int dtype, cudaStream_t stream) {
    if (g.Mout == 0 || g.Nout == 0 || g.E == 0) return B200MOE_OK;
    dim3 grid((unsigned)((g.Mout + TM - 1) / TM), (unsigned)((g.Nout + TN - 1) / TN), (unsigned)g.E);
    switch (dtype) {
        case B200MOE_F32:
            simt_w_gemm_kernel<float><<<grid, THREADS, 0, stream>>>(g);
            break;
        case B200MOE_BF16:
            simt_w_gemm_kernel<__nv_bfloat16><<<grid, THREADS, 0, stream>>>(g);
            break;
        case B200MOE_F16:
            simt_w_gemm_kernel<__half><<<grid, THREADS, 0, stream>>>(g);
            break;
        default:
            set_error_detail("unknown dtype code %d", dtype);
            return B200MOE_ERR_DTYPE;
    }
    count_launch();
    return check_launch("simt_w_gemm");
}

}  // namespace b200moe
