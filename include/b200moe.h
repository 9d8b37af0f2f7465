/*
 * b200moe — C ABI of the B200 (sm_100a) scattermoe path.
 *
 * Plain pointers and sizes only; every pointer named "device" is a CUDA device address owned by the
 * caller.  No entry point allocates device memory unless it says so; scratch memory is passed in as a
 * workspace whose size the matching *_workspace_bytes function returns.  Every launch goes to the stream
 * the caller passes (a cudaStream_t) and returns without synchronising.  Return value: 0 on success, a
 * negative B200MOE_ERR_* code otherwise (b200moe_error_string / b200moe_last_error_detail explain it).
 * Nothing throws across this boundary.
 *
 * Each entry point names the reference interface it replaces.  Reference paths are relative to the
 * reference project root; SMT/ = cute_kernels/kernels/scattermoe/triton_implementation/.
 *
 * Layout vocabulary
 *   T tokens, k experts per token, M = T*k routed rows, E experts, H hidden, I intermediate.
 *   "scattered" order: row s = t*k + j (token t, slot j).  "grouped" order: rows sorted by expert.
 *   "padded grouped" order: grouped order in which every expert's segment starts at a multiple of 128
 *   rows; the rows of an expert keep their grouped order; filler rows hold zeros.  The padded row count
 *   never exceeds b200moe_padded_rows_cap(M, E).
 *   dtype: B200MOE_F32 / B200MOE_BF16 / B200MOE_F16 — the element type of every floating-point buffer of
 *   the call, unless a parameter says otherwise.  Accumulation is always fp32.
 */
#ifndef B200MOE_H
#define B200MOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_F32 0
#define B200MOE_BF16 1
#define B200MOE_F16 2

#define B200MOE_OK 0
#define B200MOE_ERR_ARG (-1)         /* null pointer, negative size, inconsistent shapes            */
#define B200MOE_ERR_DTYPE (-2)       /* unknown dtype code                                          */
#define B200MOE_ERR_LAYOUT (-3)      /* stride / alignment the kernels do not handle                */
#define B200MOE_ERR_WORKSPACE (-4)   /* workspace too small                                         */
#define B200MOE_ERR_LAUNCH (-5)      /* CUDA reported an error at launch                            */
#define B200MOE_ERR_UNSUPPORTED (-6) /* more experts than the kernels are built for, etc.           */
#define B200MOE_ERR_DRIVER (-7)      /* tensor-map encode entry point unavailable or failed         */
#define B200MOE_ERR_DEVICE (-8)      /* a kernel gave up on a bounded wait or saw a bad index       */

#define B200MOE_MAX_EXPERTS 512

/* Engine selection for the grouped GEMMs (b200moe_set_engine).                                       */
#define B200MOE_ENGINE_AUTO 0 /* fp32 -> SIMT, bf16/fp16 -> tcgen05 when the shape allows, else SIMT */
#define B200MOE_ENGINE_SIMT 1 /* CUDA-core kernels for every dtype (exact fp32 math, cross-checks)   */
#define B200MOE_ENGINE_UMMA 2 /* tcgen05 only; shapes it cannot take return B200MOE_ERR_LAYOUT       */
#define B200MOE_ENGINE_UMMA_1CTA 3 /* like UMMA, but never the two-CTA (cta_group::2) kernels     */
#define B200MOE_ENGINE_UMMA_GATHER4 4 /* like UMMA, and operands whose rows are picked by a row map are fetched by
                                       * TMA row gather (tile::gather4) inside the two-CTA kernel instead of by the
                                       * cp.async gather warps of the one-CTA kernel; measured about 3x slower, kept
                                       * for comparison */

typedef void* b200moe_stream_t; /* cudaStream_t */

int b200moe_version(void);
const char* b200moe_error_string(int code);
/* Text describing the last failing call on this host thread (empty if none). */
const char* b200moe_last_error_detail(void);
/* Process-wide engine choice; returns the previous value. */
int b200moe_set_engine(int engine);
/* Number of kernels this library has launched since load (all streams); for launch accounting. */
int64_t b200moe_launch_count(void);
/* Reads the device status word (one int32 written by kernels that give up) after synchronising the
 * stream; returns B200MOE_OK or B200MOE_ERR_DEVICE and clears the word.  status may not be NULL. */
int b200moe_check_status(int32_t* status_device, b200moe_stream_t stream);

/* Failure-path self test (no counterpart in the reference): launches one small CTA that waits, for at most
 * limit_cycles SM cycles, on a barrier nothing arrives on, using the same bounded wait as the GEMM kernels.  The wait
 * gives up, writes code 299 to the status word and the kernel returns normally (finished, optional device int32,
 * receives 1).  b200moe_check_status then reports B200MOE_ERR_DEVICE and the context stays usable. */
int b200moe_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, int32_t* finished, b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Routing
 * ------------------------------------------------------------------------------------------------ */

/* Histogram of ids in [0, size): out[v] = #{i : x[i] == v}, int32.
 * Replaces contiguous_count_cute / contiguous_count_triton
 * (cute_kernels/kernels/contiguous_count/__init__.py:8-24,
 *  cute_kernels/kernels/contiguous_count/triton_implementation/kernels_forward.py:13-66).
 * x: device, n elements, int64 when x_is_int64 else int32.  out: device, `size` int32, overwritten. */
int b200moe_contiguous_count(const void* x, int x_is_int64, int64_t n, int32_t* out, int size,
                             b200moe_stream_t stream);

int64_t b200moe_padded_rows_cap(int64_t M, int E);
int64_t b200moe_route_workspace_bytes(int64_t M, int E);

/* Stable sort of the flat expert ids + histogram + inclusive offsets, and the row maps of the padded
 * grouped order.  Replaces `selected_experts.flatten().sort()` and
 * `contiguous_count_cute(...).cumsum(-1)` (SMT/__init__.py:79-81).  The order inside one expert's segment
 * is ascending flat index (what torch.sort(stable=True) gives).
 *   expert_ids             device int64 (M), values in [0, E)
 *   sorted_expert_idxs     device int64 (M)      or NULL
 *   sorted_scattered_idxs  device int64 (M)      or NULL
 *   expert_offsets         device int64 (E), inclusive prefix sum of the counts
 *   counts                 device int32 (E)      or NULL
 *   row_token, row_slot    device int32 (m_cap)  or NULL (both or neither): for padded grouped row p,
 *                          row_slot[p] = flat index s of the routed row, row_token[p] = s / k, and -1 on
 *                          filler rows
 * m_cap must be >= b200moe_padded_rows_cap(M, E) when the row maps are requested. */
int b200moe_route(const int64_t* expert_ids, int64_t M, int E, int k, int64_t* sorted_expert_idxs,
                  int64_t* sorted_scattered_idxs, int64_t* expert_offsets, int32_t* counts,
                  int32_t* row_token, int32_t* row_slot, int64_t m_cap, void* workspace,
                  int64_t workspace_bytes, int32_t* status, b200moe_stream_t stream);

/* b200moe_route for callers that are not allowed to allocate device memory.  It has no counterpart in the
 * reference.  Some hosts hand this library a device whose memory is already spoken for: a serving process or
 * a training framework that reserved one arena at start-up and treats any later cudaMalloc as a fault, or a
 * caller inside a latency-critical section that cannot afford the device-wide synchronisation an allocation
 * may imply.  Such a caller has nowhere to take the routing workspace from, so this variant keeps the
 * workspace inside the library: a fixed array of b200moe_route_static_scratch_bytes() = 262144 bytes of
 * device memory that is part of the library image (each GPU that loads the library carries it until the
 * process ends).  Inputs and outputs are still the caller's buffers, with the meaning they have in
 * b200moe_route.
 *   - Sizes whose workspace (b200moe_route_workspace_bytes(M, E)) exceeds the array are refused with
 *     B200MOE_ERR_UNSUPPORTED and a message naming both numbers; nothing is launched.  For example
 *     E = 8 fits up to about 33 million rows, E = 256 up to about 1 million, E = 512 up to about 0.5 million.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that device
 *     current and remembers it; make that first call before starting any stream capture.
 *   - The call never calls cudaMalloc, cudaFree or any allocating library routine.
 *   - All calls on one device share the array.  Each call overwrites every word it later reads, so the previous
 *     call's contents do no harm, but two calls that overlap on the GPU (different streams, no ordering
 *     between them) race on it: serialise them. */
int64_t b200moe_route_static_scratch_bytes(void);
int b200moe_route_static(const int64_t* expert_ids, int64_t M, int E, int k, int64_t* sorted_expert_idxs,
                         int64_t* sorted_scattered_idxs, int64_t* expert_offsets, int32_t* counts,
                         int32_t* row_token, int32_t* row_slot, int64_t m_cap, int32_t* status,
                         b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * The reference's four operators, same argument meaning (grouped order WITHOUT padding)
 * ------------------------------------------------------------------------------------------------ */

int64_t b200moe_scatter2scatter_workspace_bytes(int64_t M, int E);

/* Grouped GEMM with fused row gather / scatter.  Replaces the `scatter2scatter` op
 * (SMT/ops.py:16-63, kernel SMT/kernels.py:12-149): for m in [0, M): e = sorted_expert_idxs[m],
 * s = sorted_scattered_idxs[m]; src = m if x_grouped else s / fan_out; dst = m if y_grouped else s;
 * out[dst, :] = X[src, :] @ W[e], W element (e, kk, n) at W + e*w_se + kk*w_sk + n*w_sn.
 * X rows have inner stride 1 and row stride ldx; out likewise with ldo.  One of w_sk, w_sn must be 1. */
int b200moe_scatter2scatter(const void* X, int64_t ldx, const void* W, int64_t w_se, int64_t w_sk,
                            int64_t w_sn, const int64_t* sorted_expert_idxs,
                            const int64_t* sorted_scattered_idxs, void* out, int64_t ldo, int64_t M,
                            int K, int N, int E, int fan_out, int x_grouped, int y_grouped, int dtype,
                            void* workspace, int64_t workspace_bytes, int32_t* status,
                            b200moe_stream_t stream);

/* Per-expert weight gradient on grouped tensors.  Replaces the `group_bwd_W` op
 * (SMT/ops.py:67-94, kernel SMT/kernels.py:152-240):
 * DW[e] (K, N) = X[off[e-1]:off[e]]^T @ DY[off[e-1]:off[e]], element (e, kk, n) at
 * DW + e*d_se + kk*d_sk + n*d_sn.  Experts without rows get zeros (the reference relies on a
 * pre-zeroed DW for them, SMT/kernels.py:199).  expert_offsets: device int64 (E), inclusive. */
int b200moe_group_bwd_W(const void* DY, int64_t lddy, const void* X, int64_t ldx,
                        const int64_t* expert_offsets, void* DW, int64_t d_se, int64_t d_sk,
                        int64_t d_sn, int64_t M, int K, int N, int E, int dtype, int32_t* status,
                        b200moe_stream_t stream);

/* Row gather into grouped order with an optional per-row coefficient.  Replaces the `group` op
 * (SMT/ops.py:98-130, kernel SMT/kernels.py:243-298):
 * out[n, :] = A[idx[n] / fan_out, :] * coeff[idx[n]] for n in [0, M).  coeff may be NULL. */
int b200moe_group(const void* A, int64_t lda, const int64_t* idx, void* out, int64_t ldo,
                  const void* coeff, int fan_out, int64_t M, int K, int dtype, b200moe_stream_t stream);

/* out[t, :] = sum_j gates[t, j] * in[t*k + j, :] (gates NULL: plain sum), fp32 accumulation in slot order.
 * Replaces `torch.bmm(gates.unsqueeze(1), output_expanded)` (SMT/ops.py:160-164) and
 * `d_expanded_input.view(T, k, -1).sum(-2)` (SMT/ops.py:258-261). */
int b200moe_combine(const void* in, int64_t ldi, const void* gates, void* out, int64_t ldo, int64_t T,
                    int k, int H, int dtype, b200moe_stream_t stream);

/* y[:, :h] = x[:, :h] * silu(x[:, h:]) on a (rows, 2h) tensor, and its gradient.  Replaces
 * swiglu_unchunked forward / backward
 * (cute_kernels/kernels/swiglu_unchunked/triton_implementation/kernels_forward.py:13-38,
 *  kernels_backward.py:13-48). */
int b200moe_swiglu_unchunked_forward(const void* x, int64_t ldx, void* y, int64_t ldy, int64_t rows, int h,
                                     int dtype, b200moe_stream_t stream);
int b200moe_swiglu_unchunked_backward(const void* x, int64_t ldx, const void* dy, int64_t lddy, void* dx,
                                      int64_t lddx, int64_t rows, int h, int dtype,
                                      b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * The fused layer path (padded grouped order inside; weights as the module stores them)
 * w_fc: (E, 2I, H) contiguous, w_proj: (E, H, I) contiguous
 * (cute_kernels/kernels/scattermoe/torch_implementation.py:16).  expert_offsets, row_token, row_slot
 * come from b200moe_route.  m_cap = rows of the padded grouped buffers.
 * ------------------------------------------------------------------------------------------------ */

/* Rows of a (T, width) tensor copied into the padded grouped order: out[p, :] = src[row_map[p], :], zeros where
 * row_map[p] < 0; out has `rows` rows (the padded row count).  Replaces the `group` calls that materialise the
 * grouped input and the grouped upstream gradient (SMT/ops.py:213-233); the GEMM kernels then read the result
 * with TMA.  The kernels below also accept row_token themselves (gather fused into the operand load); the
 * layer path pre-gathers because one 16-byte-per-thread HBM pass is cheaper than a gathered operand load. */
int b200moe_gather_rows(const void* src, int64_t lds, const int32_t* row_map, void* out, int64_t ldo, int64_t rows,
                        int width, int dtype, b200moe_stream_t stream);

/* Gated activations the fused expert kernels apply between the two projections: a = h[:, :I] * m(h[:, I:]).
 * SWIGLU: m = silu (cute_kernels/kernels/swiglu_unchunked/torch_implementation.py:5-7); GLU: m = sigmoid (torch.nn.GLU,
 * the activation of the reference's MoE test, tests/test_commons.py:86-87). */
#define B200MOE_ACT_SWIGLU 0
#define B200MOE_ACT_GLU 1

/* Up projection with the token gather on the input rows and the gated activation in the epilogue:
 * h[p, :] = x[row_token[p], :] @ w_fc[e(p)]^T  (Mcap, 2I), a[p, :] = h[p, :I] * m(h[p, I:])  (Mcap, I).
 * row_token == NULL: x already holds the padded grouped rows (m_cap rows, see b200moe_gather_rows).
 * Replaces scatter2scatter for c_fc plus the activation call (SMT/__init__.py:83-91). */
int b200moe_up_forward(const void* x, int64_t ldx, const void* w_fc, const int64_t* expert_offsets,
                       const int32_t* row_token, void* h, void* a, int64_t T, int H, int I, int E,
                       int64_t m_cap, int activation, int dtype, int32_t* status, b200moe_stream_t stream);

/* Down projection scattered back to (token, slot) order and scaled by the gate of that slot:
 * y_expanded[s, :] = gates[s] * (a[p, :] @ w_proj[e(p)]^T), s = row_slot[p]; gates NULL means 1.
 * Replaces scatter2scatter for c_proj (SMT/__init__.py:92-100); b200moe_combine(gates = NULL) then gives
 * the layer output that SMT/ops.py:160-164 forms with bmm. */
int b200moe_down_forward(const void* a, const void* w_proj, const int64_t* expert_offsets,
                         const int32_t* row_slot, const void* gates, void* y_expanded, int64_t ldy,
                         int64_t M, int H, int I, int E, int64_t m_cap, int dtype, int32_t* status,
                         b200moe_stream_t stream);

/* Input gradient of the down projection fused with the gate scaling, the backward of the gated activation
 * (`activation` as in b200moe_up_forward) and the gate gradient.
 * With u[p, :] = grad_out[row_token[p], :] @ w_proj[e(p)] (Mcap, I), act = h[:, :I]*m(h[:, I:]),
 * g = gates[row_slot[p]]:
 *   d_gates[row_slot[p]] = <act[p, :], u[p, :]>          (fp32, M entries, overwritten)
 *   dh[p, :] = activation backward of h[p, :] for upstream g*u[p, :]   (Mcap, 2I)
 *   ag[p, :] = g * act[p, :]                                        (Mcap, I)
 * row_token == NULL: grad_out already holds the padded grouped rows (m_cap rows).
 * Replaces, for c_proj: the d_gates bmm, group(coeff=gates), scatter2scatter (SMT/ops.py:204-256) and the
 * activation backward between the two projections
 * (cute_kernels/kernels/swiglu_unchunked/triton_implementation/kernels_backward.py:13-48). */
int b200moe_down_dgrad(const void* grad_out, int64_t ldg, const void* w_proj, const int64_t* expert_offsets,
                       const int32_t* row_token, const int32_t* row_slot, const void* gates, const void* h,
                       void* dh, void* ag, float* d_gates, int64_t M, int H, int I, int E, int64_t m_cap,
                       int activation, int dtype, int32_t* status, b200moe_stream_t stream);

/* Weight gradient of one projection, written in the layout the module stores weights in:
 * DW[e, o, i] = sum over rows p of expert e of P[pmap(p), o] * Q[qmap(p), i], DW (E, n_out, n_in) contiguous.
 * P, Q are row-major with row strides ldp, ldq; p_map / q_map (device int32 over padded grouped rows, or
 * NULL for the identity) turn a padded grouped row into a row of P / Q, negative meaning a zero row.
 * Replaces group (of x or of grad_out), zeros_like and group_bwd_W (SMT/ops.py:213-245). */
int b200moe_wgrad(const void* P, int64_t ldp, const int32_t* p_map, const void* Q, int64_t ldq,
                  const int32_t* q_map, const int64_t* expert_offsets, void* DW, int n_out, int n_in, int E,
                  int64_t m_cap, int dtype, int32_t* status, b200moe_stream_t stream);

/* Input gradient of the up projection scattered to (token, slot) order:
 * dx_expanded[row_slot[p], :] = dh[p, :] @ w_fc[e(p)]   (M, H); b200moe_combine then sums over the slots.
 * Replaces scatter2scatter in the c_fc backward and the sum over k (SMT/ops.py:247-261). */
int b200moe_up_dgrad(const void* dh, const void* w_fc, const int64_t* expert_offsets, const int32_t* row_slot,
                     void* dx_expanded, int64_t ldd, int64_t M, int H, int I, int E, int64_t m_cap, int dtype,
                     int32_t* status, b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Expert-parallel row exchange over peer memory (no counterpart in the reference, which has no collective).
 * peer_ptrs is a HOST array of R device pointers: entry d is rank d's exchange buffer (cap_rows x width), mapped
 * into this process (CUDA IPC / symmetric memory).  start (R+1) and base (R) are device int32 arrays: the rows
 * of this rank's expert-sorted order bound for rank d are [start[d], start[d+1]) and land in d's buffer from row
 * base[d] on.  The caller orders the ranks (buffers free before, data complete after) around each call.
 * ------------------------------------------------------------------------------------------------ */

/* Token dispatch: peer d's buffer row base[d] + n - start[d] = src[idx[n] / fan_out, :] * coeff[idx[n]]
 * (idx NULL: n itself; coeff NULL: 1) for n in [0, M).  Fuses the dispatch gather (SMT/ops.py:227-233 applied to the
 * send side) with the transfer.  Rows that would fall outside cap_rows set status word 301 and are skipped. */
int b200moe_ep_push_rows(const void* src, int64_t lds, const int64_t* idx, int fan_out, const void* coeff,
                         const void* const* peer_ptrs, const int32_t* start, const int32_t* base, int R, int64_t M,
                         int width, int64_t cap_rows, int dtype, int32_t* status, b200moe_stream_t stream);

/* Return path: out[t, :] = sum_j gates[t, j] * row(inv[t*k + j]) read straight from the owning peer's buffer, where
 * row(n) sits at base[d] + n - start[d] of rank d's buffer; expanded (T*k x width, may be NULL) receives the
 * unweighted rows.  Fuses the transfer with the un-sort and the gate-weighted combine (SMT/ops.py:160-164). */
int b200moe_ep_pull_combine(const void* const* peer_ptrs, const int64_t* inv, const int32_t* start,
                            const int32_t* base, int R, const void* gates, void* out, int64_t ldo, void* expanded,
                            int64_t T, int k, int width, int dtype, b200moe_stream_t stream);

/* Gate gradient of the return path: d_gates[t, j] = <expanded[t*k + j, :], grad[t, :]> (fp32 accumulation, stored in the
 * tensor type), expanded (T*k x width) being the unweighted rows b200moe_ep_pull_combine kept.  Replaces the bmm of
 * SMT/ops.py:204 on the rank that owns the tokens. */
int b200moe_ep_gate_grad(const void* expanded, int64_t lde, const void* grad, int64_t ldg, void* d_gates, int64_t T, int k,
                         int width, int dtype, b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Fused router (the step before the path): replaces `_compute_routing_weights` + `_get_topk`
 * (cute_kernels/kernels/scattermoe/torch_implementation.py:120-133,193-199) and the histogram of the selected experts
 * (cute_kernels/kernels/contiguous_count/__init__.py:8-24) for 16-bit tensors.
 *   logits (T, E)  = x (T, H) @ gate_w (E, H)^T, fp32 accumulation on the tensor cores, rounded to the tensor type
 *   indices (T, k) = the k largest logits of each row, descending; equal logits: lower expert first (int64)
 *   weights (T, k) = scoring 0: softmax over the k selected logits; scoring 1: their sigmoids divided by their sum;
 *                    computed in fp32 from the rounded logits, stored in the tensor type
 *   counts (E)     = number of (token, slot) pairs per expert (int32; zeroed by the call)
 * Limits: E <= 256, k <= 8, bf16 / fp16.  One launch (plus the memset of counts).
 * ------------------------------------------------------------------------------------------------ */
int b200moe_router_forward(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, int64_t T, int H, int E, int k,
                           int scoring, void* logits, int64_t ldl, void* weights, int64_t* indices, int32_t* counts,
                           int dtype, int32_t* status, b200moe_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * RMSNorm (the normalisation feeding the layer's input in a transformer block): replaces `rmsnorm_cute`
 * (cute_kernels/kernels/rmsnorm/__init__.py:11-112, forward.py, backward.py and the Triton kernels under
 * triton_implementation/) whose eager definition is F.rms_norm (torch_implementation.py:5-6).
 *   y[r, :]  = x[r, :] * rstd[r] * weight,  rstd[r] = 1 / sqrt(mean(x[r, :]^2) + eps);  weight may be NULL
 *   dx[r, :] = rstd * (dy * weight) - x * rstd^3 * mean((dy * weight) * x);  dweight = sum_r dy * x * rstd
 * Arithmetic in fp32, tensors bf16 / fp16 / fp32, unit inner stride.  rstd (fp32, one per row) is optional in both
 * calls: forward stores it when given; backward recomputes it from x when NULL (the reference's memory_efficient
 * mode).  dweight may be NULL; otherwise `workspace` must hold b200moe_rmsnorm_workspace_bytes(rows, H, dtype) bytes
 * (fp32 partial sums, added up in a fixed order on the 16-byte aligned path).
 * ------------------------------------------------------------------------------------------------ */
int64_t b200moe_rmsnorm_workspace_bytes(int64_t rows, int H, int dtype);
int b200moe_rmsnorm_forward(const void* x, int64_t ldx, const void* weight, void* y, int64_t ldy, float* rstd,
                            int64_t rows, int H, float eps, int dtype, b200moe_stream_t stream);
int b200moe_rmsnorm_backward(const void* x, int64_t ldx, const void* weight, const void* dy, int64_t lddy,
                             const float* rstd, void* dx, int64_t lddx, void* dweight, void* workspace,
                             int64_t workspace_bytes, int64_t rows, int H, float eps, int dtype,
                             b200moe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H */
