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

/* Options (b200moe_set_option).  Process-wide, meant for measurements and tests; the defaults are the product path. */
#define B200MOE_OPT_DYNAMIC_TILES 1 /* two-CTA kernels, how a cluster gets its tiles: 0 = fixed stride; 1 = the weight-gradient
                                     * launches draw them from a per-launch counter, in list order (longest reduction
                                     * first); 2 (default) = those, and row launches whose reduction extent is >= 4096;
                                     * 3 = every launch */
#define B200MOE_OPT_TILE_VARIANT 2  /* -1 (default): the per-shape tile table decides; otherwise a B200MOE_TILE_* value
                                     * forced on every tensor-core launch whose operands allow it */
#define B200MOE_OPT_TILE_ORDER 3    /* row GEMMs, order of an expert's tiles: -1 (default) = by the size of the expert's weight
                                     * matrix; 1 = the column blocks of a row tile first; 0 = the row tiles of a column
                                     * block first; 2 = blocks of 8 x 8 tiles (two-CTA kernel) */
#define B200MOE_OPT_SM_LIMIT 4      /* 0 (default) = the tensor-core GEMM launches use every SM; n > 0 = at most n SMs, which
                                     * leaves the others to kernels queued on other streams (the expert-parallel
                                     * transfers: a persistent GEMM grid otherwise holds every SM until it ends) */
#define B200MOE_OPT_COUNT 5

/* Tiles of the tensor-core engine and the operations the tile table is keyed on (b200moe_tile_table_lookup).  The table
 * plays the part of the reference's autotuner configurations, which are keyed on the same quantities
 * (SMT/kernels.py:8-11,152-159: N, K), reduced to fixed entries measured on a B200. */
#define B200MOE_TILE_PAIR_256x256 0 /* cluster of two CTAs, tcgen05.mma.cta_group::2, 256 x 256 x 64, six stages */
#define B200MOE_TILE_CTA_128x256 1  /* one CTA, 128 x 256 x 64, four stages */
#define B200MOE_TILE_COUNT 2
#define B200MOE_OP_UP_FORWARD 0  /* gathered rows @ w_fc^T with the gated activation in the epilogue */
#define B200MOE_OP_ROW_STORE 1   /* row GEMM with a plain / scattered store epilogue (down forward, up dgrad) */
#define B200MOE_OP_DOWN_DGRAD 2  /* row GEMM with the activation backward in the epilogue */
#define B200MOE_OP_WGRAD 3       /* per-expert weight gradient (reduction over the expert's rows) */
#define B200MOE_OP_COUNT 4

typedef void* b200moe_stream_t; /* cudaStream_t */

int b200moe_version(void);
const char* b200moe_error_string(int code);
/* Text describing the last failing call on this host thread (empty if none). */
const char* b200moe_last_error_detail(void);
/* Process-wide engine choice; returns the previous value. */
int b200moe_set_engine(int engine);
/* Sets a B200MOE_OPT_* option; returns B200MOE_OK or B200MOE_ERR_ARG.  b200moe_get_option reads one back. */
int b200moe_set_option(int option, int value);
int b200moe_get_option(int option);
/* The tile (B200MOE_TILE_*) the table assigns to operation `op` (B200MOE_OP_*) with reduction extent K (weight
 * gradients: output rows), N output columns and about rows_per_expert rows per expert. */
int b200moe_tile_table_lookup(int op, int K, int N, int64_t rows_per_expert);
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
 *   expert_ids             device int64 (M), values in [0, E); a NEGATIVE value marks a slot that goes to no expert
 *                          (a padding token, a slot dropped by a capacity limit): it is counted nowhere and appears
 *                          in none of the outputs; a value >= E sets status word 101 and is left out as well
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

/* The same sum reading its rows through an index: out[t, :] = sum_j gates[t, j] * in[pos[t*k + j], :] (a negative
 * index contributes nothing).  With pos = the padded grouped row of every slot (b200moe_invert_row_map) it forms the
 * layer output / the input gradient straight from the grouped-order results of b200moe_down_forward / b200moe_up_dgrad,
 * i.e. the un-sort of SMT/kernels.py:97-102 moves from the GEMM epilogue into this pass.  k <= 32. */
int b200moe_combine_rows(const void* in, int64_t ldi, const int32_t* pos, const void* gates, void* out, int64_t ldo,
                         int64_t T, int k, int H, int dtype, b200moe_stream_t stream);

/* slot_row[row_slot[p]] = p for every real row p of the padded grouped order (row_slot from b200moe_route; `rows`
 * entries, M slots).  No counterpart in the reference, whose kernels scatter through sorted_scattered_idxs. */
int b200moe_invert_row_map(const int32_t* row_slot, int64_t rows, int32_t* slot_row, int64_t M, b200moe_stream_t stream);

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
/* Un-gated activation of a non-GLU expert layer: a = gelu_tanh(h), h = x @ w_fc^T with w_fc (E, I, H) (torch.nn.GELU(
 * approximate="tanh"), the activation of the reference's non-GLU MoE test, tests/test_commons.py:86-87).  With this code
 * every "2I" below reads "I": h and dh are (Mcap, I), and b200moe_up_dgrad is called with I / 2 in place of I so that
 * its reduction extent 2 * (I / 2) is the layer's I. */
#define B200MOE_ACT_GELU_TANH 2

/* Up projection with the token gather on the input rows and the gated activation in the epilogue:
 * h[p, :] = x[row_token[p], :] @ w_fc[e(p)]^T  (Mcap, 2I), a[p, :] = h[p, :I] * m(h[p, I:])  (Mcap, I).
 * h is kept for b200moe_down_dgrad only; what it holds and in which column order is the engine's own business (see there).
 * row_token == NULL: x already holds the padded grouped rows (m_cap rows, see b200moe_gather_rows).
 * Replaces scatter2scatter for c_fc plus the activation call (SMT/__init__.py:83-91). */
int b200moe_up_forward(const void* x, int64_t ldx, const void* w_fc, const int64_t* expert_offsets,
                       const int32_t* row_token, void* h, void* a, int64_t T, int H, int I, int E,
                       int64_t m_cap, int activation, int dtype, int32_t* status, b200moe_stream_t stream);

/* Down projection, optionally scattered back to (token, slot) order and scaled by the gate of that slot:
 * y_expanded[s, :] = gates[s] * (a[p, :] @ w_proj[e(p)]^T), s = row_slot[p]; gates NULL means 1.
 * row_slot == NULL (gates NULL too): the rows stay in the padded grouped order, y_expanded[p, :] for all m_cap rows
 * (zeros on filler rows), written by TMA; b200moe_combine_rows then un-sorts while it sums.
 * Replaces scatter2scatter for c_proj (SMT/__init__.py:92-100).  The layer passes gates = NULL, keeps the unweighted
 * rows for the gate gradient as the reference does (SMT/ops.py:163,173) and forms the output with
 * b200moe_combine(gates), which is the bmm of SMT/ops.py:160-164. */
int b200moe_down_forward(const void* a, const void* w_proj, const int64_t* expert_offsets,
                         const int32_t* row_slot, const void* gates, void* y_expanded, int64_t ldy,
                         int64_t M, int H, int I, int E, int64_t m_cap, int dtype, int32_t* status,
                         b200moe_stream_t stream);

/* Upstream gradient rows of the backward pass in the padded grouped order, scaled by the gate of their slot, and
 * the gate gradient, in one pass over grad_out:
 *   out[p, :]  = gates[s] * grad_out[t, :]  with s = row_slot[p], t = row_token[p]; zeros on filler rows; gates NULL: 1
 *   d_gates[s] = <y_expanded[s, :], grad_out[t, :]>   fp32 (M entries); y_expanded (the unweighted expert outputs the
 *                forward kept: M x width in (token, slot) order, or with y_grouped != 0 rows x width in the padded
 *                grouped order, row p then belongs to slot row_slot[p]) and d_gates are given together or both NULL
 * Replaces `group(grad_out, coeff=gates)` and the d_gates bmm of the c_proj backward (SMT/ops.py:200-222).  Every
 * dot product is summed in a fixed order, so the gate gradient is reproducible from run to run. */
int b200moe_gather_grad_rows(const void* grad_out, int64_t ldg, const int32_t* row_token, const int32_t* row_slot,
                             const void* gates, const void* y_expanded, int64_t ldy, int y_grouped, void* out,
                             int64_t ldo, float* d_gates, int64_t rows, int width, int dtype, b200moe_stream_t stream);

/* Input gradient of the down projection fused with the backward of the gated activation (`activation` as in
 * b200moe_up_forward).  grad_rows holds the gate-scaled upstream gradient rows in the padded grouped order (m_cap
 * rows, from b200moe_gather_grad_rows); with row_token given it holds T token rows instead and the kernel gathers
 * them (no gate scaling then).  With d[p, :] = grad_rows[p, :] @ w_proj[e(p)] rounded to the tensor type (Mcap, I):
 *   dh[p, :] = activation backward of h[p, :] for upstream d[p, :]   (Mcap, 2I), plain (up | gate) column order
 * h is the buffer b200moe_up_forward wrote IN THE SAME ENGINE; treat it as opaque between the two calls.  The CUDA-core
 * engine keeps the pre-activation (up | gate) there; the tensor-core engine keeps, interleaved per 32-column chunk, the
 * two factors of the activation's derivative (m(gate) and up * m'(gate), resp. gelu_tanh'(h)), computed in its forward
 * epilogue from h rounded to the tensor type, so that this kernel's epilogue is two multiplications per element.
 * Replaces scatter2scatter of the c_proj backward (SMT/ops.py:247-256) and the activation backward between the two
 * projections (cute_kernels/kernels/swiglu_unchunked/triton_implementation/kernels_backward.py:13-48). */
int b200moe_down_dgrad(const void* grad_rows, int64_t ldg, const void* w_proj, const int64_t* expert_offsets,
                       const int32_t* row_token, const void* h, void* dh, int64_t T, int H, int I, int E,
                       int64_t m_cap, int activation, int dtype, int32_t* status, b200moe_stream_t stream);

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
 * row_slot == NULL: dx_expanded[p, :] in the padded grouped order (m_cap rows), for b200moe_combine_rows.
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

/* The same two transfers with the destination row of every routed row given explicitly: dest_pos (device int32, M
 * entries, indexed like start's rows) is the row of the owning rank's buffer.  With dest_pos = the row's position in the
 * RECEIVER's padded grouped order (every rank can compute it from the all-gathered expert counts), dispatched rows land
 * where the receiver's expert GEMMs read them and results are fetched from where its GEMM epilogues stored them: the
 * receiver runs no sort and no gather pass of its own.  base may be NULL when dest_pos is given.  cap_rows (> 0): rows of a
 * peer buffer; a row whose place lies beyond it was never stored by the dispatch (status 301) and is read as zeros.
 * max_blocks (> 0) caps the grid of the transfer: at one block per SM (the kernels use 192 threads x 40 registers and no
 * shared memory) a transfer launched beside persistent GEMM kernels leaves room for their CTAs on every SM. */
int b200moe_ep_push_rows_at(const void* src, int64_t lds, const int64_t* idx, int fan_out, const void* coeff,
                            const void* const* peer_ptrs, const int32_t* start, const int32_t* base, const int32_t* dest_pos,
                            int R, int64_t M, int width, int64_t cap_rows, int max_blocks, int dtype, int32_t* status,
                            b200moe_stream_t stream);
int b200moe_ep_pull_combine_at(const void* const* peer_ptrs, const int64_t* inv, const int32_t* start, const int32_t* base,
                               const int32_t* dest_pos, int R, int64_t cap_rows, int max_blocks, const void* gates, void* out,
                               int64_t ldo, void* expanded, int64_t T, int k, int width, int dtype, b200moe_stream_t stream);

/* Clears the rows of a padded grouped buffer that belong to no routed row (between the end of an expert's rows and the
 * next multiple of 128): needed where the rows were written by other ranks, which only send real rows.
 * expert_offsets: device int64 (E), inclusive. */
int b200moe_zero_filler_rows(void* buf, int64_t ld, const int64_t* expert_offsets, int E, int width, int64_t cap_rows, int dtype,
                             b200moe_stream_t stream);

/* Placement plan of the direct exchange: everything a rank derives from the all-gathered expert counts of a pass, in one
 * launch.  counts_all: device int32 (R * E), entry s * E + e = rows that rank s routes to expert slot e (rank r owns the
 * slots [r * E / R, (r + 1) * E / R)).  sorted_scattered_idxs: this rank's M routed rows in expert order (b200moe_route).
 * Outputs (device): start (R + 1) and base (R) as b200moe_ep_push_rows takes them; dest_pos (M): the row every sorted row
 * occupies in its owner's padded grouped order (segments of ceil128(rows of the expert over all sources), sources in rank
 * order inside a segment); local_offsets (E / R, int64): inclusive offsets of this rank's experts over everything it
 * receives; summary (2, int64): rows this rank receives, and the most padded rows any rank's buffers must hold (the same
 * on every rank: the collective overflow decision); inverse (M, int64): inverse[sorted_scattered_idxs[i]] = i.
 * R * E <= 4096.  No counterpart in the reference (it has no multi-GPU path). */
int b200moe_ep_plan(const int32_t* counts_all, const int64_t* sorted_scattered_idxs, int R, int rank, int E, int64_t M,
                    int32_t* start, int32_t* base, int32_t* dest_pos, int64_t* local_offsets, int64_t* summary, int64_t* inverse,
                    b200moe_stream_t stream);

/* Rank barrier on the stream, over a symmetric flag array: flag_ptrs is a HOST array of R device pointers, entry d being
 * rank d's array of R int32 words (zero before the first barrier), mapped into this process.  `epoch` is the number of
 * this barrier (1, 2, 3, ... the same on every rank).  The kernel publishes the epoch to every peer and waits, for at most
 * limit_cycles SM cycles, until every peer has published it; when a peer does not arrive it writes 302 to the status word
 * and returns (b200moe_check_status then reports B200MOE_ERR_DEVICE), it never traps.  R <= 64. */
int b200moe_ep_barrier(const void* const* flag_ptrs, int rank, int R, int epoch, int64_t limit_cycles, int32_t* status,
                       b200moe_stream_t stream);

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
/* The same router with a per-row factor on the logits: logits[t, :] = row_scale[t] * (x[t, :] @ gate_w^T), rounded after
 * the scaling.  With x the un-normalised hidden states, row_scale = the rstd of b200moe_rmsnorm_forward and gate_w the
 * gate weight multiplied column-wise by the norm weight, these are the logits of the RMSNorm that feeds the layer
 * (cute_kernels/kernels/rmsnorm/triton_implementation/kernels_forward.py:19-60 followed by
 * cute_kernels/kernels/scattermoe/torch_implementation.py:120-122): the normalisation is folded into the gate
 * projection instead of being read back from memory.  row_scale: device fp32 (T), NULL = 1. */
int b200moe_router_forward_scaled(const void* x, int64_t ldx, const void* gate_w, int64_t ldw, const float* row_scale, int64_t T,
                                  int H, int E, int k, int scoring, void* logits, int64_t ldl, void* weights, int64_t* indices,
                                  int32_t* counts, int dtype, int32_t* status, b200moe_stream_t stream);

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
