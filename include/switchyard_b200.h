/* switchyard_b200 — C ABI of the sm_100a mixture-of-experts kernels.
 *
 * Every entry point takes raw device pointers, sizes, a 16-bit element type and a CUDA
 * stream (passed as void*; it is a cudaStream_t). Nothing here allocates, frees, synchronises
 * the device or takes ownership: outputs and scratch are the caller's, inputs are borrowed
 * until the enqueued work has run. Calls are asynchronous on `stream`, on the CURRENT device,
 * and may be made concurrently from several host threads (one per device).
 *
 * Return value: SY_OK (0) or a negative SY_ERR_* code; sy_last_error() gives the message of
 * the calling thread's last failure.
 *
 * Each declaration names the entry point of the reference project's extension that it
 * replaces (file:line in the reference's tree, switchyard/csrc/moe_kernels.cu).
 */
#ifndef SWITCHYARD_B200_H
#define SWITCHYARD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SY_OK 0
#define SY_ERR_ARGUMENT (-1) /* a shape, alignment or limit check failed; nothing was enqueued */
#define SY_ERR_CUDA (-2)     /* a CUDA runtime / driver call failed */
#define SY_ERR_DEVICE (-3)   /* a kernel gave up on a bounded wait (see sy_device_status) */

#define SY_DTYPE_F16 0
#define SY_DTYPE_BF16 1

/* Message of the calling thread's last failing call ("" if none). Never NULL. */
const char* sy_last_error(void);

/* Library version string. */
const char* sy_version(void);

/* Blocks until `stream` is idle, then reads the current device's kernel status word into
 * *status_out and clears it: 0, or the code of the last bounded wait that gave up (1-4: a wait
 * inside the expert kernel's pipeline, 5: a flag, 6: an index outside its array was skipped).
 * Returns SY_OK when the word is 0 and SY_ERR_DEVICE otherwise: the results of the kernels that
 * ran since the last call are then not to be trusted. The stream stays usable. Cheap enough
 * for the end of a request or a decode step; not meant for every layer. */
int sy_device_status(void* stream, int* status_out);

/* How long a kernel waits for a flag, a barrier or another block before it gives up, records
 * a status code and lets the stream go on. One value for the whole process, used by launches
 * made after the call. Default 2 s, or SY_WAIT_LIMIT_MS from the environment (read once).
 * 1 us <= limit_ns <= 60 s. No counterpart in the reference (its waits are stream events). */
int sy_set_wait_limit_ns(uint64_t limit_ns);
uint64_t sy_wait_limit_ns(void);

/* route — replaces `route` (moe_kernels.cu:73-89, kernel l.23-71).
 * logits [n_tokens, n_experts] row-major, 16-bit. One warp per token: float32 softmax,
 * top_k rounds of arg-max with ties to the lower expert index, optional renormalisation.
 * idx_out int32 [n_tokens, top_k] (descending probability), w_out 16-bit [n_tokens, top_k].
 * Limits: n_experts <= 128, top_k <= 8, top_k <= n_experts. n_tokens == 0 is a no-op. */
int sy_route(const void* logits, int n_tokens, int n_experts, int top_k, int norm_topk_prob, int dtype,
             int32_t* idx_out, void* w_out, void* stream);

/* Scratch bytes sy_sort_by_expert needs for m choices (0 when one block sorts everything). */
size_t sy_sort_scratch_bytes(int m, int n_experts);

/* sort_by_expert — replaces `sort_by_expert` (moe_kernels.cu:142-157, kernels l.94-139 and the
 * torch cumsum between them). Stable counting sort of the flat choice list (i = token*top_k +
 * slot) by expert id, no atomics, same result every run.
 * idx int32 [m] (m = n_tokens*top_k, values in [0, n_experts)), w 16-bit [m].
 * Outputs: counts int32 [n_experts]; offsets int32 [n_experts+1] (exclusive prefix);
 * token int32 [m] (= i / top_k of the choice in that sorted row); wsorted 16-bit [m];
 * pos_of int32 [m] (sorted row of choice i). m == 0 zero-fills counts and offsets.
 * scratch: sy_sort_scratch_bytes(m, n_experts) bytes of device memory (may be NULL if 0).
 * Limit: n_experts <= 256. */
int sy_sort_by_expert(const int32_t* idx, const void* w, int m, int top_k, int n_experts, int dtype,
                      int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                      void* scratch, size_t scratch_bytes, void* stream);

/* route_sort — sy_route followed by sy_sort_by_expert in ONE launch, for decode-sized batches
 * (n_tokens * top_k <= sy_route_sort_max_choices() = 8192, n_experts <= 128): blocks of sixteen
 * tokens route a token per warp, and the block that finishes last sorts all choices. Outputs are
 * those of the two separate calls, bit for bit (moe_kernels.cu:73-89 and 142-157 in one step).
 * ticket: one zero-initialised int32 of device memory, left at zero (may be NULL up to sixteen
 * tokens); launches that share it must not overlap. */
int sy_route_sort_max_choices(void);
int sy_route_sort(const void* logits, int n_tokens, int n_experts, int top_k, int norm_topk_prob, int dtype,
                  int32_t* idx, void* w, int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted,
                  int32_t* pos_of, int32_t* ticket, void* stream);

/* route_fused — router GEMM, sy_route and sy_sort_by_expert in ONE launch for decode-sized
 * batches: replaces `F.linear(h, router)` followed by `route` (switchyard/kernels.py:30-32,
 * moe_kernels.cu:73-89) and `sort_by_expert` (l.142-157).
 * h 16-bit [n_tokens, hidden]; router 16-bit [n_experts, hidden]; bias 16-bit [n_experts] or
 * NULL (added to the rounded logits in the 16-bit type, as a tensor add would).
 * logits = round16(h . router^T) with float32 accumulation in a fixed order that depends only on
 * the token's own row; they are written to logits_out [n_tokens, n_experts] when it is not NULL.
 * The routing is exactly sy_route applied to those logits and the sort exactly
 * sy_sort_by_expert, so the outputs equal the separate calls fed with logits_out. The logits
 * themselves may differ from a library GEMM's in the last bit (another summation order).
 * ticket: one zero-initialised int32 of device memory, left at zero; launches that share it
 * must not overlap. Limits: n_tokens * top_k <= 8192, n_experts a multiple of 8 up to 128,
 * hidden a multiple of 32, top_k <= 8. */
int sy_route_fused_max_tokens(void);
int sy_route_fused(const void* h, const void* router, const void* bias, int n_tokens, int n_experts, int hidden,
                   int top_k, int norm_topk_prob, int dtype, void* logits_out, int32_t* idx, void* w,
                   int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                   int32_t* ticket, void* stream);

/* sort_by_expert_static — no counterpart in the reference. The same sort, same outputs bit for
 * bit, for callers that are not allowed to allocate device memory while they run and so
 * cannot provide scratch: a server that has handed all free HBM to its own arena (cudaMalloc
 * would fail), a plugin whose host forbids allocation on the request path. The table of
 * per-block expert counts is a 128 KiB array inside the library image, present on every GPU
 * that loads the library until the process exits. This entry point calls no cudaMalloc,
 * cudaFree or other allocating routine.
 *   - At most 1 048 576 choices (m) per call and 256 experts; more is rejected with
 *     SY_ERR_ARGUMENT (use sy_sort_by_expert with your own scratch).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current): make that first call outside any
 *     stream capture.
 *   - All calls on a device share the one array. It needs no clearing between calls (every
 *     entry read is written earlier in the same call), but two calls with m > 8192 that overlap
 *     on the GPU (different streams) race on it: keep them on one stream or serialise them.
 *     Calls with m <= 8192 sort in one block and do not touch the array. */
int sy_sort_by_expert_static(const int32_t* idx, const void* w, int m, int top_k, int n_experts, int dtype,
                             int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                             void* stream);

/* grouped_gemv — replaces `grouped_gemv` (moe_kernels.cu:385-415, kernel l.306-383): the decode
 * path, for batches with few rows per expert, where the layer is bound by reading weights.
 * For every sorted row r of expert e (offsets[e] <= r < offsets[e+1]):
 *   C[r, :] = A[src(r), :] . B[e]^T,  src(r) = a_rows ? a_rows[r] : r
 * A 16-bit [*, k_dim]; B 16-bit [n_experts, n_full, k_dim] (nn.Linear layout per expert),
 * n_full = swiglu ? 2*n_out (gate rows first, then up rows) : n_out; C 16-bit [rows, n_out].
 * swiglu: C = silu(gate) * up with 16-bit rounding after each step; scale (16-bit [rows], may
 * be NULL, not with swiglu): C = round16(acc) * scale[r]. float32 accumulation in a fixed
 * order per row: a row's bits do not depend on which other rows share its expert.
 * A persistent weight stream: experts without rows are skipped, weight tiles (128 rows x 128 k,
 * with swiglu 64 gate + 64 up rows) come in by TMA through a four-stage shared-memory ring,
 * the dot products run on tcgen05 with the token rows as the N operand (N = rows rounded up
 * to 16, at most 64 per tile), accumulators in tensor memory. Any row count is accepted.
 * Requirements: k_dim % 8 == 0, n_out % 8 == 0, 16-byte aligned A, B; n_experts <= 256. */
int sy_grouped_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                    int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                    int dtype, void* stream);

/* grouped_gemm — replaces `grouped_gemm` (moe_kernels.cu:264-298, kernel l.159-261) and the
 * host-side `tile_offsets` / `total_tiles` arguments, which this implementation does not need:
 * tiles are scheduled on the device from `offsets`. Same contract as sy_grouped_gemv; the same
 * kernel in its compute-bound shape: 128 token rows (the MMA's M operand) against 256 weight
 * rows (with swiglu 128 gate + 128 up rows of the same columns) per tile, one accumulator of
 * 256 tensor-memory columns, epilogues fused. With a_rows == NULL the token rows of a tile are
 * contiguous in A and arrive as TMA boxes; with a_rows they are gathered in-kernel with 16-byte
 * copies, which is about 30 % slower at large batches: sort the rows first (sy_gather_rows) when
 * the batch is compute-bound. A then needs at least `rows` rows.
 * The bits of the two modes (gemv / gemm) may differ from each other, as in the reference. */
int sy_grouped_gemm(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                    int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                    int dtype, void* stream);

/* The compute shape has two tiles with identical results: one CTA per 128-row tile, or a CTA
 * pair (tcgen05 cta_group::2) per 256-row tile, chosen per launch from the mean rows per expert
 * (pairs from 768). This overrides the choice for plain sorted batches, for the whole process:
 * 0 = automatic, 1 = one CTA, 2 = pairs. SY_GEMM_TILE=single|pair in the environment (read once,
 * at the first launch) sets the initial value. No counterpart in the reference. */
int sy_force_compute_tile(int tile);

/* expert_ffn — the whole expert FFN of a layer in ONE launch: gate/up projection with SwiGLU
 * into `act`, then the down projection scaled by the router weights into `y`, i.e. what the
 * reference does with two grouped_gemv / grouped_gemm calls (switchyard/kernels.py:56-63). A down
 * tile of an expert starts as soon as that expert's gate/up tiles have been stored (a counter
 * per expert in `scratch`, bounded wait), so the second projection fills the SMs that the first
 * one's last tiles leave idle, and there is no launch gap between them. Arithmetic per row is
 * that of the two separate calls, bit for bit.
 * Rows come as ranges like sy_grouped_segments: range g = rows [begins[g], ends[g]); expert e owns
 * ranges [e*ranges_per_expert, (e+1)*ranges_per_expert). For the plain single-GPU layer pass
 * begins = offsets, ends = offsets + 1, n_ranges = experts, ranges_per_expert = 1.
 * x 16-bit [*, hidden] (row i of a range is x[a_rows ? a_rows[i] : i]); gate_up [experts, 2*inter,
 * hidden]; down [experts, hidden, inter]; wsorted 16-bit router weight per row; act 16-bit
 * [rows_bound, inter] scratch; y 16-bit [rows_bound, hidden], or y_table as c_table above.
 * scratch: sy_expert_ffn_scratch_bytes(experts) bytes, zero before the first call; the kernel
 * leaves it zero again. Calls that share one scratch must not overlap (one per stream).
 * compute_shape: 0 = streaming shape (decode), 1 = compute shape (prefill).
 * The launch is one persistent block per SM (or pair of SMs) whose blocks wait for one another,
 * sized by an occupancy query: all of them must be resident at once. Do not overlap it on the
 * same GPU with another kernel that holds most of an SM's shared memory (the waits are bounded:
 * the cost would be a timeout status, not a hang). */
size_t sy_expert_ffn_scratch_bytes(int n_experts);
int sy_expert_ffn(const void* x, const int32_t* a_rows, const void* gate_up, const void* down, const int32_t* begins,
                  const int32_t* ends, int n_ranges, int ranges_per_expert, int rows_bound, int hidden, int inter,
                  const void* wsorted, void* act, void* y, const uint64_t* y_table, int32_t* scratch, int dtype,
                  int compute_shape, void* stream);

/* expert_ffn_combine — sy_expert_ffn in its streaming shape with sy_combine folded into the down
 * projection's epilogue: replaces switchyard/kernels.py:56-58 and the combine that follows
 * (l.87-88) with one launch. Rows are the plain sorted batch (offsets as from sy_sort_by_expert,
 * token = the sort's token[], pos_of = its pos_of[], rows = n_tokens * top_k). Every result tile
 * counts, per token and block of 128 output columns, the rows it has stored; the tile that
 * stores a token's last row sums that token's rows in ascending row order (= ascending expert
 * id, ties by slot: sy_combine's order) in float32 and rounds once. out [n_tokens, hidden] holds
 * the same bits sy_combine would give; y [rows, hidden] is still written.
 * scratch: sy_expert_ffn_combine_scratch_bytes(...) bytes, zero before the first call, left zero. */
size_t sy_expert_ffn_combine_scratch_bytes(int n_experts, int n_tokens, int hidden);
int sy_expert_ffn_combine(const void* x, const int32_t* token, const void* gate_up, const void* down,
                          const int32_t* offsets, int n_experts, int rows, int hidden, int inter, const void* wsorted,
                          void* act, void* y, const int32_t* pos_of, int top_k, int n_tokens, void* out,
                          int32_t* scratch, int dtype, void* stream);

/* combine — replaces `combine` (moe_kernels.cu:435-444, kernel l.417-433).
 * out[t, :] = round16( sum_j float(y[pos_of[t*top_k + order_j], :]) ), the token's top_k rows
 * added in ascending expert id (ties in slot order), float32 accumulation, one rounding.
 * y 16-bit [m, hidden]; pos_of int32 [m]; idx int32 [n_tokens, top_k]; out 16-bit
 * [n_tokens, hidden]. hidden % 8 == 0, top_k <= 8. */
int sy_combine(const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden,
               void* out, int dtype, void* stream);

/* combine_add — sy_combine followed by the caller's residual add (switchyard/model.py:135,
 * `x = x + self.moe(i, h)`) in the same launch: out[t, :] = round16( float(residual[t, :]) +
 * float(round16(sum)) ), the bits of the 16-bit addition done separately. residual 16-bit
 * [n_tokens, hidden], 16-byte aligned; out must not overlap residual or y. */
int sy_combine_add(const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden,
                   const void* residual, void* out, int dtype, void* stream);

/* gather_rows — replaces `gather_rows` (moe_kernels.cu:459-467, kernel l.450-457).
 * dst[row, :] = src[index[row], :] for row < n; row_bytes % 16 == 0. dst may be memory of a
 * peer GPU (peer access enabled, or an IPC mapping): the dispatch store. */
int sy_gather_rows(const void* src, const int32_t* index, int n, int row_bytes, void* dst, void* stream);

/* copy_async — replaces `copy_async` (moe_kernels.cu:470-475): contiguous copy between any
 * two device buffers (same GPU or peers) on `stream`. */
int sy_copy_async(void* dst, const void* src, size_t bytes, void* stream);


/* enable_peer_access — replaces `enable_peer_access` (moe_kernels.cu:477-489). Sets
 * *enabled_out to 1 if `device` can (now) address `peer`'s memory, 0 if the hardware cannot.
 * Already-enabled is not an error. */
int sy_enable_peer_access(int device, int peer, int* enabled_out);

/* ---- expert parallelism over device-driven transport ----------------------------------------
 * The entry points below have no single counterpart in the reference: together they replace
 * the body of ExpertParallel.phase_send / phase_compute / phase_combine (switchyard/ep.py:174-272)
 * — per destination a gather_rows + three copy_async + an event, per received segment an ffn +
 * a copy back + an event — with three launches per rank and layer that never involve the host.
 * See csrc/ep.cu for the protocol. All pointer tables are HOST arrays of device pointers; entry
 * i belongs to rank i. Memory of other ranks is reached by peer access (one process) or through
 * the IPC mappings below (one process per GPU). */

/* grouped_segments — sy_grouped_gemv (compute_shape = 0) or sy_grouped_gemm (1) over explicit
 * row ranges. Range g is rows [begins[g], ends[g]) of A (no gather); expert e (weights B[e])
 * owns the groups_per_expert consecutive ranges starting at e*groups_per_expert, and its tiles
 * run over their concatenation, so the expert's weights are read once for all of them.
 * begins/ends are device arrays of n_groups ints. Results are stored at the same row index in C,
 * or, if c_table is not NULL, row begins[g] + i of range g goes to ((T*)c_table[g]) + i*n_out
 * (the destination may be a peer GPU's memory). rows_bound: any upper bound of the rows
 * (0 = no-op). */
int sy_grouped_segments(const void* A, const void* B, const int32_t* begins, const int32_t* ends, int n_groups,
                        int groups_per_expert, int rows_bound, int n_out, int k_dim, int swiglu, const void* scale,
                        void* C, const uint64_t* c_table, int dtype, int compute_shape, void* stream);

/* Epochs: every rank keeps one int32 layer counter in its own device memory (zero-initialised,
 * passed as epoch_counter). sy_ep_dispatch advances it and publishes the new value in the
 * receivers' arrival flags; the other entry points of the same layer read it. The host passes
 * no per-layer value, so a whole layer can be captured in a CUDA graph and replayed. */

/* ep_dispatch — sends every sorted row to the rank owning its expert (replaces
 * switchyard/ep.py:193-223): row i (expert in [d*experts_per_rank, (d+1)*experts_per_rank)) is
 * copied from h[token[i]] to row i - offsets[d*experts_per_rank] of x_dst[d], its router weight
 * to w_dst[d]; meta_dst[d] gets experts_per_rank+1 rebased offsets, the segment's first row and
 * its row count. When everything is stored, *flag_dst[d] becomes *epoch_counter + 1 (release,
 * system scope) for every d and *epoch_counter advances.
 * rows_bound: the number of sorted rows as the host knows it (sizes the grid; the kernel takes
 * the exact count from offsets; 0 still publishes empty mailboxes). counters:
 * sy_ep_dispatch_scratch_bytes(n_ranks) bytes of this rank's memory, zero before the first call,
 * left zero. stats: NULL, or two int64 that accumulate the rows sent to other ranks and the rows
 * kept. Rows past `capacity` of a mailbox are dropped and reported through the status word. */
size_t sy_ep_dispatch_scratch_bytes(int n_ranks);
int sy_ep_dispatch(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets, int rows_bound,
                   int experts_per_rank, int n_ranks, int self_rank, int row_bytes, int capacity, void* const* x_dst,
                   void* const* w_dst, int32_t* const* meta_dst, int32_t* const* flag_dst, int32_t* counters,
                   int32_t* epoch_counter, int64_t* stats, void* stream);

/* ep_expert_ffn — sy_expert_ffn over this rank's mailbox (replaces switchyard/ep.py:239-262: one
 * ffn per received segment, a copy back and an event each). The kernel waits (bounded) until
 * arrive_flags[s] has reached the layer's epoch for every sender s, builds its row ranges from the
 * senders' metadata (range e*n_ranks + s = sender s's rows of local expert e; sender s's rows
 * start at s*capacity of x_mail / w_mail; an expert's ranges share its tiles, so its weights are
 * read once), and the down projection's epilogue stores result row i of sender s's segment into
 * y_dst[s] + (first row of the segment in the sender's sort + i) * hidden * 2 bytes. When the
 * whole launch is done, *ret_flag_dst[s] = epoch (release, system scope) for every s.
 * With push_counter != NULL the launch also does the layer's dispatch in its prologue, which
 * takes sy_ep_dispatch off the critical path: the push_* arguments, self_rank, x_dst .. flag_dst,
 * push_counter and stats are sy_ep_dispatch's h, token, wsorted, offsets, rows_bound, self_rank,
 * x_dst .. flag_dst, counters and stats; the layer's epoch is then *epoch_counter + 1 and the
 * launch advances *epoch_counter when it ends. With push_counter == NULL a sy_ep_dispatch before
 * it has done both (the form for ranks that share one GPU and order their steps by events).
 * compute_shape: 0 = streaming shape; 1 / 2 = compute shape with the single-CTA / CTA-pair tile,
 * an expert's ranges sharing its tiles (rows gathered with 16-byte copies); 3 / 4 = the same
 * tiles with every sender's rows of an expert tiled on their own: a range is contiguous in the
 * mailbox, so its rows arrive as TMA boxes (about 30 % faster when a sender brings hundreds of
 * rows per expert; more padding when it brings few). The results are the same bits in all forms.
 * act: 16-bit [n_ranks*capacity, inter] scratch. scratch: sy_expert_ffn_scratch_bytes(n_ranks *
 * experts_per_rank) bytes, zero before the first call, left zero. */
int sy_ep_expert_ffn(const void* x_mail, const void* w_mail, const int32_t* meta, const int32_t* arrive_flags,
                     int32_t* epoch_counter, int n_ranks, int experts_per_rank, int capacity, const void* gate_up,
                     const void* down, int hidden, int inter, void* act, void* const* y_dst,
                     int32_t* const* ret_flag_dst, int32_t* scratch, int dtype, int compute_shape, const void* push_h,
                     const int32_t* push_token, const void* push_wsorted, const int32_t* push_offsets,
                     int push_rows_bound, int self_rank, void* const* x_dst, void* const* w_dst,
                     int32_t* const* meta_dst, int32_t* const* flag_dst, int32_t* push_counter, int64_t* stats,
                     void* stream);

/* ep_wait — one small kernel that waits (bounded, see sy_set_wait_limit_ns) until
 * flags[i] >= *epoch_counter + epoch_offset for i < n (n <= 32). The building block of the waits
 * above on its own: callers that schedule the steps themselves use it, and tests use it to see a
 * wait run out (status 5) without anything else depending on the flag. */
int sy_ep_wait(const int32_t* flags, int n, const int32_t* epoch_counter, int epoch_offset, void* stream);

/* ep_combine — waits (bounded) until ret_flags[d] >= *epoch_counter for all n_ranks owners, then
 * sums each token's rows as sy_combine does (same order, same bits; y is read with L1 bypassed,
 * its rows were stored by other GPUs). A rank with n_tokens == 0 still launches one block.
 * Replaces switchyard/ep.py:264-272 followed by the combine (moe_kernels.cu:417-444). */
int sy_ep_combine(const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter, const void* y,
                  const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden, void* out, int dtype,
                  void* stream);

/* ep_combine_add — sy_ep_combine with the residual add of sy_combine_add in the same launch. */
int sy_ep_combine_add(const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter, const void* y,
                      const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden,
                      const void* residual, void* out, int dtype, void* stream);

/* ipc_export / ipc_open / ipc_close — map one rank's window into another process (CUDA IPC).
 * export: 64-byte handle of the allocation containing ptr and ptr's offset in it.
 * open: the same address in this process (peer access enabled lazily). Set-up time only. */
int sy_ipc_export(void* ptr, unsigned char* handle64, uint64_t* offset_out);
int sy_ipc_open(const unsigned char* handle64, uint64_t offset, void** ptr_out);
int sy_ipc_close(void* ptr, uint64_t offset);

#ifdef __cplusplus
}
#endif
#endif /* SWITCHYARD_B200_H */
